// Dynamic Tanh: a norm without statistics. out = tanh(alpha * x) * weight + shift, element by element, with one
// learned scalar alpha per norm (read from device memory), a weight and a shift per column. x is the float
// residual stream; the arithmetic is float and the result is rounded once to the output type.
//
// mx_dyt:      out[r] = dyt(x[rows[r]] if rows else x[r])
// mx_dyt_sum:  x += acc + col_bias first (the residual sum that a library product left unadded), written back,
//              then out = dyt(x): epilogue and norm in one pass
#include <math.h>

#include "common.cuh"

namespace {

template <typename T>
__global__ void __launch_bounds__(256)
dyt_kernel(float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ acc,
           const float* __restrict__ col_bias, const float* __restrict__ weight, const float* __restrict__ shift,
           const float* __restrict__ alpha_ptr, T* __restrict__ out, int hidden) {
    pdl_trigger();
    const float alpha = alpha_ptr[0];
    pdl_wait();
    x = after_wait(x);
    acc = after_wait(acc);
    const int r = blockIdx.x;
    const size_t src = (size_t)(rows ? after_wait(rows)[r] : r) * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float v = x[src + c];
        if (acc) {
            v += acc[(size_t)r * hidden + c] + (col_bias ? col_bias[c] : 0.f);
            x[src + c] = v;
        }
        out[(size_t)r * hidden + c] = from_float<T>(fmaf(tanhf(alpha * v), weight[c], shift ? shift[c] : 0.f));
    }
}

// The same with four columns a thread and every load of a thread set out before anything is computed: the few
// rows of a decode step cost one trip to memory instead of one per column. hidden a multiple of 4, 16-byte
// aligned rows; blockIdx.y walks the row in pieces of 4 * blockDim.x columns.
template <typename T>
__global__ void __launch_bounds__(256)
dyt_vec_kernel(float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ acc,
               const float* __restrict__ col_bias, const float* __restrict__ weight, const float* __restrict__ shift,
               const float* __restrict__ alpha_ptr, T* __restrict__ out, int hidden) {
    pdl_trigger();
    const int c = 4 * (blockIdx.y * blockDim.x + threadIdx.x);
    const bool live = c < hidden;
    const float alpha = alpha_ptr[0];
    const float4 w4 = live ? *reinterpret_cast<const float4*>(weight + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 s4 = (live && shift) ? *reinterpret_cast<const float4*>(shift + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 b4 = (live && acc && col_bias) ? *reinterpret_cast<const float4*>(col_bias + c)
                                                : make_float4(0.f, 0.f, 0.f, 0.f);
    pdl_wait();
    if (!live) return;
    x = after_wait(x);
    acc = after_wait(acc);
    const int r = blockIdx.x;
    const size_t src = (size_t)(rows ? after_wait(rows)[r] : r) * hidden + c;
    float4 v = *reinterpret_cast<const float4*>(x + src);
    if (acc) {
        const float4 a4 = *reinterpret_cast<const float4*>(acc + (size_t)r * hidden + c);
        v.x += a4.x + b4.x; v.y += a4.y + b4.y; v.z += a4.z + b4.z; v.w += a4.w + b4.w;
        *reinterpret_cast<float4*>(x + src) = v;
    }
    const float o0 = fmaf(tanhf(alpha * v.x), w4.x, s4.x), o1 = fmaf(tanhf(alpha * v.y), w4.y, s4.y);
    const float o2 = fmaf(tanhf(alpha * v.z), w4.z, s4.z), o3 = fmaf(tanhf(alpha * v.w), w4.w, s4.w);
    T* dst = out + (size_t)r * hidden + c;
    if constexpr (sizeof(T) == 4) {
        *reinterpret_cast<float4*>(dst) = make_float4(o0, o1, o2, o3);
    } else {
        __nv_bfloat162 lo = __floats2bfloat162_rn(o0, o1), hi = __floats2bfloat162_rn(o2, o3);
        uint2 pk;
        pk.x = *reinterpret_cast<unsigned*>(&lo);
        pk.y = *reinterpret_cast<unsigned*>(&hi);
        *reinterpret_cast<uint2*>(dst) = pk;
    }
}

}  // namespace

extern "C" int mx_dyt(float* x, const int* rows, const float* acc, const float* col_bias, const float* weight,
                      const float* shift, const float* alpha, void* out, int dtype, int n_rows, int hidden,
                      cudaStream_t stream) {
    if (n_rows <= 0) return MX_OK;
    if (acc != nullptr && rows != nullptr) MX_REFUSE("dynamic tanh: a pending sum cannot be gathered by rows");
    const bool aligned = hidden % 4 == 0 && ((uintptr_t)x | (uintptr_t)out | (uintptr_t)weight | (uintptr_t)shift |
                                             (uintptr_t)acc | (uintptr_t)col_bias) % 16 == 0;
    if (aligned) {
        const int threads = hidden >= 1024 ? 256 : 128;
        const dim3 grid(n_rows, (hidden / 4 + threads - 1) / threads);
        if (dtype == MX_DTYPE_F32)
            mx_launch_chained(dyt_vec_kernel<float>, grid, dim3(threads), 0, stream, x, rows, acc, col_bias, weight,
                              shift, alpha, (float*)out, hidden);
        else
            mx_launch_chained(dyt_vec_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, x, rows, acc, col_bias,
                              weight, shift, alpha, (__nv_bfloat16*)out, hidden);
        return mx_launch_status();
    }
    const int threads = hidden >= 1024 ? 256 : 128;
    if (dtype == MX_DTYPE_F32)
        mx_launch_chained(dyt_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, x, rows, acc, col_bias, weight,
                          shift, alpha, (float*)out, hidden);
    else
        mx_launch_chained(dyt_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream, x, rows, acc, col_bias,
                          weight, shift, alpha, (__nv_bfloat16*)out, hidden);
    return mx_launch_status();
}
