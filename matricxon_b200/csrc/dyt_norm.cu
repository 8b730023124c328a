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

}  // namespace

extern "C" int mx_dyt(float* x, const int* rows, const float* acc, const float* col_bias, const float* weight,
                      const float* shift, const float* alpha, void* out, int dtype, int n_rows, int hidden,
                      cudaStream_t stream) {
    if (n_rows <= 0) return MX_OK;
    if (acc != nullptr && rows != nullptr) MX_REFUSE("dynamic tanh: a pending sum cannot be gathered by rows");
    const int threads = hidden >= 1024 ? 256 : 128;
    if (dtype == MX_DTYPE_F32)
        mx_launch_chained(dyt_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, x, rows, acc, col_bias, weight,
                          shift, alpha, (float*)out, hidden);
    else
        mx_launch_chained(dyt_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream, x, rows, acc, col_bias,
                          weight, shift, alpha, (__nv_bfloat16*)out, hidden);
    return mx_launch_status();
}
