// The steps around an attention whose keys rotate over a part of the head, whose values may be blended with
// another layer's values of the same token, and whose heads are gated by one number each.
//
// mx_rotate_mix_kv_write: the float result of a fused projection (biases already added), rows
//   [q heads x dim | k heads x dim | v heads x vdim | ...], becomes the operands of the paged attention kernels:
//     q_out [tokens][heads * hd]                 q_h with its first `rot` entries rotated, tail (dim..hd) zero
//     cache keys   [page][0][kv head][slot][hd]  k_h rotated the same way, tail zero
//     cache values [page][1][kv head][hd][slot]  (1 - mix) v_h + mix * other_h, tail (vdim..hd) zero
//   Rotation pairs entry i with entry i + rot/2 (i < rot/2): (u, v) -> (u cos a - v sin a, v cos a + u sin a),
//   a = position * freq[i] in float. `other` (float rows of kv heads x vdim, `other_ld` apart) and the device
//   scalar `mix` are optional: without them the values are stored as they are. One block per token.
// mx_head_gate: out[t][h * vdim + e] = attn[t][h * hd + e] * sigmoid(gate[t][h]): one gate per head, gate in float
//   (a column range of the same fused projection), the product rounded once.
#include <math.h>

#include "common.cuh"

namespace {

template <typename T>
__global__ void __launch_bounds__(128)
rotate_mix_kv_write_kernel(const float* __restrict__ proj, int ld, const int* __restrict__ positions,
                           const float* __restrict__ freq, int rot, const float* __restrict__ other, int other_ld,
                           const float* __restrict__ mix_ptr, const int* __restrict__ slots, T* __restrict__ cache,
                           long long n_slots, int page_size, T* __restrict__ q_out, int n_heads, int n_kv_heads,
                           int dim, int vdim, int hd, int* status) {
    const int t = blockIdx.x;
    const float* row = proj + (size_t)t * ld;
    const float pos = (float)positions[t];
    const int half = rot >> 1;
    long long slot = slots ? slots[t] : -1;
    if (slot != -1 && (slot < 0 || slot >= n_slots)) {
        if (threadIdx.x == 0) atomicOr(status, MX_STATUS_BAD_SLOT);
        slot = -1;
    }
    const long long page = slot >= 0 ? slot / page_size : 0;
    const int offset = slot >= 0 ? (int)(slot - page * page_size) : 0;
    const size_t head_stride = (size_t)page_size * hd;
    T* kbase = cache + ((size_t)page * 2 * n_kv_heads) * head_stride + (size_t)offset * hd;
    T* vbase = cache + ((size_t)page * 2 * n_kv_heads + n_kv_heads) * head_stride + offset;
    const int rot_heads = n_heads + (slot >= 0 ? n_kv_heads : 0);
    // blockIdx.y shares a token's items out between blocks: the few tokens of a decode step then cost one trip
    // to memory instead of one per 128 items
    const int stride = blockDim.x * gridDim.y, start = blockIdx.y * blockDim.x + threadIdx.x;
    for (int item = start; item < rot_heads * hd; item += stride) {
        const int h = item / hd, d = item - h * hd;
        const float* src = row + (size_t)h * dim;            // k heads follow the q heads directly
        float value = 0.f;
        if (d < rot) {
            const int i = d < half ? d : d - half;
            float s, c;
            sincosf(pos * freq[i], &s, &c);
            value = d < half ? src[d] * c - src[d + half] * s : src[d] * c + src[d - half] * s;
        } else if (d < dim) {
            value = src[d];
        }
        T* dst = h < n_heads ? q_out + ((size_t)t * n_heads + h) * hd : kbase + (size_t)(h - n_heads) * head_stride;
        dst[d] = from_float<T>(value);
    }
    if (slot < 0) return;
    const float* vrow = row + (size_t)(n_heads + n_kv_heads) * dim;
    const float mix = (other && mix_ptr) ? mix_ptr[0] : 0.f;
    for (int item = start; item < n_kv_heads * hd; item += stride) {
        const int h = item / hd, d = item - h * hd;
        float value = 0.f;
        if (d < vdim) {
            value = vrow[(size_t)h * vdim + d];
            if (other) value = (1.f - mix) * value + mix * other[(size_t)t * other_ld + (size_t)h * vdim + d];
        }
        vbase[(size_t)h * head_stride + (size_t)d * page_size] = from_float<T>(value);
    }
}

__device__ __forceinline__ float sigmoid_exact(float v) { return 1.0f / (1.0f + expf(-v)); }

template <typename T>
__global__ void head_gate_kernel(const T* __restrict__ attn, const float* __restrict__ gate, int gate_ld,
                                 T* __restrict__ out, int n_heads, int vdim, int hd, long long count) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const int width = n_heads * vdim;
    const long long t = i / width;
    const int c = (int)(i - t * width);
    const int h = c / vdim, e = c - h * vdim;
    const float a = to_float(attn[((size_t)t * n_heads + h) * hd + e]);
    out[i] = from_float<T>(a * sigmoid_exact(gate[(size_t)t * gate_ld + h]));
}

// eight neighbouring values a thread, 16-byte accesses (bfloat16, vdim and hd multiples of 8)
__global__ void head_gate_vec_kernel(const __nv_bfloat16* __restrict__ attn, const float* __restrict__ gate, int gate_ld,
                                     __nv_bfloat16* __restrict__ out, int n_heads, int vdim, int hd, long long groups) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= groups) return;
    const int per_row = n_heads * vdim / 8;
    const long long t = i / per_row;
    const int c = (int)(i - t * per_row) * 8;
    const int h = c / vdim, e = c - h * vdim;
    const float g = sigmoid_exact(gate[(size_t)t * gate_ld + h]);
    const uint4 raw = *reinterpret_cast<const uint4*>(attn + ((size_t)t * n_heads + h) * hd + e);
    const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
    uint4 oraw;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&oraw);
#pragma unroll
    for (int k = 0; k < 4; ++k) o2[k] = __floats2bfloat162_rn(__low2float(a2[k]) * g, __high2float(a2[k]) * g);
    *reinterpret_cast<uint4*>(out + (size_t)t * n_heads * vdim + c) = oraw;
}

}  // namespace

extern "C" int mx_rotate_mix_kv_write(const float* proj, int ld, const int* positions, const float* freq, int rot,
                                      const float* other, int other_ld, const float* mix, const int* slots,
                                      void* cache, long long n_pages, int page_size, void* q_out, int dtype,
                                      int n_tokens, int n_heads, int n_kv_heads, int dim, int vdim, int hd, int* status,
                                      cudaStream_t stream) {
    if (n_tokens <= 0) return MX_OK;
    if (hd < dim || hd < vdim) MX_REFUSE("attention operands: a padded head of %d holds neither %d nor %d", hd, dim, vdim);
    if (rot < 0 || rot % 2 != 0 || rot > dim) MX_REFUSE("attention operands: %d rotated entries in a head of %d", rot, dim);
    if (ld < (n_heads + n_kv_heads) * dim + n_kv_heads * vdim) MX_REFUSE("attention operands: projection rows are too short");
    const long long n_slots = n_pages * page_size;
    // few tokens: as many blocks per token as the items allow; many tokens fill the GPU by themselves
    const int pieces = n_tokens >= 512 ? 1 : max(1, min(32, ((n_heads + n_kv_heads) * hd + 127) / 128));
    const dim3 grid(n_tokens, pieces);
    if (dtype == MX_DTYPE_F32)
        rotate_mix_kv_write_kernel<float><<<grid, 128, 0, stream>>>(
            proj, ld, positions, freq, rot, other, other_ld, mix, cache ? slots : nullptr, (float*)cache, n_slots,
            page_size, (float*)q_out, n_heads, n_kv_heads, dim, vdim, hd, status);
    else
        rotate_mix_kv_write_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>(
            proj, ld, positions, freq, rot, other, other_ld, mix, cache ? slots : nullptr, (__nv_bfloat16*)cache, n_slots,
            page_size, (__nv_bfloat16*)q_out, n_heads, n_kv_heads, dim, vdim, hd, status);
    return mx_launch_status();
}

extern "C" int mx_head_gate(const void* attn, const float* gate, int gate_ld, void* out, int dtype, int n_tokens,
                            int n_heads, int vdim, int hd, cudaStream_t stream) {
    const long long count = (long long)n_tokens * n_heads * vdim;
    if (count <= 0) return MX_OK;
    const unsigned blocks = (unsigned)((count + 255) / 256);
    if (dtype == MX_DTYPE_BF16 && vdim % 8 == 0 && hd % 8 == 0 && ((uintptr_t)attn | (uintptr_t)out) % 16 == 0) {
        const long long groups = count / 8;
        head_gate_vec_kernel<<<(unsigned)((groups + 255) / 256), 256, 0, stream>>>(
            (const __nv_bfloat16*)attn, gate, gate_ld, (__nv_bfloat16*)out, n_heads, vdim, hd, groups);
        return mx_launch_status();
    }
    if (dtype == MX_DTYPE_F32)
        head_gate_kernel<float><<<blocks, 256, 0, stream>>>((const float*)attn, gate, gate_ld, (float*)out, n_heads,
                                                           vdim, hd, count);
    else
        head_gate_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)attn, gate, gate_ld,
                                                                   (__nv_bfloat16*)out, n_heads, vdim, hd, count);
    return mx_launch_status();
}
