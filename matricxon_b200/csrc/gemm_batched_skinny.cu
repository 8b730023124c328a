// Many small independent products with at most 16 rows each (the per-head and per-block products of a
// decode step): out[m][b][n] = sum_k A[m][b][k] * W[b][n][k], bfloat16 in, float accumulation.
//
// One warp per output column (b, n): the weight row is read once with 16-byte loads (lane l takes the
// elements 8l .. 8l+7 of every block of 256), every row of A against it, and the lanes' partial sums are
// added by shuffles in a fixed order, so a row's result does not depend on the other rows. The operands
// of the batch members may interleave (heads side by side in a row): rows are lda / ldo apart, members
// a_batch / w_batch / o_batch apart. Takes part in chained launches. K must be a multiple of 8 and every row 16-byte aligned.
#include "common.cuh"

namespace {

constexpr int BS_ROWS = 16;
constexpr int BS_WARPS = 8;

template <typename TOut>
__global__ void __launch_bounds__(BS_WARPS * 32)
batched_skinny_kernel(const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ W,
                      TOut* __restrict__ out, int M, int N, int K, int lda, int ldw, int ldo, int batch,
                      long long a_batch, long long w_batch, long long o_batch) {
    pdl_trigger();
    pdl_wait();
    A = after_wait(A);
    const long long column = (long long)blockIdx.x * BS_WARPS + (threadIdx.x >> 5);
    if (column >= (long long)batch * N) return;
    const int b = (int)(column / N), n = (int)(column - (long long)b * N);
    const int lane = threadIdx.x & 31;
    const __nv_bfloat16* w = W + (size_t)b * w_batch + (size_t)n * ldw;
    const __nv_bfloat16* a = A + (size_t)b * a_batch;
    float acc[BS_ROWS];
#pragma unroll
    for (int m = 0; m < BS_ROWS; ++m) acc[m] = 0.f;
    for (int k = lane * 8; k < K; k += 256) {
        const uint4 wraw = *reinterpret_cast<const uint4*>(w + k);
        const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wraw);
        float wf[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) { wf[2 * e] = __low2float(w2[e]); wf[2 * e + 1] = __high2float(w2[e]); }
#pragma unroll
        for (int m = 0; m < BS_ROWS; ++m) {
            if (m < M) {
                const uint4 araw = *reinterpret_cast<const uint4*>(a + (size_t)m * lda + k);
                const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&araw);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    acc[m] = fmaf(__low2float(a2[e]), wf[2 * e], acc[m]);
                    acc[m] = fmaf(__high2float(a2[e]), wf[2 * e + 1], acc[m]);
                }
            }
        }
    }
#pragma unroll
    for (int m = 0; m < BS_ROWS; ++m) {
        if (m < M) {
            const float total = warp_sum(acc[m]);
            if (lane == 0) out[(size_t)m * ldo + (size_t)b * o_batch + n] = from_float<TOut>(total);
        }
    }
}

}  // namespace

extern "C" int mx_gemm_batched_skinny(const void* A, const void* W, void* out, int out_dtype, int M, int N, int K,
                                      int lda, int ldw, int ldo, int batch, long long a_batch, long long w_batch,
                                      long long o_batch, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || batch <= 0) return MX_OK;
    if (M > BS_ROWS) MX_REFUSE("batched skinny product: %d rows exceed %d", M, BS_ROWS);
    if (K <= 0 || K % 8 || lda % 8 || ldw % 8 || a_batch % 8 || w_batch % 8)
        MX_REFUSE("batched skinny product: K = %d and the strides must be multiples of 8", K);
    const long long columns = (long long)batch * N;
    const unsigned blocks = (unsigned)((columns + BS_WARPS - 1) / BS_WARPS);
    if (out_dtype == MX_DTYPE_F32)
        mx_launch_chained(batched_skinny_kernel<float>, dim3(blocks), dim3(BS_WARPS * 32), 0, stream,
                          (const __nv_bfloat16*)A, (const __nv_bfloat16*)W, (float*)out, M, N, K, lda, ldw, ldo, batch,
                          a_batch, w_batch, o_batch);
    else
        mx_launch_chained(batched_skinny_kernel<__nv_bfloat16>, dim3(blocks), dim3(BS_WARPS * 32), 0, stream,
                          (const __nv_bfloat16*)A, (const __nv_bfloat16*)W, (__nv_bfloat16*)out, M, N, K, lda, ldw, ldo,
                          batch, a_batch, w_batch, o_batch);
    return mx_launch_status();
}
