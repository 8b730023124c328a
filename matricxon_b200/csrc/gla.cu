// Gated linear attention: per head a matrix state S [dim][vdim] that decays per key channel.
//
//   S_t = diag(a_t) S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t,   a_t = sigmoid(z_t)^(1/tau) per key channel,
//   z_t = A2 (A1 h_t) + b. Everything that touches the recurrence is float: q, k, v arrive as the float
//   accumulators of the projections, the decay is formed from float logits, the state lives in float.
//
// mx_gla_decay: rows `low` (the float result of the A1 projection, `rank` wide, `low_ld` apart) -> the decay of
//   every key channel, decay[t][c] = exp(log_sigmoid(A2[c] . low[t] + b[c]) / tau); A2 is float [channels][rank].
//   The small second product stays on the FP32 cores so that no rounding enters the decay.
// mx_gla_scan: every sequence's tokens in order, from and to the state slot [heads][dim][vdim] of the sequence.
//   A block owns (sequence, head, 16 value columns); a thread owns one column and every eighth key channel of it,
//   so the state stays in registers for the whole portion. Tokens arrive sixteen (eight for the widest heads) at a
//   time through shared memory.
//   q is scaled by `q_scale` on its way in. Columns of a state are independent of one another, so cutting vdim
//   into blocks changes no number.
// mx_gla_norm_gate: out[t][h][e] = o[t][h][e] / sqrt(mean_e(o^2) + eps) * weight[e] * silu(gate[t][h][e]): the
//   per-head RMS norm and the output gate, rounded once.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int GLA_COLS = 16;       // value columns per block
constexpr int GLA_SLICES = 8;      // threads per column, each with every eighth key channel
constexpr int GLA_THREADS = GLA_COLS * GLA_SLICES;

__global__ void __launch_bounds__(128)
gla_decay_kernel(const float* __restrict__ low, int low_ld, const float* __restrict__ a2, const float* __restrict__ bias,
                 float inv_tau, float* __restrict__ decay, int channels, int rank) {
    extern __shared__ float low_s[];
    const int t = blockIdx.x;
    for (int r = threadIdx.x; r < rank; r += blockDim.x) low_s[r] = low[(size_t)t * low_ld + r];
    __syncthreads();
    for (int c = threadIdx.x; c < channels; c += blockDim.x) {
        const float* w = a2 + (size_t)c * rank;
        float z = bias ? bias[c] : 0.f;
        for (int r = 0; r < rank; ++r) z = fmaf(w[r], low_s[r], z);
        // log(sigmoid(z)) without cancellation on either side
        const float log_sig = z >= 0.f ? -log1pf(expf(-z)) : z - log1pf(expf(z));
        decay[(size_t)t * channels + c] = expf(log_sig * inv_tau);
    }
}

template <int ROWS, int GLA_TOKENS>     // key channels per thread: dim <= 8 * ROWS; tokens staged per round
__global__ void __launch_bounds__(GLA_THREADS)
gla_scan_kernel(const float* __restrict__ proj, int ld, int q_col, int k_col, int v_col, const float* __restrict__ decay,
                float q_scale, float* __restrict__ state, const int* __restrict__ cu_q, const int* __restrict__ state_slots,
                float* __restrict__ out, int n_heads, int dim, int vdim) {
    __shared__ float q_s[GLA_TOKENS][8 * ROWS], k_s[GLA_TOKENS][8 * ROWS], a_s[GLA_TOKENS][8 * ROWS];
    __shared__ float v_s[GLA_TOKENS][GLA_COLS];
    const int seq = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * GLA_COLS;
    const int t0 = cu_q[seq], t1 = cu_q[seq + 1];
    if (t1 <= t0) return;
    const int tid = threadIdx.x, slice = tid & (GLA_SLICES - 1), col = col0 + (tid >> 3);
    const bool col_ok = col < vdim;
    float* s_base = state + (((size_t)state_slots[seq] * n_heads + head) * dim) * vdim;
    float S[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        const int i = slice + GLA_SLICES * r;
        S[r] = (col_ok && i < dim) ? s_base[(size_t)i * vdim + col] : 0.f;
    }
    for (int base = t0; base < t1; base += GLA_TOKENS) {
        const int n_here = min(GLA_TOKENS, t1 - base);
        __syncthreads();
        for (int item = tid; item < n_here * dim; item += GLA_THREADS) {
            const int j = item / dim, i = item - j * dim;
            const float* row = proj + (size_t)(base + j) * ld;
            q_s[j][i] = row[q_col + head * dim + i] * q_scale;
            k_s[j][i] = row[k_col + head * dim + i];
            a_s[j][i] = decay[((size_t)(base + j) * n_heads + head) * dim + i];
        }
        for (int item = tid; item < n_here * GLA_COLS; item += GLA_THREADS) {
            const int j = item / GLA_COLS, c = item - j * GLA_COLS;
            v_s[j][c] = (col0 + c < vdim) ? proj[(size_t)(base + j) * ld + v_col + head * vdim + col0 + c] : 0.f;
        }
        __syncthreads();
        for (int j = 0; j < n_here; ++j) {
            const float v = v_s[j][tid >> 3];
            float o = 0.f;
#pragma unroll
            for (int r = 0; r < ROWS; ++r) {
                const int i = slice + GLA_SLICES * r;
                if (i < dim) {
                    S[r] = fmaf(a_s[j][i], S[r], k_s[j][i] * v);
                    o = fmaf(S[r], q_s[j][i], o);
                }
            }
            o += __shfl_xor_sync(0xffffffffu, o, 1);
            o += __shfl_xor_sync(0xffffffffu, o, 2);
            o += __shfl_xor_sync(0xffffffffu, o, 4);
            if (slice == 0 && col_ok) out[((size_t)(base + j) * n_heads + head) * vdim + col] = o;
        }
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        const int i = slice + GLA_SLICES * r;
        if (col_ok && i < dim) s_base[(size_t)i * vdim + col] = S[r];
    }
}

template <typename T>
__global__ void __launch_bounds__(128)
gla_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ gate, int gate_ld,
                     const float* __restrict__ weight, float eps, T* __restrict__ out, int n_heads, int vdim) {
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    for (int h = warp; h < n_heads; h += n_warps) {
        const float* src = o + ((size_t)t * n_heads + h) * vdim;
        float s = 0.f;
        for (int e = lane; e < vdim; e += 32) s = fmaf(src[e], src[e], s);
        const float inv = 1.0f / sqrtf(warp_sum(s) / (float)vdim + eps);
        for (int e = lane; e < vdim; e += 32) {
            const float g = gate[(size_t)t * gate_ld + h * vdim + e];
            const float silu = g / (1.0f + expf(-g));
            out[((size_t)t * n_heads + h) * vdim + e] = from_float<T>(src[e] * inv * weight[e] * silu);
        }
    }
}

}  // namespace

extern "C" int mx_gla_decay(const float* low, int low_ld, const float* a2, const float* bias, float tau, float* decay,
                            int n_tokens, int channels, int rank, cudaStream_t stream) {
    if (n_tokens <= 0) return MX_OK;
    if (!(tau > 0.f)) MX_REFUSE("gated linear attention: tau %f is not positive", tau);
    if (rank <= 0 || rank > 8192) MX_REFUSE("gated linear attention: a decay rank of %d", rank);
    gla_decay_kernel<<<n_tokens, 128, (size_t)rank * sizeof(float), stream>>>(low, low_ld, a2, bias, 1.0f / tau, decay,
                                                                             channels, rank);
    return mx_launch_status();
}

extern "C" int mx_gla_scan(const float* proj, int ld, int q_col, int k_col, int v_col, const float* decay, float q_scale,
                           float* state, const int* cu_q, const int* state_slots, float* out, int n_seqs, int n_heads,
                           int dim, int vdim, cudaStream_t stream) {
    if (n_seqs <= 0) return MX_OK;
    if (dim <= 0 || dim > 256) MX_REFUSE("gated linear attention: %d key channels per head (1..256)", dim);
    if (n_heads > 65535) MX_REFUSE("gated linear attention: %d heads exceed the grid", n_heads);
    const dim3 grid(n_seqs, n_heads, (vdim + GLA_COLS - 1) / GLA_COLS);
    if (dim <= 64)
        gla_scan_kernel<8, 16><<<grid, GLA_THREADS, 0, stream>>>(proj, ld, q_col, k_col, v_col, decay, q_scale, state, cu_q,
                                                            state_slots, out, n_heads, dim, vdim);
    else if (dim <= 128)
        gla_scan_kernel<16, 16><<<grid, GLA_THREADS, 0, stream>>>(proj, ld, q_col, k_col, v_col, decay, q_scale, state, cu_q,
                                                             state_slots, out, n_heads, dim, vdim);
    else
        gla_scan_kernel<32, 8><<<grid, GLA_THREADS, 0, stream>>>(proj, ld, q_col, k_col, v_col, decay, q_scale, state, cu_q,
                                                             state_slots, out, n_heads, dim, vdim);
    return mx_launch_status();
}

extern "C" int mx_gla_norm_gate(const float* o, const float* gate, int gate_ld, const float* weight, float eps, void* out,
                                int dtype, int n_tokens, int n_heads, int vdim, cudaStream_t stream) {
    if (n_tokens <= 0) return MX_OK;
    if (dtype == MX_DTYPE_F32)
        gla_norm_gate_kernel<float><<<n_tokens, 128, 0, stream>>>(o, gate, gate_ld, weight, eps, (float*)out, n_heads, vdim);
    else
        gla_norm_gate_kernel<__nv_bfloat16><<<n_tokens, 128, 0, stream>>>(o, gate, gate_ld, weight, eps,
                                                                         (__nv_bfloat16*)out, n_heads, vdim);
    return mx_launch_status();
}
