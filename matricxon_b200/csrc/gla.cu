// Gated linear attention: per head a matrix state S [dim][vdim] that decays per key channel.
//
//   S_t = diag(a_t) S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t,   a_t = sigmoid(z_t)^(1/tau) per key channel,
//   z_t = A2 (A1 h_t) + b. Everything that touches the recurrence is float: q, k, v arrive as the float
//   accumulators of the projections, the decay is formed from float logits, the state lives in float.
//
// mx_gla_decay: rows `low` (the float result of the A1 projection, `rank` wide, `low_ld` apart) -> the decay of
//   every key channel, decay[t][c] = exp(log_sigmoid(A2[c] . low[t] + b[c]) / tau); A2 is float [channels][rank].
//   The small second product stays on the FP32 cores so that no rounding enters the decay: a thread per channel
//   keeps its row of A2 in registers for sixteen tokens.
// mx_gla_scan: every sequence's tokens in order, from and to the state slot [heads][dim][vdim] of the sequence.
//   A block owns (sequence, head, 16 value columns); a thread owns two columns and a sixteenth or a thirty-second
//   of their key channels (decay, key and query of a channel serve both columns; four or eight state rows a thread,
//   so that an SM holds eight warps of a head's 16,384 state elements), and the state stays in registers for the whole
//   portion. Tokens arrive eight or sixteen at a time through shared memory; a thread's operands of the next token are in
//   registers before it computes the current one, and the shares of an output are added up once a round.
//   q is scaled by `q_scale` on its way in. Columns of a state are independent of one another, so cutting vdim
//   into blocks changes no number.
// mx_gla_norm_gate: out[t][h][e] = o[t][h][e] / sqrt(mean_e(o^2) + eps) * weight[e] * silu(gate[t][h][e]): the
//   per-head RMS norm and the output gate, rounded once.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int GLA_COLS = 16;       // value columns per block

constexpr int DECAY_TOKENS = 16;   // tokens a block of the decay kernel walks with its rows of A2 in registers
constexpr int DECAY_CHUNK = 32;    // entries of a row of A2 a thread holds at a time

__global__ void __launch_bounds__(256)
gla_decay_kernel(const float* __restrict__ low, int low_ld, const float* __restrict__ a2, const float* __restrict__ bias,
                 float inv_tau, float* __restrict__ decay, int n_tokens, int channels, int rank, int rank_pad) {
    // a thread owns one channel: its row of A2 is read once for DECAY_TOKENS tokens, whose low-rank vectors lie in
    // shared memory (padded with zeros to a multiple of four) and are read as broadcasts
    extern __shared__ __align__(16) float low_s[];           // [DECAY_TOKENS][rank_pad]
    const int t0 = blockIdx.x * DECAY_TOKENS, n_here = min(DECAY_TOKENS, n_tokens - t0);
    for (int item = threadIdx.x; item < DECAY_TOKENS * rank_pad; item += blockDim.x) {
        const int j = item / rank_pad, r = item - j * rank_pad;
        low_s[item] = (j < n_here && r < rank) ? low[(size_t)(t0 + j) * low_ld + r] : 0.f;
    }
    __syncthreads();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const float* w = a2 + (size_t)c * rank;
    const bool vec = rank % 4 == 0 && (reinterpret_cast<uintptr_t>(a2) & 15) == 0;
    float z[DECAY_TOKENS];
    const float b = bias ? bias[c] : 0.f;
#pragma unroll
    for (int j = 0; j < DECAY_TOKENS; ++j) z[j] = b;
    for (int r0 = 0; r0 < rank; r0 += DECAY_CHUNK) {
        float4 w4[DECAY_CHUNK / 4];
#pragma unroll
        for (int u = 0; u < DECAY_CHUNK / 4; ++u) {
            const int r = r0 + 4 * u;
            if (vec) {
                w4[u] = r < rank ? *reinterpret_cast<const float4*>(w + r) : make_float4(0.f, 0.f, 0.f, 0.f);
            } else {
                w4[u].x = r < rank ? w[r] : 0.f;
                w4[u].y = r + 1 < rank ? w[r + 1] : 0.f;
                w4[u].z = r + 2 < rank ? w[r + 2] : 0.f;
                w4[u].w = r + 3 < rank ? w[r + 3] : 0.f;
            }
        }
#pragma unroll
        for (int j = 0; j < DECAY_TOKENS; ++j) {
#pragma unroll
            for (int u = 0; u < DECAY_CHUNK / 4; ++u) {
                if (r0 + 4 * u < rank_pad) {
                    const float4 l4 = *reinterpret_cast<const float4*>(&low_s[j * rank_pad + r0 + 4 * u]);
                    z[j] = fmaf(w4[u].x, l4.x, z[j]);
                    z[j] = fmaf(w4[u].y, l4.y, z[j]);
                    z[j] = fmaf(w4[u].z, l4.z, z[j]);
                    z[j] = fmaf(w4[u].w, l4.w, z[j]);
                }
            }
        }
    }
#pragma unroll
    for (int j = 0; j < DECAY_TOKENS; ++j) {
        if (j < n_here) {
            // log(sigmoid(z)) without cancellation on either side
            const float log_sig = z[j] >= 0.f ? -log1pf(expf(-z[j])) : z[j] - log1pf(expf(z[j]));
            decay[(size_t)(t0 + j) * channels + c] = expf(log_sig * inv_tau);
        }
    }
}

// GLA_SLICES threads share a pair of columns, each with ROWS of the key channels (dim <= GLA_SLICES * ROWS);
// GLA_TOKENS tokens are staged per round
template <int ROWS, int GLA_SLICES, int GLA_TOKENS>
__global__ void __launch_bounds__(GLA_COLS / 2 * GLA_SLICES)
gla_scan_kernel(const float* __restrict__ proj, int ld, int q_col, int k_col, int v_col, const float* __restrict__ decay,
                float q_scale, float* __restrict__ state, const int* __restrict__ cu_q, const int* __restrict__ state_slots,
                float* __restrict__ out, int n_heads, int dim, int vdim) {
    // a thread's ROWS channels lie side by side (four floats of padding keep the rows of neighbouring slices on
    // different banks)
    constexpr int GLA_THREADS = GLA_COLS / 2 * GLA_SLICES;
    constexpr int PAD = ROWS + 4, R4 = ROWS / 4, CH = GLA_SLICES * ROWS;
    __shared__ __align__(16) float q_s[GLA_TOKENS][GLA_SLICES][PAD], k_s[GLA_TOKENS][GLA_SLICES][PAD],
        a_s[GLA_TOKENS][GLA_SLICES][PAD];
    __shared__ __align__(8) float v_s[GLA_TOKENS][GLA_COLS];
    // a thread's share of every output of the round; the shares of an output are added up once a round
    // (a shuffle chain per token would be the longest wait of the loop)
    __shared__ __align__(8) float o_s[GLA_TOKENS][GLA_SLICES][GLA_COLS];
    const int seq = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * GLA_COLS;
    const int t0 = cu_q[seq], t1 = cu_q[seq + 1];
    if (t1 <= t0) return;
    // the eight column pairs of a slice are neighbouring lanes: a warp's state accesses are whole 64-byte row pieces,
    // its operand loads from shared memory are broadcasts
    const int tid = threadIdx.x, pair = tid & (GLA_COLS / 2 - 1), slice = tid / (GLA_COLS / 2), col = col0 + 2 * pair;
    float* s_base = state + (((size_t)state_slots[seq] * n_heads + head) * dim) * vdim;
    float S0[ROWS], S1[ROWS];          // this thread's channels of columns col and col + 1
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        const int i = slice * ROWS + r;
        S0[r] = (col < vdim && i < dim) ? s_base[(size_t)i * vdim + col] : 0.f;
        S1[r] = (col + 1 < vdim && i < dim) ? s_base[(size_t)i * vdim + col + 1] : 0.f;
    }
    // A round's tokens travel global memory -> registers -> shared memory; the registers of the next round are
    // asked for before this round is computed, so that the recurrence never waits for global memory.
    constexpr int PER = GLA_TOKENS * CH / GLA_THREADS;             // (token, channel) items a thread stages per array
    constexpr int V_PER = (GLA_TOKENS * GLA_COLS + GLA_THREADS - 1) / GLA_THREADS;
    float q_r[PER], k_r[PER], a_r[PER], v_r[V_PER];
    auto fetch = [&](int base) {
        const int n_here = min(GLA_TOKENS, t1 - base);
#pragma unroll
        for (int u = 0; u < PER; ++u) {
            const int item = tid + u * GLA_THREADS, j = item / CH, i = item % CH;
            const bool live = j < n_here && i < dim;
            const float* row = proj + (size_t)(base + j) * ld + head * dim + i;
            q_r[u] = live ? row[q_col] : 0.f;
            k_r[u] = live ? row[k_col] : 0.f;
            a_r[u] = live ? decay[((size_t)(base + j) * n_heads + head) * dim + i] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < V_PER; ++u) {
            const int item = tid + u * GLA_THREADS, j = item / GLA_COLS, c = item % GLA_COLS;
            v_r[u] = (item < GLA_TOKENS * GLA_COLS && j < n_here && col0 + c < vdim)
                         ? proj[(size_t)(base + j) * ld + v_col + head * vdim + col0 + c] : 0.f;
        }
    };
    // one token's operands of this thread, from shared memory into registers (asked for one token ahead)
    struct Operands {
        float4 a[R4], k[R4], q[R4];
        float2 v;
    };
    auto read = [&](Operands& into, int j) {
#pragma unroll
        for (int u = 0; u < R4; ++u) {
            into.a[u] = *reinterpret_cast<const float4*>(&a_s[j][slice][4 * u]);
            into.k[u] = *reinterpret_cast<const float4*>(&k_s[j][slice][4 * u]);
            into.q[u] = *reinterpret_cast<const float4*>(&q_s[j][slice][4 * u]);
        }
        into.v = *reinterpret_cast<const float2*>(&v_s[j][2 * pair]);
    };
    auto advance = [&](const Operands& now, int j) {
        float o0 = 0.f, o1 = 0.f, p0 = 0.f, p1 = 0.f;
#pragma unroll
        for (int u = 0; u < R4; ++u) {               // channels beyond dim hold zeros: no guard needed
            const float av[4] = {now.a[u].x, now.a[u].y, now.a[u].z, now.a[u].w};
            const float kv[4] = {now.k[u].x, now.k[u].y, now.k[u].z, now.k[u].w};
            const float qv[4] = {now.q[u].x, now.q[u].y, now.q[u].z, now.q[u].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                S0[4 * u + e] = fmaf(av[e], S0[4 * u + e], kv[e] * now.v.x);
                S1[4 * u + e] = fmaf(av[e], S1[4 * u + e], kv[e] * now.v.y);
                if (e & 1) {
                    o1 = fmaf(S0[4 * u + e], qv[e], o1);
                    p1 = fmaf(S1[4 * u + e], qv[e], p1);
                } else {
                    o0 = fmaf(S0[4 * u + e], qv[e], o0);
                    p0 = fmaf(S1[4 * u + e], qv[e], p0);
                }
            }
        }
        *reinterpret_cast<float2*>(&o_s[j][slice][2 * pair]) = make_float2(o0 + o1, p0 + p1);
    };
    fetch(t0);
    for (int base = t0; base < t1; base += GLA_TOKENS) {
        const int n_here = min(GLA_TOKENS, t1 - base);
        __syncthreads();
#pragma unroll
        for (int u = 0; u < PER; ++u) {
            const int item = tid + u * GLA_THREADS, j = item / CH, i = item % CH;
            q_s[j][i / ROWS][i % ROWS] = q_r[u] * q_scale;
            k_s[j][i / ROWS][i % ROWS] = k_r[u];
            a_s[j][i / ROWS][i % ROWS] = a_r[u];
        }
#pragma unroll
        for (int u = 0; u < V_PER; ++u) {
            const int item = tid + u * GLA_THREADS;
            if (item < GLA_TOKENS * GLA_COLS) v_s[item / GLA_COLS][item % GLA_COLS] = v_r[u];
        }
        __syncthreads();
        if (base + GLA_TOKENS < t1) fetch(base + GLA_TOKENS);
        Operands even, odd;
        read(even, 0);
        for (int j = 0; j < n_here; j += 2) {
            if (j + 1 < n_here) read(odd, j + 1);
            advance(even, j);
            if (j + 1 < n_here) {
                if (j + 2 < n_here) read(even, j + 2);
                advance(odd, j + 1);
            }
        }
        __syncthreads();
        for (int item = tid; item < n_here * GLA_COLS; item += GLA_THREADS) {
            const int j = item / GLA_COLS, c = item % GLA_COLS;
            float o = 0.f;
#pragma unroll
            for (int sl = 0; sl < GLA_SLICES; ++sl) o += o_s[j][sl][c];
            if (col0 + c < vdim) out[((size_t)(base + j) * n_heads + head) * vdim + col0 + c] = o;
        }
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        const int i = slice * ROWS + r;
        if (col < vdim && i < dim) s_base[(size_t)i * vdim + col] = S0[r];
        if (col + 1 < vdim && i < dim) s_base[(size_t)i * vdim + col + 1] = S1[r];
    }
}

template <typename T>
__global__ void __launch_bounds__(128)
gla_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ gate, int gate_ld,
                     const float* __restrict__ weight, float eps, T* __restrict__ out, int n_heads, int vdim) {
    const int t = blockIdx.x, lane = threadIdx.x & 31;
    const int h = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (h >= n_heads) return;
    const float* src = o + ((size_t)t * n_heads + h) * vdim;
    const float* g_row = gate + (size_t)t * gate_ld + h * vdim;
    constexpr int KEPT = 8;                       // up to 256 values of a head stay in registers
    float val[KEPT], g[KEPT];
    float s = 0.f;
#pragma unroll
    for (int u = 0; u < KEPT; ++u) {
        const int e = lane + 32 * u;
        val[u] = e < vdim ? src[e] : 0.f;
        g[u] = e < vdim ? g_row[e] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < KEPT; ++u) s = fmaf(val[u], val[u], s);
    for (int e = lane + 32 * KEPT; e < vdim; e += 32) s = fmaf(src[e], src[e], s);
    const float inv = 1.0f / sqrtf(warp_sum(s) / (float)vdim + eps);
#pragma unroll
    for (int u = 0; u < KEPT; ++u) {
        const int e = lane + 32 * u;
        if (e < vdim)
            out[((size_t)t * n_heads + h) * vdim + e] = from_float<T>(val[u] * inv * weight[e] * (g[u] / (1.0f + expf(-g[u]))));
    }
    for (int e = lane + 32 * KEPT; e < vdim; e += 32) {
        const float gv = g_row[e];
        out[((size_t)t * n_heads + h) * vdim + e] = from_float<T>(src[e] * inv * weight[e] * (gv / (1.0f + expf(-gv))));
    }
}

}  // namespace

extern "C" int mx_gla_decay(const float* low, int low_ld, const float* a2, const float* bias, float tau, float* decay,
                            int n_tokens, int channels, int rank, cudaStream_t stream) {
    if (n_tokens <= 0) return MX_OK;
    if (!(tau > 0.f)) MX_REFUSE("gated linear attention: tau %f is not positive", tau);
    const int rank_pad = (rank + 3) & ~3;
    const size_t smem = (size_t)DECAY_TOKENS * rank_pad * sizeof(float);
    if (rank <= 0 || smem > 48 * 1024) MX_REFUSE("gated linear attention: a decay rank of %d (1..768)", rank);
    gla_decay_kernel<<<dim3((n_tokens + DECAY_TOKENS - 1) / DECAY_TOKENS, (channels + 255) / 256), 256, smem, stream>>>(
        low, low_ld, a2, bias, 1.0f / tau, decay, n_tokens, channels, rank, rank_pad);
    return mx_launch_status();
}

extern "C" int mx_gla_scan(const float* proj, int ld, int q_col, int k_col, int v_col, const float* decay, float q_scale,
                           float* state, const int* cu_q, const int* state_slots, float* out, int n_seqs, int n_heads,
                           int dim, int vdim, cudaStream_t stream) {
    if (n_seqs <= 0) return MX_OK;
    if (dim <= 0 || dim > 256) MX_REFUSE("gated linear attention: %d key channels per head (1..256)", dim);
    if (n_heads > 65535 || vdim > 65535 * GLA_COLS) MX_REFUSE("gated linear attention: %d heads of %d values exceed the grid", n_heads, vdim);
    const dim3 grid(n_seqs, n_heads, (vdim + GLA_COLS - 1) / GLA_COLS);
    if (dim <= 64)
        gla_scan_kernel<4, 16, 16><<<grid, 128, 0, stream>>>(proj, ld, q_col, k_col, v_col, decay, q_scale, state, cu_q,
                                                            state_slots, out, n_heads, dim, vdim);
    else if (dim <= 128)
        gla_scan_kernel<4, 32, 8><<<grid, 256, 0, stream>>>(proj, ld, q_col, k_col, v_col, decay, q_scale, state, cu_q,
                                                             state_slots, out, n_heads, dim, vdim);
    else
        gla_scan_kernel<16, 16, 8><<<grid, 128, 0, stream>>>(proj, ld, q_col, k_col, v_col, decay, q_scale, state, cu_q,
                                                             state_slots, out, n_heads, dim, vdim);
    return mx_launch_status();
}

extern "C" int mx_gla_norm_gate(const float* o, const float* gate, int gate_ld, const float* weight, float eps, void* out,
                                int dtype, int n_tokens, int n_heads, int vdim, cudaStream_t stream) {
    if (n_tokens <= 0) return MX_OK;
    if (dtype == MX_DTYPE_F32)
        gla_norm_gate_kernel<float><<<dim3(n_tokens, (n_heads + 3) / 4), 128, 0, stream>>>(o, gate, gate_ld, weight, eps,
                                                                                          (float*)out, n_heads, vdim);
    else
        gla_norm_gate_kernel<__nv_bfloat16><<<dim3(n_tokens, (n_heads + 3) / 4), 128, 0, stream>>>(
            o, gate, gate_ld, weight, eps, (__nv_bfloat16*)out, n_heads, vdim);
    return mx_launch_status();
}
