// The real-gated linear recurrent unit with its short causal convolution, over a flattened batch of
// sequence portions with per-request state.
//
// Per request the state is a float matrix [taps][width]: rows 0 .. taps-2 hold the convolution's
// latest inputs (oldest first), row taps-1 holds the recurrent state S. A new request's slot is zero,
// which is also what the convolution reads before a sequence's start.
//
// mx_causal_conv (one thread per (token, channel)):
//   u[t][c] = conv_bias[c] + sum_k conv_weight[c][k] * x[t - (taps-1-k)][c]
//   where x is a column range of the branch projection's float result and inputs before the
//   portion's first token come from the state. Writes u as float and, when asked, a copy in the
//   activation dtype (the gate product's operand).
// mx_rglru_scan (one thread per (sequence, channel), tokens in order):
//   r = sigmoid(gates[t][b][j] + bias[b][j]), i = sigmoid(gates[t][b][bw + j] + bias[b][bw + j])   (c = b * bw + j)
//   log a = -decay * r * softplus(lambda[c]);  a = exp(log a)
//   S <- a * S + sqrt(1 - a^2) * i * u[t][c];   out[t][c] = S * gelu_tanh(y[t][c])
//   then stores S and the last taps-1 inputs. Everything is float; only `out` is rounded.
//   sqrt(1 - a^2) is taken as sqrt(-expm1(2 log a)), which keeps its digits when a is close to one.
// A sequence that brings no token in this step (a padding row of a fixed-size batch) is skipped.
// mx_rglru_scan_chunked does the same for long portions in three launches, since the recurrence is linear
// in S: per chunk of at most 32 tokens and channel, the chunk's map S -> A S + B (A the product of its
// a, B its own contribution); per sequence and channel, the chunks' start states in order, from and to
// the request's state; per chunk and channel again, the tokens from the chunk's start state. A token's
// result is the same sequence of float operations whatever else the step holds.
#include <math.h>

#include "common.cuh"

namespace {

template <typename T>
__global__ void causal_conv_kernel(const float* __restrict__ xy, int ld, int x_col,
                                   const float* __restrict__ conv_weight, const float* __restrict__ conv_bias,
                                   const float* __restrict__ state, const int* __restrict__ tok_seq,
                                   const int* __restrict__ cu_q, const int* __restrict__ state_slots,
                                   float* __restrict__ u, T* __restrict__ u_act, int width, int taps) {
    const int t = blockIdx.x;
    const int seq = tok_seq[t];
    if (seq < 0) return;
    const int local = t - cu_q[seq];
    const float* st = state + (size_t)state_slots[seq] * taps * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float v = conv_bias ? conv_bias[c] : 0.f;
        for (int k = 0; k < taps; ++k) {
            const int back = taps - 1 - k;                     // how many tokens before this one
            const float x = (local - back >= 0) ? xy[(size_t)(t - back) * ld + x_col + c]
                                                : st[(size_t)(taps - 1 + local - back) * width + c];
            v = fmaf(conv_weight[(size_t)c * taps + k], x, v);
        }
        u[(size_t)t * width + c] = v;
        if (u_act) u_act[(size_t)t * width + c] = from_float<T>(v);
    }
}

template <typename T>
__global__ void rglru_scan_kernel(const float* __restrict__ xy, int ld, int x_col, int y_col,
                                  const float* __restrict__ u, const float* __restrict__ gates,
                                  const float* __restrict__ gate_bias, const float* __restrict__ lambda,
                                  float decay, float* __restrict__ state,
                                  const int* __restrict__ cu_q, const int* __restrict__ state_slots,
                                  T* __restrict__ out, int width, int block_width, int taps) {
    const int seq = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= width) return;
    const int t0 = cu_q[seq], n = cu_q[seq + 1] - t0;
    if (n <= 0) return;
    float* st = state + (size_t)state_slots[seq] * taps * width;
    const int b = c / block_width, j = c - b * block_width;
    const size_t gate_col = (size_t)b * 2 * block_width + j;
    const float bias_r = gate_bias ? gate_bias[gate_col] : 0.f;
    const float bias_i = gate_bias ? gate_bias[gate_col + block_width] : 0.f;
    const float lam = lambda[c];
    const float rate = -decay * (lam > 20.f ? lam : log1pf(expf(lam)));
    float s = st[(size_t)(taps - 1) * width + c];
    for (int k = 0; k < n; ++k) {
        const size_t t = (size_t)(t0 + k);
        const float* g = gates + t * 2 * width + gate_col;
        const float r = 1.0f / (1.0f + expf(-(g[0] + bias_r)));
        const float i = 1.0f / (1.0f + expf(-(g[block_width] + bias_i)));
        const float log_a = rate * r;
        const float a = expf(log_a);
        const float drive = sqrtf(-expm1f(2.0f * log_a));
        s = fmaf(a, s, drive * (i * u[t * width + c]));
        const float y = gelu_tanh(xy[t * ld + y_col + c]);
        out[t * width + c] = from_float<T>(s * y);
    }
    st[(size_t)(taps - 1) * width + c] = s;
    // the convolution's memory: row r becomes the input taps-1-r tokens before the next one
    for (int r = 0; r < taps - 1; ++r) {
        const int idx = n - (taps - 1) + r;                    // within this portion when >= 0
        st[(size_t)r * width + c] = idx >= 0 ? xy[(size_t)(t0 + idx) * ld + x_col + c]
                                             : st[(size_t)(idx + taps - 1) * width + c];
    }
}

struct GateTerms { float a, b; };

__device__ __forceinline__ GateTerms gate_terms(const float* g, int block_width, float bias_r, float bias_i,
                                                float rate, float u) {
    const float r = 1.0f / (1.0f + expf(-(g[0] + bias_r)));
    const float i = 1.0f / (1.0f + expf(-(g[block_width] + bias_i)));
    const float log_a = rate * r;
    GateTerms t;
    t.a = expf(log_a);
    t.b = sqrtf(-expm1f(2.0f * log_a)) * (i * u);
    return t;
}

struct ChunkScan {
    const float* xy; const float* u; const float* gates; const float* gate_bias; const float* lambda;
    float* state; const int* cu_q; const int* state_slots;
    const int* chunks;        // [n_chunks][2]: (sequence, first token of the chunk within the sequence's portion)
    const int* seq_chunk0;    // [n_seqs + 1]: index of each sequence's first chunk
    float* chunk_a; float* chunk_b; float* chunk_start;   // [n_chunks][width]
    int ld, x_col, y_col, width, block_width, taps, chunk_tokens;
    float decay;
};

template <typename T, int PHASE>   // 0: the chunks' maps; 2: the tokens from the chunks' start states
__global__ void rglru_chunk_kernel(const ChunkScan p, T* __restrict__ out) {
    const int chunk = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= p.width) return;
    const int seq = p.chunks[2 * chunk], first = p.chunks[2 * chunk + 1];
    const int t0 = p.cu_q[seq] + first;
    const int n = min(p.chunk_tokens, p.cu_q[seq + 1] - t0);
    const int b = c / p.block_width, j = c - b * p.block_width;
    const size_t gate_col = (size_t)b * 2 * p.block_width + j;
    const float bias_r = p.gate_bias ? p.gate_bias[gate_col] : 0.f;
    const float bias_i = p.gate_bias ? p.gate_bias[gate_col + p.block_width] : 0.f;
    const float lam = p.lambda[c];
    const float rate = -p.decay * (lam > 20.f ? lam : log1pf(expf(lam)));
    if (PHASE == 0) {
        float a_all = 1.f, b_all = 0.f;
        for (int k = 0; k < n; ++k) {
            const size_t t = (size_t)(t0 + k);
            const GateTerms g = gate_terms(p.gates + t * 2 * p.width + gate_col, p.block_width, bias_r, bias_i, rate,
                                           p.u[t * p.width + c]);
            a_all *= g.a;
            b_all = fmaf(g.a, b_all, g.b);
        }
        p.chunk_a[(size_t)chunk * p.width + c] = a_all;
        p.chunk_b[(size_t)chunk * p.width + c] = b_all;
    } else {
        float s = p.chunk_start[(size_t)chunk * p.width + c];
        for (int k = 0; k < n; ++k) {
            const size_t t = (size_t)(t0 + k);
            const GateTerms g = gate_terms(p.gates + t * 2 * p.width + gate_col, p.block_width, bias_r, bias_i, rate,
                                           p.u[t * p.width + c]);
            s = fmaf(g.a, s, g.b);
            out[t * p.width + c] = from_float<T>(s * gelu_tanh(p.xy[t * p.ld + p.y_col + c]));
        }
    }
}

__global__ void rglru_carry_kernel(const ChunkScan p) {
    const int seq = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= p.width) return;
    const int t0 = p.cu_q[seq], n = p.cu_q[seq + 1] - t0;
    if (n <= 0) return;
    float* st = p.state + (size_t)p.state_slots[seq] * p.taps * p.width;
    float s = st[(size_t)(p.taps - 1) * p.width + c];
    for (int chunk = p.seq_chunk0[seq]; chunk < p.seq_chunk0[seq + 1]; ++chunk) {
        p.chunk_start[(size_t)chunk * p.width + c] = s;
        s = fmaf(p.chunk_a[(size_t)chunk * p.width + c], s, p.chunk_b[(size_t)chunk * p.width + c]);
    }
    st[(size_t)(p.taps - 1) * p.width + c] = s;
    for (int r = 0; r < p.taps - 1; ++r) {
        const int idx = n - (p.taps - 1) + r;
        st[(size_t)r * p.width + c] = idx >= 0 ? p.xy[(size_t)(t0 + idx) * p.ld + p.x_col + c]
                                               : st[(size_t)(idx + p.taps - 1) * p.width + c];
    }
}

}  // namespace

// Note on equality with mx_rglru_scan: inside a chunk the state is advanced by the same fmaf chain; across
// chunks the start state is A S + B instead of that chain, which differs by float rounding only.
extern "C" int mx_rglru_scan_chunked(const float* xy, int ld, int x_col, int y_col, const float* u,
                                     const float* gates, const float* gate_bias, const float* lambda, float decay,
                                     float* state, const int* cu_q, const int* state_slots, const int* chunks,
                                     const int* seq_chunk0, int n_chunks, int chunk_tokens, float* scratch,
                                     void* out, int out_dtype, int n_seqs, int width, int block_width, int taps,
                                     cudaStream_t stream) {
    if (n_seqs <= 0 || n_chunks <= 0) return MX_OK;
    if (block_width <= 0 || width % block_width) MX_REFUSE("recurrence: width %d in blocks of %d", width, block_width);
    ChunkScan p;
    p.xy = xy; p.u = u; p.gates = gates; p.gate_bias = gate_bias; p.lambda = lambda; p.state = state;
    p.cu_q = cu_q; p.state_slots = state_slots; p.chunks = chunks; p.seq_chunk0 = seq_chunk0;
    p.chunk_a = scratch; p.chunk_b = scratch + (size_t)n_chunks * width; p.chunk_start = scratch + 2 * (size_t)n_chunks * width;
    p.ld = ld; p.x_col = x_col; p.y_col = y_col; p.width = width; p.block_width = block_width; p.taps = taps;
    p.chunk_tokens = chunk_tokens; p.decay = decay;
    const int threads = 128;
    const dim3 per_chunk(n_chunks, (width + threads - 1) / threads), per_seq(n_seqs, (width + threads - 1) / threads);
    rglru_chunk_kernel<float, 0><<<per_chunk, threads, 0, stream>>>(p, (float*)nullptr);
    rglru_carry_kernel<<<per_seq, threads, 0, stream>>>(p);
    if (out_dtype == MX_DTYPE_F32) rglru_chunk_kernel<float, 2><<<per_chunk, threads, 0, stream>>>(p, (float*)out);
    else rglru_chunk_kernel<__nv_bfloat16, 2><<<per_chunk, threads, 0, stream>>>(p, (__nv_bfloat16*)out);
    return mx_launch_status();
}

extern "C" int mx_causal_conv(const float* xy, int ld, int x_col, const float* conv_weight,
                              const float* conv_bias, const float* state, const int* tok_seq, const int* cu_q,
                              const int* state_slots, float* u, void* u_act, int act_dtype, int n_tokens,
                              int width, int taps, cudaStream_t stream) {
    if (n_tokens <= 0) return MX_OK;
    if (taps < 1) MX_REFUSE("convolution: %d taps", taps);
    const int threads = width >= 256 ? 256 : 128;
    if (u_act == nullptr || act_dtype == MX_DTYPE_F32)
        causal_conv_kernel<float><<<n_tokens, threads, 0, stream>>>(xy, ld, x_col, conv_weight, conv_bias, state,
                                                                   tok_seq, cu_q, state_slots, u, (float*)u_act,
                                                                   width, taps);
    else
        causal_conv_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(
            xy, ld, x_col, conv_weight, conv_bias, state, tok_seq, cu_q, state_slots, u, (__nv_bfloat16*)u_act,
            width, taps);
    return mx_launch_status();
}

extern "C" int mx_rglru_scan(const float* xy, int ld, int x_col, int y_col, const float* u, const float* gates,
                             const float* gate_bias, const float* lambda, float decay, float* state, const int* cu_q,
                             const int* state_slots, void* out, int out_dtype, int n_seqs, int width,
                             int block_width, int taps, cudaStream_t stream) {
    if (n_seqs <= 0) return MX_OK;
    if (block_width <= 0 || width % block_width) MX_REFUSE("recurrence: width %d in blocks of %d", width, block_width);
    const int threads = 64;
    dim3 grid(n_seqs, (width + threads - 1) / threads);
    if (out_dtype == MX_DTYPE_F32)
        rglru_scan_kernel<float><<<grid, threads, 0, stream>>>(xy, ld, x_col, y_col, u, gates, gate_bias, lambda, decay,
                                                              state, cu_q, state_slots, (float*)out, width, block_width,
                                                              taps);
    else
        rglru_scan_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>(xy, ld, x_col, y_col, u, gates, gate_bias, lambda,
                                                                      decay, state, cu_q, state_slots,
                                                                      (__nv_bfloat16*)out, width, block_width, taps);
    return mx_launch_status();
}
