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

}  // namespace

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
