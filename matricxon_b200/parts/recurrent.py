"""A gated linear recurrence behind a short causal convolution, multiplied by a GELU branch.

Per token t and channel c (``RglruSpec``): ``u = conv(Wx h + bx)``, gates ``r, i`` from block-diagonal
matrices on u, ``a = exp(-decay r softplus(lambda))``, ``S_t = a S_(t-1) + sqrt(1 - a^2) i u`` from
S = 0, output ``Wo (S_t * gelu_tanh(Wy h + by))``. Per request the state slot holds the convolution's
latest ``taps - 1`` inputs and S, both float32; a step continues from them and leaves them for the next
one, so a sequence may be cut anywhere. Decays, gates, softplus, exponentials and the state are float;
the branch products and the gate products run in the runtime dtype with float results.
"""

from __future__ import annotations

import torch

from matricxon_b200.ops import kernels
from matricxon_b200.ops.linear import EPILOGUE_F32, EPILOGUE_RESIDUAL, batched_linear, linear
from matricxon_b200.parts.base import Mixer, StateRequest, register_part
from matricxon_b200.weights.loader import WeightSpec


@register_part("mixer", "rglru")
class GatedLinearRecurrence(Mixer):
    capturable = True

    @classmethod
    def weight_specs(cls, spec, prefix):
        s, b = spec, spec.bias_suffix
        block = s.width // s.blocks
        specs = []
        for name in (s.recurrent_branch_name, s.gate_branch_name):
            specs.append(WeightSpec(prefix + name, (s.width, s.hidden_size), role="matrix", init="weight"))
            specs.append(WeightSpec(prefix + name + b, (s.width,), role="vector", init="bias"))
        specs.append(WeightSpec(prefix + s.conv_name, (s.width, s.taps), role="vector", init="weight"))
        specs.append(WeightSpec(prefix + s.conv_name + b, (s.width,), role="vector", init="bias"))
        for name in (s.recurrence_gate_name, s.input_gate_name):
            specs.append(WeightSpec(prefix + name, (s.blocks, block, block), role="matrix", init="weight"))
            specs.append(WeightSpec(prefix + name + b, (s.blocks, block), role="vector", init="bias"))
        specs.append(WeightSpec(prefix + s.lambda_name, (s.width,), role="vector", init="bias"))
        specs.append(WeightSpec(prefix + s.output_name, (s.hidden_size, s.width), role="matrix", init="weight"))
        return specs

    @classmethod
    def state_request(cls, spec):
        # rows 0 .. taps-2: the convolution's latest inputs, oldest first; row taps-1: the recurrent state
        return StateRequest(shape=(spec.taps, spec.width), dtype=torch.float32)

    def load(self, fetch):
        p, s, b = self.prefix, self.spec, self.spec.bias_suffix
        # one product for both branches: columns [x | y]
        self.branch_weight = torch.cat([fetch(p + s.recurrent_branch_name), fetch(p + s.gate_branch_name)])
        self.branch_bias = torch.cat([fetch(p + s.recurrent_branch_name + b), fetch(p + s.gate_branch_name + b)])
        self.conv_weight = fetch(p + s.conv_name)
        self.conv_bias = fetch(p + s.conv_name + b)
        # per block one product for both gates: rows [recurrence gate | input gate]
        self.gate_weight = torch.cat([fetch(p + s.recurrence_gate_name), fetch(p + s.input_gate_name)], dim=1).contiguous()
        self.gate_bias = torch.cat([fetch(p + s.recurrence_gate_name + b), fetch(p + s.input_gate_name + b)],
                                   dim=1).contiguous()
        self.lam = fetch(p + s.lambda_name)
        self.o_weight = fetch(p + s.output_name)

    def forward(self, h, residual, ctx, binding):
        s, rt = self.spec, self.runtime
        if binding.state is None:
            raise RuntimeError("the recurrence needs a state tensor bound to it")
        n, width, block = h.shape[0], s.width, s.width // s.blocks
        branches = linear(h, self.branch_weight, self.branch_bias, EPILOGUE_F32, backend=rt.gemm_backend)
        u = torch.empty((n, width), dtype=torch.float32, device=h.device)
        u_act = u if rt.dtype == torch.float32 else torch.empty((n, width), dtype=rt.dtype, device=h.device)
        kernels.causal_conv(branches, 0, self.conv_weight, self.conv_bias, binding.state, ctx.tok_seq, ctx.cu_q,
                            ctx.state_slots, u, None if u_act is u else u_act)
        gates = torch.empty((n, s.blocks, 2 * block), dtype=torch.float32, device=h.device)
        batched_linear(u_act.view(n, s.blocks, block), self.gate_weight, None, gates)   # the scan adds the biases
        out = torch.empty((n, width), dtype=rt.dtype, device=h.device)
        if not ctx.padded and max(ctx.host.q_lens) > 2 * kernels.SCAN_CHUNK:
            # long portions: the recurrence in chunks (a token-by-token walk of thousands of tokens would
            # leave the GPU to a few warps)
            key = "scan_chunks"
            if key not in ctx.memo:
                chunks, first = kernels.scan_chunk_lists(ctx.host.q_lens)
                both = torch.tensor(chunks + first, dtype=torch.int32).to(h.device, non_blocking=True)
                ctx.memo[key] = (both[:len(chunks)], both[len(chunks):], len(chunks) // 2)
            chunks, first, n_chunks = ctx.memo[key]
            scratch = torch.empty(3 * n_chunks * width, dtype=torch.float32, device=h.device)
            kernels.rglru_scan_chunked(branches, 0, width, u, gates, self.gate_bias, self.lam, s.decay,
                                       binding.state, ctx.cu_q, ctx.state_slots, ctx.n_seqs, block, chunks, first,
                                       n_chunks, scratch, out)
        else:
            kernels.rglru_scan(branches, 0, width, u, gates, self.gate_bias, self.lam, s.decay, binding.state,
                               ctx.cu_q, ctx.state_slots, ctx.n_seqs, block, out)
        if residual is None:
            return linear(out, self.o_weight, None, EPILOGUE_F32, backend=rt.gemm_backend)
        return linear(out, self.o_weight, None, EPILOGUE_RESIDUAL, residual=residual, out=residual,
                      backend=rt.gemm_backend)
