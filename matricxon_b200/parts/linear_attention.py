"""Gated linear attention: a matrix state per head that decays per key channel.

Per token t and head (``GlaSpec``): ``q = Wq h * query_scale``, ``k = Wk h``, ``v = Wv h``, a decay per key channel
``a = sigmoid(A2 (A1 h) + b)^(1/tau)``; ``S_t = diag(a_t) S_(t-1) + k_t v_t^T`` from S = 0 and ``o_t = S_t^T q_t``.
Every head's o is RMS-normalised over its value width with one plain weight, multiplied by ``silu(Wg h)`` and
projected by Wo. Per request the state slot holds S for every head, float32; a step continues from it and leaves
it for the next one, so a sequence may be cut anywhere.

One fused product gives float rows ``[q | k | v | gate | A1 h]``; the second decay product (rank x channels, tiny)
stays on the FP32 cores with float weights, so the decays, their logarithms and exponentials, the state, the norm
and the gate are float in both dtypes; only the large projections run in the runtime dtype.
"""

from __future__ import annotations

import torch

from matricxon_b200.ops import kernels
from matricxon_b200.ops.linear import EPILOGUE_F32, EPILOGUE_RESIDUAL, linear
from matricxon_b200.parts.base import Mixer, StateRequest, register_part
from matricxon_b200.weights.loader import WeightSpec


@register_part("mixer", "gla")
class GatedLinearAttention(Mixer):
    capturable = True

    @classmethod
    def _matrices(cls, spec):
        keys, values = spec.num_heads * spec.head_dim, spec.num_heads * spec.value_dim
        return [(spec.query_name, keys), (spec.key_name, keys), (spec.value_name, values), (spec.gate_name, values),
                (spec.decay_down_name, spec.decay_rank)]

    @classmethod
    def weight_specs(cls, spec, prefix):
        s = spec
        specs = [WeightSpec(prefix + name, (rows, s.hidden_size), role="matrix", init="weight")
                 for name, rows in cls._matrices(s)]
        channels = s.num_heads * s.head_dim
        # the second decay product runs in float: its matrix is held like a vector
        specs.append(WeightSpec(prefix + s.decay_up_name, (channels, s.decay_rank), role="vector", init="weight"))
        specs.append(WeightSpec(prefix + s.decay_up_name + s.bias_suffix, (channels,), role="vector", init="bias"))
        specs.append(WeightSpec(prefix + s.norm_name, (s.value_dim,), role="vector", init="norm_weight"))
        specs.append(WeightSpec(prefix + s.output_name, (s.hidden_size, s.num_heads * s.value_dim), role="matrix",
                                init="weight"))
        return specs

    @classmethod
    def state_request(cls, spec):
        return StateRequest(shape=(spec.num_heads, spec.head_dim, spec.value_dim), dtype=torch.float32)

    def load(self, fetch):
        p, s = self.prefix, self.spec
        self.proj_weight = torch.cat([fetch(p + name) for name, _ in self._matrices(s)])
        self.decay_up = fetch(p + s.decay_up_name)
        self.decay_bias = fetch(p + s.decay_up_name + s.bias_suffix)
        self.norm_weight = fetch(p + s.norm_name)
        self.o_weight = fetch(p + s.output_name)

    def forward(self, h, residual, ctx, binding):
        s, rt = self.spec, self.runtime
        if binding.state is None:
            raise RuntimeError("gated linear attention needs a state tensor bound to it")
        n = h.shape[0]
        keys, values = s.num_heads * s.head_dim, s.num_heads * s.value_dim
        proj = linear(h, self.proj_weight, None, EPILOGUE_F32, backend=rt.gemm_backend)
        k_col, v_col, g_col, low_col = keys, 2 * keys, 2 * keys + values, 2 * keys + 2 * values
        decay = torch.empty((n, keys), dtype=torch.float32, device=h.device)
        kernels.gla_decay(proj[:, low_col:low_col + s.decay_rank], self.decay_up, self.decay_bias, s.tau, decay)
        o = torch.empty((n, values), dtype=torch.float32, device=h.device)
        kernels.gla_scan(proj, 0, k_col, v_col, decay, s.query_scale, binding.state, ctx.cu_q, ctx.state_slots,
                         ctx.n_seqs, o, s.num_heads, s.head_dim, s.value_dim)
        out = torch.empty((n, values), dtype=rt.dtype, device=h.device)
        kernels.gla_norm_gate(o, proj[:, g_col:g_col + values], self.norm_weight, s.eps, out, s.num_heads, s.value_dim)
        if residual is None:
            return linear(out, self.o_weight, None, EPILOGUE_F32, backend=rt.gemm_backend)
        return linear(out, self.o_weight, None, EPILOGUE_RESIDUAL, residual=residual, out=residual,
                      backend=rt.gemm_backend, defer_sum=getattr(ctx, "sums_may_pend", False))
