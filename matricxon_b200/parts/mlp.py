"""The plain (ungated) feed-forward: ``residual + down(act(up(h)))``.

``m = gelu_tanh(h Wfc^T + bfc)`` with ``gelu_tanh(u) = 0.5 u (1 + tanh(sqrt(2/pi)(u + 0.044715 u^3)))``,
then ``m Wproj^T + bproj`` added to the residual (app/architectures/starcoder2_layers.py:9-23,68).
The activation is applied to the float accumulator of the first product in the engine's own kernels;
for steps of 17 to 128 rows, where the library's product stands (ops/linear.py), to its bfloat16 result.
"""

from __future__ import annotations

from matricxon_b200.ops.linear import EPILOGUE_GELU, EPILOGUE_RESIDUAL, linear
from matricxon_b200.parts.base import FeedForward, register_part
from matricxon_b200.weights.loader import WeightSpec

_ACTIVATION_MODES = {"gelu_tanh": EPILOGUE_GELU}


@register_part("feed_forward", "mlp")
class Mlp(FeedForward):
    capturable = True

    def __init__(self, spec, runtime, prefix):
        super().__init__(spec, runtime, prefix)
        if spec.activation not in _ACTIVATION_MODES:
            raise ValueError(f"feed-forward activation {spec.activation!r} has no kernel")

    @classmethod
    def weight_specs(cls, spec, prefix):
        shapes = {spec.up_name: (spec.intermediate_size, spec.hidden_size),
                  spec.down_name: (spec.hidden_size, spec.intermediate_size)}
        specs = []
        for name, shape in shapes.items():
            specs.append(WeightSpec(f"{prefix}{name}.weight", shape, role="matrix", init="weight"))
            if spec.bias:
                specs.append(WeightSpec(f"{prefix}{name}.bias", (shape[0],), role="vector", init="bias"))
        return specs

    def load(self, fetch):
        p, s = self.prefix, self.spec
        self.up_weight = fetch(f"{p}{s.up_name}.weight")
        self.down_weight = fetch(f"{p}{s.down_name}.weight")
        self.up_bias = fetch(f"{p}{s.up_name}.bias") if s.bias else None
        self.down_bias = fetch(f"{p}{s.down_name}.bias") if s.bias else None

    def forward(self, h, residual, ctx):
        backend = self.runtime.gemm_backend
        mid = linear(h, self.up_weight, self.up_bias, _ACTIVATION_MODES[self.spec.activation],
                     backend=backend)
        return linear(mid, self.down_weight, self.down_bias, EPILOGUE_RESIDUAL, residual=residual,
                      out=residual, backend=backend, defer_sum=getattr(ctx, "sums_may_pend", False))


@register_part("feed_forward", "clamped_glu")
class ClampedGlu(FeedForward):
    """``down(g * sigmoid(slope g) * (u + shift))`` with the gate clamped from above and the linear branch
    from both sides (``ClampedGluSpec``): one fused product for gate and up, one activation kernel, the
    down product. ``forward(h, None, ctx)`` returns the float output without a residual."""

    capturable = True

    @classmethod
    def weight_specs(cls, spec, prefix):
        wide = (spec.intermediate_size, spec.hidden_size)
        return [WeightSpec(prefix + spec.gate_name, wide, role="matrix", init="weight"),
                WeightSpec(prefix + spec.up_name, wide, role="matrix", init="weight"),
                WeightSpec(prefix + spec.down_name, (spec.hidden_size, spec.intermediate_size), role="matrix",
                           init="weight")]

    def load(self, fetch):
        import torch

        p, s = self.prefix, self.spec
        self.gate_up_weight = torch.cat([fetch(p + s.gate_name), fetch(p + s.up_name)])
        self.down_weight = fetch(p + s.down_name)

    def forward(self, h, residual, ctx):
        import torch

        from matricxon_b200.ops import kernels
        from matricxon_b200.ops.linear import EPILOGUE_F32, EPILOGUE_NONE

        s, backend = self.spec, self.runtime.gemm_backend
        gate_up = linear(h, self.gate_up_weight, None, EPILOGUE_NONE, backend=backend)
        mid = torch.empty((h.shape[0], s.intermediate_size), dtype=gate_up.dtype, device=h.device)
        kernels.clamped_glu(gate_up, mid, s.limit if s.limit is not None else 0.0, s.slope, s.shift)
        if residual is None:
            return linear(mid, self.down_weight, None, EPILOGUE_F32, backend=backend)
        return linear(mid, self.down_weight, None, EPILOGUE_RESIDUAL, residual=residual, out=residual,
                      backend=backend)


@register_part("feed_forward", "gated_mlp")
class GatedMlp(FeedForward):
    """``down(act(gate(h)) * up(h))`` without biases (``GatedMlpSpec``): one fused product for gate and up, one
    activation kernel, the down product with the residual added. ``forward(h, None, ctx)`` returns the float
    output without a residual."""

    capturable = True

    def __init__(self, spec, runtime, prefix):
        super().__init__(spec, runtime, prefix)
        from matricxon_b200.ops import kernels

        if spec.activation not in kernels.GLU_ACTIVATIONS:
            raise ValueError(f"feed-forward activation {spec.activation!r} has no kernel")

    @classmethod
    def weight_specs(cls, spec, prefix):
        wide = (spec.intermediate_size, spec.hidden_size)
        return [WeightSpec(prefix + spec.gate_name, wide, role="matrix", init="weight"),
                WeightSpec(prefix + spec.up_name, wide, role="matrix", init="weight"),
                WeightSpec(prefix + spec.down_name, (spec.hidden_size, spec.intermediate_size), role="matrix",
                           init="weight")]

    def load(self, fetch):
        import torch

        p, s = self.prefix, self.spec
        self.gate_up_weight = torch.cat([fetch(p + s.gate_name), fetch(p + s.up_name)])
        self.down_weight = fetch(p + s.down_name)

    def forward(self, h, residual, ctx):
        import torch

        from matricxon_b200.ops import kernels
        from matricxon_b200.ops.linear import EPILOGUE_F32, EPILOGUE_NONE

        s, backend = self.spec, self.runtime.gemm_backend
        gate_up = linear(h, self.gate_up_weight, None, EPILOGUE_NONE, backend=backend)
        mid = torch.empty((h.shape[0], s.intermediate_size), dtype=gate_up.dtype, device=h.device)
        kernels.glu(gate_up, mid, s.activation)
        if residual is None:
            return linear(mid, self.down_weight, None, EPILOGUE_F32, backend=backend)
        return linear(mid, self.down_weight, None, EPILOGUE_RESIDUAL, residual=residual, out=residual,
                      backend=backend, defer_sum=getattr(ctx, "sums_may_pend", False))
