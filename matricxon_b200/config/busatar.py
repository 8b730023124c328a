"""Busatar configuration: a post-norm decoder whose layers each name their own mixer.

``config.json`` holds ``architecture: "Busatar"``, ``vocab``, ``width``, ``norm.eps``, ``postln_alpha``
and a list ``layers``; every entry gives ``type`` (``latent_attention``, ``attention`` or ``rglru``), the
mixer's sizes under ``mixer`` and its feed-forward under ``mlp`` (``kind: dense`` with ``ff`` and
``limit``, or null for a layer that has only the mixer sublayer). A layer computes
``x = norm1(alpha x + mixer(x))`` and, with a feed-forward, ``x = norm2(alpha x + ff(x))``; norms are RMS
norms whose weights are stored around zero. Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.mix.<name>``, ``l<i>.mlp.<name>``, ``final.norm``, ``head`` (no ``.weight`` suffix; biases end in
``.b``). This file is the only place that knows those names and keys; the parts are generic.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from matricxon_b200.config.base import ConfigError, ConfigReader
from matricxon_b200.parts.spec import (
    ClampedGluSpec,
    GatedAttentionSpec,
    InterpolatedRotarySpec,
    LatentAttentionSpec,
    LayerSpec,
    ModelSpec,
    RglruSpec,
    RmsNormSpec,
    sequential_schedule,
)

# what the design fixes
RGLRU_DECAY = 8.0          # log a = -8 r softplus(lambda)
GLU_SLOPE = 1.702          # g * sigmoid(1.702 g)
GLU_SHIFT = 1.0            # ... * (u + 1)
# no key of config.json limits a sequence's length; this sizes the block tables of captured steps
# (longer sequences run uncaptured)
DEFAULT_MAX_POSITIONS = 32768


@dataclass(frozen=True)
class BusatarRotary:
    dims: int
    base: float
    factor: float | None = None
    original: float = 0.0
    fast: float = 32.0
    slow: float = 1.0

    @classmethod
    def from_dict(cls, raw: Any, where: str) -> "BusatarRotary":
        r = ConfigReader(raw, where)
        dims = r.integer("dims", minimum=0)
        if dims % 2:
            raise ConfigError(f"{where}: 'dims' must be even, got {dims}")
        scaling = raw.get("scaling")
        if scaling is None:
            return cls(dims=dims, base=r.number("base", positive=True))
        sr = ConfigReader(scaling, where + ".scaling")
        return cls(dims=dims, base=r.number("base", positive=True), factor=sr.number("factor", positive=True),
                   original=sr.number("original", positive=True), fast=sr.number("fast", positive=True),
                   slow=sr.number("slow", positive=True))

    def to_dict(self) -> dict:
        out: dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.factor is not None:
            out["scaling"] = {"factor": self.factor, "fast": self.fast, "original": self.original, "slow": self.slow}
        return out


@dataclass(frozen=True)
class BusatarLayer:
    type: str
    # attention kinds
    heads: int = 0
    kv_heads: int = 0
    dim: int = 0
    vdim: int = 0
    window: int = 0
    scale: float = 0.0
    # latent attention
    rot_dim: int = 0
    kv_rank: int = 0
    rot: BusatarRotary | None = None
    # recurrence
    width: int = 0
    blocks: int = 0
    conv: int = 0
    # feed-forward (ff == 0: none)
    ff: int = 0
    limit: float = 0.0

    @classmethod
    def from_dict(cls, raw: Any, where: str) -> "BusatarLayer":
        r = ConfigReader(raw, where)
        kind = r.string("type")
        mixer = raw.get("mixer")
        if not isinstance(mixer, dict):
            raise ConfigError(f"{where}: 'mixer' must be an object")
        m = ConfigReader(mixer, where + ".mixer")
        fields: dict[str, Any] = {"type": kind}
        if kind in ("latent_attention", "attention"):
            mask = mixer.get("mask")
            if not isinstance(mask, dict):
                raise ConfigError(f"{where}.mixer: 'mask' must be an object with 'size'")
            dim = m.integer("dim", minimum=1)
            fields.update(heads=m.integer("heads", minimum=1), dim=dim,
                          vdim=m.integer("vdim", dim, minimum=1), scale=m.number("scale", positive=True),
                          window=ConfigReader(mask, where + ".mixer.mask").integer("size", minimum=1))
        if kind == "latent_attention":
            rot_dim = m.integer("rot_dim", minimum=0)
            rot = BusatarRotary.from_dict(mixer.get("rot"), where + ".mixer.rot")
            if rot.dims > rot_dim:
                raise ConfigError(f"{where}.mixer: rot.dims ({rot.dims}) exceeds rot_dim ({rot_dim})")
            fields.update(rot_dim=rot_dim, kv_rank=m.integer("kv_rank", minimum=1), rot=rot)
        elif kind == "attention":
            fields.update(kv_heads=m.integer("kv_heads", fields["heads"], minimum=1))
            if fields["heads"] % fields["kv_heads"]:
                raise ConfigError(f"{where}.mixer: heads ({fields['heads']}) must be a multiple of kv_heads "
                                  f"({fields['kv_heads']})")
            if max(fields["dim"], fields["vdim"]) > 256:
                raise ConfigError(f"{where}.mixer: head sizes above 256 have no attention kernel")
        elif kind == "rglru":
            fields.update(width=m.integer("width", minimum=1), blocks=m.integer("blocks", minimum=1),
                          conv=m.integer("conv", minimum=1))
            if fields["width"] % fields["blocks"]:
                raise ConfigError(f"{where}.mixer: width ({fields['width']}) must be a multiple of blocks "
                                  f"({fields['blocks']})")
        else:
            raise ConfigError(f"{where}: unknown layer type {kind!r}; Busatar has latent_attention, "
                              "attention and rglru")
        mlp = raw.get("mlp")
        if mlp is not None:
            f = ConfigReader(mlp, where + ".mlp")
            if f.string("kind") != "dense":
                raise ConfigError(f"{where}.mlp: unknown feed-forward kind {mlp.get('kind')!r}; Busatar has 'dense'")
            fields.update(ff=f.integer("ff", minimum=1), limit=f.number("limit", positive=True))
        return cls(**fields)

    def to_dict(self) -> dict:
        if self.type == "rglru":
            mixer: dict[str, Any] = {"blocks": self.blocks, "conv": self.conv, "width": self.width}
        else:
            mixer = {"dim": self.dim, "heads": self.heads, "mask": {"size": self.window}, "scale": self.scale,
                     "vdim": self.vdim}
            if self.type == "latent_attention":
                mixer.update(kv_rank=self.kv_rank, rot_dim=self.rot_dim, rot=self.rot.to_dict())
            else:
                mixer.update(kv_heads=self.kv_heads)
        mlp = {"ff": self.ff, "kind": "dense", "limit": self.limit} if self.ff else None
        return {"mixer": mixer, "mlp": mlp, "type": self.type}


@dataclass(frozen=True)
class BusatarConfig:
    vocab: int
    width: int
    eps: float
    postln_alpha: float
    layers: tuple[BusatarLayer, ...]
    max_positions: int = DEFAULT_MAX_POSITIONS

    architecture = "Busatar"
    model_type = "busatar"

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, raw: dict[str, Any], where: str = "config.json") -> "BusatarConfig":
        r = ConfigReader(raw, where)
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError(f"{where}: 'norm' must be an object with 'eps'")
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        return cls(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1),
                   eps=ConfigReader(norm, where + ".norm").number("eps", positive=True),
                   postln_alpha=r.number("postln_alpha"),
                   layers=tuple(BusatarLayer.from_dict(layer, f"{where}.layers[{i}]")
                                for i, layer in enumerate(layers)),
                   max_positions=r.integer("max_positions", DEFAULT_MAX_POSITIONS, minimum=1))

    def to_dict(self) -> dict[str, Any]:
        out = {"architecture": self.architecture, "layers": [layer.to_dict() for layer in self.layers],
               "norm": {"eps": self.eps}, "postln_alpha": self.postln_alpha, "vocab": self.vocab,
               "width": self.width}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        return out

    # ------------------------------------------------------------------ description
    def _mixer_spec(self, layer: BusatarLayer):
        window = layer.window
        if layer.type == "latent_attention":
            rot = layer.rot
            position = InterpolatedRotarySpec(rotary_dim=rot.dims, theta=rot.base, factor=rot.factor,
                                              original=rot.original, fast=rot.fast, slow=rot.slow)
            return LatentAttentionSpec(
                hidden_size=self.width, num_heads=layer.heads, head_dim=layer.dim, rot_dim=layer.rot_dim,
                value_dim=layer.vdim, latent_rank=layer.kv_rank, window=window, scale=layer.scale, eps=self.eps,
                position=position, query_name="q", down_name="dkv", latent_norm_name="dkv.norm",
                key_up_name="uk", value_up_name="uv", output_name="o")
        if layer.type == "attention":
            return GatedAttentionSpec(
                hidden_size=self.width, num_heads=layer.heads, num_kv_heads=layer.kv_heads, head_dim=layer.dim,
                value_dim=layer.vdim, window=window, scale=layer.scale, eps=self.eps, query_name="q",
                key_name="k", value_name="v", output_name="o", gate_name="g", query_norm_name="q.norm",
                key_norm_name="k.norm")
        return RglruSpec(hidden_size=self.width, width=layer.width, blocks=layer.blocks, taps=layer.conv,
                         decay=RGLRU_DECAY, gate_branch_name="y", recurrent_branch_name="x", conv_name="conv",
                         recurrence_gate_name="ra", input_gate_name="ri", lambda_name="lam", output_name="o",
                         bias_suffix=".b")

    def model_spec(self) -> ModelSpec:
        norm = RmsNormSpec(size=self.width, eps=self.eps, unit_offset=True, weight_name="")
        layers = []
        for layer in self.layers:
            feed_forward = None
            if layer.ff:
                feed_forward = ClampedGluSpec(hidden_size=self.width, intermediate_size=layer.ff, limit=layer.limit,
                                              gate_name="gate", up_name="up", down_name="down", slope=GLU_SLOPE,
                                              shift=GLU_SHIFT)
            layers.append(LayerSpec(
                mixer=self._mixer_spec(layer), feed_forward=feed_forward, mixer_norm=norm,
                ffn_norm=norm if feed_forward is not None else None, mixer_name="mix.", feed_forward_name="mlp.",
                mixer_norm_name="norm1", ffn_norm_name="norm2", block="post_norm_sequential",
                skip_scale=self.postln_alpha))
        return ModelSpec(
            hidden_size=self.width, vocab_size=self.vocab, layers=tuple(layers),
            schedule=sequential_schedule(len(layers)), final_norm=norm, tie_word_embeddings=False,
            max_position_embeddings=self.max_positions, embedding_name="embed", layer_prefix="l",
            final_norm_name="final.norm", head_name="head", weight_suffix="", layer_prefix_format="{prefix}{index}.",
            final_norm_prefix="final.norm")
