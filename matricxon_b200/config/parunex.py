"""Parunex configuration: a pre-norm decoder whose layers each name their own mixer and feed-forward.

``config.json`` holds ``architecture: "Parunex"``, ``vocab``, ``width``, ``norm.eps``, ``embedding.scale`` and a list
``layers``; every entry gives ``type`` (``attention`` or ``gla``), the mixer's sizes under ``mixer`` and its
feed-forward under ``mlp`` (``kind: dense`` with ``ff``, ``kind: moe`` with ``expert.ff`` and ``router``, or null for a
layer that has only the mixer sublayer). A layer computes ``x += mixer(norm1(x))`` and, with a feed-forward,
``x += ff(norm2(x))``; every norm is a Dynamic Tanh. Tensor names: ``embed``, ``l<i>.norm1`` (with ``.b`` and
``.alpha`` beside it), ``l<i>.mix.<name>``, ``l<i>.mlp.<name>`` (experts under ``l<i>.mlp.e<j>.``), ``final.norm``,
``head`` (no ``.weight`` suffix; biases end in ``.b``). This file is the only place that knows those names and keys;
the parts are generic.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from matricxon_b200.config.base import ConfigError, ConfigReader
from matricxon_b200.parts.spec import (
    DynamicTanhSpec,
    GatedMlpSpec,
    GlaSpec,
    LayerSpec,
    ModelSpec,
    RoutedExpertsSpec,
    SinkAttentionSpec,
    WavelengthRotarySpec,
    sequential_schedule,
)

# what the design fixes
DENSE_ACTIVATION = "gelu_tanh"       # the dense feed-forward's gate
EXPERT_ACTIVATION = "silu"           # an expert's gate
GROUP_BEST = 2                       # a group of experts is worth the sum of its two best scores
ROUTE_NORM_EPS = 1e-20               # added to the sum of the chosen scores
# no key of config.json limits a sequence's length; this sizes the block tables of captured steps
# (longer sequences run uncaptured)
DEFAULT_MAX_POSITIONS = 32768


def _object(raw: Any, key: str, where: str) -> dict:
    value = raw.get(key) if isinstance(raw, dict) else None
    if not isinstance(value, dict):
        raise ConfigError(f"{where}: {key!r} must be an object")
    return value


@dataclass(frozen=True)
class ParunexRotary:
    dims: int
    base: float
    factor: float | None = None
    low: float = 0.0
    high: float = 0.0
    original: float = 0.0

    @classmethod
    def from_dict(cls, raw: Any, where: str) -> "ParunexRotary":
        r = ConfigReader(raw, where)
        dims = r.integer("dims", minimum=0)
        if dims % 2:
            raise ConfigError(f"{where}: 'dims' must be even, got {dims}")
        base = r.number("base", positive=True)
        scaling = raw.get("scaling")
        if scaling is None:
            return cls(dims=dims, base=base)
        sr = ConfigReader(scaling, where + ".scaling")
        low, high = sr.number("low", positive=True), sr.number("high", positive=True)
        if not high > low:
            raise ConfigError(f"{where}.scaling: 'high' ({high}) must exceed 'low' ({low})")
        return cls(dims=dims, base=base, factor=sr.number("factor", positive=True), low=low, high=high,
                   original=sr.number("original", positive=True))

    def to_dict(self) -> dict:
        out: dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.factor is not None:
            out["scaling"] = {"factor": self.factor, "high": self.high, "low": self.low, "original": self.original}
        return out


@dataclass(frozen=True)
class ParunexFeedForward:
    kind: str                     # "dense" | "moe"
    ff: int                       # the dense width, or one expert's
    experts: int = 0
    top: int = 0
    groups: int = 1
    groups_kept: int = 1
    route_scale: float = 1.0

    @classmethod
    def from_dict(cls, raw: Any, where: str) -> "ParunexFeedForward":
        r = ConfigReader(raw, where)
        kind = r.string("kind")
        if kind == "dense":
            return cls(kind=kind, ff=r.integer("ff", minimum=1))
        if kind != "moe":
            raise ConfigError(f"{where}: unknown feed-forward kind {kind!r}; Parunex has 'dense' and 'moe'")
        expert = ConfigReader(_object(raw, "expert", where), where + ".expert")
        router_raw = _object(raw, "router", where)
        router = ConfigReader(router_raw, where + ".router")
        experts, top = router.integer("experts", minimum=1), router.integer("top", minimum=1)
        groups = kept = 1
        if router_raw.get("groups") is not None:
            g = ConfigReader(_object(router_raw, "groups", where + ".router"), where + ".router.groups")
            groups, kept = g.integer("count", minimum=1), g.integer("keep", minimum=1)
        if top > experts:
            raise ConfigError(f"{where}.router: 'top' ({top}) exceeds 'experts' ({experts})")
        if experts % groups:
            raise ConfigError(f"{where}.router: {experts} experts cannot form {groups} equal groups")
        if kept > groups or kept * (experts // groups) < top:
            raise ConfigError(f"{where}.router: keeping {kept} of {groups} groups leaves fewer than {top} experts")
        return cls(kind=kind, ff=expert.integer("ff", minimum=1), experts=experts, top=top, groups=groups,
                   groups_kept=kept, route_scale=router.number("scale", 1.0))

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return {"ff": self.ff, "kind": "dense"}
        return {"expert": {"ff": self.ff}, "kind": "moe",
                "router": {"experts": self.experts, "groups": {"count": self.groups, "keep": self.groups_kept},
                           "scale": self.route_scale, "top": self.top}}


@dataclass(frozen=True)
class ParunexLayer:
    type: str                     # "attention" | "gla"
    heads: int
    dim: int
    vdim: int
    # attention
    kv_heads: int = 0
    scale: float = 0.0
    softcap: float | None = None
    v_mix: bool = False
    rot: ParunexRotary | None = None
    # gated linear attention
    tau: float = 0.0
    feed_forward: ParunexFeedForward | None = None

    @classmethod
    def from_dict(cls, raw: Any, where: str) -> "ParunexLayer":
        r = ConfigReader(raw, where)
        kind = r.string("type")
        mixer = _object(raw, "mixer", where)
        m = ConfigReader(mixer, where + ".mixer")
        dim = m.integer("dim", minimum=1)
        fields: dict[str, Any] = {"type": kind, "heads": m.integer("heads", minimum=1), "dim": dim,
                                  "vdim": m.integer("vdim", dim, minimum=1)}
        if kind == "attention":
            fields["kv_heads"] = m.integer("kv_heads", fields["heads"], minimum=1)
            if fields["heads"] % fields["kv_heads"]:
                raise ConfigError(f"{where}.mixer: heads ({fields['heads']}) must be a multiple of kv_heads "
                                  f"({fields['kv_heads']})")
            if max(dim, fields["vdim"]) > 256:
                raise ConfigError(f"{where}.mixer: head sizes above 256 have no attention kernel")
            fields["scale"] = m.number("scale", positive=True)
            if mixer.get("softcap") is not None:
                fields["softcap"] = m.number("softcap", positive=True)
            fields["v_mix"] = m.boolean("v_mix", False)
            if mixer.get("rot") is not None:
                rot = ParunexRotary.from_dict(mixer["rot"], where + ".mixer.rot")
                if rot.dims > dim:
                    raise ConfigError(f"{where}.mixer: rot.dims ({rot.dims}) exceeds dim ({dim})")
                fields["rot"] = rot
        elif kind == "gla":
            if dim > 256:
                raise ConfigError(f"{where}.mixer: more than 256 key channels per head have no recurrence kernel")
            fields["tau"] = m.number("tau", positive=True)
        else:
            raise ConfigError(f"{where}: unknown layer type {kind!r}; Parunex has attention and gla")
        if raw.get("mlp") is not None:
            fields["feed_forward"] = ParunexFeedForward.from_dict(raw["mlp"], where + ".mlp")
        return cls(**fields)

    def to_dict(self) -> dict:
        mixer: dict[str, Any] = {"dim": self.dim, "heads": self.heads, "vdim": self.vdim}
        if self.type == "attention":
            mixer.update(kv_heads=self.kv_heads, scale=self.scale, v_mix=self.v_mix)
            if self.softcap is not None:
                mixer["softcap"] = self.softcap
            if self.rot is not None:
                mixer["rot"] = self.rot.to_dict()
        else:
            mixer["tau"] = self.tau
        return {"mixer": mixer, "mlp": self.feed_forward.to_dict() if self.feed_forward else None, "type": self.type}


@dataclass(frozen=True)
class ParunexConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    layers: tuple[ParunexLayer, ...]
    # the rank of a gla layer's decay map is no key of config.json: it is the shape of the layer's first decay
    # matrix. ``decay_ranks`` gives it per layer (0 for attention layers) to whoever builds a model from a
    # configuration alone (random weights); a model folder's tensors overrule it (``with_tensor_shapes``).
    decay_ranks: tuple[int, ...] = ()
    max_positions: int = DEFAULT_MAX_POSITIONS
    # tensors a model folder holds although the model does not use them (a mixing scalar of a layer that does not
    # mix, the second norm of a layer without a feed-forward): (name, shape), found by ``with_tensor_shapes``; they
    # are expected at the weight check and never fetched
    unused_tensors: tuple[tuple[str, tuple[int, ...]], ...] = ()

    architecture = "Parunex"
    model_type = "parunex"
    DEFAULT_DECAY_RANK = 32

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, raw: dict[str, Any], where: str = "config.json") -> "ParunexConfig":
        r = ConfigReader(raw, where)
        eps = ConfigReader(_object(raw, "norm", where), where + ".norm").number("eps", positive=True)
        scale = 1.0
        if raw.get("embedding") is not None:
            scale = ConfigReader(_object(raw, "embedding", where), where + ".embedding").number("scale", 1.0)
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        parsed = tuple(ParunexLayer.from_dict(layer, f"{where}.layers[{i}]") for i, layer in enumerate(layers))
        ranks = raw.get("decay_ranks")
        if ranks is None:
            ranks = [cls.DEFAULT_DECAY_RANK if layer.type == "gla" else 0 for layer in parsed]
        if not isinstance(ranks, list) or len(ranks) != len(parsed) or \
                any(isinstance(x, bool) or not isinstance(x, int) or x < 0 for x in ranks):
            raise ConfigError(f"{where}: 'decay_ranks' must list one non-negative integer per layer")
        config = cls(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1), eps=eps,
                     embedding_scale=scale, layers=parsed, decay_ranks=tuple(ranks),
                     max_positions=r.integer("max_positions", DEFAULT_MAX_POSITIONS, minimum=1))
        config._check_value_mix(where)
        return config

    def _check_value_mix(self, where: str) -> None:
        mixing = [layer for layer in self.layers if layer.type == "attention" and layer.v_mix]
        for layer in mixing[1:]:
            if (layer.kv_heads, layer.vdim) != (mixing[0].kv_heads, mixing[0].vdim):
                raise ConfigError(f"{where}: layers that mix values must agree on kv_heads and vdim "
                                  f"({mixing[0].kv_heads} x {mixing[0].vdim} against {layer.kv_heads} x {layer.vdim})")

    def with_tensor_shapes(self, shape_of) -> "ParunexConfig":
        """The configuration with every gla layer's decay rank read from its tensors: ``shape_of(name)`` gives a
        tensor's shape or None."""
        ranks = list(self.decay_ranks)
        unused = []
        for index, layer in enumerate(self.layers):
            if layer.type == "gla":
                shape = shape_of(f"l{index}.mix.a1")
                if shape is not None and len(shape) == 2:
                    ranks[index] = int(shape[0])
            optional = []
            if layer.type == "attention" and not layer.v_mix:
                optional.append(f"l{index}.mix.vmix")
            if layer.feed_forward is None:
                optional += [f"l{index}.norm2", f"l{index}.norm2.b", f"l{index}.norm2.alpha"]
            for name in optional:
                shape = shape_of(name)
                if shape is not None:
                    unused.append((name, tuple(int(extent) for extent in shape)))
        from dataclasses import replace

        return replace(self, decay_ranks=tuple(ranks), unused_tensors=tuple(unused))

    def to_dict(self) -> dict[str, Any]:
        out = {"architecture": self.architecture, "embedding": {"scale": self.embedding_scale},
               "layers": [layer.to_dict() for layer in self.layers], "norm": {"eps": self.eps}, "vocab": self.vocab,
               "width": self.width}
        default = [self.DEFAULT_DECAY_RANK if layer.type == "gla" else 0 for layer in self.layers]
        if list(self.decay_ranks) != default:
            out["decay_ranks"] = list(self.decay_ranks)
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        return out

    # ------------------------------------------------------------------ description
    def _mixer_spec(self, index: int, layer: ParunexLayer, first_mixing: int | None):
        if layer.type == "attention":
            position = None
            if layer.rot is not None and layer.rot.dims > 0:
                rot = layer.rot
                position = WavelengthRotarySpec(rotary_dim=rot.dims, theta=rot.base, factor=rot.factor,
                                                original=rot.original, low=rot.low, high=rot.high)
            value_mix = None
            if layer.v_mix:
                value_mix = "source" if index == first_mixing else "blend"
            return SinkAttentionSpec(
                hidden_size=self.width, num_heads=layer.heads, num_kv_heads=layer.kv_heads, head_dim=layer.dim,
                value_dim=layer.vdim, window=None, scale=layer.scale, softcap=layer.softcap, bias=True,
                position=position, query_name="q", key_name="k", value_name="v", output_name="o", gate_name="g",
                sink_name="sink", value_mix=value_mix, value_mix_name="vmix" if layer.v_mix else None, bias_suffix=".b")
        return GlaSpec(hidden_size=self.width, num_heads=layer.heads, head_dim=layer.dim, value_dim=layer.vdim,
                       decay_rank=self.decay_ranks[index] or self.DEFAULT_DECAY_RANK, tau=layer.tau,
                       query_scale=layer.dim ** -0.5, eps=self.eps, query_name="q", key_name="k", value_name="v",
                       gate_name="g", output_name="o", norm_name="norm", decay_down_name="a1", decay_up_name="a2",
                       bias_suffix=".b")

    def _feed_forward_spec(self, f: ParunexFeedForward | None):
        if f is None:
            return None
        if f.kind == "dense":
            return GatedMlpSpec(hidden_size=self.width, intermediate_size=f.ff, activation=DENSE_ACTIVATION,
                                gate_name="gate", up_name="up", down_name="down")
        expert = GatedMlpSpec(hidden_size=self.width, intermediate_size=f.ff, activation=EXPERT_ACTIVATION,
                              gate_name="gate", up_name="up", down_name="down")
        return RoutedExpertsSpec(hidden_size=self.width, num_experts=f.experts, top=f.top, num_groups=f.groups,
                                 groups_kept=f.groups_kept, route_scale=f.route_scale, expert=expert,
                                 router_name="router", expert_format="e{index}.", group_best=GROUP_BEST,
                                 norm_eps=ROUTE_NORM_EPS)

    def model_spec(self) -> ModelSpec:
        norm = DynamicTanhSpec(size=self.width, weight_name="", shift_name=".b", alpha_name=".alpha")
        first_mixing = next((i for i, layer in enumerate(self.layers)
                             if layer.type == "attention" and layer.v_mix), None)
        layers = []
        for index, layer in enumerate(self.layers):
            feed_forward = self._feed_forward_spec(layer.feed_forward)
            layers.append(LayerSpec(
                mixer=self._mixer_spec(index, layer, first_mixing), feed_forward=feed_forward, mixer_norm=norm,
                ffn_norm=norm if feed_forward is not None else None, mixer_name="mix.", feed_forward_name="mlp.",
                mixer_norm_name="norm1", ffn_norm_name="norm2", block="pre_norm_sequential", part_separator=""))
        return ModelSpec(
            hidden_size=self.width, vocab_size=self.vocab, layers=tuple(layers),
            schedule=sequential_schedule(len(layers)), final_norm=norm, tie_word_embeddings=False,
            max_position_embeddings=self.max_positions, embedding_name="embed", layer_prefix="l",
            final_norm_name="final.norm", head_name="head", embedding_scale=self.embedding_scale, weight_suffix="",
            layer_prefix_format="{prefix}{index}.", final_norm_prefix="final.norm",
            extra={"unused_tensors": self.unused_tensors})
