"""Parunex on the CPU: configuration and registry, tensor names and shapes, the cache plan, errors that name the
key, the rotary table against the plain one, and properties of the plain model itself (tests/plain_parunex.py),
which is the yardstick of the GPU tests."""

import copy
import math

import pytest
import torch

import plain_parunex as plain
from parunex_configs import MODELS, attention, dense, draw, gla, ids, model, moe, single_layer
from matricxon_b200.config.base import ConfigError
from matricxon_b200.config.parunex import ParunexConfig
from matricxon_b200.config.registry import config_from_dict, resolve_architecture
from matricxon_b200.models.decoder import model_weight_specs, plan_cache
from matricxon_b200.parts.rotary import wavelength_scaled_frequencies
from matricxon_b200.weights.loader import DictSource, WeightLoadError, check_weights

F64 = torch.float64


def test_registry_and_round_trip():
    for raw in MODELS.values():
        assert resolve_architecture(raw).config_class is ParunexConfig
        config = config_from_dict(copy.deepcopy(raw))
        again = config_from_dict(config.to_dict())
        assert again == config
    assert resolve_architecture({"model_type": "parunex"}).name == "Parunex"


def test_tensor_names_shapes_and_cache_plan():
    raw = MODELS["P"]
    config = config_from_dict(copy.deepcopy(raw))
    spec = config.model_spec()
    shapes = {s.name: tuple(s.shape) for s in model_weight_specs(spec)}
    assert shapes["embed"] == (300, 96) and shapes["head"] == (300, 96)
    assert shapes["final.norm"] == (96,) and shapes["final.norm.b"] == (96,) and shapes["final.norm.alpha"] == ()
    # layer 0: gla with 3 heads of 24 key channels and 40 values, decay rank 5, routed feed-forward of 6 experts
    assert shapes["l0.mix.q"] == (72, 96) and shapes["l0.mix.v"] == (120, 96) and shapes["l0.mix.g"] == (120, 96)
    assert shapes["l0.mix.a1"] == (5, 96) and shapes["l0.mix.a2"] == (72, 5) and shapes["l0.mix.a2.b"] == (72,)
    assert shapes["l0.mix.norm"] == (40,) and shapes["l0.mix.o"] == (96, 120)
    assert shapes["l0.mlp.router"] == (6, 96) and shapes["l0.mlp.e5.down"] == (96, 56) and "l0.mlp.e6.gate" not in shapes
    # layer 1: attention, 6 heads over 3, keys 24 wide and values 16, one gate per head
    assert shapes["l1.mix.q"] == (144, 96) and shapes["l1.mix.q.b"] == (144,) and shapes["l1.mix.k"] == (72, 96)
    assert shapes["l1.mix.v"] == (48, 96) and shapes["l1.mix.v.b"] == (48,) and shapes["l1.mix.g"] == (6, 96)
    assert shapes["l1.mix.sink"] == (6,) and shapes["l1.mix.vmix"] == () and shapes["l1.mix.o"] == (96, 96)
    assert "l2.mix.vmix" not in shapes and shapes["l4.mix.vmix"] == ()      # only layers that mix name the scalar
    assert "l1.mix.g.b" not in shapes and "l1.mix.o.b" not in shapes
    assert shapes["l1.mlp.gate"] == (136, 96) and shapes["l1.mlp.down"] == (96, 136)
    # layer 2 has no feed-forward and so no second norm
    assert "l2.norm1" in shapes and "l2.norm2" not in shapes and not any(n.startswith("l2.mlp") for n in shapes)
    plan = plan_cache(spec)
    heads = sorted((g.request.num_kv_heads, g.request.head_dim, len(g.entries)) for g in plan.groups)
    assert heads == [(1, 48, 1), (3, 16, 1), (3, 32, 1)]             # heads padded to multiples of 16
    states = [None if s is None else s.shape for s in plan.state_of_entry]
    assert states == [(3, 24, 40), None, None, (2, 56, 16), None]
    # which layer publishes its values and which blend
    mixes = [getattr(layer.mixer, "value_mix", None) for layer in spec.layers]
    assert mixes == [None, "source", None, None, "blend"]


def test_weight_errors_name_every_tensor():
    raw = MODELS["R"]
    tensors = draw(raw, 1)
    config = config_from_dict(copy.deepcopy(raw))
    specs = model_weight_specs(config.model_spec())
    check_weights(specs, DictSource(tensors))
    broken = dict(tensors)
    del broken["l0.mix.sink"]
    broken["l1.mix.a2"] = torch.zeros(100, 9)
    broken["stray"] = torch.zeros(1)
    with pytest.raises(WeightLoadError) as error:
        check_weights(specs, DictSource(broken))
    assert error.value.missing == ["l0.mix.sink"] and error.value.unexpected == ["stray"]
    assert error.value.wrong_shape[0][0] == "l1.mix.a2"


def test_decay_rank_comes_from_the_tensors():
    raw = copy.deepcopy(MODELS["R"])
    del raw["decay_ranks"]
    config = config_from_dict(raw)
    assert config.decay_ranks == (0, ParunexConfig.DEFAULT_DECAY_RANK)
    shaped = config.with_tensor_shapes(lambda name: (7, 100) if name == "l1.mix.a1" else None)
    assert shaped.decay_ranks == (0, 7)
    assert shaped.model_spec().layers[1].mixer.decay_rank == 7


@pytest.mark.parametrize("change, needle", [
    (lambda r: r["layers"][0]["mixer"].pop("scale"), "'scale'"),
    (lambda r: r["layers"][0]["mixer"].update(kv_heads=2), "multiple of kv_heads"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=7), "'dims' must be even"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=14), "exceeds dim"),
    (lambda r: r["layers"][0]["mlp"]["router"].update(top=11), "exceeds 'experts'"),
    (lambda r: r["layers"][0]["mlp"]["router"]["groups"].update(count=3), "equal groups"),
    (lambda r: r["layers"][0]["mlp"]["router"]["groups"].update(keep=1), "fewer than"),
    (lambda r: r["layers"][1]["mixer"].update(tau=0.0), "'tau'"),
    (lambda r: r["layers"][1].update(type="conv"), "unknown layer type"),
    (lambda r: r["layers"][1]["mlp"].update(kind="sparse"), "unknown feed-forward kind"),
    (lambda r: r.pop("norm"), "'norm'"),
])
def test_configuration_errors_name_the_key(change, needle):
    raw = copy.deepcopy(MODELS["R"])
    change(raw)
    with pytest.raises(ConfigError) as error:
        config_from_dict(raw)
    assert needle in str(error.value)


def test_layers_that_mix_values_must_agree():
    raw = model(64, 50, 1.0, [attention(4, 2, 16, 16, 0.25, 10.0, 8, v_mix=True),
                              attention(4, 4, 16, 16, 0.25, 10.0, 8, v_mix=True)])
    with pytest.raises(ConfigError) as error:
        config_from_dict(raw)
    assert "agree" in str(error.value)


# ---------------------------------------------------------------------------- the rotary table
@pytest.mark.parametrize("rot", [
    {"dims": 32, "base": 10000.0},
    {"dims": 12, "base": 10000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 3.0, "original": 40}},
    {"dims": 64, "base": 300.0, "scaling": {"factor": 2.0, "low": 2.0, "high": 8.0, "original": 64}},
])
def test_frequency_table_against_the_plain_one(rot):
    layer = attention(2, 2, 64, 64, 0.1, 10.0, rot["dims"], base=rot["base"], scaling=rot.get("scaling"))
    spec = config_from_dict(single_layer(layer)).model_spec().layers[0].mixer.position
    table = wavelength_scaled_frequencies(spec)
    assert torch.allclose(table, plain.rotary_frequencies(rot), rtol=1e-14, atol=0)
    if "scaling" in rot:
        s = rot["scaling"]
        plain_f = torch.tensor([rot["base"] ** (-2.0 * i / rot["dims"]) for i in range(rot["dims"] // 2)], dtype=F64)
        wavelength = 2 * math.pi / plain_f
        kept, slowed = wavelength < s["original"] / s["high"], wavelength > s["original"] / s["low"]
        assert kept.any() and slowed.any() and (~kept & ~slowed).any()      # the table has all three regimes
        assert torch.equal(table[kept], plain_f[kept])
        assert torch.allclose(table[slowed], plain_f[slowed] / s["factor"], rtol=1e-15)
        between = ~kept & ~slowed
        assert (table[between] < plain_f[between]).all() and (table[between] > plain_f[between] / s["factor"]).all()


# ---------------------------------------------------------------------------- properties of the plain model
def _attention_setup(seed=0, T=12):
    layer = attention(4, 2, 16, 8, 0.3, 5.0, 8, v_mix=True)
    raw = single_layer(layer)
    tensors = {k: v.to(F64) for k, v in draw(raw, seed, sharpen=3.0).items()}
    h = torch.randn(T, 64, dtype=F64, generator=torch.Generator().manual_seed(seed))
    return layer["mixer"], tensors, h


def test_plain_attention_is_causal_and_the_sink_takes_weight():
    m, w, h = _attention_setup()
    full, _ = plain.sink_attention(h, w, "l0.mix.", m)
    head, _ = plain.sink_attention(h[:7], w, "l0.mix.", m)
    assert torch.allclose(full[:7], head, atol=1e-12)                 # later tokens change nothing earlier
    # a huge sink swallows the softmax: the output goes to zero; a very negative one is no sink at all
    w_big = dict(w)
    w_big["l0.mix.sink"] = torch.full((4,), 60.0, dtype=F64)
    swallowed, _ = plain.sink_attention(h, w_big, "l0.mix.", m)
    assert swallowed.abs().max() < 1e-6 * full.abs().max()
    w_none = dict(w)
    w_none["l0.mix.sink"] = torch.full((4,), -1e4, dtype=F64)
    without, _ = plain.sink_attention(h, w_none, "l0.mix.", m)
    # token 0 sees only itself: without a sink its weight is exactly one, so the head's output is its gated value
    v = plain.attention_values(h, w, "l0.mix.", m)
    gate = torch.sigmoid(h @ w["l0.mix.g"].T)
    want = (v[0].repeat_interleave(2, dim=0) * gate[0][:, None]).reshape(-1) @ w["l0.mix.o"].T
    assert torch.allclose(without[0], want, atol=1e-10)
    assert not torch.allclose(full[0], want, atol=1e-3)               # with the sink it is scaled down


def test_plain_attention_caps_scores_and_blends_values():
    m, w, h = _attention_setup(seed=3)
    w_loud = dict(w)
    w_loud["l0.mix.q"] = w["l0.mix.q"] * 1e4                          # every score far beyond the cap
    w_loud["l0.mix.q.b"] = w["l0.mix.q.b"] * 1e4
    a, _ = plain.sink_attention(h, w_loud, "l0.mix.", m)
    w_louder = dict(w_loud)
    w_louder["l0.mix.q"] = w["l0.mix.q"] * 1e6
    w_louder["l0.mix.q.b"] = w["l0.mix.q.b"] * 1e6
    b, _ = plain.sink_attention(h, w_louder, "l0.mix.", m)
    assert torch.allclose(a, b, atol=1e-6)                            # saturated: +-cap whatever the size
    other = torch.randn(12, 2, 8, dtype=F64)
    blended, used = plain.sink_attention(h, w, "l0.mix.", m, v_first=other)
    lam = float(w["l0.mix.vmix"])
    assert torch.allclose(used, (1 - lam) * plain.attention_values(h, w, "l0.mix.", m) + lam * other)
    assert not torch.allclose(blended, plain.sink_attention(h, w, "l0.mix.", m)[0], atol=1e-4)


def test_plain_recurrence_equals_its_closed_form():
    layer = gla(2, 8, 6, 3.0)
    raw = single_layer(layer, rank=4)
    w = {k: v.to(F64) for k, v in draw(raw, 5).items()}
    h = torch.randn(9, 64, dtype=F64, generator=torch.Generator().manual_seed(1))
    m, p = layer["mixer"], "l0.mix."
    got = plain.gla(h, w, p, m, 1e-5)
    # o_t = sum_{s <= t} (q_t * prod_{s < r <= t} a_r) . k_s  v_s, then norm, gate and projection
    q = (h @ w[p + "q"].T).view(9, 2, 8) * 8 ** -0.5
    k = (h @ w[p + "k"].T).view(9, 2, 8)
    v = (h @ w[p + "v"].T).view(9, 2, 6)
    a = plain.gla_decay(h, w, p, m)
    assert ((a > 0) & (a < 1)).all()
    o = torch.zeros(9, 2, 6, dtype=F64)
    for t in range(9):
        for s in range(t + 1):
            decay = torch.ones(2, 8, dtype=F64)
            for r in range(s + 1, t + 1):
                decay = decay * a[r]
            o[t] += ((q[t] * decay * k[s]).sum(-1))[:, None] * v[s]
    want = ((plain.rms_unit(o, 1e-5) * w[p + "norm"]).reshape(9, 12) * plain.silu(h @ w[p + "g"].T)) @ w[p + "o"].T
    assert torch.allclose(got, want, atol=1e-10)


def test_plain_routing_keeps_the_best_groups_only():
    r = {"experts": 8, "top": 3, "groups": {"count": 4, "keep": 2}, "scale": 2.0}
    router = torch.eye(8, dtype=F64)
    # scores: group 0 = (.9, .1), group 1 = (.6, .6), group 2 = (.8, .5), group 3 = (.7, .2): worth 1.0, 1.2, 1.3, 0.9
    score = torch.tensor([[0.9, 0.1, 0.6, 0.6, 0.8, 0.5, 0.7, 0.2]], dtype=F64)
    h = torch.log(score / (1 - score))
    chosen, weights = plain.route(h, router, r)
    assert sorted(chosen[0].tolist()) == [2, 3, 4]                     # 0.9 and 0.7 sit in groups that lost
    assert torch.allclose(weights.sum(), torch.tensor(2.0, dtype=F64))
    picked = score[0, chosen[0]]
    assert torch.allclose(weights[0], picked / picked.sum() * 2.0)
    # groups of one expert are worth that expert's score
    r1 = {"experts": 8, "top": 2, "groups": {"count": 8, "keep": 3}, "scale": 1.0}
    chosen, _ = plain.route(h, router, r1)
    assert sorted(chosen[0].tolist()) == [0, 4]


def test_plain_model_is_independent_of_what_follows():
    raw = MODELS["P"]
    tensors = draw(raw, 2, sharpen=2.0)
    tokens = ids(30, raw["vocab"], 4)
    whole = plain.forward(raw, tensors, tokens)
    assert torch.allclose(plain.forward(raw, tensors, tokens[:11]), whole[:11], atol=1e-10)
    # the embedding scale, the first layer's mixing scalar (unused) and a blending layer's (used)
    scaled = copy.deepcopy(raw)
    scaled["embedding"]["scale"] = 1.0
    assert not torch.allclose(plain.forward(scaled, tensors, tokens), whole, atol=1e-3)
    unused = dict(tensors)
    unused["l1.mix.vmix"] = torch.tensor(0.99)
    assert torch.equal(plain.forward(raw, unused, tokens), whole)
    used = dict(tensors)
    used["l4.mix.vmix"] = torch.tensor(0.99)
    assert not torch.allclose(plain.forward(raw, used, tokens), whole, atol=1e-4)


def test_benchmark_configurations_describe_runnable_models():
    """The sizes ``bench.py --compare parunex`` times: they parse, name every tensor once, and plan one cache group
    and a state per recurrent layer."""
    import bench

    for size in bench.COMPARE_SIZES.values():
        config = config_from_dict(bench.parunex_config(size))
        spec = config.model_spec()
        names = [s.name for s in model_weight_specs(spec)]
        assert len(names) == len(set(names))
        plan = plan_cache(spec)
        assert len(plan.groups) == 1 and plan.groups[0].request.head_dim == 128
        assert sum(s is not None for s in plan.state_of_entry) == bench.COMPARE_LAYERS // 2


def test_tensors_that_lie_unused_in_a_model_folder_are_expected():
    """A mixing scalar of a layer that does not mix and the second norm of a layer without a feed-forward may be
    in a file: the configuration learns of them from the tensors and the weight check lets them pass."""
    raw = MODELS["P"]
    tensors = draw(raw, 1)
    config = config_from_dict(copy.deepcopy(raw))
    extra = dict(tensors)
    extra["l2.mix.vmix"] = torch.tensor(0.5)
    extra["l2.norm2"] = torch.ones(96)
    extra["l2.norm2.b"] = torch.zeros(96)
    extra["l2.norm2.alpha"] = torch.tensor(1.0)
    with pytest.raises(WeightLoadError):
        check_weights(model_weight_specs(config.model_spec()), DictSource(extra))
    shaped = config.with_tensor_shapes(lambda name: tuple(extra[name].shape) if name in extra else None)
    assert {name for name, _ in shaped.unused_tensors} == {"l2.mix.vmix", "l2.norm2", "l2.norm2.b", "l2.norm2.alpha"}
    check_weights(model_weight_specs(shaped.model_spec()), DictSource(extra))
    # without them in the file nothing is expected
    plain_shapes = config.with_tensor_shapes(lambda name: tuple(tensors[name].shape) if name in tensors else None)
    assert plain_shapes.unused_tensors == ()
    check_weights(model_weight_specs(plain_shapes.model_spec()), DictSource(tensors))
