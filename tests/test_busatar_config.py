"""Busatar on the CPU: configuration, names, registry, the rotary table, and the plain implementation's
own mechanisms checked against what they must satisfy by construction."""

import copy
import math

import pytest
import torch

import plain_busatar as plain
from busatar_configs import MODEL_X, MODEL_Y, draw, gated, ids, latent, recurrent, single_layer
from matricxon_b200.config.base import ConfigError
from matricxon_b200.config.busatar import BusatarConfig
from matricxon_b200.config.registry import config_from_dict, resolve_architecture
from matricxon_b200.models.decoder import model_weight_specs, plan_cache
from matricxon_b200.parts.rotary import interpolated_frequencies
from matricxon_b200.parts.spec import InterpolatedRotarySpec


def test_registry_reads_the_architecture_key():
    assert resolve_architecture({"architecture": "Busatar"}).config_class is BusatarConfig
    config = config_from_dict(copy.deepcopy(MODEL_X))
    assert isinstance(config, BusatarConfig) and config.vocab_size == 300
    assert config.to_dict() == MODEL_X
    assert config_from_dict(config.to_dict()) == config


@pytest.mark.parametrize("raw", [MODEL_X, MODEL_Y])
def test_tensor_names_and_shapes(raw):
    config = config_from_dict(copy.deepcopy(raw))
    specs = {s.name: s.shape for s in model_weight_specs(config.model_spec())}
    assert specs["embed"] == (raw["vocab"], raw["width"]) and specs["head"] == (raw["vocab"], raw["width"])
    assert specs["final.norm"] == (raw["width"],)
    for i, layer in enumerate(raw["layers"]):
        m = layer["mixer"]
        assert f"l{i}.norm1" in specs
        assert (f"l{i}.norm2" in specs) == (layer["mlp"] is not None)
        assert (f"l{i}.mlp.gate" in specs) == (layer["mlp"] is not None)
        if layer["type"] == "latent_attention":
            assert specs[f"l{i}.mix.q"] == (m["heads"] * (m["dim"] + m["rot_dim"]), raw["width"])
            assert specs[f"l{i}.mix.dkv"] == (m["kv_rank"] + m["rot_dim"], raw["width"])
            assert specs[f"l{i}.mix.dkv.norm"] == (m["kv_rank"],)
            assert specs[f"l{i}.mix.uk"] == (m["heads"] * m["dim"], m["kv_rank"])
            assert specs[f"l{i}.mix.uv"] == (m["heads"] * m["vdim"], m["kv_rank"])
            assert specs[f"l{i}.mix.o"] == (raw["width"], m["heads"] * m["vdim"])
        elif layer["type"] == "attention":
            assert specs[f"l{i}.mix.k"] == (m["kv_heads"] * m["dim"], raw["width"])
            assert specs[f"l{i}.mix.v"] == (m["kv_heads"] * m["vdim"], raw["width"])
            assert specs[f"l{i}.mix.g"] == (m["heads"] * m["vdim"], raw["width"])
            assert specs[f"l{i}.mix.q.norm"] == (m["dim"],) and specs[f"l{i}.mix.k.norm"] == (m["dim"],)
        else:
            block = m["width"] // m["blocks"]
            assert specs[f"l{i}.mix.conv"] == (m["width"], m["conv"])
            assert specs[f"l{i}.mix.ra"] == (m["blocks"], block, block)
            assert specs[f"l{i}.mix.ri.b"] == (m["blocks"], block)
            assert specs[f"l{i}.mix.y.b"] == (m["width"],) and specs[f"l{i}.mix.lam"] == (m["width"],)


def test_cache_plan_one_plane_for_latents_and_state_for_recurrences():
    config = config_from_dict(copy.deepcopy(MODEL_X))
    plan = plan_cache(config.model_spec())
    kinds = [layer["type"] for layer in MODEL_X["layers"]]
    for position, kind in enumerate(kinds):
        assert (plan.state_of_entry[position] is not None) == (kind == "rglru")
        assert (plan.kv_of_entry[position] is not None) == (kind != "rglru")
    requests = {group.request for group in plan.groups}
    assert {r.planes for r in requests if r.num_kv_heads == 1 and r.head_dim in (56, 32)} == {1}
    assert plan.state_of_entry[0].shape == (3, 80) and plan.state_of_entry[5].shape == (1, 48)
    # the gated attention's heads are padded to a common multiple of 16 for keys and values
    assert any(r.planes == 2 and r.head_dim == 32 and r.window == 37 for r in requests)
    assert any(r.planes == 2 and r.head_dim == 48 and r.window == 9 for r in requests)


@pytest.mark.parametrize("broken, message", [
    (lambda c: c["layers"][0].update(type="mamba"), "unknown layer type"),
    (lambda c: c["layers"][2]["mixer"].update(kv_heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mixer"].update(blocks=7), "multiple of blocks"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=18), "exceeds rot_dim"),
    (lambda c: c["layers"][1]["mlp"].update(kind="routed"), "feed-forward kind"),
    (lambda c: c.pop("postln_alpha"), "postln_alpha"),
    (lambda c: c["layers"][1]["mixer"].pop("mask"), "mask"),
])
def test_config_errors_name_the_key(broken, message):
    raw = copy.deepcopy(MODEL_X)
    broken(raw)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(raw)


@pytest.mark.parametrize("rot", [
    {"dims": 16, "base": 5000.0, "scaling": {"factor": 4.0, "original": 48, "fast": 8.0, "slow": 2.0}},
    {"dims": 32, "base": 250000.0, "scaling": {"factor": 16.0, "original": 4096, "fast": 32.0, "slow": 1.0}},
    {"dims": 8, "base": 100.0},
])
def test_rotary_table_matches_the_plain_one(rot):
    scaling = rot.get("scaling", {})
    spec = InterpolatedRotarySpec(rotary_dim=rot["dims"], theta=rot["base"], factor=scaling.get("factor"),
                                  original=scaling.get("original", 0.0), fast=scaling.get("fast", 32.0),
                                  slow=scaling.get("slow", 1.0))
    table, amplitude = interpolated_frequencies(spec)
    want, want_amplitude = plain.rotary_table(rot)
    assert torch.allclose(table, want, rtol=1e-14, atol=0) and amplitude == pytest.approx(want_amplitude, rel=1e-15)
    if scaling:
        plain_freq = torch.tensor([rot["base"] ** (-2.0 * i / rot["dims"]) for i in range(rot["dims"] // 2)],
                                  dtype=torch.float64)
        assert torch.all(table <= plain_freq * (1 + 1e-12)) and torch.all(table >= plain_freq / scaling["factor"] * (1 - 1e-12))
        assert table[0] == plain_freq[0]                      # the fastest pair keeps its frequency
        assert amplitude == pytest.approx(0.1 * math.log(scaling["factor"]) + 1.0)


def test_plain_window_and_prefix_property():
    """What the plain implementation computes for a prefix does not change when tokens are appended, and a
    token beyond every window and without recurrence does not reach a later position."""
    raw = single_layer(gated(2, 1, 16, 8, window=5, scale=0.4), width=32)
    weights = draw(raw, seed=3)
    tokens = ids(30, raw["vocab"], seed=4)
    full = plain.forward(raw, weights, tokens)
    assert torch.allclose(plain.forward(raw, weights, tokens[:17]), full[:17], rtol=0, atol=1e-12)
    changed = list(tokens)
    changed[10] = (changed[10] + 1) % raw["vocab"]
    other = plain.forward(raw, weights, changed)
    assert torch.allclose(other[15:], full[15:], rtol=0, atol=1e-12)        # 15 - 10 = 5: just outside
    assert not torch.allclose(other[14], full[14], rtol=0, atol=1e-9)       # 14 - 10 = 4: just inside


def test_plain_recurrence_carries_the_first_token_and_the_taps_reach_back():
    raw = single_layer(recurrent(32, 2, 3), width=32)
    weights = draw(raw, seed=5)
    tokens = ids(40, raw["vocab"], seed=6)
    full = plain.forward(raw, weights, tokens)
    changed = list(tokens)
    changed[0] = (changed[0] + 1) % raw["vocab"]
    assert not torch.allclose(plain.forward(raw, weights, changed)[6], full[6], rtol=0, atol=1e-12)   # beyond the taps
    x = torch.randn(6, 4, dtype=torch.float64)
    taps = torch.randn(4, 3, dtype=torch.float64)
    out = plain.causal_taps(x, taps, torch.zeros(4, dtype=torch.float64))
    assert torch.allclose(out[0], x[0] * taps[:, 2]) and torch.allclose(
        out[2], x[2] * taps[:, 2] + x[1] * taps[:, 1] + x[0] * taps[:, 0])


def test_plain_latent_attention_equals_its_folded_form():
    """Scores through expanded keys equal scores of the query folded through the key expansion against the
    latent itself: the identity the engine's kernel rests on."""
    layer = latent(3, 8, 4, 12, 6, window=7, scale=0.3, scaling={"factor": 2.0, "original": 16, "fast": 4.0, "slow": 1.0})
    m = layer["mixer"]
    torch.manual_seed(0)
    h = torch.randn(11, 20, dtype=torch.float64)
    w = {"q": torch.randn(3 * 12, 20), "dkv": torch.randn(16, 20), "dkv.norm": torch.rand(12) + 0.5,
         "uk": torch.randn(24, 12), "uv": torch.randn(18, 12), "o": torch.randn(20, 18)}
    w = {k: v.to(torch.float64) for k, v in w.items()}
    want = plain.latent_attention(h, w, m, 1e-5)
    t = h.shape[0]
    positions = torch.arange(t)
    q = (h @ w["q"].T).view(t, 3, 12)
    down = h @ w["dkv"].T
    c = plain.norm_plain(down[:, :12], w["dkv.norm"], 1e-5)
    shared = plain.rotate_half_pairs(down[:, 12:], positions, m["rot"])
    folded = torch.einsum("thd,hdr->thr", q[..., :8], w["uk"].view(3, 8, 12))
    q_rot = plain.rotate_half_pairs(q[..., 8:].transpose(0, 1), positions, m["rot"]).transpose(0, 1)
    scores = (torch.einsum("thr,sr->hts", folded, c) + torch.einsum("thd,sd->hts", q_rot, shared)) * m["scale"]
    scores = scores.masked_fill(~plain.window_mask(t, 7)[None], float("-inf"))
    mixed = torch.einsum("hts,sr->thr", torch.softmax(scores, -1), c)
    out = torch.einsum("thr,her->the", mixed, w["uv"].view(3, 6, 12)).reshape(t, -1) @ w["o"].T
    assert torch.allclose(out, want, rtol=1e-10, atol=1e-10)
