"""Small Parunex configurations of the tests (sizes, orders and constants of their own) and helpers that draw
their weights. ``sharpen`` scales the query projections, so that softmax weights concentrate on single keys and
a key wrongly seen or missed moves the logits."""

from __future__ import annotations

import copy

import torch

from matricxon_b200.config.registry import config_from_dict
from matricxon_b200.weights.random_init import RandomInit, random_tensors


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top, count, keep, scale=1.0):
    return {"kind": "moe", "expert": {"ff": ff},
            "router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}, "scale": scale}}


def attention(heads, kv_heads, dim, vdim, scale, softcap, rot_dims, v_mix=False, base=10000.0, scaling=None, mlp=None):
    rot = {"base": base, "dims": rot_dims}
    if scaling is not None:
        rot["scaling"] = scaling
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
                      "softcap": softcap, "v_mix": v_mix, "rot": rot},
            "mlp": mlp}


def gla(heads, dim, vdim, tau, mlp=None):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}, "mlp": mlp}


def model(width, vocab, embedding_scale, layers, ranks=None, eps=1e-5):
    raw = {"architecture": "Parunex", "width": width, "vocab": vocab, "embedding": {"scale": embedding_scale},
           "norm": {"eps": eps}, "layers": layers}
    if ranks is not None:
        raw["decay_ranks"] = ranks
    return raw


STRETCH = {"factor": 8.0, "low": 1.0, "high": 3.0, "original": 40}

# a recurrence first, attention without a feed-forward, odd head sizes, value width above and below the key
# width, the second mixing layer several layers after the first, a router whose groups are single experts and
# one that keeps every group, a decay rank of 5
MODEL_P = model(96, 300, 3.0, [
    gla(3, 24, 40, 4.0, mlp=moe(56, 6, 2, 6, 3, scale=1.5)),
    attention(6, 3, 24, 16, 0.3, 7.0, 12, v_mix=True, scaling=STRETCH, mlp=dense(136)),
    attention(4, 1, 40, 8, 0.2, 20.0, 40, mlp=None),
    gla(2, 56, 16, 9.0, mlp=dense(72)),
    attention(3, 3, 16, 16, 0.35, 4.0, 8, v_mix=True, base=300.0, mlp=moe(40, 8, 3, 2, 2, scale=0.7)),
], ranks=[5, 0, 0, 8, 0])

# head sizes that the tensor-core attention kernels take (64 and 128), groups of four and two query heads, all
# layers mixing values, a top-1 router, rotation over the whole head and over none of it
MODEL_Q = model(128, 257, 1.0, [
    attention(8, 2, 64, 64, 0.125, 30.0, 64, v_mix=True, mlp=moe(96, 4, 1, 2, 1, scale=2.5)),
    gla(2, 64, 64, 12.0, mlp=None),
    attention(4, 2, 128, 64, 0.09, 10.0, 0, v_mix=True, mlp=dense(256)),
    attention(2, 2, 64, 64, 0.125, 45.0, 16, v_mix=True, scaling={"factor": 2.0, "low": 2.0, "high": 8.0,
                                                                  "original": 64}, mlp=None),
    gla(1, 128, 32, 2.0, mlp=moe(64, 9, 4, 3, 2)),
], ranks=[0, 32, 0, 0, 3])

# sizes that are multiples of nothing useful: width 100, odd vocabulary, heads of 12 and 20, six rotated entries
MODEL_R = model(100, 131, 7.5, [
    attention(5, 5, 12, 20, 0.3, 15.0, 6, mlp=moe(52, 10, 3, 5, 4, scale=1.2)),
    gla(5, 20, 12, 3.0, mlp=dense(76)),
], ranks=[0, 7])

# a middle size for long prompts: products of more than a thousand rows, 128-wide heads in a group of two
MODEL_S = model(256, 640, 2.0, [
    attention(4, 2, 128, 128, 0.09, 25.0, 64, v_mix=True, scaling={"factor": 6.0, "low": 1.0, "high": 3.0,
                                                                   "original": 256}, mlp=moe(128, 8, 2, 4, 2, 1.5)),
    gla(4, 64, 64, 8.0, mlp=dense(384)),
    attention(4, 2, 128, 128, 0.09, 25.0, 64, v_mix=True, mlp=dense(256)),
], ranks=[0, 24, 0])

MODELS = {"P": MODEL_P, "Q": MODEL_Q, "R": MODEL_R, "S": MODEL_S}
INIT = RandomInit(weight_std=0.08, bias_std=0.3, norm_weight_std=0.1, norm_bias_std=0.1)


def single_layer(layer: dict, width=64, vocab=120, embedding_scale=4.0, rank=None) -> dict:
    return model(width, vocab, embedding_scale, [copy.deepcopy(layer)], ranks=None if rank is None else [rank])


def draw(raw: dict, seed: int, sharpen: float = 1.0, store_dtype=torch.float32) -> dict[str, torch.Tensor]:
    """Random weights with norms' alphas, mixing scalars and sinks away from the values that hide them."""
    tensors = random_tensors(config_from_dict(copy.deepcopy(raw)), seed, INIT, store_dtype)
    generator = torch.Generator().manual_seed(seed + 1)
    for name in tensors:
        if name.endswith(".mix.q"):
            tensors[name] = (tensors[name].float() * sharpen).to(store_dtype)
        elif name.endswith(".alpha"):
            tensors[name] = torch.tensor(0.3 + 0.4 * torch.rand((), generator=generator).item()).to(store_dtype)
        elif name.endswith(".mix.vmix"):
            tensors[name] = torch.tensor(0.2 + 0.5 * torch.rand((), generator=generator).item()).to(store_dtype)
        elif name.endswith(".mix.sink"):
            tensors[name] = (torch.randn(tensors[name].shape, generator=generator) * 1.5 + 1.0).to(store_dtype)
        elif name.endswith(".mlp.router"):
            tensors[name] = (tensors[name].float() * 6.0).to(store_dtype)      # scores away from one another
        elif name == "head":
            tensors[name] = (tensors[name].float() * 5.0).to(store_dtype)      # logits of a few units
        elif name.endswith(".mix.a2.b"):
            tensors[name] = (torch.randn(tensors[name].shape, generator=generator) + 2.0).to(store_dtype)
    return tensors


def ids(count: int, vocab: int, seed: int) -> list[int]:
    generator = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (count,), generator=generator).tolist()
