"""Small Busatar configurations of the tests (sizes, orders and constants of their own) and helpers that
draw their weights. ``sharpen`` scales the tensors that set attention scores, so that softmax weights
concentrate on single keys and a key wrongly seen or missed moves the logits."""

from __future__ import annotations

import copy

import torch

from matricxon_b200.config.registry import config_from_dict
from matricxon_b200.weights.random_init import RandomInit, random_tensors


def latent(heads, dim, rot_dim, rank, vdim, window, scale, scaling=None, base=5000.0, ff=None, limit=2.0):
    rot = {"base": base, "dims": rot_dim}
    if scaling is not None:
        rot["scaling"] = scaling
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "kv_rank": rank, "vdim": vdim,
                      "mask": {"size": window}, "scale": scale, "rot": rot},
            "mlp": {"kind": "dense", "ff": ff, "limit": limit} if ff else None}


def gated(heads, kv_heads, dim, vdim, window, scale, ff=None, limit=2.0):
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window},
                      "scale": scale},
            "mlp": {"kind": "dense", "ff": ff, "limit": limit} if ff else None}


def recurrent(width, blocks, conv, ff=None, limit=2.0):
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": conv},
            "mlp": {"kind": "dense", "ff": ff, "limit": limit} if ff else None}


def model(width, vocab, alpha, eps, layers):
    return {"architecture": "Busatar", "width": width, "vocab": vocab, "postln_alpha": alpha,
            "norm": {"eps": eps}, "layers": layers}


STRETCH = {"factor": 4.0, "original": 48, "fast": 8.0, "slow": 2.0}

# every kind, a recurrence first and last, odd head sizes, a window longer than any test sequence, a layer
# without feed-forward of each attention kind, value width above and below the key width
MODEL_X = model(96, 300, 1.5, 1e-6, [
    recurrent(80, 5, 3, ff=160, limit=0.7),
    latent(3, 24, 16, 40, 20, window=20, scale=0.2, scaling=STRETCH, ff=112, limit=1.0),
    gated(4, 2, 16, 24, window=37, scale=0.3),
    latent(2, 16, 8, 24, 16, window=500, scale=0.25),
    gated(2, 2, 40, 8, window=9, scale=0.2, ff=64),
    recurrent(48, 1, 1),
])

# head sizes that the tensor-core attention kernels take (64), a group of four query heads per key head,
# a wide latent, windows that are page multiples and one of a single token
MODEL_Y = model(128, 257, 3.0, 1e-5, [
    latent(4, 32, 32, 64, 32, window=32, scale=0.125, scaling={"factor": 16.0, "original": 32, "fast": 4.0, "slow": 1.0}, ff=256),
    gated(4, 1, 64, 64, window=33, scale=0.125, ff=128, limit=5.0),
    recurrent(128, 4, 4, ff=96),
    gated(2, 2, 64, 64, window=1, scale=0.125),
    latent(9, 16, 16, 136, 16, window=16, scale=0.3, ff=64),
])

# sizes that are multiples of nothing useful: width 100, odd vocabulary, heads of 12 and 20, a rotated part of
# 6, a latent of 20, three blocks of 20 channels, two taps
MODEL_Z = model(100, 131, 2.0, 1e-5, [
    latent(5, 12, 6, 20, 10, window=40, scale=0.3, scaling={"factor": 2.0, "original": 24, "fast": 3.0, "slow": 1.5}, ff=52),
    recurrent(60, 3, 2),
    gated(6, 3, 20, 12, window=50, scale=0.25, ff=76, limit=1.2),
])

# a middle size for long prompts: products of more than a thousand rows, tensor-core latent attention
# (latent 64, key 96), 128-wide attention heads in a group of two, a recurrence in many chunks
MODEL_W = model(256, 640, 2.0, 1e-5, [
    latent(4, 48, 32, 64, 48, window=200, scale=0.11, scaling={"factor": 8.0, "original": 512, "fast": 32.0, "slow": 1.0}, ff=512),
    gated(4, 2, 128, 128, window=150, scale=0.09, ff=384),
    recurrent(192, 3, 4, ff=256),
    latent(2, 64, 16, 128, 32, window=1500, scale=0.1),
])

MODELS = {"X": MODEL_X, "Y": MODEL_Y, "Z": MODEL_Z, "W": MODEL_W}
INIT = RandomInit(weight_std=0.08, bias_std=0.3, norm_weight_std=0.1, norm_bias_std=0.1)


def single_layer(layer: dict, width=64, vocab=120, alpha=2.0, eps=1e-5) -> dict:
    return model(width, vocab, alpha, eps, [copy.deepcopy(layer)])


def draw(raw: dict, seed: int, sharpen: float = 1.0, store_dtype=torch.float32) -> dict[str, torch.Tensor]:
    tensors = random_tensors(config_from_dict(copy.deepcopy(raw)), seed, INIT, store_dtype)
    if sharpen != 1.0:
        for name in tensors:
            if name.endswith(".mix.q") or name.endswith(".mix.q.norm"):
                tensors[name] = (tensors[name].float() * sharpen).to(store_dtype)
    return tensors


def ids(count: int, vocab: int, seed: int) -> list[int]:
    generator = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (count,), generator=generator).tolist()
