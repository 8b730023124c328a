"""A plain, slow Busatar: every mechanism as one function of float64 tensors, one sequence at a time.

This is the yardstick the engine's Busatar parts are compared with. It shares no code with the
package: it takes a configuration as the plain dictionary that ``config.json`` holds and weights as
a name -> tensor dictionary, keeps no cache (every call sees the whole sequence) and runs on the CPU.

Notation: h is a [T, width] matrix of one sequence's sublayer inputs, positions count from 0.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_around_zero(x, weight, eps):
    """RMS norm whose stored weight is the distance of the scale from one."""
    return rms_unit(x, eps) * (1.0 + weight)


def norm_plain(x, weight, eps):
    return rms_unit(x, eps) * weight


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotary_table(rot: dict) -> tuple[torch.Tensor, float]:
    """(frequency per pair [dims/2], factor on cos and sin) of a rotary description, with the
    frequency interpolation between a fast and a slow wavelength when ``scaling`` is given."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    scaling = rot.get("scaling")
    if not scaling:
        return freq, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def turning_dim(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turning_dim(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turning_dim(float(scaling["slow"]))), dims - 1)
    ramp = torch.tensor([min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(half)], dtype=F64)
    return freq / factor * ramp + freq * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_half_pairs(x: torch.Tensor, positions: torch.Tensor, rot: dict) -> torch.Tensor:
    """x [..., T, n]: the first ``dims`` entries are rotated, pair (i, i + dims/2); the rest pass."""
    dims = int(rot["dims"])
    half = dims // 2
    freq, factor = rotary_table(rot)
    angle = positions.to(F64)[:, None] * freq[None, :]
    cos, sin = torch.cos(angle) * factor, torch.sin(angle) * factor
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


def window_mask(t: int, size: int) -> torch.Tensor:
    i = torch.arange(t)[:, None]
    j = torch.arange(t)[None, :]
    return (i - j >= 0) & (i - j < size)


def softmax_attention(q, k, v, scale: float, size: int) -> torch.Tensor:
    """q [H, T, d], k [H, T, d], v [H, T, e] -> [T, H * e]."""
    t = q.shape[1]
    scores = torch.einsum("htd,hsd->hts", q, k) * scale
    scores = scores.masked_fill(~window_mask(t, size)[None], float("-inf"))
    out = torch.einsum("hts,hse->hte", torch.softmax(scores, dim=-1), v)
    return out.transpose(0, 1).reshape(t, -1)


def latent_attention(h, w: dict, m: dict, eps: float) -> torch.Tensor:
    t = h.shape[0]
    heads, dim, rot_dim, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    positions = torch.arange(t)
    q = (h @ w["q"].T).view(t, heads, dim + rot_dim).transpose(0, 1)
    down = h @ w["dkv"].T
    latent = norm_plain(down[:, :rank], w["dkv.norm"], eps)
    shared = rotate_half_pairs(down[:, rank:], positions, m["rot"])
    q_plain, q_rot = q[..., :dim], rotate_half_pairs(q[..., dim:], positions, m["rot"])
    k_plain = (latent @ w["uk"].T).view(t, heads, dim).transpose(0, 1)
    values = (latent @ w["uv"].T).view(t, heads, vdim).transpose(0, 1)
    keys = torch.cat([k_plain, shared[None].expand(heads, t, rot_dim)], dim=-1)
    queries = torch.cat([q_plain, q_rot], dim=-1)
    mixed = softmax_attention(queries, keys, values, float(m["scale"]), int(m["mask"]["size"]))
    return mixed @ w["o"].T


def gated_attention(h, w: dict, m: dict, eps: float) -> torch.Tensor:
    t = h.shape[0]
    heads, kv_heads, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = norm_plain((h @ w["q"].T).view(t, heads, dim), w["q.norm"], eps).transpose(0, 1)
    k = norm_plain((h @ w["k"].T).view(t, kv_heads, dim), w["k.norm"], eps).transpose(0, 1)
    v = (h @ w["v"].T).view(t, kv_heads, vdim).transpose(0, 1)
    share = heads // kv_heads
    k = k.repeat_interleave(share, dim=0)
    v = v.repeat_interleave(share, dim=0)
    mixed = softmax_attention(q, k, v, float(m["scale"]), int(m["mask"]["size"]))
    return (mixed * torch.sigmoid(h @ w["g"].T)) @ w["o"].T


def causal_taps(x, taps_weight, taps_bias) -> torch.Tensor:
    """x [T, C], taps_weight [C, n]: the last column multiplies the current token, zeros before the start."""
    t, n = x.shape[0], taps_weight.shape[1]
    padded = torch.cat([torch.zeros(n - 1, x.shape[1], dtype=x.dtype), x])
    out = taps_bias[None].expand(t, -1).clone()
    for k in range(n):
        out = out + padded[k:k + t] * taps_weight[:, k][None]
    return out


def gated_recurrence(h, w: dict, m: dict) -> torch.Tensor:
    t, width, blocks = h.shape[0], m["width"], m["blocks"]
    y = gelu_tanh(h @ w["y"].T + w["y.b"])
    u = causal_taps(h @ w["x"].T + w["x.b"], w["conv"], w["conv.b"])
    parts = u.view(t, blocks, width // blocks)
    r = torch.sigmoid(torch.einsum("tbi,boi->tbo", parts, w["ra"]) + w["ra.b"][None]).reshape(t, width)
    i = torch.sigmoid(torch.einsum("tbi,boi->tbo", parts, w["ri"]) + w["ri.b"][None]).reshape(t, width)
    log_a = -8.0 * r * torch.nn.functional.softplus(w["lam"])[None]
    a = torch.exp(log_a)
    drive = torch.sqrt(1.0 - a * a) * i * u
    state = torch.zeros(width, dtype=h.dtype)
    states = []
    for step in range(t):
        state = a[step] * state + drive[step]
        states.append(state)
    return (torch.stack(states) * y) @ w["o"].T


def clamped_gated_ff(h, w: dict, f: dict) -> torch.Tensor:
    limit = float(f["limit"])
    g = torch.clamp(h @ w["gate"].T, max=limit)
    u = torch.clamp(h @ w["up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w["down"].T


MIXERS = {"latent_attention": lambda h, w, m, eps: latent_attention(h, w, m, eps),
          "attention": lambda h, w, m, eps: gated_attention(h, w, m, eps),
          "rglru": lambda h, w, m, eps: gated_recurrence(h, w, m)}


def sub(weights: dict, prefix: str) -> dict:
    return {name[len(prefix):]: tensor.to(F64) for name, tensor in weights.items() if name.startswith(prefix)}


def forward(config: dict, weights: dict, tokens: list[int], layer_outputs: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] (float64) of one sequence; ``layer_outputs`` collects x after every layer."""
    eps, alpha = float(config["norm"]["eps"]), float(config["postln_alpha"])
    x = weights["embed"].to(F64)[torch.tensor(tokens, dtype=torch.long)]
    for index, layer in enumerate(config["layers"]):
        prefix = f"l{index}."
        mixed = MIXERS[layer["type"]](x, sub(weights, prefix + "mix."), layer["mixer"], eps)
        x = norm_around_zero(alpha * x + mixed, weights[prefix + "norm1"].to(F64), eps)
        if layer.get("mlp") is not None:
            fed = clamped_gated_ff(x, sub(weights, prefix + "mlp."), layer["mlp"])
            x = norm_around_zero(alpha * x + fed, weights[prefix + "norm2"].to(F64), eps)
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    x = norm_around_zero(x, weights["final.norm"].to(F64), eps)
    return x @ weights["head"].to(F64).T
