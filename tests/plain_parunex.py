"""A plain, slow Parunex: every mechanism as one function of float64 tensors, one sequence at a time.

This is the yardstick the engine's Parunex parts are compared with. It shares no code with the
package: it takes a configuration as the plain dictionary that ``config.json`` holds and weights as
a name -> tensor dictionary, keeps no cache and no state (every call sees the whole sequence) and
runs on the CPU.

Notation: h is a [T, width] matrix of one sequence's sublayer inputs, positions count from 0.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def dynamic_tanh(x, weight, shift, alpha):
    """The norm without statistics: every entry squashed on its own, then scaled and shifted."""
    return torch.tanh(float(alpha) * x) * weight + shift


def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


# ---------------------------------------------------------------------------- rotary positions
def rotary_frequencies(rot: dict) -> torch.Tensor:
    """Radians per position of every pair [dims/2]. With ``scaling``: a pair whose wavelength is shorter
    than original/high keeps its frequency, one longer than original/low turns ``factor`` times slower,
    and the pairs between are blended by where original/wavelength lies between low and high."""
    dims, base = int(rot["dims"]), float(rot["base"])
    out = []
    scaling = rot.get("scaling")
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling:
            factor, low, high = float(scaling["factor"]), float(scaling["low"]), float(scaling["high"])
            original = float(scaling["original"])
            wavelength = 2.0 * math.pi / f
            if wavelength < original / high:
                pass
            elif wavelength > original / low:
                f = f / factor
            else:
                s = (original / wavelength - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=F64)


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: dict) -> torch.Tensor:
    """x [T, heads, n]: entry i < dims/2 of every head is paired with entry i + dims/2; the entries from
    ``dims`` on pass unchanged."""
    dims = int(rot["dims"])
    half = dims // 2
    if half == 0:
        return x
    angle = positions.to(F64)[:, None] * rotary_frequencies(rot)[None, :]        # [T, half]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, x[..., dims:]], dim=-1)


# ---------------------------------------------------------------------------- attention with a sink
def attention_values(h, w: dict, p: str, m: dict) -> torch.Tensor:
    """The layer's own values [T, kv heads, vdim], before any mixing."""
    return (h @ w[p + "v"].T + w[p + "v.b"]).view(h.shape[0], int(m["kv_heads"]), int(m["vdim"]))


def sink_attention(h, w: dict, p: str, m: dict, v_first=None):
    """Causal grouped-query attention with capped scores, a keyless sink in the softmax's denominator,
    values blended with ``v_first`` (when given) and one sigmoid gate per head. Returns (output, the
    values that were attended over)."""
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    positions = torch.arange(T)
    q = rotate((h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, d), positions, m["rot"])
    k = rotate((h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, d), positions, m["rot"])
    v = attention_values(h, w, p, m)
    if v_first is not None:
        lam = float(w[p + "vmix"])
        v = (1.0 - lam) * v + lam * v_first
    gate = torch.sigmoid(h @ w[p + "g"].T)                                         # [T, H]
    cap = float(m["softcap"])
    visible = positions[None, :] <= positions[:, None]                             # [query, key]
    out = torch.zeros(T, H, dv, dtype=F64)
    for head in range(H):
        g = head // (H // G)
        score = (q[:, head] @ k[:, g].T) * float(m["scale"])
        score = cap * torch.tanh(score / cap)
        score = score.masked_fill(~visible, -math.inf)
        sink = w[p + "sink"][head]
        top = torch.maximum(score.max(dim=-1).values, sink)
        e = torch.exp(score - top[:, None])
        weights = e / (e.sum(dim=-1) + torch.exp(sink - top))[:, None]
        out[:, head] = (weights @ v[:, g]) * gate[:, head:head + 1]
    return out.reshape(T, H * dv) @ w[p + "o"].T, v


# ---------------------------------------------------------------------------- gated linear attention
def gla_decay(h, w: dict, p: str, m: dict) -> torch.Tensor:
    """The decay of every key channel [T, heads, dim]: a low-rank map, a sigmoid, the tau-th root."""
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    return (torch.sigmoid(z) ** (1.0 / float(m["tau"]))).view(h.shape[0], int(m["heads"]), int(m["dim"]))


def gla(h, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ w[p + "q"].T).view(T, H, d) * d ** -0.5
    k = (h @ w[p + "k"].T).view(T, H, d)
    v = (h @ w[p + "v"].T).view(T, H, dv)
    decay = gla_decay(h, w, p, m)
    state = torch.zeros(H, d, dv, dtype=F64)
    out = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        state = decay[t][:, :, None] * state + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hde,hd->he", state, q[t])
    out = rms_unit(out, eps) * w[p + "norm"]
    return (out.reshape(T, H * dv) * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


# ---------------------------------------------------------------------------- feed-forwards
def gated_ff(h, gate, up, down, act):
    return (act(h @ gate.T) * (h @ up.T)) @ down.T


def route(h, router_weight, r: dict):
    """(chosen experts [T, top], their weights [T, top]). Scores are sigmoids of the router's logits; the
    experts form ``groups.count`` runs of neighbours, a run is worth the sum of its two best scores, and
    only the ``groups.keep`` best runs may supply experts."""
    T = h.shape[0]
    E, top = int(r["experts"]), int(r["top"])
    count, keep = int(r["groups"]["count"]), int(r["groups"]["keep"])
    score = torch.sigmoid(h @ router_weight.T)                                     # [T, E]
    per = E // count
    runs = score.view(T, count, per)
    worth = runs.topk(min(2, per), dim=-1).values.sum(dim=-1)                      # [T, count]
    kept = worth.topk(keep, dim=-1).indices
    allowed = torch.zeros(T, count, dtype=torch.bool)
    allowed.scatter_(1, kept, True)
    masked = score.masked_fill(~allowed[:, :, None].expand(T, count, per).reshape(T, E), -1.0)
    chosen = masked.topk(top, dim=-1).indices
    picked = score.gather(1, chosen)
    return chosen, picked / (picked.sum(dim=-1, keepdim=True) + 1e-20) * float(r["scale"])


def routed_ff(h, w: dict, p: str, f: dict):
    chosen, weights = route(h, w[p + "router"], f["router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, weight in zip(chosen[t].tolist(), weights[t]):
            q = f"{p}e{e}."
            out[t] += weight * gated_ff(h[t:t + 1], w[q + "gate"], w[q + "up"], w[q + "down"], silu)[0]
    return out


# ---------------------------------------------------------------------------- the model
def forward(config: dict, weights: dict, tokens: list[int], taps: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence; ``taps`` collects the residual stream after every layer."""
    w = {name: t.to(F64) for name, t in weights.items()}
    eps = float(config["norm"]["eps"])

    def norm(x, name):
        return dynamic_tanh(x, w[name], w[name + ".b"], w[name + ".alpha"])

    x = w["embed"][torch.tensor(tokens)] * float(config["embedding"]["scale"])
    v_first = None
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = norm(x, p + "norm1")
        if layer["type"] == "attention":
            mixes = bool(m.get("v_mix"))
            mixed, v = sink_attention(h, w, p + "mix.", m, v_first if mixes else None)
            if mixes and v_first is None:
                v_first = v
        elif layer["type"] == "gla":
            mixed = gla(h, w, p + "mix.", m, eps)
        else:
            raise ValueError(layer["type"])
        x = x + mixed
        f = layer.get("mlp")
        if f is not None:
            h = norm(x, p + "norm2")
            if f["kind"] == "dense":
                q = p + "mlp."
                x = x + gated_ff(h, w[q + "gate"], w[q + "up"], w[q + "down"], gelu_tanh)
            else:
                x = x + routed_ff(h, w, p + "mlp.", f)
        if taps is not None:
            taps.append(x.clone())
    return norm(x, "final.norm") @ w["head"].T
