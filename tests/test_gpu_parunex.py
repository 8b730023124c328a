"""Parunex through the engine against the plain implementation (tests/plain_parunex.py): every mechanism alone,
then whole models cut and batched every way, in float32 and bfloat16, with pools so small that pages and state
slots are used again. Sizes, orders and constants are the tests' own."""

import copy
import json
import math
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_parunex as plain
from parunex_configs import MODELS, attention, dense, draw, gla, ids, moe, single_layer
from matricxon_b200.config.registry import config_from_dict
from matricxon_b200.engine.core import model_from_tensors
from matricxon_b200.engine.replay import TraceReplayer
from matricxon_b200.ops import kernels
from trace_utils import ROOT

pytestmark = pytest.mark.gpu

DEVICE = "cuda:0"
CHUNKS = [7, 2, 5, 3, 11, 2, 4, 13, 2, 9]
F64 = torch.float64


def limit_for(dtype: str, reference: np.ndarray) -> float:
    scale = max(1.0, float(np.abs(reference).max()))
    return (2e-4 if dtype == "float32" else 0.04) * scale


def rounded(tensors: dict, dtype: str) -> dict:
    """What the engine holds: a bfloat16 engine reads bfloat16 matrices, so the plain side gets the same."""
    if dtype == "float32":
        return tensors
    return {name: value.to(torch.bfloat16).float() for name, value in tensors.items()}


class Run:
    """One engine over one model: requests fed in portions, logits kept per (request, position)."""

    def __init__(self, raw: dict, tensors: dict, dtype: str, max_tokens: int, max_requests: int = 4,
                 page_size: int = 16) -> None:
        self.raw, self.dtype = raw, dtype
        self.weights = rounded(tensors, dtype)
        config = config_from_dict(copy.deepcopy(raw))
        model = model_from_tensors(config, self.weights, dtype=dtype, device=DEVICE, page_size=page_size)
        self.replayer = TraceReplayer(None, dtype, max_tokens, page_size=page_size, device=DEVICE,
                                      max_requests=max_requests, model=model, poison_cache=True)
        self.logits: dict[tuple[str, int], np.ndarray] = {}
        self.progress: dict[str, int] = {}
        self.slots_seen: dict[str, int] = {}
        self.reference_cache: dict[tuple, np.ndarray] = {}

    def step(self, portions: list[tuple[str, list[int]]], end=()) -> None:
        entries = []
        keys = []
        for request, tokens in portions:
            start = self.progress.get(request, 0)
            entries.append({"id": request, "tokens": tokens, "want": list(range(len(tokens)))})
            keys.extend((request, start + i) for i in range(len(tokens)))
            self.progress[request] = start + len(tokens)
        out = self.replayer.step(entries, [])
        rows = list(self.replayer.last_rows)
        for request, _ in portions:
            self.slots_seen[request] = self.replayer.core.cache.record(request).state_slot
        if end:
            self.replayer.step([], list(end))
        assert rows == keys
        for key, row in zip(keys, out.numpy()):
            self.logits[key] = row
        self.replayer.core.cache.check_invariants()

    def reference(self, tokens: list[int]) -> np.ndarray:
        key = tuple(tokens)
        if key not in self.reference_cache:
            self.reference_cache[key] = plain.forward(self.raw, self.weights, tokens).numpy()
        return self.reference_cache[key]

    def check(self, request: str, tokens: list[int], first: int = 0, allowed_over: int = 0) -> None:
        want = self.reference(tokens)
        got = np.stack([self.logits[(request, i)] for i in range(first, len(tokens))])
        worst = np.abs(got - want[first:]).max(axis=1)
        limit = limit_for(self.dtype, want)
        bad = np.nonzero(~(worst <= limit))[0]
        assert bad.size <= allowed_over, (f"{request}: first wrong position {first + bad[0]} of {len(tokens)}, "
                                          f"error {worst[bad[0]]:.3e} > {limit:.1e}; {bad.size} positions over")


# ---------------------------------------------------------------------- kernels alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden", [96, 1002, 4100])
def test_dynamic_tanh_with_rows_and_with_a_pending_sum(dtype, hidden):
    torch.manual_seed(hidden)
    x = torch.randn(7, hidden, device=DEVICE) * 3
    weight, shift = torch.randn(hidden, device=DEVICE), torch.randn(hidden, device=DEVICE)
    alpha = torch.tensor([0.37], device=DEVICE)
    rows = torch.tensor([4, 0, 6], dtype=torch.int32, device=DEVICE)
    out = torch.empty(3, hidden, dtype=dtype, device=DEVICE)
    kernels.dyt(x, weight, shift, alpha, out, rows)
    want = plain.dynamic_tanh(x.double()[rows.long()], weight.double(), shift.double(), 0.37)
    tol = 1e-5 if dtype == torch.float32 else 0.02
    assert torch.allclose(out.double(), want, rtol=tol, atol=tol)
    acc, bias = torch.randn(7, hidden, device=DEVICE), torch.randn(hidden, device=DEVICE)
    stream = x.clone()
    out = torch.empty(7, hidden, dtype=dtype, device=DEVICE)
    kernels.dyt(stream, weight, shift, alpha, out, acc=acc, col_bias=bias)
    total = x.double() + acc.double() + bias.double()
    assert torch.allclose(stream.double(), total, rtol=1e-6, atol=1e-6)
    assert torch.allclose(out.double(), plain.dynamic_tanh(total, weight.double(), shift.double(), 0.37), rtol=tol, atol=tol)


def _paged_case(dtype, n_heads, n_kv, hd, page_size, contexts, q_lens, seed, spike=None):
    """Queries and a paged cache with shuffled pages. Returns (q, cache, metadata, per-sequence keys and values).
    ``spike`` = (sequence, key position): that key is aligned with the sequence's last query and made long."""
    gen = torch.Generator().manual_seed(seed)
    n_seqs, n_tok = len(contexts), sum(q_lens)
    totals = [c + q for c, q in zip(contexts, q_lens)]
    pages_of = [-(-t // page_size) for t in totals]
    n_pages = sum(pages_of) + 3
    order = torch.randperm(n_pages, generator=gen).tolist()
    width = max(pages_of)
    tables = torch.full((n_seqs, width), -1, dtype=torch.int32)
    cache = torch.full((n_pages, 2, n_kv, page_size, hd), float("nan"))
    keys, values = [], []
    q = torch.randn(n_tok, n_heads * hd, generator=gen)
    group = n_heads // n_kv
    row = 0
    for s in range(n_seqs):
        k = torch.randn(totals[s], n_kv, hd, generator=gen)
        v = torch.randn(totals[s], n_kv, hd, generator=gen)
        last = row + q_lens[s] - 1
        if spike is not None and spike[0] == s:
            for g in range(n_kv):
                direction = q[last].view(n_heads, hd)[g * group]
                k[spike[1], g] = direction / direction.norm() * 14.0
        keys.append(k)
        values.append(v)
        for lp in range(pages_of[s]):
            page = order.pop()
            tables[s, lp] = page
            lo, hi = lp * page_size, min((lp + 1) * page_size, totals[s])
            cache[page, 0, :, :hi - lo] = k[lo:hi].transpose(0, 1)
            cache[page, 1].view(n_kv, hd, page_size)[:, :, :hi - lo] = v[lo:hi].permute(1, 2, 0)
        row += q_lens[s]
    cache = torch.nan_to_num(cache, nan=0.0) if dtype == torch.bfloat16 else cache
    tok_seq = torch.tensor([s for s in range(n_seqs) for _ in range(q_lens[s])], dtype=torch.int32)
    positions = torch.tensor([contexts[s] + i for s in range(n_seqs) for i in range(q_lens[s])], dtype=torch.int32)
    cu_q = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32)
    meta = {"tables": tables.to(DEVICE), "tok_seq": tok_seq.to(DEVICE), "positions": positions.to(DEVICE),
            "cu_q": cu_q.to(DEVICE), "contexts": torch.tensor(contexts, dtype=torch.int32, device=DEVICE)}
    return q.to(dtype).to(DEVICE), cache.to(dtype).to(DEVICE), meta, keys, values


def _plain_attend(q, keys, values, contexts, q_lens, n_heads, n_kv, hd, scale, cap, sink):
    out = torch.zeros(q.shape[0], n_heads, hd, dtype=F64)
    group = n_heads // n_kv
    row = 0
    for s, (c, n) in enumerate(zip(contexts, q_lens)):
        k, v = keys[s].double(), values[s].double()
        for i in range(n):
            qi = q[row].double().view(n_heads, hd)
            for h in range(n_heads):
                score = (k[:c + i + 1, h // group] @ qi[h]) * scale
                if cap:
                    score = cap * torch.tanh(score / cap)
                top = score.max() if sink is None else torch.maximum(score.max(), sink[h].double())
                e = torch.exp(score - top)
                total = e.sum() + (0 if sink is None else torch.exp(sink[h].double() - top))
                out[row, h] = (e / total) @ v[:c + i + 1, h // group]
            row += 1
    return out.view(q.shape[0], n_heads * hd)


@pytest.mark.parametrize("kernel, dtype, hd, group", [
    ("simt", torch.float32, 48, 3), ("simt", torch.float32, 128, 2), ("simt", torch.bfloat16, 32, 1),
    ("mma", torch.bfloat16, 64, 4), ("mma", torch.bfloat16, 128, 2), ("tc", torch.bfloat16, 128, 2),
    ("tc", torch.bfloat16, 128, 4)])
@pytest.mark.parametrize("cap, with_sink", [(6.0, True), (None, True), (3.0, False)])
def test_attention_kernels_cap_scores_and_count_the_sink(kernel, dtype, hd, group, cap, with_sink):
    """Prompt portions and single tokens in one launch, shuffled pages, key splits; a long key far back in one
    sequence saturates the cap; sinks of both signs."""
    n_kv, n_heads = 2, 2 * group
    contexts, q_lens = [70, 5, 300, 0], [1, 37, 1, 45]
    if kernel == "tc":
        contexts, q_lens = [70, 5, 130], [40, 37, 64]
    q, cache, meta, keys, values = _paged_case(dtype, n_heads, n_kv, hd, 16, contexts, q_lens, seed=hd + group,
                                               spike=(2, 11))
    sink = torch.linspace(-3.0, 4.0, n_heads) if with_sink else None
    sink_dev = sink.to(DEVICE) if with_sink else None
    status = torch.zeros(1, dtype=torch.int32, device=DEVICE)
    n_tok = sum(q_lens)
    scale = 1.0 / math.sqrt(hd)
    want = _plain_attend(q.cpu().float(), [k.to(dtype).float() for k in keys], [v.to(dtype).float() for v in values],
                         contexts, q_lens, n_heads, n_kv, hd, scale, cap, sink)
    for n_splits in (1, 3):
        out = torch.zeros(n_tok, n_heads * hd, dtype=dtype, device=DEVICE)
        scratch = None
        if n_splits > 1:
            scratch = torch.empty(kernels.attention_scratch_bytes(n_tok, n_heads, hd, n_splits) // 4 + 4,
                                  dtype=torch.float32, device=DEVICE)
        if kernel == "simt":
            kernels.paged_attention(q, q.stride(0), cache, meta["tables"], meta["tok_seq"], meta["positions"], n_tok,
                                    n_heads, n_kv, hd, None, scale, out, status, n_splits=n_splits, scratch=scratch,
                                    softcap=cap, sink=sink_dev)
        elif kernel == "tc":
            _, wide = kernels.attention_tile_lists([max(n, 17) for n in q_lens], group, True)
            tiles = torch.tensor(wide, dtype=torch.int32, device=DEVICE)
            kernels.paged_attention_tc(q, q.stride(0), cache, meta["tables"], meta["cu_q"], meta["contexts"], tiles,
                                       len(wide) // 2, n_tok, n_heads, n_kv, hd, None, scale, out, status,
                                       n_splits=n_splits, scratch=scratch, softcap=cap, sink=sink_dev)
        else:
            narrow, wide = kernels.attention_tile_lists(q_lens, group, False)
            if n_splits > 1:        # key splits need a launch that covers every token: all tiles wide
                narrow, wide = [], [x for s, n in enumerate(q_lens) for r in range(0, n * group, 64) for x in (s, r)]
            for tiles, is_narrow in ((narrow, True), (wide, False)):
                if tiles:
                    t = torch.tensor(tiles, dtype=torch.int32, device=DEVICE)
                    kernels.paged_attention_mma(q, q.stride(0), cache, meta["tables"], meta["cu_q"], meta["contexts"], t,
                                                len(tiles) // 2, is_narrow, n_tok, n_heads, n_kv, hd, None, scale, out,
                                                status, n_splits=n_splits, scratch=scratch, softcap=cap, sink=sink_dev)
        tol = 2e-5 if dtype == torch.float32 else 0.03
        assert torch.allclose(out.double().cpu(), want, rtol=tol, atol=tol), (n_splits, (out.double().cpu() - want).abs().max())
        assert int(status.item()) == 0
    # the cap really bit: without it the long key takes the softmax of the last query of its sequence
    if cap:
        free = _plain_attend(q.cpu().float(), keys, values, contexts, q_lens, n_heads, n_kv, hd, scale, None, sink)
        row = sum(q_lens[:3]) - 1
        assert (free[row] - want[row]).abs().max() > 0.1


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts, top, count, keep", [(12, 4, 4, 3), (6, 2, 6, 3), (8, 3, 1, 1), (9, 1, 3, 1),
                                                       (64, 6, 8, 4), (5, 5, 5, 5)])
def test_router_kernel_against_the_plain_choice(dtype, experts, top, count, keep):
    gen = torch.Generator().manual_seed(experts * 7 + top)
    n, width = 50, 72
    h = torch.randn(n, width, generator=gen).to(dtype)
    router = torch.randn(experts, width, generator=gen) * 0.5
    r = {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}, "scale": 1.7}
    chosen, weights = plain.route(h.double(), router.double(), r)
    ints = torch.zeros(experts + 3 * n * top, dtype=torch.int32, device=DEVICE)
    counts, got_ids, place, _ = torch.split(ints, [experts, n * top, n * top, n * top])
    got_w = torch.empty(n * top, dtype=torch.float32, device=DEVICE)
    kernels.moe_route(h.to(DEVICE), router.to(DEVICE), top, count, keep, 1.7, got_ids, got_w, counts, place)
    got_ids, got_w = got_ids.view(n, top).cpu().long(), got_w.view(n, top).cpu().double()
    assert torch.equal(got_ids, chosen), "the experts, in the order of their scores"
    assert torch.allclose(got_w, weights, rtol=1e-5, atol=1e-6)
    assert torch.equal(counts.cpu().long(), torch.bincount(chosen.flatten(), minlength=experts))
    # every pair has a place of its own among its expert's pairs
    seen = {(int(e), int(p)) for e, p in zip(got_ids.flatten(), place.cpu())}
    assert len(seen) == n * top and all(p < counts[e] for e, p in seen)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n, experts, top, width, ff", [(1, 4, 2, 64, 40), (70, 5, 3, 96, 52), (300, 3, 1, 40, 136)])
def test_routed_feed_forward_part_against_the_plain_one(dtype, n, experts, top, width, ff):
    from matricxon_b200.parts.base import Runtime, build_part
    from matricxon_b200.parts.spec import GatedMlpSpec, RoutedExpertsSpec

    gen = torch.Generator().manual_seed(n)
    expert = GatedMlpSpec(width, ff, "silu", "gate", "up", "down")
    spec = RoutedExpertsSpec(width, experts, top, 1, 1, 1.3, expert, "router")
    part = build_part("feed_forward", spec, Runtime(DEVICE, dtype), "f.")
    w = {"f.router": torch.randn(experts, width, generator=gen)}
    for e in range(experts):
        w[f"f.e{e}.gate"] = torch.randn(ff, width, generator=gen) * 0.2
        w[f"f.e{e}.up"] = torch.randn(ff, width, generator=gen) * 0.2
        w[f"f.e{e}.down"] = torch.randn(width, ff, generator=gen) * 0.2
    w = {k: (v if k == "f.router" else v.to(dtype).float()) for k, v in w.items()}
    part.load(lambda name: w[name].to(DEVICE).to(torch.float32 if name == "f.router" else dtype))
    h = torch.randn(n, width, generator=gen).to(dtype)
    residual = torch.randn(n, width, generator=gen)
    got = part.forward(h.to(DEVICE), residual.clone().to(DEVICE), None).cpu().double()
    f = {"router": {"experts": experts, "top": top, "groups": {"count": 1, "keep": 1}, "scale": 1.3}}
    want = residual.double() + plain.routed_ff(h.double(), {k: v.double() for k, v in w.items()}, "f.", f)
    tol = 1e-4 if dtype == torch.float32 else 0.05
    assert torch.allclose(got, want, rtol=tol, atol=tol), (got - want).abs().max()


@pytest.mark.parametrize("heads, dim, vdim, rank", [(3, 24, 40, 5), (2, 64, 64, 16), (1, 130, 20, 3), (2, 200, 9, 4)])
def test_recurrence_kernels_continue_from_their_state(heads, dim, vdim, rank):
    """Three sequences, one of them continued from a state that an earlier launch left, in a slot order of their
    own; against the plain recurrence over the whole sequences."""
    gen = torch.Generator().manual_seed(dim)
    lens = [(0, 37), (21, 1), (5, 18)]                      # (tokens before, tokens now)
    keys, values = heads * dim, heads * vdim
    ld = 2 * keys + values + 7
    full = [torch.randn(a + b, ld, generator=gen) for a, b in lens]
    decay = [torch.sigmoid(torch.randn(a + b, keys, generator=gen) * 2 + 2) for a, b in lens]
    state = torch.full((5, heads, dim, vdim), float("nan"), device=DEVICE)
    slots = [3, 0, 4]
    scale = dim ** -0.5

    def launch(rows, decays, cu, slot_ids):
        proj = torch.cat(rows).to(DEVICE)
        out = torch.empty(proj.shape[0], values, device=DEVICE)
        kernels.gla_scan(proj, 0, keys, 2 * keys, torch.cat(decays).to(DEVICE).contiguous(), scale, state,
                         torch.tensor(cu, dtype=torch.int32, device=DEVICE),
                         torch.tensor(slot_ids, dtype=torch.int32, device=DEVICE), len(slot_ids), out, heads, dim, vdim)
        return out.cpu()

    for s in slots:
        state[s].zero_()
    launch([full[1][:21], full[2][:5]], [decay[1][:21], decay[2][:5]], [0, 21, 26], [slots[1], slots[2]])
    got = launch([f[a:] for f, (a, b) in zip(full, lens)], [d[a:] for d, (a, b) in zip(decay, lens)],
                 [0, 37, 38, 56], slots)
    row = 0
    for f, d, (a, b) in zip(full, decay, lens):
        f, d = f.double(), d.double()
        S = torch.zeros(heads, dim, vdim, dtype=F64)
        for t in range(a + b):
            q, k = f[t, :keys].view(heads, dim) * scale, f[t, keys:2 * keys].view(heads, dim)
            v = f[t, 2 * keys:2 * keys + values].view(heads, vdim)
            S = d[t].view(heads, dim)[:, :, None] * S + k[:, :, None] * v[:, None, :]
            if t >= a:
                want = torch.einsum("hde,hd->he", S, q).reshape(-1)
                assert torch.allclose(got[row].double(), want, rtol=2e-5, atol=2e-5), (t, row)
                row += 1
    # the decay kernel: a low-rank map, a sigmoid, the tau-th root
    low = torch.randn(11, rank + 3, generator=gen)
    a2, bias = torch.randn(keys, rank, generator=gen), torch.randn(keys, generator=gen) * 3
    out = torch.empty(11, keys, device=DEVICE)
    kernels.gla_decay(low.to(DEVICE)[:, 2:2 + rank], a2.to(DEVICE), bias.to(DEVICE), 7.0, out)
    want = torch.sigmoid(low[:, 2:2 + rank].double() @ a2.double().T + bias.double()) ** (1 / 7.0)
    assert torch.allclose(out.cpu().double(), want, rtol=1e-5, atol=1e-6)


# ---------------------------------------------------------------------- each mechanism alone, as a model of one layer
SCALING = {"factor": 3.0, "low": 1.0, "high": 5.0, "original": 32}
LAYERS_ALONE = {
    "attention_narrow_values": (attention(4, 2, 24, 8, 0.3, 9.0, 12, scaling=SCALING), None),
    "attention_wide_values": (attention(3, 1, 8, 24, 0.35, 2.5, 8, base=50.0), None),
    "attention_whole_head_rotated": (attention(4, 4, 16, 16, 0.3, 30.0, 16), None),
    "attention_tensor_core_size": (attention(4, 1, 64, 64, 0.125, 12.0, 32, scaling=SCALING, mlp=dense(96)), None),
    "attention_with_experts": (attention(2, 2, 16, 16, 0.25, 5.0, 4, mlp=moe(40, 6, 2, 3, 2, scale=1.5)), None),
    "recurrence": (gla(3, 24, 40, 4.0), 5),
    "recurrence_one_head": (gla(1, 72, 16, 30.0, mlp=dense(48)), 1),
    "recurrence_with_experts": (gla(2, 16, 16, 2.0, mlp=moe(24, 4, 1, 2, 1, scale=3.0)), 8),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(LAYERS_ALONE))
def test_one_layer_models(name, dtype):
    """Whole, then one token at a time, then in portions: the three must agree with the plain model. The
    attention scores are sharpened so that a key wrongly seen or missed shows."""
    layer, rank = LAYERS_ALONE[name]
    raw = single_layer(layer, width=64, vocab=120, rank=rank)
    tensors = draw(raw, seed=len(name), sharpen=4.0)
    run = Run(raw, tensors, dtype, max_tokens=256)
    tokens = ids(75, raw["vocab"], seed=1)
    run.step([("whole", tokens)], end=["whole"])
    run.check("whole", tokens)
    for i, token in enumerate(tokens[:60]):
        run.step([("single", [token])], end=["single"] if i == 59 else [])
    run.check("single", tokens[:60])
    start = 0
    for turn in range(100):
        size = min(CHUNKS[turn % len(CHUNKS)], len(tokens) - start)
        run.step([("cut", tokens[start:start + size])], end=["cut"] if start + size == len(tokens) else [])
        start += size
        if start == len(tokens):
            break
    run.check("cut", tokens)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("decode", [False, True])
def test_a_far_key_among_hundreds_decides_the_logits(dtype, decode):
    """One token 400 positions back is made the only key the last query cares for: its value must come through,
    whole and when the tail is decoded token by token across page borders."""
    raw = single_layer(attention(2, 1, 32, 32, 0.18, 40.0, 0), width=64, vocab=90)
    tensors = draw(raw, seed=9, sharpen=1.0)
    tokens = ids(430, raw["vocab"], seed=2)
    tokens[25] = 88                                   # the only occurrence of this token ...
    tokens = [t if t != 88 or i == 25 else 87 for i, t in enumerate(tokens)]
    tokens[-1] = 89                                   # ... and of the one that asks for it
    tokens = [t if t != 89 or i == len(tokens) - 1 else 86 for i, t in enumerate(tokens)]
    # without rotation, k of token 88 and q of token 89 depend on their embeddings alone: align them, with a
    # score of 30 for that pair (under the cap of 40) and keys without a common part
    norm = lambda row: torch.tanh(float(tensors["l0.norm1.alpha"]) * row * 4.0) * tensors["l0.norm1"] + tensors["l0.norm1.b"]
    tensors["l0.mix.k.b"] = torch.zeros(32)
    k88 = tensors["l0.mix.k"] @ norm(tensors["embed"][88])
    h89 = norm(tensors["embed"][89])
    tensors["l0.mix.q"] = (torch.outer(k88.repeat(2), h89) / (h89 @ h89) * (30.0 / (0.18 * (k88 @ k88)))).contiguous()
    tensors["l0.mix.q.b"] = torch.zeros(64)
    tensors["l0.mix.o"] = tensors["l0.mix.o"] * 4.0             # what attention finds weighs in the logits
    run = Run(raw, tensors, dtype, max_tokens=512)
    if decode:
        run.step([("far", tokens[:390])])
        for i in range(390, len(tokens)):
            run.step([("far", tokens[i:i + 1])], end=["far"] if i == len(tokens) - 1 else [])
    else:
        run.step([("far", tokens)], end=["far"])
    run.check("far", tokens)
    # the far key really decides: without it the last position's logits differ by more than the tolerance
    moved = list(tokens)
    moved[25] = 87
    a, b = run.reference(tokens)[-1], plain.forward(raw, run.weights, moved).numpy()[-1]
    assert np.abs(a - b).max() > 0.3


# ---------------------------------------------------------------------- whole models
@pytest.fixture(scope="module", params=[("P", "float32"), ("P", "bfloat16"), ("Q", "float32"), ("Q", "bfloat16")],
                ids=lambda p: f"{p[0]}-{p[1]}")
def run(request):
    name, dtype = request.param
    raw = MODELS[name]
    tensors = draw(raw, seed=11 if name == "P" else 12, sharpen=2.0)
    # four live requests of at most 128 tokens: pages and slots must come back to be used again
    return Run(raw, tensors, dtype, max_tokens=4 * 128, max_requests=4)


LENGTHS = [1, 2, 17, 40, 65, 100, 128]


def prompts_of(run):
    return {f"r{n}": ids(n, run.raw["vocab"], seed=100 + n) for n in LENGTHS}


def test_whole_prompts(run):
    for request, tokens in prompts_of(run).items():
        run.step([(request + "w", tokens)], end=[request + "w"])
        run.check(request + "w", tokens)


def test_prefill_then_token_by_token(run):
    for request, tokens in prompts_of(run).items():
        head = max(len(tokens) - 70, 0)
        if head:
            run.step([(request + "d", tokens[:head])])
        for i in range(head, len(tokens)):
            run.step([(request + "d", tokens[i:i + 1])], end=[request + "d"] if i == len(tokens) - 1 else [])
        run.check(request + "d", tokens)


def test_portions_down_to_two_tokens(run):
    for shift, (request, tokens) in enumerate(prompts_of(run).items()):
        start, turn = 0, shift
        while start < len(tokens):
            size = min(CHUNKS[turn % len(CHUNKS)], len(tokens) - start)
            turn += 1
            run.step([(request + "c", tokens[start:start + size])],
                     end=[request + "c"] if start + size == len(tokens) else [])
            start += size
        run.check(request + "c", tokens)


def test_unequal_requests_batched_with_pages_and_slots_used_again(run):
    prompts = prompts_of(run)
    waiting = [(f"{request}m{again}", tokens) for again in range(2) for request, tokens in prompts.items()]
    tokens_of = dict(waiting)
    live: dict[str, int] = {}
    cache = run.replayer.core.cache
    turn = 0
    while waiting or live:
        while waiting and len(live) < 4:
            live[waiting.pop(0)[0]] = 0
        portions, ended = [], []
        for place, (request, done) in enumerate(list(live.items())):
            tokens = tokens_of[request]
            if (turn + place) % 5 == 4 and len(live) > 1:
                continue                                          # sits this step out
            remaining = len(tokens) - done
            size = 1 if (turn + place) % 3 == 0 else min(CHUNKS[(turn + place) % len(CHUNKS)], remaining)
            portions.append((request, tokens[done:done + size]))
            live[request] = done + size
            if done + size == len(tokens):
                ended.append(request)
        turn += 1
        if portions:
            run.step(portions, end=ended)
        for request in ended:
            del live[request]
    for request, tokens in tokens_of.items():
        run.check(request, tokens)
    assert cache.pages_reused > 0
    assert len(set(run.slots_seen[r] for r in tokens_of)) <= 4 < len(tokens_of)


def test_long_decoding(run):
    """Hundreds of single-token steps (the captured decode step replayed) after a short prompt, two requests
    side by side, one of them starting later."""
    a = ids(260, run.raw["vocab"], seed=7)
    b = ids(150, run.raw["vocab"], seed=8)
    run.step([("la", a[:6])])
    for i in range(6, len(a)):
        portions = [("la", a[i:i + 1])]
        j = i - 100
        if 0 <= j < len(b):
            portions.append(("lb", b[j:j + 1]))
        ended = [name for name, k, seq in (("la", i, a), ("lb", j, b)) if k == len(seq) - 1]
        run.step(portions, end=ended)
    run.check("la", a)
    run.check("lb", b)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name, length", [("R", 330), ("S", 1100)])
def test_long_prompts_and_awkward_sizes(name, length, dtype):
    """A prompt long enough for the prompt-sized product kernels, many attention tiles and many rounds of the
    recurrence: whole, then in uneven portions with the tail decoded token by token."""
    raw = MODELS[name]
    run = Run(raw, draw(raw, seed=21, sharpen=2.0), dtype, max_tokens=2 * (length + 64))
    tokens = ids(length, raw["vocab"], seed=5)
    run.step([("whole", tokens)], end=["whole"])
    # among a thousand tokens a few have two experts' scores so close that the rounding of the router's input to
    # bfloat16 decides between them (the plain model routes on unrounded input); those tokens get another expert's
    # output, which is no fault of the engine: at most 1 % of the positions may differ in bfloat16, none in float32
    slack = length // 100 if dtype == "bfloat16" else 0
    run.check("whole", tokens, allowed_over=slack)
    cuts = [0, length // 3 + 1, length // 3 + 3, length - 40]
    for a, b in zip(cuts, cuts[1:]):
        run.step([("cut", tokens[a:b])])
    for i in range(length - 40, length):
        run.step([("cut", tokens[i:i + 1])], end=["cut"] if i == length - 1 else [])
    run.check("cut", tokens, allowed_over=slack)


def test_greedy_generation_through_the_engine_entry_point():
    from matricxon_b200 import ChatEngine, GenerationRequest, SamplingConfig

    raw = MODELS["P"]
    tensors = draw(raw, seed=11, sharpen=2.0)
    config = config_from_dict(copy.deepcopy(raw))
    model = model_from_tensors(config, tensors, dtype="float32", device=DEVICE)
    engine = ChatEngine(model, max_cache_tokens=4 * 128, max_active=3, max_batched_tokens=64, prefill_chunk=24,
                        max_model_len=128)
    prompts = [ids(n, raw["vocab"], seed=40 + n) for n in (5, 33, 70, 12, 50)]
    sampling = SamplingConfig(temperature=0.0, repeat_penalty=1.0, num_predict=24, num_ctx=128, seed=0)
    results = engine.generate_batch([GenerationRequest(input_ids=p, sampling=sampling) for p in prompts])
    for prompt, result in zip(prompts, results):
        assert result.finish_reason == "length" and len(result.token_ids) == 24
        logits = plain.forward(raw, tensors, prompt + result.token_ids[:-1]).numpy()
        for k, token in enumerate(result.token_ids):
            row = logits[len(prompt) - 1 + k]
            assert row[token] >= row.max() - 2e-3, (k, token, int(row.argmax()))


def test_trace_program_and_command_line(tmp_path):
    """The replay program itself on a model folder (bfloat16 file, both dtypes; the decay rank is read from the
    tensors), and the generation command."""
    from matricxon_b200.weights.safetensors_io import write_safetensors

    raw = copy.deepcopy(MODELS["Q"])
    tensors = draw(raw, seed=12, sharpen=2.0, store_dtype=torch.bfloat16)
    del raw["decay_ranks"]                          # a model folder's config.json does not name them
    # a file may hold the second norm of a layer that has no feed-forward: expected, unused
    tensors["l1.norm2"] = torch.ones(128, dtype=torch.bfloat16)
    tensors["l1.norm2.b"] = torch.zeros(128, dtype=torch.bfloat16)
    tensors["l1.norm2.alpha"] = torch.tensor(1.0, dtype=torch.bfloat16)
    folder = tmp_path / "model"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(raw))
    write_safetensors(folder / "model.safetensors", tensors.items())
    tokens = ids(50, raw["vocab"], seed=3)
    want = plain.forward(raw, {k: v.float() for k, v in tensors.items()}, tokens).numpy()
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": tokens[:31], "want": [0, 30]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": tokens[31:33], "want": []},
                                     {"id": "b", "tokens": tokens[:9], "want": [8]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": tokens[33:], "want": [16]}], "end": ["a"]}]
    for dtype in ("float32", "bfloat16"):
        out = tmp_path / dtype
        done = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype",
                               dtype, "--out", str(out), "--max-tokens", "128"],
                              input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
                              timeout=600)
        assert done.returncode == 0, done.stderr[-2000:]
        assert [line for line in done.stdout.splitlines() if line.startswith("done")] == ["done 0", "done 1", "done 2"]
        got = {s: np.fromfile(out / f"{s}.f32", dtype="<f4").reshape(-1, raw["vocab"]) for s in (0, 1, 2)}
        limit = limit_for(dtype, want)
        assert np.abs(got[0] - want[[0, 30]]).max() <= limit
        assert np.abs(got[1] - want[[8]]).max() <= limit
        assert np.abs(got[2] - want[[49]]).max() <= limit
    config_path = tmp_path / "config.json"
    config_path.write_text(json.dumps(MODELS["R"]))
    done = subprocess.run([sys.executable, "-m", "matricxon_b200.generate", "--random-config", str(config_path),
                           "--prompt-len", "20", "--num-predict", "12"], capture_output=True, text=True,
                          timeout=600, cwd=str(ROOT))
    assert done.returncode == 0, done.stderr[-2000:]
    assert "finish_reason:  length" in done.stdout and "Parunex" in done.stdout
