"""Busatar through the engine against the plain implementation (tests/plain_busatar.py): every mechanism
alone, then whole models cut and batched every way, in float32 and bfloat16, with pools so small that
pages and state slots are used again. Sizes, orders and constants are the tests' own."""

import copy
import json
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_busatar as plain
from busatar_configs import MODELS, draw, gated, ids, latent, recurrent, single_layer
from matricxon_b200.config.registry import config_from_dict
from matricxon_b200.engine.core import model_from_tensors
from matricxon_b200.engine.replay import TraceReplayer
from matricxon_b200.ops import kernels
from trace_utils import ROOT

pytestmark = pytest.mark.gpu

DEVICE = "cuda:0"
CHUNKS = [7, 2, 5, 3, 11, 2, 4, 13, 2, 9]


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

    def check(self, request: str, tokens: list[int], first: int = 0) -> None:
        want = self.reference(tokens)
        got = np.stack([self.logits[(request, i)] for i in range(first, len(tokens))])
        worst = np.abs(got - want[first:]).max(axis=1)
        limit = limit_for(self.dtype, want)
        bad = np.nonzero(~(worst <= limit))[0]
        assert bad.size == 0, (f"{request}: first wrong position {first + bad[0]} of {len(tokens)}, "
                               f"error {worst[bad[0]]:.3e} > {limit:.1e}")


# ---------------------------------------------------------------------- kernels alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden, offset", [(96, 1.0), (1002, 0.0), (9000, 1.0), (18002, 1.0)])
def test_rms_norm_and_post_norm_sum(dtype, hidden, offset):
    torch.manual_seed(hidden)
    x = torch.randn(7, hidden, device=DEVICE) * 3
    acc = torch.randn(7, hidden, device=DEVICE)
    weight = torch.randn(hidden, device=DEVICE) * 0.2
    rows = torch.tensor([4, 0, 6], dtype=torch.int32, device=DEVICE)
    out = torch.empty(3, hidden, dtype=dtype, device=DEVICE)
    kernels.rmsnorm(x, weight, offset, 1e-3, out, rows)
    want = plain.rms_unit(x.double()[rows.long()], 1e-3) * (offset + weight.double())
    tol = 1e-5 if dtype == torch.float32 else 0.02
    assert torch.allclose(out.double(), want, rtol=tol, atol=tol)
    stream = x.clone()
    act = None if dtype == torch.float32 else torch.empty(7, hidden, dtype=dtype, device=DEVICE)
    kernels.rmsnorm_sum(stream, acc, 1.7, weight, offset, 1e-3, act)
    want = plain.rms_unit(1.7 * x.double() + acc.double(), 1e-3) * (offset + weight.double())
    assert torch.allclose(stream.double(), want, rtol=1e-5, atol=1e-5)
    if act is not None:
        assert torch.equal(act, stream.to(dtype))


def _latent_case(dtype, n_heads, rank, rot, page_size, window, contexts, q_lens, seed, spike=None,
                 tensor_cores=False, n_splits=1, no_list=False, few_rows=False):
    """Queries and a paged latent cache with shuffled pages; returns what the kernel gave and the plain sums.
    ``spike`` = (sequence, query offset, key position): that key's vector is made to dominate the query's
    scores if the query sees it."""
    gen = torch.Generator().manual_seed(seed)
    dk = rank + rot
    totals = [c + q for c, q in zip(contexts, q_lens)]
    pages_needed = [(t + page_size - 1) // page_size for t in totals]
    n_pages = sum(pages_needed) + 3
    order = torch.randperm(n_pages, generator=gen).tolist()
    width = max(pages_needed)
    tables = torch.full((len(totals), width), -1, dtype=torch.int32)
    cache = torch.full((n_pages, 1, 1, page_size, dk), float("nan"))
    vectors, q_rows, tok_seq, positions = [], [], [], []
    for s, total in enumerate(totals):
        vec = torch.randn(total, dk, generator=gen)
        q = torch.randn(q_lens[s], n_heads, dk, generator=gen)
        if spike is not None and spike[0] == s:
            _, offset, key = spike
            vec[key] = q[offset, 0] / q[offset, 0].norm() ** 2 * 10.0 * dk ** 0.5     # a score of 20
            q[offset] = q[offset, 0][None] * 1.0
        vec = vec.to(dtype).float()
        q = q.to(dtype).float()
        vectors.append(vec)
        for logical in range(pages_needed[s]):
            page = order.pop()
            tables[s, logical] = page
            chunk = vec[logical * page_size:(logical + 1) * page_size]
            cache[page, 0, 0, :chunk.shape[0]] = chunk
        q_rows.append(q)
        tok_seq += [s] * q_lens[s]
        positions += list(range(contexts[s], total))
    q_all = torch.cat(q_rows)
    out = torch.empty(q_all.shape[0], n_heads, rank, dtype=dtype, device=DEVICE)
    status = torch.zeros(1, dtype=torch.int32, device=DEVICE)
    scale = 2.0 / dk ** 0.5
    if tensor_cores:
        cu_q = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32, device=DEVICE)
        flat = kernels.latent_tile_list(q_lens, n_heads)
        tiles = None if no_list else torch.tensor(flat, dtype=torch.int32, device=DEVICE)
        scratch = None
        if n_splits > 1:
            scratch = torch.full((kernels.attention_scratch_bytes(len(tok_seq), n_heads, rank, n_splits) // 4,),
                                 float("nan"), device=DEVICE)
        kernels.latent_attention_mma(q_all.to(dtype).to(DEVICE), cache.to(dtype).to(DEVICE), tables.to(DEVICE), cu_q,
                                     torch.tensor(contexts, dtype=torch.int32, device=DEVICE), tiles,
                                     len(q_lens) if no_list else len(flat) // 2, rank, window, scale, out, status,
                                     n_splits=n_splits, scratch=scratch, few_rows=few_rows)
    else:
        kernels.latent_attention(q_all.to(dtype).to(DEVICE), cache.to(dtype).to(DEVICE), tables.to(DEVICE),
                                 torch.tensor(tok_seq, dtype=torch.int32, device=DEVICE),
                                 torch.tensor(positions, dtype=torch.int32, device=DEVICE), rank, window, scale,
                                 out, status)
    assert int(status.item()) == 0
    want = torch.empty(q_all.shape[0], n_heads, rank, dtype=torch.float64)
    for row, (s, p) in enumerate(zip(tok_seq, positions)):
        lo = max(0, p - window + 1) if window else 0
        keys = vectors[s][lo:p + 1].double()
        weights = torch.softmax(q_all[row].double() @ keys.T * scale, dim=-1)
        want[row] = weights @ keys[:, :rank]
    return out.double().cpu(), want, vectors


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_heads, rank, rot, page_size, window", [
    (3, 40, 16, 16, 20), (9, 136, 16, 8, 33), (1, 24, 0, 16, None), (8, 520, 64, 32, 64)])
def test_latent_attention_kernel(dtype, n_heads, rank, rot, page_size, window):
    got, want, _ = _latent_case(dtype, n_heads, rank, rot, page_size, window, contexts=[0, 70, 5, 129],
                                q_lens=[45, 1, 30, 2], seed=rank)
    tol = 2e-5 if dtype == torch.float32 else 0.03
    assert torch.allclose(got, want, rtol=tol, atol=tol)


@pytest.mark.parametrize("n_splits", [1, 3])
@pytest.mark.parametrize("n_heads, rank, rot, page_size, window", [
    (3, 64, 16, 16, 20), (9, 160, 16, 8, 33), (1, 32, 0, 16, None), (16, 512, 64, 32, 64), (70, 96, 32, 16, 50)])
def test_latent_attention_on_tensor_cores(n_heads, rank, rot, page_size, window, n_splits):
    """Prompt portions and single tokens in one launch; tiles that straddle tokens (heads no divisor of 64),
    more heads than a tile has rows, keys shared out between blocks."""
    got, want, _ = _latent_case(torch.bfloat16, n_heads, rank, rot, page_size, window, contexts=[0, 70, 5, 129],
                                q_lens=[45, 1, 30, 2], seed=rank, tensor_cores=True, n_splits=n_splits)
    assert torch.allclose(got, want, rtol=0.03, atol=0.03)
    # a fixed-size batch of decoding requests: no tile list, one sequence of them brings nothing
    got, want, _ = _latent_case(torch.bfloat16, n_heads, rank, rot, page_size, window, contexts=[3, 70, 0, 129],
                                q_lens=[1, 1, 1, 1], seed=rank + 1, tensor_cores=True, n_splits=n_splits,
                                no_list=True)
    assert torch.allclose(got, want, rtol=0.03, atol=0.03)
    if n_heads <= 16:       # single tokens of few heads: the deeper pipeline of key chunks, over many chunks
        got, want, _ = _latent_case(torch.bfloat16, n_heads, rank, rot, page_size, window and 8 * window,
                                    contexts=[300, 70, 0, 519], q_lens=[1, 1, 1, 1], seed=rank + 2, tensor_cores=True,
                                    n_splits=n_splits, no_list=n_splits == 1, few_rows=True)
        assert torch.allclose(got, want, rtol=0.03, atol=0.03)
    if n_heads <= 3:        # ... and a few tokens of few heads, still no more than 16 rows a sequence
        got, want, _ = _latent_case(torch.bfloat16, n_heads, rank, rot, page_size, window, contexts=[30, 0, 64, 7],
                                    q_lens=[5, 1, 2, 4], seed=rank + 3, tensor_cores=True, n_splits=n_splits,
                                    few_rows=True)
        assert torch.allclose(got, want, rtol=0.03, atol=0.03)


@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("distance, seen", [(23, True), (24, False), (16, True), (1, True), (0, True)])
def test_latent_attention_on_tensor_cores_window_edge(decode, distance, seen):
    context, q_len = (90, 1) if decode else (40, 51)
    position = context + q_len - 1
    got, want, vectors = _latent_case(torch.bfloat16, 2, 32, 16, 16, 24, contexts=[3, context], q_lens=[4, q_len],
                                      seed=distance, spike=(1, q_len - 1, position - distance), tensor_cores=True,
                                      n_splits=2 if decode else 1)
    assert torch.allclose(got, want, rtol=0.03, atol=0.03)
    row = got.shape[0] - 1
    key = vectors[1][position - distance][:32].double()
    cosine = torch.dot(got[row, 0], key) / (got[row, 0].norm() * key.norm())
    assert (cosine.item() > 0.95) == seen


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("distance, seen", [(23, True), (24, False), (16, True), (15, True), (1, True), (0, True)])
def test_latent_attention_window_edge_with_a_dominant_key(dtype, decode, distance, seen):
    """A key that would take nearly all the weight sits ``distance`` tokens back from the query; the window
    of 24 holds distances 0 .. 23. The query is the last of a portion or a decoded token."""
    context, q_len = (90, 1) if decode else (40, 51)
    position = context + q_len - 1
    got, want, vectors = _latent_case(dtype, 2, 24, 8, 16, 24, contexts=[3, context], q_lens=[4, q_len],
                                      seed=distance, spike=(1, q_len - 1, position - distance))
    tol = 2e-5 if dtype == torch.float32 else 0.03
    assert torch.allclose(got, want, rtol=tol, atol=tol)
    # the dominant key really decides the outcome: when it is visible the head's sum points along it
    row = got.shape[0] - 1
    key = vectors[1][position - distance][:24].double()
    cosine = torch.dot(want[row, 0], key) / (want[row, 0].norm() * key.norm())
    assert (cosine.item() > 0.95) == seen


# ---------------------------------------------------------------------- each mixer alone, as a model of one layer
LAYERS_ALONE = {
    "latent": latent(3, 24, 16, 40, 20, window=11, scale=0.2,
                     scaling={"factor": 4.0, "original": 32, "fast": 8.0, "slow": 2.0}),
    "latent_plain_rotation": latent(2, 16, 8, 24, 16, window=300, scale=0.25),
    "gated_equal_sizes": gated(4, 2, 16, 16, window=13, scale=0.3),
    "gated_wide_values": gated(3, 1, 8, 24, window=17, scale=0.35),
    "gated_tensor_core_size": gated(4, 1, 64, 64, window=21, scale=0.125),
    "recurrence": recurrent(80, 5, 3),
    "recurrence_one_tap": recurrent(64, 1, 1),
    "recurrence_with_ff": recurrent(32, 2, 5, ff=96, limit=0.5),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(LAYERS_ALONE))
def test_one_layer_models(name, dtype):
    """Whole, then one token at a time, then in portions: the three must agree with the plain model. The
    attention scores are sharpened so that a key wrongly seen or missed at a window's edge shows."""
    raw = single_layer(LAYERS_ALONE[name], width=64, vocab=120, alpha=1.5 if "latent" in name else 2.5)
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


# ---------------------------------------------------------------------- whole models
@pytest.fixture(scope="module", params=[("X", "float32"), ("X", "bfloat16"), ("Y", "float32"), ("Y", "bfloat16")],
                ids=lambda p: f"{p[0]}-{p[1]}")
def run(request):
    name, dtype = request.param
    raw = MODELS[name]
    tensors = draw(raw, seed=11 if name == "X" else 12, sharpen=2.0)
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
    """The tail decoded one token at a time: long enough for every window to pass over decoded tokens."""
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
@pytest.mark.parametrize("name, length", [("Z", 330), ("W", 1100)])
def test_long_prompts_and_awkward_sizes(name, length, dtype):
    """A prompt long enough for the prompt-sized product kernels, the chunked recurrence and many attention
    tiles: whole, then in uneven portions with the tail decoded token by token."""
    raw = MODELS[name]
    run = Run(raw, draw(raw, seed=21, sharpen=2.0), dtype, max_tokens=2 * (length + 64))
    tokens = ids(length, raw["vocab"], seed=5)
    run.step([("whole", tokens)], end=["whole"])
    run.check("whole", tokens)
    cuts = [0, length // 3 + 1, length // 3 + 3, length - 40]
    for a, b in zip(cuts, cuts[1:]):
        run.step([("cut", tokens[a:b])])
    for i in range(length - 40, length):
        run.step([("cut", tokens[i:i + 1])], end=["cut"] if i == length - 1 else [])
    run.check("cut", tokens)


def test_greedy_generation_through_the_engine_entry_point():
    from matricxon_b200 import ChatEngine, GenerationRequest, SamplingConfig

    raw = MODELS["X"]
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
    """The replay program itself on a model folder (bfloat16 file, both dtypes), and the generation command."""
    from matricxon_b200.weights.safetensors_io import write_safetensors

    raw = MODELS["Y"]
    tensors = draw(raw, seed=12, sharpen=2.0, store_dtype=torch.bfloat16)
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
    config_path.write_text(json.dumps(raw))
    done = subprocess.run([sys.executable, "-m", "matricxon_b200.generate", "--random-config", str(config_path),
                           "--prompt-len", "20", "--num-predict", "12"], capture_output=True, text=True,
                          timeout=600, cwd=str(ROOT))
    assert done.returncode == 0, done.stderr[-2000:]
    assert "finish_reason:  length" in done.stdout and "Busatar" in done.stdout
