"""The Mamevik decoder through the engine, and each of its mechanisms alone (GPU), against the plain
64-bit statement in plain_mamevik.py.  The configurations are in mamevik_cases.py: U (odd sizes, exact
kernels, a loop from the first layer), V (the tensor-core kernels' sizes, a loop over the last two layers that runs
three times), W (no loop, no table of pairs, a state of 200 rows, one tap, a window of one token), X (V's sizes
with every expert chosen, for long bfloat16 prompts whose routing must not flip), Y (sizes that are multiples of
nothing, a loop over all layers that runs once), Z (recurrences only: no pages, only state slots).
"""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import mamevik_cases as cases
import plain_mamevik as plain
from helpers import ROOT, Trace, assert_close, check_trace, random_tokens, run_trace_inprocess

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ENGINE_CASES = [("U", "float32"), ("U", "bfloat16"), ("V", "float32"), ("V", "bfloat16"), ("W", "float32"), ("W", "bfloat16"),
                ("Y", "float32"), ("Y", "bfloat16"), ("Z", "float32"), ("Z", "bfloat16")]


@pytest.fixture(scope="module")
def root(tmp_path_factory):
    return str(tmp_path_factory.mktemp("mamevik"))


def stored(dtype):
    return torch.bfloat16 if dtype == "bfloat16" else torch.float32


def runner_for(root, name, dtype, pages=64, requests=4, page=None):
    from inferloop_b200.engine import ModelRunner
    _, _, page_size = cases.CASES[name]
    return ModelRunner.from_folder(cases.folder(root, name, stored(dtype)), dtype=dtype, device=DEV,
                                   page_size=page or page_size, num_pages=pages, max_requests=requests)


_TOKENS = {}


def tokens_for(root, name, dtype, n, seed):
    key = (name, dtype, n, seed)
    if key not in _TOKENS:
        model = cases.plain_model(root, name, stored(dtype))
        _TOKENS[key] = cases.decided_tokens(model, n, cases.CASES[name][0]["vocab"], seed, 3e-2 if dtype == "bfloat16" else 1e-4)
    return _TOKENS[key]


def reference(root, name, dtype, tokens):
    return cases.plain_model(root, name, stored(dtype)).forward(tokens)


# ------------------------------------------------------------------------------ the engine
@pytest.mark.parametrize("name,dtype", ENGINE_CASES)
def test_whole_prompt_and_every_layer_run(root, name, dtype):
    """One prompt in one step: the residual stream after every run of a layer (a looped layer counts
    each time), and all logits."""
    from inferloop_b200.engine import StepEntry
    from inferloop_b200.parts.loop import LoopInputBlock
    r = runner_for(root, name, dtype)
    toks = tokens_for(root, name, dtype, 45, 1)
    per_run = []
    ref = cases.plain_model(root, name, stored(dtype)).forward(toks, per_run)
    got = []
    for b in r.model.blocks:
        if isinstance(b, LoopInputBlock):
            continue

        def hooked(hidden, step, cache, orig=b.forward):
            orig(hidden, step, cache)
            got.append(hidden.cpu().clone())
        b.forward = hooked
    logits = r.step([StepEntry("a", toks, list(range(len(toks))))])
    assert len(got) == len(per_run) == len(plain.run_order(cases.CASES[name][0]))
    for i, (g, w) in enumerate(zip(got, per_run)):
        assert_close(g, w, dtype, f"{name} layer run {i}", bf16_rel_of_max=2e-2)
    assert_close(logits, ref, dtype, f"{name} logits")


@pytest.mark.parametrize("name,dtype", ENGINE_CASES)
def test_prefill_against_token_by_token_and_portions(root, name, dtype):
    """The same sequence whole, token by token from the first token on, and in portions of changing size
    down to two tokens with the last tokens one by one."""
    toks = tokens_for(root, name, dtype, 70, 2)
    ref = {"a": reference(root, name, dtype, toks)}
    r = runner_for(root, name, dtype, pages=80)
    t = Trace()
    for i, tok in enumerate(toks[:40]):
        t.step([("a", [tok], [0])], end=["a"] if i == 39 else [])
    check_trace(run_trace_inprocess(r, t), t, ref, dtype, f"{name} token by token")
    t = Trace()
    at = 0
    for n in (2, 5, 3, 17, 2, 9, 16, 1, 2, 7):
        t.step([("a", toks[at:at + n], [0, n - 1])])
        at += n
    while at < len(toks):
        t.step([("a", toks[at:at + 1], [0])], end=["a"] if at == len(toks) - 1 else [])
        at += 1
    check_trace(run_trace_inprocess(r, t), t, ref, dtype, f"{name} portions")
    r.cache.check()
    assert all(n == g.pool.num_pages for g, n in zip(r.cache.groups, r.cache.free_pages().values()))


@pytest.mark.parametrize("name,dtype", ENGINE_CASES)
def test_mixed_batches_with_pages_and_slots_used_again(root, name, dtype):
    """Up to four live requests of unequal length, portions beside single tokens, four state slots for seven
    requests and a pool that cannot hold all of them: what ends gives its pages and its slot (the recurrence's
    state, the convolution's inputs, the previous token) to the next.  Every row equals the request alone."""
    lens = {"a": 37, "b": 5, "c": 64, "d": 21, "e": 50, "f": 2, "g": 33}
    toks = {k: tokens_for(root, name, dtype, n, 10 + i) for i, (k, n) in enumerate(lens.items())}
    ref = {k: reference(root, name, dtype, v) for k, v in toks.items()}
    page = cases.CASES[name][2]
    pages = -(-64 // page) + -(-50 // page) + -(-37 // page) + -(-33 // page) + 1
    r = runner_for(root, name, dtype, pages=pages, requests=4)
    t = Trace()
    cursor = {k: 0 for k in lens}
    waiting, live = list(lens), []
    portion = {"a": [2, 16, 3], "b": [5], "c": [31, 2, 20], "d": [8, 8], "e": [3, 40], "f": [2], "g": [30]}
    step = 0
    while waiting or live:
        while waiting and len(live) < 4:
            need = sum(-(-lens[k] // page) for k in live + [waiting[0]])
            if need > pages:
                break
            live.append(waiting.pop(0))
        entries, ended = [], []
        for k in live:
            plan = portion[k]
            n = plan.pop(0) if plan else 1
            n = min(n, lens[k] - cursor[k])
            entries.append((k, toks[k][cursor[k]:cursor[k] + n], sorted({0, n - 1})))
            cursor[k] += n
            if cursor[k] == lens[k]:
                ended.append(k)
        t.step(entries, end=ended)
        live = [k for k in live if k not in ended]
        step += 1
        assert step < 400
    out = run_trace_inprocess(r, t)
    check_trace(out, t, ref, dtype, f"{name} mixed")
    info = r.cache.inspect()
    assert info["begun"] == len(lens) and info["live_requests"] == 0
    if r.cache.groups:
        assert any(g["reuses"] > 0 for g in info["groups"]), "no page was used again"
    r.cache.check()


@pytest.mark.parametrize("name,dtype", [("U", "float32"), ("V", "bfloat16"), ("W", "float32"), ("W", "bfloat16")])
def test_long_decoding_through_recorded_graphs(root, name, dtype):
    """A short prompt, then 200 single tokens (recorded decode graphs after the first): every window passes
    over decoded tokens many times, and the slow heads of the recurrence still carry the prompt at the end."""
    toks = tokens_for(root, name, dtype, 220, 3)
    ref = {"a": reference(root, name, dtype, toks)}
    r = runner_for(root, name, dtype, pages=-(-230 // cases.CASES[name][2]))
    t = Trace()
    t.step([("a", toks[:20], [19])])
    for i in range(20, len(toks)):
        t.step([("a", [toks[i]], [0])], end=["a"] if i == len(toks) - 1 else [])
    check_trace(run_trace_inprocess(r, t), t, ref, dtype, f"{name} long decoding")
    assert r.graphs is not None and r.graphs.whole and r.graphs.replays > 150


@pytest.mark.parametrize("name,dtype", [("U", "float32"), ("V", "float32"), ("X", "bfloat16"), ("W", "float32")])
def test_a_long_prompt_whole_and_in_portions(root, name, dtype):
    """700 tokens in one step (the recurrence runs in chunks side by side) against the same prompt in portions
    of 128 (chunks again, other borders), 100 and 37 (one pass each): the logits at a position do not depend on
    the cut; in 32-bit, where no routing decision is close, also against the plain model."""
    from inferloop_b200.engine import StepEntry
    toks = random_tokens(700, cases.CASES[name][0]["vocab"], 77)
    want = list(range(5, 700, 10)) + [699]
    r = runner_for(root, name, dtype, pages=-(-700 // cases.CASES[name][2]) + 2)
    whole = r.step([StepEntry("w", toks, want)]).float().cpu().clone()
    r.end("w")
    if dtype == "float32":
        model = cases.plain_model(root, name, stored(dtype))
        ref = model.forward(toks)
        if model.least_margin() > 1e-4:
            assert_close(whole, ref[want], dtype, f"{name} 700 tokens whole")
    for portion in (128, 100, 37):
        rows = []
        for at in range(0, 700, portion):
            part = toks[at:at + portion]
            out = r.step([StepEntry("p", part, [w - at for w in want if at <= w < at + len(part)])])
            rows.append(out.float().cpu().clone())
        r.end("p")
        if dtype == "float32":
            # two 32-bit evaluations whose recurrences add in another order: what differs is rounding, which a recurrence
            # over hundreds of tokens amplifies about tenfold; a key outside its window or a lost state differs by percents
            err = (torch.cat(rows).double() - whole.double()).abs().max()
            assert err <= 2e-5 * whole.abs().max(), f"{name} portions of {portion}: {float(err):.3e}"
        else:
            assert_close(torch.cat(rows), whole, dtype, f"{name} portions of {portion} against the whole prompt")


@pytest.mark.parametrize("name,dtype", [("U", "float32"), ("V", "bfloat16"), ("W", "float32")])
def test_greedy_generation_through_the_entry_point(root, name, dtype):
    from inferloop_b200 import Engine, SamplingParams
    config, _, page = cases.CASES[name]
    model = cases.plain_model(root, name, stored(dtype))
    prompts = [tokens_for(root, name, dtype, n, 30 + n) for n in (3, 12, 31, 64)]
    engine = Engine(cases.folder(root, name, stored(dtype)), dtype=dtype, block_size=page, num_gpu_blocks_override=96,
                    max_num_seqs=4, prefill_chunk_tokens=32, max_num_batched_tokens=40)
    new = 12
    got = engine.generate(prompts, SamplingParams(), max_new_tokens=new)
    for p, g in zip(prompts, got):
        assert len(g) == new
        ref = model.forward(list(p) + list(g))[len(p) - 1:-1]
        bound = (1e-2 if dtype == "bfloat16" else 1e-5) * float(ref.abs().max())
        for i, tok in enumerate(g):        # teacher-forced: every chosen token is the best one within the bound
            assert ref[i, tok] >= ref[i].max() - 2 * bound
    info = engine.inspect()
    assert info["running"] == 0 and all(g["free"] == g["total"] for g in info["cache"]["groups"])


def test_the_command_line_generates_from_a_mamevik_folder(root):
    name, dtype = "W", "float32"
    prompt = tokens_for(root, name, dtype, 9, 41)
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "infer"), "generate", cases.folder(root, name, stored(dtype)),
                          "--tokens", ",".join(map(str, prompt)), "--max-new-tokens", "6", "--dtype", dtype, "--block-size", "16",
                          "--num-gpu-blocks-override", "8"], capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, out.stderr
    got = json.loads(out.stdout.strip().splitlines()[-1])["tokens"]
    ref = cases.plain_model(root, name, stored(dtype)).forward(list(prompt) + got)[len(prompt) - 1:-1]
    for i, tok in enumerate(got):
        assert ref[i, tok] >= ref[i].max() - 2e-5 * float(ref.abs().max())


def test_the_trace_program_replays_a_mamevik_folder(root, tmp_path):
    name, dtype = "U", "float32"
    toks = {"x": tokens_for(root, name, dtype, 40, 5), "y": tokens_for(root, name, dtype, 9, 6)}
    ref = {k: reference(root, name, dtype, v) for k, v in toks.items()}
    t = Trace()
    t.step([("x", toks["x"][:33], [0, 32]), ("y", toks["y"][:2], [1])])
    t.step([("x", toks["x"][33:34], [0]), ("y", toks["y"][2:], [0, 6])], end=["y"])
    for i in range(34, 40):
        t.step([("x", toks["x"][i:i + 1], [0])], end=["x"] if i == 39 else [])
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", cases.folder(root, name, stored(dtype)), "--dtype", dtype,
           "--out", str(tmp_path), "--max-tokens", "128", "--block-size", "4"]
    proc = subprocess.run(cmd, input=t.lines(), capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr
    vocab = cases.CASES[name][0]["vocab"]
    out = {s: np.fromfile(os.path.join(str(tmp_path), f"{s}.f32"), dtype="<f4").reshape(len(rows), vocab) for s, rows in t.rows.items()}
    check_trace(out, t, ref, dtype, "trace program")


# ------------------------------------------------------------------------------ each mechanism alone
class FakeStep:
    """The device arrays of a batch, for kernels called without an engine: sequences of `lens` tokens that
    start at `starts`, in slots `slots`."""

    def __init__(self, lens, starts, slots, tokens=None):
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
        self.h_q_len = list(lens)
        self.n_seqs, self.n_tokens = len(lens), sum(lens)
        self.max_q_len = max(lens)
        self.decode_only = all(n == 1 for n in lens)
        self.cu_q = i32([sum(lens[:i]) for i in range(len(lens) + 1)])
        self.positions = i32([s + j for n, s in zip(lens, starts) for j in range(n)])
        self.seq_of_token = i32([i for i, n in enumerate(lens) for _ in range(n)])
        self.slots = i32(slots)
        self.h_kv_len = [s + n for n, s in zip(lens, starts)]
        self.max_kv_len = max(self.h_kv_len)
        self.tokens = i32(tokens if tokens is not None else [0] * self.n_tokens)


def f32(t):
    return t.float().to(DEV).contiguous()


@pytest.mark.parametrize("buckets,mul_prev,mul_cur", [(97, 13, 5), (1, 1, 1), (2039, 2147483647, 2147483629)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_with_hashed_pairs(buckets, mul_prev, mul_cur, dtype):
    """Rows of the two tables, the first token's own row, the token before a portion from the state slot, slots
    that are taken over by another request; multipliers whose products need 64 bits."""
    from inferloop_b200.csrc import ops
    g = torch.Generator().manual_seed(buckets)
    V, H, eps = 50, 40, 1e-5
    E = torch.randn(V, H, generator=g).to(dtype)
    P = torch.randn(buckets + 1, H, generator=g).to(dtype)
    w = 1 + 0.1 * torch.randn(H, generator=g)
    seqs = {0: random_tokens(9, V, 1), 1: random_tokens(4, V, 2)}
    state = torch.full((3,), 12345, dtype=torch.int32, device=DEV)

    def want(tokens):
        x = E.double()[torch.tensor(tokens)] + P.double()[torch.tensor(plain.bigram_rows(tokens, dict(buckets=buckets, mul_prev=mul_prev, mul_cur=mul_cur)))]
        return plain.rms(x, eps) * w.double()

    # step 1: sequence 0 brings tokens 0..4 (slot 2), sequence 1 its first token (slot 0); step 2: the rest
    for lens, starts, parts in (([5, 1], [0, 0], [(0, 0, 5), (1, 0, 1)]), ([4, 3], [5, 1], [(0, 5, 9), (1, 1, 4)])):
        toks = [t for s, a, b in parts for t in seqs[s][a:b]]
        step = FakeStep(lens, starts, [2, 0], toks)
        out = torch.empty(sum(lens), H, dtype=torch.float32, device=DEV)
        keep = torch.empty_like(out)
        ops.embed_pairs(step, E.to(DEV), P.to(DEV), buckets, mul_prev, mul_cur, state, f32(w), eps, out, keep)
        ops.store_last_tokens(step, state)
        ref = torch.cat([want(seqs[s])[a:b] for s, a, b in parts])
        assert_close(out, ref, "float32", "embedding rows")
        assert torch.equal(out, keep)
    assert state.tolist() == [seqs[1][-1], 12345, seqs[0][-1]]


@pytest.mark.parametrize("taps,channels", [(1, 40), (2, 130), (4, 256), (5, 33), (16, 8)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_short_convolution_with_state(taps, channels, dtype):
    """Whole sequences, then the same in portions (1, 2, 17, 40 tokens; shorter and longer than the taps and than
    a block's tile) through the state slot, two sequences side by side, slots out of order."""
    from inferloop_b200.csrc import ops
    g = torch.Generator().manual_seed(taps * 1000 + channels)
    lens = [61, 23]
    raw = [torch.randn(n, channels + 7, generator=g).to(dtype) for n in lens]
    w, b = torch.randn(channels, taps, generator=g), torch.randn(channels, generator=g)
    ref = [plain.silu(plain.causal_conv(r.double()[:, 3:3 + channels], w.double(), b.double())) for r in raw]
    state = torch.full((4, max(taps - 1, 0), channels), 9.0, dtype=torch.float32, device=DEV)
    state[1].zero_(); state[3].zero_()
    cuts = [[1, 2, 17, 40, 1], [23], [], [], []]
    at = [0, 0]
    for i in range(5):
        parts = [(s, at[s], at[s] + cuts[s][i]) for s in (0, 1) if i < len(cuts[s])]
        step = FakeStep([b_ - a for _, a, b_ in parts], [a for _, a, _ in parts], [3 if s == 0 else 1 for s, _, _ in parts])
        x = torch.cat([raw[s][a:b_] for s, a, b_ in parts]).to(DEV)
        out = torch.empty(x.shape[0], channels, dtype=torch.float32, device=DEV)
        ops.ssm_conv(x, 3, channels, f32(w), f32(b), state, step, out)
        assert_close(out, torch.cat([ref[s][a:b_] for s, a, b_ in parts]), "float32", f"conv step {i}")
        for s, a, b_ in parts:
            at[s] = b_
    if taps > 1:
        assert float(state[0].min()) == 9.0 and float(state[2].min()) == 9.0      # slots of nobody are left alone
        assert torch.equal(state[3].cpu(), raw[0][61 - (taps - 1):, 3:3 + channels].float())


@pytest.mark.parametrize("heads,P,N,groups", [(4, 12, 16, 1), (6, 8, 40, 3), (2, 80, 200, 1), (8, 64, 128, 2), (3, 64, 64, 3)])
def test_recurrence_in_one_pass_in_chunks_and_in_portions(heads, P, N, groups):
    """The scan against the token-by-token recurrence in 64-bit: a whole sequence in one pass, in chunks side by
    side, and in portions through the state slot; two sequences; a head whose decay is so slow that the first
    token, made to stand out, still decides the last output."""
    from inferloop_b200.csrc import ops
    from inferloop_b200.parts.base import Workspace
    g = torch.Generator().manual_seed(heads * 100 + N)
    lens = [300, 45]
    inner, channels = heads * P, heads * P + 2 * groups * N
    act = [0.5 * torch.randn(n, channels, generator=g) for n in lens]
    act[0][0, :inner] *= 30.0                                            # the first token's input stands out
    dt_raw = [torch.randn(n, heads + 5, generator=g) for n in lens]
    dt_bias = torch.linspace(-6.0, 0.5, heads)
    a_log = torch.linspace(-4.0, 0.5, heads)
    skip = torch.randn(heads, generator=g)
    ref = []
    for a, d in zip(act, dt_raw):
        a, n = a.double(), a.shape[0]
        dd = plain.softplus(d.double()[:, 2:2 + heads] + dt_bias.double())
        ref.append(plain.recurrence(a[:, :inner].reshape(n, heads, P), a[:, inner:inner + groups * N].reshape(n, groups, N),
                                    a[:, inner + groups * N:].reshape(n, groups, N), dd, a_log.double(), skip.double(), heads,
                                    groups).reshape(n, inner))
    # without the first token the last output of the slowest head is another one: the test would see a lost state
    assert float(ref[0][-1, :P].abs().max()) > 0
    ws = Workspace(torch.device(DEV))
    for mode, cuts in (("one pass", [[300], [45]]), ("chunks", [[300], [45]]), ("portions", [[1, 2, 130, 17, 150], [40, 5]])):
        state = torch.full((3, heads, N, P), 5.0, dtype=torch.float32, device=DEV)
        state[0].zero_(); state[2].zero_()
        at = [0, 0]
        for i in range(max(len(c) for c in cuts)):
            parts = [(s, at[s], at[s] + cuts[s][i]) for s in (0, 1) if i < len(cuts[s])]
            step = FakeStep([b - a for _, a, b in parts], [a for _, a, _ in parts], [2 if s == 0 else 0 for s, _, _ in parts])
            x = torch.cat([act[s][a:b] for s, a, b in parts]).to(DEV)
            d = torch.cat([dt_raw[s][a:b] for s, a, b in parts]).to(DEV)
            y = torch.empty(x.shape[0], inner, dtype=torch.float32, device=DEV)
            chunk = {"one pass": 0, "chunks": 64, "portions": None}[mode]
            ops.ssm_scan(x, d, 2, f32(dt_bias), f32(a_log), f32(skip), state, y, step, heads, P, N, groups, workspace=ws, chunk=chunk)
            want = torch.cat([ref[s][a:b] for s, a, b in parts])
            err = (y.double().cpu() - want).abs().max() / want.abs().max()
            assert err < 2e-5, f"{mode} step {i}: {float(err):.3e}"
            for s, a, b in parts:
                at[s] = b
        assert float(state[1].min()) == 5.0


@pytest.mark.parametrize("width,groups", [(48, 1), (96, 3), (512, 2), (4096, 1), (8192, 1)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("pad", [9, 8])          # rows of the gate on odd and on 16-byte boundaries (the four-element accesses)
def test_gate_and_grouped_norm(width, groups, dtype, pad):
    from inferloop_b200.csrc import ops
    g = torch.Generator().manual_seed(width + groups)
    T = 7
    y = torch.randn(T, width, generator=g)
    z = torch.randn(T, width + pad, generator=g).to(dtype)
    w = 1 + 0.1 * torch.randn(width, generator=g)
    out = torch.empty(T, width, dtype=dtype, device=DEV)
    ops.gated_group_norm(f32(y), z.to(DEV), f32(w), 1e-5, groups, out)
    ref = plain.group_rms(y.double() * plain.silu(z.double()[:, :width]), groups, 1e-5) * w.double()
    if dtype == torch.float32:
        assert_close(out, ref, "float32", "gated norm")
    else:
        assert (out.double().cpu() - ref).abs().max() <= 2.0 ** -8 * ref.abs().max()


def _paged(c, page_size, pages_total, order):
    """A latent cache [pages, 1, page_size, rank] that holds c [n, rank] in the pages `order`."""
    n, rank = c.shape
    cache = torch.zeros(pages_total, 1, page_size, rank, dtype=c.dtype, device=DEV)
    for i in range(n):
        cache[order[i // page_size], 0, i % page_size] = c[i]
    return cache


@pytest.mark.parametrize("dtype,rank,heads,window", [
    (torch.float32, 24, 3, 7), (torch.float32, 300, 2, None), (torch.bfloat16, 64, 8, 33), (torch.bfloat16, 96, 5, 37),
    (torch.bfloat16, 128, 16, 100), (torch.bfloat16, 128, 5, None), (torch.bfloat16, 40, 2, 5), (torch.bfloat16, 32, 4, 20), (torch.bfloat16, 64, 20, 50),
    (torch.bfloat16, 96, 17, None), (torch.float32, 128, 2, 300)])
def test_attention_with_a_sink_and_a_window_over_cached_latents(dtype, rank, heads, window):
    """Keys and values are the same cached vectors; the softmax's denominator holds a sink per head.  Prompt
    portions and single tokens; pages out of order; a key that stands out sits just inside the window of one
    query and just outside the next one's; sinks that dominate, match and vanish."""
    from inferloop_b200.csrc import ops
    from inferloop_b200.parts.base import Workspace
    g = torch.Generator().manual_seed(rank + heads)
    n, page = 150, 16
    c = torch.randn(n, rank, generator=g)
    q = torch.randn(n, heads, rank, generator=g)
    scale = 1.0 / math.sqrt(rank)
    hot = 60                                            # every query likes key 60 a lot
    c[hot] *= 3.0
    q += 1.5 * c[hot] / c[hot].norm() * math.sqrt(rank) / 3.0
    sink = torch.linspace(-3.0, 6.0, heads)
    c, q = c.to(dtype), q.to(dtype)
    ref = plain.windowed_sink_attention(q.double(), c.double()[:, None, :].expand(n, heads, rank), c.double()[:, None, :].expand(n, heads, rank),
                                        scale, window, sink.double()).reshape(n, heads * rank)
    order = list(range(11, 0, -1))
    cache = _paged(c.to(DEV), page, 12, order)
    table = torch.tensor([order + [-1] * 4], dtype=torch.int32, device=DEV)
    ws = Workspace(torch.device(DEV))
    qd = q.reshape(n, heads * rank).to(DEV)

    def run(a, b):
        step = FakeStep([b - a], [a], [0])
        out = torch.empty(b - a, heads * rank, dtype=dtype, device=DEV)
        ops.attention(qd[a:b].contiguous(), out, cache, cache, step, table, window or 0, scale, heads, 1, rank, workspace=ws, sink=f32(sink))
        return out
    got = torch.cat([run(0, 50), run(50, 52), run(52, 131)] + [run(i, i + 1) for i in range(131, n)])
    if dtype == torch.float32:
        assert_close(got, ref, "float32", "attention")
    else:
        assert (got.double().cpu() - ref).abs().max() <= 2.0 ** -7 * ref.abs().max()
    if window is not None and hot + window < n:          # the edge is really seen: the row that still reads the hot key differs from the next
        assert (ref[hot + window - 1] - ref[hot + window]).abs().max() > 0.05 * ref.abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,K,N", [(3, 8, 24), (2, 40, 8), (8, 64, 64), (4, 128, 200), (1, 512, 16)])
def test_products_per_head_and_the_latent_write(dtype, heads, K, N):
    from inferloop_b200.csrc import ops
    g = torch.Generator().manual_seed(heads + K + N)
    x = torch.randn(150, heads * K + (12 if K % 16 == 0 else 11), generator=g).to(dtype)     # (even row strides reach the tensor-core form)
    w = (torch.randn(heads, K, N, generator=g) / math.sqrt(K)).to(dtype)
    for T in (150, 37, 16, 3):                # many tokens, and the few-token form whose k range is cut in four
        out = torch.empty(T, heads * N, dtype=dtype, device=DEV)
        ops.head_matmul(x[:T].to(DEV), w.to(DEV), out)
        ref = torch.einsum("thk,hkn->thn", x.double()[:T, :heads * K].reshape(T, heads, K), w.double()).reshape(T, heads * N)
        if dtype == torch.float32:
            assert_close(out, ref, "float32", f"per-head product of {T} tokens")
        else:
            assert (out.double().cpu() - ref).abs().max() <= 2.0 ** -8 * ref.abs().max()
    T = 37
    # the latent: columns heads * K - 5 .. of x, normed, into pages out of order; a dummy row (no page) is dropped
    rank, page = 16, 4
    gw = 1 + 0.1 * torch.randn(rank, generator=g)
    cache = torch.full((12, 1, page, rank), 7.0, dtype=dtype, device=DEV)
    step = FakeStep([30, 6, 1], [3, 0, 0], [0, 1, -1])
    table = torch.tensor([[5, 9, 2, 7, 0, 1, 3, 4, 6], [11, 10] + [-1] * 7, [-1] * 9], dtype=torch.int32, device=DEV)
    col0 = heads * K - 5
    ops.latent_write(x[:T].to(DEV), col0, rank, f32(gw), 1e-5, step, table, cache)
    want = plain.rms(x.double()[:T, col0:col0 + rank], 1e-5) * gw.double()
    for t, (seq, pos) in enumerate([(0, 3 + i) for i in range(30)] + [(1, i) for i in range(6)]):
        got = cache[int(table[seq, pos // page]), 0, pos % page].double().cpu()
        assert (got - want[t]).abs().max() <= (1e-5 if dtype == torch.float32 else 2.0 ** -8 * float(want[t].abs().max()))
    assert float(cache[8].min()) == 7.0
    # both at once, as steps of few tokens run them: the same latents, the same mapped queries
    if col0 + rank <= x.shape[1] and col0 >= 0:
        cache2 = torch.full((12, 1, page, rank), 7.0, dtype=dtype, device=DEV)
        few = FakeStep([9, 6, 1], [3, 0, 0], [0, 1, -1])
        q1 = torch.empty(16, heads * N, dtype=dtype, device=DEV)
        q2 = torch.empty(16, heads * N, dtype=dtype, device=DEV)
        xd = x[:16].to(DEV)
        ops.latent_input(xd, w.to(DEV), q1, col0, rank, f32(gw), 1e-5, few, table, cache2)
        ops.head_matmul(xd, w.to(DEV), q2)
        cache3 = torch.full((12, 1, page, rank), 7.0, dtype=dtype, device=DEV)
        ops.latent_write(xd, col0, rank, f32(gw), 1e-5, few, table, cache3)
        assert torch.equal(q1, q2) and torch.equal(cache2, cache3)


@pytest.mark.parametrize("experts,top", [(5, 2), (3, 3), (8, 1), (40, 4)])
def test_routing_with_a_bias_and_the_softmax_over_the_chosen(experts, top):
    from inferloop_b200.csrc import ops
    g = torch.Generator().manual_seed(experts * 10 + top)
    T = 29
    z = 3.0 * torch.randn(T, experts, generator=g)
    b = 2.0 * torch.randn(experts, generator=g)
    choice = torch.empty(T * top, dtype=torch.int32, device=DEV)
    weight = torch.empty(T * top, dtype=torch.float32, device=DEV)
    ops.moe_route(f32(z), experts, top, True, True, choice, weight, bias=f32(b))
    best = torch.topk(z.double() + b.double(), top, dim=-1)
    assert torch.equal(choice.view(T, top).cpu().long(), best.indices)
    assert_close(weight.view(T, top), torch.softmax(best.values, dim=-1), "float32", "weights")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_gated_unit_with_clamped_halves(dtype):
    from inferloop_b200.csrc import ops
    g = torch.Generator().manual_seed(5)
    x = (3.0 * torch.randn(19, 2 * 24, generator=g)).to(dtype)
    out = torch.empty(19, 24, dtype=dtype, device=DEV)
    ops.glu_mul(x.to(DEV), out, 1.25, 1.702, 1.0)
    gate, up = x.double()[:, :24].clamp(max=1.25), x.double()[:, 24:].clamp(-1.25, 1.25)
    ref = gate * torch.sigmoid(1.702 * gate) * (up + 1.0)
    assert (out.double().cpu() - ref).abs().max() <= (1e-6 if dtype == torch.float32 else 2.0 ** -8 * ref.abs().max())


def test_the_gated_unit_in_the_grouped_tensor_core_product():
    """Rows sorted by expert through the tcgen05 product with gate and up rows interleaved in blocks of 64: its
    epilogue clamps both halves, takes g * sigmoid(1.702 g) and adds one to the linear half."""
    from inferloop_b200.csrc import ops
    g = torch.Generator().manual_seed(9)
    E, I, H, rows = 3, 128, 256, 384
    a = torch.randn(rows, H, generator=g).to(torch.bfloat16)
    gate = (torch.randn(E, I, H, generator=g) / 4).to(torch.bfloat16)
    up = (torch.randn(E, I, H, generator=g) / 4).to(torch.bfloat16)
    w = torch.stack([torch.stack([gate[e].view(I // 64, 64, H), up[e].view(I // 64, 64, H)], dim=1).reshape(2 * I, H) for e in range(E)])
    blocks = torch.tensor([2, 0, 1], dtype=torch.int32, device=DEV)
    out = torch.empty(rows, I, dtype=torch.bfloat16, device=DEV)
    ops.moe_gemm_tc(a.to(DEV), w.to(DEV).contiguous(), out, blocks, swiglu=True, act=(2.0, 1.702, 1.0))
    for i, e in enumerate([2, 0, 1]):
        x = a[i * 128:(i + 1) * 128].double()
        gt, u = (x @ gate[e].double().T).clamp(max=2.0), (x @ up[e].double().T).clamp(-2.0, 2.0)
        ref = gt * torch.sigmoid(1.702 * gt) * (u + 1.0)
        assert (out[i * 128:(i + 1) * 128].double().cpu() - ref).abs().max() <= 2.0 ** -7 * ref.abs().max()
    ops.check_device_errors()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_with_a_weight_stored_around_zero_and_the_loop_input(dtype):
    from inferloop_b200.config.spec import PartSpec
    from inferloop_b200.csrc import ops
    from inferloop_b200.parts import registry
    from inferloop_b200.parts.base import BuildContext, Workspace
    from inferloop_b200.cache.manager import LayerCache
    g = torch.Generator().manual_seed(3)
    T, H = 21, 64
    ctx = BuildContext(dtype, torch.device(DEV), Workspace(torch.device(DEV)))
    norm = registry.build_norm(PartSpec.make("rms", eps=1e-5, weight_suffix="", offset=1.0), ctx, "n", width=H)
    w = 0.3 * torch.randn(H, generator=g)
    norm.bind({"n": f32(w)})
    x = torch.randn(T, H, generator=g)
    out = torch.empty(T, H, dtype=torch.float32, device=DEV)
    norm.forward(f32(x), out)
    assert_close(out, plain.norm_offset(x.double(), w.double(), 1e-5), "float32", "norm")
    block = registry.build_block(type("L", (), {"block": PartSpec.make("loop_input", hidden_size=H, times=3, source="kept")})(), ctx, "loop.")
    M = (torch.randn(H, 2 * H, generator=g) / 8).to(dtype)
    s = torch.randn(3, H, generator=g)
    block.bind({"loop.in": M.to(DEV), "loop.step": f32(s)})
    x0 = torch.randn(T, H, generator=g)
    ctx.workspace.buffer("kept", (T, H), torch.float32).copy_(x0)
    hidden = f32(x)
    block.forward(hidden, None, LayerCache(0, None, 16, None, None, True, {}, 2))
    cat = torch.cat([x, x0], dim=-1).to(dtype).double()
    ref = cat @ M.double().T + s.double()[2]
    if dtype == torch.float32:
        assert_close(hidden, ref, "float32", "loop input")
    else:
        assert (hidden.double().cpu() - ref).abs().max() <= 2.0 ** -8 * ref.abs().max()
