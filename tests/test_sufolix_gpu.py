"""The Sufolix decoder through the engine, and each of its mechanisms alone (GPU), against the
plain 64-bit statement in plain_sufolix.py.  The configurations are in sufolix_cases.py: P (odd
sizes, three streams, values wider than keys, exact kernels), Q (the serving kernels' geometry),
R (no streams, one kv head per head), S (four streams, values narrower than keys, one kv head).
"""
import math

import numpy as np
import pytest
import torch

import plain_sufolix as plain
import sufolix_cases as cases
from helpers import Trace, assert_close, check_trace, run_trace_inprocess

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def root(tmp_path_factory):
    return str(tmp_path_factory.mktemp("sufolix"))


def stored(dtype):
    return torch.bfloat16 if dtype == "bfloat16" else torch.float32


def runner_for(root, name, dtype, pages=64, requests=4, page=None):
    from inferloop_b200.engine import ModelRunner
    _, _, page_size = cases.CASES[name]
    return ModelRunner.from_folder(cases.folder(root, name, stored(dtype)), dtype=dtype, device=DEV,
                                   page_size=page or page_size, num_pages=pages, max_requests=requests)


def tokens_for(root, name, dtype, n, seed):
    model = cases.plain_model(root, name, stored(dtype))
    margin = 4e-2 if dtype == "bfloat16" else 1e-4
    return cases.decided_tokens(model, n, cases.CASES[name][0]["vocab"], seed, margin)


def reference(root, name, dtype, tokens):
    return cases.plain_model(root, name, stored(dtype)).forward(tokens)


ENGINE_CASES = [("P", "float32"), ("P", "bfloat16"), ("Q", "float32"), ("Q", "bfloat16"), ("R", "bfloat16"),
                ("R", "float32"), ("S", "float32"), ("S", "bfloat16")]


# ------------------------------------------------------------------------------ the engine
@pytest.mark.parametrize("name,dtype", ENGINE_CASES)
def test_whole_prompt_and_every_layer(root, name, dtype):
    """One prompt in one step: the sum of the streams after every layer, and all logits."""
    from inferloop_b200.engine import StepEntry
    r = runner_for(root, name, dtype)
    toks = tokens_for(root, name, dtype, 45, 1)
    per_layer = []
    ref = cases.plain_model(root, name, stored(dtype)).forward(toks, per_layer)
    got_layers = []
    S, H = r.spec.residual_streams, r.spec.hidden_size
    for b in r.model.blocks:
        def hooked(hidden, step, cache, orig=b.forward):
            orig(hidden, step, cache)
            got_layers.append(hidden.view(hidden.shape[0], S, H).sum(1).cpu().clone())
        b.forward = hooked
    logits = r.step([StepEntry("a", toks, list(range(len(toks))))])
    for i, (g, w) in enumerate(zip(got_layers, per_layer)):
        assert_close(g, w, dtype, f"{name} layer {i}", bf16_rel_of_max=2e-2)
    assert_close(logits, ref, dtype, f"{name} logits")


@pytest.mark.parametrize("name,dtype", ENGINE_CASES)
def test_prefill_against_token_by_token_and_portions(root, name, dtype):
    """The same sequence whole, token by token from the first token on, and in portions of
    changing size down to two tokens with the last tokens one by one."""
    toks = tokens_for(root, name, dtype, 70, 2)
    ref = {"a": reference(root, name, dtype, toks)}
    r = runner_for(root, name, dtype, pages=80)
    t = Trace()
    for i, tok in enumerate(toks[:40]):                           # every token alone: the first tokens of a sequence too
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
    """Up to four live requests of unequal length, portions beside single tokens, on a pool
    that cannot hold all of them at once: requests end, their pages and slots serve the next.
    Every row equals the request alone."""
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
    assert any(g["reuses"] > 0 for g in info["groups"]), "no page was used again"
    r.cache.check()


@pytest.mark.parametrize("name,dtype", [("P", "float32"), ("Q", "bfloat16"), ("S", "bfloat16")])
def test_long_decoding_through_recorded_graphs(root, name, dtype):
    """A short prompt, then 300 single tokens (recorded decode graphs after the first)."""
    toks = tokens_for(root, name, dtype, 330, 3)
    ref = {"a": reference(root, name, dtype, toks)}
    r = runner_for(root, name, dtype, pages=-(-340 // cases.CASES[name][2]))
    t = Trace()
    t.step([("a", toks[:30], [29])])
    for i in range(30, len(toks)):
        t.step([("a", [toks[i]], [0])], end=["a"] if i == len(toks) - 1 else [])
    check_trace(run_trace_inprocess(r, t), t, ref, dtype, f"{name} long decoding")
    if r.graphs is not None:
        assert r.graphs.replays > 200


@pytest.mark.parametrize("name,dtype", [("Q", "bfloat16"), ("R", "bfloat16"), ("S", "float32")])
def test_a_long_prompt_whole_and_in_portions(root, name, dtype):
    """900 tokens in one step (at Q's sizes the experts then run on the wide tiles, the attention
    on two row blocks) against the same prompt in portions of 128 and 100: the logits at a position
    do not depend on the cut.  Keys far back count: every tenth row is compared."""
    from helpers import random_tokens
    from inferloop_b200.engine import StepEntry
    vocab = cases.CASES[name][0]["vocab"]
    toks = random_tokens(900, vocab, 77)
    want = list(range(5, 900, 10)) + [899]
    r = runner_for(root, name, dtype, pages=-(-900 // cases.CASES[name][2]) + 2)
    whole = r.step([StepEntry("w", toks, want)]).float().cpu().clone()
    r.end("w")
    for portion in (128, 100):
        rows = []
        for at in range(0, 900, portion):
            part = toks[at:at + portion]
            out = r.step([StepEntry("p", part, [w - at for w in want if at <= w < at + len(part)])])
            rows.append(out.float().cpu().clone())
        r.end("p")
        assert_close(torch.cat(rows), whole, dtype, f"{name} portions of {portion} against the whole prompt")


@pytest.mark.parametrize("name,dtype", [("P", "float32"), ("Q", "bfloat16"), ("R", "float32")])
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


def test_the_command_line_generates_from_a_sufolix_folder(root):
    import json, os, subprocess, sys
    from helpers import ROOT
    name, dtype = "R", "float32"
    prompt = tokens_for(root, name, dtype, 9, 41)
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "infer"), "generate", cases.folder(root, name, stored(dtype)),
                          "--tokens", ",".join(map(str, prompt)), "--max-new-tokens", "6", "--dtype", dtype, "--block-size", "16",
                          "--num-gpu-blocks-override", "8"], capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, out.stderr
    got = json.loads(out.stdout.strip().splitlines()[-1])["tokens"]
    model = cases.plain_model(root, name, stored(dtype))
    ref = model.forward(list(prompt) + got)[len(prompt) - 1:-1]
    for i, tok in enumerate(got):
        assert ref[i, tok] >= ref[i].max() - 2e-5 * float(ref.abs().max())


def test_the_trace_program_replays_a_sufolix_folder(root, tmp_path):
    from helpers import run_trace_program
    name, dtype = "S", "float32"
    toks = {"x": tokens_for(root, name, dtype, 40, 5), "y": tokens_for(root, name, dtype, 9, 6)}
    ref = {k: reference(root, name, dtype, v) for k, v in toks.items()}
    t = Trace()
    t.step([("x", toks["x"][:33], [0, 32]), ("y", toks["y"][:2], [1])])
    t.step([("x", toks["x"][33:34], [0]), ("y", toks["y"][2:], [0, 6])], end=["y"])
    for i in range(34, 40):
        t.step([("x", toks["x"][i:i + 1], [0])], end=["x"] if i == 39 else [])
    import json, os, subprocess, sys
    from helpers import ROOT
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", cases.folder(root, name, stored(dtype)), "--dtype", dtype,
           "--out", str(tmp_path), "--max-tokens", "128", "--block-size", "4"]
    proc = subprocess.run(cmd, input=t.lines(), capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr
    vocab = cases.CASES[name][0]["vocab"]
    out = {s: np.fromfile(os.path.join(str(tmp_path), f"{s}.f32"), dtype="<f4").reshape(len(rows), vocab) for s, rows in t.rows.items()}
    check_trace(out, t, ref, dtype, "trace program")


# ------------------------------------------------------------------------------ each mechanism alone
@pytest.mark.parametrize("streams,width", [(1, 40), (2, 256), (3, 96), (4, 1536), (7, 33)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_streams_read_and_write(streams, width, out_dtype):
    from inferloop_b200.csrc import ops
    g = torch.Generator().manual_seed(streams * 100 + width)
    T = 13
    x = torch.randn(T, streams, width, generator=g, dtype=torch.float64)
    a, b = torch.randn(streams, generator=g, dtype=torch.float64), torch.randn(streams, generator=g, dtype=torch.float64)
    M = torch.randn(streams, streams, generator=g, dtype=torch.float64)
    w = 1 + 0.1 * torch.randn(width, generator=g, dtype=torch.float64)
    y = torch.randn(T, width, generator=g, dtype=torch.float64)
    f = lambda t: t.float().to(DEV)
    xd = f(x).view(T, streams * width).contiguous()
    normed = torch.empty(T, width, dtype=out_dtype, device=DEV)
    u_out = torch.empty(T, width, dtype=torch.float32, device=DEV)
    zero = torch.full((T, width), 7.0, dtype=torch.float32, device=DEV)
    ops.streams_read(xd, f(a), streams, f(w), 1e-5, normed=normed, u_out=u_out, y_zero=zero)
    u = sum(a[s] * x[:, s] for s in range(streams))
    assert_close(u_out, u, "float32", "u")
    ref = plain.rms(u.float().double(), 1e-5, w.float().double())
    if out_dtype == torch.float32:
        assert_close(normed, ref, "float32", "normed")
    else:
        assert (normed.double().cpu() - ref).abs().max() <= 2.0 ** -8 * ref.abs().max()
    assert float(zero.abs().max()) == 0.0
    ops.streams_write(xd, f(y), f(M), f(b), streams)
    want = torch.stack([sum(M[s, t] * x[:, s] for s in range(streams)) + b[t] * y for t in range(streams)], dim=1)
    assert_close(xd.view(T, streams, width), want.float().double(), "float32", "streams after the write")
    # streams = 1 with unit coefficients is the plain residual sum
    if streams == 1:
        one = torch.ones(1, device=DEV)
        x1 = f(x).view(T, width).contiguous()
        ops.streams_write(x1, f(y), one.view(1, 1), one, 1)
        assert torch.equal(x1, f(x).view(T, width) + f(y))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,d,dv,rd", [(6, 3, 16, 24, 8), (4, 1, 32, 16, 32), (2, 2, 64, 64, 2), (8, 2, 128, 128, 128),
                                            (5, 5, 128, 128, 64), (3, 1, 128, 128, 6)])
def test_rotation_of_neighbours_norm_after_it_and_mixed_values(dtype, nq, nkv, d, dv, rd):
    """The projection output through the fused kernel in the order rotation (pairs of neighbours) ->
    root-mean-square division, with the values kept by a first layer and mixed by a later one, into
    cache pages; against the plain functions."""
    from inferloop_b200.csrc import ops
    g = torch.Generator().manual_seed(nq * 7 + d)
    T, page, eps, base = 19, 4, 1e-5, 3000.0
    width = (nq + nkv) * d + nkv * dv
    qkv = torch.randn(T, width, generator=g).to(dtype)
    positions = torch.tensor([5 * i % 23 for i in range(T)], dtype=torch.int32)        # any positions, one sequence per token below
    seq = torch.arange(T, dtype=torch.int32)
    table = torch.arange(T * 8, dtype=torch.int32).view(T, 8)                        # sequence s owns pages 8 s .. 8 s + 7
    inv = torch.tensor([base ** (-2.0 * i / rd) for i in range(rd // 2)], dtype=torch.float64)
    rope = torch.empty(T, rd // 2, 2, dtype=torch.float32, device=DEV)
    ops.rope_table(positions.to(DEV), inv.to(DEV), rope)
    kc = torch.zeros(T * 8, nkv, page, d, dtype=dtype, device=DEV)
    vc = torch.zeros(T * 8, nkv, page, dv, dtype=dtype, device=DEV)
    q_out = torch.empty(T, nq * d, dtype=dtype, device=DEV)
    v_first = torch.empty(T, nkv * dv, dtype=dtype, device=DEV)
    mode = ops.ROPE_INTERLEAVED | ops.NORM_AFTER_ROTATION | ops.NORM_UNWEIGHTED
    call = lambda **kw: ops.qk_norm_rope_cache(qkv.to(DEV), q_out, None, None, eps, rope, rd, positions.to(DEV), seq.to(DEV),
                                               table.to(DEV), page, kc, vc, nq, nkv, d, dv, mode, v_first=v_first, **kw)
    call(v_keep=True)
    x = qkv.double()
    q = x[:, :nq * d].view(T, nq, d)
    k = x[:, nq * d:(nq + nkv) * d].view(T, nkv, d)
    v = x[:, (nq + nkv) * d:].view(T, nkv, dv)
    q_ref = plain.rms(plain.rotate_pairs(q, positions, base, rd), eps)
    k_ref = plain.rms(plain.rotate_pairs(k, positions, base, rd), eps)
    tol = "float32" if dtype == torch.float32 else "bfloat16"

    def cached(c, width_):
        rows = [c[int(table[t, int(positions[t]) // page]), :, int(positions[t]) % page] for t in range(T)]
        return torch.stack(rows).view(T, nkv, width_)
    assert_close(q_out.view(T, nq, d), q_ref, tol, "q")
    assert_close(cached(kc, d), k_ref, tol, "k in the cache")
    assert_close(cached(vc, dv), v, tol, "v in the cache")
    assert_close(v_first.view(T, nkv, dv), v, tol, "kept values")
    # a later layer: other values, mixed with the kept ones
    lam = torch.tensor([0.37], dtype=torch.float32, device=DEV)
    v2 = torch.randn(T, nkv * dv, generator=g).to(dtype)
    qkv = torch.cat([qkv[:, :(nq + nkv) * d], v2], dim=1).contiguous()
    call(v_lambda=lam)
    want = (1 - 0.37) * v2.double().view(T, nkv, dv) + 0.37 * v
    assert_close(cached(vc, dv), want, tol, "mixed values in the cache")
    # the stock pairing (i with i + rd/2) gives something else as soon as there are two pairs
    if rd >= 4:
        ops.qk_norm_rope_cache(qkv.to(DEV), q_out, None, None, eps, rope, rd, positions.to(DEV), seq.to(DEV), table.to(DEV), page, kc,
                               vc, nq, nkv, d, dv, ops.NORM_UNWEIGHTED)
        assert (q_out.view(T, nq, d).double().cpu() - q_ref).abs().max() > 1e-2


@pytest.mark.parametrize("d,dv", [(16, 24), (32, 16), (64, 64), (48, 200)])
def test_exact_attention_with_values_of_their_own_size_and_a_far_key(d, dv):
    """Keys of size d, values of size dv.  One key far back is made to stand out (its score is
    raised by scaling it), at a page border, so a lost page or a wrong offset shows."""
    from inferloop_b200.csrc import ops
    g = torch.Generator().manual_seed(d + dv)
    nq, nkv, page, T = 4, 2, 8, 300
    q = torch.randn(T, nq, d, generator=g, dtype=torch.float64) * 0.5
    k = torch.randn(T, nkv, d, generator=g, dtype=torch.float64) * 0.5
    v = torch.randn(T, nkv, dv, generator=g, dtype=torch.float64)
    far = 2 * page                                    # first slot of the third page
    k[far] = q[T - 1, 0] * 6.0 / q[T - 1, 0].norm()    # the last query of head 0 looks at it almost alone
    scale = 0.7
    n_pages = -(-T // page)
    perm = torch.randperm(n_pages, generator=g)
    kc = torch.zeros(n_pages, nkv, page, d, dtype=torch.float32)
    vc = torch.zeros(n_pages, nkv, page, dv, dtype=torch.float32)
    for t in range(T):
        kc[perm[t // page], :, t % page] = k[t].float()
        vc[perm[t // page], :, t % page] = v[t].float()
    out = torch.empty(T, nq * dv, dtype=torch.float32, device=DEV)
    ops.paged_attention_simple(q.float().view(T, nq * d).to(DEV), out, kc.to(DEV), vc.to(DEV), torch.arange(T, dtype=torch.int32, device=DEV),
                               torch.zeros(T, dtype=torch.int32, device=DEV), perm.to(torch.int32).view(1, -1).to(DEV), 0, scale, nq, nkv, d, dv)
    ref = plain.causal_attention(q.float().double(), k.float().double(), v.float().double(), scale)
    assert_close(out.view(T, nq, dv), ref, "float32", "attention")
    w_far = torch.softmax((k[:, 0].float().double() @ q[T - 1, 0].float().double()) * scale, 0)[far]
    assert w_far > 0.5, "the far key does not stand out; the test would not see its loss"


@pytest.mark.parametrize("experts,top,softmax,renorm", [(5, 2, False, False), (8, 1, False, False), (4, 4, False, True),
                                                      (37, 3, True, True), (160, 6, True, False), (3, 1, False, True)])
def test_routing_scores_choices_and_weights(experts, top, softmax, renorm):
    from inferloop_b200.csrc import ops
    g = torch.Generator().manual_seed(experts * 10 + top)
    T = 50
    z = torch.randn(T, experts + 1, generator=g) * 2          # one more column, as when a gate's logit rides along
    z[3, :experts] = 0.25                                     # all equal: the lower indices win
    z[4, 1] = z[4, 0]
    choice = torch.empty(T * top, dtype=torch.int32, device=DEV)
    weight = torch.empty(T * top, dtype=torch.float32, device=DEV)
    ops.moe_route(z.to(DEV), experts, top, softmax, renorm, choice, weight)
    zz = z[:, :experts].double()
    s = torch.softmax(zz, -1) if softmax else 1 / (1 + torch.exp(-zz))
    s32 = s.float()           # decisions are taken on 32-bit scores
    for t in range(T):
        ranked = sorted(range(experts), key=lambda e: (-float(s32[t, e]), e))[:top]
        got = choice.view(T, top)[t].tolist()
        if len({float(s32[t, e]) for e in range(experts)}) == experts or t in (3, 4):
            assert got == ranked, f"token {t}"
        w = s[t, got]
        if renorm:
            w = w / w.sum()
        assert_close(weight.view(T, top)[t], w, "float32", f"weights of token {t}")
    assert choice.view(T, top)[3].tolist() == list(range(top))
    if not softmax and not renorm:                         # the plain model's own routing function
        idx, w, margin = plain.route(zz, top)
        for t in range(T):
            if top == experts or margin[t] > 1e-4:
                assert choice.view(T, top)[t].tolist() == idx[t].tolist()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,rows,width", [(1, 3, 64), (9, 17, 2048), (130, 161, 96), (5, 8, 100), (33, 6, 4104)])
def test_router_logits_are_32_bit_sums(dtype, T, rows, width):
    from inferloop_b200.csrc import ops
    g = torch.Generator().manual_seed(T + rows)
    x = torch.randn(T, width, generator=g).to(dtype)
    w = torch.randn(rows, width, generator=g).to(dtype)
    out = torch.empty(T, rows, dtype=torch.float32, device=DEV)
    ops.moe_logits(x.to(DEV), w.to(DEV), out)
    assert_close(out, x.double() @ w.double().T, "float32", "router logits")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("block,tile_n", [(16, 0), (128, 128), (128, 256), (128, 257), (256, 256)])     # 257: persistent CTAs, 128 x 256 tiles
@pytest.mark.parametrize("T,experts,top,H,I", [(1, 4, 2, 64, 64), (9, 5, 2, 96, 128), (300, 8, 1, 256, 64), (77, 3, 3, 128, 192),
                                               (700, 2, 2, 320, 384)])
def test_sorted_rows_grouped_products_and_the_sum(dtype, block, tile_n, T, experts, top, H, I):
    """plan -> gather -> grouped product (exact in blocks of 16; on tensor cores in blocks of 128 and 256,
    with and without the SwiGLU epilogue) -> combine, with weights on the input and on the output,
    against per-token products."""
    from inferloop_b200.csrc import ops
    if block >= 128 and dtype != torch.bfloat16:
        pytest.skip("the tensor-core product is bfloat16")
    g = torch.Generator().manual_seed(T + experts)
    x = torch.randn(T, H, generator=g).to(dtype)
    choice = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    if T > 20:
        choice[:, 0] = torch.where(torch.arange(T) % 3 == 0, choice[:, 0], choice[0, 0])   # unequal loads, maybe an idle expert
    weight = torch.rand(T * top, generator=g) + 0.25
    w1 = (torch.randn(experts, I, H, generator=g) * 0.1).to(dtype)
    rows = ops.moe_plan_rows(T * top, experts, block)
    pos = torch.empty(T * top, dtype=torch.int32, device=DEV)
    block_expert = torch.empty(rows // block, dtype=torch.int32, device=DEV)
    ops.moe_plan(choice.view(-1).to(DEV), experts, block, pos, block_expert)
    p, be = pos.cpu(), block_expert.cpu()
    assert len(set(p.tolist())) == T * top and int(p.min()) >= 0 and int(p.max()) < rows
    for i in range(T * top):
        assert int(be[int(p[i]) // block]) == int(choice.view(-1)[i])
    for weighted_input in (True, False):
        a = torch.full((rows, H), float("nan"), dtype=dtype, device=DEV)           # rows without a pair stay as they are
        ops.moe_gather(x.to(DEV), weight.to(DEV) if weighted_input else None, pos, top, a)
        out = torch.empty(rows, I, dtype=torch.float32, device=DEV)
        if block == 16:
            ops.gemm_simt_grouped(a, w1.to(DEV), out, block_expert)
        else:
            ops.moe_gemm_tc(a, w1.to(DEV), out, block_expert, block_rows=block, tile_n=tile_n)
        y = torch.zeros(T, I, dtype=torch.float32, device=DEV)
        shared = torch.randn(T, I, generator=g)
        gate = torch.randn(T, 3, generator=g)
        ops.moe_combine(out, pos, None if weighted_input else weight.to(DEV), top, shared.to(DEV), gate.to(DEV)[:, 2], y)
        ref = torch.zeros(T, I, dtype=torch.float64)
        for t in range(T):
            for j in range(top):
                wt = float(weight[t * top + j])
                e = int(choice[t, j])
                xin = (wt * x[t].float()).to(dtype).double() if weighted_input else x[t].double()
                ref[t] += (xin @ w1[e].double().T) * (1.0 if weighted_input else wt)
            ref[t] += shared[t].double() / (1 + math.exp(-float(gate[t, 2])))
        assert_close(y, ref, "float32" if dtype == torch.float32 else "bfloat16", f"weighted_input={weighted_input}", bf16_rel_of_max=2e-3)
    if block >= 128 and I % 64 == 0:        # the SwiGLU epilogue: gate and up rows interleaved in blocks of 64
        wg, wu = (torch.randn(experts, I, H, generator=g) * 0.2).to(dtype), (torch.randn(experts, I, H, generator=g) * 0.2).to(dtype)
        inter = torch.stack([wg.view(experts, I // 64, 64, H), wu.view(experts, I // 64, 64, H)], dim=2).reshape(experts, 2 * I, H).contiguous()
        act = torch.empty(rows, I, dtype=torch.bfloat16, device=DEV)
        ops.moe_gemm_tc(a, inter.to(DEV), act, block_expert, swiglu=True, block_rows=block, tile_n=tile_n)
        for t in range(0, T, max(1, T // 7)):
            e = int(choice[t, 0])
            xin = x[t].double()
            want = plain.silu(xin @ wg[e].double().T) * (xin @ wu[e].double().T)
            got = act[int(p[t * top])].double().cpu()
            assert (got - want).abs().max() <= 2.0 ** -7 * max(1.0, float(want.abs().max())), f"SwiGLU epilogue, token {t}"
    ops.check_device_errors()
