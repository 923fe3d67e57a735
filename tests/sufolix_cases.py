"""Small Sufolix configurations for the tests, their model folders and plain logits."""
from __future__ import annotations

import json
import math
import os
import random
from typing import Dict, List

import torch

import plain_sufolix as plain


def attention(heads, kv_heads, dim, vdim, scale, rot=None, v_mix=False):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "v_mix": v_mix}
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    return m


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None):
    m = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


def layer(mixer, mlp):
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def model(vocab, width, eps, scale, streams, layers):
    c = {"architecture": "Sufolix", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale},
         "layers": layers}
    if streams is not None:
        c["streams"] = streams
    return c


# P: odd sizes everywhere: three streams, values wider than keys, rotation over part of the head,
# groups of two, a layer without rotation, one without feed-forward, one that does not mix values,
# experts with top 2 and a shared expert, experts with top 3 of 4 and none shared.  Exact kernels only.
_A = dict(heads=6, kv_heads=3, dim=16, vdim=24, scale=0.31)
CONFIG_P = model(331, 96, 2e-5, 3.0, 3, [
    layer(attention(rot=(5000.0, 8), v_mix=True, **_A), dense(80)),
    layer(attention(rot=None, v_mix=False, **_A), moe(5, 2, 24, shared=40)),
    layer(attention(rot=(5000.0, 16), v_mix=True, **_A), None),
    layer(attention(rot=(300.0, 12), v_mix=True, **_A), moe(4, 3, 40)),
])
# Q: the serving kernels' geometry: heads of 128 for keys and values (tcgen05 prefill attention,
# TMA decode attention), widths in multiples of 64 (tensor-core products, SwiGLU epilogues, the
# grouped tensor-core product of the experts), one stream with its own coefficients, top 2 of 6.
_B = dict(heads=4, kv_heads=2, dim=128, vdim=128, scale=0.09)
CONFIG_Q = model(1000, 256, 1e-6, 0.5, 1, [
    layer(attention(rot=(100000.0, 128), v_mix=True, **_B), moe(6, 2, 64, shared=128)),
    layer(attention(rot=(100000.0, 64), v_mix=True, **_B), dense(384)),
    layer(attention(rot=(100000.0, 128), v_mix=True, **_B), moe(3, 1, 128)),
])
# R: no streams at all (the plain residual), one kv head per query head, heads of 64, four streams
# are covered by S below.
_C = dict(heads=2, kv_heads=2, dim=64, vdim=64, scale=0.125)
CONFIG_R = model(257, 128, 1e-5, 1.0, None, [
    layer(attention(rot=(10000.0, 64), v_mix=False, **_C), dense(192)),
    layer(attention(rot=(10000.0, 32), v_mix=True, **_C), moe(9, 4, 64, shared=64)),
    layer(attention(rot=(10000.0, 64), v_mix=True, **_C), None),
])
# S: four streams, values narrower than keys, a single kv head.
_D = dict(heads=4, kv_heads=1, dim=32, vdim=16, scale=0.2)
CONFIG_S = model(190, 64, 1e-5, 8.0, 4, [
    layer(attention(rot=(777.0, 32), v_mix=True, **_D), moe(3, 2, 16, shared=16)),
    layer(attention(rot=(777.0, 2), v_mix=True, **_D), dense(48)),
])
CASES = {"P": (CONFIG_P, 11, 8), "Q": (CONFIG_Q, 12, 16), "R": (CONFIG_R, 13, 16), "S": (CONFIG_S, 14, 4)}   # config, seed, page size

_FOLDERS: Dict[tuple, str] = {}
_PLAIN: Dict[tuple, plain.Plain] = {}


def folder(tmp_root: str, name: str, dtype: torch.dtype) -> str:
    """The model folder of a case (weights stored in `dtype`), written once per test session.
    Router rows are scaled up so that routing decisions are rarely close."""
    from inferloop_b200.weights import write_safetensors
    from inferloop_b200.weights.safetensors_io import SafetensorsFile
    from inferloop_b200.weights import write_random_model
    key = (name, dtype)
    if key not in _FOLDERS:
        config, seed, _ = CASES[name]
        path = os.path.join(tmp_root, f"sufolix-{name}-{str(dtype).split('.')[-1]}")
        write_random_model(path, config, seed, dtype, prefix="")
        f = SafetensorsFile(os.path.join(path, "model.safetensors"))
        tensors = [(n, f.tensor(n).clone()) for n in f.names()]
        f.close()
        tensors = [(n, (t.float() * 8.0).to(t.dtype) if n.endswith(".router") else t) for n, t in tensors]
        write_safetensors(os.path.join(path, "model.safetensors"), tensors, metadata={"format": "pt"})
        _FOLDERS[key] = path
    return _FOLDERS[key]


def plain_model(tmp_root: str, name: str, dtype: torch.dtype) -> plain.Plain:
    from inferloop_b200.weights.safetensors_io import SafetensorsFile
    key = (name, dtype)
    if key not in _PLAIN:
        path = folder(tmp_root, name, dtype)
        f = SafetensorsFile(os.path.join(path, "model.safetensors"))
        weights = {n: f.tensor(n).clone() for n in f.names()}
        f.close()
        _PLAIN[key] = plain.Plain(CASES[name][0], weights)
    return _PLAIN[key]


def decided_tokens(model: plain.Plain, n: int, vocab: int, seed: int, margin: float, chunk: int = 12) -> List[int]:
    """`n` random tokens whose routing decisions, in the plain model, all have at least this
    margin, so that no comparison rests on a close call.  The sequence grows by chunks; what a
    position decides depends on the tokens up to it alone, so a chunk whose positions are not
    all decided is drawn again and the ones before it stay."""
    rng = random.Random(seed)
    tokens: List[int] = []
    failed = 0                                   # draws refused at this length: the chunk shrinks with them
    while len(tokens) < n:
        size = max(1, chunk >> (failed // 3))
        more = [rng.randrange(vocab) for _ in range(min(size, n - len(tokens)))]
        model.forward(tokens + more)
        if model.least_margin(len(tokens)) >= margin:
            tokens += more
            failed = 0
        else:
            failed += 1
            if failed > 200:
                raise AssertionError("no token sequence with decided routing found")
    return tokens
