"""Small Mamevik configurations for the tests, their model folders and plain logits."""
from __future__ import annotations

import json
import os
import random
from typing import Dict, List

import torch

import plain_mamevik as plain


def ssd(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def latent(heads, dim, vdim, kv_rank, scale, window=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    return m


def moe(experts, top, ff, limit):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}


def layer(mixer, mlp):
    return {"type": "mamba2" if "state" in mixer else "latent_attention", "mixer": mixer, "mlp": mlp}


def model(vocab, width, eps, layers, bigram=None, loop=None, logit_scale=None, logit_softcap=None):
    c = {"architecture": "Mamevik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if bigram is not None:
        c["embedding"] = {"bigram": dict(zip(("buckets", "mul_prev", "mul_cur"), bigram))}
    if loop is not None:
        c["loop"] = dict(zip(("start", "stop", "times"), loop))
    if logit_scale is not None:
        c["logit_scale"] = logit_scale
    if logit_softcap is not None:
        c["logit_softcap"] = logit_softcap
    return c


# U: odd sizes, exact kernels only.  A loop from the very first layer; a recurrence with a state of 16 rows
# and one group, another with 40 rows in three groups and two taps; a window of 7, and a layer that reads
# every earlier token; values wider and narrower than keys; a layer without feed-forward; experts of which
# all are chosen.
CONFIG_U = model(211, 72, 3e-5, [
    layer(ssd(4, 12, 16, 1, 4, 1), moe(5, 2, 24, 1.0)),
    layer(latent(3, 8, 20, 24, 0.4, window=7), None),
    layer(latent(2, 16, 8, 40, 0.3), moe(3, 3, 16, 2.5)),
    layer(ssd(6, 8, 40, 3, 2, 3), moe(4, 1, 40, 0.5)),
], bigram=(97, 13, 5), loop=(0, 2, 2), logit_scale=2.0, logit_softcap=10.0)
# V: the sizes the tensor-core kernels take: latents of 64 and 128 elements (the mma.sync attention), experts
# of 64 (the grouped tcgen05 product with the gated unit in its epilogue), a state of 128 rows (two threads a
# column), widths in multiples of 64; a loop over the last two layers that runs three times; no cap on the logits.
CONFIG_V = model(1000, 256, 1e-6, [
    layer(latent(8, 32, 64, 64, 0.17, window=33), moe(6, 2, 64, 7.0)),
    layer(ssd(8, 64, 128, 2, 4, 1), moe(6, 2, 64, 7.0)),
    layer(latent(4, 64, 32, 128, 0.12, window=100), moe(3, 1, 128, 3.0)),
    layer(latent(8, 32, 64, 64, 0.17, window=33), None),
], bigram=(509, 3, 11), loop=(2, 4, 3))
# W: no loop and no table of pairs; a state of 200 rows (four threads a column, the large shared memory), heads of
# 80 (two column tiles), a convolution of one tap and one of five; a latent of 96; a window of one token.
CONFIG_W = model(300, 128, 1e-5, [
    layer(ssd(2, 80, 200, 1, 1, 2), None),
    layer(latent(5, 16, 16, 96, 0.25, window=1), moe(4, 2, 32, 1.75)),
    layer(ssd(4, 16, 24, 2, 5, 4), None),
    layer(latent(2, 48, 24, 96, 0.2, window=19), None),
], logit_scale=0.25, logit_softcap=5.0)
# X: V's sizes with every expert chosen: no routing decision can flip, so bfloat16 runs of any prompt compare closely.
CONFIG_X = model(1000, 256, 1e-6, [
    layer(latent(8, 32, 64, 64, 0.17, window=33), moe(2, 2, 64, 7.0)),
    layer(ssd(8, 64, 128, 2, 4, 1), moe(2, 2, 64, 7.0)),
    layer(latent(4, 64, 32, 128, 0.12, window=100), moe(1, 1, 128, 3.0)),
    layer(latent(8, 32, 64, 64, 0.17), None),
], bigram=(509, 3, 11), loop=(1, 3, 2))
# Y: sizes that are multiples of nothing: width 100, heads of 5 with a state of 7, a latent of 9 with keys of 5 and
# values of 7, experts of 11; the loop covers every layer and runs once.
CONFIG_Y = model(101, 100, 1e-5, [
    layer(ssd(3, 5, 7, 3, 3, 1), moe(3, 2, 11, 1.25)),
    layer(latent(3, 5, 7, 9, 0.45, window=3), None),
    layer(ssd(2, 9, 33, 1, 7, 2), None),
], bigram=(10, 3, 1), loop=(0, 3, 1), logit_scale=3.0)
# Z: recurrences only: the model has no pages at all, only state slots.
CONFIG_Z = model(150, 64, 1e-5, [
    layer(ssd(4, 16, 32, 2, 4, 2), moe(4, 2, 32, 2.0)),
    layer(ssd(2, 32, 64, 1, 2, 1), None),
], bigram=(31, 5, 7))
CASES = {"Y": (CONFIG_Y, 25, 4), "Z": (CONFIG_Z, 26, 16), "U": (CONFIG_U, 21, 4), "V": (CONFIG_V, 22, 16), "W": (CONFIG_W, 23, 8), "X": (CONFIG_X, 24, 16)}     # config, seed, page size

_FOLDERS: Dict[tuple, str] = {}
_PLAIN: Dict[tuple, "Plain"] = {}


def _sharpen(name: str, t: torch.Tensor) -> torch.Tensor:
    """Random weights as the initialisers give them hide some faults: routers that barely prefer an expert, sinks
    and skip weights near nothing, recurrences that forget within a few tokens.  Spread them out."""
    n = t.numel()
    if name.endswith(".router"):
        return t.float() * 8.0
    if name.endswith(".sink"):
        return torch.linspace(-1.0, 2.0, n).view(t.shape)
    if name.endswith(".dt_bias"):                   # step sizes from about 0.01 to 1: heads that keep a token for hundreds of steps
        return torch.linspace(-4.5, 0.5, n).view(t.shape)
    if name.endswith(".A_log"):
        return torch.linspace(-2.0, 0.7, n).view(t.shape)
    if name == "loop.step":
        return t.float() * 10.0
    if name == "embed":                             # logits of the size of the caps
        return t.float() * 10.0
    return t


def folder(tmp_root: str, name: str, dtype: torch.dtype) -> str:
    """The model folder of a case (weights stored in `dtype`), written once per test session."""
    from inferloop_b200.weights import write_random_model, write_safetensors
    from inferloop_b200.weights.safetensors_io import SafetensorsFile
    key = (name, dtype)
    if key not in _FOLDERS:
        config, seed, _ = CASES[name]
        path = os.path.join(tmp_root, f"mamevik-{name}-{str(dtype).split('.')[-1]}")
        write_random_model(path, config, seed, dtype, prefix="")
        f = SafetensorsFile(os.path.join(path, "model.safetensors"))
        tensors = [(n, f.tensor(n).clone()) for n in f.names()]
        f.close()
        tensors = [(n, _sharpen(n, t).to(t.dtype)) for n, t in tensors]
        write_safetensors(os.path.join(path, "model.safetensors"), tensors, metadata={"format": "pt"})
        _FOLDERS[key] = path
    return _FOLDERS[key]


class Plain:
    def __init__(self, config: dict, weights: Dict[str, torch.Tensor]) -> None:
        self.config = config
        self.w = {k: v.double() for k, v in weights.items()}
        self.margins: List[torch.Tensor] = []

    def forward(self, tokens, trace=None) -> torch.Tensor:
        plain.MARGINS = self.margins = []
        try:
            return plain.forward(self.w, self.config, list(tokens), trace)
        finally:
            plain.MARGINS = None

    def least_margin(self, first: int = 0) -> float:
        """The smallest routing margin of the last forward over the positions from `first` on."""
        return min((float(m[first:].min()) for m in self.margins if m[first:].numel()), default=1.0)


def plain_model(tmp_root: str, name: str, dtype: torch.dtype) -> Plain:
    from inferloop_b200.weights.safetensors_io import SafetensorsFile
    key = (name, dtype)
    if key not in _PLAIN:
        path = folder(tmp_root, name, dtype)
        f = SafetensorsFile(os.path.join(path, "model.safetensors"))
        weights = {n: f.tensor(n).clone() for n in f.names()}
        f.close()
        _PLAIN[key] = Plain(CASES[name][0], weights)
    return _PLAIN[key]


def decided_tokens(model: Plain, n: int, vocab: int, seed: int, margin: float, chunk: int = 12) -> List[int]:
    """`n` random tokens whose routing decisions, in the plain model, all have at least this margin, so that no
    comparison rests on a close call.  The sequence grows by chunks; a position's decisions depend on the tokens
    up to it alone, so a chunk whose positions are not all decided is drawn again and the ones before it stay."""
    rng = random.Random(seed)
    tokens: List[int] = []
    failed = 0
    while len(tokens) < n:
        size = max(1, chunk >> (failed // 3))
        more = [rng.randrange(vocab) for _ in range(min(size, n - len(tokens)))]
        model.forward(tokens + more)
        if model.least_margin(len(tokens)) >= margin:
            tokens += more
            failed = 0
        else:
            failed += 1
            if failed > 300:
                raise AssertionError("no token sequence with decided routing found")
    return tokens
