"""Attention over a cached low-rank latent, without positions (mixer kind `latent_attention`).

    q = W_q h  [heads, d];   c = rms(W_dkv h) * g  [rank];   k_i = Uk_i c,  v_i = Uv_i c  (head i)
    s_ij = scale * q_i . k_j for the keys j a position reads: all earlier ones and itself, or the
    last `window` of them;  p = softmax over those, with exp(sink_i) joining the denominator when
    the layer has a sink;  out = W_o [p v]

Only c is cached (one "kv head" of `rank` elements per token, no values beside it).  The engine
never forms k and v: with q'_i = Uk_i^T q_i the score is q'_i . c_j, and sum_j p_j v_j =
Uv_i (sum_j p_j c_j), so the attention kernels run over the cached latents as keys and as values
with all heads sharing them, between two small per-head products (csrc/latent.cu; a step of up to 16
tokens writes its latents and maps its queries in one launch).  A step is the
same computation however its tokens were cut: a prompt's portion and a single token take the same
path.  W_q and W_dkv are one product.
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..csrc import ops
from ..weights.decl import WeightDecl
from . import registry
from .base import CacheNeeds, Mixer, PagedKVNeed
from .linear import linear


class LatentAttention(Mixer):
    graph_safe = True

    def __init__(self, spec, ctx, prefix: str = "") -> None:
        super().__init__(spec, ctx, prefix)
        self.hidden = int(spec["hidden_size"])
        self.heads = int(spec["heads"])
        self.d = int(spec["head_dim"])
        self.dv = int(spec.get("v_head_dim") or self.d)
        self.rank = int(spec["latent"])
        self.scale = float(spec["scale"])
        self.window = spec.get("window")
        self.has_sink = bool(spec.get("sink", False))
        self.eps = float(spec["eps"])
        # split-KV decode cuts the keys at multiples of this, fixed per model; with a window the chunks a token reads
        # are few wherever it stands, so they can be short
        self.decode_chunk = ops.DECODE_CHUNK_MIN if self.window else ops.decode_chunk_for(int(spec.get("max_positions", 4096)))
        names = {"q": "q", "down": "dkv", "down_norm": "dkv.norm", "up_k": "uk", "up_v": "uv", "sink": "sink", "o": "o"}
        for role, name in spec.get("names", ()):
            if role not in names:
                raise ValueError(f"latent attention has no tensor role {role!r}")
            names[role] = name
        self.names = {k: prefix + v for k, v in names.items()}
        self.w_in = self.w_o = self.latent_norm = self.up_k = self.up_v = self.sink = None

    def declare_weights(self) -> List[WeightDecl]:
        n, H = self.names, self.hidden
        out = [WeightDecl(n["q"], (self.heads * self.d, H)), WeightDecl(n["down"], (self.rank, H)),
               WeightDecl(n["down_norm"], (self.rank,), "vector", "norm"),
               WeightDecl(n["up_k"], (self.heads * self.d, self.rank)), WeightDecl(n["up_v"], (self.heads * self.dv, self.rank)),
               WeightDecl(n["o"], (H, self.heads * self.dv))]
        if self.has_sink:
            out.append(WeightDecl(n["sink"], (self.heads,), "vector", "around_zero"))
        return out

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        self.w_in = torch.cat([tensors[n["q"]], tensors[n["down"]]], dim=0).contiguous()
        self.latent_norm = tensors[n["down_norm"]].contiguous()
        # [heads, K, N] for out = x W: queries to the latent space (K = d, N = rank), latent sums to values (K = rank, N = dv)
        self.up_k = tensors[n["up_k"]].view(self.heads, self.d, self.rank).contiguous()
        self.up_v = tensors[n["up_v"]].view(self.heads, self.dv, self.rank).transpose(1, 2).contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        if self.has_sink:
            self.sink = tensors[n["sink"]].contiguous()

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(paged=PagedKVNeed(1, self.rank, self.window, 0))

    def scratch_bytes(self, tokens: int) -> int:
        size = torch.empty((), dtype=self.ctx.dtype).element_size()
        return tokens * size * (self.heads * (self.d + 2 * self.rank + self.dv) + self.rank)

    def forward(self, x: torch.Tensor, residual: torch.Tensor, step, cache) -> None:
        T, ws, dt = x.shape[0], self.ctx.workspace, self.ctx.dtype
        H, d, dv, r = self.heads, self.d, self.dv, self.rank
        proj = ws.buffer("latent.proj", (T, H * d + r), dt)
        ops.scope("attention.qkv_projection")
        linear(x, self.w_in, proj)
        table = step.block_tables[cache.group]
        q = ws.buffer("latent.q", (T, H * r), dt)
        if T <= ops.LATENT_INPUT_TOKENS and cache.writable and cache.k.dtype == dt:
            ops.scope("attention.input_stage (latent norm, cache write, queries to latent)")
            ops.latent_input(proj, self.up_k, q, H * d, r, self.latent_norm, self.eps, step, table, cache.k)
        else:
            ops.scope("attention.latent_norm_cache_write")
            if cache.writable:
                ops.latent_write(proj, H * d, r, self.latent_norm, self.eps, step, table, cache.k)
            ops.scope("attention.queries_to_latent")
            ops.head_matmul(proj, self.up_k, q)
        ops.scope("attention.attention")
        o = ws.buffer("latent.o", (T, H * r), dt)
        ops.attention(q, o, cache.k, cache.k, step, table, self.window or 0, self.scale, H, 1, r, workspace=ws,
                      decode_chunk=self.decode_chunk, sink=self.sink)
        ops.scope("attention.latent_to_values")
        v = ws.buffer("latent.v", (T, H * dv), dt)
        ops.head_matmul(o, self.up_v, v)
        ops.scope("attention.o_projection")
        linear(v, self.w_o, residual, accumulate=True)


registry.register("mixer", "latent_attention", LatentAttention)
