"""Pre-norm block over several copies of the residual stream ("hyper-connections").

The model keeps `streams` copies x_1 .. x_S of every token's residual stream, all equal to the
embedding at the start; their sum is what the final norm reads.  Sublayer q (the mixer, then
the feed-forward) has three learned tensors a_q [S], b_q [S] and M_q [S, S] and does

    u = sum_s a_q[s] x_s;   y = sublayer(norm_q(u));   x_t <- sum_s M_q[s, t] x_s + b_q[t] y

for all t at once from the old streams.  With S = 1, a = b = M = 1 this is the plain pre-norm
residual block.  The block sees the streams as one 32-bit row [S * hidden] per token; the read
(with the RMS norm fused in when the norm is of that kind) and the write are one kernel each
(csrc/hyper.cu), and the sublayer adds its output into a zeroed 32-bit buffer between them.
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..csrc import ops
from ..weights.decl import WeightDecl
from . import registry
from .base import Block, CacheNeeds
from .norm import RMSNorm


class HyperConnectionBlock(Block):
    """spec: hidden_size, streams, and the tensor-name pieces: mixer_prefix, ffn_prefix,
    mixer_norm, ffn_norm, mixer_streams, ffn_streams (prefixes of `in`, `out`, `mix`)."""

    def __init__(self, spec, ctx, prefix: str = "", layer=None) -> None:
        super().__init__(spec, ctx, prefix)
        self.hidden = int(spec["hidden_size"])
        self.streams = int(spec["streams"])
        if self.streams < 1:
            raise ValueError("a block needs at least one residual stream")
        self.norm1 = registry.build_norm(layer.norm, ctx, prefix + spec.get("mixer_norm", "norm1."), width=self.hidden)
        self.norm2 = registry.build_norm(layer.norm, ctx, prefix + spec.get("ffn_norm", "norm2."), width=self.hidden)
        self.mixer = registry.build("mixer", layer.mixer, ctx, prefix + spec.get("mixer_prefix", "mixer."))
        self.ffn = registry.build("feed_forward", layer.feed_forward, ctx, prefix + spec.get("ffn_prefix", "mlp."))
        self.has_ffn = not getattr(self.ffn, "absent", False)
        self.hc_names = [prefix + spec.get("mixer_streams", "hc1."), prefix + spec.get("ffn_streams", "hc2.")]
        self.hc: List[dict] = [{}, {}]

    @property
    def graph_safe(self) -> bool:
        parts = (self.norm1, self.mixer) + ((self.norm2, self.ffn) if self.has_ffn else ())
        return all(p.graph_safe for p in parts)

    def _stream_decls(self, q: int, optional: bool) -> List[WeightDecl]:
        p, S = self.hc_names[q], self.streams
        return [WeightDecl(p + "in", (S,), "vector", "norm", optional=optional),
                WeightDecl(p + "out", (S,), "vector", "norm", optional=optional),
                WeightDecl(p + "mix", (S, S), "vector", "eye", optional=optional)]

    def declare_weights(self) -> List[WeightDecl]:
        out = self.norm1.declare_weights() + self.mixer.declare_weights() + self._stream_decls(0, False)
        if self.has_ffn:
            out += self.norm2.declare_weights() + self.ffn.declare_weights() + self._stream_decls(1, False)
        else:
            # a file may still hold the absent sublayer's norm and stream tensors: they are not read
            out += [WeightDecl(d.name, d.shape, d.role, d.init, d.root, True) for d in self.norm2.declare_weights()]
            out += self._stream_decls(1, True)
        return out

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.norm1.bind(tensors)
        self.mixer.bind(tensors)
        if self.has_ffn:
            self.norm2.bind(tensors)
            self.ffn.bind(tensors)
        for q in range(2 if self.has_ffn else 1):
            p = self.hc_names[q]
            self.hc[q] = {k: tensors[p + k].contiguous() for k in ("in", "out", "mix")}

    def cache_needs(self) -> CacheNeeds:
        return self.mixer.cache_needs()

    def scratch_bytes(self, tokens: int) -> int:
        size = torch.empty((), dtype=self.ctx.dtype).element_size()
        return (tokens * self.hidden * (size + 8) + self.mixer.scratch_bytes(tokens)
                + (self.ffn.scratch_bytes(tokens) if self.has_ffn else 0))

    def _sublayer(self, q: int, norm, run, hidden: torch.Tensor) -> None:
        ws, S = self.ctx.workspace, self.streams
        T = hidden.shape[0]
        normed = ws.buffer("block.normed", (T, self.hidden), self.ctx.dtype)
        y = ws.buffer("block.sublayer_out", (T, self.hidden), torch.float32)
        hc = self.hc[q]
        ops.scope("norm")
        if isinstance(norm, RMSNorm):
            ops.streams_read(hidden, hc["in"], S, norm.weight, norm.eps, normed=normed, y_zero=y)
        else:
            u = ws.buffer("block.stream_sum", (T, self.hidden), torch.float32)
            ops.streams_read(hidden, hc["in"], S, u_out=u, y_zero=y)
            norm.forward(u, normed)
        run(normed, y)
        ops.scope("residual_streams")
        ops.streams_write(hidden, y, hc["mix"], hc["out"], S)

    def forward(self, hidden: torch.Tensor, step, cache) -> None:
        ops.scope("mixer")
        self._sublayer(0, self.norm1, lambda x, y: self.mixer.forward(x, y, step, cache), hidden)
        if self.has_ffn:
            ops.scope("feed_forward")
            self._sublayer(1, self.norm2, lambda x, y: self.ffn.forward(x, y, step), hidden)


registry.register("block", "hyper_connections", HyperConnectionBlock)
