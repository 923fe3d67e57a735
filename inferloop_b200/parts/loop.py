"""What stands before every run of a span of layers that runs several times (block kind
`loop_input`): the residual stream is mapped together with an earlier stream, and shifted by a
vector of the run:

    x <- M [x; x0] + s[r]        M [hidden, 2 hidden] (x's half first),  s [times, hidden],  r = the run's number

x0 is the workspace buffer that the spec names under `source` ([tokens, hidden] 32-bit, left
there by the part that made it; the embedding's output, say).  The run's number reaches the
block as `cache.instance`, which the run order sets.  The product takes x and x0 in the compute
dtype and sums in 32-bit; the shift rides on the product as its bias.  The block holds no cache.
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..csrc import ops
from ..weights.decl import WeightDecl
from . import registry
from .base import Block, CacheNeeds
from .linear import linear


class LoopInputBlock(Block):
    graph_safe = True

    def __init__(self, spec, ctx, prefix: str = "", layer=None) -> None:
        super().__init__(spec, ctx, prefix)
        self.hidden = int(spec["hidden_size"])
        self.times = int(spec["times"])
        self.source = str(spec["source"])
        self.matrix_name = prefix + str(spec.get("matrix", "in"))
        self.shift_name = prefix + str(spec.get("shift", "step"))
        self.matrix = self.shift = None

    def declare_weights(self) -> List[WeightDecl]:
        return [WeightDecl(self.matrix_name, (self.hidden, 2 * self.hidden)),
                WeightDecl(self.shift_name, (self.times, self.hidden), "vector", "bias")]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.matrix = tensors[self.matrix_name].contiguous()
        self.shift = tensors[self.shift_name].contiguous()

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds()

    def scratch_bytes(self, tokens: int) -> int:
        return tokens * 2 * self.hidden * torch.empty((), dtype=self.ctx.dtype).element_size()

    def forward(self, hidden: torch.Tensor, step, cache) -> None:
        run = int(cache.instance)
        if not 0 <= run < self.times:
            raise ops.KernelError(f"loop_input: run {run} of {self.times}")
        ws = self.ctx.workspace
        T = hidden.shape[0]
        x0 = ws.buffer(self.source, (T, self.hidden), torch.float32)
        both = ws.buffer("loop.both", (T, 2 * self.hidden), self.ctx.dtype)
        ops.scope("loop_input")
        ops.concat_cast(hidden, x0, both)
        linear(both, self.matrix, hidden, self.shift[run])


registry.register("block", "loop_input", LoopInputBlock)
