"""State-space recurrence with a short convolution in front (mixer kind `ssd_recurrence`; the
"state-space duality" layer of Mamba-2).

    [z | u | B | C | d] = W_in h       z, u: heads * P;  B, C: groups * N;  d: heads
    (u, B, C) <- silu(causal conv over `taps` tokens, per channel, with bias)
    d <- softplus(d + dt_bias);   per head i (group i / (heads / groups)):
    S_t = exp(-exp(A_log_i) d_t) S_{t-1} + d_t B_t u_t^T   (S is N x P),   y_t = S_t^T C_t + D_i u_t
    out = W_o (rms over `norm_groups` equal parts of (y * silu(z)) * g)

A request's state is S [heads, N, P] in 32-bit and the last taps - 1 raw inputs of the
convolution, both in its state slot (zero when the request starts).  Everything between the two
products is 32-bit (csrc/ssm.cu): the convolution, the step sizes and decays, the recurrence, the
gate and the norm; the compute dtype is the type of the two products' inputs and outputs.
A portion of 128 tokens or more runs its recurrence in chunks of 64 side by side (three passes);
shorter ones and single tokens run it in one pass from and to the slot.
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..csrc import ops
from ..weights.decl import WeightDecl
from . import registry
from .base import CacheNeeds, Mixer, SlotStateNeed
from .linear import linear


class SSDRecurrence(Mixer):
    graph_safe = True

    def __init__(self, spec, ctx, prefix: str = "") -> None:
        super().__init__(spec, ctx, prefix)
        self.hidden = int(spec["hidden_size"])
        self.heads = int(spec["heads"])
        self.P = int(spec["head_dim"])
        self.N = int(spec["state"])
        self.groups = int(spec["groups"])
        self.taps = int(spec["taps"])
        self.norm_groups = int(spec.get("norm_groups", 1))
        self.eps = float(spec["eps"])
        if self.heads % self.groups:
            raise ValueError(f"{self.heads} heads are not a multiple of {self.groups} groups")
        self.inner = self.heads * self.P
        if self.inner % self.norm_groups:
            raise ValueError(f"{self.inner} channels are not a multiple of {self.norm_groups} norm groups")
        self.channels = self.inner + 2 * self.groups * self.N           # what the convolution runs over
        self.proj_width = 2 * self.inner + 2 * self.groups * self.N + self.heads
        names = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias", "a_log": "A_log", "skip": "D",
                 "norm": "norm", "o": "o"}
        for role, name in spec.get("names", ()):
            if role not in names:
                raise ValueError(f"the recurrence has no tensor role {role!r}")
            names[role] = name
        self.names = {k: prefix + v for k, v in names.items()}
        self.w_in = self.w_o = self.conv_w = self.conv_b = self.dt_bias = self.a_log = self.skip = self.norm_w = None

    def declare_weights(self) -> List[WeightDecl]:
        n = self.names
        return [WeightDecl(n["in"], (self.proj_width, self.hidden)),
                WeightDecl(n["conv"], (self.channels, self.taps), "vector", "mix"),
                WeightDecl(n["conv_bias"], (self.channels,), "vector", "bias"),
                WeightDecl(n["dt_bias"], (self.heads,), "vector", "around_zero"),
                WeightDecl(n["a_log"], (self.heads,), "vector", "decay"),
                WeightDecl(n["skip"], (self.heads,), "vector", "norm"),
                WeightDecl(n["norm"], (self.inner,), "vector", "norm"),
                WeightDecl(n["o"], (self.hidden, self.inner))]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        self.w_in = tensors[n["in"]].contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        self.conv_w = tensors[n["conv"]].contiguous()
        self.conv_b = tensors[n["conv_bias"]].contiguous()
        self.dt_bias = tensors[n["dt_bias"]].contiguous()
        self.a_log = tensors[n["a_log"]].contiguous()
        self.skip = tensors[n["skip"]].contiguous()
        self.norm_w = tensors[n["norm"]].contiguous()

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(slots=(SlotStateNeed("state", (self.heads, self.N, self.P), torch.float32),
                                 SlotStateNeed("conv", (max(self.taps - 1, 0), self.channels), torch.float32)))

    def scratch_bytes(self, tokens: int) -> int:
        size = torch.empty((), dtype=self.ctx.dtype).element_size()
        chunks = -(-tokens // ops.SSM_CHUNK) + 1
        return (tokens * ((self.proj_width + self.inner) * size + (self.channels + self.inner) * 4)
                + chunks * self.heads * (self.N * self.P + 1) * 4)

    def forward(self, x: torch.Tensor, residual: torch.Tensor, step, cache) -> None:
        T, ws, dt = x.shape[0], self.ctx.workspace, self.ctx.dtype
        proj = ws.buffer("ssm.proj", (T, self.proj_width), dt)
        ops.scope("recurrence.in_projection")
        linear(x, self.w_in, proj)
        ops.scope("recurrence.convolution")
        act = ws.buffer("ssm.act", (T, self.channels), torch.float32)
        ops.ssm_conv(proj, self.inner, self.channels, self.conv_w, self.conv_b, cache.state["conv"], step, act)
        ops.scope("recurrence.scan")
        y = ws.buffer("ssm.y", (T, self.inner), torch.float32)
        ops.ssm_scan(act, proj, self.inner + self.channels, self.dt_bias, self.a_log, self.skip, cache.state["state"], y, step,
                     self.heads, self.P, self.N, self.groups, workspace=ws)
        ops.scope("recurrence.gate_norm")
        gated = ws.buffer("ssm.gated", (T, self.inner), dt)
        ops.gated_group_norm(y, proj, self.norm_w, self.eps, self.norm_groups, gated)
        ops.scope("recurrence.out_projection")
        linear(gated, self.w_o, residual, accumulate=True)


registry.register("mixer", "ssd_recurrence", SSDRecurrence)
