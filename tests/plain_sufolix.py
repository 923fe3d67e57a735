"""Plain 64-bit statement of the Sufolix decoder, whole sequences at a time, one function per
mechanism, written from the design's equations.  It shares no code with the engine: tensors are
looked up by their names in the weight file, the configuration is the nested dictionary of
config.json, and every sum is a torch expression over float64.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

F = torch.float64


def rms(x: torch.Tensor, eps: float, w: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) (* w), over the last dimension."""
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if w is None else y * w


def silu(z: torch.Tensor) -> torch.Tensor:
    return z / (1.0 + torch.exp(-z))


def swiglu(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """x [T, heads, d]: elements (2i, 2i + 1), i < dims / 2, are turned by the angle
    position * base^(-2i / dims); elements from `dims` on pass unchanged."""
    out = x.clone()
    for i in range(dims // 2):
        angle = positions.to(F) * base ** (-2.0 * i / dims)
        c, s = torch.cos(angle)[:, None], torch.sin(angle)[:, None]
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> torch.Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv]; head h reads kv head h // (H / G);
    token i sees tokens j <= i; ordinary softmax."""
    T, H, _ = q.shape
    G = k.shape[1]
    sees = torch.arange(T)[:, None] >= torch.arange(T)[None, :]
    out = torch.zeros(T, H, v.shape[2], dtype=F)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = torch.where(sees, s, torch.full_like(s, -math.inf))
        p = torch.exp(s - s.max(dim=-1, keepdim=True).values)
        out[:, h] = (p / p.sum(dim=-1, keepdim=True)) @ v[:, g]
    return out


def route(z: torch.Tensor, top: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Scores sigmoid(z) [T, E]; the `top` largest per token (lower index first among equals) and
    their scores as weights, not renormalised.  Also how decided each choice was: the gap between
    the last chosen and the first unchosen logit, as a fraction of the token's largest |logit|."""
    s = 1.0 / (1.0 + torch.exp(-z))
    T, E = s.shape
    idx = torch.zeros(T, top, dtype=torch.long)
    w = torch.zeros(T, top, dtype=F)
    margin = torch.full((T,), math.inf, dtype=F)
    for t in range(T):
        ranked = sorted(range(E), key=lambda e: (-float(s[t, e]), e))
        for j in range(top):
            idx[t, j] = ranked[j]
            w[t, j] = s[t, ranked[j]]
        if top < E:
            margin[t] = (z[t, ranked[top - 1]] - z[t, ranked[top]]) / z[t].abs().max()
    return idx, w, margin


class Plain:
    def __init__(self, config: dict, weights: Dict[str, torch.Tensor]) -> None:
        self.c = config
        self.w = {k: v.to(F) for k, v in weights.items()}
        self.eps = float(config["norm"]["eps"])
        self.margins: List[torch.Tensor] = []          # per routed layer of the last forward: [T]

    # ---- the parts of a layer
    def attention(self, li: int, h: torch.Tensor, positions: torch.Tensor, v_first: List[Optional[torch.Tensor]]) -> torch.Tensor:
        m, w, p = self.c["layers"][li]["mixer"], self.w, f"l{li}.mix."
        T = h.shape[0]
        q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, m["heads"], m["dim"])
        k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, m["kv_heads"], m["dim"])
        v = (h @ w[p + "v"].T + w[p + "v.b"]).view(T, m["kv_heads"], m["vdim"])
        if m.get("rot") is not None:
            q = rotate_pairs(q, positions, float(m["rot"]["base"]), int(m["rot"]["dims"]))
            k = rotate_pairs(k, positions, float(m["rot"]["base"]), int(m["rot"]["dims"]))
        q, k = rms(q, self.eps), rms(k, self.eps)
        if m.get("v_mix"):
            if v_first[0] is None:
                v_first[0] = v
            else:
                lam = w[p + "vmix"]
                v = (1.0 - lam) * v + lam * v_first[0]
        o = causal_attention(q, k, v, float(m["scale"]))
        return o.reshape(T, -1) @ w[p + "o"].T

    def feed_forward(self, li: int, h: torch.Tensor) -> torch.Tensor:
        f, w, p = self.c["layers"][li]["mlp"], self.w, f"l{li}.mlp."
        if f["kind"] == "dense":
            return swiglu(h, w[p + "gate"], w[p + "up"], w[p + "down"])
        idx, wt, margin = route(h @ w[p + "router"].T, int(f["router"]["top"]))
        self.margins.append(margin)
        y = torch.zeros_like(h)
        for t in range(h.shape[0]):
            for j in range(idx.shape[1]):
                e = int(idx[t, j])
                y[t] += swiglu(wt[t, j] * h[t], w[f"{p}e{e}.gate"], w[f"{p}e{e}.up"], w[f"{p}e{e}.down"])
        if f.get("shared") is not None:
            gate = 1.0 / (1.0 + torch.exp(-(h @ w[p + "shared.sg"].T)))
            y = y + gate * swiglu(h, w[p + "shared.gate"], w[p + "shared.up"], w[p + "shared.down"])
        return y

    def sublayer(self, li: int, q: int, xs: List[torch.Tensor], fn) -> List[torch.Tensor]:
        """Streams x_1..x_S -> the new streams, through sublayer q (1 mixer, 2 feed-forward)."""
        w, p = self.w, f"l{li}."
        if self.c.get("streams") is None:
            return [xs[0] + fn(rms(xs[0], self.eps, w[f"{p}norm{q}"]))]
        S = len(xs)
        u = sum(w[f"{p}hc{q}.in"][s] * xs[s] for s in range(S))
        y = fn(rms(u, self.eps, w[f"{p}norm{q}"]))
        return [sum(w[f"{p}hc{q}.mix"][s, t] * xs[s] for s in range(S)) + w[f"{p}hc{q}.out"][t] * y for t in range(S)]

    # ---- the model
    def forward(self, tokens: List[int], per_layer: Optional[list] = None) -> torch.Tensor:
        """Logits [T, vocab] of a whole sequence from position 0."""
        c, w = self.c, self.w
        self.margins = []
        positions = torch.arange(len(tokens))
        x0 = w["embed"][torch.tensor(tokens)] * float(c.get("embedding", {}).get("scale", 1.0))
        xs = [x0.clone() for _ in range(c.get("streams") or 1)]
        v_first: List[Optional[torch.Tensor]] = [None]
        for li, layer in enumerate(c["layers"]):
            xs = self.sublayer(li, 1, xs, lambda h: self.attention(li, h, positions, v_first))
            if layer.get("mlp") is not None:
                xs = self.sublayer(li, 2, xs, lambda h: self.feed_forward(li, h))
            if per_layer is not None:
                per_layer.append(sum(xs))
        return rms(sum(xs), self.eps, w["final.norm"]) @ w["head"].T

    def least_margin(self, first: int = 0) -> float:
        """The least decided routing choice of the last forward among positions >= first."""
        return min((float(m[first:].min()) for m in self.margins if m[first:].numel()), default=math.inf)
