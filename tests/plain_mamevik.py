"""Plain statement of the Mamevik decoder: 64-bit, whole sequences, one function per mechanism.

Written from the design's equations and sharing no code with the engine.  `w` maps tensor names
to 64-bit tensors, `cfg` is the parsed config.json.  Notation: T tokens, width W; a layer is
x <- x + mixer(n1(x)); x <- x + ff(n2(x)) with n(x) = x / sqrt(mean(x^2) + eps) * (1 + g).

  embedding     e_t = E[tok_t] + Bg[r_t],  r_0 = buckets,  r_t = (tok_{t-1} a + tok_t b) mod buckets;
                x0 = n(e)
  loop          layers start..stop-1 run `times` times; before pass p: x <- L [x; x0] + s_p
  state space   [z | u | B | C | d] = P h;  (u, B, C) <- silu(causal conv);  d <- softplus(d + d0);
                S_t = exp(-exp(a) d_t) S_{t-1} + d_t B_t u_t^T;  y_t = S_t^T C_t + D u_t;
                out = O (groupnorm(y * silu(z)) * g)
  latent attn   q = Q h;  c = rms(K h) * g;  k = Uk c;  v = Uv c;  s_ij = scale q_i.k_j for 0 <= i-j < win;
                p_ij = exp(s_ij) / (exp(sink) + sum_j exp(s_ij));  out = O (p v)
  experts       z = R h + b;  the `top` largest;  softmax over those;  expert(h) = Dn (a(min(Gt h, L)) (clamp(Up h, -L, L) + 1)),
                a(g) = g sigmoid(1.702 g)
  output        cap * tanh(scale * (E n(x)) / cap)
"""
from __future__ import annotations

import math

import torch


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_offset(x, g, eps):
    return rms(x, eps) * (1.0 + g)


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.where(x > 30.0, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def bigram_rows(tokens, big):
    rows = [int(big["buckets"])]
    for prev, cur in zip(tokens[:-1], tokens[1:]):
        rows.append((int(prev) * int(big["mul_prev"]) + int(cur) * int(big["mul_cur"])) % int(big["buckets"]))
    return rows


def embedding(w, cfg, tokens):
    x = w["embed"][torch.tensor(tokens)]
    big = (cfg.get("embedding") or {}).get("bigram")
    if big is not None:
        x = x + w["bigram"][torch.tensor(bigram_rows(tokens, big))]
    return norm_offset(x, w["embed.norm"], cfg["norm"]["eps"])


def causal_conv(x, kernel, bias):
    """x [T, C], kernel [C, taps] (last column multiplies the current token), zeros before the start."""
    T, taps = x.shape[0], kernel.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, x.shape[1], dtype=x.dtype), x])
    out = bias.expand(T, -1).clone()
    for k in range(taps):
        out = out + padded[k:k + T] * kernel[:, k]
    return out


def recurrence(u, B, C, d, a_log, D, heads, groups):
    """u [T, heads, P], B and C [T, groups, N], d [T, heads] -> y [T, heads, P], token by token."""
    T, _, P = u.shape
    per = heads // groups
    S = torch.zeros(heads, B.shape[2], P, dtype=u.dtype)
    y = torch.zeros_like(u)
    decay = torch.exp(-torch.exp(a_log)[None, :] * d)                      # [T, heads]
    Bh, Ch = B.repeat_interleave(per, dim=1), C.repeat_interleave(per, dim=1)      # [T, heads, N]: head h reads group h // per
    for t in range(T):
        S = decay[t, :, None, None] * S + d[t, :, None, None] * Bh[t, :, :, None] * u[t, :, None, :]
        y[t] = (S * Ch[t, :, :, None]).sum(1) + D[:, None] * u[t]
    return y


def group_rms(y, parts, eps):
    T, width = y.shape
    return rms(y.view(T, parts, width // parts), eps).reshape(T, width)


def state_space(h, w, p, m, eps):
    heads, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner, T = heads * P, h.shape[0]
    proj = h @ w[p + "in"].T
    z, ubc, d = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    ubc = silu(causal_conv(ubc, w[p + "conv"], w[p + "conv.b"]))
    u = ubc[:, :inner].reshape(T, heads, P)
    B = ubc[:, inner:inner + G * N].reshape(T, G, N)
    C = ubc[:, inner + G * N:].reshape(T, G, N)
    d = softplus(d + w[p + "dt_bias"])
    y = recurrence(u, B, C, d, w[p + "A_log"], w[p + "D"], heads, G).reshape(T, inner)
    y = group_rms(y * silu(z), m["norm_groups"], eps) * w[p + "norm"]
    return y @ w[p + "o"].T


def windowed_sink_attention(q, k, v, scale, window, sink):
    """q, k [T, H, d], v [T, H, dv], sink [H]; position i reads j with 0 <= i - j < window (None: all j <= i)."""
    T = q.shape[0]
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = (j <= i) if window is None else ((j <= i) & (i - j < window))
    s = s.masked_fill(~seen, -math.inf)
    top = torch.maximum(s.max(-1).values, sink[:, None])
    e = torch.exp(s - top[..., None])
    den = e.sum(-1) + torch.exp(sink[:, None] - top)
    return torch.einsum("hij,jhv->ihv", e / den[..., None], v)


def latent_attention(h, w, p, m, eps):
    T, H, d, dv = h.shape[0], m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, d)
    c = rms(h @ w[p + "dkv"].T, eps) * w[p + "dkv.norm"]
    k = (c @ w[p + "uk"].T).view(T, H, d)
    v = (c @ w[p + "uv"].T).view(T, H, dv)
    window = (m.get("mask") or {}).get("size")
    o = windowed_sink_attention(q, k, v, m["scale"], window, w[p + "sink"])
    return o.reshape(T, H * dv) @ w[p + "o"].T


def expert(h, w, p, limit):
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def router_logits(h, w, p):
    return h @ w[p + "router"].T + w[p + "router.b"]


MARGINS = None      # a list: every call of `experts` appends, per token, how far the last chosen logit lies above the first
                    # one left out, as a share of the largest logit's size (tests choose prompts whose routing is decided)


def experts(h, w, p, f):
    top, limit = f["router"]["top"], f["expert"]["limit"]
    z = router_logits(h, w, p)
    best = torch.topk(z, top, dim=-1)
    if MARGINS is not None and top < z.shape[-1]:
        ranked = torch.sort(z, dim=-1, descending=True).values
        MARGINS.append((ranked[:, top - 1] - ranked[:, top]) / ranked.abs().max(-1).values.clamp_min(1e-30))
    share = torch.softmax(best.values, dim=-1)
    out = torch.zeros_like(h)
    for e in range(z.shape[-1]):
        rows, col = torch.nonzero(best.indices == e, as_tuple=True)
        if rows.numel():
            out[rows] = out[rows] + share[rows, col][:, None] * expert(h[rows], w, f"{p}e{e}.", limit)
    return out


def layer(x, w, cfg, i):
    spec, eps, p = cfg["layers"][i], cfg["norm"]["eps"], f"l{i}."
    h = norm_offset(x, w[p + "norm1"], eps)
    mix = state_space if spec["type"] == "mamba2" else latent_attention
    x = x + mix(h, w, p + "mix.", spec["mixer"], eps)
    if spec.get("mlp") is not None:
        x = x + experts(norm_offset(x, w[p + "norm2"], eps), w, p + "mlp.", spec["mlp"])
    return x


def run_order(cfg):
    """[(layer, pass or None)] in the order the layers run."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if loop is None:
        return [(i, None) for i in range(n)]
    out = [(i, None) for i in range(loop["start"])]
    for p in range(loop["times"]):
        out += [(i, p) for i in range(loop["start"], loop["stop"])]
    return out + [(i, None) for i in range(loop["stop"], n)]


def forward(w, cfg, tokens, trace=None):
    """Logits [T, vocab]; `trace`, a list, receives the residual stream after every layer run."""
    x0 = embedding(w, cfg, tokens)
    x = x0
    loop = cfg.get("loop")
    for i, p in run_order(cfg):
        if p is not None and i == loop["start"]:
            x = torch.cat([x, x0], dim=-1) @ w["loop.in"].T + w["loop.step"][p]
        x = layer(x, w, cfg, i)
        if trace is not None:
            trace.append(x.clone())
    x = norm_offset(x, w["final.norm"], cfg["norm"]["eps"])
    z = (x @ w["embed"].T) * cfg.get("logit_scale", 1.0)
    cap = cfg.get("logit_softcap")
    return z if not cap else cap * torch.tanh(z / cap)
