"""Mamevik decoder: from its typed config to a :class:`ModelSpec`.

The embedding is the token's row plus a row of a hashed table of (previous token, token) pairs,
normed.  A layer is a pre-norm block whose norm weights are stored around zero; its mixer is a
state-space recurrence with a short convolution in front (kind `ssd_recurrence`) or attention
over a cached low-rank latent, without positions, in a sliding window, with a learned sink in
the softmax (kind `latent_attention`); its feed-forward routes every token to the `top` experts
with the largest biased router logits, weighted by the softmax over those, each expert a gated
unit with clamped inputs.  A span of layers may run several times with the same weights and a
cache of its own per run; before each run the stream is mapped, together with the embedding's
output, through a matrix and shifted by the run's vector (block kind `loop_input`).  The output
matrix is the token table; logits are scaled and soft-capped.

Tensor names: `embed`, `bigram`, `embed.norm`, `loop.in`, `loop.step`, `final.norm`, and under
`l<i>.`: `norm1`, `norm2`, `mix.{in,conv,conv.b,dt_bias,A_log,D,norm,o}` or
`mix.{q,dkv,dkv.norm,uk,uv,sink,o}`, `mlp.router`, `mlp.router.b`, `mlp.e<j>.{gate,up,down}`.
"""
from __future__ import annotations

from ..config.mamevik import MamevikConfig
from ..config.registry import Architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunEntry

# The design fixes these: the gate's activation a(g) = g * sigmoid(1.702 g), and the one added
# to the clamped linear half.
GATE_SHARPNESS = 1.702
UP_OFFSET = 1.0
# Norm weights are stored as their distance from one.
NORM_OFFSET = 1.0


def build_spec(cfg: MamevikConfig) -> ModelSpec:
    norm = PartSpec.make("rms", eps=cfg.eps, weight_suffix="", offset=NORM_OFFSET)
    layers = []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if layer.type == "mamba2":
            mixer = PartSpec.make(
                "ssd_recurrence", hidden_size=cfg.width, heads=m.heads, head_dim=m.vdim, state=m.state, groups=m.groups,
                taps=m.conv, norm_groups=m.norm_groups, eps=cfg.eps)
        else:
            mixer = PartSpec.make(
                "latent_attention", hidden_size=cfg.width, heads=m.heads, head_dim=m.dim, v_head_dim=m.vdim,
                latent=m.kv_rank, scale=m.scale, window=m.window, sink=True, eps=cfg.eps, max_positions=cfg.max_positions)
        f = layer.mlp
        if f is None:
            ffn = PartSpec.make("none")
        else:
            ffn = PartSpec.make(
                "routed_experts", hidden_size=cfg.width, experts=f.experts, top_k=f.top, expert_inter=f.ff, score="softmax",
                renormalize=True, weight_on="output", router_bias=True,
                activation=PartSpec.make("clamped_glu", limit=f.limit, sharpness=GATE_SHARPNESS, up_offset=UP_OFFSET),
                names=(("router", "router"), ("router_bias", "router.b"), ("gate", "e{e}.gate"), ("up", "e{e}.up"),
                       ("down", "e{e}.down")))
        block = PartSpec.make("pre_norm", hidden_size=cfg.width, mixer_prefix="mix.", ffn_prefix="mlp.",
                              mixer_norm="norm1", ffn_norm="norm2")
        layers.append(LayerSpec(prefix=f"l{i}.", block=block, mixer=mixer, feed_forward=ffn, norm=norm))
    n = len(cfg.layers)
    if cfg.loop is None:
        order = tuple(RunEntry(i, i) for i in range(n))
    else:
        lp = cfg.loop
        layers.append(LayerSpec(prefix="loop.", block=PartSpec.make(
            "loop_input", hidden_size=cfg.width, times=lp.times, matrix="in", shift="step", source="embedding.output")))
        order = [RunEntry(i, i) for i in range(lp.start)]
        for p in range(lp.times):
            order.append(RunEntry(n, n, instance=p))
            order += [RunEntry(i, i, instance=p) for i in range(lp.start, lp.stop)]
        order = tuple(order + [RunEntry(i, i) for i in range(lp.stop, n)])
    b = cfg.bigram
    embedding = PartSpec.make(
        "hashed_pairs", hidden_size=cfg.width, vocab_size=cfg.vocab,
        buckets=0 if b is None else b.buckets, mul_prev=0 if b is None else b.mul_prev, mul_cur=0 if b is None else b.mul_cur,
        table="bigram", norm=PartSpec.make("rms", eps=cfg.eps, weight_suffix="", offset=NORM_OFFSET), norm_name="embed.norm",
        keep="embedding.output" if cfg.loop is not None else None)
    post = None
    if cfg.logit_softcap > 0 or cfg.logit_scale != 1.0:
        post = PartSpec.make("soft_cap", cap=cfg.logit_softcap, scale=cfg.logit_scale)
    return ModelSpec(
        architecture="Mamevik",
        vocab_size=cfg.vocab,
        hidden_size=cfg.width,
        max_positions=cfg.max_positions,
        embedding_name="embed",
        head_name=None,
        final_norm_name="final.norm",
        final_norm=norm,
        layers=tuple(layers),
        run_order=order,
        weight_prefixes=("",),
        logits_post=post,
        embedding=embedding,
    )


ARCHITECTURE = Architecture(
    name="mamevik",
    claims=("Mamevik", "mamevik"),
    read_config=MamevikConfig.from_dict,
    build_spec=build_spec,
)
