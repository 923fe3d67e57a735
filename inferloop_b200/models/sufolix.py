"""Sufolix decoder: from its typed config to a :class:`ModelSpec`.

A layer is a pre-norm block over `streams` copies of the residual stream (hyper-connections;
a plain pre-norm block when the file names no streams).  Its mixer is causal grouped-query
attention with biases on q, k and v, rotary positions on interleaved pairs over the first
`rot.dims` elements of a head, q and k divided by their root mean square after the rotation,
a score multiplier from the file, values of their own head size, and (where the file says
so) values mixed with those of the first such layer.  Its feed-forward is a SwiGLU, or experts
routed by sigmoid scores whose unnormalised weights multiply the experts' inputs, plus a gated
shared expert; or none.  The embedding is multiplied by a constant; the head is its own matrix.

Tensor names: `embed`, `head`, `final.norm`, and under `l<i>.`: `norm1`, `norm2`, `mix.{q,k,v,o}`
with `.b` for the biases, `mix.vmix`, `mlp.{gate,up,down}`, `mlp.e<j>.{gate,up,down}`,
`mlp.router`, `mlp.shared.{gate,up,down,sg}`, `hc<q>.{in,out,mix}`.
"""
from __future__ import annotations

from ..config.registry import Architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec
from ..config.sufolix import SufolixConfig

_FFN_NAMES = (("gate", "gate"), ("up", "up"), ("down", "down"))


def build_spec(cfg: SufolixConfig) -> ModelSpec:
    norm = PartSpec.make("rms", eps=cfg.eps, weight_suffix="")
    layers = []
    first_mix = True
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        position = (PartSpec.make("none") if m.rot_base is None else
                    PartSpec.make("rope_interleaved", theta=m.rot_base, rotary_dim=m.rot_dims, head_dim=m.dim))
        value_mix = None
        if m.v_mix:
            value_mix, first_mix = ("first" if first_mix else "mixed"), False
        mixer = PartSpec.make(
            "gqa_attention", hidden_size=cfg.width, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim,
            v_head_dim=m.vdim, qk_norm="unweighted", qk_norm_after_rotation=True, qk_norm_eps=cfg.eps, bias="qkv",
            window=None, scale=m.scale, max_positions=cfg.max_positions, position=position, value_mix=value_mix,
            value_mix_tensor_unused=True,
            names=(("q", "q"), ("k", "k"), ("v", "v"), ("o", "o"), ("qb", "q.b"), ("kb", "k.b"), ("vb", "v.b"), ("vmix", "vmix")))
        f = layer.mlp
        if f is None:
            ffn = PartSpec.make("none")
        elif f.kind == "dense":
            ffn = PartSpec.make("swiglu", hidden_size=cfg.width, intermediate_size=f.ff, names=_FFN_NAMES)
        else:
            ffn = PartSpec.make(
                "routed_experts", hidden_size=cfg.width, experts=f.experts, top_k=f.top, expert_inter=f.ff, score="sigmoid",
                renormalize=False, weight_on="input", shared_inter=f.shared_ff, shared_gate=f.shared_ff > 0,
                names=(("router", "router"), ("gate", "e{e}.gate"), ("up", "e{e}.up"), ("down", "e{e}.down"),
                       ("shared_gate", "shared.sg"), ("shared_prefix", "shared.")),
                shared_names=_FFN_NAMES)
        pieces = dict(hidden_size=cfg.width, mixer_prefix="mix.", ffn_prefix="mlp.", mixer_norm="norm1", ffn_norm="norm2")
        block = (PartSpec.make("pre_norm", **pieces) if cfg.streams is None else
                 PartSpec.make("hyper_connections", streams=cfg.streams, mixer_streams="hc1.", ffn_streams="hc2.", **pieces))
        layers.append(LayerSpec(prefix=f"l{i}.", block=block, mixer=mixer, feed_forward=ffn, norm=norm))
    return ModelSpec(
        architecture="Sufolix",
        vocab_size=cfg.vocab,
        hidden_size=cfg.width,
        max_positions=cfg.max_positions,
        embedding_name="embed",
        head_name="head",
        final_norm_name="final.norm",
        final_norm=norm,
        layers=tuple(layers),
        weight_prefixes=("",),
        embedding_scale=cfg.embedding_scale,
        residual_streams=cfg.streams or 1,
    )


ARCHITECTURE = Architecture(
    name="sufolix",
    claims=("Sufolix", "sufolix"),
    read_config=SufolixConfig.from_dict,
    build_spec=build_spec,
)
