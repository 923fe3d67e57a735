"""Typed configuration of the Mamevik decoder, read from config.json.

The file is nested: `architecture` (the name), `vocab`, `width`, `norm.eps`, `embedding.bigram`
(`buckets`, `mul_prev`, `mul_cur`: a hashed table of token pairs added to the token's row),
`layers` (one object per layer: `type` = "mamba2" or "latent_attention", `mixer` with the
sizes of that mixer, `mlp` with `kind` "moe", `expert.ff`, `expert.limit`, `router.experts`,
`router.top`, or null), `loop` (`start`, `stop`, `times`: the layers start .. stop - 1 run
`times` times with the same weights), `logit_scale` and `logit_softcap`.  Every size and
constant comes from the file; a key that is absent means the mechanism is absent.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Any, Mapping, Optional, Tuple, Union

from .errors import ConfigError, UnsupportedConfig
from .sufolix import DEFAULT_MAX_POSITIONS, MAX_LAYERS, _int, _num, _obj


@dataclass(frozen=True)
class Bigram:
    buckets: int
    mul_prev: int
    mul_cur: int

    @classmethod
    def from_dict(cls, d: Any) -> "Bigram":
        d = _obj(d, "embedding.bigram")
        out = cls(_int(d, "buckets", "embedding.bigram"), _int(d, "mul_prev", "embedding.bigram"),
                  _int(d, "mul_cur", "embedding.bigram"))
        if max(out.buckets, out.mul_prev, out.mul_cur) >= 1 << 31:
            raise ConfigError("config.json: embedding.bigram: numbers must fit 31 bits")
        return out


@dataclass(frozen=True)
class StateSpaceMixer:
    heads: int
    vdim: int           # elements of a head
    state: int          # N: rows of a head's state matrix
    groups: int         # heads share their B and C in groups
    conv: int           # taps of the short convolution
    norm_groups: int    # parts of the output that are normed each by itself

    @classmethod
    def from_dict(cls, d: Any, what: str) -> "StateSpaceMixer":
        d = _obj(d, what)
        out = cls(*(_int(d, k, what) for k in ("heads", "vdim", "state", "groups", "conv", "norm_groups")))
        if out.heads % out.groups:
            raise ConfigError(f"config.json: {what}: {out.heads} heads are not a multiple of {out.groups} groups")
        if (out.heads * out.vdim) % out.norm_groups:
            raise ConfigError(f"config.json: {what}: heads * vdim is not a multiple of norm_groups")
        if out.conv > 16:
            raise UnsupportedConfig(f"config.json: {what}.conv: more than 16 taps are not served")
        if out.state > 256:
            raise UnsupportedConfig(f"config.json: {what}.state: more than 256 rows of state are not served")
        return out


@dataclass(frozen=True)
class LatentAttentionMixer:
    heads: int
    dim: int            # head size of queries and keys
    vdim: int           # head size of values
    kv_rank: int        # size of the cached latent
    scale: float
    window: Optional[int]   # None: every earlier token is read

    @classmethod
    def from_dict(cls, d: Any, what: str) -> "LatentAttentionMixer":
        d = _obj(d, what)
        mask = d.get("mask")
        window = None if mask is None else _int(_obj(mask, what + ".mask"), "size", what + ".mask")
        out = cls(_int(d, "heads", what), _int(d, "dim", what), _int(d, "vdim", what), _int(d, "kv_rank", what),
                  _num(d, "scale", what), window)
        if max(out.kv_rank, out.dim, out.vdim) > 512:
            raise UnsupportedConfig(f"config.json: {what}: kv_rank, dim and vdim beyond 512 are not served")
        return out


@dataclass(frozen=True)
class ExpertsFeedForward:
    experts: int
    top: int
    ff: int
    limit: float

    @classmethod
    def from_dict(cls, d: Any, what: str) -> "ExpertsFeedForward":
        d = _obj(d, what)
        if d.get("kind") != "moe":
            raise UnsupportedConfig(f"config.json: {what}.kind {d.get('kind')!r} is not served (moe)")
        router = _obj(d.get("router"), what + ".router")
        expert = _obj(d.get("expert"), what + ".expert")
        out = cls(_int(router, "experts", what + ".router"), _int(router, "top", what + ".router"),
                  _int(expert, "ff", what + ".expert"), _num(expert, "limit", what + ".expert"))
        if out.top > out.experts:
            raise ConfigError(f"config.json: {what}.router: top {out.top} of {out.experts} experts")
        if out.limit <= 0:
            raise ConfigError(f"config.json: {what}.expert.limit must be positive")
        if out.experts > 512 or out.top > 32:
            raise UnsupportedConfig(f"config.json: {what}.router: more than 512 experts or 32 a token are not served")
        return out


@dataclass(frozen=True)
class MamevikLayer:
    type: str           # "mamba2" | "latent_attention"
    mixer: Union[StateSpaceMixer, LatentAttentionMixer]
    mlp: Optional[ExpertsFeedForward]


@dataclass(frozen=True)
class Loop:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class MamevikConfig:
    vocab: int
    width: int
    eps: float
    bigram: Optional[Bigram]
    layers: Tuple[MamevikLayer, ...]
    loop: Optional[Loop]
    logit_scale: float
    logit_softcap: float            # 0: none
    max_positions: int = DEFAULT_MAX_POSITIONS

    def to_dict(self) -> dict:
        return asdict(self)

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "MamevikConfig":
        raw = _obj(raw, "the file")
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, (list, tuple)) or not layers_raw:
            raise ConfigError("config.json: layers must be a non-empty list")
        if len(layers_raw) > MAX_LAYERS:
            raise ConfigError("config.json: invalid layer count")
        layers = []
        for i, entry in enumerate(layers_raw):
            what = f"layers[{i}]"
            entry = _obj(entry, what)
            kind = entry.get("type")
            if kind == "mamba2":
                mixer = StateSpaceMixer.from_dict(entry.get("mixer"), what + ".mixer")
            elif kind == "latent_attention":
                mixer = LatentAttentionMixer.from_dict(entry.get("mixer"), what + ".mixer")
            else:
                raise UnsupportedConfig(f"config.json: {what}.type {kind!r} is not served (mamba2, latent_attention)")
            mlp = entry.get("mlp")
            layers.append(MamevikLayer(kind, mixer, None if mlp is None else ExpertsFeedForward.from_dict(mlp, what + ".mlp")))
        loop = raw.get("loop")
        if loop is not None:
            loop = _obj(loop, "loop")
            start = loop.get("start")
            if isinstance(start, bool) or not isinstance(start, int) or start < 0:
                raise ConfigError(f"config.json: loop.start must be an integer from 0, found {start!r}")
            loop = Loop(start, _int(loop, "stop", "loop"), _int(loop, "times", "loop"))
            if not loop.start < loop.stop <= len(layers):
                raise ConfigError(f"config.json: loop {loop.start} .. {loop.stop} does not lie within the {len(layers)} layers")
            if loop.times > 1024:
                raise ConfigError("config.json: loop.times is beyond any use")
        emb = raw.get("embedding")
        bigram = None
        if emb is not None and _obj(emb, "embedding").get("bigram") is not None:
            bigram = Bigram.from_dict(emb["bigram"])
        eps = _num(_obj(raw.get("norm"), "norm"), "eps", "norm")
        if eps <= 0:
            raise ConfigError("config.json: norm.eps must be positive")
        scale = _num(raw, "logit_scale", "the file") if "logit_scale" in raw else 1.0
        cap = _num(raw, "logit_softcap", "the file") if raw.get("logit_softcap") is not None else 0.0
        if cap < 0:
            raise ConfigError("config.json: logit_softcap must not be negative")
        max_positions = raw.get("max_positions", DEFAULT_MAX_POSITIONS)
        if isinstance(max_positions, bool) or not isinstance(max_positions, int) or max_positions <= 0:
            raise ConfigError("config.json: max_positions must be a positive integer")
        return cls(_int(raw, "vocab", "the file"), _int(raw, "width", "the file"), eps, bigram, tuple(layers), loop,
                   scale, cap, max_positions)
