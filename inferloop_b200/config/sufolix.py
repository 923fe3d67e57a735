"""Typed configuration of the Sufolix decoder, read from config.json.

The file is nested: `architecture` (the name), `vocab`, `width`, `norm.eps`,
`embedding.scale`, optional `streams` (copies of the residual stream), and `layers`, one
object per layer with `type`, `mixer` (its sizes and constants) and `mlp` (`kind` dense or
moe with its sizes, or null for a layer without feed-forward).  Every size and constant
comes from the file; a key that is absent means the mechanism is absent.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Any, Mapping, Optional, Tuple

from .errors import ConfigError, UnsupportedConfig

MAX_LAYERS = 10000
# The file gives no limit on positions; the engine's tables are made for this many.
DEFAULT_MAX_POSITIONS = 1 << 17


def _obj(d: Any, what: str) -> Mapping[str, Any]:
    if not isinstance(d, Mapping):
        raise ConfigError(f"config.json: {what} must be an object, found {d!r}")
    return d


def _int(d: Mapping[str, Any], key: str, what: str) -> int:
    if key not in d:
        raise ConfigError(f"config.json: {what} needs {key!r}")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {what}.{key} must be a positive integer, found {v!r}")
    return v


def _num(d: Mapping[str, Any], key: str, what: str) -> float:
    if key not in d:
        raise ConfigError(f"config.json: {what} needs {key!r}")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, (int, float)) or v != v or v in (float("inf"), float("-inf")):
        raise ConfigError(f"config.json: {what}.{key} must be a finite number, found {v!r}")
    return float(v)


@dataclass(frozen=True)
class SufolixAttention:
    heads: int
    kv_heads: int
    dim: int                     # head size of queries and keys
    vdim: int                    # head size of values
    scale: float                 # multiplier of q.k
    rot_base: Optional[float]    # None: no rotation
    rot_dims: int
    v_mix: bool

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], what: str) -> "SufolixAttention":
        d = _obj(d, what)
        heads, kv = _int(d, "heads", what), _int(d, "kv_heads", what)
        dim, vdim = _int(d, "dim", what), _int(d, "vdim", what)
        if heads % kv:
            raise ConfigError(f"config.json: {what}: {heads} heads are not a multiple of {kv} kv_heads")
        base, dims = None, 0
        rot = d.get("rot")
        if rot is not None:
            rot = _obj(rot, what + ".rot")
            base, dims = _num(rot, "base", what + ".rot"), _int(rot, "dims", what + ".rot")
            if dims % 2 or dims > dim or base <= 0:
                raise ConfigError(f"config.json: {what}.rot: dims must be even and at most dim, base positive")
        v_mix = d.get("v_mix", False)
        if not isinstance(v_mix, bool):
            raise ConfigError(f"config.json: {what}.v_mix must be true or false")
        return cls(heads, kv, dim, vdim, _num(d, "scale", what), base, dims, v_mix)


@dataclass(frozen=True)
class SufolixFeedForward:
    kind: str                    # "dense" | "moe"
    ff: int                      # dense: its inner size; moe: an expert's
    experts: int = 0
    top: int = 0
    shared_ff: int = 0           # 0: no shared expert

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], what: str) -> "SufolixFeedForward":
        d = _obj(d, what)
        kind = d.get("kind")
        if kind == "dense":
            return cls("dense", _int(d, "ff", what))
        if kind == "moe":
            router = _obj(d.get("router"), what + ".router")
            experts, top = _int(router, "experts", what + ".router"), _int(router, "top", what + ".router")
            if top > experts:
                raise ConfigError(f"config.json: {what}.router: top {top} of {experts} experts")
            shared = d.get("shared")
            shared_ff = 0 if shared is None else _int(_obj(shared, what + ".shared"), "ff", what + ".shared")
            return cls("moe", _int(_obj(d.get("expert"), what + ".expert"), "ff", what + ".expert"), experts, top, shared_ff)
        raise UnsupportedConfig(f"config.json: {what}.kind {kind!r} is not served (dense, moe)")


@dataclass(frozen=True)
class SufolixLayer:
    mixer: SufolixAttention
    mlp: Optional[SufolixFeedForward]


@dataclass(frozen=True)
class SufolixConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    streams: Optional[int]       # None: one plain residual stream
    layers: Tuple[SufolixLayer, ...]
    max_positions: int = DEFAULT_MAX_POSITIONS

    def to_dict(self) -> dict:
        return asdict(self)

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "SufolixConfig":
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
            if entry.get("type") != "attention":
                raise UnsupportedConfig(f"config.json: {what}.type {entry.get('type')!r} is not served (attention)")
            mlp = entry.get("mlp")
            layers.append(SufolixLayer(SufolixAttention.from_dict(entry.get("mixer"), what + ".mixer"),
                                       None if mlp is None else SufolixFeedForward.from_dict(mlp, what + ".mlp")))
        mixing = [l.mixer for l in layers if l.mixer.v_mix]
        if any((m.kv_heads, m.vdim) != (mixing[0].kv_heads, mixing[0].vdim) for m in mixing):
            raise ConfigError("config.json: layers that mix values must agree in kv_heads and vdim")
        streams = raw.get("streams")
        if streams is not None and (isinstance(streams, bool) or not isinstance(streams, int) or not 0 < streams <= 16):
            raise ConfigError(f"config.json: streams must be an integer from 1 to 16, found {streams!r}")
        emb = raw.get("embedding")
        scale = 1.0 if emb is None else _num(_obj(emb, "embedding"), "scale", "embedding")
        eps = _num(_obj(raw.get("norm"), "norm"), "eps", "norm")
        if eps <= 0:
            raise ConfigError("config.json: norm.eps must be positive")
        max_positions = raw.get("max_positions", DEFAULT_MAX_POSITIONS)
        if isinstance(max_positions, bool) or not isinstance(max_positions, int) or max_positions <= 0:
            raise ConfigError("config.json: max_positions must be a positive integer")
        return cls(_int(raw, "vocab", "the file"), _int(raw, "width", "the file"), eps, scale, streams, tuple(layers),
                   max_positions)
