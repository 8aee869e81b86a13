"""Typed configuration of the Zebivik decoder, read from config.json.

The file is nested: `architecture` (the name), `vocab`, `width`, `norm.eps`, `residual_mult` (the constant on what
a sublayer adds to the stream), `logit_softcap`, and `layers`, one object per layer with `type` ("parallel": softmax
attention beside a linear attention with a constant decay; "rglru": a gated linear recurrence behind a short
convolution), `mixer` (the sizes and constants of that mixer) and `mlp` (`kind` "dense" with `ff` and `limit`, or
"moe" with `router` (`experts`, `top`, `scale`, optional `groups` {`count`, `keep`}), `expert.ff` and an optional
`shared.ff`; or null for a layer without feed-forward).  Every size and constant comes from the file; a key that
is absent means the mechanism is absent.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Any, Mapping, Optional, Tuple, Union

from .errors import ConfigError, UnsupportedConfig
from .sufolix import DEFAULT_MAX_POSITIONS, MAX_LAYERS, _int, _num, _obj


@dataclass(frozen=True)
class RotaryScaling:
    factor: float
    low: float
    high: float
    original: float


@dataclass(frozen=True)
class Rotation:
    base: float
    dims: int
    scaling: Optional[RotaryScaling]


@dataclass(frozen=True)
class SoftmaxBranch:
    heads: int
    kv_heads: int
    dim: int                 # head size of queries and keys
    vdim: int                # head size of values
    scale: float             # multiplier of q.k
    rot: Optional[Rotation]

    @classmethod
    def from_dict(cls, d: Any, what: str) -> "SoftmaxBranch":
        d = _obj(d, what)
        heads, kv = _int(d, "heads", what), _int(d, "kv_heads", what)
        dim, vdim = _int(d, "dim", what), _int(d, "vdim", what)
        if heads % kv:
            raise ConfigError(f"config.json: {what}: {heads} heads are not a multiple of {kv} kv_heads")
        rot = None
        if d.get("rot") is not None:
            r = _obj(d["rot"], what + ".rot")
            dims = _int(r, "dims", what + ".rot")
            if dims % 2 or dims > dim:
                raise ConfigError(f"config.json: {what}.rot.dims must be even and at most dim, found {dims}")
            base = _num(r, "base", what + ".rot")
            if base <= 0:
                raise ConfigError(f"config.json: {what}.rot.base must be positive")
            scaling = None
            if r.get("scaling") is not None:
                s = _obj(r["scaling"], what + ".rot.scaling")
                scaling = RotaryScaling(*(_num(s, k, what + ".rot.scaling") for k in ("factor", "low", "high", "original")))
                if scaling.factor <= 0 or scaling.low <= 0 or scaling.original <= 0 or scaling.high <= scaling.low:
                    raise ConfigError(f"config.json: {what}.rot.scaling: factor, low and original must be positive and high above low")
            rot = Rotation(base, dims, scaling)
        if max(dim, vdim) > 256:
            raise UnsupportedConfig(f"config.json: {what}: head sizes beyond 256 are not served")
        return cls(heads, kv, dim, vdim, _num(d, "scale", what), rot)


@dataclass(frozen=True)
class LinearBranch:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]     # one per head

    @classmethod
    def from_dict(cls, d: Any, what: str) -> "LinearBranch":
        d = _obj(d, what)
        heads = _int(d, "heads", what)
        decay = d.get("decay")
        if not isinstance(decay, (list, tuple)) or len(decay) != heads:
            raise ConfigError(f"config.json: {what}.decay must list one number per head")
        out = []
        for v in decay:
            if isinstance(v, bool) or not isinstance(v, (int, float)) or not 0.0 <= float(v) <= 1.0:
                raise ConfigError(f"config.json: {what}.decay holds {v!r}; a decay lies in [0, 1]")
            out.append(float(v))
        dim, vdim = _int(d, "dim", what), _int(d, "vdim", what)
        if dim > 256:
            raise UnsupportedConfig(f"config.json: {what}.dim: a state of more than 256 rows is not served")
        return cls(heads, dim, vdim, tuple(out))


@dataclass(frozen=True)
class ParallelMixer:
    left: SoftmaxBranch
    right: LinearBranch
    left_scale: float
    right_scale: float

    @classmethod
    def from_dict(cls, d: Any, what: str) -> "ParallelMixer":
        d = _obj(d, what)
        return cls(SoftmaxBranch.from_dict(d.get("left"), what + ".left"), LinearBranch.from_dict(d.get("right"), what + ".right"),
                   _num(d, "left_scale", what), _num(d, "right_scale", what))


@dataclass(frozen=True)
class RecurrentMixer:
    width: int
    blocks: int
    conv: int

    @classmethod
    def from_dict(cls, d: Any, what: str) -> "RecurrentMixer":
        d = _obj(d, what)
        out = cls(_int(d, "width", what), _int(d, "blocks", what), _int(d, "conv", what))
        if out.width % out.blocks:
            raise ConfigError(f"config.json: {what}: width {out.width} is not a multiple of {out.blocks} blocks")
        if out.conv > 16:
            raise UnsupportedConfig(f"config.json: {what}.conv: more than 16 taps are not served")
        if out.width // out.blocks > 640:
            raise UnsupportedConfig(f"config.json: {what}: blocks of more than 640 channels are not served")
        return out


@dataclass(frozen=True)
class DenseFeedForward:
    ff: int
    limit: float


@dataclass(frozen=True)
class ExpertsFeedForward:
    experts: int
    top: int
    scale: float
    groups: int          # 1: no groups
    keep: int
    ff: int
    shared_ff: int       # 0: no shared expert


def _mlp(d: Any, what: str):
    d = _obj(d, what)
    kind = d.get("kind")
    if kind == "dense":
        out = DenseFeedForward(_int(d, "ff", what), _num(d, "limit", what))
        if out.limit <= 0:
            raise ConfigError(f"config.json: {what}.limit must be positive")
        return out
    if kind != "moe":
        raise UnsupportedConfig(f"config.json: {what}.kind {kind!r} is not served (dense, moe)")
    r = _obj(d.get("router"), what + ".router")
    experts, top = _int(r, "experts", what + ".router"), _int(r, "top", what + ".router")
    groups, keep = 1, 1
    if r.get("groups") is not None:
        g = _obj(r["groups"], what + ".router.groups")
        groups, keep = _int(g, "count", what + ".router.groups"), _int(g, "keep", what + ".router.groups")
        if experts % groups or keep > groups:
            raise ConfigError(f"config.json: {what}.router.groups: {groups} groups (keeping {keep}) of {experts} experts")
        if groups > 32:
            raise UnsupportedConfig(f"config.json: {what}.router.groups: more than 32 groups are not served")
    if top > experts // groups * keep:
        raise ConfigError(f"config.json: {what}.router: top {top} exceeds the experts that can be chosen")
    if experts > 512 or top > 32:
        raise UnsupportedConfig(f"config.json: {what}.router: more than 512 experts or 32 a token are not served")
    scale = _num(r, "scale", what + ".router") if "scale" in r else 1.0
    shared = d.get("shared")
    shared_ff = 0 if shared is None else _int(_obj(shared, what + ".shared"), "ff", what + ".shared")
    return ExpertsFeedForward(experts, top, scale, groups, keep, _int(_obj(d.get("expert"), what + ".expert"), "ff", what + ".expert"),
                              shared_ff)


@dataclass(frozen=True)
class ZebivikLayer:
    type: str            # "parallel" | "rglru"
    mixer: Union[ParallelMixer, RecurrentMixer]
    mlp: Union[DenseFeedForward, ExpertsFeedForward, None]


@dataclass(frozen=True)
class ZebivikConfig:
    vocab: int
    width: int
    eps: float
    residual_mult: float
    layers: Tuple[ZebivikLayer, ...]
    logit_softcap: float            # 0: none
    max_positions: int = DEFAULT_MAX_POSITIONS

    def to_dict(self) -> dict:
        return asdict(self)

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "ZebivikConfig":
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
            if kind == "parallel":
                mixer = ParallelMixer.from_dict(entry.get("mixer"), what + ".mixer")
            elif kind == "rglru":
                mixer = RecurrentMixer.from_dict(entry.get("mixer"), what + ".mixer")
            else:
                raise UnsupportedConfig(f"config.json: {what}.type {kind!r} is not served (parallel, rglru)")
            mlp = entry.get("mlp")
            layers.append(ZebivikLayer(kind, mixer, None if mlp is None else _mlp(mlp, what + ".mlp")))
        eps = _num(_obj(raw.get("norm"), "norm"), "eps", "norm")
        if eps <= 0:
            raise ConfigError("config.json: norm.eps must be positive")
        mult = _num(raw, "residual_mult", "the file") if "residual_mult" in raw else 1.0
        cap = _num(raw, "logit_softcap", "the file") if raw.get("logit_softcap") is not None else 0.0
        if cap < 0:
            raise ConfigError("config.json: logit_softcap must not be negative")
        max_positions = raw.get("max_positions", DEFAULT_MAX_POSITIONS)
        if isinstance(max_positions, bool) or not isinstance(max_positions, int) or max_positions <= 0:
            raise ConfigError("config.json: max_positions must be a positive integer")
        return cls(_int(raw, "vocab", "the file"), _int(raw, "width", "the file"), eps, mult, tuple(layers), cap, max_positions)
