"""Typed configuration of the Dalavik decoder, read from config.json.

The file is nested: `architecture` (the name), `vocab`, `width`, `norm` (`eps`, `groups`: the norm
divides each of `groups` equal parts of a row by that part's root mean square), `token_side.dim`
(width of the per-layer slice of a second token table; absent: no such input), and `layers`, one
object per layer: `type` = "latent_attention" or "attention", `mixer` with that mixer's sizes and
constants, `mlp` (`kind` "dense", `ff`) or null.

  latent_attention   heads, dim (unrotated query/key size a head), rot_dim (rotated size), vdim,
                     q_rank, kv_rank, scale, rot.base, rot.dims, and optionally kv_from: the layer
                     whose cached latent and rotated key part this one reads
  attention          heads, kv_heads, dim, vdim, scale, and optionally softcap (0: none) and
                     q_temp (coef, every)

Every size and constant comes from the file; a key that is absent means the mechanism is absent.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Any, Mapping, Optional, Tuple, Union

from .errors import ConfigError, UnsupportedConfig
from .sufolix import DEFAULT_MAX_POSITIONS, MAX_LAYERS, _int, _num, _obj


@dataclass(frozen=True)
class RotatedLatentMixer:
    heads: int
    dim: int            # unrotated elements of a head's query and key
    rot_dim: int        # rotated elements: a head's query ends in them, the keys share one such part
    vdim: int
    q_rank: int         # size of the queries' latent
    kv_rank: int        # size of the cached latent
    scale: float
    rot_base: float
    rot_dims: int       # how many of the rot_dim elements turn (in pairs of neighbours)
    kv_from: Optional[int]

    @classmethod
    def from_dict(cls, d: Any, what: str) -> "RotatedLatentMixer":
        d = _obj(d, what)
        rot = _obj(d.get("rot"), what + ".rot")
        kv_from = d.get("kv_from")
        if kv_from is not None and (isinstance(kv_from, bool) or not isinstance(kv_from, int) or kv_from < 0):
            raise ConfigError(f"config.json: {what}.kv_from must be a layer's number, found {kv_from!r}")
        out = cls(_int(d, "heads", what), _int(d, "dim", what), _int(d, "rot_dim", what), _int(d, "vdim", what),
                  _int(d, "q_rank", what), _int(d, "kv_rank", what), _num(d, "scale", what), _num(rot, "base", what + ".rot"),
                  _int(rot, "dims", what + ".rot"), kv_from)
        if out.rot_dims % 2 or out.rot_dims > out.rot_dim:
            raise ConfigError(f"config.json: {what}.rot.dims {out.rot_dims} must be even and at most rot_dim {out.rot_dim}")
        if out.rot_base <= 0:
            raise ConfigError(f"config.json: {what}.rot.base must be positive")
        if out.kv_rank + out.rot_dim > 512 or max(out.dim, out.vdim) > 512:
            raise UnsupportedConfig(f"config.json: {what}: kv_rank + rot_dim, dim and vdim beyond 512 are not served")
        return out


@dataclass(frozen=True)
class QueryTemperature:
    coef: float
    every: int


@dataclass(frozen=True)
class MixedHeadsMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float                      # 0: scores are not capped
    q_temp: Optional[QueryTemperature]

    @classmethod
    def from_dict(cls, d: Any, what: str) -> "MixedHeadsMixer":
        d = _obj(d, what)
        temp = d.get("q_temp")
        if temp is not None:
            temp = _obj(temp, what + ".q_temp")
            temp = QueryTemperature(_num(temp, "coef", what + ".q_temp"), _int(temp, "every", what + ".q_temp"))
        cap = _num(d, "softcap", what) if d.get("softcap") is not None else 0.0
        if cap < 0:
            raise ConfigError(f"config.json: {what}.softcap must not be negative")
        out = cls(_int(d, "heads", what), _int(d, "kv_heads", what), _int(d, "dim", what), _int(d, "vdim", what),
                  _num(d, "scale", what), cap, temp)
        if out.heads % out.kv_heads:
            raise ConfigError(f"config.json: {what}: {out.heads} heads are not a multiple of {out.kv_heads} kv_heads")
        if max(out.dim, out.vdim) > 512:
            raise UnsupportedConfig(f"config.json: {what}: head sizes beyond 512 are not served")
        if out.heads * out.vdim > 8192:
            raise UnsupportedConfig(f"config.json: {what}: heads * vdim beyond 8192 is not served")
        return out


@dataclass(frozen=True)
class DenseFeedForward:
    ff: int

    @classmethod
    def from_dict(cls, d: Any, what: str) -> "DenseFeedForward":
        d = _obj(d, what)
        if d.get("kind") != "dense":
            raise UnsupportedConfig(f"config.json: {what}.kind {d.get('kind')!r} is not served (dense)")
        return cls(_int(d, "ff", what))


@dataclass(frozen=True)
class DalavikLayer:
    type: str           # "latent_attention" | "attention"
    mixer: Union[RotatedLatentMixer, MixedHeadsMixer]
    mlp: Optional[DenseFeedForward]


@dataclass(frozen=True)
class DalavikConfig:
    vocab: int
    width: int
    eps: float
    norm_groups: int
    side_dim: int                   # 0: no per-layer token input
    layers: Tuple[DalavikLayer, ...]
    max_positions: int = DEFAULT_MAX_POSITIONS

    def to_dict(self) -> dict:
        return asdict(self)

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "DalavikConfig":
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
            if kind == "latent_attention":
                mixer = RotatedLatentMixer.from_dict(entry.get("mixer"), what + ".mixer")
            elif kind == "attention":
                mixer = MixedHeadsMixer.from_dict(entry.get("mixer"), what + ".mixer")
            else:
                raise UnsupportedConfig(f"config.json: {what}.type {kind!r} is not served (latent_attention, attention)")
            mlp = entry.get("mlp")
            layers.append(DalavikLayer(kind, mixer, None if mlp is None else DenseFeedForward.from_dict(mlp, what + ".mlp")))
        for i, layer in enumerate(layers):
            m = layer.mixer
            if isinstance(m, RotatedLatentMixer) and m.kv_from is not None:
                src = layers[m.kv_from].mixer if m.kv_from < len(layers) else None
                if m.kv_from >= i or not isinstance(src, RotatedLatentMixer) or src.kv_from is not None:
                    raise ConfigError(f"config.json: layers[{i}].mixer.kv_from {m.kv_from} must name an earlier latent layer "
                                      "that keeps a cache of its own")
                if (src.kv_rank, src.rot_dim, src.rot_base, src.rot_dims) != (m.kv_rank, m.rot_dim, m.rot_base, m.rot_dims):
                    raise ConfigError(f"config.json: layers[{i}].mixer reads the cache of layer {m.kv_from}, whose kv_rank, "
                                      "rot_dim or rotation differ")
        norm = _obj(raw.get("norm"), "norm")
        eps = _num(norm, "eps", "norm")
        if eps <= 0:
            raise ConfigError("config.json: norm.eps must be positive")
        groups = _int(norm, "groups", "norm") if norm.get("groups") is not None else 1
        width = _int(raw, "width", "the file")
        if width % groups or groups > 64:
            raise ConfigError(f"config.json: norm.groups {groups} must divide the width {width} (at most 64)")
        side = raw.get("token_side")
        side_dim = 0 if side is None else _int(_obj(side, "token_side"), "dim", "token_side")
        max_positions = raw.get("max_positions", DEFAULT_MAX_POSITIONS)
        if isinstance(max_positions, bool) or not isinstance(max_positions, int) or max_positions <= 0:
            raise ConfigError("config.json: max_positions must be a positive integer")
        return cls(_int(raw, "vocab", "the file"), width, eps, groups, side_dim, tuple(layers), max_positions)
