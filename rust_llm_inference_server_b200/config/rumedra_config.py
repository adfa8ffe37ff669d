"""Typed configuration of the Rumedra decoder, read from its `config.json`.

The file lists the layers one by one; every size and every constant that can differ between two models of the
design comes from it:

    {"architecture": "Rumedra", "vocab": V, "width": W, "norm": {"eps": e}, "embedding": {"scale": s},
     "layers": [{"type": "parallel" | "hgrn2", "mixer": {...}, "mlp": {...} | null}, ...]}

type "hgrn2": mixer {heads, dim, vdim}.
type "parallel": mixer {left {heads, kv_heads, dim, vdim, scale, mask {size}, rot {dims, base, scaling {factor, low,
high, original} or absent}}, right {heads, dim, vdim, decay [one a head], rot {dims, base}}, left_scale, right_scale}.
mlp: kind "dense" {ff}; kind "moe" {expert {ff}, router {experts, top, scale, identity, groups {count, keep}},
shared {ff} or absent}.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .lasapel_config import UNBOUNDED_POSITIONS, _float, _int    # the shared field readers
from .model_config import ConfigError

ARCHITECTURE = "Rumedra"


def _obj(d, key: str, where: str) -> dict:
    v = d.get(key) if isinstance(d, dict) else None
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}.{key} must be an object")
    return v


@dataclass(frozen=True)
class RotationConfig:
    """Rotate-half rotation over the first `dims` entries of a head; `factor` None: plain frequencies."""
    dims: int
    base: float
    factor: Optional[float] = None
    low: float = 0.0
    high: float = 0.0
    original: float = 0.0

    @staticmethod
    def from_dict(d: dict, where: str, head_dim: int) -> "RotationConfig":
        dims, base = _int(d, "dims", where, 2), _float(d, "base", where)
        if dims % 2 or dims > head_dim or not base > 0:
            raise ConfigError(f"config.json: {where}: dims must be even and at most the head size {head_dim}, base positive")
        sc = d.get("scaling")
        if sc is None:
            return RotationConfig(dims, base)
        if not isinstance(sc, dict):
            raise ConfigError(f"config.json: {where}.scaling must be an object or absent")
        w = where + ".scaling"
        out = RotationConfig(dims, base, _float(sc, "factor", w), _float(sc, "low", w), _float(sc, "high", w),
                             _float(sc, "original", w))
        if not out.factor > 0 or not out.low > 0 or not out.high > out.low or not out.original > 0:
            raise ConfigError(f"config.json: {w}: factor, low and original must be positive and high above low")
        return out


@dataclass(frozen=True)
class WindowAttentionConfig:
    """The left branch of a "parallel" layer."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]            # None: every earlier token is seen
    rot: Optional[RotationConfig]

    @staticmethod
    def from_dict(d: dict, where: str) -> "WindowAttentionConfig":
        heads, kv = _int(d, "heads", where), _int(d, "kv_heads", where)
        if heads % kv:
            raise ConfigError(f"config.json: {where}: {heads} heads are not a multiple of {kv} kv_heads")
        dim = _int(d, "dim", where)
        mask = d.get("mask")
        window = _int(_obj(d, "mask", where), "size", where + ".mask") if mask is not None else None
        rot = RotationConfig.from_dict(_obj(d, "rot", where), where + ".rot", dim) if d.get("rot") is not None else None
        return WindowAttentionConfig(heads, kv, dim, _int(d, "vdim", where), _float(d, "scale", where), window, rot)


@dataclass(frozen=True)
class RetentionConfig:
    """The right branch of a "parallel" layer."""
    heads: int
    dim: int
    vdim: int
    decay: tuple
    rot: Optional[RotationConfig]

    @staticmethod
    def from_dict(d: dict, where: str) -> "RetentionConfig":
        heads, dim = _int(d, "heads", where), _int(d, "dim", where)
        decay = d.get("decay")
        if not isinstance(decay, list) or len(decay) != heads or \
                any(isinstance(g, bool) or not isinstance(g, (int, float)) for g in decay):
            raise ConfigError(f"config.json: {where}.decay must list one number a head ({heads})")
        rot = RotationConfig.from_dict(_obj(d, "rot", where), where + ".rot", dim) if d.get("rot") is not None else None
        if rot is not None and rot.factor is not None:
            raise ConfigError(f"config.json: {where}.rot: this branch's rotation has no frequency scaling")
        return RetentionConfig(heads, dim, _int(d, "vdim", where), tuple(float(g) for g in decay), rot)


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: WindowAttentionConfig
    right: RetentionConfig
    left_scale: float
    right_scale: float

    @staticmethod
    def from_dict(d: dict, where: str) -> "ParallelMixerConfig":
        return ParallelMixerConfig(WindowAttentionConfig.from_dict(_obj(d, "left", where), where + ".left"),
                                   RetentionConfig.from_dict(_obj(d, "right", where), where + ".right"),
                                   _float(d, "left_scale", where), _float(d, "right_scale", where))


@dataclass(frozen=True)
class ForgetGateConfig:
    """The mixer of an "hgrn2" layer."""
    heads: int
    dim: int
    vdim: int

    @staticmethod
    def from_dict(d: dict, where: str) -> "ForgetGateConfig":
        return ForgetGateConfig(_int(d, "heads", where), _int(d, "dim", where), _int(d, "vdim", where))


@dataclass(frozen=True)
class DenseConfig:
    ff: int
    kind: str = "dense"


@dataclass(frozen=True)
class ExpertsConfig:
    ff: int
    experts: int                     # experts with tensors; the router has `experts + identity` outputs
    top: int
    scale: float
    identity: int
    groups: int
    keep: int
    shared_ff: Optional[int]         # None: no shared expert
    kind: str = "moe"

    @property
    def outputs(self) -> int:
        return self.experts + self.identity

    @staticmethod
    def from_dict(d: dict, where: str) -> "ExpertsConfig":
        ex, r = _obj(d, "expert", where), _obj(d, "router", where)
        w = where + ".router"
        experts, top = _int(r, "experts", w), _int(r, "top", w)
        identity = _int(r, "identity", w, 0) if r.get("identity") is not None else 0
        scale = _float(r, "scale", w) if r.get("scale") is not None else 1.0
        count, keep = 1, 1
        if r.get("groups") is not None:
            g = _obj(r, "groups", w)
            count, keep = _int(g, "count", w + ".groups"), _int(g, "keep", w + ".groups")
        n_out = experts + identity
        if n_out % count or keep > count:
            raise ConfigError(f"config.json: {w}: {n_out} router outputs do not form {count} equal groups, or keep {keep} "
                              f"exceeds them")
        if top > keep * (n_out // count):
            raise ConfigError(f"config.json: {w}: top {top} exceeds the {keep * (n_out // count)} outputs of the kept groups")
        shared = d.get("shared")
        shared_ff = _int(_obj(d, "shared", where), "ff", where + ".shared") if shared is not None else None
        return ExpertsConfig(_int(ex, "ff", where + ".expert"), experts, top, scale, identity, count, keep, shared_ff)


def _mlp(d, where: str):
    if d is None:
        return None
    if not isinstance(d, dict) or d.get("kind") not in ("dense", "moe"):
        raise ConfigError(f"config.json: {where} must be null or an object of kind 'dense' or 'moe'")
    if d["kind"] == "dense":
        return DenseConfig(_int(d, "ff", where))
    return ExpertsConfig.from_dict(d, where)


@dataclass(frozen=True)
class RumedraLayer:
    type: str
    mixer: object                    # ParallelMixerConfig | ForgetGateConfig
    mlp: object                      # DenseConfig | ExpertsConfig | None


@dataclass(frozen=True)
class RumedraConfig:
    architecture = ARCHITECTURE

    vocab: int
    width: int
    eps: float
    embedding_scale: float
    layers: tuple
    eos_token_ids: tuple = ()
    bos_token_id: Optional[int] = None
    max_positions: int = UNBOUNDED_POSITIONS     # the design has no positional table and no limit of its own

    MIXERS = {"parallel": ParallelMixerConfig, "hgrn2": ForgetGateConfig}

    @classmethod
    def from_dict(cls, d: dict) -> "RumedraConfig":
        vocab, width = _int(d, "vocab", "config"), _int(d, "width", "config")
        eps = _float(_obj(d, "norm", "config"), "eps", "norm")
        if not eps > 0:
            raise ConfigError("config.json: norm.eps must be positive")
        emb = d.get("embedding")
        scale = _float(emb, "scale", "embedding") if isinstance(emb, dict) and emb.get("scale") is not None else 1.0
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw):
            where = f"layers[{i}]"
            if not isinstance(entry, dict) or not isinstance(entry.get("mixer"), dict):
                raise ConfigError(f"config.json: {where} must be an object with 'type' and 'mixer'")
            kind = entry.get("type")
            if kind not in cls.MIXERS:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not one of {sorted(cls.MIXERS)}")
            layers.append(RumedraLayer(kind, cls.MIXERS[kind].from_dict(entry["mixer"], where + ".mixer"),
                                       _mlp(entry.get("mlp"), where + ".mlp")))
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else (eos,)))
        return cls(vocab, width, eps, scale, tuple(layers), eos_ids, d.get("bos_token_id"))
