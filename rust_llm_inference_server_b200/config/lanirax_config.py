"""Typed configuration of the Lanirax decoder, read from its `config.json`.

The file lists the layers one by one; every size and every constant that can differ between two
models of the design comes from it:

    {"architecture": "Lanirax", "vocab": V, "width": W, "norm": {"eps": e}, "postln_alpha": a,
     "layers": [{"type": "parallel" | "attention", "mixer": {...}, "mlp": {...} | null,
                 "weights_of": j (optional)}, ...]}

type "attention": mixer {heads, kv_heads, dim, vdim, scale, q_temp {coef, every} or absent}.
type "parallel": mixer {left {heads, kv_heads, dim, vdim, scale, mask {size}, rot {dims, base, scaling {factor,
original, fast, slow} or absent}}, right {heads, kv_heads, dim, vdim, conv}}.
mlp: kind "moe", expert {ff}, router {experts, top}.
A layer with `weights_of: j` has no tensors of its own and runs with layer j's, with a cache and a state
of its own; the rest of its entry has to equal layer j's.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .lasapel_config import UNBOUNDED_POSITIONS, RotaryConfig, _float, _int    # the shared field readers
from .model_config import ConfigError

ARCHITECTURE = "Lanirax"


def _heads(d: dict, where: str):
    heads, kv = _int(d, "heads", where), _int(d, "kv_heads", where)
    if heads % kv:
        raise ConfigError(f"config.json: {where}: {heads} heads are not a multiple of {kv} kv_heads")
    return heads, kv


@dataclass(frozen=True)
class SlopeAttentionConfig:
    """The mixer of an "attention" layer."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    q_temp_coef: Optional[float] = None     # None: no query temperature
    q_temp_every: int = 0

    @staticmethod
    def from_dict(d: dict, where: str) -> "SlopeAttentionConfig":
        heads, kv = _heads(d, where)
        qt = d.get("q_temp")
        coef, every = None, 0
        if qt is not None:
            if not isinstance(qt, dict):
                raise ConfigError(f"config.json: {where}.q_temp must be an object with 'coef' and 'every', or absent")
            coef, every = _float(qt, "coef", where + ".q_temp"), _int(qt, "every", where + ".q_temp")
        return SlopeAttentionConfig(heads, kv, _int(d, "dim", where), _int(d, "vdim", where), _float(d, "scale", where),
                                    coef, every)


@dataclass(frozen=True)
class WindowAttentionConfig:
    """The left branch of a "parallel" layer."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int
    rot: RotaryConfig

    @staticmethod
    def from_dict(d, where: str) -> "WindowAttentionConfig":
        if not isinstance(d, dict):
            raise ConfigError(f"config.json: {where} must be an object")
        heads, kv = _heads(d, where)
        mask = d.get("mask")
        if not isinstance(mask, dict):
            raise ConfigError(f"config.json: {where}.mask must be an object with 'size'")
        out = WindowAttentionConfig(heads, kv, _int(d, "dim", where), _int(d, "vdim", where), _float(d, "scale", where),
                                    _int(mask, "size", where + ".mask"), RotaryConfig.from_dict(d.get("rot"), where + ".rot"))
        if out.vdim != out.dim:
            raise ConfigError(f"config.json: {where}: the values are the keys, so vdim {out.vdim} must equal dim {out.dim}")
        if out.rot.dims > out.dim:
            raise ConfigError(f"config.json: {where}.rot.dims {out.rot.dims} exceeds dim {out.dim}")
        return out


@dataclass(frozen=True)
class DeltaRuleConfig:
    """The right branch of a "parallel" layer."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    @staticmethod
    def from_dict(d, where: str) -> "DeltaRuleConfig":
        if not isinstance(d, dict):
            raise ConfigError(f"config.json: {where} must be an object")
        heads, kv = _heads(d, where)
        return DeltaRuleConfig(heads, kv, _int(d, "dim", where), _int(d, "vdim", where), _int(d, "conv", where))


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: WindowAttentionConfig
    right: DeltaRuleConfig

    @staticmethod
    def from_dict(d: dict, where: str) -> "ParallelMixerConfig":
        return ParallelMixerConfig(WindowAttentionConfig.from_dict(d.get("left"), where + ".left"),
                                   DeltaRuleConfig.from_dict(d.get("right"), where + ".right"))


@dataclass(frozen=True)
class ExpertsConfig:
    ff: int
    experts: int
    top: int
    kind: str = "moe"

    @staticmethod
    def from_dict(d, where: str) -> "ExpertsConfig":
        if not isinstance(d, dict) or d.get("kind") != "moe":
            raise ConfigError(f"config.json: {where} must be null or an object of kind 'moe'")
        ex, r = d.get("expert"), d.get("router")
        if not isinstance(ex, dict) or not isinstance(r, dict):
            raise ConfigError(f"config.json: {where} needs the objects 'expert' and 'router'")
        experts, top = _int(r, "experts", where + ".router"), _int(r, "top", where + ".router")
        if top > experts:
            raise ConfigError(f"config.json: {where}.router: top {top} exceeds experts {experts}")
        return ExpertsConfig(_int(ex, "ff", where + ".expert"), experts, top)


@dataclass(frozen=True)
class LaniraxLayer:
    type: str
    mixer: object                    # SlopeAttentionConfig | ParallelMixerConfig
    mlp: Optional[ExpertsConfig]
    weights_of: Optional[int] = None  # the layer whose tensors this one runs with (None: its own)


@dataclass(frozen=True)
class LaniraxConfig:
    architecture = ARCHITECTURE

    vocab: int
    width: int
    eps: float
    alpha: float
    layers: tuple
    eos_token_ids: tuple = ()
    bos_token_id: Optional[int] = None
    max_positions: int = UNBOUNDED_POSITIONS     # the design has no positional table and no limit of its own

    MIXERS = {"attention": SlopeAttentionConfig, "parallel": ParallelMixerConfig}

    def owner(self, i: int) -> int:
        """The layer whose tensors layer i runs with."""
        j = self.layers[i].weights_of
        return i if j is None else j

    @classmethod
    def from_dict(cls, d: dict) -> "LaniraxConfig":
        vocab, width = _int(d, "vocab", "config"), _int(d, "width", "config")
        norm = d.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: 'norm' must be an object with 'eps'")
        eps = _float(norm, "eps", "norm")
        if not eps > 0:
            raise ConfigError("config.json: norm.eps must be positive")
        alpha = _float(d, "postln_alpha", "config")
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
            mixer = cls.MIXERS[kind].from_dict(entry["mixer"], where + ".mixer")
            mlp = entry.get("mlp")
            if mlp is not None:
                mlp = ExpertsConfig.from_dict(mlp, where + ".mlp")
            src = entry.get("weights_of")
            if src is not None:
                if not isinstance(src, int) or isinstance(src, bool) or not 0 <= src < len(raw) or src == i:
                    raise ConfigError(f"config.json: {where}.weights_of must name another layer, got {src!r}")
            layers.append(LaniraxLayer(kind, mixer, mlp, src))
        # a layer that borrows tensors names a layer that has them, and is the same layer otherwise
        resolved = []
        for i, layer in enumerate(layers):
            j, seen = layer.weights_of, {i}
            while j is not None and layers[j].weights_of is not None:
                if j in seen:
                    raise ConfigError(f"config.json: layers[{i}].weights_of leads back to itself")
                seen.add(j)
                j = layers[j].weights_of
            if j is not None and (layers[j].type, layers[j].mixer, layers[j].mlp) != (layer.type, layer.mixer, layer.mlp):
                raise ConfigError(f"config.json: layers[{i}] runs with the tensors of layers[{j}] and differs from it")
            resolved.append(LaniraxLayer(layer.type, layer.mixer, layer.mlp, j))
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else (eos,)))
        return cls(vocab, width, eps, alpha, tuple(resolved), eos_ids, d.get("bos_token_id"))
