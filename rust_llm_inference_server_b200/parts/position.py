"""Position encodings of the attention mixer.

Rotary encoding with the reference's frequency rules (crates/model/src/rope.rs:19-49): inverse
frequencies in float32, scaled per frequency when rope_type is "llama3".  Angles position * f are
formed in float32 inside the kernel, so no table bounds the position.
"""

from __future__ import annotations

import math

import numpy as np
import torch

from .. import ops
from .base import PositionEncoding, register_position


def rope_inverse_frequencies(head_dim: int, theta: float, scaling=None) -> np.ndarray:
    """float32 [head_dim / 2].  1 / theta^(2j/d); for llama3 scaling a frequency whose wavelength
    is shorter than original/high is kept, longer than original/low is divided by `factor`, and
    between the two is blended linearly in original/wavelength (rope.rs:26-46)."""
    one = np.float32(1.0)
    th = np.float32(theta)
    exps = np.arange(0, head_dim, 2, dtype=np.float32) / np.float32(head_dim)
    freqs = (one / np.power(th, exps, dtype=np.float32)).astype(np.float32)
    if scaling is None or getattr(scaling, "rope_type", None) != "llama3":
        return freqs
    factor = np.float32(scaling.factor)
    low = np.float32(scaling.low_freq_factor)
    high = np.float32(scaling.high_freq_factor)
    orig = np.float32(scaling.original_max_position_embeddings)
    wavelen = (np.float32(2.0) * np.float32(math.pi) / freqs).astype(np.float32)
    smooth = ((orig / wavelen - low) / (high - low)).astype(np.float32)
    blended = ((one - smooth) * freqs / factor + smooth * freqs).astype(np.float32)
    out = np.where(wavelen < orig / high, freqs,
                   np.where(wavelen > orig / low, (freqs / factor).astype(np.float32), blended))
    return out.astype(np.float32)


def rope_inverse_frequencies_exact(head_dim: int, theta: float, scaling=None) -> np.ndarray:
    """The same rule as `rope_inverse_frequencies`, worked out in float64 and rounded to float32 once."""
    f = np.power(float(theta), -np.arange(0, head_dim, 2, dtype=np.float64) / float(head_dim))
    if scaling is None or getattr(scaling, "rope_type", None) != "llama3":
        return f.astype(np.float32)
    factor, low, high = float(scaling.factor), float(scaling.low_freq_factor), float(scaling.high_freq_factor)
    orig = float(scaling.original_max_position_embeddings)
    wavelen = 2.0 * math.pi / f
    smooth = (orig / wavelen - low) / (high - low) if high != low else np.zeros_like(f)
    blended = (1.0 - smooth) * f / factor + smooth * f
    return np.where(wavelen < orig / high, f, np.where(wavelen > orig / low, f / factor, blended)).astype(np.float32)


def yarn_inverse_frequencies(dims: int, base: float, factor=None, original: float = 0.0, fast: float = 0.0,
                             slow: float = 0.0):
    """(float32 [dims / 2] frequencies, multiplier of cos and sin) of `YarnRopeSpec`'s rule, worked out
    in float64 and rounded once."""
    half = dims // 2
    i = np.arange(half, dtype=np.float64)
    f = np.power(float(base), -2.0 * i / dims)
    if factor is None:
        return f.astype(np.float32), 1.0

    def dim_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(dim_of(fast)), 0)
    hi = min(math.ceil(dim_of(slow)), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    f = f / factor * ramp + f * (1.0 - ramp)
    return f.astype(np.float32), 0.1 * math.log(factor) + 1.0


class Rope(PositionEncoding):
    pairing = "half"         # entry i turns with entry i + head_dim / 2

    def __init__(self, spec, dtype, device):
        if spec.head_dim <= 0 or spec.head_dim % 2:
            raise ValueError(f"a rotation in pairs takes an even number of entries, got {spec.head_dim}")
        self.head_dim = spec.head_dim
        rule = rope_inverse_frequencies_exact if getattr(spec, "exact", False) else rope_inverse_frequencies
        inv = rule(spec.head_dim, spec.theta, spec.scaling)
        self.inv_freq = torch.from_numpy(inv).to(device)

    def rotation(self):
        return self.inv_freq, self.head_dim, 1.0

    def encode_and_store(self, qkv, q_out, cache, step, n_heads, n_kv_heads, head_dim, store):
        slots = step.slots[cache.group] if (store and cache is not None) else None
        ops.rope_cache(qkv, q_out, cache.k if slots is not None else None,
                       cache.v if slots is not None else None, step.positions, slots,
                       self.inv_freq, n_heads, n_kv_heads, head_dim,
                       cache.page_size if cache is not None else 1)

    def rotate_half_table(self):
        return self.inv_freq


class NoPosition(PositionEncoding):
    """No encoding: q is copied out and k, v are stored as they are."""

    def __init__(self, spec, dtype, device):
        pass

    def encode_and_store(self, qkv, q_out, cache, step, n_heads, n_kv_heads, head_dim, store):
        slots = step.slots[cache.group] if (store and cache is not None) else None
        ops.rope_cache(qkv, q_out, cache.k if slots is not None else None,
                       cache.v if slots is not None else None, step.positions, slots,
                       None, n_heads, n_kv_heads, head_dim,
                       cache.page_size if cache is not None else 1)

    def rotate_half_table(self):
        return None


class YarnRope(PositionEncoding):
    """A rotation a mixer applies itself: `rotation()` gives (float32 frequencies on the device, how
    many leading entries are rotated, the multiplier of cos and sin); `pairing` says which entries turn
    together ("half" or "adjacent")."""

    def __init__(self, spec, dtype, device):
        if spec.dims <= 0 or spec.dims % 2:
            raise ValueError(f"a rotation in pairs takes an even number of entries, got {spec.dims}")
        self.pairing = getattr(spec, "pairing", "half")
        if self.pairing not in ("half", "adjacent"):
            raise ValueError(f"a rotation pairs entries by 'half' or 'adjacent', got {self.pairing!r}")
        inv, self.magnitude = yarn_inverse_frequencies(spec.dims, spec.base, spec.factor, spec.original,
                                                       spec.fast, spec.slow)
        self.dims = int(spec.dims)
        self.inv_freq = torch.from_numpy(inv).to(device)

    def rotation(self):
        return self.inv_freq, self.dims, float(self.magnitude)


register_position("rope", Rope)
register_position("yarn_rope", YarnRope)
register_position("none", NoPosition)
