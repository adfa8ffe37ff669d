"""Causal grouped-query attention with per-head RMS norms of queries and keys, a learned bias by
distance, values of their own width that a layer may mix with another layer's, and a gate on every head's
output; optionally a rotation of part of every head before the norms, keys that double as values, a query
temperature by position, a penalty linear in the distance, a window, and a sink in the softmax."""

from __future__ import annotations

import math

import numpy as np
import torch

from .. import ops
from ..ops.profile import span
from .base import KVCacheSpec, Mixer, build_position, register_mixer


def log_bucket(n: int, rows: int, far: float) -> int:
    """The table row of a key n positions back (see `parts.spec.DistanceBiasSpec`)."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def bias_by_distance(table: torch.Tensor, far: float) -> torch.Tensor:
    """float32 [n_dist, heads]: the bias of a key n positions back, for every n up to the first distance
    from which all share the table's last row (the kernels clamp larger distances to the last entry)."""
    rows = table.shape[0]
    if rows < 2 or not far > rows // 2:
        raise ValueError(f"a distance-bias table of {rows} rows does not reach up to distance {far}")
    buckets, n = [], 0
    while True:
        b = log_bucket(n, rows, far)
        buckets.append(b)
        if b == rows - 1 and n >= far:
            break
        n += 1
    return table.float()[torch.tensor(buckets, dtype=torch.long, device=table.device)].contiguous()


class BiasedAttention(Mixer):
    """One stacked product makes q | k | v | gate logits; one kernel norms q and k per head, mixes the
    values where the layer does and stores keys and values in the paged cache; attention adds the bias by
    distance to every score and applies the gate to every head's result; then the output projection.

    The layer with `value_source` leaves its values (a view of its projection's rows) in `step.carry`
    for the layers that mix them in: they concern the same tokens of the same step, so nothing has to be
    kept between steps.  Norms, scores, softmax, value sums, mixing and gate are float32."""

    graph_safe = True

    CARRY_KEY = "biased_attention.values"

    def __init__(self, spec, dtype, device):
        self.spec = spec
        self.dtype = dtype
        if spec.n_heads % spec.n_kv_heads:
            raise ValueError(f"{spec.n_heads} query heads are not a multiple of {spec.n_kv_heads} key/value heads")
        if spec.dim > 256 or spec.v_dim > 256:
            raise ValueError(f"attention kernels take head sizes up to 256, got {spec.dim} / {spec.v_dim}")
        self.eps = float(np.float32(spec.eps))
        self.scale = float(spec.scale)
        self.window = int(spec.window) if spec.window else 0
        self.q_off = 0
        self.k_off = spec.n_heads * spec.dim
        self.v_off = self.k_off + spec.n_kv_heads * spec.dim
        self.g_off = self.v_off + spec.n_kv_heads * spec.v_dim
        if spec.v_proj is None:
            # the values are the keys as projected: the same columns, read before rotation and norm
            if spec.v_dim != spec.dim or spec.value_mix is not None or spec.value_source:
                raise ValueError("keys that double as values have the keys' width and are not mixed with another layer's")
            self.v_off = self.k_off
            self.g_off = self.k_off + spec.n_kv_heads * spec.dim
        self.lam = 0.0
        self.bias = self.q_w = self.k_w = self.sinks = self.slopes = None
        self.rotation = None
        self.rot_half = False
        if spec.rotation is not None:
            pos = build_position(spec.rotation, dtype, device)
            if getattr(pos, "pairing", None) not in ("adjacent", "half") or not hasattr(pos, "rotation"):
                raise ValueError("this mixer rotates entry 2i with entry 2i + 1 or entry i with entry i + dims / 2 "
                                 "(a rotary spec with pairing 'adjacent' or 'half')")
            self.rotation = pos.rotation()
            self.rot_half = pos.pairing == "half"
            if self.rotation[1] > spec.dim:
                raise ValueError(f"the rotation covers {self.rotation[1]} entries, a head has {spec.dim}")
        if spec.unit_norm and (spec.q_norm is not None or spec.k_norm is not None):
            raise ValueError("queries and keys are normed with a weight or without, not both")
        self.q_temp = None
        if spec.q_temp is not None:
            coef, every = float(spec.q_temp[0]), int(spec.q_temp[1])
            if every <= 0:
                raise ValueError(f"the query temperature steps every {every} positions")
            self.q_temp = (coef, every)
        if spec.slopes is not None:
            if len(spec.slopes) != spec.n_heads:
                raise ValueError(f"{len(spec.slopes)} slopes for {spec.n_heads} heads")
            self.slopes = torch.tensor([float(v) for v in spec.slopes], dtype=torch.float64).to(torch.float32).to(device)
        if spec.unit_norm:
            self.q_w = self.k_w = torch.ones((spec.dim,), dtype=torch.float32, device=device)
        if spec.out_gate is not None and spec.head_gate is not None:
            raise ValueError("a head's output is gated as a whole or channel by channel, not both")
        self.gate_cols = spec.n_heads * spec.v_dim if spec.out_gate is not None else spec.n_heads
        self.proj_bias = None

    def tensors(self) -> dict:
        s = self.spec
        out = {s.q_proj: (s.n_heads * s.dim, s.hidden), s.k_proj: (s.n_kv_heads * s.dim, s.hidden),
               s.o_proj: (s.hidden, s.n_heads * s.v_dim)}
        if s.v_proj is not None:
            out[s.v_proj] = (s.n_kv_heads * s.v_dim, s.hidden)
        if s.sink is not None:
            out[s.sink] = (s.n_heads,)
        if s.q_norm is not None:
            out[s.q_norm] = (s.dim,)
        if s.k_norm is not None:
            out[s.k_norm] = (s.dim,)
        if s.bias is not None:
            out[s.bias.table] = (s.bias.rows, s.n_heads)
        if s.head_gate is not None:
            out[s.head_gate] = (s.n_heads, s.hidden)
        if s.out_gate is not None:
            out[s.out_gate] = (s.n_heads * s.v_dim, s.hidden)
        for name, rows in ((s.q_bias, s.n_heads * s.dim), (s.k_bias, s.n_kv_heads * s.dim), (s.v_bias, s.n_kv_heads * s.v_dim)):
            if name is not None:
                out[name] = (rows,)
        if s.value_mix is not None:
            out[s.value_mix] = ()
        return out

    def load(self, src) -> None:
        s = self.spec
        parts = [src.get(s.q_proj), src.get(s.k_proj)] + ([src.get(s.v_proj)] if s.v_proj is not None else [])
        if s.head_gate is not None:
            parts.append(src.get(s.head_gate))
        if s.out_gate is not None:
            parts.append(src.get(s.out_gate))
        w = torch.cat(parts, dim=0)
        pad = -w.shape[0] % 8             # rows of the stacked projection stay 16-byte multiples
        if pad:
            w = torch.cat([w, w.new_zeros((pad, w.shape[1]))], dim=0)
        self.w_in = w.contiguous()
        self.w_o = src.get(s.o_proj).contiguous()
        if s.q_bias is not None or s.k_bias is not None or s.v_bias is not None:
            if s.v_proj is None and s.v_bias is not None:
                raise ValueError("keys that double as values have no value bias")
            # one float32 entry a column of the stacked projection's row; the kernel that reads q, k and v adds it
            bias = torch.zeros((self.w_in.shape[0],), dtype=torch.float32, device=self.w_in.device)
            for name, off in ((s.q_bias, self.q_off), (s.k_bias, self.k_off), (s.v_bias, self.v_off)):
                if name is not None:
                    b = src.get(name, "vector")
                    bias[off:off + b.shape[0]] = b
            self.proj_bias = bias.contiguous()
        if not s.unit_norm:
            self.q_w = src.get(s.q_norm, "vector").contiguous() if s.q_norm is not None else None
            self.k_w = src.get(s.k_norm, "vector").contiguous() if s.k_norm is not None else None
        if s.sink is not None:
            self.sinks = src.get(s.sink, "vector").contiguous()
        if s.bias is not None:
            self.bias = bias_by_distance(src.get(s.bias.table, "vector"), float(s.bias.far))
        if s.value_mix is not None:
            self.lam = float(src.get(s.value_mix, "vector").reshape(-1)[0].item())

    def cache_spec(self):
        s = self.spec
        return KVCacheSpec(s.n_kv_heads, s.dim, s.window, v_head_dim=s.v_dim if s.v_dim != s.dim else None)

    def _fast(self) -> bool:
        s = self.spec
        return ops.biased_attention_takes_mma(self.dtype, s.n_heads, s.n_kv_heads, s.dim, s.v_dim)

    @property
    def prefill_tile(self):
        return ops.prefill_tile() if self._fast() else None

    def launch_variant(self, step):
        if not step.n_decode or not self._fast():
            return None
        s = self.spec
        return ops.biased_decode_pieces(step.n_decode, s.n_kv_heads, step.max_decode_ctx)

    def forward(self, x, step, cache, state, writes_cache=True):
        s = self.spec
        T = x.shape[0]
        with span("q|k|v|gate proj"):
            proj = ops.linear(x, self.w_in)
        other = None
        if s.value_source:
            step.carry[self.CARRY_KEY] = proj[:, self.v_off:self.v_off + s.n_kv_heads * s.v_dim]
        elif s.value_mix is not None:
            other = step.carry.get(self.CARRY_KEY)
            if other is None:
                raise RuntimeError("a layer mixes in another layer's values, and no layer of this step has left any")
        q = step.buffer("attn_q", (T, s.n_heads * s.dim), self.dtype)
        with span("q, k norms + value mix + kv write"):
            ops.qk_norm_store(proj, self.q_off, self.k_off, self.v_off, self.q_w, self.k_w, self.eps, other, self.lam, q,
                              cache.k, cache.v, step.slots[cache.group] if writes_cache else None, s.n_heads,
                              s.n_kv_heads, s.dim, s.v_dim, cache.page_size, rotation=self.rotation,
                              positions=step.positions, q_temp=self.q_temp, rot_half=self.rot_half,
                              proj_bias=self.proj_bias)
        o = step.buffer("attn_o", (T, s.n_heads * s.v_dim), self.dtype)
        gate = proj[:, self.g_off:self.g_off + self.gate_cols] if (s.head_gate is not None or s.out_gate is not None) else None
        with span("attention"):
            ops.attention_biased(q, cache.k, cache.v, o, self.bias, gate, step, cache.group, s.n_heads, s.n_kv_heads,
                                 s.dim, s.v_dim, cache.page_size, self.scale, self.window, sinks=self.sinks,
                                 slopes=self.slopes)
        with span("o proj"):
            return ops.linear(o, self.w_o)


register_mixer("biased_attention", BiasedAttention)
