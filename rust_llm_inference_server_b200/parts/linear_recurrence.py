"""Linear-attention recurrences over a float32 state per request: retention (a fixed decay a head, rotated
queries and keys) and the recurrence with a gate a channel whose complement is the key (a decay a token and channel)."""

from __future__ import annotations

import numpy as np
import torch

from .. import ops
from ..ops.profile import span
from .base import Mixer, StateSpec, build_position, register_mixer


class _Recurrence(Mixer):
    """What both share: one stacked projection, a kernel that makes the recurrence's float32 inputs [q | k | v (| a)]
    of every token, the walk S <- diag(a) S + k v^T, o = S^T q from the request's state slot (S is kept
    transposed), a norm a head, and the output projection.  Everything between the two projections is float32."""

    graph_safe = True

    def state_spec(self):
        s = self.spec
        return StateSpec((s.n_heads, s.v_dim, s.dim), torch.float32)     # S transposed: a column's entries are contiguous

    def fuses_norms(self, step) -> bool:
        # in steps of a few rows the first product scales the rows of the norm before it and the last one adds to the
        # stream itself (both are the streaming product)
        s = self.spec
        return ops.fuses_norms(step.n_tokens, self.dtype, s.hidden, s.n_heads * s.v_dim)

    def _walk(self, proj, step, state, decay, complement_key=False, **inputs):
        s = self.spec
        T, H = proj.shape[0], s.n_heads
        qk, hv = H * s.dim, H * s.v_dim
        if T < ops.RECURRENCE_INPUT_PASS_TOKENS:
            # short steps: the walk makes its inputs while it stages the tokens (one kernel)
            o = step.buffer("recurrence_o", (T, hv), torch.float32)
            with span("recurrence"):
                return ops.recurrence_scan_rows(proj, self.q_off, self.k_off, self.v_off, o, state, decay, step, H, s.dim,
                                                s.v_dim, rotation=inputs.get("rotation"), k_scale=inputs.get("k_scale", 1.0),
                                                lower=inputs.get("lower"), gate_bias=inputs.get("gate_bias"))
        rows = step.buffer("recurrence_in", (T, 2 * qk + hv + (qk if decay is None else 0)), torch.float32)
        with span("recurrence inputs"):
            ops.recurrence_inputs(proj, self.q_off, self.k_off, self.v_off, rows, H, s.dim, s.v_dim, **inputs)
        o = step.buffer("recurrence_o", (T, hv), torch.float32)
        with span("recurrence"):
            return ops.recurrence_scan(rows, o, state, decay, step, H, s.dim, s.v_dim, complement_key=complement_key)


class Retention(_Recurrence):
    """q | k | v | gate come from one stacked projection; q and k are rotated by position in float32 and k is scaled;
    S <- decay_h S + k v^T, o = S^T q; each head's o is divided by its root mean square, gated and projected."""

    def __init__(self, spec, dtype, device):
        self.spec = spec
        self.dtype = dtype
        if len(spec.decay) != spec.n_heads:
            raise ValueError(f"{len(spec.decay)} decay factors for {spec.n_heads} heads")
        if spec.gate_act not in ops.GATE_ACTIVATIONS:
            raise ValueError(f"unknown gate activation {spec.gate_act!r}; known: {sorted(ops.GATE_ACTIVATIONS)}")
        self.eps = float(np.float32(spec.eps))
        self.decay = torch.tensor([float(g) for g in spec.decay], dtype=torch.float64).to(torch.float32).to(device)
        self.k_scale = float(spec.dim) ** -0.5 if spec.k_scale is None else float(spec.k_scale)
        self.rotation = None
        if spec.rotation is not None:
            pos = build_position(spec.rotation, dtype, device)
            if getattr(pos, "pairing", "half") != "half" or not hasattr(pos, "rotation"):
                raise ValueError("this mixer rotates entry i with entry i + dims / 2 (a rotate-half spec)")
            inv_freq, dims, magnitude = pos.rotation()
            if dims > spec.dim or magnitude != 1.0:
                raise ValueError(f"the rotation covers {dims} entries (a head has {spec.dim}) with magnitude {magnitude}")
            self.rotation = (inv_freq, dims)
        qk = spec.n_heads * spec.dim
        self.q_off, self.k_off, self.v_off, self.g_off = 0, qk, 2 * qk, 2 * qk + spec.n_heads * spec.v_dim
        self.out_norm = None

    def tensors(self) -> dict:
        s = self.spec
        out = {s.q_proj: (s.n_heads * s.dim, s.hidden), s.k_proj: (s.n_heads * s.dim, s.hidden),
               s.v_proj: (s.n_heads * s.v_dim, s.hidden), s.o_proj: (s.hidden, s.n_heads * s.v_dim)}
        if s.gate_proj is not None:
            out[s.gate_proj] = (s.n_heads * s.v_dim, s.hidden)
        if s.out_norm is not None:
            out[s.out_norm] = (s.v_dim,)
        return out

    def load(self, src) -> None:
        s = self.spec
        parts = [src.get(s.q_proj), src.get(s.k_proj), src.get(s.v_proj)]
        if s.gate_proj is not None:
            parts.append(src.get(s.gate_proj))
        w = torch.cat(parts, dim=0)
        pad = -w.shape[0] % 8             # rows of the stacked projection stay 16-byte multiples
        if pad:
            w = torch.cat([w, w.new_zeros((pad, w.shape[1]))], dim=0)
        self.w_in = w.contiguous()
        self.out_norm = src.get(s.out_norm, "vector").contiguous() if s.out_norm is not None else None
        self.w_o = src.get(s.o_proj).contiguous()

    def forward(self, x, step, cache, state, writes_cache=True, sink=None):
        s = self.spec
        T, hv = x.shape[0], s.n_heads * s.v_dim
        with span("q|k|v|gate proj"):
            proj = ops.linear(x, self.w_in)
        o = self._walk(proj, step, state, self.decay, rotation=self.rotation, positions=step.positions,
                       k_scale=self.k_scale)
        y = step.buffer("recurrence_y", (T, hv), self.dtype)
        with span("head norm * gate"):
            ops.head_norm_gate(o, self.out_norm, self.eps, y, s.n_heads,
                               gate=proj[:, self.g_off:self.g_off + hv] if s.gate_proj is not None else None,
                               activation=s.gate_act)
        with span("o proj"):
            return ops.linear(y, self.w_o, sink=sink)


class ForgetGateRecurrence(_Recurrence):
    """q | f | v come from one stacked projection; q = silu(q), the forget gate a = l + (1 - l) sigmoid(f + b) per head
    and channel and the key 1 - a are made in float32; S <- diag(a) S + (1 - a) v^T, o = S^T q; each head's o is
    RMS-normed with one weight shared by the heads and projected."""

    def __init__(self, spec, dtype, device):
        self.spec = spec
        self.dtype = dtype
        self.eps = float(np.float32(spec.eps))
        qk = spec.n_heads * spec.dim
        self.q_off, self.k_off, self.v_off = 0, qk, 2 * qk
        self.lower = self.f_bias = self.out_norm = None

    def tensors(self) -> dict:
        s = self.spec
        qk = s.n_heads * s.dim
        out = {s.q_proj: (qk, s.hidden), s.f_proj: (qk, s.hidden), s.lower: (qk,),
               s.v_proj: (s.n_heads * s.v_dim, s.hidden), s.o_proj: (s.hidden, s.n_heads * s.v_dim)}
        if s.f_bias is not None:
            out[s.f_bias] = (qk,)
        if s.out_norm is not None:
            out[s.out_norm] = (s.v_dim,)
        return out

    def load(self, src) -> None:
        s = self.spec
        w = torch.cat([src.get(s.q_proj), src.get(s.f_proj), src.get(s.v_proj)], dim=0)
        pad = -w.shape[0] % 8             # rows of the stacked projection stay 16-byte multiples
        if pad:
            w = torch.cat([w, w.new_zeros((pad, w.shape[1]))], dim=0)
        self.w_in = w.contiguous()
        self.lower = src.get(s.lower, "vector").contiguous()
        self.f_bias = src.get(s.f_bias, "vector").contiguous() if s.f_bias is not None else None
        self.out_norm = src.get(s.out_norm, "vector").contiguous() if s.out_norm is not None else None
        self.w_o = src.get(s.o_proj).contiguous()

    def forward(self, x, step, cache, state, writes_cache=True, sink=None):
        s = self.spec
        T, hv = x.shape[0], s.n_heads * s.v_dim
        with span("q|f|v proj"):
            proj = ops.linear(x, self.w_in)
        o = self._walk(proj, step, state, None, complement_key=True, q_silu=True, lower=self.lower, gate_bias=self.f_bias)
        y = step.buffer("recurrence_y", (T, hv), self.dtype)
        with span("head norm"):
            ops.head_norm_gate(o, self.out_norm, self.eps, y, s.n_heads)
        with span("o proj"):
            return ops.linear(y, self.w_o, sink=sink)


register_mixer("retention", Retention)
register_mixer("forget_gate_recurrence", ForgetGateRecurrence)
