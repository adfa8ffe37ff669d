"""The gated delta rule: a linear recurrence over a float32 state per request whose update corrects the
state towards the token's value along its key, behind short causal convolutions of q, k and v."""

from __future__ import annotations

import numpy as np
import torch

from .. import ops
from ..ops.profile import span
from .base import Mixer, StateSpec, register_mixer


class GatedDeltaRule(Mixer):
    """q | k | v | gate | beta logits | decay logits come from one stacked projection.  One kernel applies the
    convolutions (their tail of taps - 1 inputs is part of the request's state), silu, the unit norms of q and k,
    the sigmoid of beta and the decay g = exp(-exp(a_log) softplus(. + dt_bias)); a second one walks the step's
    tokens per (request, head): S <- g S, u = beta (v - S^T k), S <- S + k u^T, o = S^T q.  The heads' outputs are
    normed per head, gated by silu(W_g h) and projected.  Everything between the two projections is float32."""

    graph_safe = True

    def __init__(self, spec, dtype, device):
        self.spec = spec
        self.dtype = dtype
        if spec.n_heads % spec.n_qk_heads:
            raise ValueError(f"{spec.n_heads} heads are not a multiple of {spec.n_qk_heads} query/key heads")
        if spec.conv < 1:
            raise ValueError(f"a convolution has at least one tap, got {spec.conv}")
        self.eps = float(np.float32(spec.eps))
        qk, hv = spec.n_qk_heads * spec.dim, spec.n_heads * spec.v_dim
        self.channels = 2 * qk + hv
        self.g_off = self.channels
        self.b_off = self.g_off + hv
        self.a_off = self.b_off + spec.n_heads
        self.state_floats = ops.gated_delta_state_floats(spec.n_heads, spec.n_qk_heads, spec.dim, spec.v_dim, spec.conv)

    def tensors(self) -> dict:
        s = self.spec
        qk, hv = s.n_qk_heads * s.dim, s.n_heads * s.v_dim
        return {s.q_proj: (qk, s.hidden), s.k_proj: (qk, s.hidden), s.v_proj: (hv, s.hidden),
                s.q_conv: (qk, s.conv), s.k_conv: (qk, s.conv), s.v_conv: (hv, s.conv),
                s.beta_proj: (s.n_heads, s.hidden), s.decay_proj: (s.n_heads, s.hidden), s.a_log: (s.n_heads,),
                s.dt_bias: (s.n_heads,), s.gate_proj: (hv, s.hidden), s.out_norm: (s.v_dim,),
                s.o_proj: (s.hidden, hv)}

    def load(self, src) -> None:
        s = self.spec
        w = torch.cat([src.get(s.q_proj), src.get(s.k_proj), src.get(s.v_proj), src.get(s.gate_proj),
                       src.get(s.beta_proj), src.get(s.decay_proj)], dim=0)
        pad = -w.shape[0] % 8             # rows of the stacked projection stay 16-byte multiples
        if pad:
            w = torch.cat([w, w.new_zeros((pad, w.shape[1]))], dim=0)
        self.w_in = w.contiguous()
        self.conv_w = torch.cat([src.get(s.q_conv, "vector"), src.get(s.k_conv, "vector"),
                                 src.get(s.v_conv, "vector")], dim=0).contiguous()
        self.a_log = src.get(s.a_log, "vector").contiguous()
        self.dt_bias = src.get(s.dt_bias, "vector").contiguous()
        self.out_norm = src.get(s.out_norm, "vector").contiguous()
        self.w_o = src.get(s.o_proj).contiguous()

    def state_spec(self):
        return StateSpec((self.state_floats,), torch.float32)

    def forward(self, x, step, cache, state, writes_cache=True):
        s = self.spec
        T, hv = x.shape[0], s.n_heads * s.v_dim
        with span("q|k|v|gate|beta|decay proj"):
            proj = ops.linear(x, self.w_in)
        o = step.buffer("gated_delta_o", (T, hv), torch.float32)
        with span("conv + delta rule"):
            ops.gated_delta(proj, 0, self.b_off, self.a_off, self.conv_w, self.a_log, self.dt_bias, state, o, step,
                            s.n_heads, s.n_qk_heads, s.dim, s.v_dim, s.conv, s.unit_eps, float(s.dim) ** -0.5)
        y = step.buffer("gated_delta_y", (T, hv), self.dtype)
        with span("head norm * gate"):
            ops.head_norm_gate(o, self.out_norm, self.eps, y, s.n_heads, gate=proj[:, self.g_off:self.g_off + hv],
                               activation="silu")
        with span("o proj"):
            return ops.linear(y, self.w_o)


register_mixer("gated_delta", GatedDeltaRule)
