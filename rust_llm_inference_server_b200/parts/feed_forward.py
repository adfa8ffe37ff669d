"""Dense SwiGLU feed-forward (crates/model/src/layers.rs:156-187): down(silu(gate x) * up x)."""

from __future__ import annotations

import torch

from .. import ops
from ..ops.profile import span
from .base import FeedForward, register_feed_forward


class SwiGLU(FeedForward):
    """gate and up are stacked into one (2I, hidden) matrix at load time, rows interleaved in
    blocks of 4 (4 gate rows, their 4 up rows, ...), so one product feeds the gating and the
    decode kernel can gate in its epilogue; a pure change of layout."""

    graph_safe = True    # launches depend on the step's device arrays and shapes only

    def __init__(self, spec, dtype, device):
        self.spec = spec
        self.dtype = dtype
        self.w_gate_up = None
        self.w_down = None
        # the form g sigmoid(slope g) * u has kernels that gate inside a product (silu at slope 1, relu at an infinite
        # one); a clipping limit or a shifted linear branch go through the gating kernel that takes them as parameters
        self.slope = float(getattr(spec, "slope", 1.0))
        self.plain = getattr(spec, "limit", None) is None and float(getattr(spec, "up_shift", 0.0)) == 0.0

    def tensors(self) -> dict:
        s = self.spec
        return {s.gate_proj: (s.intermediate, s.hidden), s.up_proj: (s.intermediate, s.hidden),
                s.down_proj: (s.hidden, s.intermediate)}

    def load(self, src) -> None:
        s = self.spec
        g, u = src.get(s.gate_proj), src.get(s.up_proj)
        self.interleave = 4 if s.intermediate % 4 == 0 else 0
        if self.interleave:
            self.w_gate_up = torch.stack([g.view(-1, 4, s.hidden), u.view(-1, 4, s.hidden)], dim=1) \
                .reshape(2 * s.intermediate, s.hidden).contiguous()
        else:
            self.w_gate_up = torch.cat([g, u], dim=0).contiguous()
        self.w_down = src.get(s.down_proj).contiguous()

    def fuses_norms(self, step) -> bool:
        return self.plain and ops.fuses_norms(step.n_tokens, self.dtype, self.spec.hidden, self.spec.intermediate)

    def forward(self, x, step, sink=None):
        if not self.plain:
            s = self.spec
            if (self.dtype == torch.bfloat16 and self.interleave == 4 and s.hidden % 8 == 0 and x.shape[0] >= 128
                    and s.intermediate % 128 == 0):
                # prefill: the tcgen05 product with the clipped gating in its epilogue
                with span("mlp gate+up, clipped gating"):
                    act = ops.gemm_tcgen05(x, self.w_gate_up, "glu4", glu=(s.slope, s.limit, s.up_shift))
            else:
                with span("mlp gate+up"):
                    gu = ops.linear(x, self.w_gate_up)
                with span("clipped gating"):
                    act = step.buffer("ffn_act", (x.shape[0], s.intermediate), self.dtype)
                    ops.glu_act(gu, act, s.slope, s.limit, s.up_shift, self.interleave)
            with span("mlp down proj"):
                return ops.linear(act, self.w_down)
        fusable = self.dtype == torch.bfloat16 and self.interleave == 4 and self.spec.hidden % 8 == 0
        silu = self.slope == 1.0
        with span("mlp gate+up, silu*up" if silu else "mlp gate+up, gate*up"):
            if fusable and x.shape[0] <= ops.STREAM_GEMM_ROWS:
                act = ops.stream_gemm(x, self.w_gate_up, swiglu4=True, slope=self.slope)   # product and gating in one kernel
            elif fusable and x.shape[0] >= 128 and self.spec.intermediate % 128 == 0:
                # prefill: the tcgen05 product with the gating in its epilogue (the gate|up activations
                # never reach HBM)
                act = ops.gemm_tcgen05(x, self.w_gate_up, "swiglu4") if silu \
                    else ops.gemm_tcgen05(x, self.w_gate_up, "glu4", glu=(self.slope, None, 0.0))
            else:
                gu = ops.linear(x, self.w_gate_up)
                act = step.buffer("ffn_act", (x.shape[0], self.spec.intermediate), self.dtype)
                if silu:
                    ops.swiglu(gu, act, self.interleave)
                else:
                    ops.glu_act(gu, act, self.slope, None, 0.0, self.interleave)
        with span("mlp down proj"):
            return ops.linear(act, self.w_down, sink=sink)


class DenseFF(FeedForward):
    """W_down act(W_up x + b_up) + b_down.  The bias and the activation after the first product are
    one kernel; the second bias is returned as `pending_bias` for an arrangement that norms the
    result (it adds the bias while it reads the row), and added here otherwise."""

    graph_safe = True

    def __init__(self, spec, dtype, device):
        self.spec = spec
        self.dtype = dtype
        if spec.activation not in ops.BIAS_ACTIVATIONS:
            raise ValueError(f"unknown activation {spec.activation!r}; known: {sorted(ops.BIAS_ACTIVATIONS)}")

    def tensors(self) -> dict:
        s = self.spec
        out = {s.up_proj: (s.intermediate, s.hidden), s.down_proj: (s.hidden, s.intermediate)}
        if s.up_bias is not None:
            out[s.up_bias] = (s.intermediate,)
        if s.down_bias is not None:
            out[s.down_bias] = (s.hidden,)
        return out

    def load(self, src) -> None:
        s = self.spec
        self.w_up = src.get(s.up_proj).contiguous()
        self.w_down = src.get(s.down_proj).contiguous()
        self.b_up = src.get(s.up_bias, "vector") if s.up_bias is not None else None
        self.b_down = src.get(s.down_bias, "vector") if s.down_bias is not None else None

    def forward(self, x, step, defer_bias: bool = False):
        """With `defer_bias` the caller adds `self.b_down` itself (in float32, while norming)."""
        with span("mlp up proj"):
            u = ops.linear(x, self.w_up)
        with span("bias + activation"):
            act = ops.bias_act(u, self.b_up, step.buffer("ffn_act", tuple(u.shape), self.dtype), self.spec.activation)
        with span("mlp down proj"):
            y = ops.linear(act, self.w_down)
        if self.b_down is not None and not defer_bias:
            y = ops.bias_act(y, self.b_down, step.buffer("ffn_out", tuple(y.shape), self.dtype), "none")
        return y


register_feed_forward("swiglu", SwiGLU)
register_feed_forward("dense_ff", DenseFF)
