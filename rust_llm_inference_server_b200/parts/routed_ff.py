"""A feed-forward that routes every token to a few of many small gated feed-forwards, beside an optional
shared one that every token runs through."""

from __future__ import annotations

import torch

from .. import ops
from ..ops.profile import span
from .base import FeedForward, build_feed_forward, register_feed_forward


class RoutedFF(FeedForward):
    """Router scores in float32 from float32 copies of the router matrix (and of the shared expert's
    gate row, which rides along as one more row); choice, weights and the sort of (token, choice) pairs
    by expert happen on the device, so launches depend on the step's shape only.  The experts' matrices
    are stacked at load time: both branches of the first product in one stack [expert, 2 I, in], the second
    product's [expert, out, I].  Steps with many pairs an expert (portions of prompts) take the grouped
    tcgen05 products, steps with few (decode) the mma.sync ones, float32 the FFMA ones (`ops.moe_up`)."""

    graph_safe = True

    def __init__(self, spec, dtype, device):
        self.spec = spec
        self.dtype = dtype
        self.limit = float("inf") if spec.limit is None else float(spec.limit)
        self.shared = build_feed_forward(spec.shared, dtype, device) if spec.shared is not None else None
        if spec.shared_gate is not None and self.shared is None:
            raise ValueError("a gate on the shared expert, and no shared expert")
        if spec.scoring not in ("sigmoid", "softmax_chosen", "softmax"):
            raise ValueError(f"experts are scored by 'sigmoid', 'softmax_chosen' or 'softmax', got {spec.scoring!r}")
        self.n_identity = int(getattr(spec, "n_identity", 0) or 0)
        self.groups = tuple(int(g) for g in spec.groups) if getattr(spec, "groups", None) is not None else None
        n_out = spec.n_experts + self.n_identity
        if self.groups is not None:
            count, keep = self.groups
            if count < 1 or n_out % count or not 1 <= keep <= count or spec.top > keep * (n_out // count):
                raise ValueError(f"{n_out} router outputs do not form {count} equal groups of which {keep} hold {spec.top} choices")
        if self.n_identity and spec.shared_gate is not None:
            raise ValueError("the gate of a shared expert rides on the router's last row, where identity experts sit")
        self.router_bias = None

    def _names(self, pattern: str):
        return [pattern.format(e=e) for e in range(self.spec.n_experts)]

    def tensors(self) -> dict:
        s = self.spec
        n_out = s.n_experts + self.n_identity
        out = {s.router: (n_out, s.hidden)}
        if s.correction is not None:
            out[s.correction] = (n_out,)
        if s.router_bias is not None:
            out[s.router_bias] = (n_out,)
        for n in self._names(s.gate_proj) + self._names(s.up_proj):
            out[n] = (s.intermediate, s.hidden)
        for n in self._names(s.down_proj):
            out[n] = (s.hidden, s.intermediate)
        if self.shared is not None:
            out.update(self.shared.tensors())
        if s.shared_gate is not None:
            out[s.shared_gate] = (1, s.hidden)
        return out

    def load(self, src) -> None:
        s = self.spec
        rows = [src.get(s.router, "vector")]
        if s.shared_gate is not None:
            rows.append(src.get(s.shared_gate, "vector"))
        self.w_router = torch.cat(rows, dim=0).contiguous()              # float32 [experts (+ 1), hidden]
        self.correction = src.get(s.correction, "vector").contiguous() if s.correction is not None else None
        self.router_bias = src.get(s.router_bias, "vector").contiguous() if s.router_bias is not None else None
        # one stack [expert, 2 I, in] of both branches: gate and linear rows interleaved in blocks of 4 (what
        # the gated epilogue of the grouped product over prompts wants) where I allows, else gate rows first
        I, W = s.intermediate, s.hidden
        self.interleave = 4 if I % 4 == 0 else 0
        per_expert = []
        for gn, un in zip(self._names(s.gate_proj), self._names(s.up_proj)):
            g, u = src.get(gn), src.get(un)
            if self.interleave:
                per_expert.append(torch.stack([g.view(-1, 4, W), u.view(-1, 4, W)], dim=1).reshape(2 * I, W))
            else:
                per_expert.append(torch.cat([g, u], dim=0))
        self.w_gate_up = torch.stack(per_expert).contiguous()
        self.w_down = torch.stack([src.get(n) for n in self._names(s.down_proj)]).contiguous()
        if self.shared is not None:
            self.shared.load(src)

    def forward(self, x, step):
        s = self.spec
        T = x.shape[0]
        with span("router"):
            plan = ops.moe_route(x, self.w_router, self.correction, s.n_experts, s.top, s.route_scale,
                                 s.shared_gate is not None, step, router_bias=self.router_bias, scoring=s.scoring,
                                 groups=self.groups, normalize=bool(getattr(s, "normalize", False)),
                                 n_identity=self.n_identity)
        y_shared = self.shared.forward(x, step) if self.shared is not None else None
        with span("experts"):
            act = ops.moe_up(x, self.w_gate_up, plan, s.slope, self.limit, s.up_shift, step, self.interleave)
            y = ops.moe_down(act, self.w_down, plan, step)
        out = step.buffer("ffn_out", (T, s.hidden), self.dtype)
        with span("combine"):
            return ops.moe_combine(y, plan, y_shared, out, x=x)


register_feed_forward("routed_ff", RoutedFF)
