"""Several mixers side by side on the same input."""

from __future__ import annotations

import numpy as np

from .. import ops
from ..ops.profile import span
from .base import Mixer, Part, build_mixer, register_mixer


class ParallelMixer(Mixer):
    """Every branch reads the mixer's input; the result is the mean of the branches' outputs, each first
    RMS-normed over the model width with a weight of its own (or, as the spec says, their weighted sum as they are).  A call of the run order has one cache slot and
    one state, so at most one branch keeps a paged cache and at most one a state; they get the call's.

    An arrangement that can take the sum into a kernel of its own asks `forward_branches` for the outputs with
    their weights and coefficients instead of `forward`."""

    def __init__(self, spec, dtype, device):
        self.spec = spec
        self.dtype = dtype
        if not spec.branches or (spec.out_norms is not None and len(spec.branches) != len(spec.out_norms)):
            raise ValueError("a parallel mixer takes one output norm a branch")
        coefficients = getattr(spec, "coefficients", None)
        if coefficients is not None and len(coefficients) != len(spec.branches):
            raise ValueError("a parallel mixer takes one coefficient a branch")
        self.coefficients = [float(c) for c in coefficients] if coefficients is not None \
            else [1.0 / len(spec.branches)] * len(spec.branches)
        self.branches = [build_mixer(b, dtype, device) for b in spec.branches]
        if sum(b.cache_spec() is not None for b in self.branches) > 1:
            raise ValueError("at most one branch of a parallel mixer keeps a paged cache")
        if sum(b.state_spec() is not None for b in self.branches) > 1:
            raise ValueError("at most one branch of a parallel mixer keeps a per-request state")
        self.eps = float(np.float32(spec.eps))
        self.out_w = None
        self.graph_safe = all(getattr(b, "graph_safe", False) for b in self.branches)

    def tensors(self) -> dict:
        out = {n: (self.spec.hidden,) for n in (self.spec.out_norms or ())}
        for b in self.branches:
            out.update(b.tensors())
        return out

    def load(self, src) -> None:
        self.out_w = [src.get(n, "vector").contiguous() for n in self.spec.out_norms] \
            if self.spec.out_norms is not None else [None] * len(self.branches)
        for b in self.branches:
            b.load(src)

    def cache_spec(self):
        return next((cs for cs in (b.cache_spec() for b in self.branches) if cs is not None), None)

    def state_spec(self):
        return next((ss for ss in (b.state_spec() for b in self.branches) if ss is not None), None)

    @property
    def prefill_tile(self):
        tiles = {b.prefill_tile for b in self.branches if getattr(b, "prefill_tile", None)}
        if len(tiles) > 1:
            raise ValueError(f"the branches ask for prompt tiles of different sizes: {sorted(tiles)}")
        return tiles.pop() if tiles else None

    def launch_variant(self, step):
        return tuple(b.launch_variant(step) if getattr(type(b), "launch_variant", Part.launch_variant)
                     is not Part.launch_variant else None for b in self.branches)

    def forward_branches(self, x, step, cache, state, writes_cache=True):
        """([(output, norm weight, coefficient), ...], eps of the norms): the terms of the result."""
        outs = []
        for b, w, c in zip(self.branches, self.out_w, self.coefficients):
            y = b.forward(x, step, cache if b.cache_spec() is not None else None,
                          state if b.state_spec() is not None else None, writes_cache)
            outs.append((y, w, c))
        return outs, self.eps

    def forward(self, x, step, cache, state, writes_cache=True):
        terms, eps = self.forward_branches(x, step, cache, state, writes_cache)
        out = step.buffer("parallel_out", (x.shape[0], self.spec.hidden), self.dtype)
        with span("branch norms + mean"):
            ops.sum_norm(None, 0.0, terms[:2], None, 0.0, out=out, eps_branch=eps)
            for term in terms[2:]:                  # two branches a launch; more are added one by one
                ops.sum_norm(None, 0.0, [term, (out, None, 1.0)], None, 0.0, out=out, eps_branch=eps)
        return out


register_mixer("parallel", ParallelMixer)
