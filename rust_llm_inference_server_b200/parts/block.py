"""Arrangements of parts into a block.

"prenorm" (crates/model/src/llama.rs:264-271): x += mixer(norm1(x)); x += feed_forward(norm2(x)).
The residual stream is float32; each addition is fused into the norm that follows it, so a block
takes (resid, pending delta) and returns (resid, its own pending delta).

In steps of a few rows a norm is a kernel that moves a few kilobytes.  Where the parts on both
sides of a norm say that they can (`Part.fuses_norms`) and the norm offers it (`Norm.sink`), the
block hands the norm's sink to the part before it, which adds its result to the residual stream in
its last product, and passes the `ops.ScaledRows` it gets back to the part after it, whose first
product applies the scale; "pending" is then such rows instead of a delta.  The same holds across
blocks: the model names the next block, and `entry_sink` answers for its first norm."""

from __future__ import annotations

import torch

from .. import ops
from .base import (Part, build_feed_forward, build_mixer, build_norm, register_arrangement)


class PreNormBlock:
    def __init__(self, spec, dtype, device):
        self.norm1 = build_norm(spec.norm1, dtype, device)
        self.mixer = build_mixer(spec.mixer, dtype, device)
        # a layer may have no feed-forward: its mixer's result is then the block's pending addition
        self.feed_forward = build_feed_forward(spec.feed_forward, dtype, device) if spec.feed_forward is not None else None
        self.norm2 = build_norm(spec.norm2, dtype, device) if self.feed_forward is not None else None

    def parts(self):
        return tuple(p for p in (self.norm1, self.mixer, self.norm2, self.feed_forward) if p is not None)

    chains_norms = True      # `forward` takes `next_block`

    def entry_sink(self, resid, step):
        """For the block that runs before this one: the sink of this block's first norm, if its
        mixer takes the rows that come out of it."""
        return self.norm1.sink(resid, step) if self.mixer.fuses_norms(step) else None

    def forward(self, resid, pending, step, cache, state, writes_cache=True, next_block=None):
        h = pending if isinstance(pending, ops.ScaledRows) else self.norm1.forward(resid, pending, step)
        if self.feed_forward is None:
            sink = next_block.entry_sink(resid, step) if self.mixer.fuses_norms(step) and next_block is not None else None
            if sink is not None:
                return resid, self.mixer.forward(h, step, cache, state, writes_cache, sink=sink)
            return resid, self.mixer.forward(h, step, cache, state, writes_cache)
        mixer_fuses, ff_fuses = self.mixer.fuses_norms(step), self.feed_forward.fuses_norms(step)
        sink = self.norm2.sink(resid, step) if mixer_fuses and ff_fuses else None
        if sink is not None:
            h = self.mixer.forward(h, step, cache, state, writes_cache, sink=sink)
        else:
            a = self.mixer.forward(h, step, cache, state, writes_cache)
            h = self.norm2.forward(resid, a, step)
        sink = next_block.entry_sink(resid, step) if ff_fuses and next_block is not None else None
        if sink is not None:
            return resid, self.feed_forward.forward(h, step, sink=sink)
        return resid, self.feed_forward.forward(h, step)


class SandwichBlock:
    """x += scale1 * post_norm1(mixer(norm1(x))); x += scale2 * post_norm2(feed_forward(norm2(x))),
    the second line only when the layer has a feed-forward.  The residual stream and both norms of
    a sublayer's result are float32: one kernel norms the result, scales it, adds it to the stream
    and norms the stream for the sublayer that follows, also when that is the first sublayer of the
    next block of this kind (the block then returns those rows as `NormedRows`).  A block returns no
    pending delta: its additions are done when it returns."""

    def __init__(self, spec, dtype, device):
        self.dtype = dtype
        self.norm1 = build_norm(spec.norm1, dtype, device)
        self.mixer = build_mixer(spec.mixer, dtype, device)
        self.post_norm1 = build_norm(spec.post_norm1, dtype, device)
        self.scale1_name, self.scale2_name = spec.scale1, spec.scale2
        self.hidden = spec.norm1.dim
        self.feed_forward = build_feed_forward(spec.feed_forward, dtype, device) if spec.feed_forward is not None else None
        self.norm2 = build_norm(spec.norm2, dtype, device) if self.feed_forward is not None else None
        self.post_norm2 = build_norm(spec.post_norm2, dtype, device) if self.feed_forward is not None else None
        self.scale1 = self.scale2 = None
        for n in (self.norm1, self.post_norm1, self.norm2, self.post_norm2):
            if n is not None and not hasattr(n, "weight"):
                raise ValueError("the sandwich arrangement takes norms that are a weight and an eps (RMSNorm)")

    chains_norms = True      # `forward` takes `next_block`

    def entry_sink(self, resid, step):
        return None          # nothing is left to the product before this block

    def parts(self):
        own = _BlockTensors(self)
        return tuple(p for p in (self.norm1, self.mixer, self.post_norm1, self.norm2, self.feed_forward,
                                 self.post_norm2, own) if p is not None)

    def _last(self, sub, resid, post_norm, scale, step, next_block, bias=None):
        """The block's last addition; norms the stream for the next block when that is a sandwich too."""
        if isinstance(next_block, SandwichBlock):
            h = step.buffer("norm_out", (resid.shape[0], self.hidden), self.dtype)
            ops.post_norm_residual(sub, resid, post_norm.weight, post_norm.eps, scale, bias=bias,
                                   w_next=next_block.norm1.weight, eps_next=next_block.norm1.eps, out=h)
            return resid, NormedRows(h)
        ops.post_norm_residual(sub, resid, post_norm.weight, post_norm.eps, scale, bias=bias)
        return resid, None

    def forward(self, resid, pending, step, cache, state, writes_cache=True, next_block=None):
        h = pending.x if isinstance(pending, NormedRows) else self.norm1.forward(resid, pending, step)
        a = self.mixer.forward(h, step, cache, state, writes_cache)
        if self.feed_forward is None:
            return self._last(a, resid, self.post_norm1, self.scale1, step, next_block)
        h = step.buffer("norm_out", (resid.shape[0], self.hidden), self.dtype)
        ops.post_norm_residual(a, resid, self.post_norm1.weight, self.post_norm1.eps, self.scale1,
                               w_next=self.norm2.weight, eps_next=self.norm2.eps, out=h)
        defer = getattr(self.feed_forward, "b_down", None) is not None
        f = self.feed_forward.forward(h, step, defer_bias=True) if defer else self.feed_forward.forward(h, step)
        return self._last(f, resid, self.post_norm2, self.scale2, step, next_block,
                          bias=self.feed_forward.b_down if defer else None)


class OutNormBlock:
    """x += m * norm1(mixer(x)); x += m * norm2(feed_forward(x)), the second line only when the layer has a
    feed-forward.  The sublayers read the stream as it is, and only their results are normed.  The stream
    and the norms are float32: one kernel norms a result, adds it to the stream and leaves the stream,
    rounded to the compute type, for the sublayer that follows (in float32 that sublayer reads the stream
    itself).  A block returns no pending delta, and hands the next block of its kind the rounded stream."""

    def __init__(self, spec, dtype, device):
        self.dtype = dtype
        self.mult = float(spec.residual_mult)
        self.hidden = spec.norm1.dim
        self.mixer = build_mixer(spec.mixer, dtype, device)
        self.norm1 = build_norm(spec.norm1, dtype, device)
        self.feed_forward = build_feed_forward(spec.feed_forward, dtype, device) if spec.feed_forward is not None else None
        self.norm2 = build_norm(spec.norm2, dtype, device) if self.feed_forward is not None else None
        for n in (self.norm1, self.norm2):
            if n is not None and not hasattr(n, "weight"):
                raise ValueError("the outnorm arrangement takes norms that are a weight and an eps (RMSNorm)")

    chains_norms = True      # `forward` takes `next_block`

    def entry_sink(self, resid, step):
        return None

    def parts(self):
        return tuple(p for p in (self.mixer, self.norm1, self.feed_forward, self.norm2) if p is not None)

    def _stream(self, resid, step):
        """The stream as a sublayer reads it."""
        if self.dtype == torch.float32:
            return resid
        h = step.buffer("stream_copy", (resid.shape[0], self.hidden), self.dtype)
        return ops.post_norm_residual(None, resid, None, 0.0, out=h)

    def _join(self, sub, norm, resid, step, wanted: bool):
        """resid += m * norm(sub); returns the stream for the next sublayer if one is `wanted`."""
        if not wanted or self.dtype == torch.float32:
            ops.post_norm_residual(sub, resid, norm.weight, norm.eps, mult=self.mult)
            return resid if wanted else None
        h = step.buffer("stream_copy", (resid.shape[0], self.hidden), self.dtype)
        return ops.post_norm_residual(sub, resid, norm.weight, norm.eps, mult=self.mult, out=h)

    def forward(self, resid, pending, step, cache, state, writes_cache=True, next_block=None):
        h = pending.x if isinstance(pending, StreamRows) else self._stream(resid, step)
        a = self.mixer.forward(h, step, cache, state, writes_cache)
        chained = isinstance(next_block, OutNormBlock) and next_block.dtype == self.dtype
        if self.feed_forward is None:
            h = self._join(a, self.norm1, resid, step, chained)
        else:
            h = self._join(a, self.norm1, resid, step, True)
            f = self.feed_forward.forward(h, step)
            h = self._join(f, self.norm2, resid, step, chained)
        return resid, (StreamRows(h) if chained else None)


class PostNormBlock:
    """x = norm1(a x + mixer(x)); x = norm2(a x + feed_forward(x)), the second line only when the layer has a
    feed-forward; a is a constant.  The sublayers read the stream as it is.  The stream, the sums and the norms
    are float32: one kernel adds a sublayer's result to the scaled stream, norms the sum into the stream and
    leaves the stream, rounded to the compute type, for the sublayer that follows (in float32 that sublayer reads
    the stream itself).  A mixer of several branches (`forward_branches`) has its branches normed and averaged in
    the same kernel.  A block returns no pending delta, and hands the next block of its kind the rounded stream."""

    def __init__(self, spec, dtype, device):
        self.dtype = dtype
        self.alpha = float(spec.stream_mult)
        self.hidden = spec.norm1.dim
        self.mixer = build_mixer(spec.mixer, dtype, device)
        self.norm1 = build_norm(spec.norm1, dtype, device)
        self.feed_forward = build_feed_forward(spec.feed_forward, dtype, device) if spec.feed_forward is not None else None
        self.norm2 = build_norm(spec.norm2, dtype, device) if self.feed_forward is not None else None
        for n in (self.norm1, self.norm2):
            if n is not None and not hasattr(n, "weight"):
                raise ValueError("the postnorm arrangement takes norms that are a weight and an eps (RMSNorm)")

    chains_norms = True      # `forward` takes `next_block`

    def entry_sink(self, resid, step):
        return None

    def parts(self):
        return tuple(p for p in (self.mixer, self.norm1, self.feed_forward, self.norm2) if p is not None)

    def _stream(self, resid, step):
        if self.dtype == torch.float32:
            return resid
        h = step.buffer("stream_copy", (resid.shape[0], self.hidden), self.dtype)
        return ops.post_norm_residual(None, resid, None, 0.0, out=h)

    def _join(self, terms, eps_branch, norm, resid, step, wanted: bool):
        """resid = norm(alpha * resid + sum of the terms); returns the stream for the next sublayer if `wanted`."""
        h = None
        if wanted and self.dtype != torch.float32:
            h = step.buffer("stream_copy", (resid.shape[0], self.hidden), self.dtype)
        ops.sum_norm(resid, self.alpha, terms, norm.weight, norm.eps, out=h, eps_branch=eps_branch)
        return (h if h is not None else resid) if wanted else None

    def forward(self, resid, pending, step, cache, state, writes_cache=True, next_block=None):
        h = pending.x if isinstance(pending, StreamRows) else self._stream(resid, step)
        chained = isinstance(next_block, (PostNormBlock, OutNormBlock)) and next_block.dtype == self.dtype
        branches = getattr(self.mixer, "forward_branches", None)
        if branches is not None and len(self.mixer.branches) <= 2:      # the joining kernel takes two terms
            terms, eps_b = branches(h, step, cache, state, writes_cache)
        else:
            terms, eps_b = [(self.mixer.forward(h, step, cache, state, writes_cache), None, 1.0)], 0.0
        h = self._join(terms, eps_b, self.norm1, resid, step, chained or self.feed_forward is not None)
        if self.feed_forward is not None:
            f = self.feed_forward.forward(h, step)
            h = self._join([(f, None, 1.0)], 0.0, self.norm2, resid, step, chained)
        return resid, (StreamRows(h) if chained else None)


class StreamRows:
    """What an outnorm block hands the next one: `x`, the (complete) residual stream in the compute type."""

    def __init__(self, x):
        self.x = x


class NormedRows:
    """What a block hands the next one when it has already normed the stream for it: `x`, the next
    block's first norm applied to the (complete) residual stream."""

    def __init__(self, x):
        self.x = x


class _BlockTensors(Part):
    """The block's own tensors (the per-channel scales), loaded with its parts."""

    graph_safe = True

    def __init__(self, block):
        self.block = block

    def tensors(self) -> dict:
        b = self.block
        return {n: (b.hidden,) for n in (b.scale1_name, b.scale2_name if b.feed_forward is not None else None)
                if n is not None}

    def load(self, src) -> None:
        b = self.block
        b.scale1 = src.get(b.scale1_name, "vector") if b.scale1_name is not None else None
        b.scale2 = src.get(b.scale2_name, "vector") if (b.scale2_name is not None and b.feed_forward is not None) else None


register_arrangement("prenorm", PreNormBlock)
register_arrangement("sandwich", SandwichBlock)
register_arrangement("outnorm", OutNormBlock)
register_arrangement("postnorm", PostNormBlock)
