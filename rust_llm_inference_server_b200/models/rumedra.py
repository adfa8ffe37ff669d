"""The Rumedra decoder as a description: pre-norm layers over a scaled embedding, x += mixer(norm1(x)), x +=
feed_forward(norm2(x)), with two kinds of mixer.  "hgrn2": a linear recurrence with one gate a channel, bounded from
below, that keeps f of the state and writes 1 - f of the new value.  "parallel": two mixers side by side whose outputs are added
with a constant each: sliding-window grouped-query attention with biased projections, a rotate-half rotation of
part of every head with frequencies scaled by wavelength, values of their own width and a sigmoid gate on every
output channel; and retention, a linear recurrence with a fixed decay a head over rotated queries and keys.
Feed-forwards are units gated by relu, or a mixture of silu-gated experts chosen by softmax scores within the best
groups of router outputs, some of which are identity experts, beside a shared expert.  The logits come from the
embedding table.  This file holds no size: everything comes from RumedraConfig and the order of its layers.
"""

from __future__ import annotations

import math

from ..config.model_config import RopeScaling
from ..config.registry import register_architecture
from ..config.rumedra_config import ARCHITECTURE, RumedraConfig
from ..parts.spec import (BiasedAttentionSpec, EmbeddingSpec, ForgetGateRecurrenceSpec, LayerCall, LayerSpec, LMHeadSpec,
                          ModelSpec, ParallelMixerSpec, RetentionSpec, RMSNormSpec, RopeSpec, RoutedFFSpec, SwiGLUSpec)

# The design fixes these: a dense unit is gated by relu (the limit of g sigmoid(slope g) for a growing slope), an
# expert by silu.
RELU_SLOPE = math.inf
SILU_SLOPE = 1.0


def _rotation(rot):
    if rot is None:
        return None
    scaling = None
    if rot.factor is not None:
        scaling = RopeScaling("llama3", rot.factor, rot.low, rot.high, rot.original)
    return RopeSpec(rot.dims, rot.base, scaling, exact=True)


def _window_attention(cfg: RumedraConfig, m, q: str) -> BiasedAttentionSpec:
    return BiasedAttentionSpec(
        hidden=cfg.width, n_heads=m.heads, n_kv_heads=m.kv_heads, dim=m.dim, v_dim=m.vdim, scale=m.scale, eps=cfg.eps,
        q_proj=q + "q", k_proj=q + "k", v_proj=q + "v", o_proj=q + "o", q_bias=q + "q.b", k_bias=q + "k.b",
        v_bias=q + "v.b", out_gate=q + "g", window=m.window, rotation=_rotation(m.rot))


def _retention(cfg: RumedraConfig, m, q: str) -> RetentionSpec:
    return RetentionSpec(
        hidden=cfg.width, n_heads=m.heads, dim=m.dim, v_dim=m.vdim, decay=m.decay, eps=cfg.eps, q_proj=q + "q",
        k_proj=q + "k", v_proj=q + "v", o_proj=q + "o", gate_proj=q + "g", gate_act="silu", rotation=_rotation(m.rot))


def _mixer(cfg: RumedraConfig, layer, p: str):
    q, m = p + "mix.", layer.mixer
    if layer.type == "hgrn2":
        return ForgetGateRecurrenceSpec(
            hidden=cfg.width, n_heads=m.heads, dim=m.dim, v_dim=m.vdim, eps=cfg.eps, q_proj=q + "q", f_proj=q + "f",
            f_bias=q + "f.b", lower=q + "lower", v_proj=q + "v", out_norm=q + "norm", o_proj=q + "o")
    return ParallelMixerSpec(
        hidden=cfg.width, eps=cfg.eps, out_norms=None, coefficients=(m.left_scale, m.right_scale),
        branches=(_window_attention(cfg, m.left, q + "left."), _retention(cfg, m.right, q + "right.")))


def _gated(cfg: RumedraConfig, ff: int, p: str, slope: float) -> SwiGLUSpec:
    return SwiGLUSpec(cfg.width, ff, p + "gate", p + "up", p + "down", slope=slope)


def _feed_forward(cfg: RumedraConfig, x, p: str):
    if x is None:
        return None
    if x.kind == "dense":
        return _gated(cfg, x.ff, p, RELU_SLOPE)
    return RoutedFFSpec(
        hidden=cfg.width, intermediate=x.ff, n_experts=x.experts, top=x.top, router=p + "router",
        gate_proj=p + "e{e}.gate", up_proj=p + "e{e}.up", down_proj=p + "e{e}.down", correction=p + "correction",
        route_scale=x.scale, slope=SILU_SLOPE, scoring="softmax", n_identity=x.identity, groups=(x.groups, x.keep),
        normalize=True, shared=_gated(cfg, x.shared_ff, p + "shared.", SILU_SLOPE) if x.shared_ff is not None else None)


def describe_rumedra(cfg: RumedraConfig) -> ModelSpec:
    W = cfg.width
    norm = lambda name: RMSNormSpec(W, cfg.eps, name)
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        ff = _feed_forward(cfg, layer.mlp, p + "mlp.")
        layers.append(LayerSpec(norm1=norm(p + "norm1"), mixer=_mixer(cfg, layer, p), norm2=norm(p + "norm2") if ff else None,
                                feed_forward=ff, arrangement="prenorm"))
    return ModelSpec(
        vocab_size=cfg.vocab, hidden=W, embedding=EmbeddingSpec(cfg.vocab, W, "embed", scale=cfg.embedding_scale),
        layers=tuple(layers), order=tuple(LayerCall(i, i) for i in range(len(layers))), final_norm=norm("final.norm"),
        lm_head=LMHeadSpec(cfg.vocab, W, "embed"), max_positions=cfg.max_positions,
        eos_token_ids=tuple(cfg.eos_token_ids))


def rumedra_tensor_kinds(cfg: RumedraConfig) -> dict:
    """{name: (shape, kind)} of every checkpoint tensor, for the random-weights mode.  Kinds: "matrix" N(0, 0.02);
    "norm" N(1, 0.02); "offset" N(0, 0.1) for biases and corrections; "fraction" numbers between 0 and 1 for the lower
    bounds of the forget gates."""
    W = cfg.width
    out = {"embed": ((cfg.vocab, W), "matrix"), "final.norm": ((W,), "norm")}
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        out[p + "norm1"] = ((W,), "norm")
        if layer.type == "hgrn2":
            q, qk, hv = p + "mix.", m.heads * m.dim, m.heads * m.vdim
            out[q + "q"] = ((qk, W), "matrix")
            out[q + "f"] = ((qk, W), "matrix")
            out[q + "f.b"] = ((qk,), "offset")
            out[q + "lower"] = ((qk,), "fraction")
            out[q + "v"] = ((hv, W), "matrix")
            out[q + "norm"] = ((m.vdim,), "norm")
            out[q + "o"] = ((W, hv), "matrix")
        else:
            q, a = p + "mix.left.", m.left
            for name, rows in (("q", a.heads * a.dim), ("k", a.kv_heads * a.dim), ("v", a.kv_heads * a.vdim)):
                out[q + name] = ((rows, W), "matrix")
                out[q + name + ".b"] = ((rows,), "offset")
            out[q + "g"] = ((a.heads * a.vdim, W), "matrix")
            out[q + "o"] = ((W, a.heads * a.vdim), "matrix")
            q, r = p + "mix.right.", m.right
            for name, rows in (("q", r.heads * r.dim), ("k", r.heads * r.dim), ("v", r.heads * r.vdim),
                               ("g", r.heads * r.vdim)):
                out[q + name] = ((rows, W), "matrix")
            out[q + "o"] = ((W, r.heads * r.vdim), "matrix")
        x = layer.mlp
        if x is None:
            continue
        out[p + "norm2"] = ((W,), "norm")
        q = p + "mlp."
        if x.kind == "dense":
            groups = [(q, x.ff)]
        else:
            groups = [(f"{q}e{e}.", x.ff) for e in range(x.experts)]
            if x.shared_ff is not None:
                groups.append((q + "shared.", x.shared_ff))
            out[q + "router"] = ((x.outputs, W), "matrix")
            out[q + "correction"] = ((x.outputs,), "offset")
        for g, ff in groups:
            out[g + "gate"] = ((ff, W), "matrix")
            out[g + "up"] = ((ff, W), "matrix")
            out[g + "down"] = ((W, ff), "matrix")
    return out


register_architecture(ARCHITECTURE, RumedraConfig.from_dict, describe_rumedra, rumedra_tensor_kinds)
