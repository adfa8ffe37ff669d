"""The Lanirax decoder as a description: layers whose sum of stream and sublayer is normed (x = norm(a x +
sublayer(x)), a constant a), with two kinds of mixer.  "attention": causal attention without rotation, queries
and keys normed per head, a query temperature that grows in steps with the position, and a penalty linear in
the distance with one slope a head.  "parallel": two mixers side by side whose normed outputs are averaged: a
sliding-window attention whose keys double as values, with a rotation of adjacent pairs on part of every head
(YaRN's frequency blend), unit root mean square of queries and keys and a learned sink in the softmax; and a
gated delta rule behind short convolutions.  Feed-forwards route every token to a few of many gated experts,
with weights that are the softmax over the chosen logits.  A layer may run with another layer's tensors and a
cache and state of its own.  This file holds no size: everything comes from LaniraxConfig and the order of its
layers.
"""

from __future__ import annotations

from ..config.lanirax_config import ARCHITECTURE, LaniraxConfig
from ..config.registry import register_architecture
from ..parts.spec import (BiasedAttentionSpec, EmbeddingSpec, GatedDeltaSpec, LayerCall, LayerSpec, LMHeadSpec,
                          ModelSpec, ParallelMixerSpec, RMSNormSpec, RoutedFFSpec, YarnRopeSpec)

# The design fixes these: the slopes of the distance penalty, and the epsilon under the root of the unit norms
# of the recurrent branch's queries and keys.
SLOPE_EXPONENT = 8.0
UNIT_EPS = 1e-6


def head_slopes(n_heads: int) -> tuple:
    """slope_h = 2^(-8 (h + 1) / H), h = 0 .. H - 1."""
    return tuple(2.0 ** (-SLOPE_EXPONENT * (h + 1) / n_heads) for h in range(n_heads))


def _slope_attention(cfg: LaniraxConfig, m, q: str) -> BiasedAttentionSpec:
    return BiasedAttentionSpec(
        hidden=cfg.width, n_heads=m.heads, n_kv_heads=m.kv_heads, dim=m.dim, v_dim=m.vdim, scale=m.scale, eps=cfg.eps,
        q_proj=q + "q", k_proj=q + "k", v_proj=q + "v", o_proj=q + "o", q_norm=q + "q.norm", k_norm=q + "k.norm",
        q_temp=(m.q_temp_coef, m.q_temp_every) if m.q_temp_coef is not None else None, slopes=head_slopes(m.heads))


def _window_attention(cfg: LaniraxConfig, m, q: str) -> BiasedAttentionSpec:
    r = m.rot
    return BiasedAttentionSpec(
        hidden=cfg.width, n_heads=m.heads, n_kv_heads=m.kv_heads, dim=m.dim, v_dim=m.vdim, scale=m.scale, eps=cfg.eps,
        q_proj=q + "q", k_proj=q + "k", v_proj=None, o_proj=q + "o", window=m.window, unit_norm=True, sink=q + "sink",
        rotation=YarnRopeSpec(r.dims, r.base, r.factor, r.original, r.fast, r.slow, pairing="adjacent"))


def _delta_rule(cfg: LaniraxConfig, m, q: str) -> GatedDeltaSpec:
    return GatedDeltaSpec(
        hidden=cfg.width, n_heads=m.heads, n_qk_heads=m.kv_heads, dim=m.dim, v_dim=m.vdim, conv=m.conv, eps=cfg.eps,
        q_proj=q + "q", k_proj=q + "k", v_proj=q + "v", q_conv=q + "q.conv", k_conv=q + "k.conv", v_conv=q + "v.conv",
        beta_proj=q + "b", decay_proj=q + "a", a_log=q + "A_log", dt_bias=q + "dt_bias", gate_proj=q + "g",
        out_norm=q + "norm", o_proj=q + "o", unit_eps=UNIT_EPS)


def _mixer(cfg: LaniraxConfig, layer, p: str):
    q = p + "mix."
    if layer.type == "attention":
        return _slope_attention(cfg, layer.mixer, q)
    return ParallelMixerSpec(
        hidden=cfg.width, eps=cfg.eps, out_norms=(q + "left.out", q + "right.out"),
        branches=(_window_attention(cfg, layer.mixer.left, q + "left."), _delta_rule(cfg, layer.mixer.right, q + "right.")))


def _feed_forward(cfg: LaniraxConfig, x, p: str):
    if x is None:
        return None
    return RoutedFFSpec(
        hidden=cfg.width, intermediate=x.ff, n_experts=x.experts, top=x.top, router=p + "router",
        gate_proj=p + "e{e}.gate", up_proj=p + "e{e}.up", down_proj=p + "e{e}.down", router_bias=p + "router.b",
        scoring="softmax_chosen")


def describe_lanirax(cfg: LaniraxConfig) -> ModelSpec:
    W = cfg.width
    norm = lambda name: RMSNormSpec(W, cfg.eps, name)
    layers, order, index = [], [], {}
    for i, layer in enumerate(cfg.layers):
        if layer.weights_of is not None:
            continue
        p = f"l{i}."
        ff = _feed_forward(cfg, layer.mlp, p + "mlp.")
        index[i] = len(layers)
        layers.append(LayerSpec(norm1=norm(p + "norm1"), mixer=_mixer(cfg, layer, p), norm2=norm(p + "norm2") if ff else None,
                                feed_forward=ff, arrangement="postnorm", stream_mult=cfg.alpha))
    for i in range(len(cfg.layers)):
        # a layer that runs with another's tensors is a second call of that layer, with cache slot and state of its own
        order.append(LayerCall(index[cfg.owner(i)], i))
    return ModelSpec(
        vocab_size=cfg.vocab, hidden=W, embedding=EmbeddingSpec(cfg.vocab, W, "embed", norm=norm("embed.norm")),
        layers=tuple(layers), order=tuple(order), final_norm=norm("final.norm"), lm_head=LMHeadSpec(cfg.vocab, W, "head"),
        max_positions=cfg.max_positions, eos_token_ids=tuple(cfg.eos_token_ids))


def lanirax_tensor_kinds(cfg: LaniraxConfig) -> dict:
    """{name: (shape, kind)} of every checkpoint tensor, for the random-weights mode.  Kinds: "matrix" N(0, 0.02);
    "norm" N(1, 0.02); "offset" N(0, 0.1) for biases, decay logarithms and step biases; "gain" N(0, 1) for sinks;
    "taps" N(0, 0.5) for the short convolutions."""
    W = cfg.width
    out = {"embed": ((cfg.vocab, W), "matrix"), "embed.norm": ((W,), "norm"), "head": ((cfg.vocab, W), "matrix"),
           "final.norm": ((W,), "norm")}
    for i, layer in enumerate(cfg.layers):
        if layer.weights_of is not None:
            continue
        p, m = f"l{i}.", layer.mixer
        out[p + "norm1"] = ((W,), "norm")
        if layer.type == "attention":
            q = p + "mix."
            out[q + "q"] = ((m.heads * m.dim, W), "matrix")
            out[q + "k"] = ((m.kv_heads * m.dim, W), "matrix")
            out[q + "v"] = ((m.kv_heads * m.vdim, W), "matrix")
            out[q + "q.norm"] = ((m.dim,), "norm")
            out[q + "k.norm"] = ((m.dim,), "norm")
            out[q + "o"] = ((W, m.heads * m.vdim), "matrix")
        else:
            q, a = p + "mix.left.", m.left
            out[q + "q"] = ((a.heads * a.dim, W), "matrix")
            out[q + "k"] = ((a.kv_heads * a.dim, W), "matrix")
            out[q + "sink"] = ((a.heads,), "gain")
            out[q + "o"] = ((W, a.heads * a.vdim), "matrix")
            q, r = p + "mix.right.", m.right
            qk, hv = r.kv_heads * r.dim, r.heads * r.vdim
            for name, rows in (("q", qk), ("k", qk), ("v", hv)):
                out[q + name] = ((rows, W), "matrix")
                out[q + name + ".conv"] = ((rows, r.conv), "taps")
            out[q + "b"] = ((r.heads, W), "matrix")
            out[q + "a"] = ((r.heads, W), "matrix")
            out[q + "A_log"] = ((r.heads,), "offset")
            out[q + "dt_bias"] = ((r.heads,), "offset")
            out[q + "g"] = ((hv, W), "matrix")
            out[q + "norm"] = ((r.vdim,), "norm")
            out[q + "o"] = ((W, hv), "matrix")
            out[p + "mix.left.out"] = ((W,), "norm")
            out[p + "mix.right.out"] = ((W,), "norm")
        x = layer.mlp
        if x is None:
            continue
        out[p + "norm2"] = ((W,), "norm")
        for e in range(x.experts):
            out[f"{p}mlp.e{e}.gate"] = ((x.ff, W), "matrix")
            out[f"{p}mlp.e{e}.up"] = ((x.ff, W), "matrix")
            out[f"{p}mlp.e{e}.down"] = ((W, x.ff), "matrix")
        out[p + "mlp.router"] = ((x.experts, W), "matrix")
        out[p + "mlp.router.b"] = ((x.experts,), "offset")
    return out


register_architecture(ARCHITECTURE, LaniraxConfig.from_dict, describe_lanirax, lanirax_tensor_kinds)
