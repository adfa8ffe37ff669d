"""Lanirax without a GPU: the configuration reader and what it refuses, the description against an
independent list of tensors, the order of the runs and who keeps a cache and a state, the plain restatement
against closed forms, and that the test models' logits move far beyond the tolerances when a mechanism is
left out."""

import copy
import math

import numpy as np
import pytest

from tests import lanirax_util as U
from tests.plain import lanirax_plain as P


def test_reader_takes_every_size_and_constant_from_the_file():
    from rust_llm_inference_server_b200.config import ConfigError
    from rust_llm_inference_server_b200.config.lanirax_config import LaniraxConfig
    cfg = LaniraxConfig.from_dict(U.CONFIGS["A"])
    assert (cfg.vocab, cfg.width, cfg.eps, cfg.alpha, len(cfg.layers)) == (211, 96, 1e-5, 1.8, 5)
    m = cfg.layers[0].mixer
    assert (m.heads, m.kv_heads, m.dim, m.vdim, m.scale, m.q_temp_coef, m.q_temp_every) == (4, 2, 32, 16, 0.35, 0.7, 5)
    a, r = cfg.layers[1].mixer.left, cfg.layers[1].mixer.right
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.window) == (4, 2, 32, 32, 0.4, 9)
    assert (a.rot.dims, a.rot.base, a.rot.factor, a.rot.original, a.rot.fast, a.rot.slow) == (16, 10000.0, 4.0, 64, 16.0, 2.0)
    assert (r.heads, r.kv_heads, r.dim, r.vdim, r.conv) == (4, 2, 16, 24, 3)
    x = cfg.layers[1].mlp
    assert (x.experts, x.top, x.ff) == (6, 3, 40)
    assert cfg.layers[3].mlp is None and cfg.layers[3].mixer.left.rot.factor is None      # no blend of frequencies
    assert [cfg.owner(i) for i in range(5)] == [0, 1, 0, 3, 1]
    b = LaniraxConfig.from_dict(U.CONFIGS["B"])
    assert b.layers[1].mixer.q_temp_coef is None and b.alpha == 1.0

    def broken(edit):
        c = copy.deepcopy(U.CONFIGS["A"])
        edit(c)
        with pytest.raises(ConfigError):
            LaniraxConfig.from_dict(c)
    broken(lambda c: c["layers"][0]["mixer"].update(heads=3))                     # not a multiple of kv_heads
    broken(lambda c: c["layers"][0].update(type="convolution"))
    broken(lambda c: c["layers"][1]["mlp"]["router"].update(top=9))
    broken(lambda c: c["layers"][1]["mixer"]["left"].update(vdim=16))             # the values are the keys
    broken(lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=40))      # more than a head
    broken(lambda c: c["layers"][1]["mixer"]["left"].pop("mask"))
    broken(lambda c: c["layers"][1]["mixer"].pop("right"))
    broken(lambda c: c.pop("norm"))
    broken(lambda c: c.pop("postln_alpha"))
    broken(lambda c: c["layers"][1]["mlp"].update(kind="dense"))
    broken(lambda c: c["layers"][2].update(weights_of=2))                         # itself
    broken(lambda c: c["layers"][2].update(weights_of=7))
    broken(lambda c: c["layers"][2].update(weights_of=1))                         # another kind of layer
    broken(lambda c: c["layers"][2]["mixer"].update(scale=0.5))                   # differs from the layer it borrows from


@pytest.mark.parametrize("which", sorted(U.CONFIGS))
def test_description_lists_the_tensors_and_the_runs(which):
    from rust_llm_inference_server_b200.models.model import build_model
    cfg = U.CONFIGS[which]
    model = build_model(cfg, "float32", "cpu")
    want = U.tensor_shapes(cfg)
    got = model.tensors()
    assert set(got) == set(want)
    for name, shape in got.items():
        assert tuple(shape) == tuple(want[name]), name
    layers = cfg["layers"]
    # one run a listed layer, each with a cache of its own; a parallel layer also keeps a state
    specs, states = model.cache_slot_specs, model.call_state_specs
    assert len(specs) == len(layers) == len(states)
    for sp, st, l in zip(specs, states, layers):
        if l["type"] == "attention":
            m = l["mixer"]
            assert (sp.n_kv_heads, sp.head_dim, sp.v_head_dim or sp.head_dim, sp.window) == (m["kv_heads"], m["dim"], m["vdim"], None)
            assert st is None
        else:
            a, r = l["mixer"]["left"], l["mixer"]["right"]
            assert (sp.n_kv_heads, sp.head_dim, sp.window) == (a["kv_heads"], a["dim"], a["mask"]["size"])
            floats = r["heads"] * r["vdim"] * r["dim"] + (r["conv"] - 1) * (2 * r["kv_heads"] * r["dim"] + r["heads"] * r["vdim"])
            assert tuple(st.shape) == (floats,)
    assert model.graph_safe


def test_random_weights_mode_lists_the_same_tensors():
    from rust_llm_inference_server_b200.config.lanirax_config import LaniraxConfig
    from rust_llm_inference_server_b200.models.lanirax import head_slopes, lanirax_tensor_kinds
    for which, cfg in U.CONFIGS.items():
        kinds = lanirax_tensor_kinds(LaniraxConfig.from_dict(cfg))
        assert {k: tuple(v[0]) for k, v in kinds.items()} == {k: tuple(v) for k, v in U.tensor_shapes(cfg).items()}, which
    assert np.allclose(head_slopes(4), [0.25, 0.0625, 0.015625, 0.00390625])
    assert np.allclose(head_slopes(3), P.head_slopes(3))


def test_blended_frequencies_of_the_package_and_the_plain_form():
    import torch
    from rust_llm_inference_server_b200.parts.base import build_position
    from rust_llm_inference_server_b200.parts.spec import YarnRopeSpec
    for dims, base, sc in ((16, 10000.0, (4.0, 64, 16.0, 2.0)), (48, 50000.0, (16.0, 128, 8.0, 0.5)), (12, 20000.0, (2.0, 32, 4.0, 1.0)),
                           (10, 777.0, (3.0, 50, 10.0, 1.5)), (8, 100.0, None)):
        rot = {"dims": dims, "base": base}
        if sc:
            rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), sc))
        f, mag = P.blended_frequencies(rot)
        spec = YarnRopeSpec(dims, base, *(sc or (None,)), pairing="adjacent") if sc else YarnRopeSpec(dims, base, pairing="adjacent")
        inv, r, m = build_position(spec, torch.float32, "cpu").rotation()
        assert r == dims and abs(m - mag) < 1e-6
        assert np.allclose(inv.double().numpy(), f, rtol=2e-6, atol=0)
    # the blend: the fastest pairs keep their frequency, the slowest are divided by the factor
    f, mag = P.blended_frequencies({"dims": 64, "base": 10000.0, "scaling": {"factor": 8.0, "original": 256, "fast": 32.0, "slow": 1.0}})
    plain = 10000.0 ** (-np.arange(32) / 32.0)
    assert np.isclose(f[0], plain[0]) and np.isclose(f[-1], plain[-1] / 8.0) and np.isclose(mag, 0.1 * math.log(8.0) + 1.0)
    assert np.all(f <= plain + 1e-15) and np.all(f >= plain / 8.0 - 1e-15)


def test_plain_functions_against_closed_forms():
    rng = np.random.default_rng(0)
    # a rotation keeps a pair's length (times the multiplier) and turns (1, 0) to (cos, sin)
    x = np.zeros((3, 1, 6))
    x[:, 0, 0] = 1.0
    x[:, 0, 4] = 7.0
    y = P.rotate_adjacent_pairs(x, np.array([0.0, 1.0, 2.0]), np.array([0.5, 0.1]), 1.2)
    assert np.allclose(y[2, 0, :2], [1.2 * math.cos(1.0), 1.2 * math.sin(1.0)]) and np.allclose(y[:, 0, 4], 7.0)
    assert np.allclose(y[0, 0, :2], [1.2, 0.0])
    # window and sink: with a window of 2 the third token sees two keys and the sink
    q, k = rng.standard_normal((3, 1, 4)), rng.standard_normal((3, 1, 4))
    v = rng.standard_normal((3, 1, 2))
    o = P.masked_attention(q, k, v, 0.5, window=2, sinks=np.array([0.3]))
    s = np.array([k[1, 0] @ q[2, 0], k[2, 0] @ q[2, 0]]) * 0.5
    e = np.exp(s)
    assert np.allclose(o[2, 0], (e[0] * v[1, 0] + e[1] * v[2, 0]) / (e.sum() + math.exp(0.3)))
    # slopes: the penalty grows with the distance
    o = P.masked_attention(q, k, v, 0.5, slopes=np.array([0.7]))
    s = np.array([k[j, 0] @ q[2, 0] * 0.5 - 0.7 * (2 - j) for j in range(3)])
    assert np.allclose(o[2, 0], (np.exp(s) / np.exp(s).sum()) @ v[:, 0])
    # the temperature steps with the position
    t = P.temperature(12, {"coef": 0.5, "every": 5})
    assert np.allclose(t[:4], 1.0) and np.allclose(t[4:9], 1 + 0.5 * math.log(2)) and np.allclose(t[9:], 1 + 0.5 * math.log(3))
    # the convolution: the last tap is the current token's
    c = P.short_conv(np.array([[1.0], [2.0], [4.0]]), np.array([[100.0, 10.0, 1.0]]))
    assert c[:, 0].tolist() == [1.0, 12.0, 124.0]
    # the delta rule with beta 1 and no decay stores v along a unit key, and the read-out sees the write
    kk = np.array([[1.0, 0.0], [0.0, 1.0], [1.0, 0.0]])
    vv = np.array([[3.0], [5.0], [11.0]])
    o = P.delta_rule(kk, kk, vv, np.ones(3), np.ones(3))
    assert o[:, 0].tolist() == [3.0, 5.0, 11.0]                 # the third write replaces the first along the same key
    o = P.delta_rule(kk, kk, vv, np.array([1.0, 1.0, 0.5]), np.array([1.0, 1.0, 0.5]))
    assert np.isclose(o[2, 0], 1.5 + 0.5 * (11.0 - 1.5))        # decayed, then corrected half of the way
    # routing: the largest logits, softmax over those alone
    w = {"r.router": np.array([[1.0, 0.0], [0.0, 1.0], [-1.0, 0.0]]), "r.router.b": np.array([0.0, 0.0, 4.0])}
    for e in range(3):
        w[f"r.e{e}.gate"], w[f"r.e{e}.up"], w[f"r.e{e}.down"] = np.eye(2) * (e + 1), np.eye(2), np.eye(2)
    out = P.routed_ff(np.array([[2.0, 1.0]]), w, "r.", {"router": {"experts": 3, "top": 2}})
    z = np.array([2.0, 1.0, 2.0])                                # experts 0 and 2 (a tie goes to the lower index)
    g = np.exp(z[[0, 2]]) / np.exp(z[[0, 2]]).sum()
    h = np.array([2.0, 1.0])
    want = sum(gi * (P.silu(h * (e + 1)) * h) for gi, e in zip(g, (0, 2)))
    assert np.allclose(out[0], want)


def _logits(which, edit=None, cfg_edit=None, n=70):
    cfg = copy.deepcopy(U.CONFIGS[which])
    if cfg_edit:
        cfg_edit(cfg)
    w = {k: v.double().numpy() for k, v in U.draw_weights(U.CONFIGS[which], U.SEEDS[which]).items()}
    if edit:
        edit(w)
    toks = np.random.default_rng(4).integers(0, cfg["vocab"], size=n).tolist()
    return P.forward(cfg, w, toks)[0]


def test_the_plain_model_is_causal_and_runs_borrowed_layers():
    cfg = U.CONFIGS["A"]
    w = {k: v.double().numpy() for k, v in U.draw_weights(cfg, 3).items()}
    toks = np.random.default_rng(1).integers(0, cfg["vocab"], size=30).tolist()
    full, streams = P.forward(cfg, w, toks)
    assert streams.shape == (5, 30, 96)
    assert np.allclose(full[:17], P.forward(cfg, w, toks[:17])[0], atol=1e-9)


@pytest.mark.parametrize("which", ["A", "D"])
def test_a_missing_mechanism_shows_in_the_logits(which):
    base = _logits(which)

    def moved(**kw):
        d = _logits(which, **kw) - base
        return float(np.sqrt(np.mean(d * d, axis=-1)).max())

    def scaled(suffix, by):
        return lambda w: [w.__setitem__(k, v * by) for k, v in list(w.items()) if k.endswith(suffix)]
    par = [i for i, l in enumerate(U.CONFIGS[which]["layers"]) if l["type"] == "parallel"][0]
    att = [i for i, l in enumerate(U.CONFIGS[which]["layers"]) if l["type"] == "attention"][0]

    def left(c):
        return c["layers"][par]["mixer"]["left"]
    # no sink; a window one token longer or shorter; no rotation; the other pairing is another model; no blend
    assert moved(edit=lambda w: [w.__setitem__(k, v - 30.0) for k, v in list(w.items()) if k.endswith(".sink")]) > 0.1
    assert moved(cfg_edit=lambda c: left(c)["mask"].update(size=left(c)["mask"]["size"] + 1)) > 0.05
    assert moved(cfg_edit=lambda c: left(c)["mask"].update(size=left(c)["mask"]["size"] - 1)) > 0.05
    assert moved(cfg_edit=lambda c: left(c)["rot"].update(base=1.0000001, scaling=None)) > 0.05
    assert moved(cfg_edit=lambda c: left(c)["rot"].pop("scaling")) > 0.02
    # a temperature that is not applied or steps one position late; no slopes is another scale of the penalty
    assert moved(cfg_edit=lambda c: c["layers"][att]["mixer"].pop("q_temp")) > 0.05
    assert moved(cfg_edit=lambda c: c["layers"][att]["mixer"]["q_temp"].update(every=c["layers"][att]["mixer"]["q_temp"]["every"] + 1)) > 0.02
    # the recurrent branch: no decay, no step bias, a tap left out, the branch's norm weight
    assert moved(edit=scaled("A_log", 0.0)) > 0.02
    assert moved(edit=scaled("dt_bias", 0.0)) > 0.01
    assert moved(edit=lambda w: [w.__setitem__(k, np.concatenate([v[:, :1] * 0, v[:, 1:]], 1)) for k, v in list(w.items()) if k.endswith(".conv")]) > 0.05
    assert moved(edit=scaled("right.out", 0.0)) > 0.1
    assert moved(edit=scaled("left.out", 0.0)) > 0.1
    # the router's bias; the factor on the stream; the embedding's norm
    assert moved(edit=scaled("router.b", 0.0)) > 0.05
    assert moved(cfg_edit=lambda c: c.update(postln_alpha=1.0)) > 0.1
    assert moved(edit=lambda w: w.__setitem__("embed.norm", w["embed.norm"] * 0 + 1)) > 0.02
