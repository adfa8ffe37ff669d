"""Rumedra without a GPU: the configuration reader and what it refuses, the description against an independent
list of tensors, who keeps a cache and a state, the frequency rule and the plain restatement against closed forms,
and that the test models' logits move far beyond the tolerances when a mechanism is left out."""

import copy
import math

import numpy as np
import pytest

from tests import rumedra_util as U
from tests.plain import rumedra_plain as P


def test_reader_takes_every_size_and_constant_from_the_file():
    from rust_llm_inference_server_b200.config import ConfigError
    from rust_llm_inference_server_b200.config.rumedra_config import RumedraConfig
    cfg = RumedraConfig.from_dict(U.CONFIGS["A"])
    assert (cfg.vocab, cfg.width, cfg.eps, cfg.embedding_scale, len(cfg.layers)) == (211, 96, 1e-5, 2.0, 5)
    m = cfg.layers[0].mixer
    assert (m.heads, m.dim, m.vdim) == (3, 8, 16)
    x = cfg.layers[0].mlp
    assert (x.kind, x.experts, x.top, x.ff, x.identity, x.groups, x.keep, x.scale, x.shared_ff, x.outputs) == \
        ("moe", 7, 3, 24, 2, 3, 2, 1.6, 16, 9)
    p = cfg.layers[1].mixer
    a, r = p.left, p.right
    assert (p.left_scale, p.right_scale) == (0.7, 0.4)
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.window) == (4, 2, 32, 16, 0.3, 9)
    assert (a.rot.dims, a.rot.base, a.rot.factor, a.rot.low, a.rot.high, a.rot.original) == (16, 10000.0, 4.0, 1.0, 4.0, 64)
    assert (r.heads, r.dim, r.vdim, r.decay, r.rot.dims, r.rot.base, r.rot.factor) == (2, 16, 24, (0.9, 0.97), 8, 500.0, None)
    assert (cfg.layers[1].mlp.kind, cfg.layers[1].mlp.ff) == ("dense", 40)
    assert cfg.layers[2].mlp is None and cfg.layers[2].mixer.left.rot.factor is None
    y = cfg.layers[4].mlp
    assert (y.identity, y.groups, y.keep, y.shared_ff) == (0, 2, 1, None)

    def broken(edit):
        c = copy.deepcopy(U.CONFIGS["A"])
        edit(c)
        with pytest.raises(ConfigError):
            RumedraConfig.from_dict(c)
    broken(lambda c: c["layers"][1]["mixer"]["left"].update(heads=3))               # not a multiple of kv_heads
    broken(lambda c: c["layers"][0].update(type="convolution"))
    broken(lambda c: c["layers"][0]["mlp"]["router"].update(top=7))                 # more than the kept groups hold
    broken(lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4))     # 9 outputs in 4 groups
    broken(lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(keep=4))
    broken(lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=40))        # more than a head
    broken(lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=7))
    broken(lambda c: c["layers"][1]["mixer"]["right"].update(decay=[0.9]))          # one a head
    broken(lambda c: c["layers"][1]["mixer"].pop("right"))
    broken(lambda c: c["layers"][1]["mixer"].pop("left_scale"))
    broken(lambda c: c.pop("norm"))
    broken(lambda c: c["layers"][1]["mlp"].update(kind="gated"))
    broken(lambda c: c["layers"][3]["mixer"].pop("vdim"))


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
    specs, states = model.cache_slot_specs, model.call_state_specs
    assert len(states) == len(layers)
    for i, (st, l) in enumerate(zip(states, layers)):
        sp = specs[i] if i < len(specs) else None
        if l["type"] == "hgrn2":
            m = l["mixer"]
            assert sp is None and tuple(st.shape) == (m["heads"], m["vdim"], m["dim"])
        else:
            a, r = l["mixer"]["left"], l["mixer"]["right"]
            assert (sp.n_kv_heads, sp.head_dim, sp.v_head_dim or sp.head_dim, sp.window) == \
                (a["kv_heads"], a["dim"], a["vdim"], a["mask"]["size"])
            assert tuple(st.shape) == (r["heads"], r["vdim"], r["dim"])
    assert model.graph_safe


def test_random_weights_mode_knows_the_design():
    from rust_llm_inference_server_b200.weights.random_init import random_tensors
    w = random_tensors(U.CONFIGS["D"], 4)
    want = U.tensor_shapes(U.CONFIGS["D"])
    assert {k: tuple(v.shape) for k, v in w.items()} == {k: tuple(v) for k, v in want.items()}
    lower = w["l1.mix.lower"].float()
    assert float(lower.min()) > 0 and float(lower.max()) < 1


def test_frequencies_by_wavelength():
    from rust_llm_inference_server_b200.config.model_config import RopeScaling
    from rust_llm_inference_server_b200.parts.position import rope_inverse_frequencies_exact
    rot = {"dims": 32, "base": 10000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 256}}
    f = P.rotary_frequencies(rot)
    plain = 10000.0 ** (-2.0 * np.arange(16) / 32)
    wl = 2 * math.pi / plain
    assert np.array_equal(f[wl < 64], plain[wl < 64]) and (wl < 64).any()
    assert np.allclose(f[wl > 256], plain[wl > 256] / 8.0) and (wl > 256).any()
    mid = (wl >= 64) & (wl <= 256)
    assert mid.any() and ((f[mid] < plain[mid]) & (f[mid] > plain[mid] / 8.0)).all()
    got = rope_inverse_frequencies_exact(32, 10000.0, RopeScaling("llama3", 8.0, 1.0, 4.0, 256))
    np.testing.assert_allclose(got, f, rtol=1e-7)
    np.testing.assert_allclose(rope_inverse_frequencies_exact(32, 10000.0), plain, rtol=1e-7)


def test_plain_mechanisms_against_closed_forms():
    rng = np.random.default_rng(0)
    # rotation: a pair (u, v) at distance dims / 2 turns by position * f; dot products depend on the distance only
    rot = {"dims": 4, "base": 100.0}
    x = rng.standard_normal((1, 1, 6))
    y = P.rotate(x, [3], rot)
    f = P.rotary_frequencies(rot)
    assert np.allclose(y[0, 0, 0], x[0, 0, 0] * math.cos(3 * f[0]) - x[0, 0, 2] * math.sin(3 * f[0]))
    assert np.allclose(y[0, 0, 3], x[0, 0, 3] * math.cos(3 * f[1]) + x[0, 0, 1] * math.sin(3 * f[1]))
    assert np.array_equal(y[0, 0, 4:], x[0, 0, 4:])
    a, b = rng.standard_normal((1, 1, 4)), rng.standard_normal((1, 1, 4))
    d1 = (P.rotate(a, [10], rot) * P.rotate(b, [7], rot)).sum()
    d2 = (P.rotate(a, [103], rot) * P.rotate(b, [100], rot)).sum()
    assert np.allclose(d1, d2)
    # retention: o_t = sum_j decay^(t - j) (q_t . k_j) v_j with rotated q, k
    T, d, dv = 7, 4, 3
    m = {"heads": 1, "dim": d, "vdim": dv, "decay": [0.8], "rot": rot}
    h = rng.standard_normal((T, 5))
    w = {"q": rng.standard_normal((d, 5)), "k": rng.standard_normal((d, 5)), "v": rng.standard_normal((dv, 5)),
         "g": rng.standard_normal((dv, 5)), "o": np.eye(dv)}
    got = P.retention(h, w, "", m, np.arange(T), 1e-6)
    q = P.rotate((h @ w["q"].T).reshape(T, 1, d), np.arange(T), rot)[:, 0]
    k = P.rotate((h @ w["k"].T).reshape(T, 1, d), np.arange(T), rot)[:, 0] * d ** -0.5
    v = h @ w["v"].T
    o = np.stack([sum(0.8 ** (t - j) * (q[t] @ k[j]) * v[j] for j in range(t + 1)) for t in range(T)])
    assert np.allclose(got, P.rms_unit(o, 1e-6) * P.silu(h @ w["g"].T))
    # the forget-gate recurrence with a constant gate f: o_t = sum_j f^(t - j) (1 - f) (q_t . 1) v_j per channel
    m = {"heads": 1, "dim": 2, "vdim": dv}
    w = {"q": rng.standard_normal((2, 5)), "f": np.zeros((2, 5)), "f.b": np.zeros(2), "lower": np.array([0.5, 0.5]),
         "v": rng.standard_normal((dv, 5)), "norm": np.ones(dv), "o": np.eye(dv)}
    got = P.hgrn2(h, w, "", m, 1e-6)
    fgate = 0.5 + 0.5 * 0.5
    q, v = P.silu(h @ w["q"].T), h @ w["v"].T
    o = np.stack([sum(fgate ** (t - j) * (1 - fgate) * q[t].sum() * v[j] for j in range(t + 1)) for t in range(T)])
    assert np.allclose(got, P.rms_unit(o, 1e-6))
    # routing: groups, identity, normalised weights
    r = {"experts": 4, "identity": 2, "top": 2, "scale": 1.5, "groups": {"count": 3, "keep": 1}}
    wr = {"router": np.eye(6), "correction": np.array([0.0, 0.0, 0.0, 0.0, 0.5, -0.9])}
    hh = np.array([[0.0, 0.1, 3.0, 0.2, 0.0, 0.0],      # group 1 has the best score: outputs 2 and 3
                   [0.0, 0.1, 1.0, 0.2, 0.9, 0.0]])     # the correction lifts group 2: outputs 4 and 5 (both identity)
    idx, wt = P.route(hh, wr, "", r)
    assert idx.tolist() == [[2, 3], [4, 5]]
    s = np.exp(hh[1]) / np.exp(hh[1]).sum()
    assert np.allclose(wt[1], s[[4, 5]] / s[[4, 5]].sum() * 1.5) and np.allclose(wt.sum(-1), 1.5)


@pytest.mark.parametrize("which", ["A", "B"])
def test_every_mechanism_counts_in_the_test_models(which, tmp_path):
    """The logits of the test models move far beyond the tolerances when a mechanism is left out or read one off."""
    cfg = U.CONFIGS[which]
    w = {k: v.to(dtype=__import__("torch").float64).numpy() for k, v in U.draw_weights(cfg, U.SEEDS[which]).items()}
    toks = np.random.default_rng(1).integers(0, cfg["vocab"], size=60).tolist()
    base = P.forward(cfg, w, toks)[0]

    def moved(cfg2=None, w2=None, least=0.05):
        got = P.forward(cfg2 or cfg, w2 or w, toks)[0]
        d = (got - base)[20:]
        assert np.sqrt((d * d).mean()) / base.std() > least

    def edited(fn):
        c = copy.deepcopy(cfg)
        fn(c)
        return c
    par = next(i for i, l in enumerate(cfg["layers"]) if l["type"] == "parallel" and l["mixer"]["left"]["mask"]["size"] > 1)
    rec = next(i for i, l in enumerate(cfg["layers"]) if l["type"] == "hgrn2")
    routed = max(i for i, l in enumerate(cfg["layers"]) if l["mlp"] and l["mlp"]["kind"] == "moe" and l["mlp"]["router"]["identity"])
    moved(edited(lambda c: c["layers"][par]["mixer"]["left"]["mask"].update(size=c["layers"][par]["mixer"]["left"]["mask"]["size"] + 1)), least=0.003)
    moved(edited(lambda c: c["layers"][par]["mixer"]["left"]["rot"].update(base=3.0)))
    moved(edited(lambda c: c["layers"][par]["mixer"].update(right_scale=0.0)))
    moved(edited(lambda c: c["layers"][par]["mixer"]["right"].update(decay=[0.0] * c["layers"][par]["mixer"]["right"]["heads"])))
    moved(edited(lambda c: c["embedding"].update(scale=c["embedding"]["scale"] * 1.5)), least=0.01)
    moved(edited(lambda c: c["layers"][routed]["mlp"]["router"]["groups"].update(count=1, keep=1)), least=0.01)
    moved(edited(lambda c: c["layers"][routed]["mlp"]["router"].update(scale=0.0)))
    for name in (f"l{par}.mix.left.q.b", f"l{par}.mix.left.v.b", f"l{rec}.mix.f.b", f"l{rec}.mix.lower", f"l{routed}.mlp.correction"):
        w2 = dict(w)
        w2[name] = np.zeros_like(w[name])
        moved(w2=w2, least=0.01)
    w2 = dict(w)
    w2[f"l{par}.mix.left.g"] = np.zeros_like(w[f"l{par}.mix.left.g"])            # every gate at a half
    moved(w2=w2)
