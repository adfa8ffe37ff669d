"""Lanirax on the GPU against the plain restatement: every kernel alone (keys far back, at page borders and
just inside and outside a window made to carry a head's weight, sinks that outweigh every key, slopes, first
tokens, the recurrence cut into portions over slots that held something else, routing by the logits), every
kind of layer alone in a small model, the stream after every run of a layer, whole prompts against portions,
single tokens and mixed batches in pools so small that pages and slots are used again, long decoding, and
greedy generation through the entry point and the command line."""

from types import SimpleNamespace

import numpy as np
import pytest
import torch

from tests import lanirax_util as U
from tests import replay_util as R
from tests.plain import lanirax_plain as P
from tests.test_gavodra_gpu import dev, fill_pools, hand_step, host, position_error, requests_for

pytestmark = pytest.mark.gpu

# A position's error is the root mean square, over the vocabulary, of the difference of its logits, as a part
# of the spread of the logits there.  float32: sums in another order than the plain float64 ones.  bfloat16:
# every product's inputs are rounded to 8 bits, and attention here is peaked, which amplifies it at some
# positions tenfold; so the bfloat16 limit of a position is three times what rounding alone does there in the
# plain restatement (its products and kept queries and keys rounded to bfloat16, nothing else changed), and
# no less than three times the median of that over the prompt, nor than FLOOR.
TOL = {"float32": 5e-5}
# (between two ways of cutting a prompt: portions of more than four tokens a request go through the recurrence 16
# tokens at a time, shorter ones token by token, which are two orders of summation)
TOL_BETWEEN = {"float32": 2.5e-5}
FLOOR = 0.03


def to_bfloat16(x):
    return torch.from_numpy(np.asarray(x, dtype=np.float32)).to(torch.bfloat16).to(torch.float64).numpy()


class Limits(dict):
    """The plain logits of every request, name -> [tokens, vocab], with `limit[(name, position)]`."""

    def worst(self, got, ref=None, between=False):
        """The largest error of `got` ((name, position) -> logits), against the plain logits or `ref`, as a part
        of the position's limit, and where."""
        worst, where = 0.0, None
        for (name, pos), row in got.items():
            lim = self.limit[(name, pos)] if self.limit else (TOL_BETWEEN if between else TOL)["float32"]
            e = position_error(row, self[name][pos] if ref is None else ref[(name, pos)]) / lim
            if e >= worst:
                worst, where = e, (name, pos, e * lim)
        return worst, where


def plain_logits(model_dir, reqs, dtype="float32"):
    cfg, w = U.read_config(model_dir), U.plain_weights(model_dir)
    out = Limits({name: P.forward(cfg, w, toks)[0] for name, toks in reqs.items()})
    out.limit = {}
    if dtype == "bfloat16":
        for name, toks in reqs.items():
            with P.coarse_products(to_bfloat16):
                rounded = P.forward(cfg, w, toks)[0]
            e = np.array([position_error(rounded[i], out[name][i]) for i in range(len(toks))])
            for i, x in enumerate(np.maximum(np.maximum(e, np.median(e)) * 3.0, FLOOR)):
                out.limit[(name, i)] = float(x)
    return out


def session(model_dir, dtype, max_tokens, page=16, max_live=4):
    from rust_llm_inference_server_b200.engine.replay import ReplaySession
    return ReplaySession(model_dir, dtype, max_tokens, page, max_live=max_live)


def model_dir(root, which, dtype, cfg=None, seed=None):
    """The model folder of a run: the bfloat16 runs take weights whose routing does not hang on close logits."""
    if dtype == "bfloat16":
        return U.make_dir(root, which + "_settled", cfg or U.CONFIGS[which], U.SEEDS.get(which, 0) if seed is None else seed,
                          edit=U.settle_routing)
    return U.make_dir(root, which, cfg, seed)


# ---- the kernels, one by one -------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden", [40, 96, 1030])
def test_normed_sum_of_stream_and_branches(dtype, hidden):
    from rust_llm_inference_server_b200 import ops
    rng = np.random.default_rng(hidden)
    T = 5
    a, b = dev(rng.standard_normal((T, hidden)) * 3, dtype), dev(rng.standard_normal((T, hidden)) * 0.2, dtype)
    wa, wb, wo = (dev(1 + 0.3 * rng.standard_normal(hidden)) for _ in range(3))
    tol = 3e-6 if dtype == torch.float32 else 0.02
    # the stream times a constant plus the mean of two normed branches, normed
    resid = dev(rng.standard_normal((T, hidden)))
    r0 = host(resid)
    want = P.rms_unit(2.5 * r0 + 0.5 * P.rms_unit(host(a), 1e-4) * host(wa) + 0.5 * P.rms_unit(host(b), 1e-4) * host(wb), 1e-5) * host(wo)
    out = torch.empty((T, hidden), dtype=dtype, device="cuda")
    assert ops.sum_norm(resid, 2.5, [(a, wa, 0.5), (b, wb, 0.5)], wo, 1e-5, out=out, eps_branch=1e-4) is out
    np.testing.assert_allclose(host(resid), want, rtol=0, atol=3e-6)                  # float32 whatever the type
    assert torch.equal(out, resid.to(dtype))                                         # the stream, rounded once
    # one branch taken as it is, no copy asked for
    r0 = host(resid)
    ops.sum_norm(resid, 0.7, [(a, None, 1.0)], wo, 1e-6)
    np.testing.assert_allclose(host(resid), P.rms_unit(0.7 * r0 + host(a), 1e-6) * host(wo), rtol=0, atol=3e-6)
    # no stream and no final norm: the mean of the normed branches
    out.zero_()
    ops.sum_norm(None, 0.0, [(a, wa, 0.5), (b, wb, 0.5)], None, 0.0, out=out, eps_branch=1e-4)
    want = 0.5 * P.rms_unit(host(a), 1e-4) * host(wa) + 0.5 * P.rms_unit(host(b), 1e-4) * host(wb)
    np.testing.assert_allclose(host(out), want, rtol=0, atol=tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,dv", [(4, 24), (1, 16), (3, 64), (2, 200)])
def test_norm_of_every_head_times_gate(dtype, nh, dv):
    from rust_llm_inference_server_b200 import ops
    rng = np.random.default_rng(dv)
    T = 6
    x = dev(rng.standard_normal((T, nh * dv)) * 4)
    w = dev(1 + 0.3 * rng.standard_normal(dv))
    wide = dev(rng.standard_normal((T, nh * dv + 11)) * 2, dtype)
    gate = wide[:, 8:8 + nh * dv]                        # a column slice of wider rows
    out = torch.empty((T, nh * dv), dtype=dtype, device="cuda")
    ops.head_norm_gate(x, w, 1e-5, out, nh, gate=gate, activation="silu")
    want = (P.rms_unit(host(x).reshape(T, nh, dv), 1e-5) * host(w)).reshape(T, -1) * P.silu(host(gate))
    np.testing.assert_allclose(host(out), want, rtol=0, atol=1e-5 if dtype == torch.float32 else 0.05)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,rot,sc", [(4, 2, 32, 16, (4.0, 64, 16.0, 2.0)), (3, 3, 24, 12, (2.0, 32, 4.0, 1.0)), (1, 1, 8, 8, None),
                                          (6, 2, 64, 48, (16.0, 128, 8.0, 0.5)), (2, 1, 128, 64, (8.0, 256, 32.0, 1.0)),
                                          (5, 5, 24, 10, (3.0, 50, 10.0, 1.5))])
def test_rotation_unit_norms_temperature_and_the_paged_write(dtype, H, G, d, rot, sc):
    """Keys that double as values: the cache's value rows hold the keys as projected, its key rows the rotated
    and normed ones.  Positions far from 0, portions that start in the middle of a page."""
    from rust_llm_inference_server_b200 import ops
    rng = np.random.default_rng(d + rot)
    page, n_pages = 8, 140
    st = hand_step([1019, 5, 30], [7, 1, 30], page, n_pages, rng)
    T = st.n_tokens
    lead = 8
    N = lead + H * d + G * d + 8
    proj = dev(rng.standard_normal((T, N)) * 2, dtype)
    kc = torch.full((n_pages, G, page, d), 7.0, dtype=dtype, device="cuda")
    vc = torch.full((n_pages, G, page, d), 7.0, dtype=dtype, device="cuda")
    q_out = torch.empty((T, H * d), dtype=dtype, device="cuda")
    q_off, k_off = lead, lead + H * d
    tol = 2e-5 if dtype == torch.float32 else 0.05
    rd = {"dims": rot, "base": 5000.0}
    if sc:
        rd["scaling"] = dict(zip(("factor", "original", "fast", "slow"), sc))
    freqs, mag = P.blended_frequencies(rd)
    inv = dev(freqs)
    ones = torch.ones((d,), dtype=torch.float32, device="cuda")
    x = host(proj)
    pos = np.asarray(st.host_pos, dtype=np.float64)
    # float32 angles: at position 1,000 an angle is exact to about 1e-4 radians
    want_q = P.rms_unit(P.rotate_adjacent_pairs(x[:, q_off:k_off].reshape(T, H, d), pos, host(inv), mag), 1e-5).reshape(T, -1)
    want_k = P.rms_unit(P.rotate_adjacent_pairs(x[:, k_off:k_off + G * d].reshape(T, G, d), pos, host(inv), mag), 1e-5)
    ops.qk_norm_store(proj, q_off, k_off, k_off, ones, ones, 1e-5, None, 0.0, q_out, kc, vc, st.slots[0], H, G, d, d, page,
                      rotation=(inv, rot, mag), positions=st.positions)
    np.testing.assert_allclose(host(q_out), want_q, rtol=0, atol=max(tol, 3e-4))
    for t in range(T):
        pg = st.host_tables[st.host_seq[t], st.host_pos[t] // page]
        np.testing.assert_allclose(host(kc[pg, :, st.host_pos[t] % page]), want_k[t], rtol=0, atol=max(tol, 3e-4))
        np.testing.assert_allclose(host(vc[pg, :, st.host_pos[t] % page]), x[t, k_off:k_off + G * d].reshape(G, d), rtol=0, atol=0)
    # the temperature, with weights, without rotation: a step at every multiple of `every`, counted from position 1
    qw, kw = dev(1 + 0.5 * rng.standard_normal(d)), dev(1 + 0.5 * rng.standard_normal(d))
    for coef, every in ((0.5, 7), (1.25, 1), (0.3, 1020)):
        ops.qk_norm_store(proj, q_off, k_off, k_off, qw, kw, 1e-5, None, 0.0, q_out, kc, vc, None, H, G, d, d, page,
                          positions=st.positions, q_temp=(coef, every))
        temp = 1.0 + coef * np.log(np.floor((pos + 1) / every) + 1.0)
        want = (P.rms_unit(x[:, q_off:k_off].reshape(T, H, d), 1e-5) * host(qw) * temp[:, None, None]).reshape(T, -1)
        np.testing.assert_allclose(host(q_out), want, rtol=0, atol=tol * max(1.0, float(temp.max())))


def plain_rows(q, keys, vals, scale, st, H, G, window, sinks, slopes):
    """q [T, H, d]; keys/vals: per request the whole context [ctx, G, d | dv]."""
    T = q.shape[0]
    out = np.zeros((T, H, vals[0].shape[-1]))
    for t in range(T):
        b, pos = st.host_seq[t], st.host_pos[t]
        lo = max(0, pos - window + 1) if window else 0
        for h in range(H):
            g = h // (H // G)
            js = np.arange(lo, pos + 1)
            s = keys[b][lo:pos + 1, g] @ q[t, h] * scale
            if slopes is not None:
                s = s - slopes[h] * (pos - js)
            m = max(s.max(), sinks[h]) if sinks is not None else s.max()
            e = np.exp(s - m)
            den = e.sum() + (np.exp(sinks[h] - m) if sinks is not None else 0.0)
            out[t, h] = (e / den) @ vals[b][lo:pos + 1, g]
    return out


SHAPES = [(4, 2, 32, 16, 8), (3, 3, 24, 24, 16), (1, 1, 8, 24, 16), (6, 2, 64, 64, 16), (2, 1, 128, 32, 8),
          (4, 2, 128, 64, 16), (8, 4, 64, 64, 32), (2, 1, 128, 128, 16), (10, 5, 12, 20, 16)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv,page", SHAPES)
def test_attention_windows_sinks_and_slopes(dtype, H, G, d, dv, page):
    """Whole prompts, portions that start in the middle of a page, and single tokens in one launch.  Per head one
    key is made to carry the weight (query and key scaled, the slope's penalty made up for): the first token, a
    page's last and first slot, a key far back, and, with a window, the oldest key inside it and the first
    outside, which must not count however well it matches."""
    from rust_llm_inference_server_b200 import ops
    rng = np.random.default_rng(H * 100 + d)
    ctx = [333, 70, 129, 1, 2, 1100, 65, 150]
    qn = [333, 1, 37, 1, 2, 1, 64, 1]
    n_pages = sum(-(-c // page) for c in ctx) + 3
    st = hand_step(ctx, qn, page, n_pages, rng)
    T = st.n_tokens
    keys = [rng.standard_normal((c, G, d)) for c in ctx]
    vals = [rng.standard_normal((c, G, dv)) for c in ctx]
    scale = 0.9 / np.sqrt(d)
    slopes = P.head_slopes(H)
    sinks = rng.uniform(-2.0, 2.0, H)
    if H > 1:
        sinks[0] = 14.0                                 # head 0 gives nearly everything to its sink
        sinks[1] = -40.0                                # head 1's sink is as good as absent
    tol = 2e-5 if dtype == torch.float32 else 0.03
    out = torch.empty((T, H * dv), dtype=dtype, device="cuda")
    starts = np.concatenate([[0], np.cumsum(qn)])
    marked = [(int(starts[0] + qn[0] - 1), 0), (int(starts[5]), 5), (int(starts[2] + 20), 2), (int(starts[7]), 7),
              (int(starts[6] + 63), 6)]
    for window, use_sinks, use_slopes in ((0, False, True), (72, True, False), (100, True, True), (1, True, False), (0, False, False)):
        q = rng.standard_normal((T, H, d))
        for t, b in marked:
            pos = st.host_pos[t]
            far = [0, page - 1, page, 3 * page, pos // 2, pos - 1, pos]
            if window:
                far = [pos - window + 1, pos - window, pos - window + 1, max(pos - window - 1, 0), pos, pos - window // 2]
                if H == 1:
                    far = [pos - window]
            for h in range(H):
                j = min(max(far[h % len(far)], 0), pos)
                g = h // (H // G)
                boost = 9.0 + (slopes[h] * (pos - j) if use_slopes else 0.0)
                q[t, h] = keys[b][j, g] * (boost / scale / float(keys[b][j, g] @ keys[b][j, g]))
        qd = dev(q.reshape(T, -1), dtype)
        kr = [host(dev(k, dtype)) for k in keys]
        vr = [host(dev(v, dtype)) for v in vals]
        kc, vc = fill_pools(st, kr, vr, page, n_pages, dtype)
        out.fill_(float("nan"))
        sk, sl = (dev(sinks) if use_sinks else None), (dev(slopes) if use_slopes else None)
        ops.attention_biased(qd, kc, vc, out, None, None, st, 0, H, G, d, dv, page, scale, window, sinks=sk, slopes=sl)
        want = plain_rows(host(qd).reshape(T, H, d), kr, vr, scale, st, H, G, window, host(sk) if use_sinks else None,
                          host(sl) if use_slopes else None)
        got = host(out).reshape(T, H, dv)
        err = np.abs(got - want).max(axis=(1, 2))
        assert np.isfinite(got).all() and err.max() <= tol, f"window {window}: row {int(err.argmax())}: {err.max()}"
        if window > 1:
            # the test bites: with the key just outside the window let in, a marked row would differ
            t, b = marked[0]
            moved = plain_rows(host(qd).reshape(T, H, d)[t:t + 1], kr, vr, scale,
                               SimpleNamespace(host_seq=[b], host_pos=[st.host_pos[t]]), H, G, window + 1,
                               host(sk) if use_sinks else None, host(sl) if use_slopes else None)
            assert np.abs(moved[0] - want[t])[min(1, H - 1)].max() > 0.2
    if dtype == torch.bfloat16 and ops.biased_attention_takes_mma(dtype, H, G, d, dv):
        assert ops.launches_by_kernel.get("attention_bias.decode.mma.split") and ops.launches_by_kernel.get("attention_bias.prefill.mma")


def plain_recurrent_rows(x, taps_w, a_log, dt_bias, nh, nqk, d, dv):
    """x [T, C + 2 nh] float64: one request's rows q | k | v | beta logits | decay logits -> o [T, nh, dv]."""
    T, qk = x.shape[0], nqk * d
    C = 2 * qk + nh * dv
    y = P.silu(P.short_conv(x[:, :C], taps_w))
    q, k, v = y[:, :qk].reshape(T, nqk, d), y[:, qk:2 * qk].reshape(T, nqk, d), y[:, 2 * qk:].reshape(T, nh, dv)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * d ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = 1.0 / (1.0 + np.exp(-x[:, C:C + nh]))
    decay = np.exp(-np.exp(a_log) * P.softplus(x[:, C + nh:] + dt_bias))
    o = np.zeros((T, nh, dv))
    for h in range(nh):
        g = h // (nh // nqk)
        o[:, h] = P.delta_rule(q[:, g], k[:, g], v[:, h], beta[:, h], decay[:, h])
    return o


RECURRENCE_SCHEDULES = {
    # portions that go 16 tokens at a time (ending in the middle of a chunk, beside single tokens) and a single token
    "long": ([70, 1, 33, 150, 2, 9], [[(0, 40), (1, 1), (2, 2)], [(0, 1), (2, 31), (3, 5)], [(3, 1), (0, 29), (4, 2)],
                                      [(5, 3), (3, 144)], [(5, 1)], [(5, 5)]]),
    # steps of at most four tokens a request: the token-by-token kernel
    "short": ([7, 1, 6, 12, 2, 9], [[(0, 4), (1, 1), (2, 2)], [(0, 1), (2, 4), (3, 4)], [(3, 4), (0, 2), (4, 2)],
                                    [(5, 3), (3, 4)], [(5, 1)], [(5, 4)], [(5, 1)]]),
}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("portions", ["long", "short"])
@pytest.mark.parametrize("nh,nqk,d,dv,taps", [(4, 2, 16, 24, 3), (1, 1, 8, 16, 1), (3, 1, 24, 16, 5), (2, 1, 64, 32, 4),
                                              (4, 4, 32, 64, 4), (6, 3, 12, 20, 4), (2, 2, 128, 128, 2), (2, 1, 200, 40, 8),
                                              (2, 1, 300, 16, 2)])
def test_recurrence_cut_into_portions_over_slots_that_held_something_else(dtype, portions, nh, nqk, d, dv, taps):
    """Six requests over three state slots: portions of one and two tokens beside long ones, requests that sit
    out a step, a slot taken over by a new request in the step after its owner ended; the slots start full of
    junk.  Every output row against the plain recurrence over the whole request."""
    from rust_llm_inference_server_b200 import ops
    rng = np.random.default_rng(d * 7 + taps)
    lens, schedule = RECURRENCE_SCHEDULES[portions]
    ops.launches_by_kernel.clear()
    C = 2 * nqk * d + nh * dv
    lead, gap = 8, 5
    q_off, b_off = lead, lead + C + gap
    a_off = b_off + nh + 3
    N = -(-(a_off + nh) // 8) * 8
    rows = [np.concatenate([rng.standard_normal((n, a_off)) * 1.5, rng.standard_normal((n, N - a_off)) * 2.0], axis=1) for n in lens]
    rows = [host(dev(r, dtype)) for r in rows]                      # what the kernel reads, exactly
    taps_w = dev(rng.standard_normal((C, taps)) * 0.6 + 0.3)
    a_log, dt_bias = dev(rng.uniform(-1.5, 0.5, nh)), dev(rng.uniform(-1.0, 1.0, nh))
    want = [plain_recurrent_rows(np.concatenate([r[:, q_off:q_off + C], r[:, b_off:b_off + nh], r[:, a_off:a_off + nh]], axis=1),
                                 host(taps_w), host(a_log), host(dt_bias), nh, nqk, d, dv) for r in rows]
    state = torch.full((3, ops.gated_delta_state_floats(nh, nqk, d, dv, taps)), 30.0, dtype=torch.float32, device="cuda")
    free, slot_of, done = [2, 0, 1], {}, {r: 0 for r in range(len(lens))}
    worst = 0.0
    for entries in schedule:
        for r, _ in entries:
            if r not in slot_of:
                slot_of[r] = free.pop()
        ctx = [done[r] + n for r, n in entries]
        st = hand_step(ctx, [n for _, n in entries], 16, sum(-(-c // 16) for c in ctx) + 1, rng)
        st.state_slots = dev([slot_of[r] for r, _ in entries], torch.int32)
        proj = dev(np.concatenate([rows[r][done[r]:done[r] + n] for r, n in entries]), dtype)
        out = torch.full((st.n_tokens, nh * dv), float("nan"), dtype=torch.float32, device="cuda")
        ops.gated_delta(proj, q_off, b_off, a_off, taps_w, a_log, dt_bias, state, out, st, nh, nqk, d, dv, taps, 1e-6, d ** -0.5,
                        chunks=st.n_tokens > 4 * st.n_seqs)
        got, at = host(out).reshape(-1, nh, dv), 0
        for r, n in entries:
            worst = max(worst, float(np.abs(got[at:at + n] - want[r][done[r]:done[r] + n]).max()))
            at += n
            done[r] += n
            if done[r] == lens[r]:
                free.append(slot_of[r])
    assert done == dict(enumerate(lens)) and worst <= 5e-5, worst
    assert ops.launches_by_kernel.get("gated_delta.scan") and bool(ops.launches_by_kernel.get("gated_delta.chunks")) == (portions == "long")
    # the test bites: without the state the later rows differ
    assert portions == "short" or d > 200 or np.abs(want[3][10:] - plain_recurrent_rows(
        np.concatenate([rows[3][10:, q_off:q_off + C], rows[3][10:, b_off:b_off + nh], rows[3][10:, a_off:a_off + nh]], axis=1),
        host(taps_w), host(a_log), host(dt_bias), nh, nqk, d, dv)).max() > 0.05
    ops.check_device_errors()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,E,top,W,I", [(1, 3, 1, 40, 24), (37, 5, 2, 96, 40), (150, 9, 3, 64, 72), (64, 4, 4, 32, 16),
                                          (5, 16, 16, 48, 8), (600, 3, 2, 256, 128)])
def test_routing_by_the_logits_with_softmax_over_the_chosen(dtype, T, E, top, W, I):
    from rust_llm_inference_server_b200 import ops
    rng = np.random.default_rng(T + E)
    x = dev(rng.standard_normal((T, W)), dtype)
    wr = dev(rng.standard_normal((E, W)) * 2 / np.sqrt(W))
    b = rng.standard_normal(E) * 0.5
    b[0] += 2.0                                         # a crowded expert
    b = dev(b)
    st = SimpleNamespace(buffer=hand_step([1], [1], 8, 1, rng).buffer)
    plan = ops.moe_route(x, wr, None, E, top, 1.0, False, st, router_bias=b, softmax_chosen=True)
    idx, wts = P.choose_experts(host(x) @ host(wr).T + host(b), top)
    got_idx, got_w = plan.top_idx.view(T, top).cpu().numpy(), host(plan.top_w).reshape(T, top)
    for t in range(T):
        assert dict(zip(got_idx[t].tolist(), got_w[t])) == pytest.approx(dict(zip(idx[t].tolist(), wts[t])), abs=2e-5)
    np.testing.assert_allclose(got_w.sum(axis=1), 1.0, atol=1e-5)
    wg, wu = (dev(rng.standard_normal((E, I, W)) / np.sqrt(W), dtype) for _ in range(2))
    wd = dev(rng.standard_normal((E, W, I)) / np.sqrt(I), dtype)
    stack = torch.stack([wg.view(E, -1, 4, W), wu.view(E, -1, 4, W)], dim=2).reshape(E, 2 * I, W).contiguous()
    y = ops.moe_down(ops.moe_up(x, stack, plan, 1.0, float("inf"), 0.0, st, 4), wd, plan, st)
    out = torch.empty((T, W), dtype=dtype, device="cuda")
    ops.moe_combine(y, plan, None, out)
    want = np.zeros((T, W))
    for t in range(T):
        for e, g in zip(idx[t], wts[t]):
            want[t] += g * P.gated_expert(host(x)[t], host(wg)[e], host(wu)[e], host(wd)[e])
    np.testing.assert_allclose(host(out), want, rtol=0, atol=3e-5 if dtype == torch.float32 else 0.06)
    ops.check_device_errors()


# ---- whole models ------------------------------------------------------------------------------

_P0 = U.parallel(U.window_attn(2, 1, 16, 0.5, 7, 8, 100.0, (2.0, 16, 4.0, 1.0)), U.delta(2, 1, 8, 12, 3))
ALONE = {
    "slopes_only": U.model(61, 48, 1e-5, 1.7, [U.attention(U.slope_attn(3, 1, 16, 8, 0.3, (0.6, 3)))]),
    "two_branches": U.model(61, 48, 1e-5, 2.0, [_P0]),
    "with_routed": U.model(61, 48, 1e-5, 1.3, [U.attention(U.slope_attn(2, 2, 24, 16, 0.25), U.moe(4, 2, 16))]),
    "run_twice": U.model(61, 48, 1e-6, 2.4, [_P0, U._with(_P0, 0), U._with(_P0, 0)]),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", sorted(ALONE))
def test_each_kind_of_layer_alone(model_root, which, dtype):
    d = model_dir(model_root, which, dtype, ALONE[which], seed=11)
    reqs = requests_for(ALONE[which], [1, 2, 37, 90])
    ref = plain_logits(d, reqs, dtype)
    for fam, steps in (("whole", R.whole_trace(reqs)), ("decode", R.decode_trace(reqs, tail=20)),
                       ("chunks", R.chunk_trace(reqs, seed=2))):
        s = session(d, dtype, R.live_token_peak(steps), 8)
        worst, where = ref.worst(R.collect(s.step, steps))
        assert worst <= 1.0, f"{which} {dtype} {fam}: {worst} of the limit at {where}"


@pytest.mark.parametrize("which", ["A", "D"])
def test_the_stream_after_every_run_of_a_layer(model_root, which):
    """float32: the stream as every block leaves it, a block that runs twice counted each time."""
    d = model_dir(model_root, which, "float32")
    cfg, w = U.read_config(d), U.plain_weights(d)
    toks = requests_for(cfg, [45], seed=4)["r0"]
    want = P.forward(cfg, w, toks)[1]
    s = session(d, "float32", 64, 16)
    seen = []
    for blk in set(s.model.blocks):
        def tapped(*a, _inner=blk.forward, **k):
            r = _inner(*a, **k)
            seen.append(host(r[0]))
            return r
        blk.forward = tapped
    s.step({"step": 0, "entries": [{"id": "x", "tokens": toks, "want": [len(toks) - 1]}], "end": ["x"]})
    assert len(seen) == len(cfg["layers"])
    for i, (got, ref) in enumerate(zip(seen, want)):
        np.testing.assert_allclose(got, ref, rtol=0, atol=2e-4, err_msg=f"after run {i}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which,page,lens", [("A", 16, [1, 50, 97, 200, 64, 17, 2]), ("A", 8, [130, 33, 2, 71, 40]),
                                             ("B", 16, [3, 150, 40, 2, 129, 1]), ("B", 32, [260, 31, 5, 90]),
                                             ("C", 16, [1, 70, 333, 2, 129, 64, 65]), ("C", 8, [200, 31, 5, 400]),
                                             ("D", 16, [90, 1, 33, 150, 2]), ("E", 16, [420, 3, 200, 77])])
def test_all_ways_of_cutting_give_the_plain_logits(model_root, which, page, lens, dtype, monkeypatch):
    from rust_llm_inference_server_b200 import ops
    ops.launches_by_kernel.clear()
    # portions of five tokens and more go through the recurrence's chunk kernels, shorter ones token by token: every
    # family of cuts mixes the two
    monkeypatch.setattr(ops, "GATED_DELTA_CHUNKS_FROM", 5)
    d = model_dir(model_root, which, dtype)
    reqs = requests_for(U.CONFIGS[which], lens, seed=page)
    ref = plain_logits(d, reqs, dtype)
    families = {
        "whole": (R.whole_trace(reqs), 4),
        "decode": (R.decode_trace(reqs, tail=40), 4),
        "chunks": (R.chunk_trace(reqs, seed=3), 4),
        "mixed": (R.mixed_trace(reqs, seed=4), 4),
        "mixed2": (R.mixed_trace(dict(reversed(list(reqs.items()))), seed=5, max_live=2), 2),   # two state slots for all
    }
    results = {}
    for fam, (steps, live) in families.items():
        s = session(d, dtype, R.live_token_peak(steps, max(64, page)), page, max_live=live)
        for pool in s.storage.pools:                         # whatever a page or a slot held before must not matter
            for t in (pool if isinstance(pool, tuple) else (pool,)):
                t.fill_(30.0)
        for state in s.storage.states:
            if state is not None:
                state.fill_(3.0)
        results[fam] = R.collect(s.step, steps)
        assert s.cache.check_invariants() == ""
        assert s.cache.num_free_pages(0) == s.cache.group(0).num_pages, fam
        assert s.cache.num_free_state_slots() == live, fam
        worst, where = ref.worst(results[fam])
        assert worst <= 1.0, f"{which} {dtype} {fam} vs plain: {worst} of the limit at {where}"
    for fam in ("decode", "chunks", "mixed", "mixed2"):
        worst, where = ref.worst(results[fam], results["whole"], between=True)
        assert worst <= 1.0, f"{which} {dtype}: {fam} differs from whole by {worst} of the limit at {where}"
    fast = dtype == "bfloat16" and which in ("C", "E")
    for k in (("attention_bias.decode.mma", "attention_bias.prefill.mma") if fast else ("attention_bias",)) + \
            (("moe_gemm.mma.glu", "moe_gemm.mma.down") if dtype == "bfloat16" and which != "D" else ("moe_gemm.glu", "moe_gemm.down")) + \
            ("qk_norm_store", "qk_norm_store.rot", "gated_delta.prepare", "gated_delta.scan", "gated_delta.gram",
             "gated_delta.chunks", "head_norm_gate", "moe_route",
             "moe_align", "moe_combine"):
        assert ops.launches_by_kernel.get(k), f"never launched {k}; launched {sorted(ops.launches_by_kernel)}"
    assert any(k.startswith("sum_norm") for k in ops.launches_by_kernel)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which,n,tail", [("A", 230, 215), ("B", 180, 170)])
def test_long_decoding_while_the_windows_pass_over_decoded_tokens(model_root, which, n, tail, dtype):
    d = model_dir(model_root, which, dtype)
    reqs = requests_for(U.CONFIGS[which], [n], seed=9)
    ref = plain_logits(d, reqs, dtype)
    steps = R.decode_trace(reqs, tail=tail)             # a page border every 8 tokens; every window slides many times over
    s = session(d, dtype, R.live_token_peak(steps), 8)
    worst, where = ref.worst(R.collect(s.step, steps))
    assert worst <= 1.0, f"{worst} of the limit at {where}"


def plain_greedy(cfg, w, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(np.argmax(P.forward(cfg, w, toks)[0][-1])))
    return toks[len(prompt):]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(model_root, dtype):
    """Prompts of unequal length batched by the scheduler, portions of 16 tokens, decode steps from CUDA
    graphs and launched ahead; two seats, so the later prompts take over pages and state slots."""
    from rust_llm_inference_server_b200 import LLM, SamplingParams
    d = model_dir(model_root, "A", dtype)
    cfg, w = U.read_config(d), U.plain_weights(d)
    prompts = list(requests_for(cfg, [1, 9, 40, 23, 3], seed=12).values())
    llm = LLM(d, dtype=dtype, max_seq_len=128, num_blocks=40, block_size=8, max_num_seqs=2, max_batched_tokens=16)
    outs = llm.generate(prompts, SamplingParams(max_tokens=12))
    for p, o in zip(prompts, outs):
        want = plain_greedy(cfg, w, p, 12)
        assert o.finish_reason == "length" and len(o.token_ids) == 12
        if o.token_ids != want:
            i = next(k for k, (a, b) in enumerate(zip(o.token_ids, want)) if a != b)
            lg = P.forward(cfg, w, p + want[:i])[0][-1]
            gap = lg[want[i]] - lg[o.token_ids[i]]
            assert dtype == "bfloat16" and gap < 0.15, f"parted at token {i} with a gap of {gap}"
    assert llm.engine.cache.check_invariants() == ""


def test_command_line_serves_the_design(tmp_path):
    """random-weights and generate of the command line with a Lanirax folder."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

    def rlis(*args):
        return subprocess.run([sys.executable, os.path.join(root, "bin", "rlis"), *args], capture_output=True,
                              text=True, timeout=600)

    cfg_file = tmp_path / "c.json"
    cfg_file.write_text(json.dumps(U.CONFIGS["A"]))
    d = str(tmp_path / "m")
    r = rlis("random-weights", "--config", str(cfg_file), "--seed", "21", "--out", d)
    assert r.returncode == 0, r.stderr[-2000:]
    cfg, w = U.read_config(d), U.plain_weights(d)
    assert cfg["architecture"] == "Lanirax" and set(w) == set(U.tensor_shapes(cfg))
    prompt = [5, 9, 200, 31, 7]
    r = rlis("generate", "--model", d, "--dtype", "f32", "--prompt-ids", ",".join(map(str, prompt)),
             "--max-tokens", "8", "--max-seq-len", "64", "--kv-cache-gb", "0.001", "--block-size", "8",
             "--max-num-seqs", "2")
    assert r.returncode == 0, r.stderr[-2000:]
    assert [int(t) for t in r.stdout.split()] == plain_greedy(cfg, w, prompt, 8)
