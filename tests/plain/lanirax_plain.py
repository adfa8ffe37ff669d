"""The Lanirax decoder restated plainly in float64 numpy: whole sequences, no cache, no batching, one
function per mechanism.  It shares no code with the package; the tests compare the package against it.

`forward(cfg, w, tokens)` takes the dictionary of a config.json, a dictionary name -> float array of the
checkpoint's tensors, and one sequence of token ids; it returns the logits of every position and the
stream after every layer run.
"""

from __future__ import annotations

import math

import numpy as np


_coarse = [lambda x: x]


class coarse_products:
    """Within this context every matrix product takes its inputs, and leaves its result, through `fn` (the
    rounding of a narrower number type), and so do the queries and keys that attention keeps; everything else
    stays float64.  It models what rounding alone does to the logits: the tests take their tolerance for a
    narrow type from it."""

    def __init__(self, fn):
        self.fn = fn

    def __enter__(self):
        _coarse.append(self.fn)

    def __exit__(self, *exc):
        _coarse.pop()


def kept(x):
    return _coarse[-1](x)


def linear(h, weight, exact_result=False):
    y = kept(h) @ weight.T
    return y if exact_result else kept(y)


def rms_unit(x, eps):
    """x divided by its root mean square over the last axis (eps under the root)."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def silu(z):
    return z / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


# ---- rotation -------------------------------------------------------------------------------------


def blended_frequencies(rot: dict):
    """Frequencies of the rotated pairs and the factor on cos and sin."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    f = np.array([base ** (-2.0 * i / dims) for i in range(half)])
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def pair_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(sc["slow"]))), dims - 1)
    out = np.empty(half)
    for i in range(half):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out[i] = f[i] / factor * ramp + f[i] * (1.0 - ramp)
    return out, 0.1 * math.log(factor) + 1.0


def rotate_adjacent_pairs(x, positions, freqs, mag):
    """x [T, heads, dim]: entries (2i, 2i+1), i < len(freqs), turn by position * freqs[i]; the rest stay."""
    y = x.copy()
    for i, f in enumerate(freqs):
        a = positions * f
        c, s = np.cos(a)[:, None] * mag, np.sin(a)[:, None] * mag
        u, v = x[:, :, 2 * i], x[:, :, 2 * i + 1]
        y[:, :, 2 * i] = u * c - v * s
        y[:, :, 2 * i + 1] = v * c + u * s
    return y


# ---- attention ------------------------------------------------------------------------------------


def masked_attention(q, k, v, scale, window=None, sinks=None, slopes=None):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv].  Query i sees keys j <= i, with a window only
    those with i - j < window.  `sinks` [H]: one more term exp(sink) in the denominator.  `slopes` [H]:
    slope * (i - j) is subtracted from the score."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            lo = 0 if window is None else max(0, i - window + 1)
            js = np.arange(lo, i + 1)
            s = (k[js, g] @ q[i, h]) * scale
            if slopes is not None:
                s = s - slopes[h] * (i - js)
            m = s.max() if sinks is None else max(s.max(), sinks[h])
            e = np.exp(s - m)
            den = e.sum() + (math.exp(sinks[h] - m) if sinks is not None else 0.0)
            out[i, h] = (e / den) @ v[js, g]
    return out


def window_sink_mixer(h, w, p, m, eps):
    """The rotating branch: keys double as values (as projected), rotation on part of a head, then unit
    root mean square, a window and a sink."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = linear(h, w[p + "q"]).reshape(T, H, d)
    k = linear(h, w[p + "k"]).reshape(T, G, d)
    v = k.copy()
    freqs, mag = blended_frequencies(m["rot"])
    pos = np.arange(T, dtype=np.float64)
    q = kept(rms_unit(rotate_adjacent_pairs(q, pos, freqs, mag), eps))
    k = kept(rms_unit(rotate_adjacent_pairs(k, pos, freqs, mag), eps))
    o = masked_attention(q, k, v, m["scale"], window=m["mask"]["size"], sinks=w[p + "sink"])
    return linear(o.reshape(T, -1), w[p + "o"])


def temperature(T, q_temp):
    p = np.arange(T)
    return 1.0 + q_temp["coef"] * np.log(np.floor((p + 1) / q_temp["every"]) + 1.0)


def head_slopes(H):
    return np.array([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)])


def slope_mixer(h, w, p, m, eps):
    """The layer kind without rotation: normed queries and keys, a temperature on the queries that grows
    in steps with the position, and a penalty linear in the distance."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_unit(linear(h, w[p + "q"]).reshape(T, H, d), eps) * w[p + "q.norm"]
    k = rms_unit(linear(h, w[p + "k"]).reshape(T, G, d), eps) * w[p + "k.norm"]
    v = linear(h, w[p + "v"]).reshape(T, G, dv)
    if m.get("q_temp") is not None:
        q = q * temperature(T, m["q_temp"])[:, None, None]
    o = masked_attention(kept(q), kept(k), v, m["scale"], slopes=head_slopes(H))
    return linear(o.reshape(T, -1), w[p + "o"])


# ---- the recurrent branch -------------------------------------------------------------------------


def short_conv(x, taps):
    """x [T, C], taps [C, n]: y[t, c] = sum_j taps[c, j] * x[t - (n - 1 - j), c], zeros before the start."""
    T, C = x.shape
    n = taps.shape[1]
    padded = np.concatenate([np.zeros((n - 1, C)), x], axis=0)
    y = np.zeros((T, C))
    for j in range(n):
        y += padded[j:j + T] * taps[:, j]
    return y


def delta_rule(q, k, v, beta, decay):
    """One head: q, k [T, d], v [T, dv], beta, decay [T].  The state decays, is corrected towards v along
    k, and is read after the write."""
    T, d = q.shape
    S = np.zeros((d, v.shape[1]))
    out = np.zeros((T, v.shape[1]))
    for t in range(T):
        S = decay[t] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + np.outer(k[t], u)
        out[t] = S.T @ q[t]
    return out


def delta_mixer(h, w, p, m, eps):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(linear(h, w[p + "q"]), w[p + "q.conv"])).reshape(T, G, d)
    k = silu(short_conv(linear(h, w[p + "k"]), w[p + "k.conv"])).reshape(T, G, d)
    v = silu(short_conv(linear(h, w[p + "v"]), w[p + "v.conv"])).reshape(T, H, dv)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * d ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = 1.0 / (1.0 + np.exp(-linear(h, w[p + "b"])))
    decay = np.exp(-np.exp(w[p + "A_log"]) * softplus(linear(h, w[p + "a"]) + w[p + "dt_bias"]))
    o = np.zeros((T, H, dv))
    for i in range(H):
        g = i // (H // G)
        o[:, i] = delta_rule(q[:, g], k[:, g], v[:, i], beta[:, i], decay[:, i])
    o = rms_unit(o, eps) * w[p + "norm"] * silu(linear(h, w[p + "g"])).reshape(T, H, dv)
    return linear(o.reshape(T, -1), w[p + "o"])


def parallel_mixer(h, w, p, m, eps):
    a = rms_unit(window_sink_mixer(h, w, p + "left.", m["left"], eps), eps) * w[p + "left.out"]
    b = rms_unit(delta_mixer(h, w, p + "right.", m["right"], eps), eps) * w[p + "right.out"]
    return 0.5 * (a + b)


# ---- feed-forward ---------------------------------------------------------------------------------


def choose_experts(z, top):
    """z [T, n] router logits -> (indices [T, top], weights [T, top]): the `top` largest logits of every row
    (the lower index wins a tie), weighted by the softmax over those logits alone."""
    idx = np.stack([np.array(sorted(range(z.shape[1]), key=lambda e: (-row[e], e))[:top]) for row in z])
    chosen = np.take_along_axis(z, idx, axis=1)
    e_w = np.exp(chosen - chosen.max(axis=1, keepdims=True))
    return idx, e_w / e_w.sum(axis=1, keepdims=True)


def gated_expert(h, gate, up, down):
    return linear(kept(silu(linear(h, gate, True)) * linear(h, up, True)), down, True)


def routed_ff(h, w, p, mlp):
    n, top = mlp["router"]["experts"], mlp["router"]["top"]
    idx, wts = choose_experts(linear(h, w[p + "router"], exact_result=True) + w[p + "router.b"], top)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, g in zip(idx[t], wts[t]):
            q = f"{p}e{e}."
            out[t] += g * gated_expert(h[t], w[q + "gate"], w[q + "up"], w[q + "down"])
    return out


# ---- the model ------------------------------------------------------------------------------------

MIXERS = {"parallel": parallel_mixer, "attention": slope_mixer}


def forward(cfg: dict, w: dict, tokens):
    """Returns (logits [T, vocab], stream after every layer run [runs, T, width])."""
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    x = rms_unit(w["embed"][np.asarray(tokens)], eps) * w["embed.norm"]
    streams = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{layer.get('weights_of', i)}."
        x = rms_unit(alpha * x + MIXERS[layer["type"]](x, w, p + "mix.", layer["mixer"], eps), eps) * w[p + "norm1"]
        if layer.get("mlp") is not None:
            x = rms_unit(alpha * x + routed_ff(x, w, p + "mlp.", layer["mlp"]), eps) * w[p + "norm2"]
        streams.append(x)
    logits = linear(rms_unit(x, eps) * w["final.norm"], w["head"], exact_result=True)
    return logits, np.stack(streams)
