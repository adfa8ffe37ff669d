"""The Rumedra decoder restated plainly in float64 numpy: whole sequences, no cache, no batching, one
function per mechanism.  It shares no code with the package; the tests compare the package against it.

`forward(cfg, w, tokens)` takes the dictionary of a config.json, a dictionary name -> float array of the
checkpoint's tensors, and one sequence of token ids; it returns the logits of every position and the
stream after every layer.
"""

from __future__ import annotations

import math

import numpy as np


_coarse = [lambda x: x]


class coarse_products:
    """Within this context every matrix product takes its inputs, and leaves its result, through `fn` (the
    rounding of a narrower number type), and so do the queries, keys and values that attention keeps;
    everything else stays float64.  It models what rounding alone does to the logits: the tests take their
    tolerance for a narrow type from it."""

    def __init__(self, fn):
        self.fn = fn

    def __enter__(self):
        _coarse.append(self.fn)

    def __exit__(self, *exc):
        _coarse.pop()


def kept(x):
    return _coarse[-1](x)


def linear(h, weight, bias=None, exact_result=False):
    y = kept(h) @ weight.T
    if bias is not None:
        y = y + bias
    return y if exact_result else kept(y)


def rms_unit(x, eps):
    """x divided by its root mean square over the last axis (eps under the root)."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, weight, eps):
    return rms_unit(x, eps) * weight


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


# ---- rotation -------------------------------------------------------------------------------------


def rotary_frequencies(rot: dict):
    """f_i = base^(-2i / dims), i < dims / 2; with `scaling`, by wavelength 2 pi / f: short ones (below
    original / high) keep f, long ones (above original / low) get f / factor, the ones between a blend
    that is linear in original / wavelength."""
    dims = int(rot["dims"])
    i = np.arange(dims // 2, dtype=np.float64)
    f = float(rot["base"]) ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if sc is None:
        return f
    factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
    out = np.empty_like(f)
    for n, fi in enumerate(f):
        wavelength = 2.0 * math.pi / fi
        if wavelength < orig / high:
            out[n] = fi
        elif wavelength > orig / low:
            out[n] = fi / factor
        else:
            s = (orig / wavelength - low) / (high - low)
            out[n] = (1.0 - s) * fi / factor + s * fi
    return out


def rotate(x, positions, rot: dict):
    """x [T, heads, d]: entry i of the first `dims` turns with entry i + dims / 2 by position * f_i."""
    dims = int(rot["dims"])
    half = dims // 2
    f = rotary_frequencies(rot)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]          # [T, half]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    out = x.copy()
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


# ---- the left branch: sliding-window attention with an output gate ---------------------------------


def window_attention(h, w, p, m, positions):
    """Grouped-query attention over the last `mask.size` positions (the query's own included), biased
    projections, rotation of part of each head, scores times `scale`, softmax, sigmoid gate, projection."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = linear(h, w[p + "q"], w[p + "q.b"]).reshape(T, H, d)
    k = linear(h, w[p + "k"], w[p + "k.b"]).reshape(T, G, d)
    v = linear(h, w[p + "v"], w[p + "v.b"]).reshape(T, G, dv)
    q, k = kept(rotate(q, positions, m["rot"])), kept(rotate(k, positions, m["rot"]))
    size = int(m["mask"]["size"])
    out = np.zeros((T, H, dv))
    for hd in range(H):
        g = hd // (H // G)
        for i in range(T):
            lo = max(0, i - size + 1)
            s = (k[lo:i + 1, g] @ q[i, hd]) * float(m["scale"])
            e = np.exp(s - s.max())
            out[i, hd] = (e / e.sum()) @ v[lo:i + 1, g]
    gate = sigmoid(linear(h, w[p + "g"]))
    return linear(out.reshape(T, H * dv) * gate, w[p + "o"])


# ---- the right branch: retention --------------------------------------------------------------------


def retention(h, w, p, m, positions, eps):
    """S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t per head (scores as they are, nothing exponentiated or
    normalised); q and k rotated, k times dim^(-1/2); o divided by its root mean square, gated by silu, projected."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = rotate(linear(h, w[p + "q"]).reshape(T, H, d), positions, m["rot"])
    k = rotate(linear(h, w[p + "k"]).reshape(T, H, d), positions, m["rot"]) * d ** -0.5
    v = linear(h, w[p + "v"]).reshape(T, H, dv)
    o = np.zeros((T, H, dv))
    for hd in range(H):
        S = np.zeros((d, dv))
        for t in range(T):
            S = float(m["decay"][hd]) * S + np.outer(k[t, hd], v[t, hd])
            o[t, hd] = S.T @ q[t, hd]
    o = rms_unit(o, eps).reshape(T, H * dv)
    return linear(o * silu(linear(h, w[p + "g"])), w[p + "o"])


def parallel_mixer(h, w, p, m, positions, eps):
    left = window_attention(h, w, p + "left.", m["left"], positions)
    right = retention(h, w, p + "right.", m["right"], positions, eps)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


# ---- the recurrence with one gate a channel that keeps f and writes 1 - f ---------------------------


def hgrn2(h, w, p, m, eps):
    """f = l + (1 - l) sigmoid(W_f h + b) per head and channel; S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T;
    o_t = S_t^T q_t with q = silu(W_q h); each head normed over its value width with one shared weight."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(linear(h, w[p + "q"])).reshape(T, H, d)
    v = linear(h, w[p + "v"]).reshape(T, H, dv)
    lower = w[p + "lower"]
    f = (lower + (1.0 - lower) * sigmoid(linear(h, w[p + "f"], w[p + "f.b"]))).reshape(T, H, d)
    o = np.zeros((T, H, dv))
    for hd in range(H):
        S = np.zeros((d, dv))
        for t in range(T):
            S = f[t, hd][:, None] * S + np.outer(1.0 - f[t, hd], v[t, hd])
            o[t, hd] = S.T @ q[t, hd]
    o = rms_norm(o, w[p + "norm"], eps).reshape(T, H * dv)
    return linear(o, w[p + "o"])


# ---- feed-forwards ------------------------------------------------------------------------------------


def gated_ff(h, w, p, act):
    return linear(act(linear(h, w[p + "gate"])) * linear(h, w[p + "up"]), w[p + "down"])


def relu(z):
    return np.maximum(z, 0.0)


def route(h, w, p, r):
    """(chosen router outputs [T, top], weights [T, top]).  Softmax over all router outputs; the correction
    only chooses; only outputs of the `keep` groups with the largest member can be chosen; weights are
    the chosen scores over their sum, times `scale`."""
    z = h @ w[p + "router"].T                       # float64: the router is not a coarse product
    z = z - z.max(axis=-1, keepdims=True)
    s = np.exp(z) / np.exp(z).sum(axis=-1, keepdims=True)
    choice = s + w[p + "correction"]
    T, N = s.shape
    count, keep = int(r["groups"]["count"]), int(r["groups"]["keep"])
    per = N // count
    best = choice.reshape(T, count, per).max(axis=-1)
    idx = np.zeros((T, int(r["top"])), dtype=np.int64)
    wt = np.zeros((T, int(r["top"])))
    for t in range(T):
        groups = sorted(range(count), key=lambda g: (-best[t, g], g))[:keep]
        allowed = [e for e in range(N) if e // per in groups]
        chosen = sorted(allowed, key=lambda e: (-choice[t, e], e))[:int(r["top"])]
        idx[t] = chosen
        sc = s[t, chosen]
        wt[t] = sc / (sc.sum() + 1e-20) * float(r["scale"])
    return idx, wt


def routed_ff(h, w, p, mlp):
    r = mlp["router"]
    n_real = int(r["experts"])
    idx, wt = route(kept(h), w, p, r)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(idx[t], wt[t]):
            if e >= n_real:                         # an identity expert hands the input back
                out[t] += a * kept(h[t])
            else:
                out[t] += a * gated_ff(h[t:t + 1], w, f"{p}e{e}.", silu)[0]
    if mlp.get("shared") is not None:
        out = out + gated_ff(h, w, p + "shared.", silu)
    return kept(out)


# ---- the model ----------------------------------------------------------------------------------------


def forward(cfg: dict, w: dict, tokens, start: int = 0):
    """(logits [T, vocab], stream after every layer [layers, T, width])."""
    eps = float(cfg["norm"]["eps"])
    positions = np.arange(start, start + len(tokens))
    x = w["embed"][np.asarray(tokens)] * float(cfg["embedding"]["scale"])
    streams = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = rms_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "hgrn2":
            x = x + hgrn2(h, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "parallel":
            x = x + parallel_mixer(h, w, p + "mix.", layer["mixer"], positions, eps)
        else:
            raise ValueError(layer["type"])
        mlp = layer.get("mlp")
        if mlp is not None:
            h = rms_norm(x, w[p + "norm2"], eps)
            if mlp["kind"] == "dense":
                x = x + gated_ff(h, w, p + "mlp.", relu)
            else:
                x = x + routed_ff(h, w, p + "mlp.", mlp)
        streams.append(x.copy())
    h = rms_norm(x, w["final.norm"], eps)
    return linear(h, w["embed"], exact_result=True), np.stack(streams)
