"""Small Lanirax configurations and weights for the tests.  The weights are drawn here (not by the package's
random-weights mode) so that attention is peaked, sinks weigh as much as a key, decays are neither 0 nor 1
and the convolutions' taps all count: a key that is one position off a window's edge, a sink that is left
out, a lost state or convolution tail moves the logits far beyond rounding."""

from __future__ import annotations

import json
import os

import numpy as np
import torch


def slope_attn(heads, kv_heads, dim, vdim, scale, q_temp=None):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if q_temp is not None:
        out["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return out


def window_attn(heads, kv_heads, dim, scale, window, rot_dims, base, scaling=None):
    rot = {"dims": rot_dims, "base": base}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale, "mask": {"size": window},
            "rot": rot}


def delta(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def attention(mixer, mlp=None, weights_of=None):
    out = {"type": "attention", "mixer": mixer, "mlp": mlp}
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


def parallel(left, right, mlp=None, weights_of=None):
    out = {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp}
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


def model(vocab, width, eps, alpha, layers):
    return {"architecture": "Lanirax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "postln_alpha": alpha,
            "layers": layers}


def _with(layer, weights_of):
    out = json.loads(json.dumps(layer))
    out["weights_of"] = weights_of
    return out


_A0 = attention(slope_attn(4, 2, 32, 16, 0.35, (0.7, 5)), moe(5, 2, 24))
_A1 = parallel(window_attn(4, 2, 32, 0.4, 9, 16, 10000.0, (4.0, 64, 16.0, 2.0)), delta(4, 2, 16, 24, 3), moe(6, 3, 40))
_C0 = parallel(window_attn(6, 2, 64, 0.2, 100, 48, 50000.0, (16.0, 128, 8.0, 0.5)), delta(2, 1, 64, 32, 4), moe(4, 2, 64))
CONFIGS = {
    # both kinds of layer, each also run a second time with the first run's tensors (a cache and a state of their
    # own), a layer without feed-forward, a window shorter than a page, rotation of half a head, a temperature
    # that steps every five positions, more value heads than query/key heads in the recurrent branch
    "A": model(211, 96, 1e-5, 1.8, [
        _A0, _A1, _with(_A0, 0), parallel(window_attn(2, 2, 16, 0.6, 21, 16, 300.0), delta(2, 2, 8, 8, 2)), _with(_A1, 1)]),
    # ones: one head, one expert a token, one tap (no convolution tail), a window of one (a token sees itself and
    # the sink), a factor on the stream of 1, rotation of the whole head without a blend, no temperature
    "B": model(97, 64, 1e-6, 1.0, [
        parallel(window_attn(1, 1, 8, 0.9, 1, 8, 100.0), delta(1, 1, 8, 16, 1), moe(3, 1, 16)),
        attention(slope_attn(1, 1, 8, 24, 0.8)),
        parallel(window_attn(3, 3, 24, 0.45, 40, 12, 20000.0, (2.0, 32, 4.0, 1.0)), delta(3, 1, 24, 16, 5), moe(2, 2, 24)),
        attention(slope_attn(3, 3, 24, 48, 0.4, (0.25, 1)), moe(3, 1, 16)),
    ]),
    # head sizes that the tensor-core kernels take, a window beyond a tile of keys, experts the grouped product takes
    "C": model(157, 128, 1e-5, 3.0, [
        _C0,
        attention(slope_attn(2, 1, 128, 32, 0.09, (0.5, 64)), moe(6, 2, 32)),
        attention(slope_attn(4, 2, 128, 64, 0.08, (1.5, 200))),
        _with(_C0, 0),
    ]),
    # sizes that are multiples of nothing in particular
    "D": model(131, 100, 1e-5, 2.2, [
        parallel(window_attn(5, 5, 24, 0.4, 33, 10, 777.0, (3.0, 50, 10.0, 1.5)), delta(6, 3, 12, 20, 4), moe(7, 3, 36)),
        attention(slope_attn(10, 5, 12, 20, 0.5, (0.3, 17)), moe(7, 4, 20)),
    ]),
    # wide experts over long prompts
    "E": model(89, 256, 1e-5, 2.0, [
        attention(slope_attn(4, 2, 64, 64, 0.16, (0.4, 100)), moe(4, 2, 128)),
        parallel(window_attn(2, 1, 128, 0.1, 150, 64, 10000.0, (8.0, 256, 32.0, 1.0)), delta(4, 4, 32, 64, 4), moe(3, 1, 256)),
    ]),
}
SEEDS = {"A": 3, "B": 5, "C": 8, "D": 13, "E": 21}


def tensor_shapes(cfg: dict) -> dict:
    """Names and shapes, listed here independently of the package."""
    W = cfg["width"]
    out = {"embed": (cfg["vocab"], W), "embed.norm": (W,), "final.norm": (W,), "head": (cfg["vocab"], W)}
    for i, l in enumerate(cfg["layers"]):
        if "weights_of" in l:
            continue
        p = f"l{i}."
        out[p + "norm1"] = (W,)
        if l["type"] == "attention":
            m, q = l["mixer"], p + "mix."
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({q + "q": (H * d, W), q + "k": (G * d, W), q + "v": (G * dv, W), q + "q.norm": (d,),
                        q + "k.norm": (d,), q + "o": (W, H * dv)})
        else:
            m, q = l["mixer"]["left"], p + "mix.left."
            H, G, d = m["heads"], m["kv_heads"], m["dim"]
            out.update({q + "q": (H * d, W), q + "k": (G * d, W), q + "sink": (H,), q + "o": (W, H * d),
                        p + "mix.left.out": (W,), p + "mix.right.out": (W,)})
            m, q = l["mixer"]["right"], p + "mix.right."
            H, G, d, dv, n = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            out.update({q + "q": (G * d, W), q + "k": (G * d, W), q + "v": (H * dv, W), q + "q.conv": (G * d, n),
                        q + "k.conv": (G * d, n), q + "v.conv": (H * dv, n), q + "b": (H, W), q + "a": (H, W),
                        q + "A_log": (H,), q + "dt_bias": (H,), q + "g": (H * dv, W), q + "norm": (dv,),
                        q + "o": (W, H * dv)})
        x = l["mlp"]
        if x is None:
            continue
        out[p + "norm2"] = (W,)
        for e in range(x["router"]["experts"]):
            ff = x["expert"]["ff"]
            out.update({f"{p}mlp.e{e}.gate": (ff, W), f"{p}mlp.e{e}.up": (ff, W), f"{p}mlp.e{e}.down": (W, ff)})
        out.update({p + "mlp.router": (x["router"]["experts"], W), p + "mlp.router.b": (x["router"]["experts"],)})
    return out


def draw_weights(cfg: dict, seed: int) -> dict:
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.split(".")[-1]
        if last == "sink":
            x = rng.uniform(-1.0, 3.0, shape)              # as heavy as a well-matched key
        elif last == "conv":
            x = rng.standard_normal(shape) * 0.6 + 0.3     # every tap counts
        elif last == "A_log":
            x = rng.uniform(-1.5, 0.5, shape)
        elif last == "dt_bias":
            x = rng.uniform(-1.0, 1.0, shape)
        elif last == "b" and len(shape) == 1:
            x = rng.standard_normal(shape) * 0.5           # router bias
        elif last == "router":
            x = rng.standard_normal(shape) * 2.0 / np.sqrt(shape[1])
        elif len(shape) == 2:
            std = 2.0 if last in ("a", "b") else (1.5 if name == "embed" else 1.0)
            x = rng.standard_normal(shape) * std / np.sqrt(shape[1])
        elif name.endswith("q.norm") or name.endswith("k.norm"):
            x = 1.0 + 0.3 * rng.standard_normal(shape)
        else:
            x = 1.0 + 0.2 * rng.standard_normal(shape)
        out[name] = torch.from_numpy(np.asarray(x, dtype=np.float32)).to(torch.bfloat16)
    return out


def settle_routing(w: dict) -> None:
    """Router biases so far apart, under routers so small, that the choice of experts no longer hangs on the
    logits: a choice that flips under bfloat16 rounding would move a token's logits as much as a fault does, and
    some tokens' logits always lie close.  The weights of the chosen experts still follow the logits.  The
    bfloat16 runs of whole models use such weights; the float32 runs, and the routing kernel's own test in both
    types, choose by the logits."""
    for name in [n for n in w if n.endswith(".router.b")]:
        n = w[name].shape[0]
        order = np.random.default_rng(n + len(name)).permutation(n)
        w[name] = torch.from_numpy((order * 3.0).astype(np.float32)).to(torch.bfloat16)
        w[name[:-2]] = (w[name[:-2]].float() * 0.25).to(torch.bfloat16)


def make_dir(root: str, which: str, cfg: dict | None = None, seed: int | None = None, edit=None) -> str:
    """Writes config.json and model.safetensors (with the `safetensors` package) once; `edit(weights)` may
    change tensors before they are stored."""
    from safetensors.torch import save_file
    out = os.path.join(root, f"lanirax_{which}")
    if not os.path.isfile(os.path.join(out, "model.safetensors")):
        os.makedirs(out, exist_ok=True)
        cfg = cfg or CONFIGS[which]
        w = draw_weights(cfg, SEEDS.get(which, 0) if seed is None else seed)
        if edit is not None:
            edit(w)
        save_file({k: v.contiguous() for k, v in w.items()}, os.path.join(out, "model.safetensors"))
        with open(os.path.join(out, "config.json"), "w") as f:
            json.dump(cfg, f)
    return out


def plain_weights(model_dir: str) -> dict:
    from safetensors.torch import load_file
    return {k: v.to(torch.float64).numpy() for k, v in load_file(os.path.join(model_dir, "model.safetensors")).items()}


def read_config(model_dir: str) -> dict:
    with open(os.path.join(model_dir, "config.json")) as f:
        return json.load(f)
