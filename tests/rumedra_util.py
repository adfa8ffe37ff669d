"""Small Rumedra configurations and weights for the tests.  The weights are drawn here (not by the package's
random-weights mode) so that attention is peaked, the forget gates spread between their lower bounds and 1, the
retention's state matters and every router output gets chosen: a key that is one position off a window's edge, a
lost state, a bias, gate, group or identity expert that is left out moves the logits far beyond rounding."""

from __future__ import annotations

import json
import os

import numpy as np
import torch


def window_attn(heads, kv_heads, dim, vdim, scale, window, rot_dims, base, scaling=None):
    rot = {"dims": rot_dims, "base": base}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": window},
            "rot": rot}


def retention(heads, dim, vdim, decay, rot_dims, base):
    assert len(decay) == heads
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay), "rot": {"dims": rot_dims, "base": base}}


def parallel(left, right, left_scale, right_scale, mlp=None):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale,
                                          "right_scale": right_scale}, "mlp": mlp}


def hgrn2(heads, dim, vdim, mlp=None):
    return {"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim}, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, identity=0, groups=(1, 1), scale=1.0, shared=None):
    out = {"kind": "moe", "expert": {"ff": ff},
           "router": {"experts": experts, "top": top, "identity": identity, "scale": scale,
                      "groups": {"count": groups[0], "keep": groups[1]}}}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


def model(vocab, width, eps, emb_scale, layers):
    return {"architecture": "Rumedra", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "embedding": {"scale": emb_scale}, "layers": layers}


CONFIGS = {
    # both kinds of layer with all three kinds of feed-forward and none; a window shorter than a page; rotation of half a
    # head on the left and of part of a head on the right; values wider and narrower than keys; two of three groups
    # kept; identity experts
    "A": model(211, 96, 1e-5, 2.0, [
        hgrn2(3, 8, 16, moe(7, 3, 24, identity=2, groups=(3, 2), scale=1.6, shared=16)),
        parallel(window_attn(4, 2, 32, 16, 0.3, 9, 16, 10000.0, (4.0, 1.0, 4.0, 64)),
                 retention(2, 16, 24, (0.9, 0.97), 8, 500.0), 0.7, 0.4, dense(40)),
        parallel(window_attn(2, 2, 16, 24, 0.5, 21, 16, 300.0), retention(3, 8, 8, (0.8, 0.95, 0.99), 8, 100.0), 1.2, 0.6),
        hgrn2(2, 24, 8, dense(64)),
        parallel(window_attn(6, 3, 16, 16, 0.4, 40, 8, 5000.0, (2.0, 0.5, 2.0, 32)),
                 retention(2, 32, 16, (0.93, 0.999), 32, 20000.0), 0.5, 0.5, moe(4, 2, 16, groups=(2, 1), scale=0.8)),
    ]),
    # ones: one head, one expert a token, one group, a window of one (a token sees itself only), an embedding scale of 1,
    # a scale of 1 on both branches and on the router, no identity experts, no shared expert, a decay of 1
    "B": model(97, 64, 1e-6, 1.0, [
        parallel(window_attn(1, 1, 8, 8, 0.9, 1, 8, 100.0), retention(1, 8, 16, (1.0,), 8, 50.0), 1.0, 1.0, moe(3, 1, 16)),
        hgrn2(1, 8, 24),
        parallel(window_attn(3, 3, 24, 8, 0.45, 40, 12, 20000.0, (2.0, 1.0, 3.0, 32)),
                 retention(3, 24, 16, (0.5, 0.9, 0.99), 12, 1000.0), 0.3, 1.1, moe(2, 2, 24, identity=1)),
        hgrn2(4, 4, 4, moe(5, 2, 8, identity=3, groups=(4, 1), scale=2.0, shared=24)),
    ]),
    # head sizes that the tensor-core kernels take, a window beyond a tile of keys, heads of 128
    "C": model(157, 128, 1e-5, 3.0, [
        parallel(window_attn(4, 2, 64, 32, 0.16, 100, 48, 50000.0, (16.0, 1.0, 8.0, 128)),
                 retention(2, 64, 32, (0.95, 0.995), 64, 10000.0), 0.6, 0.5, moe(6, 2, 32, identity=2, groups=(4, 3), shared=32)),
        hgrn2(2, 64, 64, dense(128)),
        parallel(window_attn(2, 1, 128, 64, 0.09, 150, 64, 10000.0), retention(1, 128, 128, (0.99,), 32, 10000.0), 0.8, 0.3),
        parallel(window_attn(4, 4, 64, 128, 0.12, 70, 64, 1000.0, (8.0, 2.0, 6.0, 256)),
                 retention(4, 16, 16, (0.9, 0.95, 0.98, 0.999), 16, 100.0), 0.5, 0.7, dense(128)),
    ]),
    # sizes that are multiples of nothing in particular
    "D": model(131, 100, 1e-5, 1.7, [
        parallel(window_attn(5, 5, 24, 20, 0.4, 33, 10, 777.0, (3.0, 1.5, 5.0, 50)), retention(3, 12, 20, (0.9, 0.97, 0.99), 6, 333.0),
                 0.9, 0.35, moe(7, 3, 36, identity=2, groups=(3, 2), scale=1.3, shared=20)),
        hgrn2(5, 12, 20, dense(52)),
    ]),
    # wide experts and wide dense units over long prompts
    "E": model(89, 320, 1e-5, 2.5, [
        hgrn2(4, 16, 64, moe(3, 1, 256, identity=1, groups=(2, 1), scale=1.7, shared=128)),
        parallel(window_attn(4, 2, 64, 64, 0.16, 130, 32, 10000.0, (6.0, 1.0, 3.0, 256)), retention(2, 64, 128, (0.97, 0.999), 64, 10000.0),
                 0.7, 0.45, dense(384)),
    ]),
    # larger: one key/value head for eight query heads of 128 with values of 96, many experts in many groups, more identity
    # experts than half the experts, a layer of each kind without a feed-forward of its own kind before it
    "F": model(1000, 384, 1e-6, 4.0, [
        parallel(window_attn(8, 1, 128, 96, 0.09, 64, 64, 1e6, (8.0, 1.0, 4.0, 2048)), retention(3, 96, 48, (0.9, 0.99, 0.999), 32, 1e4), 0.5, 0.5,
                 moe(32, 6, 64, identity=0, groups=(8, 4), scale=2.0, shared=128)),
        hgrn2(4, 48, 80, dense(512)),
        hgrn2(2, 96, 96, moe(10, 2, 48, identity=6, groups=(4, 2), scale=1.0)),
        parallel(window_attn(8, 1, 128, 96, 0.09, 64, 64, 1e6, (8.0, 1.0, 4.0, 2048)), retention(3, 96, 48, (0.9, 0.99, 0.999), 32, 1e4), 0.5, 0.5),
    ]),
}
SEEDS = {"A": 3, "B": 5, "C": 8, "D": 13, "E": 21, "F": 34}


def tensor_shapes(cfg: dict) -> dict:
    """Names and shapes, listed here independently of the package."""
    W = cfg["width"]
    out = {"embed": (cfg["vocab"], W), "final.norm": (W,)}
    for i, l in enumerate(cfg["layers"]):
        p = f"l{i}."
        out[p + "norm1"] = (W,)
        if l["type"] == "hgrn2":
            m, q = l["mixer"], p + "mix."
            H, d, dv = m["heads"], m["dim"], m["vdim"]
            out.update({q + "q": (H * d, W), q + "f": (H * d, W), q + "f.b": (H * d,), q + "lower": (H * d,),
                        q + "v": (H * dv, W), q + "norm": (dv,), q + "o": (W, H * dv)})
        else:
            m, q = l["mixer"]["left"], p + "mix.left."
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({q + "q": (H * d, W), q + "q.b": (H * d,), q + "k": (G * d, W), q + "k.b": (G * d,),
                        q + "v": (G * dv, W), q + "v.b": (G * dv,), q + "g": (H * dv, W), q + "o": (W, H * dv)})
            m, q = l["mixer"]["right"], p + "mix.right."
            H, d, dv = m["heads"], m["dim"], m["vdim"]
            out.update({q + "q": (H * d, W), q + "k": (H * d, W), q + "v": (H * dv, W), q + "g": (H * dv, W),
                        q + "o": (W, H * dv)})
        x = l["mlp"]
        if x is None:
            continue
        out[p + "norm2"] = (W,)
        q = p + "mlp."
        if x["kind"] == "dense":
            units = [(q, x["ff"])]
        else:
            r = x["router"]
            units = [(f"{q}e{e}.", x["expert"]["ff"]) for e in range(r["experts"])]
            if x.get("shared") is not None:
                units.append((q + "shared.", x["shared"]["ff"]))
            n_out = r["experts"] + r.get("identity", 0)
            out.update({q + "router": (n_out, W), q + "correction": (n_out,)})
        for u, ff in units:
            out.update({u + "gate": (ff, W), u + "up": (ff, W), u + "down": (W, ff)})
    return out


def draw_weights(cfg: dict, seed: int) -> dict:
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.split(".")[-1]
        if last == "lower":
            x = rng.uniform(0.05, 0.9, shape)              # the bounds differ by channel and are felt
        elif last == "correction":
            x = rng.standard_normal(shape) * 0.2           # as large as the scores themselves
        elif last == "b":
            x = rng.standard_normal(shape) * 0.7           # biases of projections and of the forget gate
        elif last == "router":
            x = rng.standard_normal(shape) * 2.0 / np.sqrt(shape[1])
        elif len(shape) == 2:
            std = 2.0 if last == "f" else (1.5 if name == "embed" else 1.0)
            x = rng.standard_normal(shape) * std / np.sqrt(shape[1])
        else:
            x = 1.0 + 0.2 * rng.standard_normal(shape)
        out[name] = torch.from_numpy(np.asarray(x, dtype=np.float32)).to(torch.bfloat16)
    return out


def settle_routing(w: dict) -> None:
    """Corrections so far apart that the choice of experts no longer hangs on the scores: a choice that flips under
    bfloat16 rounding would move a token's logits as much as a fault does, and some tokens' scores always lie close.
    The weights of the chosen experts still follow the scores.  The bfloat16 runs of whole models use such weights;
    the float32 runs, and the routing kernel's own test in both types, choose by the scores."""
    for name in [n for n in w if n.endswith(".correction")]:
        n = w[name].shape[0]
        order = np.random.default_rng(n + len(name)).permutation(n)
        w[name] = torch.from_numpy((order * 3.0).astype(np.float32)).to(torch.bfloat16)


def make_dir(root: str, which: str, cfg: dict | None = None, seed: int | None = None, edit=None) -> str:
    """Writes config.json and model.safetensors (with the `safetensors` package) once; `edit(weights)` may
    change tensors before they are stored."""
    from safetensors.torch import save_file
    out = os.path.join(root, f"rumedra_{which}")
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
