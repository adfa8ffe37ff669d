#!/usr/bin/env python3
"""Benchmark of the decode step (and a 2,048-token prefill) at the Llama-3.2-1B layer sizes with
random bfloat16 weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  `value` is decoded tokens a second over K device-timed decode steps of a
batch of 8 requests whose context ends at 4,096 tokens (teacher-forced random tokens, sampler
kernel included, CUDA events around the K steps).  `e2e` is the same quantity through the Python
entry point (`LLM.stream`): every step uploads its inputs from pinned host memory and reads its
sampled token ids back.  Method after the reference's own micro-benchmarks (warm-up, then a timed
loop with a device synchronisation on both sides, crates/model/examples/decode_profile.rs:47-62).
"""

from __future__ import annotations

import argparse
import json
import os
import shutil
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# configs[2] of the baseline description: Llama-3.2-1B sizes
CONFIG_1B = {
    "architectures": ["LlamaForCausalLM"],
    "hidden_size": 2048, "intermediate_size": 8192, "num_hidden_layers": 16,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64, "vocab_size": 128256,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "max_position_embeddings": 131072,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "tie_word_embeddings": True,
}
CONTEXT = 4096
PREFILL_TOKENS = 2048
SEED = 4

# configs[3] and configs[4] of the baseline description: Llama-3.2-3B and Llama-3.1-8B sizes
CONFIG_3B = {
    "architectures": ["LlamaForCausalLM"],
    "hidden_size": 3072, "intermediate_size": 8192, "num_hidden_layers": 28,
    "num_attention_heads": 24, "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 128256,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "max_position_embeddings": 131072,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "tie_word_embeddings": True,
}
CONFIG_8B = {
    "architectures": ["LlamaForCausalLM"],
    "hidden_size": 4096, "intermediate_size": 14336, "num_hidden_layers": 32,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 128256,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "max_position_embeddings": 131072,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "tie_word_embeddings": False,
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks() -> tuple:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            out = dict(FALLBACK_PEAKS)
            for k in out:
                if isinstance(d.get(k), (int, float)):
                    out[k] = float(d[k])
            return out, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


def _peak_extra(key: str, default: float) -> float:
    """A number of MEASURED_PEAKS.json beyond the three peaks (the SMs' maximum clock)."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            v = json.load(f).get(key)
        return float(v) if isinstance(v, (int, float)) else default
    except (OSError, ValueError):
        return default


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.lines: list = []

    def start(self):
        exe = shutil.which("nvidia-smi")
        if not exe:
            return
        idx = os.environ.get("CUDA_VISIBLE_DEVICES", "0").split(",")[0] or "0"
        try:
            self.proc = subprocess.Popen(
                [exe, "-i", idx, f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(sm)}


def weight_bytes(cfg: dict, n_layers: int, elem: int = 2) -> int:
    """What a decode step reads of the weights: every layer's matrices and the LM head's table once
    (the embedding rows of a few tokens do not count)."""
    H, I, d = cfg["hidden_size"], cfg["intermediate_size"], cfg["head_dim"]
    nh, nkv, V = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["vocab_size"]
    per_layer = ((nh + 2 * nkv) * d * H + H * nh * d + 3 * I * H) * elem + 2 * H * 4
    return n_layers * per_layer + V * H * elem + H * 4


def kv_bytes_per_token(cfg: dict, n_layers: int, elem: int = 2) -> int:
    return 2 * n_layers * cfg["num_key_value_heads"] * cfg["head_dim"] * elem


def prefill_flops(cfg: dict, n_layers: int, T: int) -> float:
    H, I, d = cfg["hidden_size"], cfg["intermediate_size"], cfg["head_dim"]
    nh, nkv, V = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["vocab_size"]
    proj = 2.0 * T * ((nh + 2 * nkv) * d * H + H * nh * d + 3 * I * H)
    attn = 2.0 * T * T * nh * d          # causal: QK^T and PV over half the square
    return n_layers * (proj + attn) + 2.0 * V * H


def run_reference(args) -> int:
    print(json.dumps({
        "impl": "reference",
        "unavailable": "the reference is a Rust workspace on the candle library (Metal kernels); pip finds "
                       "neither setup.py nor pyproject.toml and there is no cargo/rustc here, so it cannot be installed",
    }))
    return 0


def decode_run(llm, B: int, steps: int, warmup: int, ctx_end: int, torch, fill: bool = True, clocks=None):
    """Device-timed decode: B requests, each step one teacher-forced token per request and the
    sampler kernel; the last step's context is `ctx_end`.  Returns (ms per step, launches per step)."""
    import numpy as np
    from rust_llm_inference_server_b200.engine import StepEntry
    from rust_llm_inference_server_b200.ops import profile

    eng = llm.engine
    runner, cache = eng.runner, eng.cache
    V = llm.model.spec.vocab_size
    rng = np.random.default_rng(B)
    total = warmup + steps
    ctx0 = ctx_end - total
    ids = list(range(10_000, 10_000 + B))
    for sid in ids:
        assert cache.acquire_state_slot(sid) >= 0
        assert cache.reserve(sid, ctx_end), "cache pool too small for the benchmark"
    # fill the cache up to ctx0 with a prompt cut into portions of at most 2,048 tokens
    for sid in ids:
        pos = 0 if fill else ctx0      # (profiler captures skip the fill: the pages then hold zeros)
        while pos < ctx0:
            n = min(2048, ctx0 - pos)
            runner.step([StepEntry(sid, rng.integers(0, V, size=n).tolist(), pos, [])])
            pos += n
    params = torch.zeros((B, 2), dtype=torch.int32, device=llm.model.device)     # greedy rows
    out_ids = torch.empty((B,), dtype=torch.int32, device=llm.model.device)
    toks = rng.integers(0, V, size=(total, B))
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    launches = 0
    if clocks is not None:          # sample clocks over the warm-up and the timed steps only
        clocks.start()
        time.sleep(0.5)             # let nvidia-smi come up before anything is timed
    for i in range(total):
        if i == warmup:
            torch.cuda.synchronize()
            if profile.enabled:
                profile.take_report()       # the table covers the timed steps only
            l0 = runner.launches
            start.record()
        logits = runner.step([StepEntry(sid, [int(toks[i, b])], ctx0 + i, [0]) for b, sid in enumerate(ids)])
        runner.sample(logits, params, out_ids)
    end.record()
    torch.cuda.synchronize()
    launches = runner.launches - l0
    ms = start.elapsed_time(end) / steps
    for sid in ids:
        cache.free(sid)
    return ms, launches / steps


def percentile(xs, q):
    if not xs:
        return None
    xs = sorted(xs)
    return xs[min(len(xs) - 1, int(round(q / 100.0 * (len(xs) - 1))))]


def serve_poisson(llm, prompts, outputs, arrivals, torch):
    """Feeds requests to the engine loop as their arrival times come (wall clock) and steps it
    until all have finished.  Returns per-request time to first token (from the intended arrival),
    the gaps between a request's tokens, and the wall time from the first arrival to the last token."""
    from rust_llm_inference_server_b200 import SamplingParams
    eng = llm.engine
    n = len(prompts)
    first, last, gaps, done = {}, {}, [], {}
    nxt = 0
    rid_of = {}
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    while len(done) < n:
        now = time.perf_counter() - t0
        while nxt < n and arrivals[nxt] <= now:
            rid = eng.add_request(prompts[nxt], SamplingParams(max_tokens=outputs[nxt], ignore_eos=True))
            rid_of[rid] = nxt
            nxt += 1
        if not eng.has_work():
            time.sleep(max(0.0, min(0.001, arrivals[nxt] - now)))
            continue
        finished = eng.step()
        t = time.perf_counter() - t0
        for rid in eng.last_step.new_tokens:
            i = rid_of[rid]
            if i not in first:
                first[i] = t - arrivals[i]
            else:
                gaps.append(t - last[i])
            last[i] = t
        for o in finished:
            done[rid_of[o.request_id]] = o
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    return first, gaps, wall, done


def workload_3b(args, torch, np) -> dict:
    """configs[3]: 64 requests, prompts U[128, 2048], outputs U[64, 512], seeded Poisson arrivals,
    prompts cut into portions of 512 tokens, through `LLMEngine.add_request` / `step` (the numbers
    the reference publishes for its server sweep, README.md:187-191,208-214: throughput, time to the
    first token, time between tokens, preemptions, prefix hits)."""
    from rust_llm_inference_server_b200 import LLM
    cfg = dict(CONFIG_3B)
    n_full = cfg["num_hidden_layers"]
    cfg["num_hidden_layers"] = args.layers or n_full
    rng = np.random.default_rng(5)
    n = 64
    p_lens = rng.integers(128, 2049, size=n).tolist()
    o_lens = rng.integers(64, 513, size=n).tolist()
    prompts = [rng.integers(0, cfg["vocab_size"], size=k).tolist() for k in p_lens]
    arrivals = np.cumsum(rng.exponential(1.0 / args.rate, size=n)).tolist()
    page = 16
    kv_tok = kv_bytes_per_token(cfg, cfg["num_hidden_layers"])
    runs = {}
    llm = None
    for name, pool_tokens in (("roomy", sum(p + o for p, o in zip(p_lens, o_lens)) + 64 * page),
                              ("tight", 40960)):
        del llm
        torch.cuda.empty_cache()
        llm = LLM.from_random(cfg, 5, dtype="bfloat16", on_device=True, max_seq_len=2048 + 512 + page,
                              num_blocks=pool_tokens // page, block_size=page, max_num_seqs=64,
                              max_batched_tokens=512, prefix_caching=True)
        # warm-up outside the timed region: a stream of the same shape (other tokens), so that the
        # decode shapes the run meets have their graphs; a serving process does this once at start-up
        w_prompts = [rng.integers(0, cfg["vocab_size"], size=k).tolist() for k in p_lens]
        serve_poisson(llm, w_prompts, o_lens, arrivals, torch)
        st = llm.engine.stats
        pre0, hit0, steps0 = st.preemptions, st.prefix_hit_tokens, st.steps
        clocks = ClockSampler()
        clocks.start()
        time.sleep(0.3)
        first, gaps, wall, done = serve_poisson(llm, prompts, o_lens, arrivals, torch)
        clk = clocks.stop()
        assert all(len(done[i].token_ids) == o_lens[i] for i in range(n))
        out_tokens = sum(o_lens)
        ms = lambda x: None if x is None else round(x * 1e3, 2)
        runs[name] = {
            "pool_tokens": pool_tokens, "pool_gb": round(pool_tokens * kv_tok / 2 ** 30, 2),
            "wall_s": round(wall, 3), "output_tokens_per_s": round(out_tokens / wall, 1),
            "total_tokens_per_s": round((out_tokens + sum(p_lens)) / wall, 1),
            "ttft_ms_p50": ms(percentile(list(first.values()), 50)), "ttft_ms_p99": ms(percentile(list(first.values()), 99)),
            "itl_ms_p50": ms(percentile(gaps, 50)), "itl_ms_p99": ms(percentile(gaps, 99)),
            "preemptions": st.preemptions - pre0, "prefix_hit_tokens": st.prefix_hit_tokens - hit0,
            "steps": st.steps - steps0, "failed": st.failed_requests, "clocks": clk,
        }
    return {
        "workload": "3b", "metric": "continuous batching, 64 requests in a Poisson stream (Llama-3.2-3B sizes, random bf16 weights)",
        "impl": "ours", "dtype": "bf16", "n_gpus": 1,
        "data": "synthetic: uniform-random token ids, random-init weights N(0,0.02) seed 5 (device generator)",
        "config": {"model": "llama-3.2-3b-sizes", "layers": cfg["num_hidden_layers"], "layers_in_config": n_full,
                   "hidden": 3072, "heads": 24, "kv_heads": 8, "head_dim": 128, "intermediate": 8192, "vocab": 128256,
                   "requests": n, "prompt_tokens": sum(p_lens), "output_tokens": sum(o_lens), "rate_per_s": args.rate,
                   "max_batched_tokens": 512, "max_num_seqs": 64, "page_size": page, "prefix_caching": True},
        "runs": runs,
    }


def workload_8b(args, torch, np) -> dict:
    """configs[4]: 32 requests with 2,048-token prompts, a quarter of which share their first
    1,024 tokens, through the engine (prefill in portions, prefix reuse), then device-timed decode
    steps of the 32 whose context ends at 8,192 tokens, against the HBM roofline."""
    from rust_llm_inference_server_b200 import LLM, SamplingParams
    cfg = dict(CONFIG_8B)
    n_full = cfg["num_hidden_layers"]
    n_layers = args.layers or n_full
    cfg["num_hidden_layers"] = n_layers
    pk, pk_src = peaks()
    rng = np.random.default_rng(6)
    B, ctx, page = 32, 8192, 16
    llm = LLM.from_random(cfg, 6, dtype="bfloat16", on_device=True, max_seq_len=ctx + page,
                          num_blocks=B * (ctx + page) // page + 64, block_size=page, max_num_seqs=B,
                          max_batched_tokens=2048, prefix_caching=True)
    V = cfg["vocab_size"]
    shared = rng.integers(0, V, size=1024).tolist()
    prompts = [(shared + rng.integers(0, V, size=1024).tolist()) if i % 4 == 0 else rng.integers(0, V, size=2048).tolist()
               for i in range(B)]
    sp = SamplingParams(max_tokens=16, ignore_eos=True)
    llm.generate([rng.integers(0, V, size=300).tolist()], SamplingParams(max_tokens=4, ignore_eos=True))   # warm-up
    st = llm.engine.stats
    hit0 = st.prefix_hit_tokens
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = llm.generate(prompts, sp)
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    assert all(len(o.token_ids) == 16 for o in outs)
    engine_part = {"prompt_tokens": 2048 * B, "prefix_hit_tokens": st.prefix_hit_tokens - hit0, "wall_s": round(wall, 3),
                   "prompt_tokens_per_s": round(2048 * B / wall, 1), "preemptions": st.preemptions}
    steps = min(args.steps, 64)
    clocks = ClockSampler()
    ms, launches = decode_run(llm, B, steps, args.warmup, ctx, torch, clocks=clocks)
    clk = clocks.stop()
    mean_ctx = ctx - steps / 2
    step_bytes = weight_bytes(cfg, n_layers) + B * mean_ctx * kv_bytes_per_token(cfg, n_layers)
    achieved = step_bytes / (ms / 1e3) / 1e9
    return {
        "workload": "8b", "metric": "decode tokens/s, batch 32, context 8192 (Llama-3.1-8B sizes, random bf16 weights)",
        "value": round(B / (ms / 1e3), 1), "unit": "tokens/s", "ms_per_step": round(ms, 4), "steps": steps, "warmup": args.warmup,
        "impl": "ours", "dtype": "bf16", "n_gpus": 1,
        "data": "synthetic: uniform-random token ids, random-init weights N(0,0.02) seed 6 (device generator)",
        "config": {"model": "llama-3.1-8b-sizes", "layers": n_layers, "layers_in_config": n_full, "hidden": 4096,
                   "heads": 32, "kv_heads": 8, "head_dim": 128, "intermediate": 14336, "vocab": V, "tied": False,
                   "global_batch": B, "seq_len": ctx, "page_size": page, "kv_dtype": "bf16"},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk_src,
                     "bytes_per_step": int(step_bytes)},
        "prompts_through_the_engine": engine_part, "gpu_launches": int(round(launches * steps)), "clocks": clk,
    }


def workload_1b_fp32(args, torch, np) -> dict:
    """The true 32-bit path at the 1B sizes: a 2,048-token prefill and decode steps of a batch of 8
    at a context of 4,096 (FFMA products, float32 cache and attention; no tensor cores)."""
    from rust_llm_inference_server_b200 import LLM
    from rust_llm_inference_server_b200.engine import StepEntry
    cfg = dict(CONFIG_1B)
    n_full = cfg["num_hidden_layers"]
    n_layers = args.layers or n_full
    cfg["num_hidden_layers"] = n_layers
    B, ctx, page = 8, CONTEXT, 16
    llm = LLM.from_random(cfg, SEED, dtype="float32", on_device=True, max_seq_len=ctx + page,
                          num_blocks=B * (ctx + page) // page + 64, block_size=page, max_num_seqs=B,
                          max_batched_tokens=2048, prefix_caching=False)
    runner, cache = llm.engine.runner, llm.engine.cache
    rng = np.random.default_rng(0)
    pre = []
    for it in range(4):
        sid = 500 + it
        cache.acquire_state_slot(sid)
        assert cache.reserve(sid, PREFILL_TOKENS)
        toks = rng.integers(0, cfg["vocab_size"], size=PREFILL_TOKENS).tolist()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        runner.step([StepEntry(sid, toks, 0, [PREFILL_TOKENS - 1])])
        e.record()
        torch.cuda.synchronize()
        pre.append(s.elapsed_time(e))
        cache.free(sid)
    prefill_ms = statistics.median(pre[1:])
    steps = min(args.steps, 32)
    clocks = ClockSampler()
    ms, launches = decode_run(llm, B, steps, args.warmup, ctx, torch, clocks=clocks)
    clk = clocks.stop()
    pk, pk_src = peaks()
    step_bytes = weight_bytes(cfg, n_layers, 4) + B * (ctx - steps / 2) * kv_bytes_per_token(cfg, n_layers, 4)
    achieved = step_bytes / (ms / 1e3) / 1e9
    return {
        "workload": "1b-fp32", "metric": "decode tokens/s, batch 8, context 4096, true float32 path (Llama-3.2-1B sizes)",
        "value": round(B / (ms / 1e3), 1), "unit": "tokens/s", "ms_per_step": round(ms, 4), "steps": steps, "warmup": args.warmup,
        "impl": "ours", "dtype": "fp32", "n_gpus": 1,
        "config": {"model": "llama-3.2-1b-sizes", "layers": n_layers, "layers_in_config": n_full, "global_batch": B,
                   "seq_len": ctx, "page_size": page, "kv_dtype": "fp32"},
        "prefill": {"value": round(PREFILL_TOKENS / (prefill_ms / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(prefill_ms, 3),
                    "tflops": round(prefill_flops(cfg, n_layers, PREFILL_TOKENS) / (prefill_ms / 1e3) / 1e12, 2)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk_src},
        "gpu_launches": int(round(launches * steps)), "clocks": clk,
    }


def lasapel_config(width: int, vocab: int = 32000) -> dict:
    """Four Lasapel layers at a real model's proportions: heads of 128, a latent of 512 with 64
    rotated entries, a query latent of 3/4 of the width, feed-forwards of four widths."""
    H = width // 128
    rot = {"dims": 64, "base": 10000.0, "scaling": {"factor": 40.0, "original": 4096, "fast": 32.0, "slow": 1.0}}
    lat = {"heads": H, "dim": 128, "rot_dim": 64, "vdim": 128, "q_rank": 3 * width // 4, "kv_rank": 512,
           "scale": (128 + 64) ** -0.5, "rot": rot}
    lin = {"heads": H, "dim": 128, "vdim": 128, "decay": [1.0 - 2.0 ** (-5 - 3 * h / max(1, H - 1)) for h in range(H)]}
    mlp = {"kind": "dense", "ff": 4 * width}
    return {"architecture": "Lasapel", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "layers": [
        {"type": "lightning", "mixer": lin, "mlp": mlp}, {"type": "latent_attention", "mixer": lat, "mlp": mlp},
        {"type": "lightning", "mixer": lin, "mlp": None}, {"type": "latent_attention", "mixer": dict(lat, kv_from=1), "mlp": mlp}]}


def llama_config_like(width: int, vocab: int = 32000) -> dict:
    """The closest existing model at the same width and depth: heads of 64, four query heads a key
    head, a gated feed-forward of the same parameter count as the dense one of four widths (8/3)."""
    return {"architectures": ["LlamaForCausalLM"], "hidden_size": width, "intermediate_size": width * 8 // 3 // 128 * 128,
            "num_hidden_layers": 4, "num_attention_heads": width // 64, "num_key_value_heads": width // 256,
            "head_dim": 64, "vocab_size": vocab, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
            "max_position_embeddings": 131072, "tie_word_embeddings": False}


def prefill_run(llm, tokens: int, iters: int, warmup: int, torch, np) -> float:
    """Median device time (ms) of one prompt of `tokens` tokens run whole, logits at its last place."""
    from rust_llm_inference_server_b200.engine import StepEntry
    rng = np.random.default_rng(1)
    V, cache, runner = llm.model.spec.vocab_size, llm.engine.cache, llm.engine.runner
    times = []
    for it in range(warmup + iters):
        sid = 700 + it
        cache.acquire_state_slot(sid)
        assert cache.reserve(sid, tokens)
        toks = rng.integers(0, V, size=tokens).tolist()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        runner.step([StepEntry(sid, toks, 0, [tokens - 1])])
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
        cache.free(sid)
    return statistics.median(times[warmup:])


class _KernelStep:
    """The device arrays of a step that the mixers' kernels read, for requests given as (tokens cached
    before, tokens now); every request gets pages of its own in shuffled order."""

    def __init__(self, reqs, page, torch, np, tile=64):
        dev = lambda x: torch.as_tensor(np.asarray(x), dtype=torch.int32).cuda().contiguous()
        lens = [n for _, n in reqs]
        cu = np.cumsum([0] + lens)
        pages = [-(-(s + n) // page) for s, n in reqs]
        perm = np.random.default_rng(0).permutation(sum(pages))
        tables = np.full((len(reqs), max(pages)), -1, dtype=np.int32)
        k = 0
        for b, m in enumerate(pages):
            tables[b, :m] = perm[k:k + m]
            k += m
        self.n_pages, self.n_tokens, self.n_seqs = int(sum(pages)), int(cu[-1]), len(reqs)
        self.block_tables = [dev(tables)]
        self.positions = dev(np.concatenate([np.arange(s, s + n) for s, n in reqs]))
        self.seq_of_token = dev(np.concatenate([np.full(n, b) for b, (_, n) in enumerate(reqs)]))
        self.cu_seqlens, self.ctx_lens = dev(cu), dev([s + n for s, n in reqs])
        self.state_slots = dev(list(range(len(reqs))))
        dec = [b for b, (_, n) in enumerate(reqs) if n == 1]
        self.n_decode, self.dec_seqs, self.dec_rows = len(dec), dev(dec), dev([cu[b] for b in dec])
        self.max_decode_ctx = max([reqs[b][0] + 1 for b in dec], default=0)
        self.max_ctx_len = max(s + n for s, n in reqs)
        tiles = [(b, t0) for b, (_, n) in enumerate(reqs) if n > 1 for t0 in range(0, n, tile)]
        self.n_prefill_tiles, self.n_prefill_tokens = len(tiles), sum(n for _, n in reqs if n > 1)
        self.prefill_tiles = dev(np.asarray(tiles).reshape(-1, 2)) if tiles else None
        self._bufs, self._torch = {}, torch

    def buffer(self, name, shape, dtype):
        key = (name, tuple(shape), dtype)
        if key not in self._bufs:
            self._bufs[key] = self._torch.empty(tuple(shape), dtype=dtype, device="cuda")
        return self._bufs[key]


def _graph_time_us(fn, torch, iters: int = 20) -> float:
    """Device time of one call of `fn` replayed from a CUDA graph (no host time between its kernels),
    L2 flushed before every replay."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    total = 0.0
    for _ in range(iters):
        flush.zero_()
        s.record()
        g.replay()
        e.record()
        torch.cuda.synchronize()
        total += s.elapsed_time(e)
    return total / iters * 1e3


def mixer_kernel_rooflines(width: int, B: int, ctx: int, T: int, pk: dict, torch, np) -> dict:
    """The mixers' kernels alone at the sizes of `lasapel_config(width)` and `llama_config_like(width)`:
    {name: {"us", "ideal_us", "frac"}}.  Ideal: bytes that must move over the measured copy bandwidth, or
    FLOPs over the measured bfloat16 GEMM rate (attention over prompts), or float32 FMAs over the FFMA
    rate of the SMs at their maximum clock (the recurrence over prompts, which is float32 by design)."""
    from rust_llm_inference_server_b200 import ops
    hbm, tf = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    ffma = sms * 128 * 2 * pk.get("sm_max_mhz", 1965.0) * 1e6
    page, H, rank, rot, d = 16, width // 128, 512, 64, 128
    dk = rank + rot
    nh, nkv, hd = width // 64, width // 256, 64
    bf, out = torch.bfloat16, {}
    rnd = lambda *shape: torch.randn(*shape, device="cuda") * 0.3

    def row(name, us, ideal_s):
        out[name] = {"us": round(us, 1), "ideal_us": round(ideal_s * 1e6, 1), "frac": round(ideal_s * 1e6 / us, 3)}

    for kind, reqs in (("decode", [(ctx - 1, 1)] * B), ("prefill", [(0, T)])):
        st = _KernelStep(reqs, page, torch, np)
        n, keys = st.n_tokens, (B * ctx if kind == "decode" else T * (T + 1) // 2)
        cache, qa = rnd(st.n_pages, 1, page, dk).to(bf), rnd(n, H * dk).to(bf)
        o, sinks = torch.empty(n, H * rank, dtype=bf, device="cuda"), torch.zeros(H, device="cuda")
        us = _graph_time_us(lambda: ops.attention_latent(qa, cache, o, st, 0, H, rank, page, 0.07, sinks, 0), torch)
        row(f"latent_attention_{kind}", us, max(B * ctx * dk * 2 / hbm, 2 * H * keys * (dk + rank) / tf) if kind == "decode"
            else 2 * H * keys * (dk + rank) / tf)
        kc, vc, q = rnd(st.n_pages, nkv, page, hd).to(bf), rnd(st.n_pages, nkv, page, hd).to(bf), rnd(n, nh * hd).to(bf)
        o2 = torch.empty_like(q)
        us = _graph_time_us(lambda: ops.attention(q, kc, vc, o2, st, 0, nh, nkv, hd, page, 0.125, 0), torch)
        row(f"gqa_attention_{kind}", us, B * ctx * nkv * hd * 2 * 2 / hbm if kind == "decode" else 2 * nh * keys * 2 * hd / tf)
        proj = rnd(n, 2 * H * d + 2 * H * d).to(bf)
        state, decay = torch.zeros(len(reqs), H, d, d, device="cuda"), torch.full((H,), 0.97, device="cuda")
        o3 = torch.empty(n, H * d, device="cuda")
        us = _graph_time_us(lambda: ops.lightning_scan(proj, 0, H * d, 2 * H * d, o3, state, decay, st, H, d, d), torch)
        row(f"recurrence_{kind}", us, B * H * d * d * 4 * 2 / hbm if kind == "decode" else 2 * 2 * T * H * d * d / ffma)
    return out


def workload_lasapel(args, torch, np) -> dict:
    """Prefill (one 2,048-token prompt) and decode (batch 8, context 4,096) of four Lasapel layers
    at two widths beside four Llama layers of the same width, random bfloat16 weights; then the
    stages of one step by CUDA-event spans (eager launches: host time between kernels is in them), and
    the mixers' kernels alone, replayed from CUDA graphs, against their rooflines."""
    from rust_llm_inference_server_b200 import LLM
    from rust_llm_inference_server_b200.ops import profile
    pk, pk_src = peaks()
    pk["sm_max_mhz"] = _peak_extra("sm_max_mhz", 1965.0)
    B, ctx, page, T = args.batch, args.context, 16, PREFILL_TOKENS
    steps = min(args.steps, 64)
    out = {"workload": "lasapel", "metric": "prefill and decode tokens/s of four layers, Lasapel beside Llama at equal width",
           "unit": "tokens/s", "impl": "ours", "dtype": "bf16", "n_gpus": 1, "steps": steps, "warmup": args.warmup,
           "data": "synthetic: uniform-random token ids, random-init weights (device generator)",
           "config": {"global_batch": B, "seq_len": ctx, "prefill_tokens": T, "page_size": page, "layers": 4},
           "peaks": dict(pk, source=pk_src), "sizes": {}}
    clocks = ClockSampler()
    clocks.start()
    for width in (1024, 2048):
        row = {}
        for name, cfg in (("lasapel", lasapel_config(width)), ("llama", llama_config_like(width))):
            llm = LLM.from_random(cfg, 8, dtype="bfloat16", on_device=True, max_seq_len=ctx + page,
                                  num_blocks=B * (ctx + page) // page + 64, block_size=page, max_num_seqs=B,
                                  max_batched_tokens=max(2048, B), prefix_caching=False)
            pre = prefill_run(llm, T, 5, 3, torch, np)
            ms, launches = decode_run(llm, B, steps, args.warmup, ctx, torch)
            profile.enable(True)                      # the same two steps by stages (eager, events around each)
            prefill_run(llm, T, 3, 2, torch, np)
            profile.take_report()
            prefill_run(llm, T, 3, 0, torch, np)
            pre_stages = {k: round(v[0] / 3 * 1e3, 1) for k, v in profile.take_report().items()}
            decode_run(llm, B, 8, 4, ctx, torch, fill=False)
            dec_stages = {k: round(v[0] / 8 * 1e3, 1) for k, v in profile.take_report().items()}
            profile.enable(False)
            row[name] = {"prefill_tokens_per_s": round(T / (pre / 1e3), 1), "prefill_ms": round(pre, 3),
                         "decode_tokens_per_s": round(B / (ms / 1e3), 1), "decode_ms_per_step": round(ms, 4),
                         "launches_per_decode_step": launches,
                         "weight_bytes": int(sum(p.numel() * p.element_size() for p in _model_tensors(llm.model))),
                         "prefill_stage_us": pre_stages, "decode_stage_us": dec_stages}
            del llm
            torch.cuda.empty_cache()
        row["rooflines"] = mixer_kernel_rooflines(width, B, ctx, T, pk, torch, np)
        out["sizes"][f"width{width}"] = row
    out["clocks"] = clocks.stop()
    head = out["sizes"]["width2048"]["lasapel"]
    out["value"] = head["decode_tokens_per_s"]
    out["ms_per_step"] = head["decode_ms_per_step"]
    out["gpu_launches"] = int(round(head["launches_per_decode_step"] * steps))
    return out


def gavodra_config(width: int, vocab: int = 32000) -> dict:
    """Four Gavodra layers at a real model's proportions: heads of 64 with four query heads a key head (as
    the Llama layers beside them), a bias table of 48 rows reaching 128 positions back, one dense gated
    feed-forward of 8/3 widths and three routed ones (32 experts of half a width, 4 a token, beside a shared
    one of half a width: 2.5 widths of feed-forward a token)."""
    H = width // 64
    mix = {"heads": H, "kv_heads": max(1, H // 4), "dim": 64, "vdim": 64, "scale": 0.125, "bias_max": 128, "v_mix": True,
           "bias_rows": 48}
    moe = {"kind": "moe", "expert": {"ff": width // 2, "limit": 7.0}, "router": {"experts": 32, "top": 4, "scale": 2.5},
           "shared": {"ff": width // 2, "limit": 7.0}}
    dense = {"kind": "dense", "ff": width * 8 // 3 // 128 * 128, "limit": 7.0}
    return {"architecture": "Gavodra", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "residual_mult": 0.5,
            "embedding": {"scale": 8.0}, "logit_scale": 0.5, "logit_softcap": 30.0,
            "layers": [{"type": "attention", "mixer": mix, "mlp": m} for m in (dense, moe, moe, moe)]}


def gavodra_kernel_rooflines(width: int, B: int, ctx: int, T: int, pk: dict, torch, np) -> dict:
    """The new kernels alone at the sizes of `gavodra_config(width)`, each beside the like kernel of the Llama
    layers: {name: {"us", "ideal_us", "frac"}}.  Ideal: bytes that must move over the measured copy bandwidth
    (single tokens) or FLOPs over the measured bfloat16 GEMM rate (prompts)."""
    from rust_llm_inference_server_b200 import ops
    hbm, tf = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    page, nh, nkv, hd = 16, width // 64, max(1, width // 256), 64
    E, top, ff = 32, 4, width // 2
    bf, out = torch.bfloat16, {}
    rnd = lambda *shape: torch.randn(*shape, device="cuda") * 0.3

    def row(name, us, ideal_s):
        out[name] = {"us": round(us, 1), "ideal_us": round(ideal_s * 1e6, 1), "frac": round(ideal_s * 1e6 / us, 3)}

    bias = rnd(129, nh).contiguous()
    for kind, reqs in (("decode", [(ctx - 1, 1)] * B), ("prefill", [(0, T)])):
        st = _KernelStep(reqs, page, torch, np)
        st.n_prefill_tokens = st.n_prefill_tokens if kind == "prefill" else 0
        n, keys = st.n_tokens, (B * ctx if kind == "decode" else T * (T + 1) // 2)
        kc, vc, q = rnd(st.n_pages, nkv, page, hd).to(bf), rnd(st.n_pages, nkv, page, hd).to(bf), rnd(n, nh * hd).to(bf)
        gate = rnd(n, nh + 8).to(bf)[:, :nh]
        o = torch.empty_like(q)
        ideal = B * ctx * nkv * hd * 2 * 2 / hbm if kind == "decode" else 2 * nh * keys * 2 * hd / tf
        us = _graph_time_us(lambda: ops.attention_biased(q, kc, vc, o, bias, gate, st, 0, nh, nkv, hd, hd, page, 0.125, 0), torch)
        row(f"biased_attention_{kind}", us, ideal)
        us = _graph_time_us(lambda: ops.attention(q, kc, vc, o, st, 0, nh, nkv, hd, page, 0.125, 0), torch)
        row(f"gqa_attention_{kind}", us, ideal)
        # the routed products (route + sort + both products + the weighted sum) beside Llama's gated
        # feed-forward products at the same number of feed-forward columns a token (top * ff)
        x = rnd(n, width).to(bf)
        wr, corr = rnd(E, width).contiguous(), rnd(E).contiguous()
        wgu, wd = rnd(E, 2 * ff, width).to(bf), rnd(E, width, ff).to(bf)     # gate and linear rows in blocks of 4
        y = torch.empty(n, width, dtype=bf, device="cuda")

        def routed():
            plan = ops.moe_route(x, wr, corr, E, top, 2.5, False, st)
            act = ops.moe_up(x, wgu, plan, 1.702, 7.0, 1.0, st, 4)
            return ops.moe_combine(ops.moe_down(act, wd, plan, st), plan, None, y)
        used = min(E, n * top)
        flops = 2.0 * n * top * 3 * ff * width
        ideal = used * 3 * ff * width * 2 / hbm if kind == "decode" else flops / tf
        row(f"routed_ff_{kind}", _graph_time_us(routed, torch), ideal)
        I = top * ff
        wgu = torch.stack([rnd(I // 4, 4, width), rnd(I // 4, 4, width)], dim=1).reshape(2 * I, width).to(bf).contiguous()
        wdn = rnd(width, I).to(bf)

        def gated():
            if n <= ops.STREAM_GEMM_ROWS:
                return ops.linear(ops.stream_gemm(x, wgu, swiglu4=True), wdn)
            return ops.linear(ops.gemm_tcgen05(x, wgu, "swiglu4"), wdn)
        row(f"gated_ff_{kind}", _graph_time_us(gated, torch), 3 * I * width * 2 / hbm if kind == "decode" else flops / tf)
    return out


def workload_gavodra(args, torch, np) -> dict:
    """Prefill (one 2,048-token prompt) and decode (batch 8, context 4,096) of four Gavodra layers at two
    widths beside four Llama layers of the same width, random bfloat16 weights; then the stages of one step
    by CUDA-event spans (eager launches), and the new kernels alone, replayed from CUDA graphs, against
    their rooflines beside Llama's like kernels."""
    from rust_llm_inference_server_b200 import LLM
    from rust_llm_inference_server_b200.ops import profile
    pk, pk_src = peaks()
    B, ctx, page, T = args.batch, args.context, 16, PREFILL_TOKENS
    steps = min(args.steps, 64)
    out = {"workload": "gavodra", "metric": "prefill and decode tokens/s of four layers, Gavodra beside Llama at equal width",
           "unit": "tokens/s", "impl": "ours", "dtype": "bf16", "n_gpus": 1, "steps": steps, "warmup": args.warmup,
           "data": "synthetic: uniform-random token ids, random-init weights (device generator)",
           "config": {"global_batch": B, "seq_len": ctx, "prefill_tokens": T, "page_size": page, "layers": 4},
           "peaks": dict(pk, source=pk_src), "sizes": {}}
    clocks = ClockSampler()
    clocks.start()
    for width in (1024, 2048):
        row = {}
        for name, cfg in (("gavodra", gavodra_config(width)), ("llama", llama_config_like(width))):
            llm = LLM.from_random(cfg, 8, dtype="bfloat16", on_device=True, max_seq_len=ctx + page,
                                  num_blocks=B * (ctx + page) // page + 64, block_size=page, max_num_seqs=B,
                                  max_batched_tokens=max(2048, B), prefix_caching=False)
            pre = prefill_run(llm, T, 5, 3, torch, np)
            ms, launches = decode_run(llm, B, steps, args.warmup, ctx, torch)
            profile.enable(True)
            prefill_run(llm, T, 3, 2, torch, np)
            profile.take_report()
            prefill_run(llm, T, 3, 0, torch, np)
            pre_stages = {k: round(v[0] / 3 * 1e3, 1) for k, v in profile.take_report().items()}
            decode_run(llm, B, 8, 4, ctx, torch, fill=False)
            dec_stages = {k: round(v[0] / 8 * 1e3, 1) for k, v in profile.take_report().items()}
            profile.enable(False)
            row[name] = {"prefill_tokens_per_s": round(T / (pre / 1e3), 1), "prefill_ms": round(pre, 3),
                         "decode_tokens_per_s": round(B / (ms / 1e3), 1), "decode_ms_per_step": round(ms, 4),
                         "launches_per_decode_step": launches,
                         "weight_bytes": int(sum(p.numel() * p.element_size() for p in _model_tensors(llm.model))),
                         "prefill_stage_us": pre_stages, "decode_stage_us": dec_stages}
            del llm
            torch.cuda.empty_cache()
        row["rooflines"] = gavodra_kernel_rooflines(width, B, ctx, T, pk, torch, np)
        out["sizes"][f"width{width}"] = row
    out["clocks"] = clocks.stop()
    head = out["sizes"]["width2048"]["gavodra"]
    out["value"] = head["decode_tokens_per_s"]
    out["ms_per_step"] = head["decode_ms_per_step"]
    out["gpu_launches"] = int(round(head["launches_per_decode_step"] * steps))
    return out


def lanirax_config(width: int, vocab: int = 32000) -> dict:
    """Four Lanirax layers at a real model's proportions.  Parallel layers: a window of 1,024 over heads of 64
    in groups of four (keys double as values, three quarters of a head rotated) beside a gated delta rule with heads of
    128 x 128, two value heads a query/key head, four taps.  Slope layers: heads of 64 in groups of four.
    Every layer routes to 4 of 32 experts of half a width (2 widths of feed-forward a token)."""
    H = width // 64
    rot = {"dims": 48, "base": 10000.0, "scaling": {"factor": 4.0, "original": 8192, "fast": 16.0, "slow": 2.0}}
    left = {"heads": H, "kv_heads": max(1, H // 4), "dim": 64, "vdim": 64, "scale": 0.125, "mask": {"size": 1024}, "rot": rot}
    right = {"heads": width // 128, "kv_heads": max(1, width // 256), "dim": 128, "vdim": 128, "conv": 4}
    slope = {"heads": H, "kv_heads": max(1, H // 4), "dim": 64, "vdim": 64, "scale": 0.125, "q_temp": {"coef": 0.3, "every": 1024}}
    moe = {"kind": "moe", "expert": {"ff": width // 2}, "router": {"experts": 32, "top": 4}}
    par = {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": moe}
    att = {"type": "attention", "mixer": slope, "mlp": moe}
    return {"architecture": "Lanirax", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "postln_alpha": 2.0,
            "layers": [par, att, par, att]}


def lanirax_kernel_rooflines(width: int, B: int, ctx: int, T: int, pk: dict, torch, np) -> dict:
    """The kernels that Lanirax adds or extends, alone, at the sizes of `lanirax_config(width)`, each beside
    the like kernel of the closest models: {name: {"us", "ideal_us", "frac"}}.  Ideal: bytes that must move over
    the measured copy bandwidth (single tokens, norms), FLOPs over the measured bfloat16 GEMM rate (attention
    over prompts), or float32 FMAs over the FFMA rate of the SMs at their maximum clock (the recurrences over
    prompts, float32 by design)."""
    from rust_llm_inference_server_b200 import ops
    hbm, tf = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    ffma = sms * 128 * 2 * pk.get("sm_max_mhz", 1965.0) * 1e6
    page, nh, nkv, hd, window = 16, width // 64, max(1, width // 256), 64, 1024
    rh, rqk, rd, taps = width // 128, max(1, width // 256), 128, 4
    bf, out = torch.bfloat16, {}
    rnd = lambda *shape: torch.randn(*shape, device="cuda") * 0.3

    def row(name, us, ideal_s):
        out[name] = {"us": round(us, 1), "ideal_us": round(ideal_s * 1e6, 1), "frac": round(ideal_s * 1e6 / us, 3)}

    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / nh) for h in range(nh)], device="cuda")
    sinks, bias = rnd(nh).contiguous(), rnd(129, nh).contiguous()
    for kind, reqs in (("decode", [(ctx - 1, 1)] * B), ("prefill", [(0, T)])):
        st = _KernelStep(reqs, page, torch, np)
        st.n_prefill_tokens = st.n_prefill_tokens if kind == "prefill" else 0
        n = st.n_tokens
        keys = B * ctx if kind == "decode" else T * (T + 1) // 2
        seen = B * min(ctx, window) if kind == "decode" else sum(min(i + 1, window) for i in range(T))
        kc, vc, q = rnd(st.n_pages, nkv, page, hd).to(bf), rnd(st.n_pages, nkv, page, hd).to(bf), rnd(n, nh * hd).to(bf)
        gate = rnd(n, nh + 8).to(bf)[:, :nh]
        o = torch.empty_like(q)
        attn = lambda k: k * nkv * hd * 2 * 2 / hbm if kind == "decode" else 2 * nh * k * 2 * hd / tf
        us = _graph_time_us(lambda: ops.attention_biased(q, kc, vc, o, None, None, st, 0, nh, nkv, hd, hd, page, 0.125, 0,
                                                         slopes=slopes), torch)
        row(f"slope_attention_{kind}", us, attn(keys))
        us = _graph_time_us(lambda: ops.attention_biased(q, kc, vc, o, None, None, st, 0, nh, nkv, hd, hd, page, 0.125, window,
                                                         sinks=sinks), torch)
        row(f"window_sink_attention_{kind}", us, attn(seen))
        us = _graph_time_us(lambda: ops.attention_biased(q, kc, vc, o, bias, gate, st, 0, nh, nkv, hd, hd, page, 0.125, 0), torch)
        row(f"table_bias_attention_{kind}", us, attn(keys))
        # the recurrences: the gated delta rule (convolutions, unit norms and gates in its first kernel) beside the
        # decayed linear attention at the same head sizes
        C = 2 * rqk * rd + rh * rd
        proj = rnd(n, C + rh * rd + 2 * rh + (-(2 * rh) % 8)).to(bf)
        conv_w, a_log, dt_bias = rnd(C, taps).contiguous(), rnd(rh).contiguous(), rnd(rh).contiguous()
        state = torch.zeros(len(reqs), ops.gated_delta_state_floats(rh, rqk, rd, rd, taps), device="cuda")
        o3 = torch.empty(n, rh * rd, device="cuda")
        us = _graph_time_us(lambda: ops.gated_delta(proj, 0, C + rh * rd, C + rh * rd + rh, conv_w, a_log, dt_bias, state, o3, st,
                                                    rh, rqk, rd, rd, taps, 1e-6, rd ** -0.5), torch)
        row(f"gated_delta_{kind}", us, B * rh * rd * rd * 4 * 2 / hbm if kind == "decode" else 3 * 2 * T * rh * rd * rd / ffma)
        proj2 = rnd(n, 3 * rh * rd).to(bf)
        state2, decay = torch.zeros(len(reqs), rh, rd, rd, device="cuda"), torch.full((rh,), 0.97, device="cuda")
        us = _graph_time_us(lambda: ops.lightning_scan(proj2, 0, rh * rd, 2 * rh * rd, o3, state2, decay, st, rh, rd, rd), torch)
        row(f"decayed_linear_attention_{kind}", us, B * rh * rd * rd * 4 * 2 / hbm if kind == "decode" else 2 * 2 * T * rh * rd * rd / ffma)
        # the normed sum of stream and two normed branches beside the norm of one sublayer's result
        resid, wv = rnd(n, width).contiguous(), torch.ones(width, device="cuda")
        a, b, y = rnd(n, width).to(bf), rnd(n, width).to(bf), torch.empty(n, width, dtype=bf, device="cuda")
        us = _graph_time_us(lambda: ops.sum_norm(resid, 2.5, [(a, wv, 0.5), (b, wv, 0.5)], wv, 1e-6, out=y, eps_branch=1e-6), torch)
        row(f"sum_norm_two_branches_{kind}", us, n * width * (4 + 4 + 2 + 2 + 2) / hbm)
        us = _graph_time_us(lambda: ops.post_norm_residual(a, resid, wv, 1e-6, out=y, mult=0.5), torch)
        row(f"post_norm_residual_{kind}", us, n * width * (4 + 4 + 2 + 2) / hbm)
    return out


def workload_lanirax(args, torch, np) -> dict:
    """Prefill (one 2,048-token prompt) and decode (batch 8, context 4,096) of four Lanirax layers at two
    widths beside four Gavodra layers (the closest model: the same attention kernels and routed feed-forwards) and
    four Llama layers of the same width, random bfloat16 weights; then the stages of one step by CUDA-event spans
    (eager launches), and the kernels alone, replayed from CUDA graphs, against their rooflines."""
    from rust_llm_inference_server_b200 import LLM
    from rust_llm_inference_server_b200.ops import profile
    pk, pk_src = peaks()
    B, ctx, page, T = args.batch, args.context, 16, PREFILL_TOKENS
    steps = min(args.steps, 64)
    out = {"workload": "lanirax", "metric": "prefill and decode tokens/s of four layers, Lanirax beside Gavodra and Llama at equal width",
           "unit": "tokens/s", "impl": "ours", "dtype": "bf16", "n_gpus": 1, "steps": steps, "warmup": args.warmup,
           "data": "synthetic: uniform-random token ids, random-init weights (device generator)",
           "config": {"global_batch": B, "seq_len": ctx, "prefill_tokens": T, "page_size": page, "layers": 4},
           "peaks": dict(pk, source=pk_src), "sizes": {}}
    clocks = ClockSampler()
    clocks.start()
    for width in (1024, 2048):
        row = {}
        for name, cfg in (("lanirax", lanirax_config(width)), ("gavodra", gavodra_config(width)), ("llama", llama_config_like(width))):
            llm = LLM.from_random(cfg, 8, dtype="bfloat16", on_device=True, max_seq_len=ctx + page,
                                  num_blocks=B * (ctx + page) // page + 64, block_size=page, max_num_seqs=B,
                                  max_batched_tokens=max(2048, B), prefix_caching=False)
            pre = prefill_run(llm, T, 5, 3, torch, np)
            ms, launches = decode_run(llm, B, steps, args.warmup, ctx, torch)
            profile.enable(True)
            prefill_run(llm, T, 3, 2, torch, np)
            profile.take_report()
            prefill_run(llm, T, 3, 0, torch, np)
            pre_stages = {k: round(v[0] / 3 * 1e3, 1) for k, v in profile.take_report().items()}
            decode_run(llm, B, 8, 4, ctx, torch, fill=False)
            dec_stages = {k: round(v[0] / 8 * 1e3, 1) for k, v in profile.take_report().items()}
            profile.enable(False)
            row[name] = {"prefill_tokens_per_s": round(T / (pre / 1e3), 1), "prefill_ms": round(pre, 3),
                         "decode_tokens_per_s": round(B / (ms / 1e3), 1), "decode_ms_per_step": round(ms, 4),
                         "launches_per_decode_step": launches,
                         "weight_bytes": int(sum(p.numel() * p.element_size() for p in _model_tensors(llm.model))),
                         "prefill_stage_us": pre_stages, "decode_stage_us": dec_stages}
            del llm
            torch.cuda.empty_cache()
        row["rooflines"] = lanirax_kernel_rooflines(width, B, ctx, T, pk, torch, np)
        out["sizes"][f"width{width}"] = row
    out["clocks"] = clocks.stop()
    head = out["sizes"]["width2048"]["lanirax"]
    out["value"] = head["decode_tokens_per_s"]
    out["ms_per_step"] = head["decode_ms_per_step"]
    out["gpu_launches"] = int(round(head["launches_per_decode_step"] * steps))
    return out


def rumedra_config(width: int, vocab: int = 32000) -> dict:
    """Four Rumedra layers at a real model's proportions.  Parallel layers: a window of 1,024 over heads of 64 in groups
    of four with values as wide as keys, half of every head rotated, a gate a channel, beside retention with heads of
    128 x 128.  Forget-gate layers: heads of 128 x 128.  Feed-forwards: relu-gated units of 8/3 widths, and routing to 4
    of 32 router outputs (28 experts of half a width and 4 identity experts, in 4 groups of which 2 are kept) beside a
    shared expert of half a width."""
    H, R = width // 64, width // 128
    rot = {"dims": 32, "base": 500000.0, "scaling": {"factor": 16.0, "low": 1.0, "high": 8.0, "original": 8192}}
    left = {"heads": H, "kv_heads": max(1, H // 4), "dim": 64, "vdim": 64, "scale": 0.125, "mask": {"size": 1024}, "rot": rot}
    right = {"heads": R, "dim": 128, "vdim": 128, "decay": [1.0 - 2.0 ** (-5 - 3 * h / max(1, R - 1)) for h in range(R)],
             "rot": {"dims": 128, "base": 500000.0}}
    par = {"left": left, "right": right, "left_scale": 0.7, "right_scale": 0.4}
    rec = {"heads": R, "dim": 128, "vdim": 128}
    moe = {"kind": "moe", "expert": {"ff": width // 2}, "shared": {"ff": width // 2},
           "router": {"experts": 28, "identity": 4, "top": 4, "scale": 2.5, "groups": {"count": 4, "keep": 2}}}
    dense = {"kind": "dense", "ff": width * 8 // 3 // 128 * 128}
    return {"architecture": "Rumedra", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
            "layers": [{"type": "parallel", "mixer": par, "mlp": dense}, {"type": "hgrn2", "mixer": rec, "mlp": moe},
                       {"type": "parallel", "mixer": par, "mlp": moe}, {"type": "hgrn2", "mixer": rec, "mlp": dense}]}


def rumedra_kernel_rooflines(width: int, B: int, ctx: int, T: int, pk: dict, torch, np) -> dict:
    """The kernels that Rumedra adds or extends, alone, at the sizes of `rumedra_config(width)`, each beside the like
    kernel of the closest models: {name: {"us", "ideal_us", "frac"}}.  Ideal: bytes that must move over the measured
    copy bandwidth (single tokens, elementwise kernels), FLOPs over the measured bfloat16 GEMM rate (attention and
    feed-forwards over prompts), or float32 FMAs over the FFMA rate of the SMs at their maximum clock (the recurrences
    over prompts, float32 by design)."""
    from rust_llm_inference_server_b200 import ops
    hbm, tf = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    ffma = sms * 128 * 2 * pk.get("sm_max_mhz", 1965.0) * 1e6
    page, nh, nkv, hd, window = 16, width // 64, max(1, width // 256), 64, 1024
    rh, rd = width // 128, 128
    E, ident, top, ff = 28, 4, 4, width // 2
    bf, out = torch.bfloat16, {}
    rnd = lambda *shape: torch.randn(*shape, device="cuda") * 0.3

    def row(name, us, ideal_s):
        out[name] = {"us": round(us, 1), "ideal_us": round(ideal_s * 1e6, 1), "frac": round(ideal_s * 1e6 / us, 3)}

    sinks = rnd(nh).contiguous()
    inv64, inv32 = torch.rand(64, device="cuda"), torch.rand(16, device="cuda")
    for kind, reqs in (("decode", [(ctx - 1, 1)] * B), ("prefill", [(0, T)])):
        st = _KernelStep(reqs, page, torch, np)
        st.n_prefill_tokens = st.n_prefill_tokens if kind == "prefill" else 0
        n = st.n_tokens
        seen = B * min(ctx, window) if kind == "decode" else sum(min(i + 1, window) for i in range(T))
        kc, vc, q = rnd(st.n_pages, nkv, page, hd).to(bf), rnd(st.n_pages, nkv, page, hd).to(bf), rnd(n, nh * hd).to(bf)
        gate = rnd(n, nh * hd + 8).to(bf)[:, :nh * hd]
        o = torch.empty_like(q)
        attn = seen * nkv * hd * 2 * 2 / hbm if kind == "decode" else 2 * nh * seen * 2 * hd / tf
        us = _graph_time_us(lambda: ops.attention_biased(q, kc, vc, o, None, gate, st, 0, nh, nkv, hd, hd, page, 0.125, window), torch)
        row(f"window_gate_attention_{kind}", us, attn)
        us = _graph_time_us(lambda: ops.attention_biased(q, kc, vc, o, None, None, st, 0, nh, nkv, hd, hd, page, 0.125, window,
                                                         sinks=sinks), torch)
        row(f"window_sink_attention_{kind}", us, attn)
        # rotation by halves with biases and the paged write, beside the rotation of adjacent pairs with unit norms
        N = (nh + 2 * nkv) * hd
        proj, pb = rnd(n, N).to(bf), rnd(N).contiguous()
        slots = torch.arange(n, device="cuda", dtype=torch.int32)
        ones = torch.ones(hd, device="cuda")
        moved = n * (N * 2 + (nh + 2 * nkv) * hd * 2) / hbm
        us = _graph_time_us(lambda: ops.qk_norm_store(proj, 0, nh * hd, (nh + nkv) * hd, None, None, 1e-5, None, 0.0, q, kc, vc, slots,
                                                      nh, nkv, hd, hd, page, rotation=(inv32, 32, 1.0), positions=st.positions,
                                                      rot_half=True, proj_bias=pb), torch)
        row(f"rotate_halves_bias_store_{kind}", us, moved)
        us = _graph_time_us(lambda: ops.qk_norm_store(proj, 0, nh * hd, (nh + nkv) * hd, ones, ones, 1e-5, None, 0.0, q, kc, vc, slots,
                                                      nh, nkv, hd, hd, page, rotation=(inv32, 32, 1.0), positions=st.positions), torch)
        row(f"rotate_pairs_norm_store_{kind}", us, moved)
        # the recurrences: inputs + walk, with a decay a head and a decay a channel, beside the decayed linear attention
        # (silu inputs, one kernel or two) at the same head sizes
        qk = rh * rd
        proj3 = rnd(n, 3 * qk).to(bf)
        state, decay = torch.zeros(len(reqs), rh, rd, rd, device="cuda"), torch.full((rh,), 0.97, device="cuda")
        o3 = torch.empty(n, qk, device="cuda")
        rows3, rows4 = torch.empty(n, 3 * qk, device="cuda"), torch.empty(n, 4 * qk, device="cuda")
        lower, gb = torch.rand(qk, device="cuda"), rnd(qk).contiguous()
        walk = B * rh * rd * rd * 4 * 2 / hbm if kind == "decode" else 2 * 2 * T * rh * rd * rd / ffma

        def retention():
            if n < ops.RECURRENCE_INPUT_PASS_TOKENS:
                return ops.recurrence_scan_rows(proj3, 0, qk, 2 * qk, o3, state, decay, st, rh, rd, rd, rotation=(inv64, 128),
                                                k_scale=rd ** -0.5)
            ops.recurrence_inputs(proj3, 0, qk, 2 * qk, rows3, rh, rd, rd, rotation=(inv64, 128), positions=st.positions,
                                  k_scale=rd ** -0.5)
            return ops.recurrence_scan(rows3, o3, state, decay, st, rh, rd, rd)

        def forget_gate():
            if n < ops.RECURRENCE_INPUT_PASS_TOKENS:
                return ops.recurrence_scan_rows(proj3, 0, qk, 2 * qk, o3, state, None, st, rh, rd, rd, lower=lower, gate_bias=gb)
            ops.recurrence_inputs(proj3, 0, qk, 2 * qk, rows4, rh, rd, rd, q_silu=True, lower=lower, gate_bias=gb)
            return ops.recurrence_scan(rows4, o3, state, None, st, rh, rd, rd, complement_key=True)
        row(f"retention_{kind}", _graph_time_us(retention, torch), walk)
        row(f"forget_gate_recurrence_{kind}", _graph_time_us(forget_gate, torch), walk)
        us = _graph_time_us(lambda: ops.lightning_scan(proj3, 0, qk, 2 * qk, o3, state, decay, st, rh, rd, rd), torch)
        row(f"decayed_linear_attention_{kind}", us, walk)
        # routing by softmax in groups with identity experts (route + sort + both products + the weighted sum), beside
        # routing by sigmoid scores over as many outputs that are all experts
        x = rnd(n, width).to(bf)
        y = torch.empty(n, width, dtype=bf, device="cuda")
        for name, n_exp, n_id, kw in (("routed_ff_groups_identity", E, ident, dict(scoring="softmax", groups=(4, 2), normalize=True)),
                                      ("routed_ff_sigmoid", E + ident, 0, {})):
            wr, corr = rnd(n_exp + n_id, width).contiguous(), rnd(n_exp + n_id).contiguous()
            wgu, wd = rnd(n_exp, 2 * ff, width).to(bf), rnd(n_exp, width, ff).to(bf)

            def routed(wr=wr, corr=corr, wgu=wgu, wd=wd, n_exp=n_exp, n_id=n_id, kw=kw):
                plan = ops.moe_route(x, wr, corr, n_exp, top, 2.5, False, st, n_identity=n_id, **kw)
                act = ops.moe_up(x, wgu, plan, 1.0, float("inf"), 0.0, st, 4)
                return ops.moe_combine(ops.moe_down(act, wd, plan, st), plan, None, y, x=x)
            share = n_exp / (n_exp + n_id)              # of the pairs that reach an expert
            flops = 2.0 * n * top * share * 3 * ff * width
            row(f"{name}_{kind}", _graph_time_us(routed, torch),
                min(n_exp, n * top) * 3 * ff * width * 2 / hbm if kind == "decode" else flops / tf)
        # the unit gated by relu beside the unit gated by silu (gating in the first product's epilogue over prompts)
        I = width * 8 // 3 // 128 * 128
        wgu = torch.stack([rnd(I // 4, 4, width), rnd(I // 4, 4, width)], dim=1).reshape(2 * I, width).to(bf).contiguous()
        wdn, act = rnd(width, I).to(bf), torch.empty(n, I, dtype=bf, device="cuda")

        def relu_unit():
            if n <= ops.STREAM_GEMM_ROWS:
                return ops.linear(ops.stream_gemm(x, wgu, swiglu4=True, slope=float("inf")), wdn)
            return ops.linear(ops.gemm_tcgen05(x, wgu, "glu4", glu=(float("inf"), None, 0.0)), wdn)

        def silu_unit():
            if n <= ops.STREAM_GEMM_ROWS:
                return ops.linear(ops.stream_gemm(x, wgu, swiglu4=True), wdn)
            return ops.linear(ops.gemm_tcgen05(x, wgu, "swiglu4"), wdn)
        ideal = 3 * I * width * 2 / hbm if kind == "decode" else 2.0 * n * 3 * I * width / tf
        row(f"relu_gated_ff_{kind}", _graph_time_us(relu_unit, torch), ideal)
        row(f"silu_gated_ff_{kind}", _graph_time_us(silu_unit, torch), ideal)
    return out


def workload_rumedra(args, torch, np) -> dict:
    """Prefill (one 2,048-token prompt) and decode (batch 8, context 4,096) of four Rumedra layers at two widths beside
    four Lanirax layers (the closest model: a parallel mixer of window attention and a recurrence, routed feed-forwards)
    and four Llama layers of the same width, random bfloat16 weights; then the stages of one step by CUDA-event spans
    (eager launches), and the kernels alone, replayed from CUDA graphs, against their rooflines."""
    from rust_llm_inference_server_b200 import LLM
    from rust_llm_inference_server_b200.ops import profile
    pk, pk_src = peaks()
    B, ctx, page, T = args.batch, args.context, 16, PREFILL_TOKENS
    steps = min(args.steps, 64)
    out = {"workload": "rumedra", "metric": "prefill and decode tokens/s of four layers, Rumedra beside Lanirax and Llama at equal width",
           "unit": "tokens/s", "impl": "ours", "dtype": "bf16", "n_gpus": 1, "steps": steps, "warmup": args.warmup,
           "data": "synthetic: uniform-random token ids, random-init weights (device generator)",
           "config": {"global_batch": B, "seq_len": ctx, "prefill_tokens": T, "page_size": page, "layers": 4},
           "peaks": dict(pk, source=pk_src), "sizes": {}}
    clocks = ClockSampler()
    clocks.start()
    for width in (1024, 2048):
        row = {}
        for name, cfg in (("rumedra", rumedra_config(width)), ("lanirax", lanirax_config(width)), ("llama", llama_config_like(width))):
            llm = LLM.from_random(cfg, 8, dtype="bfloat16", on_device=True, max_seq_len=ctx + page,
                                  num_blocks=B * (ctx + page) // page + 64, block_size=page, max_num_seqs=B,
                                  max_batched_tokens=max(2048, B), prefix_caching=False)
            pre = prefill_run(llm, T, 5, 3, torch, np)
            ms, launches = decode_run(llm, B, steps, args.warmup, ctx, torch)
            profile.enable(True)
            prefill_run(llm, T, 3, 2, torch, np)
            profile.take_report()
            prefill_run(llm, T, 3, 0, torch, np)
            pre_stages = {k: round(v[0] / 3 * 1e3, 1) for k, v in profile.take_report().items()}
            decode_run(llm, B, 8, 4, ctx, torch, fill=False)
            dec_stages = {k: round(v[0] / 8 * 1e3, 1) for k, v in profile.take_report().items()}
            profile.enable(False)
            row[name] = {"prefill_tokens_per_s": round(T / (pre / 1e3), 1), "prefill_ms": round(pre, 3),
                         "decode_tokens_per_s": round(B / (ms / 1e3), 1), "decode_ms_per_step": round(ms, 4),
                         "launches_per_decode_step": launches,
                         "weight_bytes": int(sum(p.numel() * p.element_size() for p in _model_tensors(llm.model))),
                         "prefill_stage_us": pre_stages, "decode_stage_us": dec_stages}
            del llm
            torch.cuda.empty_cache()
        row["rooflines"] = rumedra_kernel_rooflines(width, B, ctx, T, pk, torch, np)
        out["sizes"][f"width{width}"] = row
    out["clocks"] = clocks.stop()
    head = out["sizes"]["width2048"]["rumedra"]
    out["value"] = head["decode_tokens_per_s"]
    out["ms_per_step"] = head["decode_ms_per_step"]
    out["gpu_launches"] = int(round(head["launches_per_decode_step"] * steps))
    return out


def _model_tensors(model):
    seen = {}
    for part in model.parts():
        for v in vars(part).values():
            if isinstance(v, type(model.embedding.weight)) and v.is_cuda:
                seen[v.data_ptr()] = v
    return seen.values()


def print_timeline(records: list) -> None:
    """One decode step product by product (microseconds since the first product of the step started):
    when the launch's first CTA started, when its wait for the kernel before it passed, when its
    products were done, and when it ended; the gap is from the end of the product before to this
    one's wait passing, which for QKV -> O holds the attention kernel."""
    if not records:
        return
    t0 = records[0]["start"]
    us = lambda v: "      -" if v is None else f"{(v - t0) / 1e3:7.2f}"
    print(f"{'N x K':>15} | {'start':>7} {'waited':>7} {'done':>7} {'barrier':>7} {'sent':>7} {'arrived':>7} {'end':>7} | after the wait | gap before | grid before done",
          file=sys.stderr)
    prev = None
    for r in records:
        gap = "" if prev is None else f"{(r['wait_passed'] - prev) / 1e3:6.2f}"
        print(f"{r['N']:>7} x {r['K']:>5} | {us(r['start'])} {us(r['wait_passed'])} {us(r['products_done'])} {us(r['cluster_barrier'])} "
              f"{us(r['sent'])} {us(r['sums_arrived'])} {us(r['end'])} | {(r['end'] - r['wait_passed']) / 1e3:14.2f} | {gap:>10} | {us(r['grid_before_done'])}",
              file=sys.stderr)
        prev = r["end"]


WORKLOADS = {"3b": workload_3b, "8b": workload_8b, "1b-fp32": workload_1b_fp32, "lasapel": workload_lasapel,
             "gavodra": workload_gavodra, "lanirax": workload_lanirax, "rumedra": workload_rumedra}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (both numbers are reported)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=CONTEXT, help="context length at the last timed decode step")
    ap.add_argument("--no-fill", action="store_true",
                    help="with --only decode: do not compute the cached context first (keeps profiler captures short)")
    ap.add_argument("--only", default=None, choices=["decode", "prefill"],
                    help="run one part only and print a short line (for profiler captures of a small case)")
    ap.add_argument("--sizes", default="1b", choices=["1b", "3b", "8b"],
                    help="with --only: the layer sizes to run it at (the default line is always the 1B's)")
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS),
                    help="one of the other measured configurations instead of the default line: 3b (continuous "
                         "batching under a Poisson stream), 8b (batch 32 at 8,192 of context), 1b-fp32")
    ap.add_argument("--rate", type=float, default=48.0, help="--workload 3b: mean arrivals a second")
    ap.add_argument("--timeline", action="store_true",
                    help="with --only decode and RLIS_TIMELINE=1 in the environment (a build of the kernels with "
                         "the stamps compiled in): lay the last step out product by product from the stamps the "
                         "streaming products' first CTAs take of the device's timer (printed to stderr)")
    ap.add_argument("--spans", action="store_true",
                    help="with --only: time the stages of the step with CUDA-event spans (RLIS_PROFILE) and "
                         "print the table to stderr; steps then run eagerly, not from graphs")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)

    import numpy as np
    import torch

    from rust_llm_inference_server_b200 import LLM, SamplingParams, ops
    from rust_llm_inference_server_b200.ops import profile

    if args.workload:
        print(json.dumps(WORKLOADS[args.workload](args, torch, np)))
        return 0
    pk, pk_src = peaks()
    cfg = dict({"1b": CONFIG_1B, "3b": CONFIG_3B, "8b": CONFIG_8B}[args.sizes if args.only else "1b"])
    n_layers_full = cfg["num_hidden_layers"]
    n_layers = args.layers or n_layers_full
    cfg["num_hidden_layers"] = n_layers
    B = args.batch
    total = args.warmup + args.steps
    page = 16
    max_b = max(B, 64)
    context = args.context
    if args.only:
        max_b = B
    pool_tokens = max_b * (context + page)
    llm = LLM.from_random(cfg, SEED, dtype="bfloat16", on_device=True, max_seq_len=max(context, PREFILL_TOKENS) + page,
                          num_blocks=pool_tokens // page + 64, block_size=page, max_num_seqs=max_b,
                          max_batched_tokens=max(2048, max_b), prefix_caching=False)
    runner = llm.engine.runner

    # ---- prefill of one 2,048-token prompt ----
    from rust_llm_inference_server_b200.engine import StepEntry
    rng = np.random.default_rng(0)
    V = cfg["vocab_size"]
    cache = llm.engine.cache
    if args.only and args.spans:
        profile.enable(True)
    if args.only == "decode":
        if args.timeline:
            ops.stream_timeline(True)
        ms, launches = decode_run(llm, B, args.steps, args.warmup, context, torch, fill=not args.no_fill)
        print(json.dumps({"only": "decode", "batch": B, "context": context, "ms_per_step": round(ms, 4),
                          "launches_per_step": launches}))
        if args.timeline:
            print_timeline(ops.read_stream_timeline(4 * n_layers + 1))
        if args.spans:
            print(profile.format_report(profile.take_report()), file=sys.stderr)
        return 0
    pre_ms = []
    for it in range(5 if not args.only else args.warmup + args.steps):
        sid = 500 + it
        cache.acquire_state_slot(sid)
        assert cache.reserve(sid, PREFILL_TOKENS)
        toks = rng.integers(0, V, size=PREFILL_TOKENS).tolist()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        if args.only and args.spans and it == args.warmup:
            profile.take_report()           # the table covers the timed steps only
        s.record()
        runner.step([StepEntry(sid, toks, 0, [PREFILL_TOKENS - 1])])
        e.record()
        torch.cuda.synchronize()
        pre_ms.append(s.elapsed_time(e))
        cache.free(sid)
    prefill_ms = statistics.median(pre_ms[2:] if not args.only else pre_ms[args.warmup:])
    if args.only == "prefill":
        print(json.dumps({"only": "prefill", "tokens": PREFILL_TOKENS, "ms": round(prefill_ms, 3)}))
        if args.spans:
            print(profile.format_report(profile.take_report()), file=sys.stderr)
        return 0
    pf = prefill_flops(cfg, n_layers, PREFILL_TOKENS)
    prefill = {"value": round(PREFILL_TOKENS / (prefill_ms / 1e3), 1), "tokens": PREFILL_TOKENS,
               "ms": round(prefill_ms, 3),
               "frac": round(pf / (prefill_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}

    # ---- decode points at batch 1 and 64, then the headline batch under the clock sampler ----
    points = {}
    for b in (1, 64):
        ms, _ = decode_run(llm, b, max(16, min(args.steps, 64)), args.warmup, context, torch)
        points[f"decode_b{b}"] = round(b / (ms / 1e3), 1)
    clocks = ClockSampler()
    ms, launches = decode_run(llm, B, args.steps, args.warmup, context, torch, clocks=clocks)
    clk = clocks.stop()
    value = B / (ms / 1e3)
    mean_ctx = context - args.steps / 2
    step_bytes = weight_bytes(cfg, n_layers) + B * mean_ctx * kv_bytes_per_token(cfg, n_layers)
    achieved = step_bytes / (ms / 1e3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk_src}

    # ---- end to end through the Python entry point ----
    # The prompts finish their prefill in different steps (the token budget cuts them), so the
    # requests do not decode in lockstep; each gets enough output that all B decode together for
    # warmup + steps steps, the last of which sees a context of about `context` tokens.
    stagger = B * (context // 2048 + 1)
    e2e_out = total + stagger + 8
    prompts = [rng.integers(0, V, size=context - e2e_out - 1).tolist() for _ in range(B)]
    sp = SamplingParams(max_tokens=e2e_out, ignore_eos=True)
    eng = llm.engine
    h2d0 = d2h0 = h2d1 = d2h1 = 0
    t0 = t1 = None
    n_decode = 0
    for ev in llm.stream(prompts, sp):
        if not (ev.all_decoding and ev.n_seqs == B) or t1 is not None:
            continue
        n_decode += 1
        if n_decode == args.warmup:
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            h2d0, d2h0 = eng.stats.h2d_bytes, eng.stats.d2h_bytes
        elif n_decode == args.warmup + args.steps:
            torch.cuda.synchronize()
            t1 = time.perf_counter()
            h2d1, d2h1 = eng.stats.h2d_bytes, eng.stats.d2h_bytes
    e2e_ms = (t1 - t0) * 1e3 / args.steps
    e2e = {"value": round(B / (e2e_ms / 1e3), 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
           "h2d_bytes_per_step": (h2d1 - h2d0) // args.steps, "d2h_bytes_per_step": (d2h1 - d2h0) // args.steps}

    line = {
        "metric": "decode tokens/s, batch 8, context 4096 (Llama-3.2-1B sizes, random bf16 weights)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: uniform-random token ids, random-init weights N(0,0.02) seed 4",
        "impl": "ours",
        "config": {
            "model": "llama-3.2-1b-sizes", "layers": n_layers, "layers_in_config": n_layers_full,
            "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": V,
            "tied": True, "rope": "theta 5e5 llama3 32/1/4/8192", "eps": 1e-5,
            "global_batch": B, "seq_len": context, "page_size": page, "parallelism": "single GPU",
            "l2": "inputs larger than L2 (weights 2.47 GB per step)", "kv_dtype": "bf16",
        },
        "prefill": prefill, "roofline": roofline, "points": points, "e2e": e2e,
        "gpu_launches": int(round(launches * args.steps)), "clocks": clk,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
