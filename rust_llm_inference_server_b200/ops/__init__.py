"""The hot ops of the forward pass: thin, checked wrappers over the sm_100a kernels.

Every function takes CUDA tensors, checks element types, shapes and contiguity, and launches on
the current stream.  A size that a kernel does not take is refused with an error; nothing here
falls back to a tensor library's model code or to the CPU.  Matrix products in bfloat16 go to the
library GEMM (cuBLAS through `torch.mm`), as the reference's go to its tensor library
(crates/model/src/layers.rs:82); in float32 they go to this package's own FFMA kernel so that
no reduced-precision matrix mode can enter.
"""

from __future__ import annotations

import functools

import torch

from . import library
from .library import KernelError, check, debug_set, lib

_DT = {torch.float32: 0, torch.bfloat16: 1}

# Number of launches of this package's kernels since the last reset (a claim the benchmark
# reports; launches replayed from a captured graph are counted by the graph's owner).
launch_count = 0


def set_programmatic_launch(on: bool) -> None:
    """Whether kernels are launched with the programmatic-serialization attribute (on unless
    switched off, here or by RLIS_DEBUG=pdl=0): the next kernel's CTAs start their prologue while
    the current kernel drains; see csrc/kernels/common.cuh."""
    debug_set("pdl", 1 if on else 0)


def _code(dtype) -> int:
    try:
        return _DT[dtype]
    except KeyError:
        raise KernelError(f"element type {dtype} is not supported (float32 and bfloat16 are)") from None


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current CUDA stream's handle.  (The raw lookup takes a microsecond; building a
    `torch.cuda.Stream` object for it took eighteen, three times a decode step.)"""
    if _raw_stream is not None:
        return _raw_stream(-1)
    return torch.cuda.current_stream().cuda_stream


def _req(t: torch.Tensor, name: str, dtype=None, shape=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name}: expected a CUDA tensor; there is no CPU path")
    if not t.is_contiguous():
        raise KernelError(f"{name}: expected a contiguous tensor, got strides {t.stride()}")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: expected {dtype}, got {t.dtype}")
    if shape is not None:
        if t.dim() != len(shape) or any(s is not None and s != g for s, g in zip(shape, t.shape)):
            raise KernelError(f"{name}: expected shape {shape}, got {tuple(t.shape)}")


# The same by kernel, for tests that have to know which kernel a step went through:
# {"stream_gemm.sink": 12, "attention_decode_qkv.mma.tma": 4, ...}.
launches_by_kernel: dict = {}


def _count(name: str) -> None:
    global launch_count
    launch_count += 1
    launches_by_kernel[name] = launches_by_kernel.get(name, 0) + 1


def _decode_variant() -> str:
    """Which decode-attention kernel the launcher just chose."""
    v = lib().rlis_attention_decode_last_variant()
    if not v & 1:
        return ".cuda_core"
    return ".mma" + (".tma" if v & 2 else "") + (".cluster" if v & 4 else "")


def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, scale: float | None = None) -> torch.Tensor:
    """out[t, :] = table[ids[t], :] widened to float32 (times `scale` if given).  ids int32 [T];
    out float32 [T, H]."""
    V, H = table.shape
    T = ids.shape[0]
    _req(ids, "ids", torch.int32, (T,))
    _req(table, "table")
    _req(out, "out", torch.float32, (T, H))
    check(lib().rlis_embedding(ids.data_ptr(), table.data_ptr(), out.data_ptr(), T, H, V,
                               1.0 if scale is None else float(scale), _code(table.dtype), _stream()), "embedding")
    _count("embedding")
    return out


def embedding_sink(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, scale: float | None, sink):
    """`embedding` for a step whose first norm is left to the product after it (`sink`, a
    ResidualSink over `out`): also returns that norm's ScaledRows, bf16(row * weight) and the sums of
    squares of every 128 features.  bfloat16 tables whose width is a multiple of 8."""
    V, H = table.shape
    T = ids.shape[0]
    _req(ids, "ids", torch.int32, (T,))
    _req(table, "table", torch.bfloat16)
    _req(out, "out", torch.float32, (T, H))
    _req(sink.weight, "sink.weight", torch.float32, (H,))
    if sink.resid.data_ptr() != out.data_ptr() or H % 8:
        raise KernelError("embedding_sink: the sink is over another residual stream, or the width is no multiple of 8")
    xn = torch.empty((T, H), dtype=torch.bfloat16, device=out.device)
    partials = torch.empty(((H + 127) // 128, T), dtype=torch.float32, device=out.device)
    check(lib().rlis_embedding_sink(ids.data_ptr(), table.data_ptr(), out.data_ptr(), sink.weight.data_ptr(),
                                    xn.data_ptr(), partials.data_ptr(), T, H, V,
                                    1.0 if scale is None else float(scale), _stream()), "embedding_sink")
    _count("embedding.sink")
    return ScaledRows(xn, partials, H, sink.eps)


def logit_transform(logits: torch.Tensor, scale: float | None, soft_cap: float | None) -> torch.Tensor:
    """In place on float32 logits [R, V]: x <- x * scale, then x <- cap * tanh(x / cap) (each only
    where given)."""
    R, V = logits.shape
    if logits.dtype != torch.float32 or not logits.is_cuda or logits.stride(1) != 1:
        raise KernelError("logit_transform: logits must be float32 CUDA rows with unit stride")
    if soft_cap is not None and not soft_cap > 0:
        raise KernelError(f"logit_transform: the cap must be positive, got {soft_cap}")
    check(lib().rlis_logit_transform(logits.data_ptr(), R, V, logits.stride(0), 1.0 if scale is None else float(scale),
                                     0.0 if soft_cap is None else float(soft_cap), _stream()), "logit_transform")
    _count("logit_transform")
    return logits


def rmsnorm(resid: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            delta: torch.Tensor | None = None, rows: torch.Tensor | None = None) -> torch.Tensor:
    """If `delta` is given: resid += delta (float32).  out = rmsnorm(resid) * weight, rounded once.

    resid float32 [T, H] (updated in place), weight float32 [H], out and delta in the activation
    type.  With `rows` (int32 [R]): out [R, H] is computed from rows resid[rows] (+ delta[rows])
    and resid is left unchanged."""
    T, H = resid.shape
    _req(resid, "resid", torch.float32)
    _req(weight, "weight", torch.float32, (H,))
    n_out = T
    if rows is not None:
        _req(rows, "rows", torch.int32, (None,))
        n_out = rows.shape[0]
    _req(out, "out", None, (n_out, H))
    if delta is not None:
        _req(delta, "delta", out.dtype, (T, H))
    check(lib().rlis_rmsnorm(resid.data_ptr(), delta.data_ptr() if delta is not None else None,
                             weight.data_ptr(), out.data_ptr(),
                             rows.data_ptr() if rows is not None else None, n_out, H, float(eps),
                             _code(out.dtype), _stream()), "rmsnorm")
    _count("rmsnorm" if rows is None else "rmsnorm.rows")
    return out


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, interleave: int = 0) -> torch.Tensor:
    """out[t, i] = silu(gate_i) * up_i; gate_up [T, 2I], out [T, I].  interleave 0: gate columns
    first, then up columns; B > 0: blocks of B gate columns each followed by their B up columns."""
    T, I2 = gate_up.shape
    if I2 % 2:
        raise KernelError(f"swiglu: the fused gate|up width must be even, got {I2}")
    _req(gate_up, "gate_up")
    _req(out, "out", gate_up.dtype, (T, I2 // 2))
    check(lib().rlis_swiglu(gate_up.data_ptr(), out.data_ptr(), T, I2 // 2, int(interleave),
                            _code(out.dtype), _stream()), "swiglu")
    _count("swiglu")
    return out


def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """out[M, N] = a[M, K] @ w[N, K]^T in true float32 (FFMA, fixed order over K)."""
    M, K = a.shape
    N = w.shape[0]
    _req(a, "a", torch.float32)
    _req(w, "w", torch.float32, (N, K))
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=a.device)
    _req(out, "out", torch.float32, (M, N))
    check(lib().rlis_gemm_f32_nt(a.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, _stream()),
          "gemm_f32")
    _count("gemm_f32")
    return out


def gemm_f32_batched(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[:, b, :] = a[:, b, :] @ w[b]^T for every b, in true float32 (the same kernel and k order as
    `gemm_f32`).  a [M, B, K], out [M, B, N]: views whose last axis has unit stride (the per-head
    slices of wider rows); w [B, N, K] contiguous."""
    M, B, K = a.shape
    N = w.shape[1]
    for t, nm in ((a, "a"), (out, "out")):
        if t.dtype != torch.float32 or not t.is_cuda or t.stride(2) != 1:
            raise KernelError(f"gemm_f32_batched: {nm} must be float32 on the device with unit stride in its last axis")
    _req(w, "w", torch.float32, (B, N, K))
    if tuple(out.shape) != (M, B, N):
        raise KernelError(f"gemm_f32_batched: expected out of shape {(M, B, N)}, got {tuple(out.shape)}")
    check(lib().rlis_gemm_f32_nt_batched(a.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), K,
                                         out.stride(0), B, a.stride(1), N * K, out.stride(1), _stream()),
          "gemm_f32_batched")
    _count("gemm_f32.batched")
    return out


def per_head_linear(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t, h, :] = w[h] @ a[t, h, :]: one small product a head (a [T, H, K] and out [T, H, N] may be
    slices of wider rows, w [H, N, K]).  float32: this package's FFMA kernel; bfloat16 operands: the
    library's batched GEMM with float32 accumulation, into `out`'s element type."""
    if a.dtype == torch.float32:
        return gemm_f32_batched(a, w, out)
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not a.is_cuda:
        raise KernelError(f"per_head_linear: expected float32 or bfloat16 operands on the device, got {a.dtype}, {w.dtype}")
    # [H, T, N] view of `out` (rows H * width apart, heads one head's width apart): the library writes it in place
    if out.dtype != a.dtype:
        torch.bmm(a.transpose(0, 1), w.transpose(1, 2), out_dtype=out.dtype, out=out.transpose(0, 1))
    else:
        torch.bmm(a.transpose(0, 1), w.transpose(1, 2), out=out.transpose(0, 1))
    return out


def post_norm_residual(sub: torch.Tensor | None, resid: torch.Tensor, w_post: torch.Tensor | None, eps_post: float,
                       scale: torch.Tensor | None = None, bias: torch.Tensor | None = None,
                       w_next: torch.Tensor | None = None, eps_next: float = 0.0,
                       out: torch.Tensor | None = None, mult: float = 1.0):
    """resid += mult * scale * rmsnorm(sub + bias) * w_post, all in float32 and in place (`mult` a number,
    `scale` a vector); with `w_next` also out = rmsnorm(resid) * w_next (the norm in front of the next
    sublayer), rounded once to sub's type.  `out` without `w_next`: out = resid rounded to out's type, for a
    sublayer that reads the stream as it is; `sub` None: nothing is added and only that copy is made.
    sub [T, H] in the activation type; resid float32 [T, H]; the vectors float32 [H]."""
    T, H = resid.shape
    _req(resid, "resid", torch.float32)
    if sub is not None:
        _req(sub, "sub", None, (T, H))
        _req(w_post, "w_post", torch.float32, (H,))
    elif out is None or w_next is not None:
        raise KernelError("post_norm_residual: without a sublayer result only the copy of the stream is made")
    for v, nm in ((scale, "scale"), (bias, "bias"), (w_next, "w_next")):
        if v is not None:
            _req(v, nm, torch.float32, (H,))
    if w_next is not None or out is not None:
        _req(out, "out", sub.dtype if sub is not None else None, (T, H))
    dtype = sub.dtype if sub is not None else out.dtype
    check(lib().rlis_post_norm_residual(sub.data_ptr() if sub is not None else None,
                                        bias.data_ptr() if bias is not None else None,
                                        w_post.data_ptr() if sub is not None else None,
                                        scale.data_ptr() if scale is not None else None,
                                        resid.data_ptr(), w_next.data_ptr() if w_next is not None else None,
                                        out.data_ptr() if out is not None else None, T, H, float(eps_post),
                                        float(eps_next), float(mult), _code(dtype), _stream()), "post_norm_residual")
    _count("post_norm_residual" + (".next" if w_next is not None else ".copy" if out is not None else ""))
    return out


def act_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
             gate: torch.Tensor | None = None) -> torch.Tensor:
    """out = x / sqrt(mean(x^2) + eps) * weight (* sigmoid(gate)) per row, statistics in float32.  x is
    float32 or out's type; x, gate and out [T, W] may be column slices of wider rows (unit stride in
    the last axis)."""
    T, W = x.shape
    for t, nm in ((x, "x"), (out, "out")) + (((gate, "gate"),) if gate is not None else ()):
        if not t.is_cuda or t.dim() != 2 or tuple(t.shape) != (T, W) or t.stride(1) != 1:
            raise KernelError(f"act_norm: {nm} must be [T, W] rows on the device with unit stride")
    if x.dtype not in (torch.float32, out.dtype) or (gate is not None and gate.dtype != out.dtype):
        raise KernelError(f"act_norm: element types {x.dtype} / {out.dtype} are not taken")
    _req(weight, "weight", torch.float32, (W,))
    check(lib().rlis_act_norm(x.data_ptr(), x.stride(0), 1 if x.dtype == torch.float32 else 0, weight.data_ptr(),
                              gate.data_ptr() if gate is not None else None,
                              gate.stride(0) if gate is not None else 0, out.data_ptr(), out.stride(0), T, W,
                              float(eps), _code(out.dtype), _stream()), "act_norm")
    _count("act_norm" + (".gate" if gate is not None else ""))
    return out


def sum_norm(resid: torch.Tensor | None, alpha: float, branches, w_out: torch.Tensor | None, eps_out: float,
             out: torch.Tensor | None = None, eps_branch: float = 0.0) -> torch.Tensor | None:
    """y = alpha * resid + sum over `branches` (x, w, c) of c * (x / sqrt(mean(x^2) + eps_branch) * w, or x itself
    where w is None); with `w_out`, y = y / sqrt(mean(y^2) + eps_out) * w_out.  y is written back to `resid`
    (float32 [T, H], in place; None: there is no stream term) and, rounded once, to `out` (the activation type;
    None: no copy).  Up to two branches [T, H] in the activation type; all sums float32."""
    branches = list(branches)
    if len(branches) > 2:
        raise KernelError("sum_norm: up to two branches")
    ref = resid if resid is not None else out
    if ref is None:
        raise KernelError("sum_norm: nothing to write")
    T, H = ref.shape
    if resid is not None:
        _req(resid, "resid", torch.float32, (T, H))
    dtype = out.dtype if out is not None else (branches[0][0].dtype if branches else torch.float32)
    if out is not None:
        _req(out, "out", dtype, (T, H))
    args = []
    for x, w, c in branches:
        _req(x, "branch", dtype, (T, H))
        if w is not None:
            _req(w, "branch weight", torch.float32, (H,))
        args += [x.data_ptr(), w.data_ptr() if w is not None else None, float(c)]
    while len(args) < 6:
        args += [None, None, 0.0]
    if w_out is not None:
        _req(w_out, "w_out", torch.float32, (H,))
    check(lib().rlis_sum_norm(*args, resid.data_ptr() if resid is not None else None, float(alpha),
                              w_out.data_ptr() if w_out is not None else None,
                              out.data_ptr() if out is not None else None, T, H, float(eps_branch), float(eps_out),
                              _code(dtype), _stream()), "sum_norm")
    _count("sum_norm" + (".%d" % len(branches)) + (".norm" if w_out is not None else ""))
    return out if out is not None else resid


GATE_ACTIVATIONS = {"sigmoid": 0, "silu": 1}


def head_norm_gate(x: torch.Tensor, weight: torch.Tensor | None, eps: float, out: torch.Tensor, n_heads: int,
                   gate: torch.Tensor | None = None, activation: str = "sigmoid") -> torch.Tensor:
    """out[t, h, :] = x[t, h, :] / sqrt(mean(x[t, h, :]^2) + eps) * weight * act(gate[t, h, :]): one norm a head,
    one weight vector [dv] for all heads (None: no weight).  x float32 [T, nh dv]; gate [T, nh dv] in out's type (may be a column
    slice of wider rows); activation "sigmoid" or "silu"."""
    T, W = x.shape
    dv = W // n_heads
    _req(x, "x", torch.float32, (T, n_heads * dv))
    if weight is not None:
        _req(weight, "weight", torch.float32, (dv,))
    _req(out, "out", None, (T, W))
    gp, gs = None, 0
    if gate is not None:
        if gate.dtype != out.dtype or tuple(gate.shape) != (T, W) or gate.stride(1) != 1 or not gate.is_cuda:
            raise KernelError("head_norm_gate: the gate must be [T, nh dv] rows with unit stride in out's type")
        gp, gs = gate.data_ptr(), gate.stride(0)
    if activation not in GATE_ACTIVATIONS:
        raise KernelError(f"head_norm_gate: unknown activation {activation!r}; known: {sorted(GATE_ACTIVATIONS)}")
    check(lib().rlis_head_norm_gate(x.data_ptr(), weight.data_ptr() if weight is not None else None, gp, gs, out.data_ptr(),
                                    T, n_heads, dv, float(eps),
                                    GATE_ACTIVATIONS[activation], _code(out.dtype), _stream()), "head_norm_gate")
    _count("head_norm_gate")
    return out


def gated_delta_state_floats(n_heads: int, n_qk_heads: int, d: int, dv: int, taps: int) -> int:
    """float32 entries of a request's state for `gated_delta`: S of every head, then the convolution's tail."""
    return n_heads * dv * d + (taps - 1) * (2 * n_qk_heads * d + n_heads * dv)


# Portions of this many tokens a request (on average over the step) go through the recurrence 16 tokens at a time,
# unless the step has so many requests that the token-by-token kernel fills the SMs by itself (more than three
# CTAs an SM): measured on a B200 at heads of 128 x 128, one or four prompts of 512 and more tokens run 1.1 to 1.4
# times faster in chunks, eight prompts of 256 and less 1.1 to 1.5 times faster token by token.
GATED_DELTA_CHUNKS_FROM = 256


@functools.lru_cache(maxsize=None)
def _sm_count(device) -> int:
    return torch.cuda.get_device_properties(device).multi_processor_count


def gated_delta(proj: torch.Tensor, qkv_off: int, b_off: int, a_off: int, conv_w: torch.Tensor, a_log: torch.Tensor,
                dt_bias: torch.Tensor, state: torch.Tensor, out: torch.Tensor, step, n_heads: int, n_qk_heads: int,
                d: int, dv: int, taps: int, unit_eps: float, q_scale: float, chunks: bool | None = None) -> torch.Tensor:
    """The gated delta rule over the step's tokens (csrc/kernels/gated_delta.cu): from the rows of a stacked
    projection `proj` [T, N] (q | k | v from column qkv_off: n_qk_heads heads of d twice, then n_heads of dv; one
    logit a head of beta from b_off and of the decay from a_off), a causal convolution of `taps` taps per channel
    (conv_w float32 [C, taps]) and silu, unit vectors q (times q_scale) and k, then per head S <- g S, u = beta
    (v - S^T k), S <- S + k u^T, o = S^T q.  `state` float32 [slots, gated_delta_state_floats(...)] holds S and
    the convolution's tail between steps; out float32 [T, nh dv].

    A step of long portions of few requests (GATED_DELTA_CHUNKS_FROM) goes through the kernels that take 16 tokens
    of a request at a time; other steps walk token by token (`chunks` says which, for any step)."""
    T, N = proj.shape
    C = 2 * n_qk_heads * d + n_heads * dv
    _req(proj, "proj")
    _req(conv_w, "conv_w", torch.float32, (C, taps))
    _req(a_log, "a_log", torch.float32, (n_heads,))
    _req(dt_bias, "dt_bias", torch.float32, (n_heads,))
    _req(out, "out", torch.float32, (T, n_heads * dv))
    _req(state, "state", torch.float32, (None, gated_delta_state_floats(n_heads, n_qk_heads, d, dv, taps)))
    if qkv_off + C > N or b_off + n_heads > N or a_off + n_heads > N:
        raise KernelError("gated_delta: the column offsets reach beyond the projection's rows")
    act = step.buffer("gated_delta_act", (T, C + 2 * n_heads), torch.float32)
    if chunks is None:
        chunks = T >= GATED_DELTA_CHUNKS_FROM * step.n_seqs and \
            step.n_seqs * n_heads * -(-dv // 16) <= 3 * _sm_count(proj.device)
    gram = step.buffer("gated_delta_gram", (T, n_qk_heads * 32 + n_heads * 16), torch.float32).data_ptr() if chunks else 0
    check(lib().rlis_gated_delta(proj.data_ptr(), proj.stride(0), int(qkv_off), int(b_off), int(a_off), conv_w.data_ptr(),
                                 a_log.data_ptr(), dt_bias.data_ptr(), state.data_ptr(), state.stride(0),
                                 step.cu_seqlens.data_ptr(), step.ctx_lens.data_ptr(), step.state_slots.data_ptr(),
                                 step.seq_of_token.data_ptr(), act.data_ptr(), gram, out.data_ptr(), T, step.n_seqs, n_heads,
                                 n_qk_heads, d, dv, taps, float(unit_eps), float(q_scale), _code(proj.dtype), _stream()),
          "gated_delta")
    _count("gated_delta.prepare")
    if chunks:
        _count("gated_delta.gram")
        _count("gated_delta.solve")
    _count("gated_delta.chunks" if chunks else "gated_delta.scan")
    return out


BIAS_ACTIVATIONS = {"none": 0, "relu2": 1}


def bias_act(x: torch.Tensor, bias: torch.Tensor | None, out: torch.Tensor, activation: str = "none") -> torch.Tensor:
    """out = act(x + bias): "none", or "relu2" (the square of max(., 0)); float32 inside."""
    T, W = x.shape
    _req(x, "x")
    _req(out, "out", x.dtype, (T, W))
    if bias is not None:
        _req(bias, "bias", torch.float32, (W,))
    if activation not in BIAS_ACTIVATIONS:
        raise KernelError(f"bias_act: unknown activation {activation!r}; known: {sorted(BIAS_ACTIVATIONS)}")
    check(lib().rlis_bias_act(x.data_ptr(), bias.data_ptr() if bias is not None else None, out.data_ptr(), T, W,
                              BIAS_ACTIVATIONS[activation], _code(x.dtype), _stream()), "bias_act")
    _count("bias_act." + activation)
    return out


def latent_kv_store(z: torch.Tensor, weight: torch.Tensor, eps: float, inv_freq: torch.Tensor, rot_dims: int,
                    magnitude: float, positions: torch.Tensor, slots: torch.Tensor, cache: torch.Tensor,
                    rank: int, page_size: int, q_latent: torch.Tensor | None = None,
                    q_weight: torch.Tensor | None = None, q_out: torch.Tensor | None = None) -> None:
    """Writes one row per token into a paged cache of latents [pages, 1, page_size, rank + rot]:
    rmsnorm(z[:, :rank]) * weight, then z[:, rank:] with its first `rot_dims` entries rotated
    (rotate-half, angle position * inv_freq, cos and sin times `magnitude`).  z may be a column slice.
    With `q_latent` (another column slice of the same rows), `q_weight` and `q_out` [T, q_rank]
    (contiguous) the same launch also leaves q_out = rmsnorm(q_latent) * q_weight."""
    T, Wd = z.shape
    zq = wq = cq = None
    q_rank = 0
    if q_latent is not None:
        q_rank = q_latent.shape[1]
        if q_latent.dtype != z.dtype or q_latent.stride(0) != z.stride(0) or q_latent.stride(1) != 1 or q_latent.shape[0] != T:
            raise KernelError("latent_kv_store: the query latent must be a column slice of the same rows as z")
        _req(q_weight, "q_weight", torch.float32, (q_rank,))
        _req(q_out, "q_out", z.dtype, (T, q_rank))
        zq, wq, cq = q_latent.data_ptr(), q_weight.data_ptr(), q_out.data_ptr()
    rot = Wd - rank
    if not z.is_cuda or z.stride(1) != 1 or rot < 0:
        raise KernelError("latent_kv_store: z must be [T, rank + rot] rows on the device with unit stride")
    _req(weight, "weight", torch.float32, (rank,))
    _req(inv_freq, "inv_freq", torch.float32, (rot_dims // 2,))
    _req(positions, "positions", torch.int32, (T,))
    _req(slots, "slots", torch.int32, (T,))
    _req(cache, "cache", z.dtype, (None, 1, page_size, Wd))
    check(lib().rlis_latent_kv_store(z.data_ptr(), z.stride(0), weight.data_ptr(), inv_freq.data_ptr(),
                                     positions.data_ptr(), slots.data_ptr(), cache.data_ptr(), T, rank, rot,
                                     int(rot_dims), float(magnitude), float(eps), _code(z.dtype), zq, wq, cq, q_rank,
                                     _stream()),
          "latent_kv_store")
    _count("latent_kv_store" + (".q_norm" if q_latent is not None else ""))


def latent_q_rope(q: torch.Tensor, qa: torch.Tensor, inv_freq: torch.Tensor, rot_dims: int, magnitude: float,
                  positions: torch.Tensor, n_heads: int, d_plain: int, rot: int, rank: int) -> torch.Tensor:
    """qa[t, h, rank:] = the rotated part q[t, h, d_plain:] after rotation, in float32.  q [T, nh (d_plain
    + rot)] in the activation type; qa [T, nh (rank + rot)] float32, or bfloat16 for the tensor-core
    attention kernels."""
    T = q.shape[0]
    _req(q, "q", None, (T, n_heads * (d_plain + rot)))
    _req(qa, "qa", None, (T, n_heads * (rank + rot)))
    if qa.dtype not in (torch.float32, torch.bfloat16) or (qa.dtype == torch.bfloat16 and q.dtype != torch.bfloat16):
        raise KernelError(f"latent_q_rope: qa of {qa.dtype} for q of {q.dtype} is not taken")
    _req(inv_freq, "inv_freq", torch.float32, (rot_dims // 2,))
    _req(positions, "positions", torch.int32, (T,))
    check(lib().rlis_latent_q_rope(q.data_ptr(), qa.data_ptr(), inv_freq.data_ptr(), positions.data_ptr(), T,
                                   n_heads, d_plain, rot, int(rot_dims), rank, float(magnitude), _code(q.dtype),
                                   1 if qa.dtype == torch.bfloat16 else 0, _stream()), "latent_q_rope")
    _count("latent_q_rope")
    return qa


LATENT_DECODE_CTAS_PER_SM = 2   # debug switch "latent_ctas_per_sm": how full decode attention over latents fills the SMs
LATENT_MMA = True          # debug switch "latent_mma": 0 takes the one-warp-a-row kernel for every size


def latent_attention_takes_mma(dtype, dk: int, rank: int) -> bool:
    """Whether the tensor-core kernels for attention over latent rows exist for these sizes."""
    return bool(LATENT_MMA and dtype == torch.bfloat16 and _latent_mma_sizes(int(dk), int(rank)))


@functools.lru_cache(maxsize=None)
def _latent_mma_sizes(dk: int, rank: int) -> bool:
    return bool(lib().rlis_attention_latent_mma_takes(dk, rank))


@functools.lru_cache(maxsize=4096)
def _latent_decode_pieces(n_decode: int, head_tiles: int, max_ctx: int, sms: int) -> tuple:
    """(pieces, keys a piece) for decode attention over latent rows: a CTA takes 16 heads of one
    token and two fit an SM's shared memory, so the context is cut until the CTAs about fill the SMs
    twice, in pieces that are multiples of 64 keys and at least 128 long."""
    ctas = max(1, n_decode * head_tiles)
    want = max(1, min(LATENT_DECODE_CTAS_PER_SM * sms // ctas, max_ctx // 128))
    keys = -(-max_ctx // want)
    keys = -(-keys // 64) * 64
    return max(1, -(-max_ctx // keys)), keys


def latent_decode_pieces(n_decode: int, n_heads: int, max_ctx: int) -> tuple:
    return _latent_decode_pieces(int(n_decode), (int(n_heads) + 15) // 16, max(1, int(max_ctx)), num_sms())


def _latent_step_takes_mma(step, dtype, dk: int, rank: int) -> bool:
    """Whether every token of the step goes to the tensor-core kernels: the sizes fit, and the step's
    prompt portions (if any) are listed in tiles."""
    n_dec, n_tiles = getattr(step, "n_decode", 0), getattr(step, "n_prefill_tiles", 0)
    return bool(latent_attention_takes_mma(dtype, dk, rank) and (n_dec or n_tiles)
                and (n_tiles or not getattr(step, "n_prefill_tokens", 0)))


def latent_attention_queries_dtype(step, dtype, dk: int, rank: int):
    """The element type `attention_latent` wants its folded queries in for this step: bfloat16 when all
    of it goes to the tensor-core kernels (they copy the queries into shared memory as they are),
    float32 otherwise."""
    return torch.bfloat16 if _latent_step_takes_mma(step, dtype, dk, rank) else torch.float32


def attention_latent(qa: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, step, group: int, n_heads: int,
                     rank: int, page_size: int, scale: float, sinks: torch.Tensor | None = None,
                     window: int = 0) -> torch.Tensor:
    """Causal attention of every token of the step over its request's cached latent rows, which all
    heads share: score = scale * qa[t, h] . row, out[t, h] = sum of softmax weights times row[:rank].
    `sinks` float32 [nh]: exp(sink_h) joins the denominator of head h and nothing else.  qa float32
    [T, nh dk] (bfloat16 is taken too when the whole step goes to the tensor-core kernels, see
    `latent_attention_queries_dtype`); cache [pages, 1, page_size, dk]; out [T, nh rank] in the cache's type.

    bfloat16 with sizes the tensor-core kernels take: single decoded tokens go to the split decode
    kernel, portions of prompts (the step's tile list) to the flash kernel.  Everything else, and all
    of float32, to the kernel that takes one warp a (token, head)."""
    T = qa.shape[0]
    dk = cache.shape[-1]
    _req(qa, "qa", None, (T, n_heads * dk))
    _req(cache, "cache", None, (None, 1, page_size, dk))
    _req(out, "out", cache.dtype, (T, n_heads * rank))
    if sinks is not None:
        _req(sinks, "sinks", torch.float32, (n_heads,))
    if qa.dtype != latent_attention_queries_dtype(step, cache.dtype, dk, rank) and qa.dtype != torch.float32:
        raise KernelError(f"attention_latent: queries of {qa.dtype} where this step takes float32")
    q16 = 1 if qa.dtype == torch.bfloat16 else 0
    tables = step.block_tables[group]
    sink_ptr = sinks.data_ptr() if sinks is not None else None
    n_dec = getattr(step, "n_decode", 0)
    n_tiles = getattr(step, "n_prefill_tiles", 0)
    if _latent_step_takes_mma(step, cache.dtype, dk, rank):
        if n_dec:
            pieces, keys = latent_decode_pieces(n_dec, n_heads, step.max_decode_ctx)
            scratch = None
            if pieces > 1:
                scratch = step.buffer("latent_partial", (n_dec * ((n_heads + 15) // 16) * pieces * 16 * (rank + 2),),
                                      torch.float32)
            check(lib().rlis_attention_latent_decode(
                qa.data_ptr(), q16, cache.data_ptr(), out.data_ptr(), sink_ptr,
                scratch.data_ptr() if scratch is not None else None, step.dec_rows.data_ptr(),
                step.dec_seqs.data_ptr(), step.ctx_lens.data_ptr(), tables.data_ptr(), tables.shape[1], n_dec,
                n_heads, dk, rank, page_size, float(scale), int(window), pieces, keys, _stream()),
                "attention_latent_decode")
            _count("attention_latent.decode.mma" + (".split" if pieces > 1 else ""))
        if n_tiles:
            check(lib().rlis_attention_latent_prefill(
                qa.data_ptr(), q16, cache.data_ptr(), out.data_ptr(), sink_ptr, step.prefill_tiles.data_ptr(), n_tiles,
                step.cu_seqlens.data_ptr(), step.ctx_lens.data_ptr(), tables.data_ptr(), tables.shape[1], n_heads,
                dk, rank, page_size, float(scale), int(window), _stream()), "attention_latent_prefill")
            _count("attention_latent.prefill.mma")
        return out
    check(lib().rlis_attention_latent(qa.data_ptr(), cache.data_ptr(), out.data_ptr(), sink_ptr,
                                      step.seq_of_token.data_ptr(), step.positions.data_ptr(), tables.data_ptr(),
                                      None, tables.shape[1], T, n_heads, dk, rank, page_size, float(scale),
                                      int(window), _code(cache.dtype), _stream()), "attention_latent")
    _count("attention_latent")
    return out


LIGHTNING_SILU_PASS_TOKENS = 64


def lightning_scan(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, out: torch.Tensor, state: torch.Tensor,
                   decay: torch.Tensor, step, n_heads: int, d: int, dv: int) -> torch.Tensor:
    """The decayed linear-attention recurrence over the step's tokens: per request and head
    S <- decay_h S + k v^T, o = S^T q, with q, k, v = silu of columns q_off.., k_off.., v_off.. of
    `proj` [T, *].  `state` float32 [slots, nh, dv, d] holds S, transposed, between steps (a request
    whose first token is in this step starts from zero); out float32 [T, nh dv]."""
    T = proj.shape[0]
    _req(proj, "proj")
    _req(out, "out", torch.float32, (T, n_heads * dv))
    _req(state, "state", torch.float32, (None, n_heads, dv, d))
    _req(decay, "decay", torch.float32, (n_heads,))
    if max(q_off, k_off) + n_heads * d > proj.shape[1] or v_off + n_heads * dv > proj.shape[1]:
        raise KernelError("lightning_scan: the column offsets reach beyond the projection's rows")
    # Steps of many tokens: silu is applied once, into a float32 buffer that every CTA of a head then
    # reads (each would otherwise apply it to the head's q and k again).
    activated = None
    if T >= LIGHTNING_SILU_PASS_TOKENS and q_off == 0 and k_off <= v_off and hasattr(step, "buffer"):
        activated = step.buffer("lightning_act", (T, v_off + n_heads * dv), torch.float32)
    check(lib().rlis_lightning_scan(proj.data_ptr(), proj.stride(0), q_off, k_off, v_off, out.data_ptr(),
                                    state.data_ptr(), decay.data_ptr(), step.cu_seqlens.data_ptr(),
                                    step.ctx_lens.data_ptr(), step.state_slots.data_ptr(), step.n_seqs, n_heads, d,
                                    dv, _code(proj.dtype), activated.data_ptr() if activated is not None else None,
                                    T, _stream()), "lightning_scan")
    _count("lightning_scan" + (".silu_pass" if activated is not None else ""))
    return out


def recurrence_inputs(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, out: torch.Tensor, n_heads: int, d: int,
                      dv: int, rotation: tuple | None = None, positions: torch.Tensor | None = None,
                      k_scale: float = 1.0, q_silu: bool = False, lower: torch.Tensor | None = None,
                      gate_bias: torch.Tensor | None = None) -> torch.Tensor:
    """The float32 inputs of a linear recurrence, one row [q | k | v (| a)] a token, from the rows of a stacked
    projection `proj` [T, N] (queries at column q_off, keys at k_off: n_heads heads of d; values at v_off: heads of
    dv).  `rotation` = (float32 frequencies [r / 2], r): entry i < r / 2 of every query and key head turns with
    entry i + r / 2 by the angle positions[t] * frequency i.  Keys are multiplied by `k_scale`; `q_silu`: q =
    silu(q).  `lower` (float32 [n_heads d]): the columns at k_off are the logits z of a forget gate a = lower + (1 -
    lower) sigmoid(z + gate_bias); the row then holds k = 1 - a and, as a fourth segment, a."""
    T, N = proj.shape
    qk, hv = n_heads * d, n_heads * dv
    _req(proj, "proj")
    _req(out, "out", torch.float32, (T, 2 * qk + hv + (qk if lower is not None else 0)))
    if max(q_off, k_off) + qk > N or v_off + hv > N:
        raise KernelError("recurrence_inputs: the column offsets reach beyond the projection's rows")
    inv_freq, rot_dims = rotation if rotation is not None else (None, 0)
    if rot_dims:
        _req(inv_freq, "rotation frequencies", torch.float32, (rot_dims // 2,))
        _req(positions, "positions", torch.int32, (T,))
        if rot_dims % 2 or rot_dims > d or q_silu or lower is not None:
            raise KernelError(f"recurrence_inputs: {rot_dims} rotated entries do not fit plain heads of {d} in pairs")
    for v, nm in ((lower, "lower"), (gate_bias, "gate_bias")):
        if v is not None:
            _req(v, nm, torch.float32, (qk,))
    check(lib().rlis_recurrence_inputs(proj.data_ptr(), proj.stride(0), int(q_off), int(k_off), int(v_off), out.data_ptr(),
                                       T, n_heads, d, dv, inv_freq.data_ptr() if rot_dims else None, int(rot_dims),
                                       positions.data_ptr() if rot_dims else None, float(k_scale), 1 if q_silu else 0,
                                       lower.data_ptr() if lower is not None else None,
                                       gate_bias.data_ptr() if gate_bias is not None else None, _code(proj.dtype),
                                       _stream()), "recurrence_inputs")
    _count("recurrence_inputs" + (".rot" if rot_dims else "") + (".gate" if lower is not None else ""))
    return out


def recurrence_scan(rows: torch.Tensor, out: torch.Tensor, state: torch.Tensor, decay: torch.Tensor | None, step,
                    n_heads: int, d: int, dv: int, complement_key: bool = False) -> torch.Tensor:
    """The linear recurrence over the step's tokens from prepared float32 rows [T, q | k | v (| a)] (see
    `recurrence_inputs`): per request and head S <- diag(a_t) S + k_t v_t^T, o_t = S^T q_t, with a_t = decay[head]
    for every channel (`decay` float32 [n_heads]) or, with `decay` None, the rows' fourth segment.  `state` float32
    [slots, nh, dv, d] holds S, transposed, between steps (a request whose first token is in this step starts from
    zero); out float32 [T, nh dv].  `complement_key` (with a decay a channel): the rows' keys are 1 - a, as a forget
    gate's are, and the walk takes them from the decays instead of staging them (a stage then holds twice the tokens)."""
    T, W = rows.shape
    qk, hv = n_heads * d, n_heads * dv
    _req(rows, "rows", torch.float32, (T, 2 * qk + hv + (qk if decay is None else 0)))
    _req(out, "out", torch.float32, (T, hv))
    _req(state, "state", torch.float32, (None, n_heads, dv, d))
    if decay is not None:
        _req(decay, "decay", torch.float32, (n_heads,))
    check(lib().rlis_recurrence_scan(rows.data_ptr(), W, 0, qk, 2 * qk, 2 * qk + hv, out.data_ptr(), state.data_ptr(),
                                     decay.data_ptr() if decay is not None else None, step.cu_seqlens.data_ptr(),
                                     step.ctx_lens.data_ptr(), step.state_slots.data_ptr(), step.n_seqs, n_heads, d, dv,
                                     1 if (complement_key and decay is None) else 0, _stream()), "recurrence_scan")
    _count("recurrence_scan" + (".channel_decay" if decay is None else ""))
    return out


RECURRENCE_INPUT_PASS_TOKENS = 64   # steps of this many tokens and more make the recurrence's inputs in a pass of their own


def recurrence_scan_rows(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, out: torch.Tensor, state: torch.Tensor,
                         decay: torch.Tensor | None, step, n_heads: int, d: int, dv: int, rotation: tuple | None = None,
                         k_scale: float = 1.0, lower: torch.Tensor | None = None,
                         gate_bias: torch.Tensor | None = None) -> torch.Tensor:
    """`recurrence_inputs` and `recurrence_scan` in one kernel, for short steps: the walk makes its inputs from the
    projection's rows while it stages them.  With `decay` (float32 [n_heads]): q and k rotated by halves at the tokens'
    positions (`rotation` = (frequencies, r)), k times `k_scale`.  With `lower` (and no `decay`): q = silu(q), the forget
    gate a = lower + (1 - lower) sigmoid(z + gate_bias) from the columns at k_off is the decay a channel and k = 1 - a."""
    T, N = proj.shape
    qk, hv = n_heads * d, n_heads * dv
    _req(proj, "proj")
    _req(out, "out", torch.float32, (T, hv))
    _req(state, "state", torch.float32, (None, n_heads, dv, d))
    if (decay is None) == (lower is None):
        raise KernelError("recurrence_scan_rows: a decay a head, or the lower bounds of a forget gate")
    if max(q_off, k_off) + qk > N or v_off + hv > N:
        raise KernelError("recurrence_scan_rows: the column offsets reach beyond the projection's rows")
    inv_freq, rot_dims = rotation if rotation is not None else (None, 0)
    if rot_dims:
        _req(inv_freq, "rotation frequencies", torch.float32, (rot_dims // 2,))
        if rot_dims % 2 or rot_dims > d or lower is not None:
            raise KernelError(f"recurrence_scan_rows: {rot_dims} rotated entries do not fit plain heads of {d} in pairs")
    for v, nm, n in ((decay, "decay", n_heads), (lower, "lower", qk), (gate_bias, "gate_bias", qk)):
        if v is not None:
            _req(v, nm, torch.float32, (n,))
    ptr = lambda t: t.data_ptr() if t is not None else None
    check(lib().rlis_recurrence_scan_rows(proj.data_ptr(), proj.stride(0), int(q_off), int(k_off), int(v_off), out.data_ptr(),
                                          state.data_ptr(), ptr(decay), step.cu_seqlens.data_ptr(), step.ctx_lens.data_ptr(),
                                          step.state_slots.data_ptr(), step.n_seqs, n_heads, d, dv,
                                          inv_freq.data_ptr() if rot_dims else None, int(rot_dims), float(k_scale), ptr(lower),
                                          ptr(gate_bias), _code(proj.dtype), _stream()), "recurrence_scan_rows")
    _count("recurrence_scan_rows" + (".channel_decay" if decay is None else ""))
    return out


FUSE_NORMS = True          # debug switch "fuse_norms": 0 runs every norm as a kernel
STREAM_MAX_ROWS = 128     # what the weight-streaming kernel takes
DECODE_GEMM_ROWS = 16     # up to this many rows its sink epilogue works: the norms go into the products
STREAM_GEMM_ROWS = 16     # up to this many rows `linear` uses it; longer batches go to the library GEMM
                          # (debug switch "stream_rows"; measured in the decode step with 32 rows: at the 1B
                          # sizes, context 4096, 1.540 ms with it and 1.541 ms with the library; at the 8B
                          # sizes, two layers, context 8192, 0.863 against 0.770 ms; with 48 and 64 rows at
                          # the 1B sizes 1.976 and 2.369 ms against 1.894 and 2.226 ms)


class ScaledRows:
    """Rows of a norm's output whose scale is still to be applied: `x` = bf16(resid * weight) [T, dim]
    and `partials` float32 [P, T], the sums of resid^2 over P slices of the width.  The product that
    takes them multiplies its result by 1 / sqrt(sum of a row's partials / dim + eps): the norm
    between two decode products without a kernel of its own.  Made by `stream_gemm(..., sink=)`."""

    def __init__(self, x, partials, dim, eps):
        self.x, self.partials, self.dim, self.eps = x, partials, int(dim), float(eps)

    shape = property(lambda self: self.x.shape)
    dtype = property(lambda self: self.x.dtype)
    device = property(lambda self: self.x.device)


class ResidualSink:
    """Where the last product of a part may put its result itself: added to the float32 residual
    stream `resid` [T, dim] in place, and handed on as the ScaledRows of the RMSNorm that follows
    (`weight` float32 [dim], `eps`)."""

    def __init__(self, resid, weight, eps):
        self.resid, self.weight, self.eps = resid, weight, float(eps)


def stream_gemm(x, w: torch.Tensor, out_dtype=torch.bfloat16, swiglu4: bool = False, sink: ResidualSink | None = None,
                slope: float = 1.0):
    """y = x @ w^T for at most 128 rows of bfloat16 x: the decode step's weight-streaming product on
    the tcgen05 tensor cores (TMA-fed, weights as the M side, k split over CTAs).  `swiglu4`: w is a
    gate|up matrix interleaved in blocks of 4 rows and the result is silu(gate) * up, [M, N / 2]; with a `slope`,
    gate sigmoid(slope gate) * up (+inf: max(gate, 0) * up).  `x` may be ScaledRows: the rows' scale is applied to the result.  `sink` (up to 16 rows): the
    result, rounded to bfloat16, is added to sink.resid in place and the ScaledRows of the norm that
    follows are returned instead of y."""
    scaled = x if isinstance(x, ScaledRows) else None
    if scaled is not None:
        x = scaled.x
    M, K = x.shape
    N = w.shape[0]
    _req(x, "x", torch.bfloat16)
    _req(w, "w", torch.bfloat16, (N, K))
    if M > STREAM_MAX_ROWS or K % 8 or (swiglu4 and N % 8):
        raise KernelError(f"stream_gemm: takes up to {STREAM_MAX_ROWS} rows and K a multiple of 8, got M={M}, K={K}")
    if scaled is None and sink is None:
        out = torch.empty((M, N // 2 if swiglu4 else N), dtype=out_dtype, device=x.device)
        check(lib().rlis_stream_gemm_bf16(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, _code(out_dtype),
                                          1 if swiglu4 else 0, float(slope), _stream()), "stream_gemm")
        _count("stream_gemm.swiglu" if swiglu4 else "stream_gemm")
        return out
    in_p, n_p, dim, eps = 0, 0, 0, 0.0
    if scaled is not None:
        if sink is not None:
            raise KernelError("stream_gemm: scaled rows into a sink are not supported")
        n_p = scaled.partials.shape[0]
        _req(scaled.partials, "partials", torch.float32, (n_p, M))
        if scaled.dim != K:
            raise KernelError(f"stream_gemm: scaled rows of width {scaled.dim} for a product over {K}")
        in_p, dim, eps = scaled.partials.data_ptr(), scaled.dim, scaled.eps
    if sink is None:
        out = torch.empty((M, N // 2 if swiglu4 else N), dtype=out_dtype, device=x.device)
        check(lib().rlis_stream_gemm_fused(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, _code(out_dtype),
                                           1 if swiglu4 else 0, in_p, n_p, dim, eps, 0, 0, 0, 0, float(slope), _stream()),
              "stream_gemm")
        _count("stream_gemm.scaled.swiglu" if swiglu4 else "stream_gemm.scaled")
        return out
    if swiglu4 or M > DECODE_GEMM_ROWS:
        raise KernelError(f"stream_gemm: a sink takes a plain product of up to {DECODE_GEMM_ROWS} rows")
    _req(sink.resid, "sink.resid", torch.float32, (M, N))
    _req(sink.weight, "sink.weight", torch.float32, (N,))
    xn = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    partials = torch.empty(((N + 127) // 128, M), dtype=torch.float32, device=x.device)
    check(lib().rlis_stream_gemm_fused(x.data_ptr(), w.data_ptr(), 0, M, N, K, _code(torch.bfloat16), 2, 0, 0, 0, 0.0,
                                       sink.resid.data_ptr(), sink.weight.data_ptr(), xn.data_ptr(),
                                       partials.data_ptr(), 1.0, _stream()), "stream_gemm")
    _count("stream_gemm.sink")
    return ScaledRows(xn, partials, N, sink.eps)


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, epilogue: str = "plain", glu: tuple | None = None) -> torch.Tensor:
    """y = x @ w^T on the tcgen05 tensor cores (TMA-fed, accumulator in tensor memory), bfloat16
    operands.  epilogue "plain": bf16 [M, N]; "float32": float32 [M, N]; "swiglu4": w is a gate|up
    matrix interleaved in blocks of 4 rows and the result is silu(gate) * up, bf16 [M, N / 2]; "glu4":
    the same layout with the gating of `glu` = (slope, limit or None, up_shift), see `glu_act`."""
    M, K = x.shape
    N = w.shape[0]
    _req(x, "x", torch.bfloat16)
    _req(w, "w", torch.bfloat16, (N, K))
    code = {"plain": 0, "swiglu4": 1, "float32": 2, "glu4": 3}[epilogue]
    gated = code in (1, 3)
    if M < 128 or N < 256 or K % 8 or N % (16 if gated else 8):
        raise KernelError(f"gemm_tcgen05: takes M >= 128, N >= 256, K a multiple of 8 and N a multiple of 8 "
                          f"(16 with a gated epilogue); got M={M}, N={N}, K={K}")
    out = torch.empty((M, N // 2 if gated else N), dtype=torch.float32 if code == 2 else torch.bfloat16,
                      device=x.device)
    if code == 3:
        slope, limit, shift = glu
        check(lib().rlis_gemm_tcgen05_glu(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, float(slope),
                                          float("inf") if limit is None else float(limit), float(shift), _stream()),
              "gemm_tcgen05")
    else:
        check(lib().rlis_gemm_tcgen05(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, code, _stream()),
              "gemm_tcgen05")
    _count("gemm_tcgen05." + epilogue)
    return out


def take_device_errors(out: torch.Tensor) -> torch.Tensor:
    """Reads and clears, in stream order, the error words of the kernels' bounded waits and leaves
    their union in `out` (int32 [1] on the device): non-zero when a wait ran out in a kernel launched
    before this call and after the last one.  No synchronisation; copy `out` to the host with
    whatever else the step brings back."""
    _req(out, "out", torch.int32, (1,))
    check(lib().rlis_take_errors(out.data_ptr(), _stream()), "take_errors")
    _count("take_errors")
    return out


def stream_timeline(on: bool) -> None:
    """Switches the streaming products' timeline on or off (and empties it): the first CTA of every
    launch stamps the device's global timer at its phases.  A measurement tool; synchronises.  Only in
    a library built with it: set RLIS_TIMELINE=1 in the environment before the first use."""
    torch.cuda.synchronize()
    check(lib().rlis_stream_gemm_timeline(1 if on else 0), "stream_timeline")


def read_stream_timeline(last: int) -> list:
    """The last `last` launches of the streaming product (oldest first), each a dict with N, K and,
    in nanoseconds of the global timer: start, wait_passed (the kernel before has finished),
    products_done, cluster_barrier, sent, sums_arrived (the last three None for a launch that does
    not split k), end, and grid_before_done: the latest end of any CTA of the streaming product launched
    before this one (meaningful when that product is the kernel right before)."""
    import ctypes
    torch.cuda.synchronize()
    buf = (ctypes.c_ulonglong * (512 * 10))()
    n = ctypes.c_uint(0)
    check(lib().rlis_stream_gemm_timeline_read(buf, ctypes.byref(n)), "stream_timeline_read")
    count = min(int(last), n.value, 512)
    out = []
    for i in range(n.value - count, n.value):
        r = buf[(i % 512) * 10:(i % 512) * 10 + 10]
        split = r[3] >= r[2] and r[3] <= r[7]          # records of launches without a split keep stale stamps there
        out.append({"N": int(r[6] // 100000), "K": int(r[6] % 100000), "start": int(r[0]), "wait_passed": int(r[1]),
                    "products_done": int(r[2]), "cluster_barrier": int(r[3]) if split else None,
                    "sent": int(r[4]) if split else None, "sums_arrived": int(r[5]) if split else None,
                    "end": int(r[7]), "grid_before_done": int(r[8])})
    return out


def check_device_errors() -> None:
    """Raises if a bounded wait inside a kernel ever ran out on this device (the kernel then
    finished without its data; results since are not to be trusted).  Synchronises the device."""
    code = (lib().rlis_gemm_tcgen05_error() or lib().rlis_stream_gemm_error() or lib().rlis_attention_prefill_tc_error()
            or lib().rlis_attention_decode_error())
    if code != 0:
        raise KernelError(f"a bounded mbarrier wait of a tcgen05 kernel ran out on the device (code {code})")


def fuses_norms(n_rows: int, dtype, *widths: int) -> bool:
    """Whether products over `widths` of a step of `n_rows` rows go to the kernel that takes
    ScaledRows and a ResidualSink."""
    return (FUSE_NORMS and dtype == torch.bfloat16 and 0 < n_rows <= DECODE_GEMM_ROWS
            and all(w % 8 == 0 for w in widths))


def linear(x, w: torch.Tensor, out_dtype=None, sink: ResidualSink | None = None):
    """y = x @ w^T for w stored (out, in).  float32: this package's FFMA kernel.  bfloat16: up to
    16 rows go to this package's weight-streaming tcgen05 kernel, more to the library GEMM; both
    accumulate in float32, and `out_dtype=torch.float32` keeps that precision (used for logits).
    ScaledRows as x and a `sink` are for the streaming kernel only (see `fuses_norms`)."""
    if isinstance(x, ScaledRows) or sink is not None:
        if not fuses_norms(x.shape[0], x.dtype, x.shape[1]):
            raise KernelError("linear: scaled rows or a sink with a product that does not take them")
        return stream_gemm(x, w, out_dtype or torch.bfloat16, sink=sink)
    if x.dtype == torch.float32:
        return gemm_f32(x, w)
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"linear: expected matching float32 or bfloat16 operands, got {x.dtype}, {w.dtype}")
    if not x.is_cuda:
        raise KernelError("linear: expected CUDA tensors; there is no CPU path")
    if x.shape[1] % 8 == 0 and x.is_contiguous() and (
            x.shape[0] <= STREAM_GEMM_ROWS or (x.shape[0] <= STREAM_MAX_ROWS and w.shape[0] >= 256 * num_sms())):
        # few rows, or up to 128 rows over a matrix so tall that the streaming kernel does not split k
        # (two tiles of 128 features an SM and more: an LM head).  Measured at 128256 x 2048: 48 rows
        # 88 against 97 us for the library, 64 rows 91 against 99, 128 rows 104 against 111; at 17 to
        # 32 rows the two are within 1 us.
        return stream_gemm(x, w, out_dtype or torch.bfloat16)
    if out_dtype is None or out_dtype == torch.bfloat16:
        return torch.mm(x, w.t())
    return torch.mm(x, w.t(), out_dtype=out_dtype)


def rope_cache(qkv: torch.Tensor, q_out: torch.Tensor, k_cache: torch.Tensor | None,
               v_cache: torch.Tensor | None, positions: torch.Tensor, slots: torch.Tensor | None,
               inv_freq: torch.Tensor | None, n_heads: int, n_kv_heads: int, head_dim: int,
               page_size: int) -> torch.Tensor:
    """Rotates q and k by their positions and stores k, v at `slots` of one layer's paged cache.

    qkv [T, (nh + 2 nkv) d]; q_out [T, nh d]; caches [pages, nkv, page_size, d]; positions and
    slots int32 [T] (slots None: nothing is stored); inv_freq float32 [d/2] (None: no rotation)."""
    T = qkv.shape[0]
    _req(qkv, "qkv", None, (T, (n_heads + 2 * n_kv_heads) * head_dim))
    _req(q_out, "q_out", qkv.dtype, (T, n_heads * head_dim))
    _req(positions, "positions", torch.int32, (T,))
    if slots is not None:
        _req(slots, "slots", torch.int32, (T,))
        for c, nm in ((k_cache, "k_cache"), (v_cache, "v_cache")):
            _req(c, nm, qkv.dtype, (None, n_kv_heads, page_size, head_dim))
    if inv_freq is not None:
        _req(inv_freq, "inv_freq", torch.float32, (head_dim // 2,))
    check(lib().rlis_rope_cache(
        qkv.data_ptr(), q_out.data_ptr(),
        k_cache.data_ptr() if slots is not None else None,
        v_cache.data_ptr() if slots is not None else None,
        positions.data_ptr(), slots.data_ptr() if slots is not None else None,
        inv_freq.data_ptr() if inv_freq is not None else None,
        T, n_heads, n_kv_heads, head_dim, page_size, _code(qkv.dtype), _stream()), "rope_cache")
    _count("rope_cache")
    return q_out


def attention_generic(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                      out: torch.Tensor, seq_of_token: torch.Tensor, positions: torch.Tensor,
                      block_tables: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                      page_size: int, scale: float, window: int = 0,
                      token_rows: torch.Tensor | None = None) -> torch.Tensor:
    """Causal grouped-query attention over paged keys and values for any mix of query lengths.

    q, out [T, nh d]; caches [pages, nkv, page_size, d]; seq_of_token, positions int32 [T];
    block_tables int32 [B, max_blocks].  window 0 = all earlier keys.  `token_rows` (int32):
    compute these rows of the step only."""
    T = q.shape[0]
    _req(q, "q", None, (T, n_heads * head_dim))
    _req(out, "out", q.dtype, (T, n_heads * head_dim))
    _req(k_cache, "k_cache", q.dtype, (None, n_kv_heads, page_size, head_dim))
    _req(v_cache, "v_cache", q.dtype, (None, n_kv_heads, page_size, head_dim))
    _req(seq_of_token, "seq_of_token", torch.int32, (T,))
    _req(positions, "positions", torch.int32, (T,))
    _req(block_tables, "block_tables", torch.int32, (None, None))
    if head_dim % 16 or head_dim > 256:
        raise KernelError(f"attention: head sizes are multiples of 16 up to 256, got {head_dim}")
    if n_heads % n_kv_heads:
        raise KernelError(f"attention: {n_heads} query heads are not a multiple of {n_kv_heads} key/value heads")
    check(lib().rlis_attention_generic(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
        seq_of_token.data_ptr(), positions.data_ptr(), block_tables.data_ptr(),
        token_rows.data_ptr() if token_rows is not None else None,
        block_tables.shape[1], T if token_rows is None else token_rows.shape[0], n_heads,
        n_kv_heads, head_dim, page_size, float(scale), int(window), _code(q.dtype), _stream()),
        "attention_generic")
    _count("attention_generic")
    return out


DECODE_MIN_KEYS_PER_SPLIT = 128


@functools.lru_cache(maxsize=None)
def num_sms() -> int:
    """Streaming multiprocessors of the current device (what the launchers ask the runtime for)."""
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device; there is no CPU path")
    return int(torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count)


def decode_splits(n_decode: int, n_kv_heads: int, max_ctx: int, sms: int | None = None) -> int:
    """How many pieces the context is cut into for decode attention on a device of `sms`
    multiprocessors (None: the current device); see `_decode_splits`."""
    return _decode_splits(n_decode, n_kv_heads, max_ctx, num_sms() if sms is None else int(sms))


@functools.lru_cache(maxsize=4096)
def _decode_splits(n_decode: int, n_kv_heads: int, max_ctx: int, sms: int) -> int:
    """Role of `split_plan`, crates/model/src/paged_attention.rs:21-36, re-tuned by measurement
    (on 148 multiprocessors, which the numbers below are for).  Few requests:
    enough CTAs (kv heads x requests x pieces) to fill the SMs about twice, each piece at least
    128 keys long.  From 64 (request, kv head) pairs on, pieces of at least 512 keys and no more
    than about 384 CTAs; from 256 pairs on, one piece at every context: the pairs fill the SMs by
    themselves, and cutting only adds the merge (batch 32, context 2048: 22.6 us whole, 33.8 us
    in 4 pieces; batch 64, context 4096: 82.5 against 95.9 us).  Up to 8 pieces of a small grid are
    merged inside a thread-block cluster, and clusters of 2, 4 and 8 are the sizes that schedule
    well (batch 8, context 4096: 17.4 us with 4 pieces, 29.2 with 5)."""
    groups = max(1, n_decode * n_kv_heads)
    cluster_max_ctas = 4 * sms     # larger grids merge their pieces through global memory instead
    want = -(-2 * sms // groups)
    min_keys = DECODE_MIN_KEYS_PER_SPLIT
    if groups >= 64:
        want = min(want, max(1, 384 // groups))
        min_keys = 512
    want = max(1, min(want, max_ctx // min_keys, 32))
    if want > 1 and groups * min(want, 8) <= cluster_max_ctas:
        # merged inside a cluster: 2, 4 or 8 pieces; with few requests 8, until a piece gets long
        # (batch 1, context 4096: 6.7 us with 8 pieces in a cluster, 12.6 us with 32 and tickets)
        pieces = 1 << (min(want, 8).bit_length() - 1)
        while 8 <= pieces < 32 and want >= 2 * pieces and max_ctx // pieces > 1536:
            pieces *= 2
        want = pieces
    return want


def attention_decode(q, k_cache, v_cache, out, dec_rows, dec_seqs, ctx_lens, block_tables,
                     n_heads: int, n_kv_heads: int, head_dim: int, page_size: int, scale: float,
                     window: int, splits: int, scratch: torch.Tensor | None) -> torch.Tensor:
    """Attention of single decoded tokens (bfloat16): request i's token sits in row dec_rows[i] of
    q/out and belongs to batch entry dec_seqs[i]; it sees keys 0 .. ctx_lens[seq]-1.  `scratch`:
    float32, at least n_decode * n_heads * splits * (d + 2) elements when splits > 1."""
    n = dec_rows.shape[0]
    _req(q, "q", torch.bfloat16, (None, n_heads * head_dim))
    _req(out, "out", torch.bfloat16, tuple(q.shape))
    _req(k_cache, "k_cache", torch.bfloat16, (None, n_kv_heads, page_size, head_dim))
    _req(v_cache, "v_cache", torch.bfloat16, (None, n_kv_heads, page_size, head_dim))
    for t, nm in ((dec_rows, "dec_rows"), (dec_seqs, "dec_seqs"), (ctx_lens, "ctx_lens")):
        _req(t, nm, torch.int32, (None,))
    _req(block_tables, "block_tables", torch.int32, (None, None))
    if head_dim % 8 or head_dim > 256 or n_heads % n_kv_heads or n_heads // n_kv_heads > 8:
        raise KernelError(f"decode attention: head size {head_dim} / group of {n_heads // max(1, n_kv_heads)} "
                          "heads is not taken (multiples of 8 up to 256, groups up to 8)")
    if splits > 1:
        need = n * n_heads * splits * (head_dim + 2)
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need:
            raise KernelError(f"decode attention: scratch of {need} float32 elements is needed")
    check(lib().rlis_attention_decode_pages(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
        scratch.data_ptr() if splits > 1 else None, dec_rows.data_ptr(), dec_seqs.data_ptr(),
        ctx_lens.data_ptr(), block_tables.data_ptr(), block_tables.shape[1], n, n_heads,
        n_kv_heads, head_dim, page_size, k_cache.shape[0], float(scale), int(window), int(splits),
        _code(q.dtype), _stream()), "attention_decode")
    _count("attention_decode" + _decode_variant())
    return out


def decode_attention_takes_qkv(dtype, n_heads: int, n_kv_heads: int, head_dim: int) -> bool:
    """Whether `attention_decode_from_qkv` exists for these sizes (the tensor-core decode kernel)."""
    return (dtype == torch.bfloat16 and head_dim in (64, 128) and n_heads % n_kv_heads == 0
            and n_heads // n_kv_heads <= 8)


def attention_decode_from_qkv(qkv, k_cache, v_cache, out, step, group: int, inv_freq, store: bool,
                              n_heads: int, n_kv_heads: int, head_dim: int, page_size: int,
                              scale: float, window: int = 0) -> torch.Tensor:
    """Decode attention of a step of single tokens straight from the q|k|v projection
    [T, (nh + 2 nkv) d]: rotates q and each request's newest key (`inv_freq` float32 [d / 2], None:
    no rotation) inside the attention kernel, which also stores the newest key and value at the
    step's slots (`store` False: the layer reads another layer's cache)."""
    T = qkv.shape[0]
    n = step.n_decode
    _req(qkv, "qkv", torch.bfloat16, (T, (n_heads + 2 * n_kv_heads) * head_dim))
    _req(out, "out", torch.bfloat16, (T, n_heads * head_dim))
    _req(k_cache, "k_cache", torch.bfloat16, (None, n_kv_heads, page_size, head_dim))
    _req(v_cache, "v_cache", torch.bfloat16, (None, n_kv_heads, page_size, head_dim))
    if not decode_attention_takes_qkv(qkv.dtype, n_heads, n_kv_heads, head_dim):
        raise KernelError(f"decode attention from q|k|v: head size {head_dim} / {n_heads}:{n_kv_heads} heads is not taken")
    if inv_freq is not None:
        _req(inv_freq, "inv_freq", torch.float32, (head_dim // 2,))
    slots = step.slots[group] if store else None
    tables = step.block_tables[group]
    splits = decode_splits(n, n_kv_heads, step.max_decode_ctx)
    scratch = None
    if splits > 1:
        scratch = step.buffer("attn_partial", (n * n_heads * splits * (head_dim + 2),), torch.float32)
    check(lib().rlis_attention_decode_qkv(
        qkv.data_ptr(), step.positions.data_ptr(), slots.data_ptr() if slots is not None else None,
        inv_freq.data_ptr() if inv_freq is not None else None, k_cache.data_ptr(), v_cache.data_ptr(),
        out.data_ptr(), scratch.data_ptr() if splits > 1 else None, step.dec_rows.data_ptr(),
        step.dec_seqs.data_ptr(), step.ctx_lens.data_ptr(), tables.data_ptr(), tables.shape[1], n, n_heads,
        n_kv_heads, head_dim, page_size, k_cache.shape[0], float(scale), int(window), int(splits),
        _code(qkv.dtype), _stream()),
        "attention_decode_qkv")
    _count("attention_decode_qkv" + _decode_variant())
    return out


@functools.lru_cache(maxsize=None)
def prefill_tile() -> int:
    """Tokens of a portion that one CTA of the flash kernels for prompt portions takes; the step's
    tile list (`attention_prefill`'s `tiles`) is cut to this size."""
    return int(lib().rlis_attention_prefill_tile())


PREFILL_TCGEN05 = True     # debug switch "prefill_tcgen05": 0 takes the mma.sync kernel for every size


def _set_flag(name):
    def setter(value):
        globals()[name] = bool(value)
    return setter


def _set_latent_ctas(value):
    global LATENT_DECODE_CTAS_PER_SM
    LATENT_DECODE_CTAS_PER_SM = max(1, int(value))
    _latent_decode_pieces.cache_clear()


def _set_stream_rows(value):
    global STREAM_GEMM_ROWS
    STREAM_GEMM_ROWS = max(DECODE_GEMM_ROWS, min(int(value), STREAM_MAX_ROWS))


library.PYTHON_SWITCHES.update(biased_mma=_set_flag("BIASED_MMA"), moe_mma=_set_flag("MOE_MMA"),
                               moe_grouped=_set_flag("MOE_GROUPED"), fuse_norms=_set_flag("FUSE_NORMS"), prefill_tcgen05=_set_flag("PREFILL_TCGEN05"),
                               latent_mma=_set_flag("LATENT_MMA"), latent_ctas_per_sm=_set_latent_ctas,
                               stream_rows=_set_stream_rows)


def attention_prefill(q, k_cache, v_cache, out, tiles, cu_seqlens, ctx_lens, block_tables,
                      n_heads: int, n_kv_heads: int, head_dim: int, page_size: int, scale: float,
                      window: int = 0, max_ctx: int = 0) -> torch.Tensor:
    """Causal flash attention of portions of prompts over the paged cache (bfloat16, head sizes 64
    and 128).  tiles int32 [n, 2] = (batch entry, first token of the tile within the entry's
    portion; a tile is `prefill_tile()` tokens); cu_seqlens int32 [B + 1] = rows of the entries' first tokens.  max_ctx: the
    longest context of the step if known (with few tiles and long contexts several CTAs then
    share a tile's keys)."""
    _req(q, "q", torch.bfloat16, (None, n_heads * head_dim))
    _req(out, "out", torch.bfloat16, tuple(q.shape))
    _req(k_cache, "k_cache", torch.bfloat16, (None, n_kv_heads, page_size, head_dim))
    _req(v_cache, "v_cache", torch.bfloat16, (None, n_kv_heads, page_size, head_dim))
    _req(tiles, "tiles", torch.int32, (None, 2))
    _req(cu_seqlens, "cu_seqlens", torch.int32, (None,))
    _req(ctx_lens, "ctx_lens", torch.int32, (None,))
    _req(block_tables, "block_tables", torch.int32, (None, None))
    if head_dim not in (64, 128) or n_heads % n_kv_heads:
        raise KernelError(f"prefill attention: head size {head_dim} is not taken (64 and 128 are)")
    if PREFILL_TCGEN05 and lib().rlis_attention_prefill_tc_takes(n_heads, n_kv_heads, head_dim, page_size):
        # the tcgen05 kernel: head sizes 64 and 128, two or more query heads a kv head, pages that divide a block of keys
        check(lib().rlis_attention_prefill_tc(
            q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), tiles.data_ptr(),
            tiles.shape[0], cu_seqlens.data_ptr(), ctx_lens.data_ptr(), block_tables.data_ptr(),
            block_tables.shape[1], q.shape[0], k_cache.shape[0], n_heads, n_kv_heads, head_dim, page_size,
            float(scale), int(window), _code(q.dtype), int(max_ctx), _stream()), "attention_prefill_tc")
        _count("attention_prefill.tcgen05")
        return out
    check(lib().rlis_attention_prefill(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), tiles.data_ptr(),
        tiles.shape[0], cu_seqlens.data_ptr(), ctx_lens.data_ptr(), block_tables.data_ptr(),
        block_tables.shape[1], n_heads, n_kv_heads, head_dim, page_size, float(scale), int(window),
        _code(q.dtype), _stream()), "attention_prefill")
    _count("attention_prefill.mma")
    return out


def attention(q, k_cache, v_cache, out, step, group: int, n_heads: int, n_kv_heads: int,
              head_dim: int, page_size: int, scale: float, window: int = 0) -> torch.Tensor:
    """Attention of every token of the step over its request's cached keys, by the kernels that
    fit the step.  bfloat16: single decoded tokens go to the split decode kernel, portions of
    prompts to the flash kernel (head sizes 64 and 128); everything else, and all of float32, to
    the kernel for any query length.  The choice never changes the result beyond rounding."""
    tables = step.block_tables[group]
    bf = q.dtype == torch.bfloat16
    dec_fast = bf and step.n_decode > 0 and n_heads // n_kv_heads <= 8 and head_dim % 8 == 0
    pf_fast = bf and step.n_prefill_tiles > 0 and head_dim in (64, 128)
    if dec_fast:
        splits = decode_splits(step.n_decode, n_kv_heads, step.max_decode_ctx)
        scratch = None
        if splits > 1:
            scratch = step.buffer("attn_partial", (step.n_decode * n_heads * splits * (head_dim + 2),), torch.float32)
        attention_decode(q, k_cache, v_cache, out, step.dec_rows, step.dec_seqs, step.ctx_lens, tables,
                         n_heads, n_kv_heads, head_dim, page_size, scale, window, splits, scratch)
    if pf_fast:
        attention_prefill(q, k_cache, v_cache, out, step.prefill_tiles, step.cu_seqlens, step.ctx_lens,
                          tables, n_heads, n_kv_heads, head_dim, page_size, scale, window,
                          getattr(step, "max_ctx_len", 0))
    if dec_fast and pf_fast:
        return out
    if not dec_fast and not pf_fast:
        rows = None                                   # every token of the step
    elif dec_fast:
        if step.n_prefill_tokens == 0:
            return out
        rows = step.prefill_rows                      # the portions only
    else:
        if step.n_decode == 0:
            return out
        rows = step.dec_rows                          # the single tokens only
    return attention_generic(q, k_cache, v_cache, out, step.seq_of_token, step.positions, tables,
                             n_heads, n_kv_heads, head_dim, page_size, scale, window, token_rows=rows)


def glu_act(gate_up: torch.Tensor, out: torch.Tensor, slope: float = 1.0, limit: float | None = None,
            up_shift: float = 0.0, interleave: int = 0) -> torch.Tensor:
    """out[t, i] = g sigmoid(slope g) (u + up_shift) with g = gate_up[t, i] and u = gate_up[t, I + i], both in
    float32 (slope +inf: max(g, 0) (u + up_shift)); with a `limit`, g is cut at limit from above and u clipped to [-limit, limit] first.
    interleave B > 0: blocks of B gate columns each followed by their B columns of u."""
    T, I2 = gate_up.shape
    if I2 % 2:
        raise KernelError(f"glu_act: the stacked gate|up width must be even, got {I2}")
    _req(gate_up, "gate_up")
    _req(out, "out", gate_up.dtype, (T, I2 // 2))
    check(lib().rlis_glu_act(gate_up.data_ptr(), out.data_ptr(), T, I2 // 2, float(slope),
                             float("inf") if limit is None else float(limit), float(up_shift), int(interleave),
                             _code(out.dtype), _stream()), "glu_act")
    _count("glu_act")
    return out


def qk_norm_store(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, q_w, k_w, eps: float, v_other, lam: float,
                  q_out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, slots, n_heads: int,
                  n_kv_heads: int, dim: int, v_dim: int, page_size: int, rotation: tuple | None = None,
                  positions: torch.Tensor | None = None, q_temp: tuple | None = None, rot_half: bool = False,
                  proj_bias: torch.Tensor | None = None) -> torch.Tensor:
    """From the rows of a stacked projection `proj` [T, N] (queries at column q_off, keys at k_off, values
    at v_off): q_out [T, nh dim] = per-head rmsnorm(q) * q_w, and at `slots` of the paged caches the keys
    rmsnorm(k) * k_w and the values, mixed as (1 - lam) v + lam v_other where `v_other` (a [T, nkv v_dim]
    column slice of another projection's rows) is given.  q_w, k_w float32 [dim] or None (no norm); slots
    None: nothing is stored.  Statistics and the mixing are float32.

    `rotation` = (float32 frequencies [r / 2], r, multiplier): before the norm, entries (2i, 2i + 1) of every
    query and key head, i < r / 2, turn by the angle position * frequency i, cos and sin times the multiplier
    (values are taken as projected, so v_off = k_off caches the unrotated keys as values).  `q_temp` = (coef,
    every): queries are multiplied by 1 + coef * ln(floor((p + 1) / every) + 1) at position p.  Both take
    `positions` (int32 [T]).  `rot_half`: entry i turns with entry i + r / 2 instead of its neighbour.  `proj_bias`
    (float32 [N]): added to the queries, keys and values as they are read from `proj`."""
    T, N = proj.shape
    _req(proj, "proj")
    _req(q_out, "q_out", proj.dtype, (T, n_heads * dim))
    for w, nm in ((q_w, "q_w"), (k_w, "k_w")):
        if w is not None:
            _req(w, nm, torch.float32, (dim,))
    if v_off + n_kv_heads * v_dim > N or k_off + n_kv_heads * dim > N or q_off + n_heads * dim > N:
        raise KernelError("qk_norm_store: the column offsets reach beyond the projection's rows")
    if slots is not None:
        _req(slots, "slots", torch.int32, (T,))
        _req(k_cache, "k_cache", proj.dtype, (None, n_kv_heads, page_size, dim))
        _req(v_cache, "v_cache", proj.dtype, (None, n_kv_heads, page_size, v_dim))
    vo, vo_stride = None, 0
    if v_other is not None:
        if (v_other.dtype != proj.dtype or tuple(v_other.shape) != (T, n_kv_heads * v_dim) or v_other.stride(1) != 1
                or not v_other.is_cuda):
            raise KernelError("qk_norm_store: the other layer's values must be [T, nkv v_dim] rows with unit stride")
        vo, vo_stride = v_other.data_ptr(), v_other.stride(0)
    inv_freq, rot_dims, rot_mag = rotation if rotation is not None else (None, 0, 1.0)
    if rot_dims:
        _req(inv_freq, "rotation frequencies", torch.float32, (rot_dims // 2,))
        if rot_dims % 2 or rot_dims > dim:
            raise KernelError(f"qk_norm_store: {rot_dims} rotated entries do not fit heads of {dim} in pairs")
    coef, every = q_temp if q_temp is not None else (0.0, 0)
    if rot_dims or every:
        _req(positions, "positions", torch.int32, (T,))
    if proj_bias is not None:
        _req(proj_bias, "proj_bias", torch.float32, (N,))
    check(lib().rlis_qk_norm_store(proj.data_ptr(), N, int(q_off), int(k_off), int(v_off),
                                   q_w.data_ptr() if q_w is not None else None,
                                   k_w.data_ptr() if k_w is not None else None, float(eps), vo, vo_stride, float(lam),
                                   q_out.data_ptr(), k_cache.data_ptr() if slots is not None else None,
                                   v_cache.data_ptr() if slots is not None else None,
                                   slots.data_ptr() if slots is not None else None, T, n_heads, n_kv_heads, dim, v_dim,
                                   page_size, inv_freq.data_ptr() if rot_dims else None, int(rot_dims), float(rot_mag),
                                   positions.data_ptr() if (rot_dims or every) else None, float(coef), int(every),
                                   1 if rot_half else 0, proj_bias.data_ptr() if proj_bias is not None else None,
                                   _code(proj.dtype), _stream()), "qk_norm_store")
    _count("qk_norm_store" + (".mix" if v_other is not None else "") + (".rot" if rot_dims else ""))
    return q_out


BIASED_MMA = True          # debug switch "biased_mma": 0 takes the one-warp-a-row kernel for every size


@functools.lru_cache(maxsize=None)
def _biased_mma_sizes(dim: int, v_dim: int) -> bool:
    return bool(lib().rlis_attention_bias_mma_takes(dim, v_dim))


def biased_attention_takes_mma(dtype, n_heads: int, n_kv_heads: int, dim: int, v_dim: int) -> bool:
    """Whether the tensor-core kernels for attention with a bias by distance exist for these sizes."""
    return bool(BIASED_MMA and dtype == torch.bfloat16 and n_heads % n_kv_heads == 0
                and _biased_mma_sizes(int(dim), int(v_dim)))


@functools.lru_cache(maxsize=4096)
def _biased_decode_pieces(n_decode: int, n_kv_heads: int, max_ctx: int, sms: int) -> int:
    """Pieces a context is cut into for single tokens: a CTA takes one key/value head of one request, so
    the context is cut until there are about four CTAs an SM, in pieces of at least 128 keys."""
    ctas = max(1, n_decode * n_kv_heads)
    return max(1, min(-(-4 * sms // ctas), max_ctx // 128, 64))


def biased_decode_pieces(n_decode: int, n_kv_heads: int, max_ctx: int) -> int:
    return _biased_decode_pieces(int(n_decode), int(n_kv_heads), max(1, int(max_ctx)), num_sms())


def attention_biased(q, k_cache, v_cache, out, bias, gate, step, group: int, n_heads: int, n_kv_heads: int,
                     dim: int, v_dim: int, page_size: int, scale: float, window: int = 0,
                     sinks: torch.Tensor | None = None, slopes: torch.Tensor | None = None) -> torch.Tensor:
    """Causal grouped-query attention of every token of the step over its request's cached keys:
    score = scale * q . k + bias[min(distance, len(bias) - 1), head] - slopes[head] * distance; a head's
    result is multiplied by sigmoid(gate[t, head]); exp(sinks[head]) joins the softmax's denominator
    (`slopes`, `sinks` float32 [nh] or None).  q [T, nh dim]; k_cache [pages, nkv, page_size, dim]; v_cache [pages, nkv,
    page_size, v_dim]; out [T, nh v_dim]; bias float32 [n_dist, nh] or None; gate [T, nh] (a column slice
    of wider rows) or None.

    bfloat16 with sizes the tensor-core kernels take: single decoded tokens go to the split decode kernel
    (groups of up to 16 query heads), portions of prompts (the step's tile list) to the flash kernel.
    Everything else, and all of float32, to the kernel that takes one warp a (token, head)."""
    T = q.shape[0]
    _req(q, "q", None, (T, n_heads * dim))
    _req(out, "out", q.dtype, (T, n_heads * v_dim))
    _req(k_cache, "k_cache", q.dtype, (None, n_kv_heads, page_size, dim))
    _req(v_cache, "v_cache", q.dtype, (None, n_kv_heads, page_size, v_dim))
    n_dist, bp = 0, None
    if bias is not None:
        _req(bias, "bias", torch.float32, (None, n_heads))
        n_dist, bp = bias.shape[0], bias.data_ptr()
    gp, gs, gc = None, 0, 1
    if gate is not None:
        # one logit a head, or one a channel of every head
        if (gate.dtype != q.dtype or tuple(gate.shape) not in ((T, n_heads), (T, n_heads * v_dim)) or gate.stride(1) != 1
                or not gate.is_cuda):
            raise KernelError("attention_biased: the gate must be [T, nh] or [T, nh v_dim] rows with unit stride in q's type")
        gp, gs = gate.data_ptr(), gate.stride(0)
        gc = v_dim if gate.shape[1] == n_heads * v_dim and v_dim > 1 else 1
    for v, nm in ((sinks, "sinks"), (slopes, "slopes")):
        if v is not None:
            _req(v, nm, torch.float32, (n_heads,))
    sp = sinks.data_ptr() if sinks is not None else None
    lp = slopes.data_ptr() if slopes is not None else None
    tables = step.block_tables[group]
    fast = biased_attention_takes_mma(q.dtype, n_heads, n_kv_heads, dim, v_dim)
    n_dec = getattr(step, "n_decode", 0) if fast and n_heads // n_kv_heads <= 16 else 0
    n_tiles = getattr(step, "n_prefill_tiles", 0) if fast else 0
    if n_dec:
        pieces = biased_decode_pieces(n_dec, n_kv_heads, step.max_decode_ctx)
        scratch = step.buffer("attn_partial", (n_dec * n_heads * pieces * (v_dim + 2),), torch.float32) if pieces > 1 else None
        check(lib().rlis_attention_bias_decode(
            q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
            scratch.data_ptr() if scratch is not None else None, bp, n_dist, gp, gs, step.dec_rows.data_ptr(),
            step.dec_seqs.data_ptr(), step.ctx_lens.data_ptr(), tables.data_ptr(), tables.shape[1], n_dec, n_heads,
            n_kv_heads, dim, v_dim, page_size, float(scale), int(window), pieces, sp, lp, gc, _stream()), "attention_bias_decode")
        _count("attention_bias.decode.mma" + (".split" if pieces > 1 else ""))
    if n_tiles:
        check(lib().rlis_attention_bias_prefill(
            q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), bp, n_dist, gp, gs,
            step.prefill_tiles.data_ptr(), n_tiles, step.cu_seqlens.data_ptr(), step.ctx_lens.data_ptr(),
            tables.data_ptr(), tables.shape[1], n_heads, n_kv_heads, dim, v_dim, page_size, float(scale), int(window),
            sp, lp, gc, _stream()), "attention_bias_prefill")
        _count("attention_bias.prefill.mma")
    # what the tensor-core kernels did not take: nothing, the portions only, the single tokens only, or everything
    rows, n_rows = None, T
    if n_dec and n_tiles:
        return out
    if n_dec:
        if step.n_prefill_tokens == 0:
            return out
        rows, n_rows = step.prefill_rows, step.n_prefill_tokens
    elif n_tiles:
        if getattr(step, "n_decode", 0) == 0:
            return out
        rows, n_rows = step.dec_rows, step.n_decode
    check(lib().rlis_attention_bias(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), bp, n_dist, gp,
                                    gs, step.seq_of_token.data_ptr(), step.positions.data_ptr(), tables.data_ptr(),
                                    rows.data_ptr() if rows is not None else None, tables.shape[1], n_rows, n_heads,
                                    n_kv_heads, dim, v_dim, page_size, float(scale), int(window), sp, lp, gc,
                                    _code(q.dtype), _stream()), "attention_bias")
    _count("attention_bias")
    return out


class MoePlan:
    """Where a step's (token, choice) pairs go: the chosen experts and weights, the pairs sorted by expert
    into slots in tiles of `tile` rows, and the shared expert's gate; all on the device."""

    def __init__(self, **kw):
        self.__dict__.update(kw)


MOE_MMA = True             # debug switch "moe_mma": 0 takes the FFMA products for bfloat16 too


def moe_tile_rows(n_pairs: int, n_experts: int) -> int:
    """Rows of a tile of the sort: 128 when an expert gets about a tile's worth of pairs or more (a prompt's
    portion: wide tiles read the weights fewer times), else 32 (a few tokens: little padding)."""
    return 128 if n_pairs >= 96 * n_experts else 32


MOE_GROUPED = True         # debug switch "moe_grouped": 0 keeps the experts' products over prompts on mma.sync


def _moe_gemm(a, wg_ptr: int, wu_ptr, w_stride: int, interleave: int, out, plan, N: int, K: int, glu: bool,
              slope: float, limit: float, shift: float, name: str):
    """One of the routed products: tensor cores for bfloat16 rows that are 16-byte multiples, FFMA otherwise."""
    args = (a.data_ptr(), wg_ptr, wu_ptr, out.data_ptr(), plan.sorted_pair.data_ptr(), plan.tile_expert.data_ptr(),
            plan.max_tiles, plan.tile, plan.top, N, K, 1 if glu else 0, float(slope), float(limit), float(shift),
            int(w_stride), int(interleave))
    if (MOE_MMA and a.dtype == torch.bfloat16 and K % 8 == 0 and interleave in (0, 4)
            and lib().rlis_moe_mma_takes_tile(plan.tile)):
        check(lib().rlis_moe_gemm_mma(*args, _stream()), name)
        _count("moe_gemm.mma" + (".glu" if glu else ".down"))
    else:
        check(lib().rlis_moe_gemm(*args, _code(a.dtype), _stream()), name)
        _count("moe_gemm" + (".glu" if glu else ".down"))


def moe_route(x: torch.Tensor, w_router: torch.Tensor, correction, n_experts: int, top: int, route_scale: float,
              shared_gate: bool, step, router_bias: torch.Tensor | None = None,
              softmax_chosen: bool = False, scoring: str | None = None, groups: tuple | None = None,
              normalize: bool = False, n_identity: int = 0) -> MoePlan:
    """Scores s = sigmoid(w_router x + router_bias) in float32; the `top` experts with the largest s +
    correction; weights s * route_scale.  `softmax_chosen`: the logits themselves are the scores, and the
    weights are the softmax over the chosen logits alone (times route_scale).  w_router float32 [n_experts (+ 1), width]: with `shared_gate` its last row is the logit
    of the shared expert's gate.  Then the pairs are sorted by expert on the device.

    `scoring` "softmax": s = softmax over all router outputs.  `n_identity`: the router has that many more outputs
    after the experts' (identity experts: they return their input, see `moe_combine`), which are scored and chosen
    like the rest.  `groups` = (count, keep): the outputs form `count` equal groups of neighbours, ranked by their
    largest s + correction, and only outputs of the `keep` best groups can be chosen.  `normalize`: the chosen
    scores are divided by their sum (+ 1e-20) before route_scale."""
    T, W = x.shape
    _req(x, "x")
    n_real, n_experts = n_experts, n_experts + int(n_identity)          # the kernel scores outputs; only experts get slots
    mode = {None: 1 if softmax_chosen else 0, "sigmoid": 0, "softmax_chosen": 1, "softmax": 2}[scoring]
    n_groups, keep = groups if groups is not None else (1, 1)
    rows = n_experts + (1 if shared_gate else 0)
    _req(w_router, "w_router", torch.float32, (rows, W))
    if correction is not None:
        _req(correction, "correction", torch.float32, (n_experts,))
    if router_bias is not None:
        _req(router_bias, "router_bias", torch.float32, (n_experts,))
    pairs = T * top
    tile = moe_tile_rows(pairs, n_real)
    max_tiles = min(pairs, n_real) + pairs // tile         # every expert in use ends in at most one partial tile
    ints = step.buffer("moe_ints", (2 * pairs + max_tiles * tile + max_tiles + 1,), torch.int32)
    flts = step.buffer("moe_floats", (pairs + T,), torch.float32)
    top_idx, pair_slot = ints[:pairs], ints[pairs:2 * pairs]
    sorted_pair = ints[2 * pairs:2 * pairs + max_tiles * tile]
    tile_expert = ints[2 * pairs + max_tiles * tile:]
    top_w, gate = flts[:pairs], flts[pairs:]
    check(lib().rlis_moe_route(x.data_ptr(), w_router.data_ptr(), correction.data_ptr() if correction is not None else None,
                               top_idx.data_ptr(), top_w.data_ptr(), gate.data_ptr() if shared_gate else None, T, W,
                               n_experts, top, float(route_scale),
                               router_bias.data_ptr() if router_bias is not None else None, mode, int(n_groups), int(keep),
                               1 if normalize else 0, _code(x.dtype), _stream()), "moe_route")
    _count("moe_route")
    check(lib().rlis_moe_align(top_idx.data_ptr(), sorted_pair.data_ptr(), pair_slot.data_ptr(), tile_expert.data_ptr(),
                               pairs, n_real, max_tiles, tile, _stream()), "moe_align")
    _count("moe_align")
    return MoePlan(n_tokens=T, top=top, n_experts=n_real, n_identity=int(n_identity), tile=tile, max_tiles=max_tiles, top_idx=top_idx,
                   top_w=top_w, pair_slot=pair_slot, sorted_pair=sorted_pair, tile_expert=tile_expert,
                   shared_gate=gate if shared_gate else None)


def _moe_grouped(plan: MoePlan, dtype, N: int, K: int) -> bool:
    """Whether a routed product of this step goes to the grouped tcgen05 product: bfloat16, the sort's wide
    tiles (its row tile), extents that its tensor maps take."""
    return bool(MOE_GROUPED and dtype == torch.bfloat16 and plan.tile == 128 and K % 8 == 0 and N % 8 == 0 and N >= 256)


def gemm_tcgen05_grouped(x: torch.Tensor, w: torch.Tensor, tile_expert: torch.Tensor, out: torch.Tensor,
                         glu: tuple | None = None) -> torch.Tensor:
    """out[m] = x[m] @ w[e]^T for every row tile of 128 rows of x, e = tile_expert[tile] (-1: the tile is left
    out and its rows of `out` keep what they held; such tiles come last, and tile_expert[M / 128] says how many
    tiles have an expert); on the tcgen05 tensor cores, one SM a tile.  x [M, K]
    bfloat16 with M a multiple of 128; w [experts, N, K] bfloat16 contiguous; out [M, N] bfloat16 or float32.
    With `glu` = (slope, limit or None, up_shift): w's rows are gate and linear branch interleaved in blocks of
    4 and out [M, N / 2] bfloat16 is the gated result (see `glu_act`)."""
    M, K = x.shape
    E, N, _ = w.shape
    _req(x, "x", torch.bfloat16)
    _req(w, "w", torch.bfloat16, (E, N, K))
    _req(tile_expert, "tile_expert", torch.int32, (None,))
    _req(out, "out", torch.bfloat16 if glu is not None else None, (M, N // 2 if glu is not None else N))
    if M % 128 or tile_expert.shape[0] < M // 128 + 1 or out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError(f"gemm_tcgen05_grouped: rows in tiles of 128 with an expert each and their count, got M={M} and "
                          f"{tile_expert.shape[0]} tiles; out in bfloat16 or float32, got {out.dtype}")
    slope, limit, shift = glu if glu is not None else (1.0, None, 0.0)
    code = 3 if glu is not None else 2 if out.dtype == torch.float32 else 0
    check(lib().rlis_gemm_tcgen05_grouped(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, E, tile_expert.data_ptr(),
                                          code, float(slope), float("inf") if limit is None else float(limit),
                                          float(shift), _stream()), "gemm_tcgen05_grouped")
    _count("gemm_tcgen05.grouped" + (".glu4" if glu is not None else ""))
    return out


def moe_up(x: torch.Tensor, w_gate_up: torch.Tensor, plan: MoePlan, slope: float, limit: float, up_shift: float,
           step, interleave: int = 0) -> torch.Tensor:
    """act[slot, :] = glu(w_gate[e] x_t, w_up[e] x_t) for the token t and expert e of every slot (see `glu_act`).
    w_gate_up [experts, 2 I, width] holds both branches of every expert: interleave 0: the I gate rows, then the
    I rows of the linear branch; interleave B > 0: blocks of B gate rows, each followed by its B rows of the
    linear branch (4 is what the gated epilogue of the grouped tcgen05 product over prompts wants).  Returns
    [slots, I] in x's type."""
    T, W = x.shape
    E, I2, _ = w_gate_up.shape
    I = I2 // 2
    _req(x, "x")
    _req(w_gate_up, "w_gate_up", x.dtype, (plan.n_experts, 2 * I, W))
    if interleave < 0 or (interleave > 0 and I % interleave):
        raise KernelError(f"moe_up: blocks of {interleave} rows do not divide {I}")
    S = plan.max_tiles * plan.tile
    act = step.buffer("moe_act", (S, I), x.dtype)
    limit_or_none = None if limit == float("inf") else limit
    if interleave in (0, 4) and _moe_grouped(plan, x.dtype, 2 * I, W) and (interleave == 0 or I % 8 == 0):
        # rows into slot order, then one grouped product for both branches; in blocks of 4 it gates on its
        # accumulators, otherwise the gating is a pass of its own
        xs = step.buffer("moe_rows", (S, W), x.dtype)
        check(lib().rlis_moe_gather_rows(x.data_ptr(), xs.data_ptr(), plan.sorted_pair.data_ptr(), S, plan.top, W,
                                         _code(x.dtype), _stream()), "moe_gather_rows")
        _count("moe_gather_rows")
        if interleave == 4:
            return gemm_tcgen05_grouped(xs, w_gate_up, plan.tile_expert, act, glu=(slope, limit_or_none, up_shift))
        gu = gemm_tcgen05_grouped(xs, w_gate_up, plan.tile_expert, step.buffer("moe_gate_up", (S, 2 * I), x.dtype))
        return glu_act(gu, act, slope, limit_or_none, up_shift)
    rows_to_up = (interleave if interleave > 0 else I) * W * w_gate_up.element_size()
    _moe_gemm(x, w_gate_up.data_ptr(), w_gate_up.data_ptr() + rows_to_up, 2 * I * W, interleave, act, plan, I, W, True,
              slope, limit, up_shift, "moe_up")
    return act


def moe_down(act: torch.Tensor, w_down: torch.Tensor, plan: MoePlan, step) -> torch.Tensor:
    """y[slot, :] = w_down[e] act[slot, :] in float32; w_down [experts, width, I]."""
    S, I = act.shape
    E, W, _ = w_down.shape
    _req(act, "act", None, (plan.max_tiles * plan.tile, I))
    _req(w_down, "w_down", act.dtype, (plan.n_experts, W, I))
    y = step.buffer("moe_y", (S, W), torch.float32)
    if _moe_grouped(plan, act.dtype, W, I):
        return gemm_tcgen05_grouped(act, w_down, plan.tile_expert, y)
    _moe_gemm(act, w_down.data_ptr(), None, W * I, 0, y, plan, W, I, False, 1.0, 0.0, 0.0, "moe_down")
    return y


def moe_combine(y: torch.Tensor, plan: MoePlan, shared, out: torch.Tensor, x: torch.Tensor | None = None) -> torch.Tensor:
    """out[t] = sum over a token's choices of weight * y[slot] (+ gate[t] * shared[t], gate 1 without one),
    summed in float32 in the order of the choices.  A choice beyond the experts (an identity expert of the plan)
    adds weight * x[t]; `x` [T, W] is then the feed-forward's input."""
    T, W = out.shape
    if getattr(plan, "n_identity", 0):
        _req(x, "x", out.dtype, (T, W))
    else:
        x = None
    _req(y, "y", torch.float32, (None, W))
    _req(out, "out")
    if shared is not None:
        _req(shared, "shared", out.dtype, (T, W))
    check(lib().rlis_moe_combine(y.data_ptr(), plan.pair_slot.data_ptr(), plan.top_w.data_ptr(),
                                 shared.data_ptr() if shared is not None else None,
                                 plan.shared_gate.data_ptr() if plan.shared_gate is not None else None, out.data_ptr(),
                                 T, W, plan.top, x.data_ptr() if x is not None else None, plan.top_idx.data_ptr(),
                                 plan.n_experts, _code(out.dtype), _stream()), "moe_combine")
    _count("moe_combine")
    return out


def sample_rows(logits: torch.Tensor, params: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """One token id per row of float32 logits [R, V].  params int32 [R, 2] = (key, bits of 1/T);
    (0, 0) is greedy.  Returns int32 [R]."""
    R, V = logits.shape
    if logits.dtype != torch.float32 or not logits.is_cuda or logits.stride(1) != 1:
        raise KernelError("sample_rows: logits must be float32 CUDA rows with unit stride")
    _req(params, "params", torch.int32, (R, 2))
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    _req(out, "out", torch.int32, (R,))
    check(lib().rlis_sample_rows(logits.data_ptr(), params.data_ptr(), out.data_ptr(), R, V,
                                 logits.stride(0), _stream()), "sample_rows")
    _count("sample_rows")
    return out


def repetition_penalty(logits: torch.Tensor, rows: torch.Tensor, history: torch.Tensor, offsets: torch.Tensor,
                       penalties: torch.Tensor) -> torch.Tensor:
    """In place on float32 logits [R, V]: for row rows[i], every distinct token of
    history[offsets[i]:offsets[i + 1]] has its logit divided by penalties[i] if positive, multiplied
    otherwise (once, however often the token occurs)."""
    R, V = logits.shape
    n = rows.shape[0]
    if logits.dtype != torch.float32 or not logits.is_cuda or logits.stride(1) != 1:
        raise KernelError("repetition_penalty: logits must be float32 CUDA rows with unit stride")
    _req(rows, "rows", torch.int32, (n,))
    _req(history, "history", torch.int32, (None,))
    _req(offsets, "offsets", torch.int32, (n + 1,))
    _req(penalties, "penalties", torch.float32, (n,))
    check(lib().rlis_repetition_penalty(logits.data_ptr(), rows.data_ptr(), history.data_ptr(), offsets.data_ptr(),
                                        penalties.data_ptr(), n, V, logits.stride(0), _stream()), "repetition_penalty")
    _count("repetition_penalty")
    return logits


def sample_filtered(logits: torch.Tensor, params: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """One token id per row of float32 logits [R, V] by temperature sampling with top-k and/or
    top-p filtering on the device.  params int32 [R, 5] = (bits of 1/T, top_k (0: off), bits of
    top_p, low word, high word of a 53-bit uniform).  Returns int32 [R]."""
    R, V = logits.shape
    if logits.dtype != torch.float32 or not logits.is_cuda or logits.stride(1) != 1:
        raise KernelError("sample_filtered: logits must be float32 CUDA rows with unit stride")
    _req(params, "params", torch.int32, (R, 5))
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    _req(out, "out", torch.int32, (R,))
    check(lib().rlis_sample_filtered(logits.data_ptr(), params.data_ptr(), out.data_ptr(), R, V,
                                     logits.stride(0), _stream()), "sample_filtered")
    _count("sample_filtered")
    return out


def nll_rows(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """Negative log-likelihood of targets[r] under softmax(logits[r]); float32 [R]."""
    R, V = logits.shape
    if logits.dtype != torch.float32 or not logits.is_cuda or logits.stride(1) != 1:
        raise KernelError("nll_rows: logits must be float32 CUDA rows with unit stride")
    _req(targets, "targets", torch.int32, (R,))
    out = torch.empty((R,), dtype=torch.float32, device=logits.device)
    check(lib().rlis_nll_rows(logits.data_ptr(), targets.data_ptr(), out.data_ptr(), R, V,
                              logits.stride(0), _stream()), "nll_rows")
    _count("nll_rows")
    return out
