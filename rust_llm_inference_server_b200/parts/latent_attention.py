"""Causal attention over a cache of latents: per token one row [c | k_rot] shared by all heads;
keys and values of a head are linear maps of c."""

from __future__ import annotations

import numpy as np
import torch

from .. import ops
from ..ops.profile import span
from .base import KVCacheSpec, Mixer, build_position, register_mixer


class LatentAttention(Mixer):
    """The key map is folded into the query, so attention runs on the cached rows themselves:

        qa[t, h] = [W_uk_h^T q_plain[t, h] | rotate(q_rot[t, h])]        float32
        lat[t, h] = sum_j softmax_j(scale * qa[t, h] . row_j) * row_j[:kv_rank]
        out = W_o concat_h(W_uv_h lat[t, h])

    which equals scoring against [W_uk_h c_j | k_rot_j] and summing W_uv_h c_j.  Norms of the two
    latents, the rotation, scores, softmax (with the optional sink term) and value sums are float32.
    A spec without `kv_down` stores nothing: its call reads the slot another call has filled."""

    graph_safe = True

    def __init__(self, spec, dtype, device):
        self.spec = spec
        self.dtype = dtype
        self.position = build_position(spec.position, dtype, device)
        rot = getattr(self.position, "rotation", None)
        if getattr(self.position, "pairing", "half") != "half":
            raise ValueError("latent attention rotates entry i with entry i + dims / 2")
        self.inv_freq, self.rot_dims, self.magnitude = rot() if rot is not None else (None, 0, 1.0)
        if self.inv_freq is None:
            self.inv_freq = torch.zeros((0,), dtype=torch.float32, device=device)
        if self.rot_dims > spec.rot_dim:
            raise ValueError(f"the rotation covers {self.rot_dims} entries, the rotated part has {spec.rot_dim}")
        self.eps = float(np.float32(spec.eps))
        self.scale = float(spec.scale)
        self.window = int(spec.window) if spec.window else 0
        self.own_kv = spec.kv_down is not None

    def tensors(self) -> dict:
        s = self.spec
        out = {s.q_down: (s.q_rank, s.hidden), s.q_norm: (s.q_rank,),
               s.q_up: (s.n_heads * (s.dim + s.rot_dim), s.q_rank),
               s.k_up: (s.n_heads * s.dim, s.kv_rank), s.v_up: (s.n_heads * s.v_dim, s.kv_rank),
               s.o_proj: (s.hidden, s.n_heads * s.v_dim)}
        if self.own_kv:
            out[s.kv_down] = (s.kv_rank + s.rot_dim, s.hidden)
            out[s.kv_norm] = (s.kv_rank,)
        if s.sink is not None:
            out[s.sink] = (s.n_heads,)
        return out

    def load(self, src) -> None:
        s = self.spec
        down = [src.get(s.q_down)] + ([src.get(s.kv_down)] if self.own_kv else [])
        self.w_down = torch.cat(down, dim=0).contiguous()          # q latent | kv latent | shared key part
        self.q_norm = src.get(s.q_norm, "vector")
        self.kv_norm = src.get(s.kv_norm, "vector") if self.own_kv else None
        self.w_q_up = src.get(s.q_up).contiguous()
        # [head, kv_rank, dim]: the key map transposed, so that it applies to queries
        self.w_k_fold = src.get(s.k_up).view(s.n_heads, s.dim, s.kv_rank).transpose(1, 2).contiguous()
        self.w_v_up = src.get(s.v_up).view(s.n_heads, s.v_dim, s.kv_rank).contiguous()
        self.w_o = src.get(s.o_proj).contiguous()
        self.sinks = src.get(s.sink, "vector").contiguous() if s.sink is not None else None

    def cache_spec(self):
        s = self.spec
        return KVCacheSpec(1, s.kv_rank + s.rot_dim, s.window, values=False)

    def _mma(self) -> bool:
        s = self.spec
        return ops.latent_attention_takes_mma(self.dtype, s.kv_rank + s.rot_dim, s.kv_rank)

    @property
    def prefill_tile(self):
        # the flash kernel for prompt portions takes one tile of this many tokens a CTA
        return ops.prefill_tile() if self.dtype == torch.bfloat16 and self._mma() else None

    def launch_variant(self, step):
        # decode attention cuts the context into pieces by the longest context of the step
        if not step.n_decode or not self._mma():
            return None
        return ops.latent_decode_pieces(step.n_decode, self.spec.n_heads, step.max_decode_ctx)

    def forward(self, x, step, cache, state, writes_cache=True):
        s = self.spec
        T, H = x.shape[0], s.n_heads
        dk = s.kv_rank + s.rot_dim
        with span("latent down proj"):
            down = ops.linear(x, self.w_down)
        cq = step.buffer("latent_cq", (T, s.q_rank), self.dtype)
        if self.own_kv and writes_cache:
            # one launch: the kv latent's norm, the shared key part's rotation, the paged write, and the
            # query latent's norm
            with span("latent norms + rope + cache write"):
                ops.latent_kv_store(down[:, s.q_rank:], self.kv_norm, self.eps, self.inv_freq, self.rot_dims,
                                    self.magnitude, step.positions, step.slots[cache.group], cache.k, s.kv_rank,
                                    cache.page_size, q_latent=down[:, :s.q_rank], q_weight=self.q_norm, q_out=cq)
        else:
            with span("q latent norm"):
                ops.act_norm(down[:, :s.q_rank], self.q_norm, self.eps, cq)
        with span("q up proj"):
            q = ops.linear(cq, self.w_q_up)
        # float32, or bfloat16 when the whole step goes to the tensor-core attention kernels
        qa_dtype = ops.latent_attention_queries_dtype(step, self.dtype, dk, s.kv_rank)
        qa = step.buffer("latent_qa" if qa_dtype == torch.float32 else "latent_qa16", (T, H * dk), qa_dtype)
        with span("q fold + rope"):
            ops.per_head_linear(q.view(T, H, s.dim + s.rot_dim)[:, :, :s.dim], self.w_k_fold,
                                qa.view(T, H, dk)[:, :, :s.kv_rank])
            ops.latent_q_rope(q, qa, self.inv_freq, self.rot_dims, self.magnitude, step.positions, H, s.dim,
                              s.rot_dim, s.kv_rank)
        lat = step.buffer("latent_o", (T, H * s.kv_rank), self.dtype)
        with span("attention"):
            ops.attention_latent(qa, cache.k, lat, step, cache.group, H, s.kv_rank, cache.page_size, self.scale,
                                 self.sinks, self.window)
        o = step.buffer("attn_o", (T, H * s.v_dim), self.dtype)
        with span("v up proj"):
            ops.per_head_linear(lat.view(T, H, s.kv_rank), self.w_v_up, o.view(T, H, s.v_dim))
        with span("o proj"):
            return ops.linear(o, self.w_o)


register_mixer("latent_attention", LatentAttention)
