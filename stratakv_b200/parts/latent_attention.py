"""Causal attention over one compressed vector per position.

``c = rmsnorm(Wdkv h) * w`` is what the cache keeps (``latent_dim`` numbers a position, cache kind ``latent``).
Head h's keys and values are ``Wuk[h] c`` and ``Wuv[h] c``; they are never made.  Since
``q . (Wuk[h] c) = (Wuk[h]^T q) . c`` and ``sum_j p_j Wuv[h] c_j = Wuv[h] (sum_j p_j c_j)``, the mixer folds the
keys' up-projection into the queries (``headwise_linear`` with the transposed matrices), attends with every head over
the same cached vectors as keys and as values (the attention kernels with one key/value head of ``latent_dim``), and
applies the values' up-projection to each head's result.  No position encoding.
"""
from __future__ import annotations

import torch

from .. import ops as _ops
from ..cache.kinds import CacheKind, register_cache_kind
from .attention import _residual_mode, _residual_stats
from .base import CacheRequest, Mixer, TensorRequest
from .registry import register_mixer

register_cache_kind(CacheKind("latent", paged=True, windowed=False,
                              block_tensors=lambda request, block_size: {"c": (1, block_size, request.head_dim)}))


class LatentAttention(Mixer):
    graph_safe = True
    stores_branch = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if runtime.dtype == torch.bfloat16 and spec.hidden_size % 8 != 0:
            raise ValueError(f"latent attention: hidden size {spec.hidden_size} is not supported in bfloat16 "
                             "(rows of 16 bytes are needed: a multiple of 8); float32 takes any size")
        if spec.latent_dim > 512:
            raise ValueError(f"latent attention: a latent of {spec.latent_dim} numbers is not supported (at most 512)")
        self.q_dim = spec.num_heads * spec.head_dim
        self.ctx_dim = spec.num_heads * spec.v_head_dim
        self.ctx_width = -(-self.ctx_dim // 8) * 8          # whole 16 bytes for the output projection
        self.fused_width = -(-(self.q_dim + spec.latent_dim) // 8) * 8

    @classmethod
    def expected_tensors(cls, spec):
        return {spec.q_weight: TensorRequest((spec.num_heads * spec.head_dim, spec.hidden_size)),
                spec.down_weight: TensorRequest((spec.latent_dim, spec.hidden_size)),
                spec.latent_norm: TensorRequest((spec.latent_dim,), "around_one"),
                spec.k_up_weight: TensorRequest((spec.num_heads * spec.head_dim, spec.latent_dim)),
                spec.v_up_weight: TensorRequest((spec.num_heads * spec.v_head_dim, spec.latent_dim)),
                spec.o_weight: TensorRequest((spec.hidden_size, spec.num_heads * spec.v_head_dim))}

    @classmethod
    def cache_request(cls, spec):
        return CacheRequest("latent", 1, spec.latent_dim)

    def bind(self, tensors):
        s = self.spec
        parts = [self.rt.upload(tensors[s.q_weight]), self.rt.upload(tensors[s.down_weight])]
        rows = sum(part.shape[0] for part in parts)
        if rows < self.fused_width:                 # (zero rows: what they produce is never read)
            parts.append(parts[0].new_zeros(self.fused_width - rows, s.hidden_size))
        self.w_q_down = torch.cat(parts, dim=0).contiguous()
        del parts
        self.latent_gamma = self.rt.upload(tensors[s.latent_norm], torch.float32)
        k_up = self.rt.upload(tensors[s.k_up_weight]).view(s.num_heads, s.head_dim, s.latent_dim)
        self.w_k_up_t = k_up.transpose(1, 2).contiguous()       # [heads, latent, head_dim]: q -> q in latent space
        self.w_v_up = self.rt.upload(tensors[s.v_up_weight]).view(s.num_heads, s.v_head_dim, s.latent_dim).contiguous()
        w_o = self.rt.upload(tensors[s.o_weight])
        if self.ctx_width != self.ctx_dim:
            w_o = torch.cat([w_o, w_o.new_zeros(s.hidden_size, self.ctx_width - self.ctx_dim)], dim=1)
        self.w_o = w_o.contiguous()

    def forward(self, step, h, x, cache_entry, writes_cache=True):
        s, rt = self.spec, self.rt
        ops = rt.kernels()
        n = h.shape[0]
        fused = rt.workspace.get("qkv", (n, self.fused_width), torch.float32)
        ops.linear(h, self.w_q_down, fused, _ops.MODE_STORE_F32)
        latents = step.cache.entry_storage(cache_entry)["c"]
        table = step.block_tables[step.cache.entry_group_index(cache_entry)]
        block_size = step.cache.block_size
        q = rt.workspace.get("q", (n, self.q_dim), rt.dtype)
        # queries pass as they are; the one "key head" of a row is the latent, normed with its weight and cached
        ops.qkv_finish(fused, q, latents, None, step.positions, step.token_seq, table, s.num_heads, 1, s.head_dim, 0,
                       block_size, write_kv=writes_cache, k_norm=True, qk_norm_eps=s.eps,
                       k_norm_weight=self.latent_gamma, key_dim=s.latent_dim)
        q_latent = rt.workspace.get("q_latent", (n, s.num_heads * s.latent_dim), rt.dtype)
        ops.headwise_linear(q, self.w_k_up_t, q_latent, s.num_heads)
        mixed = rt.workspace.get("latent_ctx", (n, s.num_heads * s.latent_dim), rt.dtype)
        ops.attention_general(q_latent, latents, latents, table, step.positions, step.token_seq, mixed, s.num_heads, 1,
                              s.latent_dim, s.latent_dim, block_size, s.scale)
        ctx = rt.workspace.get("attn_ctx", (n, self.ctx_width), rt.dtype)
        ops.headwise_linear(mixed, self.w_v_up, ctx, s.num_heads, zero_pad=self.ctx_width != self.ctx_dim)
        ops.linear(ctx, self.w_o, x, _residual_mode(step), stats=_residual_stats(step))


register_mixer("latent_attention", LatentAttention)
