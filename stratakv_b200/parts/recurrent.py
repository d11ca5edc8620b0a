"""A recurrent block around a real-gated linear recurrent unit (the block of the Griffin models).

For the mixer's input h and ``C`` channels::

    y = gelu_tanh(Wy h + by)                                       the gate branch
    u = conv(Wx h + bx)                                            causal, per channel, `taps` wide, no activation
    r = sigmoid(Ra u + ba),  i = sigmoid(Ri u + bi)                Ra, Ri block-diagonal
    a = exp(-8 r softplus(lam)),  S <- a S + sqrt(1 - a^2) i u     S = 0 before the first token
    x += Wo (S * y)

Kernels: one projection for both branches (float32 out), the convolution, the gates' block-diagonal products
(``headwise_linear`` on float32 inputs), the gates themselves, the scan, the output projection.  Everything between
the two projections is float32.  Per sequence the cache's state area keeps S and the convolution's last inputs
(``csrc/recurrent.cu`` says how a step that runs twice stays correct); nothing is kept per position.
"""
from __future__ import annotations

import torch

from .. import ops as _ops
from .attention import _residual_mode, _residual_stats
from .base import CacheRequest, Mixer, TensorRequest
from .registry import register_mixer


class RgLru(Mixer):
    graph_safe = True
    stores_branch = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if spec.parts <= 0 or spec.channels % spec.parts != 0:
            raise ValueError(f"rglru: {spec.channels} channels do not split into {spec.parts} equal parts")
        if spec.taps <= 0:
            raise ValueError("rglru: the convolution needs at least one tap")
        if runtime.dtype == torch.bfloat16 and spec.hidden_size % 8 != 0:
            raise ValueError(f"rglru: hidden size {spec.hidden_size} is not supported in bfloat16 "
                             "(rows of 16 bytes are needed: a multiple of 8); float32 takes any size")
        self.part = spec.channels // spec.parts
        self.padded = -(-spec.channels // 8) * 8             # rows of whole 16 bytes for both projections
        self.state_floats = (2 + spec.taps) * spec.channels

    @classmethod
    def expected_tensors(cls, spec):
        c, part = spec.channels, spec.channels // spec.parts
        return {spec.y_weight: TensorRequest((c, spec.hidden_size)), spec.y_bias: TensorRequest((c,)),
                spec.x_weight: TensorRequest((c, spec.hidden_size)), spec.x_bias: TensorRequest((c,)),
                spec.conv_weight: TensorRequest((c, spec.taps)), spec.conv_bias: TensorRequest((c,)),
                spec.r_weight: TensorRequest((spec.parts, part, part)), spec.r_bias: TensorRequest((spec.parts, part)),
                spec.i_weight: TensorRequest((spec.parts, part, part)), spec.i_bias: TensorRequest((spec.parts, part)),
                spec.decay: TensorRequest((c,)), spec.o_weight: TensorRequest((spec.hidden_size, c))}

    @classmethod
    def cache_request(cls, spec):
        return CacheRequest(kind="none", state_bytes=4 * (2 + spec.taps) * spec.channels)

    def bind(self, tensors):
        s, rt = self.spec, self.rt
        pad = self.padded - s.channels
        branches = []
        for name in (s.y_weight, s.x_weight):
            w = rt.upload(tensors[name])
            if pad:
                w = torch.cat([w, w.new_zeros(pad, s.hidden_size)], dim=0)
            branches.append(w)
        self.w_yx = torch.cat(branches, dim=0).contiguous()
        del branches
        as_float = lambda name: rt.upload(tensors[name], torch.float32).reshape(-1).contiguous()
        self.y_bias, self.x_bias = as_float(s.y_bias), as_float(s.x_bias)
        self.conv_w = rt.upload(tensors[s.conv_weight], torch.float32).contiguous()
        self.conv_b = as_float(s.conv_bias)
        lam = as_float(s.decay)
        self.decay_rate = rt.kernels().rglru_rate(lam, torch.empty_like(lam))     # 8 * softplus(lam), once
        self.r_bias, self.i_bias = as_float(s.r_bias), as_float(s.i_bias)
        # per part the r rows, then the i rows: one block-diagonal product makes both gates' inputs
        self.w_gates = torch.cat([rt.upload(tensors[s.r_weight]), rt.upload(tensors[s.i_weight])], dim=1).contiguous()
        w_o = rt.upload(tensors[s.o_weight])
        if pad:
            w_o = torch.cat([w_o, w_o.new_zeros(s.hidden_size, pad)], dim=1)
        self.w_o = w_o.contiguous()

    def forward(self, step, h, x, cache_entry, writes_cache=True):
        s, rt = self.spec, self.rt
        ops = rt.kernels()
        n, c = h.shape[0], s.channels
        yx = rt.workspace.get("rglru_yx", (n, 2 * self.padded), torch.float32)
        ops.linear(h, self.w_yx, yx, _ops.MODE_STORE_F32)
        state = step.cache.state(cache_entry).view(torch.float32)
        meta = (step.positions, step.token_seq, step.cu_q, step.slot_ids)
        u = rt.workspace.get("rglru_u", (n, c), torch.float32)
        ops.rglru_conv(yx, self.padded, self.x_bias, self.conv_w, self.conv_b, u, meta, state)
        gates = rt.workspace.get("rglru_gates", (n, 2 * c), torch.float32)
        ops.headwise_linear(u, self.w_gates, gates, s.parts)
        ops.rglru_gates(gates, u, yx, self.y_bias, self.r_bias, self.i_bias, self.decay_rate, self.part)
        mixed = rt.workspace.get("rglru_out", (n, self.padded), rt.dtype, zero=self.padded != c)
        need = ops.rglru_scan_scratch(step.n_seqs, step.max_q_len, c)
        summary = rt.workspace.get("rglru_chunks", (need,), torch.float32) if need else None
        ops.rglru_scan(gates, yx, self.padded, self.x_bias, mixed, self.part, s.taps, meta, state, step.max_q_len, summary)
        ops.linear(mixed, self.w_o, x, _residual_mode(step), stats=_residual_stats(step))


register_mixer("rglru", RgLru)
