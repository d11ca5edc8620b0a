"""A per-layer input that depends on the token, added to the stream at the end of a layer.

One table ``[vocab, layers * dim]`` serves all layers; layer i reads the columns ``[i * dim, (i + 1) * dim)`` of the
token's row: ``e``.  Then ``g = gelu_tanh(gate x) * e``, ``y = proj g`` and ``x += rmsnorm(y) * norm`` (a plain-weight
RMS norm).  ``dim`` is small, so the whole thing is one kernel with a block per token (``csrc/stream_ops.cu``), which
can also leave the next layer's first norm of the new stream.
"""
from __future__ import annotations

import torch

from .base import Part, TensorRequest
from .registry import register_token_input


class TokenSide(Part):
    role = "token_input"
    graph_safe = True

    @classmethod
    def expected_tensors(cls, spec):
        return {spec.table: TensorRequest((spec.vocab_size, spec.table_width)),
                spec.gate_weight: TensorRequest((spec.dim, spec.hidden_size)),
                spec.proj_weight: TensorRequest((spec.hidden_size, spec.dim)),
                spec.norm_weight: TensorRequest((spec.hidden_size,), "around_one")}

    def bind(self, tensors):
        s = self.spec
        self.table = self.rt.upload_shared(s.table, tensors[s.table])
        self.w_gate = self.rt.upload(tensors[s.gate_weight]).contiguous()
        self.w_proj_t = self.rt.upload(tensors[s.proj_weight]).t().contiguous()     # [dim, hidden]
        self.gamma = self.rt.upload(tensors[s.norm_weight], torch.float32)

    # The kernel can first add a sublayer's branch through the norm after it (``forward``'s ``branch``, ``post_norm``),
    # but measured slower than ``rmsnorm_add`` followed by this kernel (16,320 tokens of width 2,048: 931 us against
    # 115 + 490 us; a decode step of 8 sequences 0.80 against 0.78 ms), so the arrangement is told not to ask for it.
    adds_branch = False

    def forward(self, step, x, next_norm=None, next_out=None, branch=None, post_norm=None) -> None:
        """Adds the input into ``x``; with ``next_norm`` (an RMS norm part) and ``next_out`` also writes that norm of
        the new stream.  ``branch`` (float32) and ``post_norm`` (an RMS norm part): the sublayer in front has not been
        added yet; ``x += post_norm(branch)`` is done first, in the same kernel."""
        s = self.spec
        self.rt.kernels().token_side(
            x, step.token_ids, self.table, s.offset, s.dim, self.w_gate, self.w_proj_t, self.gamma, s.eps,
            next_gamma=next_norm.gamma if next_norm is not None else None,
            next_eps=next_norm.spec.eps if next_norm is not None else 0.0, next_out=next_out,
            branch=branch, post_gamma=post_norm.gamma if branch is not None else None,
            post_eps=post_norm.spec.eps if branch is not None else 0.0)


register_token_input("token_side", TokenSide)
