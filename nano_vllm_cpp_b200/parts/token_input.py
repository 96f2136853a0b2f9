"""Per-layer token input: a branch made from the residual stream's rows and a table row of the row's own token."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import TokenInput, TensorSpec
from .linear import linear
from .registry import register_part


class GatedTokenInput(TokenInput):
    """``e = table[token, index * dim : (index + 1) * dim]``; ``g = gelu_tanh(W_gate h) * e``; the branch is
    ``W_proj g``.  ``table`` ([vocab, layers * dim]) is one tensor of the whole model (``table_name``, an absolute
    name); ``gate`` and ``proj`` are this layer's."""

    def __init__(self, hidden_size: int, vocab_size: int, dim: int, index: int, count: int, table_name: str):
        self.hidden, self.vocab, self.dim, self.index, self.count = hidden_size, vocab_size, dim, index, count
        self.table_name = "/" + table_name.lstrip("/")

    def tensor_specs(self, available=None):
        return {self.table_name: TensorSpec((self.vocab, self.count * self.dim)),
                "gate": TensorSpec((self.dim, self.hidden)), "proj": TensorSpec((self.hidden, self.dim))}

    def load(self, fetch, ctx):
        self.ctx = ctx
        self.table = fetch(self.table_name)
        self.w_gate, self.w_proj = fetch("gate"), fetch("proj")

    def forward(self, h, batch):
        ctx = self.ctx
        gate = linear(ctx, h, self.w_gate, torch.float32)
        g = torch.empty((h.shape[0], self.dim), dtype=ctx.act_dtype, device=h.device)
        ops.token_gate(gate, batch.input_ids, self.table, self.index * self.dim, g, ctx.err, feed=ctx.feed)
        return linear(ctx, g, self.w_proj, torch.float32)


register_part("token_input", "gated_table", GatedTokenInput)
