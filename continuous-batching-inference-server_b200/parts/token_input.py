"""A token's own input of a layer: a row of a second token table, gated by the residual stream."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import Delta, FeedForward, register_feed_forward
from .rmsnorm import RMSNorm


class TokenGatedInput(FeedForward):
    """y = proj(act(gate x) * e) with x the residual stream as it is (the block hands it over unnormalised) and e the
    layer's own ``dim`` columns of the token's row of a second table ``[vocab, table_width]``, from column ``col0``.
    What is added is unit_rms(y) * weight: the part names a root-mean-square norm of its own (plain weight, ``eps``
    inside the root) that the norm adding the result applies in its pass (``Delta.post``).

    ``table``: the table's full tensor name (shared by all layers, no layer prefix); ``names``: what follows the
    layer's prefix in the names of the gate ``[dim, width]``, the projection ``[width, dim]`` and the norm's weight.
    A layer keeps its own columns of the table only, so all layers together hold the table once."""

    def __init__(self, width: int, dim: int, vocab_size: int, table_width: int, col0: int, eps: float,
                 activation: str = "gelu_tanh", table: str = "side.embed", names=("side.gate", "side.proj", "side.norm")):
        if activation not in ops.ACT or not activation:
            raise ValueError(f"activation {activation!r} is not one of {sorted(k for k in ops.ACT if k)}")
        self.width, self.dim, self.vocab_size = int(width), int(dim), int(vocab_size)
        self.table_width, self.col0 = int(table_width), int(col0)
        if not 0 <= self.col0 <= self.table_width - self.dim:
            raise ValueError(f"columns {self.col0}..{self.col0 + self.dim} lie outside a table of width {self.table_width}")
        self.activation, self.table_name = activation, table
        self.gate_name, self.proj_name, self.norm_name = names
        self.norm = RMSNorm(self.width, eps, 0.0, self.norm_name)
        self.w_gate = self.w_proj = self.rows = None

    def tensors(self, prefix):
        return [TensorDecl(self.table_name, (self.vocab_size, self.table_width), "table"),
                TensorDecl(prefix + self.gate_name, (self.dim, self.width)),
                TensorDecl(prefix + self.proj_name, (self.width, self.dim))] + self.norm.tensors(prefix)

    def load(self, prefix, tensors, dtype, device):
        self.w_gate = self._matrix(tensors[prefix + self.gate_name], dtype, device)
        self.w_proj = self._matrix(tensors[prefix + self.proj_name], dtype, device)
        self.rows = self._matrix(tensors[self.table_name][:, self.col0:self.col0 + self.dim], dtype, device)
        self.norm.load(prefix, tensors, dtype, device)

    def streamed_weights(self):
        return [self.w_gate, self.w_proj]

    def forward(self, ctx, h):
        T = h.shape[0]
        g = ops.linear(h, self.w_gate, None)
        ops.gate_mul(g, self.rows, self.activation, g, b_rows=ctx.tokens[:T])
        return Delta(ops.linear(g, self.w_proj, None, None, out_dtype=torch.float32), None, self.norm)


register_feed_forward("token_gated", TokenGatedInput)
