"""LayerNorm with the residual add folded in."""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import Delta, Norm, register_norm, settle_delta


class LayerNorm(Norm):
    """y = (x - mean) * rsqrt(var + eps) * weight + bias over the last dim, biased variance,
    statistics in 32-bit (reference: kernels/elementwise.cu:21-57; eps is a literal there, :51)."""

    def __init__(self, width: int, eps: float, names=("weight", "bias")):
        """``names``: what follows the norm's prefix in the names of its weight and its bias."""
        self.width, self.eps = int(width), float(eps)
        self.weight_name, self.bias_name = names
        if not 0 < self.width <= ops.NORM_MAX_WIDTH:
            raise ValueError(f"LayerNorm: width {self.width} is outside 1..{ops.NORM_MAX_WIDTH}, the widest row the kernel takes")
        self.weight = self.bias = None

    def tensors(self, prefix):
        return [TensorDecl(prefix + self.weight_name, (self.width,), "norm_weight"),
                TensorDecl(prefix + self.bias_name, (self.width,), "norm_bias")]

    def load(self, prefix, tensors, dtype, device):
        self.weight = self._vector(tensors[prefix + self.weight_name], device)
        self.bias = self._vector(tensors[prefix + self.bias_name], device)

    def as_layernorm(self):
        return (self.weight, self.bias, self.eps) if self.weight is not None and self.bias is not None else None

    def forward(self, ctx, x, delta: Optional[Delta], rows=None, out_dtype=None):
        n = rows.shape[0] if rows is not None else x.shape[0]
        delta = settle_delta(ctx, self, delta)
        out = torch.empty((n, self.width), dtype=out_dtype or ctx.dtype, device=x.device)
        ops.add_layernorm(x, delta.value if delta else None, delta.bias if delta else None,
                          self.weight, self.bias, self.eps, out, rows)
        return out


class NoNorm(Norm):
    """No normalisation: adds what is pending to the residual stream and hands the rows on in the
    compute dtype (for a model without a final norm, and for a part that reads the stream as it is).  What is pending
    may name a root-mean-square norm of its own (a layer that normalises a part's RESULT): it is applied in the same
    pass over the row."""

    def __init__(self, width: int):
        self.width = int(width)
        if not 0 < self.width <= ops.NORM_MAX_WIDTH:
            raise ValueError(f"width {self.width} is outside 1..{ops.NORM_MAX_WIDTH}, the widest row the kernel takes")

    def takes_post(self, post):
        return (getattr(post, "width", None) == self.width and self.width <= ops.RMS_RESIDUAL_MAX_WIDTH
                and post.as_rmsnorm() is not None)

    @property
    def takes_scale(self):
        return self.width <= ops.RMS_RESIDUAL_MAX_WIDTH

    def forward(self, ctx, x, delta: Optional[Delta], rows=None, out_dtype=None):
        n = rows.shape[0] if rows is not None else x.shape[0]
        delta = settle_delta(ctx, self, delta)
        out = torch.empty((n, self.width), dtype=out_dtype or ctx.dtype, device=x.device)
        if delta is not None and (delta.post is not None or delta.scale != 1.0):
            # x += post(delta) * scale; the rows go on as they are
            ops.add_rmsnorm(x, delta.value, delta.bias, delta.post.as_rmsnorm() if delta.post is not None else None,
                            None, 0.0, 0.0, out, rows, delta_scale=delta.scale)
            return out
        ops.add_layernorm(x, delta.value if delta else None, delta.bias if delta else None, None, None, 0.0, out, rows)
        return out


register_norm("layernorm", LayerNorm)
register_norm("none", NoNorm)
