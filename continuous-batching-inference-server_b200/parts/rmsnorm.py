"""Root-mean-square norm with the residual add folded in."""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import Delta, Norm, register_norm, settle_delta


class RMSNorm(Norm):
    """y = x / sqrt(mean(x^2) + eps) * (offset + weight) over the last dim, eps inside the root, in 32-bit.
    ``offset`` 1 is for weights stored around zero, 0 for weights stored as they are applied.  ``name``: what
    follows the norm's prefix in its weight's tensor name.

    The norm that adds a delta to the residual stream also applies the delta's own norm (``Delta.post``, if that is an
    ``RMSNorm`` too) in the same pass over the row: in a block with norms before and after every part, each part costs
    one norm kernel, not two and an add."""

    def __init__(self, width: int, eps: float, offset: float = 0.0, name: str = "weight"):
        self.width, self.eps, self.offset, self.name = int(width), float(eps), float(offset), name
        if not 0 < self.width <= ops.RMS_RESIDUAL_MAX_WIDTH:
            raise ValueError(f"RMSNorm: width {self.width} is outside 1..{ops.RMS_RESIDUAL_MAX_WIDTH}, the widest row "
                             f"the kernel takes")
        self.weight = None

    def tensors(self, prefix):
        return [TensorDecl(prefix + self.name, (self.width,), "norm_zero" if self.offset else "norm_weight")]

    def load(self, prefix, tensors, dtype, device):
        self.weight = self._vector(tensors[prefix + self.name], device)

    takes_scale = True

    def as_rmsnorm(self):
        return (self.weight, self.eps, self.offset) if self.weight is not None else None

    def takes_post(self, post):
        return isinstance(post, RMSNorm) and post.width == self.width and post.weight is not None

    def forward(self, ctx, x, delta: Optional[Delta], rows=None, out_dtype=None):
        n = rows.shape[0] if rows is not None else x.shape[0]
        delta = settle_delta(ctx, self, delta)
        out = torch.empty((n, self.width), dtype=out_dtype or ctx.dtype, device=x.device)
        post = None
        if delta is not None and delta.post is not None:
            post = (delta.post.weight, delta.post.eps, delta.post.offset)
        ops.add_rmsnorm(x, delta.value if delta else None, delta.bias if delta else None, post, self.weight, self.eps,
                        self.offset, out, rows, delta_scale=delta.scale if delta else 1.0)
        return out

    def apply(self, ctx, value, bias=None):
        out = torch.zeros(value.shape, dtype=torch.float32, device=value.device)
        ops.add_rmsnorm(out, value, bias, (self.weight, self.eps, self.offset), None, 0.0, 0.0, None)
        return out


register_norm("rmsnorm", RMSNorm)
