"""Dense feed-forward."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import Delta, FeedForward, register_feed_forward


class DenseFeedForward(FeedForward):
    """act(h @ W1 + b1) @ W2 + b2 with the activation taken on the 32-bit sum
    (reference: python/model.py:50, src/transformer.cpp:86-88).  Weights come in GPT-2's
    Conv1D layout [in, out] and are kept transposed, [out, in].

    ``plain`` True is the other storage: the two matrices as ``[out, in]`` under the very names ``names`` gives
    (no ``.weight``), and no biases."""

    def __init__(self, width: int, inner: int, activation: str,
                 names=("mlp.c_fc", "mlp.c_proj"), plain: bool = False):
        if activation not in ops.ACT:
            raise ValueError(f"activation {activation!r} is not one of {sorted(k for k in ops.ACT if k)}")
        self.width, self.inner, self.activation = int(width), int(inner), activation
        self.fc, self.proj = names
        self.plain = bool(plain)
        self.w1 = self.b1 = self.w2 = self.b2 = None

    def tensors(self, prefix):
        if self.plain:
            return [TensorDecl(prefix + self.fc, (self.inner, self.width)), TensorDecl(prefix + self.proj, (self.width, self.inner))]
        return [TensorDecl(f"{prefix}{self.fc}.weight", (self.width, self.inner)),
                TensorDecl(f"{prefix}{self.fc}.bias", (self.inner,), "vector"),
                TensorDecl(f"{prefix}{self.proj}.weight", (self.inner, self.width)),
                TensorDecl(f"{prefix}{self.proj}.bias", (self.width,), "vector")]

    def load(self, prefix, tensors, dtype, device):
        if self.plain:
            self.w1 = self._matrix(tensors[prefix + self.fc], dtype, device)
            self.w2 = self._matrix(tensors[prefix + self.proj], dtype, device)
            return
        self.w1 = self._matrix_nk(tensors[f"{prefix}{self.fc}.weight"], dtype, device)
        self.b1 = self._vector(tensors[f"{prefix}{self.fc}.bias"], device)
        self.w2 = self._matrix_nk(tensors[f"{prefix}{self.proj}.weight"], dtype, device)
        self.b2 = self._vector(tensors[f"{prefix}{self.proj}.bias"], device)

    def streamed_weights(self):
        return [self.w1, self.w2]

    def fuses_norm(self, ctx, norm):
        return not self.plain and ops.ln_linear_takes(ctx, norm, self.w1) and self.inner % 8 == 0

    def forward_residual(self, ctx, x, norm):
        a = torch.empty((ctx.n_rows, self.inner), dtype=ctx.dtype, device=x.device)
        ops.ln_linear(x, *norm.as_layernorm(), self.w1, self.b1, self.activation, a)
        ops.gemm_small_m(a, self.w2, self.b2, None, x, accumulate=True)

    def forward(self, ctx, h):
        a = ops.linear(h, self.w1, self.b1, self.activation)
        if self.b2 is None:
            if ops.linear_residual(a, self.w2, ctx.residual):
                return None
        elif ops.linear_add_takes(a, self.w2, ctx.residual):       # the product adds into the residual stream itself
            ops.linear_add(a, self.w2, self.b2, ctx.residual)
            return None
        return Delta(ops.linear(a, self.w2, None, None, out_dtype=torch.float32), self.b2)


register_feed_forward("dense", DenseFeedForward)


class GatedFeedForward(FeedForward):
    """down(act(gate h) * (up h)): three matrices stored ``[out, in]``, no biases; the gate's and the up
    projection's rows form one matrix, so one product gives both, and the activation and the product of the two
    halves are taken in 32-bit and rounded once.  With ``biases`` each of the three has a bias (its matrix's name with
    ``.b``), added to the 32-bit sums.  ``names``: what follows the layer's prefix in the names of the gate, up and
    down matrices."""

    def __init__(self, width: int, inner: int, activation: str = "silu", names=("mlp.gate", "mlp.up", "mlp.down"),
                 biases: bool = False):
        if activation not in ops.ACT or not activation:
            raise ValueError(f"activation {activation!r} is not one of {sorted(k for k in ops.ACT if k)}")
        self.width, self.inner, self.activation = int(width), int(inner), activation
        self.gate_name, self.up_name, self.down_name = names
        self.biases = bool(biases)
        self.w_gate_up = self.w_down = self.b_gate_up = self.b_down = None

    def tensors(self, prefix):
        out = [TensorDecl(prefix + self.gate_name, (self.inner, self.width)),
               TensorDecl(prefix + self.up_name, (self.inner, self.width)),
               TensorDecl(prefix + self.down_name, (self.width, self.inner))]
        if self.biases:
            out += [TensorDecl(prefix + self.gate_name + ".b", (self.inner,), "vector"),
                    TensorDecl(prefix + self.up_name + ".b", (self.inner,), "vector"),
                    TensorDecl(prefix + self.down_name + ".b", (self.width,), "vector")]
        return out

    def load(self, prefix, tensors, dtype, device):
        self.w_gate_up = torch.cat([self._matrix(tensors[prefix + self.gate_name], dtype, device),
                                    self._matrix(tensors[prefix + self.up_name], dtype, device)]).contiguous()
        self.w_down = self._matrix(tensors[prefix + self.down_name], dtype, device)
        if self.biases:
            self.b_gate_up = torch.cat([self._vector(tensors[prefix + self.gate_name + ".b"], device),
                                        self._vector(tensors[prefix + self.up_name + ".b"], device)]).contiguous()
            self.b_down = self._vector(tensors[prefix + self.down_name + ".b"], device)

    def streamed_weights(self):
        return [self.w_gate_up, self.w_down]

    def forward(self, ctx, h):
        F = self.inner
        gu = ops.linear(h, self.w_gate_up, self.b_gate_up)
        a = torch.empty((h.shape[0], F), dtype=h.dtype, device=h.device)
        ops.gate_mul(gu[:, :F], gu[:, F:], self.activation, a)
        if self.b_down is None:
            if ops.linear_residual(a, self.w_down, ctx.residual):   # the product adds into the residual stream itself
                return None
        elif ops.linear_add_takes(a, self.w_down, ctx.residual):
            ops.linear_add(a, self.w_down, self.b_down, ctx.residual)
            return None
        return Delta(ops.linear(a, self.w_down, None, None, out_dtype=torch.float32), self.b_down)


    def forward_into(self, h, out) -> None:
        """out += this feed-forward of h; ``out``: 32-bit rows (another part's result that this one joins)."""
        F = self.inner
        gu = ops.linear(h, self.w_gate_up, self.b_gate_up)
        a = torch.empty((h.shape[0], F), dtype=h.dtype, device=h.device)
        ops.gate_mul(gu[:, :F], gu[:, F:], self.activation, a)
        if self.b_down is None and ops.linear_residual(a, self.w_down, out):
            return
        ops.add_delta(out, ops.linear(a, self.w_down, None, None, out_dtype=torch.float32), self.b_down)


class NoFeedForward(FeedForward):
    """A layer without a feed-forward: nothing is added."""

    def __init__(self, width: int):
        self.width = int(width)

    def forward(self, ctx, h):
        return None


register_feed_forward("gated", GatedFeedForward)
register_feed_forward("nothing", NoFeedForward)
