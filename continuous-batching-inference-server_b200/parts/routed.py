"""A routed mixture of gated feed-forwards."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import Delta, FeedForward, register_feed_forward
from .dense import GatedFeedForward


class RoutedFeedForward(FeedForward):
    """``experts`` gated feed-forwards (down(act(gate v) * (up v)), no biases) of which every row uses ``top``.

    The router's logits ``router h`` are taken in 32-bit; ``score`` ("sigmoid", or "softmax" over all experts) turns
    them into scores; the ``top`` largest are chosen; their weights are the scores as they are, or divided by their
    sum with ``renormalize``.  ``weight_on`` says what a weight multiplies: "input" (the result is the sum of
    expert(w h)) or "output" (the sum of w expert(h)).  ``renorm_eps`` joins the sum the weights are divided by;
    ``weight_scale`` multiplies every weight afterwards.  ``shared_inner`` > 0: one more gated feed-forward of that
    inner width (``<names[2]>.gate|up|down``) that every row uses, unweighted, added to the experts' sum.  Tensors: ``<names[0]>`` the router ``[experts, width]``,
    ``<names[1]><i>.gate|up|down`` expert i's matrices, stored ``[out, in]``; they are kept stacked,
    ``[experts, 2 inner, width]`` and ``[experts, width, inner]``, so a kernel finds an expert by its index."""

    def __init__(self, width: int, inner: int, experts: int, top: int, activation: str = "silu", score: str = "sigmoid",
                 renormalize: bool = False, weight_on: str = "input", names=("mlp.router", "mlp.e", "mlp.shared"),
                 renorm_eps: float = 0.0, weight_scale: float = 1.0, shared_inner: int = 0):
        if activation not in ops.ACT or not activation:
            raise ValueError(f"activation {activation!r} is not one of {sorted(k for k in ops.ACT if k)}")
        if score not in ops.ROUTE_SCORE:
            raise ValueError(f"score {score!r} is not one of {sorted(ops.ROUTE_SCORE)}")
        if weight_on not in ("input", "output"):
            raise ValueError(f"weight_on {weight_on!r} is not 'input' or 'output'")
        if not 0 < int(top) <= int(experts):
            raise ValueError(f"top={top} must lie in 1..experts={experts}")
        self.width, self.inner, self.experts, self.top = int(width), int(inner), int(experts), int(top)
        self.activation, self.score, self.renormalize = activation, score, bool(renormalize)
        self.weight_on_input = weight_on == "input"
        self.router_name, self.expert_prefix = names[0], names[1]
        self.renorm_eps, self.weight_scale = float(renorm_eps), float(weight_scale)
        self.shared = None
        if int(shared_inner) > 0:
            stem = names[2] if len(names) > 2 else "mlp.shared"
            self.shared = GatedFeedForward(self.width, int(shared_inner), activation,
                                           names=(stem + ".gate", stem + ".up", stem + ".down"))
        self.w_router = self.w_gate_up = self.w_down = None

    def tensors(self, prefix):
        out = [TensorDecl(prefix + self.router_name, (self.experts, self.width))]
        for e in range(self.experts):
            p = f"{prefix}{self.expert_prefix}{e}."
            out += [TensorDecl(p + "gate", (self.inner, self.width)), TensorDecl(p + "up", (self.inner, self.width)),
                    TensorDecl(p + "down", (self.width, self.inner))]
        return out + (self.shared.tensors(prefix) if self.shared is not None else [])

    def load(self, prefix, tensors, dtype, device):
        self.w_router = self._matrix(tensors[prefix + self.router_name], dtype, device)
        gu, down = [], []
        for e in range(self.experts):
            p = f"{prefix}{self.expert_prefix}{e}."
            gu.append(torch.cat([self._matrix(tensors[p + "gate"], dtype, device),
                                 self._matrix(tensors[p + "up"], dtype, device)]))
            down.append(self._matrix(tensors[p + "down"], dtype, device))
        self.w_gate_up = torch.stack(gu).contiguous()
        self.w_down = torch.stack(down).contiguous()
        if self.shared is not None:
            self.shared.load(prefix, tensors, dtype, device)

    def streamed_weights(self):
        return self.shared.streamed_weights() if self.shared is not None else []

    def forward(self, ctx, h):
        T = h.shape[0]
        ids = torch.empty((T, self.top), dtype=torch.int32, device=h.device)
        weights = torch.empty((T, self.top), dtype=torch.float32, device=h.device)
        ops.route_topk(h, self.w_router, self.top, self.score, self.renormalize, ids, weights, self.renorm_eps,
                       self.weight_scale)
        # the result goes straight into the 32-bit residual rows where a block offers them
        into = ctx.residual if ctx.residual is not None and ctx.residual.shape == (T, self.width) else None
        out = into if into is not None else torch.empty((T, self.width), dtype=torch.float32, device=h.device)
        if ops.routed_tiles_takes(h, self.w_gate_up, self.w_down):
            # many rows: sorted by expert, tiles on the tensor cores
            ops.routed_tiles(h, self.w_gate_up, self.w_down, ids, weights, self.activation, self.weight_on_input, out,
                             accumulate=into is not None)
        else:
            # a few rows (decoding), and the 32-bit path: every (row, choice) streams its expert's matrices
            hidden = torch.empty((T * self.top, self.inner), dtype=h.dtype, device=h.device)
            ops.routed_gate_up(h, self.w_gate_up, ids, weights, self.activation, self.weight_on_input, hidden)
            ops.routed_down(hidden, self.w_down, ids, weights, self.weight_on_input, out, accumulate=into is not None)
        if self.shared is not None:
            self.shared.forward_into(h, out)        # the expert every row uses adds to the same 32-bit rows
        return None if into is not None else Delta(out)


register_feed_forward("routed", RoutedFeedForward)
