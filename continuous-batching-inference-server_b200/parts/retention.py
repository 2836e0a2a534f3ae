"""Retention: linear attention with a fixed decay per head."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import Delta, Mixer, StateNeed, register_mixer
from .rotation import rotary_frequencies


class RetentionMixer(Mixer):
    """Per head: q and k (``dim`` wide) and v (``v_dim``) from the mixer's input, no biases.  The first ``rot_dims``
    entries of every head's q and k are rotated by the token's position (pairs i, i + rot_dims/2, angle
    p * rot_base^(-2i/rot_dims), optionally stretched, see ``rotary_frequencies``); k is then multiplied by
    ``k_scale`` (default dim^-1/2).  In 32-bit, with the head's fixed decay:

        S <- decay_h S + k v^T;   o = S^T q                  (no softmax, no denominator)

    Each head's o is divided by its root mean square (eps inside the root, no weight); the heads side by side are
    multiplied by ``gate_act`` of a gate as wide as they are (from the mixer's input) and projected out.

    Per request the mixer keeps S (zero at the start), 32-bit; a step walks each segment's rows in order from that
    state, so prompt portions cut anywhere, single decoded tokens and whole prompts give the same values.  Nothing is
    cached per token.  Long segments of a step with little parallel work are cut into pieces that run side by side
    (``ops.retention``; the results differ from the walk in one piece by rounding only).  q | k | v | gate are one product; rotation and scale happen inside the recurrence kernel, on
    32-bit values.  ``names``: what follows the layer's prefix in the tensors' names (q, k, v, the gate, the output
    matrix)."""

    def __init__(self, width: int, heads: int, dim: int, v_dim: int, decays, eps: float, rot_base: float = 10000.0,
                 rot_dims: int = 0, rot_stretch=None, k_scale: float = None, gate_act: str = "silu",
                 names=("mix.q", "mix.k", "mix.v", "mix.g", "mix.o")):
        self.width, self.heads, self.dim, self.v_dim = int(width), int(heads), int(dim), int(v_dim)
        if not 0 < self.dim <= ops.RETENTION_MAX_DIM:
            raise ValueError(f"dim={dim} is outside 1..{ops.RETENTION_MAX_DIM}, what the recurrence kernel takes")
        self.decays = tuple(float(d) for d in decays)
        if len(self.decays) != self.heads or not all(0.0 <= d <= 1.0 for d in self.decays):
            raise ValueError(f"decays: {self.heads} numbers between 0 and 1 are needed, one per head, got {list(decays)!r}")
        self.rot_base, self.rot_dims = float(rot_base), int(rot_dims)
        if self.rot_dims % 2 or not 0 <= self.rot_dims <= self.dim:
            raise ValueError(f"rot_dims={self.rot_dims} must be even and at most dim={self.dim}")
        self.rot_stretch = None if rot_stretch is None else tuple(float(v) for v in rot_stretch)
        if gate_act not in ops.ACT or not gate_act:
            raise ValueError(f"gate_act {gate_act!r} is not one of {sorted(k for k in ops.ACT if k)}")
        self.eps, self.gate_act = float(eps), gate_act
        self.k_scale = float(k_scale) if k_scale is not None else self.dim ** -0.5
        self.d_qk, self.d_v = self.heads * self.dim, self.heads * self.v_dim
        self.names = tuple(names)
        self.w_in = self.w_out = self.freqs = self.one_minus_decay = self.piece_decays = None

    def state_need(self):
        return StateNeed((self.heads * self.v_dim * self.dim,), torch.float32)

    def tensors(self, prefix):
        n = [prefix + s for s in self.names]
        W = self.width
        return [TensorDecl(n[0], (self.d_qk, W)), TensorDecl(n[1], (self.d_qk, W)), TensorDecl(n[2], (self.d_v, W)),
                TensorDecl(n[3], (self.d_v, W)), TensorDecl(n[4], (W, self.d_v))]

    def load(self, prefix, tensors, dtype, device):
        n = [prefix + s for s in self.names]
        self.w_in = torch.cat([self._matrix(tensors[k], dtype, device) for k in n[:4]]).contiguous()    # q | k | v | gate
        self.w_out = self._matrix(tensors[n[4]], dtype, device)
        self.freqs = rotary_frequencies(self.rot_base, self.rot_dims, self.rot_stretch).to(device)
        # 1 - decay in 64-bit, rounded once: a decay near 1 keeps its digits
        self.one_minus_decay = torch.tensor([1.0 - d for d in self.decays], dtype=torch.float64).to(torch.float32).to(device)
        self.piece_decays = ops.retention_piece_decays(self.decays).to(device)

    def streamed_weights(self):
        return [self.w_in, self.w_out]

    def forward(self, ctx, h, cache, state):
        T = h.shape[0]
        proj = ops.linear(h, self.w_in, None)                                            # q | k | v | gate
        y = torch.empty((T, self.d_v), dtype=torch.float32, device=h.device)
        ops.retention(proj, 0, self.d_qk, 2 * self.d_qk, ctx.positions, self.freqs, self.rot_dims, self.k_scale,
                      self.one_minus_decay, state, ctx.seg_slot, ctx.cu_rows, ctx.n_segments, self.heads, self.dim,
                      self.v_dim, y, max_seg_rows=ctx.max_seg_rows, piece_decays=self.piece_decays)
        g = torch.empty((T, self.d_v), dtype=h.dtype, device=h.device)
        g0 = 2 * self.d_qk + self.d_v
        ops.rms_norm(y, None, self.eps, g, parts=self.heads, gate=proj[:, g0:g0 + self.d_v], gate_act=self.gate_act,
                     gate_after=True)
        if ops.linear_residual(g, self.w_out, ctx.residual):
            return None
        return Delta(ops.linear(g, self.w_out, None, None, out_dtype=torch.float32))


register_mixer("retention", RetentionMixer)
