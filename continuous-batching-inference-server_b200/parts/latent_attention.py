"""Attention whose keys and values are projections of one cached latent vector per token."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import CacheArray, CacheNeed, Delta, Mixer, register_mixer
from .rotation import blended_frequencies, rotary_frequencies


class LatentAttention(Mixer):
    """The latent c = unit_rms(W_dkv h) * weight (``rank`` wide, eps inside the root) is cached per token; per head
    k = W_uk c (``qk_dim`` wide), v = W_uv c (``v_dim`` wide).  Scores (q . k) * scale over the keys inside ``window``
    (0: all), softmax in 32-bit; the heads' outputs side by side are gated and projected out.  With ``own_latent``
    False the layer has no W_dkv and reads the latents another layer cached (its own W_uk, W_uv, window and the rest).

    Options, each a parameter:

    * ``q_rank`` > 0: queries go through a latent of their own, q = W_uq (unit_rms(W_dq h) * weight); 0: q = W_q h.
    * ``rot_dim`` > 0: every head's query carries ``rot_dim`` more entries after its ``qk_dim``, and W_dkv ``rot_dim``
      more rows after the latent's: ONE more key part per token, shared by all heads and not normalised.  Both are
      rotated by the token's position (pairs i, i + rot_dims/2 of their first ``rot_dims`` entries, angle
      p * rot_base^(-2i/rot_dims), in 32-bit) and their product joins the score.  The rotated key part is cached
      behind the latent, in the same array.  ``rot_pairs`` "neighbours" pairs entry 2i with 2i + 1 instead;
      ``rot_blend`` = (factor, original, fast, slow) slows the slow pairs down and lengthens cosines and sines
      (``parts.rotation.blended_frequencies``); the score's ``scale`` is used as it is given either way.
    * ``sinks``: a learned number per head whose exponential joins the softmax's denominator (no key, no value).
    * ``gate``: "element" (sigmoid of a projection as wide as the heads' outputs), "head" (one number per head) or
      None (the heads' outputs go to the output projection as they are; no gate tensor).

    The scores never need k: q . (W_uk c) = (W_uk^T q) . c, so queries are carried into the latent space (one
    product per head) and the paged attention kernels run with ONE shared key/value head whose keys are the cached
    rows (latent, then rotated part) and whose values are the latents, the rows' first ``rank`` entries; their
    output, still in the latent space, goes through W_uv per head.
    ``names``: what follows the layer's prefix in the tensors' names (q, dkv, the latent's norm weight, uk, uv, the
    output gate, the output projection, and with their options dq, its norm weight, uq, the sinks)."""

    kv_arrays = ("c", "c")      # the pages that stand for keys and for values

    def __init__(self, width: int, n_head: int, qk_dim: int, v_dim: int, rank: int, scale: float, window: int = 0,
                 eps: float = 1e-5, own_latent: bool = True, q_rank: int = 0, rot_dim: int = 0, rot_base: float = 10000.0,
                 rot_dims: int = None, sinks: bool = False, gate: str = "element", rot_pairs: str = "half", rot_blend=None,
                 names=("mix.q", "mix.dkv", "mix.dkv.norm", "mix.uk", "mix.uv", "mix.g", "mix.o", "mix.dq", "mix.dq.norm",
                        "mix.uq", "mix.sink")):
        self.width, self.n_head, self.qk_dim, self.v_dim, self.rank = int(width), int(n_head), int(qk_dim), int(v_dim), int(rank)
        self.q_rank, self.rot_dim = int(q_rank), int(rot_dim)
        self.rot_dims = self.rot_dim if rot_dims is None else int(rot_dims)
        self.rot_base = float(rot_base)
        if self.rot_dims % 2 or not 0 <= self.rot_dims <= self.rot_dim:
            raise ValueError(f"rot_dims={self.rot_dims} must be even and at most rot_dim={self.rot_dim}")
        if gate not in ("element", "head", None):
            raise ValueError(f"gate {gate!r} is not one of ['element', 'head', None]")
        if rot_pairs not in ("half", "neighbours"):
            raise ValueError(f"rot_pairs {rot_pairs!r} is not one of ['half', 'neighbours']")
        self.rot_neighbours = rot_pairs == "neighbours"
        self.rot_blend = None if rot_blend is None else tuple(float(v) for v in rot_blend)
        self.rot_length = 1.0
        self.key_dim = self.rank + self.rot_dim               # a cached row: the latent, then the rotated key part
        if not 0 < self.key_dim <= ops.ATTENTION_MAX_HEAD_DIM:
            raise ValueError(f"rank + rot_dim = {self.key_dim} is outside 1..{ops.ATTENTION_MAX_HEAD_DIM}, the widest key "
                             f"any attention kernel takes")
        self.scale, self.window, self.eps, self.own_kv = float(scale), int(window), float(eps), bool(own_latent)
        self.has_sinks, self.gate = bool(sinks), gate
        # what the attention kernels read off a mixer: one key/value head shared by all query heads
        self.n_kv_head, self.head_dim, self.v_head_dim = 1, self.key_dim, self.rank
        self.d_q, self.d_kv = self.n_head * self.key_dim, self.key_dim
        self.q_head = self.qk_dim + self.rot_dim              # a head's query as projected
        self.d_gate = 0 if gate is None else (self.n_head if gate == "head" else self.n_head * self.v_dim)
        self.names = tuple(names)
        self.w_in = self.w_uq = self.w_uk_t = self.w_uv = self.w_out = self.norm_w = self.q_norm_w = None
        self.sinks = self.freqs = None

    def cache_need(self):
        return CacheNeed((CacheArray("c", 1, self.key_dim),), self.window) if self.own_kv else None

    def tensors(self, prefix):
        n = [prefix + s for s in self.names]
        H, D, V, R, W = self.n_head, self.qk_dim, self.v_dim, self.rank, self.width
        if self.q_rank:
            q = [TensorDecl(n[7], (self.q_rank, W)), TensorDecl(n[8], (self.q_rank,), "norm_weight"),
                 TensorDecl(n[9], (H * self.q_head, self.q_rank))]
        else:
            q = [TensorDecl(n[0], (H * self.q_head, W))]
        own = [TensorDecl(n[1], (self.key_dim, W)), TensorDecl(n[2], (R,), "norm_weight")] if self.own_kv else []
        extra = [TensorDecl(n[10], (H,), "vector")] if self.has_sinks else []
        gate = [TensorDecl(n[5], (self.d_gate, W))] if self.gate is not None else []
        return q + own + [TensorDecl(n[3], (H * D, R)), TensorDecl(n[4], (H * V, R))] + gate + [TensorDecl(n[6], (W, H * V))] + extra

    def load(self, prefix, tensors, dtype, device):
        n = [prefix + s for s in self.names]
        H, D, V, R = self.n_head, self.qk_dim, self.v_dim, self.rank
        rows = ([tensors[n[7] if self.q_rank else n[0]]] + ([tensors[n[5]]] if self.gate is not None else [])
                + ([tensors[n[1]]] if self.own_kv else []))
        self.w_in = torch.cat([self._matrix(t, dtype, device) for t in rows]).contiguous()       # q (or its latent) | gate | latent
        if self.q_rank:
            self.q_norm_w = self._vector(tensors[n[8]], device)
            self.w_uq = self._matrix(tensors[n[9]], dtype, device)
        if self.own_kv:
            self.norm_w = self._vector(tensors[n[2]], device)
        # per head [rank, qk_dim]: carries a head's query into the latent space
        self.w_uk_t = self._matrix(tensors[n[3]], dtype, device).view(H, D, R).transpose(1, 2).contiguous()
        self.w_uv = self._matrix(tensors[n[4]], dtype, device).view(H, V, R).contiguous()
        self.w_out = self._matrix(tensors[n[6]], dtype, device)
        if self.has_sinks:
            self.sinks = self._vector(tensors[n[10]], device)
        if self.rot_dims:
            if self.rot_blend is not None:
                table, self.rot_length = blended_frequencies(self.rot_base, self.rot_dims, *self.rot_blend)
            else:
                table = rotary_frequencies(self.rot_base, self.rot_dims)
            self.freqs = table.to(device)

    def streamed_weights(self):
        return [self.w_in, self.w_out]

    def forward(self, ctx, h, cache, state):
        if cache is None:
            raise RuntimeError("latent attention needs a cache of latents: its own or the layer's it reads")
        T, H, R, KD = h.shape[0], self.n_head, self.rank, self.key_dim
        HV = H * self.v_dim
        proj = ops.linear(h, self.w_in, None)
        n_q = self.q_rank or H * self.q_head
        gate0, lat0 = n_q, n_q + self.d_gate
        if self.q_rank:
            cq = torch.empty((T, self.q_rank), dtype=h.dtype, device=h.device)
            ops.rms_norm(proj[:, :n_q], self.q_norm_w, self.eps, cq)
            q = ops.linear(cq, self.w_uq, None)
        else:
            q = proj[:, :n_q]
        # per row: every head's query in the latent space (then its rotated part), then this token's key row
        qc = torch.empty((T, self.d_q + (KD if self.own_kv else 0)), dtype=h.dtype, device=h.device)
        ops.linear_heads(q, self.w_uk_t, qc, x_head_stride=self.q_head, out_head_stride=KD)
        if self.rot_dim:
            ops.rope_rows(q, self.qk_dim, self.q_head, qc, R, KD, ctx.positions, H, self.rot_dim, self.rot_dims, self.freqs,
                          neighbours=self.rot_neighbours, length=self.rot_length)
        if self.own_kv:
            ops.rms_norm(proj[:, lat0:lat0 + R], self.norm_w, self.eps, qc[:, self.d_q:self.d_q + R])
            if self.rot_dim:
                ops.rope_rows(proj, lat0 + R, 0, qc, self.d_q + R, 0, ctx.positions, 1, self.rot_dim, self.rot_dims,
                              self.freqs, neighbours=self.rot_neighbours, length=self.rot_length)
        mixed = torch.empty((T, H * KD), dtype=h.dtype, device=h.device)
        # stores the key rows (if its own), then attends; a head's result takes `stride` columns of `mixed`
        stride = ctx.attention(self, qc, cache, ctx.groups[cache.group], mixed) or KD
        out = torch.empty((T, HV), dtype=h.dtype, device=h.device)
        ops.linear_heads(mixed, self.w_uv, out, x_head_stride=stride)
        if self.gate == "head":
            ops.head_gate_mul(out, proj[:, gate0:gate0 + H], H, out)
        elif self.gate == "element":
            ops.gate_mul(proj[:, gate0:gate0 + HV], out, "sigmoid", out)
        if ops.linear_residual(out, self.w_out, ctx.residual):      # the product adds into the residual stream itself
            return None
        return Delta(ops.linear(out, self.w_out, None, None, out_dtype=torch.float32))


register_mixer("latent_attention", LatentAttention)
