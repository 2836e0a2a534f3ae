"""Attention over the paged cache with rotated queries and keys, a norm over the whole projections, a sink of
score zero and values blended across layers."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import CacheArray, CacheNeed, Delta, Mixer, register_mixer
from .rotation import rotary_frequencies


class RotaryAttention(Mixer):
    """q, k, v from three matrices stored ``[out, in]`` without biases, run as ONE product.  Keys are ``head_dim``
    wide, values ``v_head_dim``; query head h reads key/value head h // (n_head / n_kv_head).  Then, each optional:

    * ``qk_norm``: ALL of q, before it is split into heads, is divided by its root mean square (eps inside the root)
      and multiplied by a weight as wide as q (``<q>.norm``); the same for all of k.  One norm per projection, not
      one per head.
    * rotation: the first ``rot_dims`` entries of every head of q and k turn by the token's position (pairs i,
      i + rot_dims/2, angle p * rot_base^(-2i/rot_dims), optionally stretched: ``rotary_frequencies``).  Keys are
      cached rotated.
    * ``unit_sink``: the softmax's denominator holds 1 more than the sum over the keys, p_j = exp(s_j) / (1 + sum
      exp(s)): the weights of the keys sum to less than one, what is missing goes nowhere.
    * ``value_blend``: "source": this layer's values, as projected, are left for the later layers of the step;
      "blend": v <- (1 - lambda) v + lambda v_source with the source layer's values of the same token and lambda
      the layer's own scalar ``<blend>``; the blended values are what is cached.  None: neither.

    * ``bias``: q and k (and v, where there is one) have biases, their matrices' names with ``.b``, added to the
      32-bit sums of the projection.
    * ``values_from_keys``: there is no value matrix; a token's values are its keys AS PROJECTED, before the rotation
      (with their bias).  Rotated keys and unrotated values are cached side by side.
    * ``rot_divide``: every frequency of the rotation is divided by it.
    * ``block`` > 0: the query at position p sees only the keys of its own block of ``block`` positions, those from
      p - p mod block on, blocks counted from position 0 of the sequence however a prompt was cut (instead of a
      sliding ``window``; the kernels take both in one signed number, ``mask``).
    * ``head_gate``: head h's output is multiplied by sigmoid of one number per token and head, a projection of the
      mixer's input (``<gate>``, no bias).

    score = (q . k) * scale over the keys up to the query's position (inside ``window``, 0: all), softmax in
    32-bit; the heads side by side are projected out.  ``names``: what follows the layer's prefix in the names of
    q, k, v, the output matrix, the blend scalar and the gate; a norm's weight is its matrix's name with ``.norm``."""

    def __init__(self, width: int, n_head: int, n_kv_head: int, head_dim: int, v_head_dim: int, scale: float,
                 window: int = 0, qk_norm: bool = False, eps: float = 1e-5, rot_base: float = 10000.0, rot_dims: int = 0,
                 rot_stretch=None, unit_sink: bool = False, value_blend: str = None,
                 names=("mix.q", "mix.k", "mix.v", "mix.o", "mix.vmix", "mix.g"), bias: bool = False,
                 values_from_keys: bool = False, rot_divide: float = 1.0, block: int = 0, head_gate: bool = False):
        if n_head % n_kv_head:
            raise ValueError(f"n_head={n_head} is not a multiple of n_kv_head={n_kv_head}")
        for what, v in (("head_dim", head_dim), ("v_head_dim", v_head_dim)):
            if not 0 < int(v) <= ops.ATTENTION_MAX_HEAD_DIM:
                raise ValueError(f"{what}={v} is outside 1..{ops.ATTENTION_MAX_HEAD_DIM}, the widest head any "
                                 f"attention kernel takes")
        if value_blend not in (None, "source", "blend"):
            raise ValueError(f"value_blend {value_blend!r} is not one of [None, 'source', 'blend']")
        self.width, self.n_head, self.n_kv_head = int(width), int(n_head), int(n_kv_head)
        self.head_dim, self.v_head_dim = int(head_dim), int(v_head_dim)
        self.scale, self.own_kv = float(scale), True
        self.block = int(block)
        if self.block < 0 or int(window) < 0 or (self.block and int(window)):
            raise ValueError(f"window={window} and block={block} must not be negative, and only one of them may be set")
        # what the attention kernels are told: w > 0 a sliding window, w < 0 blocks of -w positions, 0 every key
        self.window = -self.block if self.block else int(window)
        self.bias, self.values_from_keys, self.head_gate = bool(bias), bool(values_from_keys), bool(head_gate)
        self.rot_divide = float(rot_divide)
        if self.values_from_keys and (qk_norm or value_blend is not None or int(v_head_dim) != int(head_dim)):
            raise ValueError("values taken from the keys go with neither a norm over the projections nor blended values, "
                             "and are as wide as the keys")
        self.qk_norm, self.eps = bool(qk_norm), float(eps)
        self.rot_base, self.rot_dims = float(rot_base), int(rot_dims)
        if self.rot_dims % 2 or not 0 <= self.rot_dims <= self.head_dim:
            raise ValueError(f"rot_dims={self.rot_dims} must be even and at most head_dim={self.head_dim}")
        self.rot_stretch = None if rot_stretch is None else tuple(float(v) for v in rot_stretch)
        self.unit_sink, self.value_blend = bool(unit_sink), value_blend
        self.d_q, self.d_kv, self.d_v = self.n_head * self.head_dim, self.n_kv_head * self.head_dim, self.n_kv_head * self.v_head_dim
        # wider rows than the kernel that prepares q and k in one pass holds: the same in kernels of their own
        self.one_pass = self.d_q + self.d_kv <= ops.QK_PREPARE_MAX_WIDTH
        defaults = ("mix.q", "mix.k", "mix.v", "mix.o", "mix.vmix", "mix.g")
        self.names = tuple(names) + defaults[len(tuple(names)):]
        self.w_in = self.b_in = self.w_out = self.q_norm_w = self.k_norm_w = self.freqs = self.sinks = None
        self.blend = 0.0

    def cache_need(self):
        # behind a sliding window pages go back; blocks keep theirs (0: nothing is given back)
        return CacheNeed((CacheArray("k", self.n_kv_head, self.head_dim), CacheArray("v", self.n_kv_head, self.v_head_dim)),
                         max(self.window, 0))

    def _inputs(self):
        """(tensor name, rows, has a bias) of the matrices that form the one input product, in its column order."""
        n = self.names
        out = [(n[0], self.d_q, self.bias), (n[1], self.d_kv, self.bias)]
        if not self.values_from_keys:
            out.append((n[2], self.d_v, self.bias))
        if self.head_gate:
            out.append((n[5], self.n_head, False))
        return out

    def tensors(self, prefix):
        n = [prefix + s for s in self.names]
        W = self.width
        out = []
        for name, rows, biased in self._inputs():
            out.append(TensorDecl(prefix + name, (rows, W)))
            if biased:
                out.append(TensorDecl(prefix + name + ".b", (rows,), "vector"))
        out.append(TensorDecl(n[3], (W, self.n_head * self.v_head_dim)))
        if self.qk_norm:
            out += [TensorDecl(n[0] + ".norm", (self.d_q,), "norm_weight"), TensorDecl(n[1] + ".norm", (self.d_kv,), "norm_weight")]
        if self.value_blend is not None:      # the source layer stores the scalar too, unused
            out.append(TensorDecl(n[4], (), "vector"))
        return out

    def load(self, prefix, tensors, dtype, device):
        n = [prefix + s for s in self.names]
        parts = self._inputs()
        self.w_in = torch.cat([self._matrix(tensors[prefix + k], dtype, device) for k, _, _ in parts]).contiguous()   # q | k | v | gate
        if self.bias:
            self.b_in = torch.cat([self._vector(tensors[prefix + k + ".b"], device) if biased
                                   else torch.zeros(rows, dtype=torch.float32, device=device)
                                   for k, rows, biased in parts]).contiguous()
        self.w_out = self._matrix(tensors[n[3]], dtype, device)
        if self.qk_norm:
            self.q_norm_w, self.k_norm_w = self._vector(tensors[n[0] + ".norm"], device), self._vector(tensors[n[1] + ".norm"], device)
        if self.value_blend == "blend":
            self.blend = float(tensors[n[4]].to(torch.float32).reshape(()).item())      # a constant of the model
        self.freqs = rotary_frequencies(self.rot_base, self.rot_dims, self.rot_stretch, self.rot_divide).to(device)
        if self.unit_sink:      # a sink of score 0: exp(0) joins the denominator
            self.sinks = torch.zeros(self.n_head, dtype=torch.float32, device=device)

    def streamed_weights(self):
        return [self.w_in, self.w_out]

    def forward(self, ctx, h, cache, state):
        if cache is None:
            raise RuntimeError("attention needs a cache")
        T = h.shape[0]
        k0, v0 = self.d_q, self.d_q + self.d_kv
        proj = ops.linear(h, self.w_in, self.b_in)
        if self.values_from_keys:
            return self._finish(ctx, h, cache, self._keys_as_values(ctx, proj), proj)
        other = None
        if self.value_blend == "source":
            ctx.shared["value_blend_source"] = proj[:, v0:v0 + self.d_v]       # stays as projected: this layer blends nothing
        elif self.value_blend == "blend":
            other = ctx.shared.get("value_blend_source")
            if other is None or other.shape != (T, self.d_v):
                raise RuntimeError("a layer that blends its values needs an earlier layer of the step that left values "
                                   f"of the same shape [{T}, {self.d_v}]")
        if ops.USE_QK_PREPARE and self.one_pass:
            if self.qk_norm or self.rot_dims or other is not None:
                ops.qk_prepare(proj, 0, self.n_head, k0, self.n_kv_head, self.head_dim, self.q_norm_w, self.k_norm_w,
                               self.eps, ctx.positions, self.freqs, self.rot_dims, v0, self.d_v, other, self.blend)
        else:       # the same in kernels of their own
            q, k, v = proj[:, :k0], proj[:, k0:v0], proj[:, v0:v0 + self.d_v]
            if self.qk_norm:
                ops.rms_norm(q, self.q_norm_w, self.eps, q)
                ops.rms_norm(k, self.k_norm_w, self.eps, k)
            if self.rot_dims:
                ops.rope_rows(proj, 0, self.head_dim, proj, 0, self.head_dim, ctx.positions, self.n_head, self.head_dim,
                              self.rot_dims, self.freqs)
                ops.rope_rows(proj, k0, self.head_dim, proj, k0, self.head_dim, ctx.positions, self.n_kv_head,
                              self.head_dim, self.rot_dims, self.freqs)
            if other is not None:
                ops.blend_rows(v, other, self.blend, v)
        return self._finish(ctx, h, cache, proj, proj)

    def _keys_as_values(self, ctx, proj):
        """q | k | v for the attention kernels from the product's q | k: q and k rotated, and the keys as they were
        projected once more behind them, as the values.  One kernel."""
        T, D = proj.shape[0], self.head_dim
        qkv = torch.empty((T, self.d_q + 2 * self.d_kv), dtype=proj.dtype, device=proj.device)
        ops.rope_rows(proj, 0, D, qkv, 0, D, ctx.positions, self.n_head + self.n_kv_head, D, self.rot_dims, self.freqs,
                      keep_col0=self.d_q + self.d_kv, keep_head0=self.n_head)
        return qkv

    def _finish(self, ctx, h, cache, qkv, proj):
        T = h.shape[0]
        out = torch.empty((T, self.n_head * self.v_head_dim), dtype=h.dtype, device=h.device)
        ctx.attention(self, qkv, cache, ctx.groups[cache.group], out)     # stores k and v, then attends
        if self.head_gate:
            g0 = proj.shape[1] - self.n_head
            ops.head_gate_mul(out, proj[:, g0:g0 + self.n_head], self.n_head, out)
        if ops.linear_residual(out, self.w_out, ctx.residual):
            return None
        return Delta(ops.linear(out, self.w_out, None, None, out_dtype=torch.float32))


register_mixer("rotary_attention", RotaryAttention)
