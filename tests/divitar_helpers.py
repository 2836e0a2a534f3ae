"""Small Divitar configurations with random weights, an engine over them, and the plain implementation's logits."""
import copy

import numpy as np
import torch

import plain_divitar
from figotar_helpers import assert_same, as_numpy, mixed_schedule  # noqa: F401  (the same comparisons and schedules)
from vekedra_helpers import make_engine, run_cut, tokens_of, tolerance  # noqa: F401  (the same engine plumbing)


def blend(factor, original, fast, slow):
    return {"factor": factor, "original": original, "fast": fast, "slow": slow}


def attn(heads, kv_heads, dim, block, scale, base=10000.0, rot_dims=None, factor=None, mlp=None):
    rot = {"base": base, "dims": dim if rot_dims is None else rot_dims}
    if factor is not None:
        rot["scaling"] = {"factor": factor}
    m = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "rot": rot, "scale": scale, "vdim": dim}
    if block:
        m["mask"] = {"size": block}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def latent(heads, dim, rot_dim, vdim, rank, window, scale, base=10000.0, scaling=None, kv_from=None, mlp=None):
    m = {"dim": dim, "heads": heads, "kv_rank": rank, "rot_dim": rot_dim, "scale": scale, "vdim": vdim}
    if rot_dim:
        m["rot"] = {"base": base, "dims": rot_dim}
        if scaling is not None:
            m["rot"]["scaling"] = scaling
    if window:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, scale=None, shared=None):
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if scale is not None:
        f["router"]["scale"] = scale
    if shared:
        f["shared"] = {"ff": shared}
    return f


def config(width, vocab, layers, mult=0.5, logit_scale=0.5, side=None, eps=1e-5):
    d = {"architecture": "Divitar", "layers": copy.deepcopy(layers), "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if mult is not None:
        d["residual_mult"] = mult
    if logit_scale is not None:
        d["logit_scale"] = logit_scale
    if side:
        d["token_side"] = {"dim": side}
    return d


# every mechanism several times: blocks and windows shorter than the prompts, grouped heads, part of a head rotated,
# frequencies of which some stay, some are blended and some are slowed down, latents read from an earlier layer with
# another window, routed experts with and without the expert for all, a layer without a feed-forward
MIXED = config(64, 96, [
    latent(2, 16, 8, 24, 32, 19, 0.25, base=100.0, scaling=blend(4.0, 40, 4.0, 1.0), mlp=dense(80)),
    attn(4, 2, 16, 23, 0.25, base=1000.0, rot_dims=8, factor=4.0, mlp=moe(5, 2, 24, scale=2.5, shared=40)),
    latent(4, 8, 16, 16, 24, 30, 0.3, base=50.0, mlp=moe(6, 3, 16, scale=0.75)),
    attn(2, 2, 24, 64, 0.2, base=30.0, mlp=None),
    latent(2, 16, 8, 8, 32, 41, 0.3, base=100.0, scaling=blend(4.0, 40, 4.0, 1.0), kv_from=0, mlp=dense(48)),
    latent(3, 8, 16, 24, 24, 7, 0.35, base=50.0, kv_from=2, mlp=moe(4, 1, 32, shared=16)),
], mult=0.7, logit_scale=0.5, side=8)
# odd sizes and values that models tend to make equal or 1: widths that are no multiples of 8, one key/value head
# under three query heads and as many key/value heads as query heads, nothing rotated in one layer and two entries in
# another, every expert chosen, one expert, no constant on the results, no scale on the logits, no second table, a
# window of one token and a block of one position, no mask at all
ODD = config(40, 61, [
    attn(3, 1, 12, 1, 0.3, base=20.0, rot_dims=2, mlp=moe(3, 3, 20)),
    latent(3, 12, 6, 20, 20, 1, 0.25, base=9.0, scaling=blend(1.5, 16, 3.0, 0.5), mlp=moe(2, 1, 12, scale=1.0, shared=20)),
    attn(5, 5, 6, 0, 0.4, rot_dims=0, factor=3.0, mlp=dense(56)),
    latent(1, 20, 0, 12, 12, 0, 0.2, mlp=None),
    latent(2, 6, 6, 10, 20, 500, 0.3, base=9.0, scaling=blend(1.5, 16, 3.0, 0.5), kv_from=1, mlp=dense(24)),
], mult=None, logit_scale=None, side=None, eps=1e-4)
# sizes that take the tiled kernels: head sizes 64 and 128 (TMA + tcgen05 prefill, tensor-core decoding), widths in
# multiples of 16, cached rows of 128 and 192, several cache groups
WIDE = config(128, 200, [
    attn(4, 2, 64, 70, 0.12, factor=2.0, mlp=moe(8, 2, 64, scale=1.5, shared=64)),
    latent(4, 32, 32, 48, 96, 50, 0.12, base=1000.0, scaling=blend(8.0, 64, 16.0, 2.0), mlp=dense(192)),
    attn(2, 1, 128, 33, 0.09, rot_dims=64, mlp=None),
    latent(8, 16, 64, 16, 128, 128, 0.15, mlp=dense(96)),
    attn(8, 8, 32, 128, 0.17, base=300.0, factor=8.0, mlp=dense(64)),
    latent(2, 64, 32, 64, 96, 64, 0.1, base=1000.0, scaling=blend(8.0, 64, 16.0, 2.0), kv_from=1, mlp=moe(4, 1, 32)),
], mult=0.4, logit_scale=2.0, side=16)

# layers as wide as a small real model's: products of hundreds of rows on the TMA + tcgen05 kernels with their
# epilogues, routed experts in tiles, head size 64 on the tensor-core attention kernels, a cached row of 128
REAL = config(512, 1000, [
    latent(8, 64, 32, 64, 96, 100, 0.1, base=10000.0, scaling=blend(4.0, 256, 16.0, 1.0), mlp=dense(2048)),
    attn(8, 2, 64, 128, 0.125, factor=4.0, mlp=moe(8, 2, 352, scale=2.0, shared=352)),
    latent(8, 64, 32, 64, 96, 60, 0.1, base=10000.0, scaling=blend(4.0, 256, 16.0, 1.0), kv_from=0, mlp=moe(8, 2, 352, scale=2.0)),
], mult=0.5, logit_scale=0.25, side=32)

ONE_LAYER = {
    "attention": config(64, 80, [attn(4, 2, 16, 21, 0.25, base=500.0, rot_dims=12, factor=2.0, mlp=None)], side=None),
    "latent": config(64, 80, [latent(3, 16, 8, 24, 40, 17, 0.2, base=200.0, scaling=blend(2.0, 32, 8.0, 1.0), mlp=None)], side=None),
    "dense": config(64, 80, [attn(2, 2, 8, 0, 0.3, rot_dims=0, mlp=dense(96))], side=None),
    "routed": config(64, 80, [attn(2, 2, 8, 0, 0.3, rot_dims=0, mlp=moe(6, 2, 24, scale=1.5, shared=32))], side=None),
    "side": config(64, 80, [attn(2, 2, 8, 0, 0.3, rot_dims=0, mlp=None)], side=12),
}


def unrouted(cfgd):
    """The configuration with dense feed-forwards in place of its routed ones: for comparisons of chosen tokens in
    bfloat16, where rounding may send a token to another expert."""
    out = copy.deepcopy(cfgd)
    for layer in out["layers"]:
        if layer["mlp"] is not None and layer["mlp"]["kind"] == "moe":
            layer["mlp"] = dense(48)
    return out


def make_weights(cfgd, seed, std=0.25, tweak=None):
    """Random tensors of the configuration, values exact in bfloat16 (both precisions and the plain implementation
    then see the same numbers); ``tweak(tensors)`` may change some before they are rounded."""
    import cbis_b200 as cb
    from cbis_b200.models import Model
    from cbis_b200.weights import InitScheme, random_tensors
    spec = cb.config_from_dict(cfgd).model_spec()
    tensors = random_tensors(Model(spec).declared(), seed, InitScheme(std, 0.3, 0.2, 0.2), torch.float32, draw_on="cpu")
    W = cfgd["width"]
    for name, t in tensors.items():
        if t.dim() == 2 and name not in ("embed", "side.embed"):
            t.mul_((W / t.shape[1]) ** 0.5)         # keep activations of order one
        if name.endswith(".side.gate"):
            t.mul_(0.3)                             # it reads the stream itself, which is not of order one
        if name.endswith(".sink"):
            t.add_(1.0)                             # a sink that takes a visible share of the denominator
        if name.endswith(".router"):
            t.mul_(4.0)                             # scores apart from one another: few close calls
    if tweak is not None:
        tweak(tensors)
    return {k: v.to(torch.bfloat16).float() for k, v in tensors.items()}


def plain_all(cfgd, tensors, tokens):
    """Logits, the stream after every layer, and the first position at which some routed layer's choice hangs on
    less than 0.02 between two scores (the length if there is none)."""
    logits, streams, gaps = plain_divitar.forward(cfgd, as_numpy(tensors), list(tokens))
    close = [int(np.nonzero(g < 0.02)[0][0]) for g in gaps.values() if (g < 0.02).any()]
    return torch.from_numpy(logits), torch.from_numpy(streams), min(close, default=len(tokens))


def plain(cfgd, tensors, tokens):
    return plain_all(cfgd, tensors, tokens)[0]


def assert_close(got, ref, dtype, what="", first_close=None, tol32=2e-4):
    """32-bit: every row within ``tol32``.  bfloat16: every row before the sequence's first routing close call
    (``first_close``; None: there is no routing) within 4 % of the largest logit, and the median row of all too: an
    expert that rounding flips moves a few rows, a fault moves most."""
    err = (got - ref).abs().max(1).values
    assert torch.isfinite(got).all(), what
    if dtype == "float32":
        assert err.max() < tol32, (what, int(err.argmax()), err.max().item())
        return
    tol = 0.04 * max(1.0, ref.abs().max().item())
    n = len(err) if first_close is None else first_close
    assert n == 0 or err[:n].max() < tol, (what, int(err[:n].argmax()), err[:n].max().item(), n)
    assert err.median() < tol, (what, err.median().item())
