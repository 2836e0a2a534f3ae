"""Small Vatevik configurations with random weights, an engine over them, and the plain implementation's logits."""
import copy

import torch

import plain_vatevik
from figotar_helpers import assert_close, assert_same, as_numpy, mixed_schedule  # noqa: F401  (the same comparisons)
from vekedra_helpers import make_engine, run_cut, tokens_of, tolerance  # noqa: F401  (the same engine plumbing)


def stretch(factor, low, high, original):
    return {"factor": factor, "low": low, "high": high, "original": original}


def ret(heads, dim, vdim, decay, base=10000.0, rot_dims=None, mlp=None):
    m = {"decay": list(decay), "dim": dim, "heads": heads, "rot": {"base": base, "dims": dim if rot_dims is None else rot_dims},
         "vdim": vdim}
    return {"type": "retention", "mixer": m, "mlp": mlp}


def attn(heads, kv_heads, dim, vdim, scale, base=10000.0, rot_dims=None, scaling=None, v_mix=False, mlp=None):
    rot = {"base": base, "dims": dim if rot_dims is None else rot_dims}
    if scaling is not None:
        rot["scaling"] = scaling
    m = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "rot": rot, "scale": scale, "v_mix": v_mix, "vdim": vdim}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def config(width, vocab, layers, emb_scale=4.0, logit_scale=0.5, softcap=20.0, eps=1e-5):
    d = {"architecture": "Vatevik", "embedding": {"scale": emb_scale}, "layers": copy.deepcopy(layers),
         "logit_scale": logit_scale, "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if softcap:
        d["logit_softcap"] = softcap
    return d


# both mixers several times: an attention layer that blends nothing before the one whose values the later ones take,
# grouped heads, values wider and narrower than keys, half of a head rotated, frequencies of which one stays, one is
# blended and two are slowed down, a decay of exactly 1 and one that forgets within a few tokens, a layer without a
# feed-forward, retention with keys and values of unlike widths
MIXED = config(64, 96, [
    attn(4, 2, 16, 24, 0.25, base=1000.0, rot_dims=8, scaling=stretch(8.0, 1.0, 4.0, 64), mlp=dense(80)),
    ret(2, 16, 24, [0.9, 0.995], base=100.0, mlp=dense(48)),
    attn(4, 2, 8, 12, 0.3, base=50.0, v_mix=True, mlp=None),
    ret(4, 8, 8, [1.0, 0.5, 0.98, 0.9990234375], rot_dims=4, mlp=dense(40)),
    attn(6, 2, 8, 12, 0.35, base=500.0, rot_dims=6, scaling=stretch(2.0, 2.0, 8.0, 32), v_mix=True, mlp=dense(32)),
    attn(2, 2, 16, 12, 0.2, v_mix=True, mlp=dense(24)),
])
# odd sizes: three heads over one key/value head, widths that are no multiples of 8, nothing rotated in one layer and
# two entries in another, one head of retention, a retention wider than 32 columns, no cap on the logits
ODD = config(40, 61, [
    ret(1, 12, 20, [0.97], base=20.0, rot_dims=2, mlp=dense(24)),
    attn(3, 1, 12, 20, 0.3, rot_dims=0, v_mix=True, mlp=None),
    attn(2, 1, 20, 20, 0.2, base=30.0, rot_dims=10, v_mix=True, mlp=dense(16)),
    ret(3, 20, 44, [0.8, 0.99, 0.999], rot_dims=0, mlp=None),
    attn(5, 5, 6, 10, 0.4, base=9.0, mlp=dense(56)),
], emb_scale=2.5, logit_scale=1.5, softcap=0.0, eps=1e-4)
# sizes that take the tiled kernels: widths in multiples of 8 and 16 up to 128, several cache groups, retention of 64
# and 128 with 48 and 80 columns
WIDE = config(128, 200, [
    attn(4, 2, 48, 80, 0.14, base=10000.0, scaling=stretch(4.0, 1.0, 4.0, 128), v_mix=True, mlp=dense(192)),
    ret(2, 64, 48, [0.99, 0.999], mlp=dense(128)),
    attn(2, 1, 128, 64, 0.09, rot_dims=64, mlp=None),
    attn(8, 2, 32, 80, 0.17, base=300.0, v_mix=True, mlp=dense(64)),
    ret(1, 128, 80, [0.995], rot_dims=32, mlp=None),
    attn(8, 8, 24, 40, 0.2, mlp=dense(64)),
], emb_scale=6.0)


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
        if t.dim() == 2 and name != "embed":
            t.mul_((W / t.shape[1]) ** 0.5 / cfgd["embedding"]["scale"] ** 0.5)     # parts read the stream itself: keep them of order one
        if name.endswith(".vmix"):
            t.copy_(0.5 + 0.35 * torch.tanh(4 * t))                                   # a share between 0.15 and 0.85
    if tweak is not None:
        tweak(tensors)
    return {k: v.to(torch.bfloat16).float() for k, v in tensors.items()}


def plain(cfgd, tensors, tokens):
    logits, _ = plain_vatevik.forward(cfgd, as_numpy(tensors), list(tokens))
    return torch.from_numpy(logits)
