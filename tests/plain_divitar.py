"""A plain, slow implementation of the Divitar design in float64, one function per mechanism.

It shares no code with the engine: it takes a configuration dict (the keys of config.json) and a dict of tensors by
name (numpy arrays), runs one whole sequence, and returns the logits and the residual stream after every layer.
Everything is written from the design's equations:

* the input: a token's row of the table;
* a layer: x += m mixer(norm1(x)); x += m ff(norm2(x)); then the token's own input of the layer:
  y = proj(gelu_tanh(gate x) * e_token), x += m unit_rms(y) * w, with e_token the layer's part of a second table's row;
  all norms are r / sqrt(mean(r^2) + eps) * w;
* mixer "attention": grouped heads, biases on q and k, the values are the keys as projected (before the rotation),
  rotate-half pairs turned by position with all frequencies divided by a factor, keys seen only inside the query's own
  block of positions, ordinary softmax, one sigmoid gate per head and token;
* mixer "latent_attention": one cached latent (normalised) and one rotated key part per token, keys and values per
  head from the latent, neighbouring pairs turned by position with frequencies blended between f and f / factor and
  lengthened cosines and sines, a sliding window, a learned number per head in the softmax's denominator; a layer may
  read the latent and rotated part of an earlier layer;
* feed-forward: down(relu(up h)^2), or experts down(silu(gate h) * (up h)) chosen by the largest sigmoid scores,
  weighted by their scores over their sum times a constant, plus one expert that every token uses;
* the output: the final norm, the head matrix, a scale.
"""
from __future__ import annotations

import math

import numpy as np


def unit_rms(x, eps):
    x = np.asarray(x, dtype=np.float64)
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, w, eps):
    return unit_rms(x, eps) * np.asarray(w, dtype=np.float64)


def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def linear(x, tensors, name, bias=False):
    y = x @ np.asarray(tensors[name], dtype=np.float64).T
    if bias:
        y = y + np.asarray(tensors[name + ".b"], dtype=np.float64)
    return y


# ---- rotations ---------------------------------------------------------------------------------------------------
def plain_frequencies(base, dims):
    return np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=np.float64)


def divided_frequencies(base, dims, factor):
    """Every frequency divided by one factor."""
    return plain_frequencies(base, dims) / factor


def blended_frequencies(base, dims, factor, original, fast, slow):
    """Pair i keeps f_i below ``lo``, gets f_i / factor above ``hi`` and a blend between; lo and hi are the pairs that
    make ``fast`` and ``slow`` turns within ``original`` positions.  Returns the frequencies and the factor by which
    cosines and sines are lengthened."""
    def pair_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(pair_of(fast)), 0)
    hi = min(math.ceil(pair_of(slow)), dims - 1)
    f = plain_frequencies(base, dims)
    out = np.empty_like(f)
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out[i] = fi / factor * ramp + fi * (1.0 - ramp)
    return out, 0.1 * math.log(factor) + 1.0


def rotate_half(x, positions, freqs, dims):
    """x [T, heads, width]: entries i and i + dims/2 (i < dims/2) of every head turn by positions * freqs[i]."""
    x = np.array(x, dtype=np.float64)
    half = dims // 2
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freqs[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    a, b = x[..., :half].copy(), x[..., half:dims].copy()
    x[..., :half] = a * c - b * s
    x[..., half:dims] = b * c + a * s
    return x


def rotate_neighbours(x, positions, freqs, dims, length=1.0):
    """x [T, heads, width]: entries 2i and 2i + 1 (i < dims/2) of every head turn by positions * freqs[i]; cosine and
    sine are multiplied by ``length``."""
    x = np.array(x, dtype=np.float64)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freqs[None, :]
    c, s = (np.cos(ang) * length)[:, None, :], (np.sin(ang) * length)[:, None, :]
    a, b = x[..., 0:dims:2].copy(), x[..., 1:dims:2].copy()
    x[..., 0:dims:2] = a * c - b * s
    x[..., 1:dims:2] = b * c + a * s
    return x


# ---- which keys a query sees ---------------------------------------------------------------------------------------
def sees_block(i, j, size):
    """Keys of the query's own block of ``size`` positions, up to itself (``size`` 0: all keys up to itself)."""
    return j <= i and (size == 0 or i // size == j // size)


def sees_window(i, j, size):
    """The query itself and the size - 1 positions before it (``size`` 0: all before it)."""
    return 0 <= i - j and (size == 0 or i - j < size)


def softmax_rows(scores, positions, sees, sink=None):
    """scores [T, T] (query, key): weights over the keys a query sees; ``sink``: a number whose exponential joins the
    denominator."""
    T = scores.shape[0]
    w = np.zeros_like(scores)
    for a in range(T):
        vis = [b for b in range(T) if sees(positions[a], positions[b])]
        s = scores[a, vis]
        m = s.max() if sink is None else max(s.max(), sink)
        e = np.exp(s - m)
        den = e.sum() + (0.0 if sink is None else math.exp(sink - m))
        w[a, vis] = e / den
    return w


# ---- mixers --------------------------------------------------------------------------------------------------------
def attention(m, tensors, prefix, h, positions):
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    rot = m.get("rot")
    q = linear(h, tensors, prefix + "mix.q", bias=True).reshape(T, H, D)
    k = linear(h, tensors, prefix + "mix.k", bias=True).reshape(T, G, D)
    v = k.copy()                                  # the values are the keys as projected
    if rot is not None and rot["dims"]:
        factor = (rot.get("scaling") or {}).get("factor", 1.0)
        freqs = divided_frequencies(rot["base"], rot["dims"], factor)
        q = rotate_half(q, positions, freqs, rot["dims"])
        k = rotate_half(k, positions, freqs, rot["dims"])
    gate = sigmoid(linear(h, tensors, prefix + "mix.g"))          # [T, H]
    size = (m.get("mask") or {}).get("size", 0)
    out = np.zeros((T, H, D))
    for head in range(H):
        g = head // (H // G)
        scores = (q[:, head] @ k[:, g].T) * m["scale"]
        w = softmax_rows(scores, positions, lambda i, j: sees_block(i, j, size))
        out[:, head] = (w @ v[:, g]) * gate[:, head:head + 1]
    return linear(out.reshape(T, H * D), tensors, prefix + "mix.o")


def latent_and_key_part(m, tensors, prefix, h, positions, eps):
    """What a layer with a down-projection of its own caches per token: the normalised latent and the rotated part."""
    R, P = m["kv_rank"], m.get("rot_dim", 0)
    ckv = linear(h, tensors, prefix + "mix.dkv")
    c = rms_norm(ckv[:, :R], tensors[prefix + "mix.dkv.norm"], eps)
    if not P:
        return c, np.zeros((h.shape[0], 0))
    freqs, length = latent_rotation(m)
    kr = rotate_neighbours(ckv[:, None, R:R + P], positions, freqs, m["rot"]["dims"], length)[:, 0]
    return c, kr


def latent_rotation(m):
    rot = m["rot"]
    sc = rot.get("scaling")
    if sc is None:
        return plain_frequencies(rot["base"], rot["dims"]), 1.0
    return blended_frequencies(rot["base"], rot["dims"], sc["factor"], sc["original"], sc["fast"], sc["slow"])


def latent_attention(m, tensors, prefix, h, positions, c, kr):
    """``c`` [T, rank] and ``kr`` [T, rot_dim]: the latents and rotated key parts (this layer's or another's)."""
    T = h.shape[0]
    H, D, P, V, R = m["heads"], m["dim"], m.get("rot_dim", 0), m["vdim"], m["kv_rank"]
    q = linear(h, tensors, prefix + "mix.q").reshape(T, H, D + P)
    qr = q[:, :, D:]
    if P:
        freqs, length = latent_rotation(m)
        qr = rotate_neighbours(qr, positions, freqs, m["rot"]["dims"], length)
    k = linear(c, tensors, prefix + "mix.uk").reshape(T, H, D)
    v = linear(c, tensors, prefix + "mix.uv").reshape(T, H, V)
    sinks = np.asarray(tensors[prefix + "mix.sink"], dtype=np.float64)
    size = (m.get("mask") or {}).get("size", 0)
    out = np.zeros((T, H, V))
    for head in range(H):
        scores = (q[:, head, :D] @ k[:, head].T + qr[:, head] @ kr.T) * m["scale"]
        w = softmax_rows(scores, positions, lambda i, j: sees_window(i, j, size), sink=float(sinks[head]))
        out[:, head] = w @ v[:, head]
    return linear(out.reshape(T, H * V), tensors, prefix + "mix.o")


# ---- feed-forwards -------------------------------------------------------------------------------------------------
def dense_ff(tensors, prefix, h):
    a = np.maximum(linear(h, tensors, prefix + "up"), 0.0) ** 2
    return linear(a, tensors, prefix + "down")


def expert(tensors, prefix, h):
    return linear(silu(linear(h, tensors, prefix + "gate")) * linear(h, tensors, prefix + "up"), tensors, prefix + "down")


def route(tensors, prefix, h, top, scale):
    """Per row: the chosen experts, their weights, and the gap between the last chosen score and the next one."""
    s = sigmoid(linear(h, tensors, prefix + "router"))
    order = np.argsort(-s, axis=-1, kind="stable")
    ids = order[:, :top]
    chosen = np.take_along_axis(s, ids, axis=-1)
    weights = chosen / (chosen.sum(axis=-1, keepdims=True) + 1e-20) * scale
    gap = (chosen[:, -1] - np.take_along_axis(s, order[:, top:top + 1], axis=-1)[:, 0]) if s.shape[1] > top else np.full(len(s), np.inf)
    return ids, weights, gap


def routed_ff(f, tensors, prefix, h):
    ids, weights, gap = route(tensors, prefix, h, f["router"]["top"], f["router"].get("scale", 1.0))
    out = np.zeros((h.shape[0], np.asarray(tensors[prefix + "e0.down"]).shape[0]))
    for t in range(h.shape[0]):
        for e, w in zip(ids[t], weights[t]):
            out[t] += w * expert(tensors, f"{prefix}e{e}.", h[t:t + 1])[0]
    if f.get("shared") is not None:
        out += expert(tensors, prefix + "shared.", h)
    return out, gap


# ---- the token's own input of a layer ------------------------------------------------------------------------------
def token_side(tensors, prefix, x, tokens, layer, dim, eps):
    e = np.asarray(tensors["side.embed"], dtype=np.float64)[tokens, layer * dim:(layer + 1) * dim]
    g = gelu_tanh(linear(x, tensors, prefix + "side.gate")) * e
    y = linear(g, tensors, prefix + "side.proj")
    return unit_rms(y, eps) * np.asarray(tensors[prefix + "side.norm"], dtype=np.float64)


# ---- the model -----------------------------------------------------------------------------------------------------
def forward(cfg, tensors, tokens, positions=None):
    """Logits [T, vocab], the residual stream after every layer [L, T, width], and per routed layer the rows' gaps
    between the last chosen expert's score and the first one left out."""
    tokens = list(tokens)
    T = len(tokens)
    positions = list(range(T)) if positions is None else list(positions)
    eps, m = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    side = cfg.get("token_side")
    x = np.asarray(tensors["embed"], dtype=np.float64)[tokens]
    kept, streams, gaps = {}, [], {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        mix = layer["mixer"]
        h = rms_norm(x, tensors[p + "norm1"], eps)
        if layer["type"] == "attention":
            y = attention(mix, tensors, p, h, positions)
        else:
            src = mix.get("kv_from")
            if src is None:
                kept[i] = latent_and_key_part(mix, tensors, p, h, positions, eps)
                src = i
            y = latent_attention(mix, tensors, p, h, positions, *kept[src])
        x = x + m * y
        f = layer.get("mlp")
        if f is not None:
            h = rms_norm(x, tensors[p + "norm2"], eps)
            if f["kind"] == "dense":
                y = dense_ff(tensors, p + "mlp.", h)
            else:
                y, gaps[i] = routed_ff(f, tensors, p + "mlp.", h)
            x = x + m * y
        if side is not None:
            x = x + m * token_side(tensors, p, x, tokens, i, side["dim"], eps)
        streams.append(x.copy())
    h = rms_norm(x, tensors["final.norm"], eps)
    logits = linear(h, tensors, "head") * cfg.get("logit_scale", 1.0)
    return logits, np.stack(streams), gaps


def attention_rows(q, k, v, scale, sees, sinks=None, positions=None):
    """Attention alone: q [T, H, D], k [T, G, D], v [T, G, V] of one sequence; ``sees(i, j)`` says which keys the
    query at position i takes; ``sinks`` [H] join the denominators.  Returns [T, H, V]."""
    q, k, v = (np.asarray(a, dtype=np.float64) for a in (q, k, v))
    T, H, _ = q.shape
    G = k.shape[1]
    positions = list(range(T)) if positions is None else list(positions)
    out = np.zeros((T, H, v.shape[2]))
    for head in range(H):
        g = head // (H // G)
        w = softmax_rows((q[:, head] @ k[:, g].T) * scale, positions, sees, None if sinks is None else float(sinks[head]))
        out[:, head] = w @ v[:, g]
    return out
