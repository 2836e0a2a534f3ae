"""A plain, slow implementation of the Vatevik design in float64, one function per mechanism.

It shares no code with the engine: it takes a configuration dict (the keys of config.json) and a dict of tensors by
name (numpy arrays), runs one whole sequence, and returns the logits and the residual stream after every layer.
Everything is written from the design's equations:

* the input: a token's row of the table times a constant;
* a layer: x += norm1(mixer(x)); x += norm2(ff(x)): a part reads the stream as it is, only its result is normalised
  (y = r / sqrt(mean(r^2) + eps) * w);
* mixer "retention": per head S <- decay S + k v^T, o = S^T q, with q and k rotated by position and k shortened by
  sqrt(dim); each head's o over its root mean square, times silu of a gate, projected out;
* mixer "attention": grouped heads, one root-mean-square norm over ALL of q (and all of k) before the rotation, a
  rotation whose slow frequencies are stretched, softmax with 1 added to the denominator, values blended with the
  values of the first such layer;
* feed-forward: down(silu(gate h) * (up h));
* the output: the final norm, the token table again (without the constant), a scale and a tanh cap.
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


def linear(x, tensors, name):
    return x @ np.asarray(tensors[name], dtype=np.float64).T


def frequencies(base, dims, scaling=None):
    """f_i = base^(-2i/dims), i < dims/2.  With ``scaling`` (factor, low, high, original): a frequency whose
    wavelength 2 pi / f is shorter than original/high stays; one longer than original/low is divided by factor; in
    between the two are blended by s = (original / wavelength - low) / (high - low): (1 - s) f / factor + s f."""
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=np.float64)
    if scaling is None:
        return f
    factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    out = f.copy()
    for i, fi in enumerate(f):
        wave = 2.0 * math.pi / fi
        if wave < orig / high:
            continue
        if wave > orig / low:
            out[i] = fi / factor
        else:
            s = (orig / wave - low) / (high - low)
            out[i] = (1.0 - s) * fi / factor + s * fi
    return out


def rotate(x, positions, freqs, dims):
    """x [T, heads, width]: in every head the entries i and i + dims/2 (i < dims/2) turn by positions * freqs[i];
    entries from ``dims`` on stay."""
    x = np.array(x, dtype=np.float64)
    half = dims // 2
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freqs[None, :]          # [T, half]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    a, b = x[..., :half].copy(), x[..., half:dims].copy()
    x[..., :half] = a * c - b * s
    x[..., half:dims] = b * c + a * s
    return x


def retention_rows(q, k, v, decays, state=None):
    """q, k [T, H, D], v [T, H, V] (already rotated and scaled); per head S <- decay S + k v^T, o = S^T q.
    Returns o [T, H, V] and the states [H, D, V]."""
    T, H, D = q.shape
    V = v.shape[2]
    S = np.zeros((H, D, V)) if state is None else np.array(state, dtype=np.float64)
    o = np.zeros((T, H, V))
    for t in range(T):
        for h in range(H):
            S[h] = decays[h] * S[h] + np.outer(k[t, h], v[t, h])
            o[t, h] = S[h].T @ q[t, h]
    return o, S


def retention_mixer(h, m, tensors, p, eps, positions=None):
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    positions = np.arange(T) if positions is None else positions
    q = linear(h, tensors, p + "mix.q").reshape(T, H, D)
    k = linear(h, tensors, p + "mix.k").reshape(T, H, D)
    v = linear(h, tensors, p + "mix.v").reshape(T, H, V)
    f = frequencies(m["rot"]["base"], m["rot"]["dims"], m["rot"].get("scaling"))
    q = rotate(q, positions, f, m["rot"]["dims"])
    k = rotate(k, positions, f, m["rot"]["dims"]) * D ** -0.5
    o, _ = retention_rows(q, k, v, [float(d) for d in m["decay"]])
    o = unit_rms(o, eps).reshape(T, H * V)
    return linear(o * silu(linear(h, tensors, p + "mix.g")), tensors, p + "mix.o")


def softmax_plus_one(scores):
    """Weights exp(s_j) / (1 + sum exp(s)): a key-less, value-less entry of score 0 shares the softmax."""
    m = max(scores.max(), 0.0)
    e = np.exp(scores - m)
    return e / (math.exp(-m) + e.sum())


def attention_rows(q, k, v, scale):
    """q [T, H, D], k [T, G, D], v [T, G, V] of one sequence from position 0, causal.  Returns [T, H, V]."""
    T, H = q.shape[:2]
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    for i in range(T):
        for a in range(H):
            g = a // (H // G)
            s = (k[:i + 1, g] @ q[i, a]) * scale
            out[i, a] = softmax_plus_one(s) @ v[:i + 1, g]
    return out


def attention_mixer(h, m, tensors, p, eps, shared, positions=None):
    """``shared``: a dict that lives for one forward pass; the first layer with ``v_mix`` leaves its values there."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    positions = np.arange(T) if positions is None else positions
    q = rms_norm(linear(h, tensors, p + "mix.q"), tensors[p + "mix.q.norm"], eps).reshape(T, H, D)
    k = rms_norm(linear(h, tensors, p + "mix.k"), tensors[p + "mix.k.norm"], eps).reshape(T, G, D)
    v = linear(h, tensors, p + "mix.v").reshape(T, G, V)
    f = frequencies(m["rot"]["base"], m["rot"]["dims"], m["rot"].get("scaling"))
    q = rotate(q, positions, f, m["rot"]["dims"])
    k = rotate(k, positions, f, m["rot"]["dims"])
    if m.get("v_mix"):
        if "v_first" not in shared:
            shared["v_first"] = v
        else:
            lam = float(np.asarray(tensors[p + "mix.vmix"], dtype=np.float64))
            v = (1.0 - lam) * v + lam * shared["v_first"]
    o = attention_rows(q, k, v, m["scale"]).reshape(T, H * V)
    return linear(o, tensors, p + "mix.o")


def feed_forward(h, tensors, p):
    return linear(silu(linear(h, tensors, p + "mlp.gate")) * linear(h, tensors, p + "mlp.up"), tensors, p + "mlp.down")


def forward(cfg, tensors, tokens):
    """Logits [T, vocab] and the residual stream after every layer [layers, T, width] of one whole sequence."""
    eps = cfg["norm"]["eps"]
    table = np.asarray(tensors["embed"], dtype=np.float64)
    x = table[np.asarray(tokens)] * cfg["embedding"]["scale"]
    shared, streams = {}, []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        if layer["type"] == "retention":
            r = retention_mixer(x, layer["mixer"], tensors, p, eps)
        elif layer["type"] == "attention":
            r = attention_mixer(x, layer["mixer"], tensors, p, eps, shared)
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(r, tensors[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + rms_norm(feed_forward(x, tensors, p), tensors[p + "norm2"], eps)
        streams.append(x.copy())
    logits = (rms_norm(x, tensors["final.norm"], eps) @ table.T) * cfg["logit_scale"]
    cap = cfg.get("logit_softcap", 0.0)
    if cap:
        logits = cap * np.tanh(logits / cap)
    return logits, np.stack(streams)
