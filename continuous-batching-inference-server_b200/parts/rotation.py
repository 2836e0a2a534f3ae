"""Frequencies of a rotation of queries and keys by position."""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch


def rotary_frequencies(base: float, dims: int, stretch: Optional[Sequence[float]] = None) -> torch.Tensor:
    """f_i = base^(-2 i / dims) for i < dims / 2, as 32-bit numbers made in 64-bit and rounded once; the angle of
    pair i at position p is p * f_i.

    ``stretch`` = (factor, low, high, original) slows the slow pairs down so that a model reaches further than the
    ``original`` positions it was made for (the scheme of Llama 3.1): with the wavelength l = 2 pi / f, a pair with
    l < original / high keeps f; one with l > original / low gets f / factor; between the two, with
    s = (original / l - low) / (high - low), it gets (1 - s) f / factor + s f."""
    if dims < 0 or dims % 2:
        raise ValueError(f"rotated dims={dims} must be even and not negative")
    out = []
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        if stretch is not None:
            factor, low, high, original = (float(v) for v in stretch)
            wave = 2.0 * math.pi / f
            if wave > original / low:
                f = f / factor
            elif wave >= original / high:
                s = (original / wave - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=torch.float64).to(torch.float32)
