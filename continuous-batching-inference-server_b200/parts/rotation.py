"""Frequencies of a rotation of queries and keys by position."""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch


def rotary_frequencies(base: float, dims: int, stretch: Optional[Sequence[float]] = None,
                       divide: float = 1.0) -> torch.Tensor:
    """f_i = base^(-2 i / dims) for i < dims / 2, as 32-bit numbers made in 64-bit and rounded once; the angle of
    pair i at position p is p * f_i.

    ``stretch`` = (factor, low, high, original) slows the slow pairs down so that a model reaches further than the
    ``original`` positions it was made for (the scheme of Llama 3.1): with the wavelength l = 2 pi / f, a pair with
    l < original / high keeps f; one with l > original / low gets f / factor; between the two, with
    s = (original / l - low) / (high - low), it gets (1 - s) f / factor + s f.

    ``divide``: every frequency is divided by it (positions stretched evenly)."""
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
        out.append(f / float(divide))
    return torch.tensor(out, dtype=torch.float64).to(torch.float32)


def blended_frequencies(base: float, dims: int, factor: float, original: float, fast: float, slow: float):
    """Frequencies slowed down by pair INDEX (the scheme known as YaRN), and the factor by which the rotation's cosines
    and sines are lengthened.  With pair(t) = dims * ln(original / (2 pi t)) / (2 ln base), the pair that makes t turns
    within ``original`` positions, lo = max(floor(pair(fast)), 0) and hi = min(ceil(pair(slow)), dims - 1): pair i
    gets f_i / factor * r + f_i * (1 - r) with r = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), so pairs up to lo keep
    f_i and pairs from hi on get f_i / factor.  The length is 0.1 ln(factor) + 1.  Returns (table as 32-bit numbers
    made in 64-bit and rounded once, length)."""
    if dims < 0 or dims % 2:
        raise ValueError(f"rotated dims={dims} must be even and not negative")
    base, factor, original = float(base), float(factor), float(original)

    def pair(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * float(turns))) / (2.0 * math.log(base))

    lo = max(math.floor(pair(fast)), 0)
    hi = min(math.ceil(pair(slow)), dims - 1)
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        r = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * r + f * (1.0 - r))
    return torch.tensor(out, dtype=torch.float64).to(torch.float32), 0.1 * math.log(factor) + 1.0
