"""Rotary position encoding as a table of frequencies.

Dimension i of the rotated part is paired with dimension i + dims/2 ("rotate half"); the pair (u, v) at
position p becomes (u cos a - v sin a, v cos a + u sin a) with a = p * f_i, f_i = base^(-2i/dims).

YaRN scaling (``scaling`` = {factor, original, fast, slow}) stretches the slow pairs for contexts beyond the
``original`` length: a pair that makes t turns over the original context sits at
d(t) = dims * ln(original / (2 pi t)) / (2 ln base); with lo = max(floor(d(fast)), 0), hi = min(ceil(d(slow)), dims - 1)
and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1) the frequency is f_i / factor * ramp_i + f_i * (1 - ramp_i),
and cos and sin are multiplied by 0.1 * ln(factor) + 1.  The kernels take the table (float32) and the factor; they
compute the angle, cos and sin in 32-bit at the token's position.

Scaling by wavelength (``scaling`` = {factor, low, high, original}; the form Llama 3.1 uses): a pair whose wavelength
l_i = 2 pi / f_i is shorter than original / high keeps its frequency, one longer than original / low turns ``factor``
times slower, and between the two the frequency is (1 - s) f_i / factor + s f_i with s = (original / l_i - low) /
(high - low); cos and sin keep their size.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple


def rotary_table(dims: int, base: float, scaling: Optional[dict] = None) -> Tuple[list, float]:
    """(frequencies [dims/2] as Python floats, the factor on cos and sin)."""
    if dims < 0 or dims % 2:
        raise ValueError(f"rotary: {dims} rotated dimensions (an even number)")
    half = dims // 2
    f = [float(base) ** (-2.0 * i / dims) for i in range(half)]
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])
    if "low" in scaling or "high" in scaling:
        low, high = float(scaling["low"]), float(scaling["high"])
        if not (high > low > 0 and factor > 0 and orig > 0):
            raise ValueError(f"rotary: scaling by wavelength needs high > low > 0 and positive factor and original, got {scaling!r}")
        scaled = []
        for fi in f:
            turns = orig * fi / (2.0 * math.pi)          # original / wavelength: turns over the original context
            if turns > high:
                scaled.append(fi)
            elif turns < low:
                scaled.append(fi / factor)
            else:
                s = (turns - low) / (high - low)
                scaled.append((1.0 - s) * fi / factor + s * fi)
        return scaled, 1.0

    def at(turns: float) -> float:
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(float(base)))

    lo = max(math.floor(at(float(scaling["fast"]))), 0)
    hi = min(math.ceil(at(float(scaling["slow"]))), dims - 1)
    out = []
    for i in range(half):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f[i] / factor * ramp + f[i] * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0
