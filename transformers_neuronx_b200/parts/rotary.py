"""Rotation of pairs of dims by position ("rotary" encoding), as constants for the kernels that apply it:
pair i of `dims` dims turns by position * base^(-2 i / dims), optionally stretched for long contexts
(spec.FrequencyRampSpec).  The frequencies are computed in 64-bit on the host and rounded once to 32-bit; the angle
itself (position * frequency) and its sine and cosine are computed in 32-bit inside the kernels."""
from __future__ import annotations

import math

import torch


def inverse_frequencies(dims: int, base: float, device, scaling=None) -> torch.Tensor:
    if dims <= 0 or dims % 2:
        raise ValueError(f"a rotation needs an even, positive number of dims, got {dims}")
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims)
    if scaling is not None:
        def turns(t):
            return dims * math.log(scaling.original / (2.0 * math.pi * t)) / (2.0 * math.log(base))
        lo = max(math.floor(turns(scaling.fast)), 0)
        hi = min(math.ceil(turns(scaling.slow)), dims - 1)
        ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        f = f / float(scaling.factor) * ramp + f * (1.0 - ramp)
    return f.to(torch.float32).to(device)


def rotation_magnitude(scaling=None) -> float:
    """What sines and cosines are multiplied by: 1, or 0.1 ln(factor) + 1 with stretched frequencies."""
    return 1.0 if scaling is None else 0.1 * math.log(float(scaling.factor)) + 1.0
