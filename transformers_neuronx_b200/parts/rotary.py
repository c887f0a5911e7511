"""Rotation of pairs of dims by position ("rotary" encoding), as constants for the kernels that apply it:
pair i of `dims` dims turns by position * base^(-2 i / dims).  The frequencies are computed in 64-bit on the
host and rounded once to 32-bit; the angle itself (position * frequency) and its sine and cosine are
computed in 32-bit inside the kernels."""
from __future__ import annotations

import torch


def inverse_frequencies(dims: int, base: float, device) -> torch.Tensor:
    if dims <= 0 or dims % 2:
        raise ValueError(f"a rotation needs an even, positive number of dims, got {dims}")
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims)
    return f.to(torch.float32).to(device)
