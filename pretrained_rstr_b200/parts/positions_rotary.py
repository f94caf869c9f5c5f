"""Frequencies of rotary positions in the rotate-half layout: coordinate i < dims / 2 pairs
with i + dims / 2 and the pair at position p turns by p * base^(-2 i / dims).  The mixers'
kernels compute the angles in 32-bit from this table and the tokens' positions."""
from __future__ import annotations

import torch


def rotary_frequencies(base: float, dims: int, device) -> torch.Tensor:
    """float32 [max(1, dims / 2)] (a table of one zero when nothing is rotated)."""
    if dims < 0 or dims % 2:
        raise ValueError(f"rotary positions need an even number of coordinates, got {dims}")
    half = dims // 2
    freq = [float(base) ** (-2.0 * i / dims) for i in range(half)] or [0.0]
    return torch.tensor(freq, dtype=torch.float64).to(torch.float32).to(device)
