"""Rotary position encoding as a table of cosines and sines.

``inv_freq[j] = 1 / theta^(2j / rotary_dim)`` and ``angle[p, j] = float(p) * inv_freq[j]``
are computed on the CPU in float32, as the reference does so that no device or
dtype conversion can round the frequencies (qil/model.py:99-108); cosine and sine
are then rounded to the activation dtype as in ``rotate`` (qil/model.py:42-46) and
kept as float32.  Mixers hand the table to their kernels: a kernel never derives
an angle itself, so another encoding (partial rotation, scaled frequencies) is
another table.
"""
from __future__ import annotations

import math

import torch

from .base import PositionEncoding


def rotary_table(rotary_dim, theta, positions, dtype) -> torch.Tensor:
    """float32 [positions, rotary_dim]: cos of the rotary_dim/2 angles, then their sines."""
    exponent = torch.arange(0, rotary_dim, 2, device="cpu", dtype=torch.float32) / rotary_dim
    inv_freq = 1.0 / (theta ** exponent)
    angles = torch.arange(positions, device="cpu").float()[:, None] * inv_freq[None, :]
    table = torch.cat((angles.cos(), angles.sin()), dim=-1)
    return table.to(dtype).float().contiguous()


class RotaryEmbedding(PositionEncoding):
    graph_safe = True

    def __init__(self, rotary_dim, theta, max_positions):
        if rotary_dim % 2 or rotary_dim <= 0:
            raise ValueError(f"rotary_dim must be positive and even, got {rotary_dim}")
        self.rotary_dim, self.theta, self.max_positions = int(rotary_dim), float(theta), int(max_positions)
        self.table = None

    def finalize(self, device, dtype):
        self.table = rotary_table(self.rotary_dim, self.theta, self.max_positions, dtype).to(device)


class RotaryFrequencies(PositionEncoding):
    """Rotation whose angles the kernels compute themselves, in float32: pair i at position p turns by
    ``float(p) * freq[i]`` with ``freq[i] = base^(-2 i / dims)``, i < dims / 2.  No table: a request may be as long
    as the cache allows.  ``layout`` says which of the ``dims`` rotated dimensions of a vector pair up:
    ``"halves"`` (i with i + dims / 2) or ``"interleaved"`` (2 i with 2 i + 1); dimensions from ``dims`` on pass
    unchanged.  The frequencies are made on the host in float64 and rounded once to float32.

    ``scaling`` = (factor, low, high, original) stretches long waves for contexts beyond the ``original`` one: with
    wavelength l = 2 pi / freq, a frequency stays when l < original / high, becomes freq / factor when
    l > original / low, and between the two is (1 - s) freq / factor + s freq with
    s = (original / l - low) / (high - low)."""
    graph_safe = True
    LAYOUTS = {"halves": 0, "interleaved": 1}

    def __init__(self, dims, base, layout="halves", scaling=None):
        if dims % 2 or dims <= 0:
            raise ValueError(f"the number of rotated dimensions must be positive and even, got {dims}")
        if layout not in self.LAYOUTS:
            raise ValueError(f"unknown rotary layout {layout!r} (known: {sorted(self.LAYOUTS)})")
        self.rotary_dim, self.base, self.layout = int(dims), float(base), self.LAYOUTS[layout]
        self.scaling = None if scaling is None else tuple(float(v) for v in scaling)
        if self.scaling is not None and (len(self.scaling) != 4 or self.scaling[0] <= 0 or self.scaling[3] <= 0
                                         or not 0 < self.scaling[1] < self.scaling[2]):
            raise ValueError(f"frequency scaling wants (factor, low, high, original) with 0 < low < high, got {scaling}")
        self.freq = None

    def frequencies(self) -> list:
        """The frequency of every rotated pair as Python floats (float64)."""
        values = [self.base ** (-2.0 * i / self.rotary_dim) for i in range(self.rotary_dim // 2)]
        if self.scaling is None:
            return values
        factor, low, high, original = self.scaling
        for i, f in enumerate(values):
            wave = 2.0 * math.pi / f
            if wave > original / low:
                values[i] = f / factor
            elif wave >= original / high:
                s = (original / wave - low) / (high - low)
                values[i] = (1.0 - s) * f / factor + s * f
        return values

    def finalize(self, device, dtype):
        values = self.frequencies()
        self.freq = torch.tensor(values, dtype=torch.float64).to(torch.float32).to(device)
