"""Rotary position encoding (python/helios/exec/model.py:117-153), rotate-half
convention, with the ``llama3`` frequency scaling (not in the reference).

Frequencies are computed once on the host in float64.  Each step the part turns
the batch's positions into a cos/sin table [T, rot/2] (float32, angles taken in
float64), kept for the step under the encoding's own identity: a mixer that was
handed an encoding reads that encoding's table, so layers may rotate by different
bases.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..csrc import ops
from .base import PositionEncoding, register_part


def rotary_frequencies(rotary_dim: int, theta: float, scaling=None) -> torch.Tensor:
    """inv_freq[j] = theta^(-2j/rotary_dim) in float64; with ``scaling`` (an object with
    factor, low_freq_factor, high_freq_factor, original_max_position_embeddings):
    wavelengths below P/high stay, above P/low are divided by factor, between are
    interpolated linearly in (P/wavelength - low) / (high - low)."""
    j = torch.arange(0, rotary_dim, 2, dtype=torch.float64)
    inv = 1.0 / (float(theta) ** (j / rotary_dim))
    if scaling is None:
        return inv
    f, lo, hi = float(scaling.factor), float(scaling.low_freq_factor), float(scaling.high_freq_factor)
    P = float(scaling.original_max_position_embeddings)
    if hi <= lo:
        raise ValueError("rope_scaling: high_freq_factor must exceed low_freq_factor")
    wavelen = 2.0 * math.pi / inv
    smooth = (P / wavelen - lo) / (hi - lo)
    mid = (1.0 - smooth) * inv / f + smooth * inv
    out = torch.where(wavelen > P / lo, inv / f, mid)
    out = torch.where(wavelen < P / hi, inv, out)
    return out


class RotaryEncoding(PositionEncoding):
    def __init__(self, rotary_dim: int, theta: float, scaling=None) -> None:
        if rotary_dim % 2:
            raise ValueError(f"rotary dimension {rotary_dim} must be even")
        self.rotary_dim = rotary_dim
        self.theta = float(theta)
        self.scaling = scaling
        self.inv_freq64 = rotary_frequencies(rotary_dim, theta, scaling)
        self._dev: Optional[torch.Tensor] = None

    def tables(self, ctx):
        """(cos, sin) [T, rot/2] for the step's positions, computed once per step."""
        hit = ctx.step_tables.get(id(self))
        if hit is None:
            if self._dev is None or self._dev.device != ctx.positions.device:
                self._dev = self.inv_freq64.to(ctx.positions.device)
            hit = ctx.step_tables[id(self)] = ops.rotary_table(ctx.positions, self._dev)
        return hit

    def prepare(self, ctx) -> None:
        # the plan's own encoding also serves the mixers that were given none
        ctx.rotary_cos, ctx.rotary_sin = self.tables(ctx)


register_part("position_encoding", "rotary", RotaryEncoding)
