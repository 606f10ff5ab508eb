"""Rotary position encoding with half-split pairs (element i with i + head_dim/2),
angle = position * f_i, f_i = theta^(-2i/head_dim)
(internal/device/kernels.metal:430-463 rope_f16; internal/device/cpu_ref.go:100-131).

The reference has no frequency scaling.  `scaling` of type "llama3" rescales f_i by
wavelength: kept above the high-frequency bound, divided by `factor` below the
low-frequency bound, blended in between.  Frequencies and angles are worked out in
float64 on the host and tabulated as float32 cos/sin, so every kernel and every
way of cutting the work reads the same angles.

`rotary_dims` r < head_dim rotates only the first r dimensions of a head (pairs i,
i + r/2, f_i = theta^(-2i/r)); the tables are then [positions, r/2].  `scaling` may
also be a `LinearScaling(factor)`: every f_i divided by the factor; or a `YarnScaling`: fast
dimensions keep f_i, slow ones get f_i / factor, the ones in between a blend along a linear ramp
over the dimension index, and cos and sin are both multiplied by 0.1 ln(factor) + 1.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .base import PositionEncoding, Runtime
from .registry import register_part


@dataclass(frozen=True)
class LinearScaling:
    """Positions stretched by `factor`: every frequency is divided by it."""
    factor: float


@dataclass(frozen=True)
class YarnScaling:
    """Frequencies blended between f_i (dimensions that turn more than `fast` times over `original` positions)
    and f_i / factor (fewer than `slow` turns).  With d(t) = dims ln(original / (2 pi t)) / (2 ln base),
    lo = max(floor(d(fast)), 0), hi = min(ceil(d(slow)), dims - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1):
    f_i' = f_i / factor * ramp_i + f_i (1 - ramp_i).  The tables' cos and sin carry the factor 0.1 ln(factor) + 1."""
    factor: float
    original: float
    fast: float
    slow: float

    @property
    def table_factor(self) -> float:
        return 0.1 * math.log(self.factor) + 1.0


def rope_frequencies(head_dim: int, theta: float, scaling=None) -> torch.Tensor:
    """f_i for i < head_dim / 2, float64 (head_dim: the number of rotated dimensions)."""
    i = torch.arange(head_dim // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -2.0 * i / head_dim)
    if scaling is None:
        return f
    if isinstance(scaling, LinearScaling):
        return f / float(scaling.factor)
    if isinstance(scaling, YarnScaling):
        def turn_dim(turns: float) -> float:
            return head_dim * math.log(scaling.original / (2.0 * math.pi * turns)) / (2.0 * math.log(float(theta)))
        lo = max(math.floor(turn_dim(scaling.fast)), 0)
        hi = min(math.ceil(turn_dim(scaling.slow)), head_dim - 1)
        ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        return f / float(scaling.factor) * ramp + f * (1.0 - ramp)
    n0 = float(scaling.original_max_position_embeddings)
    lo, hi, factor = float(scaling.low_freq_factor), float(scaling.high_freq_factor), float(scaling.factor)
    wavelen = 2.0 * math.pi / f
    smooth = (n0 / wavelen - lo) / (hi - lo)
    blended = (1.0 - smooth) * f / factor + smooth * f
    out = torch.where(wavelen > n0 / lo, f / factor, blended)
    return torch.where(wavelen < n0 / hi, f, out)


@register_part("position", "rope")
class Rope(PositionEncoding):
    graph_safe = True

    def __init__(self, runtime: Runtime, head_dim: int, theta: float, scaling=None, rotary_dims: int | None = None):
        self.runtime, self.head_dim, self.theta, self.scaling = runtime, head_dim, float(theta), scaling
        self.rotary_dims = head_dim if rotary_dims is None else int(rotary_dims)
        if self.rotary_dims % 2 or not 0 < self.rotary_dims <= head_dim:
            raise ValueError(f"rope: {self.rotary_dims} rotated dimensions must be even and at most head_dim {head_dim}")
        self._tables = None

    def tables(self):
        if self._tables is None:
            key = ("rope", self.rotary_dims, self.theta, self.scaling, self.runtime.max_context)
            if key not in self.runtime.shared:
                f = rope_frequencies(self.rotary_dims, self.theta, self.scaling)
                pos = torch.arange(self.runtime.max_context, dtype=torch.float64)
                ang = pos[:, None] * f[None, :]
                mult = float(getattr(self.scaling, "table_factor", 1.0))
                self.runtime.shared[key] = ((torch.cos(ang) * mult).to(torch.float32).to(self.runtime.device).contiguous(),
                                            (torch.sin(ang) * mult).to(torch.float32).to(self.runtime.device).contiguous())
            self._tables = self.runtime.shared[key]
        return self._tables
