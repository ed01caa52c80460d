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
over the dimension index, and cos and sin are both multiplied by 0.1 ln(factor) + 1; or a `WavelengthScaling`,
the same rescaling by wavelength as "llama3" with its four constants given directly.

`layout="interleaved"` pairs dimension 2i with 2i + 1 instead of i with i + r/2.  The kernels keep their
half-split form: a mixer that uses this part reorders the rows of its query and key projections once, at load
(`pair_order`), so that the interleaved pairs land where the kernels look for them.  Scores are sums over a head's
dimensions and do not change when queries and keys are reordered alike; only the order inside a cached key differs.
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


@dataclass(frozen=True)
class WavelengthScaling:
    """With wavelength l = 2 pi / f: f kept where l < original / high, f / factor where l > original / low, and between
    the two (1 - s) f / factor + s f with s = (original / l - low) / (high - low)."""
    factor: float
    low: float
    high: float
    original: float

    # the names under which `rope_frequencies` reads the same four constants of a "llama3" rope_scaling
    @property
    def low_freq_factor(self) -> float:
        return self.low

    @property
    def high_freq_factor(self) -> float:
        return self.high

    @property
    def original_max_position_embeddings(self) -> float:
        return self.original


def pair_order(head_dim: int, rotary_dims: int) -> list[int]:
    """Where each dimension of a head comes from when interleaved pairs (2i, 2i + 1) of the first `rotary_dims`
    dimensions are laid out half-split (i, i + rotary_dims / 2): [0, 2, 4, ..., 1, 3, 5, ..., the rest in place]."""
    return list(range(0, rotary_dims, 2)) + list(range(1, rotary_dims, 2)) + list(range(rotary_dims, head_dim))


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
    smooth = (n0 / wavelen - lo) / ((hi - lo) or 1.0)
    blended = (1.0 - smooth) * f / factor + smooth * f
    out = torch.where(wavelen > n0 / lo, f / factor, blended)
    return torch.where(wavelen < n0 / hi, f, out)


@register_part("position", "rope")
class Rope(PositionEncoding):
    graph_safe = True

    def __init__(self, runtime: Runtime, head_dim: int, theta: float, scaling=None, rotary_dims: int | None = None,
                 layout: str = "half"):
        if layout not in ("half", "interleaved"):
            raise ValueError(f"rope: layout {layout!r} is not supported (supported: 'half', 'interleaved')")
        self.runtime, self.head_dim, self.theta, self.scaling = runtime, head_dim, float(theta), scaling
        self.interleaved = layout == "interleaved"
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
