"""Two mixers side by side in one layer: both read the same normed rows, and their outputs join the stream as
left_scale * left + right_scale * right.  Either side is any registered mixer that can hand back its output as
float32 rows; what each keeps in the cache (keys and values, a state) lives under the layer's one cache entry."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Mixer, Runtime, SeveralNeeds, StepContext
from .registry import make_part, register_part
from .spec import PartSpec


@register_part("mixer", "side_by_side")
class SideBySide(Mixer):
    """Two mixers that read the same rows; their outputs join the stream as left_scale * left + right_scale * right.
    Each keeps what it needs in the cache under the one cache entry of the layer (`SeveralNeeds`: the views come as a
    pair).  Both hand back their branches as float32 rows; with `returns_sum` the block takes (branches, scales) and
    adds them in the kernel that makes its next norm's rows."""
    returns_branch = True

    def __init__(self, runtime: Runtime, left: PartSpec, right: PartSpec, left_scale: float = 1.0, right_scale: float = 1.0,
                 left_prefix: str = "left.", right_prefix: str = "right."):
        self.runtime = runtime
        self.left, self.right = make_part("mixer", left, runtime), make_part("mixer", right, runtime)
        for side in (self.left, self.right):
            if not getattr(side, "returns_branch", False):
                raise ValueError(f"side_by_side: the mixer {type(side).__name__} cannot hand back its output")
        self.scales = (float(left_scale), float(right_scale))
        self.prefixes = (left_prefix, right_prefix)

    def sides(self):
        return (self.left, self.right)

    @property
    def graph_safe(self):
        return all(s.graph_safe for s in self.sides())

    @property
    def kernel_libraries(self):
        return tuple(lib for s in self.sides() for lib in getattr(s, "kernel_libraries", ()))

    def cache_need(self):
        return SeveralNeeds(tuple(s.cache_need() for s in self.sides()))

    def step_needs(self):
        out = {}
        for s in self.sides():
            out.update(s.step_needs())
        return out

    def weights(self):
        return {p + name: spec for p, s in zip(self.prefixes, self.sides()) for name, spec in s.weights().items()}

    def load(self, tensors):
        for p, s in zip(self.prefixes, self.sides()):
            s.load({name: tensors[p + name] for name in s.weights()})

    def branches(self, h, ctx: StepContext, cache_view, writes_cache: bool = True):
        """((left rows, left scale), (right rows, right scale)): float32 [T, D] each, not yet added."""
        return tuple((s.forward(h, ctx, view, None, writes_cache), m)
                     for s, view, m in zip(self.sides(), cache_view, self.scales))

    def forward(self, h, ctx: StepContext, cache_view, residual, writes_cache: bool = True):
        pairs = self.branches(h, ctx, cache_view, writes_cache)
        if residual is None:
            (a, ma), (b, mb) = pairs
            out = torch.zeros_like(a)
            ops.add_scaled(out, a, ma)
            return ops.add_scaled(out, b, mb)
        for y, m in pairs:
            ops.add_scaled(residual, y, m)
        return None
