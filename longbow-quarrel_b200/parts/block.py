"""The arrangement of parts in a layer.

"pre_norm": x += mixer(norm1(x)); x += ffn(norm2(x)) (norm2 and ffn together, or a layer of a mixer
alone), the order of the reference's
block (internal/device/metal.go:1347-1527), with the residual stream x in 32-bit
throughout (internal/engine/engine.go:1375).

Two options of "pre_norm" that other designs use: a part in the place `conv1` (role "conv": a short causal
convolution over time) filters what the mixer reads, h <- conv1(norm1(x)), with the rows it needs from earlier
steps kept as the layer's own state; and `residual_scale` m, x += m * mixer(...), x += m * ffn(...), for which
the mixer and the feed-forward hand back their branches as float32 rows.

"stream_mix": no mixer and no feed-forward; the stream is replaced by a product over the stream and the embedding's
rows side by side, x <- W [x; e] (what a pass over repeated layers starts with).

"sandwich_norm": every branch is normed on both sides, x += norm1b(mixer(norm1(x)));
x += norm2b(ffn(norm2(x))), and a layer may have no feed-forward.  The branch's own norm,
the addition and the norm that reads the stream next are one kernel."""
from __future__ import annotations

import torch

from ..kernels import linear, ops
from ..weights.spec import WeightSpec
from .base import Part, Runtime, StepContext
from .norm import RMSNorm
from .registry import make_part, register_part
from .spec import LayerSpec


@register_part("block", "pre_norm")
class PreNormBlock(Part):
    def __init__(self, runtime: Runtime, layer: LayerSpec, residual_scale: float = 1.0):
        self.prefix = layer.prefix
        unknown = set(layer.parts) - {"norm1", "conv1", "mixer", "norm2", "ffn"}
        if unknown:
            raise ValueError(f"layer {layer.prefix!r}: the arrangement 'pre_norm' has no place {sorted(unknown)}")
        if len(set(layer.parts) & {"norm2", "ffn"}) == 1:
            raise ValueError(f"layer {layer.prefix!r}: norm2 and ffn come together or not at all")
        self.norm1 = make_part("norm", layer.part("norm1"), runtime)
        self.conv1 = make_part("conv", layer.part("conv1"), runtime) if "conv1" in layer.parts else None
        self.mixer = make_part("mixer", layer.part("mixer"), runtime)
        self.has_ffn = "ffn" in layer.parts
        self.norm2 = make_part("norm", layer.part("norm2"), runtime) if self.has_ffn else None
        self.ffn = make_part("ffn", layer.part("ffn"), runtime) if self.has_ffn else None
        self.scale = float(residual_scale)
        if self.scale != 1.0 and not getattr(self.mixer, "returns_branch", False):
            raise ValueError(f"layer {layer.prefix!r}: the mixer {layer.part('mixer').kind!r} cannot hand back its output "
                             f"for a multiplier on the branch")
        # The products that fold norms add their output straight into the stream and read the norm's unfinished rows:
        # neither goes with a multiplier on the branch or with a filter between the norm and the mixer.
        self.folds_norm = self.scale == 1.0 and self.conv1 is None

    def parts(self):
        return tuple(p for p in (self.norm1, self.conv1, self.mixer, self.norm2, self.ffn) if p is not None)

    def cache_need(self):
        """What the layer's cache entry must hold: its mixer's need."""
        return self.mixer.cache_need()

    def state_need(self):
        """What every run of the layer keeps for each sequence beside its mixer's cache entry: the filter's rows."""
        return self.conv1.state_need() if self.conv1 is not None else None

    def step_needs(self):
        out = {}
        for part in self.parts():
            out.update(part.step_needs())
        return out

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self.parts())

    def weights(self):
        out = {}
        for part in self.parts():
            for name, spec in part.weights().items():
                if name in out:
                    raise ValueError(f"layer {self.prefix}: two parts name the tensor {name!r}")
                out[name] = spec
        return out

    def load(self, tensors):
        for part in self.parts():
            part.load({n: tensors[n] for n in part.weights()})

    def input_norm(self, n_rows: int):
        """(gain, eps) when the layer ahead of this one may leave this layer's first norm to the
        products on either side of it; None otherwise."""
        return self.norm1.foldable(n_rows) if self.mixer.folds_norm else None

    def _forward_plain(self, x, ctx: StepContext, cache_view, writes_cache: bool, state):
        """The layer with a filter ahead of its mixer or a multiplier on its branches: the norms are kernels of their own,
        except that the mixer's branch joins the stream in the kernel that makes the second norm's rows."""
        h = self.norm1.forward(x)
        if self.conv1 is not None:
            h = self.conv1.forward(h, ctx, state)
        h2 = None
        if self.scale == 1.0:
            self.mixer.forward(h, ctx, cache_view, x, writes_cache)
        else:
            branch = self.mixer.forward(h, ctx, cache_view, None, writes_cache)
            gain = self.norm2.gain if self.has_ffn and isinstance(self.norm2, RMSNorm) else None
            if gain is not None and gain.dtype == x.dtype == branch.dtype and x.is_contiguous() and branch.is_contiguous():
                h2 = ops.add_scaled_norm(x, branch, self.scale, gain, self.norm2.eps, self.norm2.runtime.act_dtype)
            else:
                ops.add_scaled(x, branch, self.scale)
        if self.has_ffn:
            h = h2 if h2 is not None else self.norm2.forward(x)
            if self.scale == 1.0:
                self.ffn.forward(h, ctx, x)
            elif getattr(self.ffn, "takes_scale", False):
                self.ffn.forward(h, ctx, x, scale=self.scale)          # the feed-forward's last kernel multiplies as it adds
            else:
                ops.add_scaled(x, self.ffn.forward(h, ctx, None), self.scale)
        return None

    def forward(self, x, ctx: StepContext, cache_view, writes_cache: bool = True, normed=None, emit=None, state=None):
        """`normed`: the rows of norm1, when the layer ahead made them (see input_norm).  `emit`: the
        input_norm() of the layer that follows.  `state`: the view of what `state_need` asked for.  Returns the
        next layer's rows, or None."""
        if not self.folds_norm:
            return self._forward_plain(x, ctx, cache_view, writes_cache, state)
        n_rows = x.shape[0]
        h = normed if normed is not None else self.norm1.forward(x)
        if self.has_ffn and hasattr(self.mixer, "branches") and getattr(self.norm2, "takes_branches", False):
            # A mixer of several sides: its branches join the stream in the kernel that makes the second norm's rows.
            h = self.norm2.forward(x, add=self.mixer.branches(h, ctx, cache_view, writes_cache))
            self.ffn.forward(h, ctx, x)
            return None
        if not self.has_ffn:
            if emit is not None and self.mixer.folds_norm:
                return self.mixer.forward(h, ctx, cache_view, x, writes_cache, emit=emit)
            self.mixer.forward(h, ctx, cache_view, x, writes_cache)
            return None
        fold2 = self.norm2.foldable(n_rows) if (self.mixer.folds_norm and self.ffn.folds_norm) else None
        h = self.mixer.forward(h, ctx, cache_view, x, writes_cache, emit=fold2) if fold2 is not None \
            else self.mixer.forward(h, ctx, cache_view, x, writes_cache)
        if fold2 is None or h is None:
            h = self.norm2.forward(x)
        if emit is not None and self.ffn.folds_norm:
            return self.ffn.forward(h, ctx, x, emit=emit)
        self.ffn.forward(h, ctx, x)
        return None


@register_part("block", "sandwich_norm")
class SandwichNormBlock(Part):
    """Places: norm1, mixer, norm1b, and (all three or none) norm2, ffn, norm2b.  The mixer and the
    feed-forward hand back their outputs as float32 rows (`returns_branch`) instead of adding them."""

    folds_norm = True

    def __init__(self, runtime: Runtime, layer: LayerSpec):
        self.prefix, self.runtime = layer.prefix, runtime
        places = set(layer.parts)
        unknown = places - {"norm1", "mixer", "norm1b", "norm2", "ffn", "norm2b"}
        if unknown:
            raise ValueError(f"layer {layer.prefix!r}: the arrangement 'sandwich_norm' has no place {sorted(unknown)}")
        if len(places & {"norm2", "ffn", "norm2b"}) not in (0, 3):
            raise ValueError(f"layer {layer.prefix!r}: norm2, ffn and norm2b come together or not at all")
        self.norm1 = make_part("norm", layer.part("norm1"), runtime)
        self.mixer = make_part("mixer", layer.part("mixer"), runtime)
        self.norm1b = make_part("norm", layer.part("norm1b"), runtime)
        self.has_ffn = "ffn" in places
        self.norm2 = make_part("norm", layer.part("norm2"), runtime) if self.has_ffn else None
        self.ffn = make_part("ffn", layer.part("ffn"), runtime) if self.has_ffn else None
        self.norm2b = make_part("norm", layer.part("norm2b"), runtime) if self.has_ffn else None
        if not getattr(self.mixer, "returns_branch", False):
            raise ValueError(f"layer {layer.prefix!r}: the mixer {layer.part('mixer').kind!r} cannot hand back its "
                             f"output for a norm of its own")
        for norm in self.norms():
            if not hasattr(norm, "gain") or not hasattr(norm, "eps"):
                raise ValueError(f"layer {layer.prefix!r}: the arrangement 'sandwich_norm' needs RMS norms with a gain")

    def norms(self):
        return tuple(n for n in (self.norm1, self.norm1b, self.norm2, self.norm2b) if n is not None)

    def parts(self):
        return tuple(p for p in (self.norm1, self.mixer, self.norm1b, self.norm2, self.ffn, self.norm2b) if p is not None)

    def cache_need(self):
        return self.mixer.cache_need()

    def step_needs(self):
        out = {}
        for part in self.parts():
            out.update(part.step_needs())
        return out

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self.parts())

    def weights(self):
        out = {}
        for part in self.parts():
            for name, spec in part.weights().items():
                if name in out:
                    raise ValueError(f"layer {self.prefix}: two parts name the tensor {name!r}")
                out[name] = spec
        return out

    def load(self, tensors):
        for part in self.parts():
            part.load({n: tensors[n] for n in part.weights()})

    def input_norm(self, n_rows: int):
        """(gain, eps) of norm1: the layer ahead may make its rows in the kernel that ends it."""
        return (self.norm1.gain, self.norm1.eps) if self.norm1.gain is not None else None

    def forward(self, x, ctx: StepContext, cache_view, writes_cache: bool = True, normed=None, emit=None):
        """`normed`: the rows of norm1 when the layer ahead made them; `emit`: the next layer's
        input_norm().  Returns the next layer's rows, or None."""
        act = self.runtime.act_dtype
        if isinstance(normed, ops.NormedRows):
            normed = normed.finish()
        h = normed if normed is not None else self.norm1.forward(x)
        y = self.mixer.forward(h, ctx, cache_view, None, writes_cache)
        if not self.has_ffn:
            return ops.rmsnorm_add(y, self.norm1b.gain, self.norm1b.eps, x, emit, act)
        h = ops.rmsnorm_add(y, self.norm1b.gain, self.norm1b.eps, x, (self.norm2.gain, self.norm2.eps), act)
        y = self.ffn.forward(h, ctx, None)
        return ops.rmsnorm_add(y, self.norm2b.gain, self.norm2b.eps, x, emit, act)


@register_part("block", "stream_mix")
class StreamMixBlock(Part):
    """x <- W [x; e]: W [D, 2 D], x the stream, e the embedding's output for the same rows.  The product reads both in
    the model's precision and leaves the new stream in 32-bit.  It keeps nothing in the cache."""
    graph_safe = True
    folds_norm = False
    replaces_stream = True       # forward returns the new stream instead of changing x in place
    reads_embedding = True       # forward is given the embedding's rows as `embedded`

    def __init__(self, runtime: Runtime, layer: LayerSpec, hidden_size: int, name: str = "in"):
        if layer.parts:
            raise ValueError(f"layer {layer.prefix!r}: the arrangement 'stream_mix' has no places for parts")
        self.prefix, self.runtime, self.D, self.name = layer.prefix, runtime, int(hidden_size), name
        self.w: linear.LinearWeight | None = None

    def parts(self):
        return ()

    def cache_need(self):
        return None

    def weights(self):
        return {self.name: WeightSpec((self.D, 2 * self.D))}

    def load(self, tensors):
        self.w = linear.LinearWeight(tensors[self.name])

    def forward(self, x, ctx: StepContext, embedded):
        return linear.linear(ops.side_by_side(x, embedded, self.runtime.act_dtype), self.w, torch.float32)
