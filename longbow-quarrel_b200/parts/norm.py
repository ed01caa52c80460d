"""RMS norm: y = x / sqrt(mean(x^2) + eps) * gain, computed in 32-bit
(internal/device/kernels.metal:905-942 rmsnorm_f32_to_f16_v4; the gains are
promoted to 32-bit at load, internal/engine/engine.go:788-792)."""
from __future__ import annotations

import torch

from ..kernels import linear, ops
from ..weights.spec import WeightSpec
from .base import Norm, Runtime
from .registry import register_part


@register_part("norm", "rms_norm")
class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, runtime: Runtime, size: int, eps: float, name: str = "weight", offset: float = 0.0,
                 scalar: bool = False):
        """offset: what is added to the stored tensor to give the gain (1 for checkpoints that keep their
        gains minus one: y = x / rms(x) * (1 + w)); the sum is made once, in 32-bit, when the tensor is loaded.
        scalar: the stored gain is one number (a tensor without dimensions) that serves every coordinate."""
        self.runtime, self.size, self.eps, self.name, self.offset = runtime, size, float(eps), name, float(offset)
        self.scalar = bool(scalar)
        self.gain: torch.Tensor | None = None

    def weights(self):
        shape = () if self.scalar else (self.size,)
        return {self.name: WeightSpec(shape, init="gain" if self.offset == 0.0 else "small", full_precision=True)}

    def load(self, tensors):
        gain = tensors[self.name].to(torch.float32) + self.offset
        # One number for all coordinates is kept as a row of equal gains: every kernel that reads gains takes it as it is.
        self.gain = (gain.reshape(1).expand(self.size) if self.scalar else gain).contiguous()

    def forward(self, x, rows=None):
        return ops.rmsnorm(x, self.gain, self.eps, self.runtime.act_dtype, rows)

    def foldable(self, n_rows):
        if self.gain is None or not linear.can_defer_norm(n_rows, self.size, self.runtime.act_dtype):
            return None
        return self.gain, self.eps


@register_part("norm", "layer_norm")
class LayerNorm(Norm):
    """y = (x - mean(x)) / sqrt(var(x) + eps) * gain + bias, var the mean of the squared deviations, in 32-bit.  The
    bias tensor is named `bias_name` (default: the gain's name with ".b" behind it)."""
    graph_safe = True

    def __init__(self, runtime: Runtime, size: int, eps: float, name: str = "weight", bias_name: str | None = None):
        self.runtime, self.size, self.eps, self.name = runtime, size, float(eps), name
        self.bias_name = bias_name if bias_name is not None else name + ".b"
        self.gain: torch.Tensor | None = None
        self.bias: torch.Tensor | None = None

    def weights(self):
        return {self.name: WeightSpec((self.size,), init="gain", full_precision=True),
                self.bias_name: WeightSpec((self.size,), init="small", full_precision=True)}

    def load(self, tensors):
        self.gain = tensors[self.name].to(torch.float32).contiguous()
        self.bias = tensors[self.bias_name].to(torch.float32).contiguous()

    def forward(self, x, rows=None, add=()):
        """add: ((y, m), ...) branches that join the stream (x += m * y, in place) in the same pass."""
        return ops.layernorm(x, self.gain, self.bias, self.eps, self.runtime.act_dtype, rows, add=add)

    takes_branches = True       # forward(add=...) adds a mixer's branches as it norms
