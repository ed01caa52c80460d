"""Short causal convolution over time on each channel of what a mixer reads:

    out_t = h_t + sum_j w[:, j] * h_(t - taps + 1 + j)        (j = 0 .. taps - 1; rows before a sequence's start are zero)

The weight is stored [channels, taps], without bias.  The last taps - 1 rows that a sequence has brought are part
of its state (`state_need`): a step's first rows read them, and the step's own last rows replace them.  Sums in
32-bit; the rows keep their dtype."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.spec import WeightSpec
from .base import Part, Runtime, StateNeed, StepContext
from .registry import register_part


@register_part("conv", "causal_conv")
class CausalConv(Part):
    graph_safe = True

    def __init__(self, runtime: Runtime, channels: int, taps: int, name: str, add_input: bool = True):
        """add_input False: the convolution alone, without the row itself added."""
        if taps < 1:
            raise ValueError(f"causal_conv: {taps} taps")
        self.runtime, self.channels, self.taps, self.name, self.add_input = runtime, channels, int(taps), name, bool(add_input)
        self.w: torch.Tensor | None = None
        self.w_by_taps: torch.Tensor | None = None       # [taps, channels]: the layout the kernel of 16-byte pieces reads

    def weights(self):
        return {self.name: WeightSpec((self.channels, self.taps))}

    def load(self, tensors):
        self.w = tensors[self.name].to(torch.float32).contiguous()
        self.w_by_taps = self.w.t().contiguous()

    def state_need(self):
        return StateNeed((self.taps - 1, self.channels), torch.float32) if self.taps > 1 else None

    def forward(self, h: torch.Tensor, ctx: StepContext, state) -> torch.Tensor:
        return ops.causal_conv(h, self.w, state, ctx.tok_seq, ctx.slots, ctx.cu_rows, ctx.B, self.add_input, w_by_taps=self.w_by_taps)
