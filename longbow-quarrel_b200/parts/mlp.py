"""Gated feed-forward: y = (up(x) * act(gate(x))) . Wd^T, act = SiLU without clamp
(internal/device/metal.go:1464-1474; internal/device/cpu_ref.go:133-149 CPUSwiGLU).
Gate and up are one matrix product over the stacked weight [2F, D].

Options that other designs use: `activation` "gelu_tanh" or "gelu" (the erf form) instead of "silu", and
`bias` (each of the three projections with a bias: y = W_down (act(W_gate h + b_g) * (W_up h + b_u)) + b_d).
With either the activation is a kernel of its own behind the product (whose sums it reads in 32-bit where
biases are added); the fused SwiGLU epilogues serve the plain form."""
from __future__ import annotations

import torch

from ..kernels import linear, ops
from ..weights.spec import WeightSpec
from .base import FeedForward, Runtime, StepContext
from .registry import register_part

DEFAULT_NAMES = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}


@register_part("ffn", "gated_mlp")
class GatedMLP(FeedForward):
    graph_safe = True

    def __init__(self, runtime: Runtime, hidden_size: int, intermediate_size: int, activation: str = "silu",
                 names: dict | None = None, bias: bool = False):
        if activation not in ("silu", "gelu_tanh", "gelu"):
            raise ValueError(f"gated_mlp: activation {activation!r} is not supported (supported: 'silu', 'gelu_tanh', 'gelu')")
        self.runtime, self.D, self.F = runtime, hidden_size, intermediate_size
        self.activation, self.bias = activation, bool(bias)
        self.plain = activation == "silu" and not self.bias
        self.folds_norm = self.plain        # the products of the plain form can take and leave unfinished rows of a norm
        self.names = {**DEFAULT_NAMES, **(names or {})}
        for key in ("gate", "up", "down"):
            self.names.setdefault(key + "_bias", self.names[key].replace(".weight", "") + ".bias")
        self.b_gu = self.b_down = None
        self.w_gu: linear.LinearWeight | None = None
        self.block = 0
        self.w_down: linear.LinearWeight | None = None

    def weights(self):
        n = self.names
        out = {n["gate"]: WeightSpec((self.F, self.D)), n["up"]: WeightSpec((self.F, self.D)),
               n["down"]: WeightSpec((self.D, self.F))}
        if self.bias:
            out.update({n["gate_bias"]: WeightSpec((self.F,), init="small", full_precision=True),
                        n["up_bias"]: WeightSpec((self.F,), init="small", full_precision=True),
                        n["down_bias"]: WeightSpec((self.D,), init="small", full_precision=True)})
        return out

    def load(self, tensors):
        n = self.names
        gate, up = tensors[n["gate"]], tensors[n["up"]]
        if gate.dtype != up.dtype:
            gate, up = gate.to(torch.float32), up.to(torch.float32)
        # bfloat16 kernels apply SwiGLU in the product's epilogue over interleaved rows.
        self.block = linear.GATE_UP_BLOCK if (self.plain and self.runtime.dtype == torch.bfloat16 and gate.dtype == torch.bfloat16
                                              and self.F % linear.GATE_UP_BLOCK == 0) else 0
        stacked = linear.interleave_gate_up(gate, up) if self.block else torch.cat([gate, up], dim=0)
        self.w_gu = linear.LinearWeight(stacked)
        self.w_down = linear.LinearWeight(tensors[n["down"]])
        if self.bias:
            self.b_gu = torch.cat([tensors[n["gate_bias"]], tensors[n["up_bias"]]]).to(torch.float32).contiguous()
            self.b_down = tensors[n["down_bias"]].to(torch.float32).contiguous()

    def forward(self, h, ctx: StepContext, residual, emit=None):
        """With `residual` None the output comes back as float32 [T, D] instead of being added."""
        if residual is None:
            if self.plain:
                return linear.linear(linear.linear_swiglu(h, self.w_gu, self.block), self.w_down, torch.float32)
            gu = linear.linear(h, self.w_gu, torch.float32 if self.bias else self.runtime.act_dtype)
            out = linear.linear(ops.gated_act(gu, self.b_gu, self.activation, self.runtime.act_dtype), self.w_down, torch.float32)
            return ops.add_bias(out, self.b_down) if self.bias else out
        if not self.plain:
            # Biases meet the product's 32-bit sums before anything is rounded.
            gu = linear.linear(h, self.w_gu, torch.float32 if self.bias else self.runtime.act_dtype)
            act = ops.gated_act(gu, self.b_gu, self.activation, self.runtime.act_dtype)
            linear.linear(act, self.w_down, self.runtime.act_dtype, residual=residual)
            if self.bias:
                ops.add_bias(residual, self.b_down)
            return None
        act = linear.linear_swiglu(h, self.w_gu, self.block)
        if emit is None:
            linear.linear(act, self.w_down, self.runtime.act_dtype, residual=residual)
            return None
        return linear.linear(act, self.w_down, self.runtime.act_dtype, residual=residual, emit=emit)[1]
