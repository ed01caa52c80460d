"""Feed-forward of many small experts, of which each token uses a few.

    z = W_router h (32-bit)        s = sigmoid(z)
    experts form `groups` equal groups of neighbours; a group's score is the sum of its two largest s;
    only experts of the `keep` best groups can be chosen; of those, the `top` with the largest s are
    g_e = s_e / (sum of the chosen s + 1e-20) * route_scale
    y = sum_e g_e W_down,e act(W_up,e h)  [ + sigmoid(w_sg . h) * shared(h) ]

The experts have no gate and no bias.  A shared expert (a `dense_mlp` of its own size) runs for every
token behind one sigmoid number per token.

Options that other designs use, each a parameter: `score` "softmax" (over all router outputs) instead of "sigmoid";
`correction` (a tensor of one number per router output that is added to the scores for the choice only: groups and
experts are chosen by s + correction, the weights are the plain s); `group_rule` "max" (a group's score is its best
choice score) instead of "top2"; `normalize` False (the weights are the chosen scores as they are); `gated` (an expert
is W_down (act(W_gate h) * (W_up h)), and so is the shared expert); `identity` n (the router has n more outputs than
there are experts; a token that chooses one of those gets its own input h back, times the weight; they have no tensors,
and groups are formed over experts and identity outputs together).  The router's logits and the shared expert's gate come
from one 32-bit product; choice and weights are one kernel.  Few tokens (a decode step): the experts' two
products are one kernel each that streams every token's own experts (`csrc/moe.cu`), the second of which also
adds the shared expert's rows and joins the stream.  Many tokens (a prompt, bfloat16): the (token, choice) pairs
are sorted by expert on the device and each product is one grouped tensor-core launch: on tcgen05 for a long
prompt (`lq_gemm_tc_grouped`: every expert's rows padded to whole tiles), on mma.sync for a short one
(`csrc/grouped_gemm.cu`).
Every kernel reads the chosen experts from device memory, so a step can be captured and replayed.
"""
from __future__ import annotations

import torch

from ..kernels import linear, ops
from ..weights.spec import WeightSpec
from .base import FeedForward, Runtime, StepContext
from .registry import make_part, register_part
from .spec import PartSpec


@register_part("ffn", "routed_experts")
class RoutedExperts(FeedForward):
    graph_safe = True
    GROUPED_FROM = 256       # (token, choice) pairs from which the experts' products run as grouped tensor-core products
    TILED_FROM = 2048        # ... and from which they run on tcgen05, every expert's rows padded to whole tiles of 128

    @property
    def kernel_libraries(self):
        # `recurrent` holds the 32-bit product for weights of few rows (the router).
        return ("moe", "recurrent", "grouped_gemm") if self.runtime.dtype == torch.bfloat16 else ("moe", "recurrent")

    def __init__(self, runtime: Runtime, hidden_size: int, n_experts: int, top: int, expert_size: int,
                 activation: str = "gelu", groups: int = 1, keep_groups: int = 1, route_scale: float = 1.0,
                 shared_size: int | None = None, shared_activation: str | None = None, names: dict | None = None,
                 score: str = "sigmoid", correction: bool = False, group_rule: str = "top2", normalize: bool = True,
                 gated: bool = False, identity: int = 0):
        if activation not in ops.MOE_ACTS:
            raise ValueError(f"routed_experts: activation {activation!r} is not one of {', '.join(map(str, ops.MOE_ACTS))}")
        if score not in ops.SCORE_FNS or group_rule not in ops.GROUP_RULES:
            raise ValueError(f"routed_experts: score {score!r} / group rule {group_rule!r} (scores: {', '.join(ops.SCORE_FNS)}; "
                             f"group rules: {', '.join(ops.GROUP_RULES)})")
        routed = n_experts + int(identity)              # what the router chooses from
        if identity < 0 or routed % groups or not 1 <= keep_groups <= groups:
            raise ValueError(f"routed_experts: {n_experts} experts and {identity} identity outputs in {groups} groups, {keep_groups} kept")
        if not 1 <= top <= keep_groups * (routed // groups):
            raise ValueError(f"routed_experts: {top} experts per token, but only {keep_groups * (routed // groups)} can be chosen")
        self.runtime, self.D, self.E, self.top, self.F = runtime, hidden_size, n_experts, top, expert_size
        self.routed, self.identity = routed, int(identity)
        self.activation, self.groups, self.keep, self.route_scale = activation, groups, keep_groups, float(route_scale)
        self.score, self.has_correction, self.group_rule, self.normalize = score, bool(correction), group_rule, bool(normalize)
        self.gated = bool(gated)
        self.names = {"router": "router", "expert": "e{}", "gate": "gate", "up": "up", "down": "down", "shared": "shared",
                      "shared_gate": "shared.sg", "correction": "correction", **(names or {})}
        self.shared = None
        if shared_size:
            n = self.names
            if self.gated:
                self.shared = make_part("ffn", PartSpec("gated_mlp", {
                    "hidden_size": hidden_size, "intermediate_size": shared_size, "activation": shared_activation or activation,
                    "names": {"gate": f"{n['shared']}.{n['gate']}", "up": f"{n['shared']}.{n['up']}",
                              "down": f"{n['shared']}.{n['down']}"}}), runtime)
            else:
                self.shared = make_part("ffn", PartSpec("dense_mlp", {
                    "hidden_size": hidden_size, "intermediate_size": shared_size, "activation": shared_activation or activation,
                    "names": {"up": f"{n['shared']}.{n['up']}", "down": f"{n['shared']}.{n['down']}"}}), runtime)
        self.w_route = self.w_up = self.w_down = self.correction = None
        self.up_block = 0        # gated: how an expert's gate and up rows lie in w_up (see load)

    takes_scale = True        # forward(..., scale=m): the whole output times m as it joins the stream

    def _expert(self, e: int, which: str) -> str:
        return f"{self.names['expert'].format(e)}.{self.names[which]}"

    def weights(self):
        out = {self.names["router"]: WeightSpec((self.routed, self.D))}
        if self.has_correction:
            out[self.names["correction"]] = WeightSpec((self.routed,), init="small", full_precision=True)
        for e in range(self.E):
            if self.gated:
                out[self._expert(e, "gate")] = WeightSpec((self.F, self.D))
            out[self._expert(e, "up")] = WeightSpec((self.F, self.D))
            out[self._expert(e, "down")] = WeightSpec((self.D, self.F))
        if self.shared is not None:
            out.update(self.shared.weights())
            out[self.names["shared_gate"]] = WeightSpec((1, self.D))
        return out

    def load(self, tensors):
        rows = [tensors[self.names["router"]]] + ([tensors[self.names["shared_gate"]]] if self.shared is not None else [])
        self.w_route = torch.cat(rows, dim=0).contiguous()           # the shared expert's gate rides behind the router's rows
        if self.has_correction:
            self.correction = tensors[self.names["correction"]].to(torch.float32).contiguous()
        if self.gated:
            # One stream of [2F, D] per expert: gate and up rows by turns in blocks of 8 where the tensor-core products'
            # gated epilogue can read them (silu, F a multiple of 8), else the gate rows ahead of the up rows.
            self.up_block = linear.GATE_UP_BLOCK if self.activation == "silu" and self.F % linear.GATE_UP_BLOCK == 0 else 0
            join = linear.interleave_gate_up if self.up_block else (lambda g, u: torch.cat([g, u]))
            self.w_up = torch.stack([join(tensors[self._expert(e, "gate")], tensors[self._expert(e, "up")])
                                     for e in range(self.E)]).contiguous()
        else:
            self.w_up = torch.stack([tensors[self._expert(e, "up")] for e in range(self.E)]).contiguous()
        self.w_down = torch.stack([tensors[self._expert(e, "down")] for e in range(self.E)]).contiguous()
        if self.w_up.dtype != self.runtime.act_dtype:
            # The experts' kernels read rows and weights of one dtype.
            self.w_up, self.w_down = self.w_up.to(self.runtime.act_dtype), self.w_down.to(self.runtime.act_dtype)
        if self.shared is not None:
            self.shared.load({name: tensors[name] for name in self.shared.weights()})

    def forward(self, h, ctx: StepContext, residual, scale: float = 1.0):
        """scale: a multiplier on the whole output (the chosen experts' weights and the shared expert's gate carry it)."""
        z = ops.small_proj(h, self.w_route)                          # float32 [T, routed (+ 1)]
        ids, weights = ops.moe_route(z, self.routed, self.groups, self.keep, self.top, self.route_scale * scale, score=self.score,
                                     correction=self.correction, group_rule=self.group_rule, normalize=self.normalize)
        shared = self.shared.forward(h, ctx, None) if self.shared is not None else None
        gate = z[:, self.routed] if self.shared is not None else None
        T = h.shape[0]
        grouped = self.F % 8 == 0 and ops.grouped_gemm_takes(h, self.w_up)
        # Identity outputs have no rows in the grouped products; the combination adds their tokens' own input instead.
        more = dict(ids=ids, E=self.E, h=h) if self.identity else {}
        if grouped and T * self.top >= self.TILED_FROM:
            # A prompt: the pairs in the order of their experts, every expert padded to whole row tiles, so that each
            # tile of the tcgen05 product reads one expert's weight; the second product reads the first one's rows as
            # they lie, and the combination finds each pair's row through the order's inverse.
            src, dst, tile_group = ops.group_rows_padded(ids.view(-1), self.E)
            u = ops.gemm_tc_grouped(ops.gather_rows(h, src, self.top), self.w_up, tile_group, h.dtype,
                                    swiglu=self.gated and self.up_block > 0)     # silu(gate) * up in the product's epilogue
            if self.gated and not self.up_block:
                u = ops.gated_act(u, None, self.activation, h.dtype)     # [rows, 2F] -> act(gate columns) * up columns
            elif not self.gated and self.activation is not None:
                ops.activation(u, self.activation, out=u)
            y = ops.gemm_tc_grouped(u, self.w_down, tile_group, torch.float32)
            out = residual if residual is not None else torch.empty((T, self.D), dtype=torch.float32, device=h.device)
            ops.moe_combine(y, weights, out, accumulate=residual is not None, shared=shared, shared_gate=gate, place=dst,
                            shared_scale=scale, **more)
            return None if residual is not None else out
        if grouped and T * self.top >= self.GROUPED_FROM:
            # Many tokens: the pairs sorted by expert (on the device), each expert's rows as tiles of a tensor-core product.
            listed = ops.group_rows(ids.view(-1), self.routed)
            n_up = self.w_up.shape[1]
            u = torch.empty((T * self.top, n_up), dtype=h.dtype, device=h.device)
            ops.grouped_gemm(h, self.w_up, u, listed=listed, a_div=self.top, act=None if self.gated else self.activation)
            if self.gated:
                u = ops.swiglu(u, self.up_block) if self.up_block else ops.gated_act(u, None, self.activation, h.dtype)
            y = torch.empty((T * self.top, self.D), dtype=torch.float32, device=h.device)
            ops.grouped_gemm(u, self.w_down, y, listed=listed)
            out = residual if residual is not None else torch.empty((T, self.D), dtype=torch.float32, device=h.device)
            ops.moe_combine(y, weights, out, accumulate=residual is not None, shared=shared, shared_gate=gate,
                            shared_scale=scale, **more)
            return None if residual is not None else out
        u = ops.moe_up(h, self.w_up, ids, self.activation, gated=self.gated, block=self.up_block)
        more = dict(h=h if self.identity else None, shared_scale=scale)
        if residual is None:
            out = torch.empty((h.shape[0], self.D), dtype=torch.float32, device=h.device)
            return ops.moe_down(u, self.w_down, ids, weights, out, accumulate=False, shared=shared, shared_gate=gate, **more)
        ops.moe_down(u, self.w_down, ids, weights, residual, accumulate=True, shared=shared, shared_gate=gate, **more)
        return None
