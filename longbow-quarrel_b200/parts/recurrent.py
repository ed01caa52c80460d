"""Mixers that keep a matrix of fixed size per head and sequence instead of keys and values.

Both carry S (key size x value size, float32) from token to token in the cache's
fixed-size state of the sequence's slot, which is zero when a sequence starts:

    S_t = a_t S_(t-1) + b_t k_t v_t^T        o_t = S_t^T q_t

"retention"  a_t = the head's fixed decay, b_t = 1; q and k rotated by position (optional),
             k scaled by dim^-1/2 after the rotation; no softmax and no denominator.
             Output: each head over its root mean square, times silu(W_g h), then W_o.
"mlstm"      exponential input gate and sigmoid forget gate, both from the layer's input
             through a soft cap c tanh(. / c), stabilised by a running maximum m (m_0 = 0):
             i = cap(W_i h + b_i), f = logsigmoid(cap(W_f h + b_f)), m_t = max(f + m_(t-1), i),
             a_t = exp(f + m_(t-1) - m_t), b_t = exp(i - m_t); a normaliser n_t follows the
             same recurrence with k alone; q scaled by dim^-1/2;
             o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6).
             Output: each head over its root mean square, times a weight, times sigmoid(W_g h),
             then W_o.

"lightning"  a_t = the head's fixed decay, b_t = 1; q, k and v each pass through silu; no rotation and no
             scale.  Output: all heads together over their root mean square, times a weight, times
             sigmoid(W_g h), then W_o.

"channel_decay"  a_t is a vector over the key channels, S_t = diag(a_t) S_(t-1) + k_t v_t^T (the rows of S that belong
             to a key channel decay by that channel's a_t), a_t = sigmoid(W_a2 (W_a1 h) + b)^(1/tau) through two small
             32-bit products and the logarithm of the sigmoid; q scaled by dim^-1/2, b_t = 1.  Output: each head over
             its root mean square, times a weight of the head's size that all heads share, times silu(W_g h), then W_o.

Gates, decays, the state and the per-head norms are 32-bit in both precisions; the
gates' pre-activations come from a 32-bit product of their own.  A sequence's tokens
are walked in order from the state in its slot (`csrc/recurrent.cu`: one kernel for
prompts and portions, one for steps of a single token per sequence), so a position's
result does not depend on how its prompt was cut, beyond rounding.
"""
from __future__ import annotations

import torch

from ..kernels import linear, ops
from ..weights.spec import WeightSpec
from .base import Mixer, Runtime, StateNeed, StepContext
from .registry import make_part, register_part
from .spec import PartSpec


class _MatrixStateMixer(Mixer):
    graph_safe = True
    returns_branch = True
    kernel_libraries = ("recurrent",)

    def __init__(self, runtime: Runtime, hidden_size: int, n_heads: int, key_dim: int, value_dim: int, eps: float,
                 names: dict | None = None):
        if key_dim > 256:
            raise ValueError(f"{type(self).__name__}: key size {key_dim} exceeds 256")
        self.runtime, self.D, self.H, self.dk, self.dv, self.eps = runtime, hidden_size, n_heads, key_dim, value_dim, float(eps)
        self.names = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", **(names or {})}
        self.w_in: linear.LinearWeight | None = None
        self.w_o: linear.LinearWeight | None = None

    def _base_weights(self):
        n, H, dk, dv, D = self.names, self.H, self.dk, self.dv, self.D
        return {n["q"]: WeightSpec((H * dk, D)), n["k"]: WeightSpec((H * dk, D)), n["v"]: WeightSpec((H * dv, D)),
                n["g"]: WeightSpec((H * dv, D)), n["o"]: WeightSpec((D, H * dv))}

    def _load_base(self, tensors):
        n = self.names
        rows = [tensors[n[k]] for k in ("q", "k", "v", "g")]
        if len({r.dtype for r in rows}) > 1:
            rows = [r.to(torch.float32) for r in rows]
        self.w_in = linear.LinearWeight(torch.cat(rows, dim=0))       # q, k, v and the gate in one product
        self.w_o = linear.LinearWeight(tensors[n["o"]])

    def _finish(self, out, residual):
        if residual is None:
            return linear.linear(out, self.w_o, torch.float32)
        linear.linear(out, self.w_o, self.runtime.act_dtype, residual=residual)
        return None


@register_part("mixer", "retention")
class Retention(_MatrixStateMixer):
    def __init__(self, runtime: Runtime, hidden_size: int, n_heads: int, key_dim: int, value_dim: int, decay, eps: float,
                 position: PartSpec | None = None, names: dict | None = None):
        super().__init__(runtime, hidden_size, n_heads, key_dim, value_dim, eps, names)
        if len(decay) != n_heads:
            raise ValueError(f"retention: {len(decay)} decays for {n_heads} heads")
        self.decay_values = tuple(float(d) for d in decay)
        self.decay = None
        self.position = make_part("position", position, runtime) if position is not None else None

    def cache_need(self):
        return StateNeed((self.H, self.dk, self.dv), torch.float32)

    def weights(self):
        return self._base_weights()

    def load(self, tensors):
        self._load_base(tensors)
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=self.runtime.device)

    def forward(self, h, ctx: StepContext, cache_view, residual, writes_cache: bool = True):
        H, dk, dv = self.H, self.dk, self.dv
        rows = linear.linear(h, self.w_in, self.runtime.act_dtype)
        rot = None
        if self.position is not None:
            cos, sin = self.position.tables()
            rot = (cos, sin, self.position.rotary_dims)
        raw, _ = ops.linear_scan(rows, 0, H * dk, 2 * H * dk, cache_view, ctx.cu_rows, ctx.slots, ctx.tok_pos, ctx.B,
                                 H, dk, dv, k_scale=dk ** -0.5, decay=self.decay, rot=rot, single=ctx.decode)
        g_off = 2 * H * dk + H * dv
        out = ops.head_norm_gate(raw, dv, self.eps, self.runtime.act_dtype, gate=rows[:, g_off:g_off + H * dv], act="silu")
        return self._finish(out, residual)


@register_part("mixer", "lightning")
class Lightning(_MatrixStateMixer):
    def __init__(self, runtime: Runtime, hidden_size: int, n_heads: int, key_dim: int, value_dim: int, decay, eps: float,
                 names: dict | None = None):
        super().__init__(runtime, hidden_size, n_heads, key_dim, value_dim, eps, {"norm": "norm", **(names or {})})
        if len(decay) != n_heads:
            raise ValueError(f"lightning: {len(decay)} decays for {n_heads} heads")
        self.decay_values = tuple(float(d) for d in decay)
        self.decay = self.norm_weight = None

    def cache_need(self):
        return StateNeed((self.H, self.dk, self.dv), torch.float32)

    def weights(self):
        return {**self._base_weights(), self.names["norm"]: WeightSpec((self.H * self.dv,), init="gain", full_precision=True)}

    def load(self, tensors):
        self._load_base(tensors)
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=self.runtime.device)
        self.norm_weight = tensors[self.names["norm"]].to(torch.float32).contiguous()

    def forward(self, h, ctx: StepContext, cache_view, residual, writes_cache: bool = True):
        H, dk, dv = self.H, self.dk, self.dv
        rows = linear.linear(h, self.w_in, self.runtime.act_dtype)
        # silu meets q, k and v in 32-bit as the scan reads them: nothing that enters the recurrence is rounded again.
        raw, _ = ops.linear_scan(rows, 0, H * dk, 2 * H * dk, cache_view, ctx.cu_rows, ctx.slots, ctx.tok_pos, ctx.B,
                                 H, dk, dv, decay=self.decay, single=ctx.decode, in_act="silu")
        g_off = 2 * H * dk + H * dv
        # One norm over all heads: the heads' outputs as a single "head" of H * dv numbers.
        out = ops.head_norm_gate(raw.view(raw.shape[0], 1, H * dv), H * dv, self.eps, self.runtime.act_dtype,
                                 weight=self.norm_weight, gate=rows[:, g_off:g_off + H * dv], act="sigmoid")
        return self._finish(out, residual)


@register_part("mixer", "mlstm")
class MLSTM(_MatrixStateMixer):
    def __init__(self, runtime: Runtime, hidden_size: int, n_heads: int, key_dim: int, value_dim: int, gate_cap: float,
                 eps: float, names: dict | None = None):
        super().__init__(runtime, hidden_size, n_heads, key_dim, value_dim, eps,
                         {"norm": "norm", "i": "i", "i_bias": "i.b", "f": "f", "f_bias": "f.b", **(names or {})})
        self.cap = float(gate_cap)
        self.w_gates = self.b_gates = self.head_weight = None

    def cache_need(self):
        # One more row for the running maximum and one more column for the normaliser.
        return StateNeed((self.H, self.dk + 1, self.dv + 1), torch.float32)

    def weights(self):
        n, H = self.names, self.H
        return {**self._base_weights(),
                n["norm"]: WeightSpec((H * self.dv,), init="gain", full_precision=True),
                n["i"]: WeightSpec((H, self.D)), n["f"]: WeightSpec((H, self.D)),
                n["i_bias"]: WeightSpec((H,), init="small", full_precision=True),
                n["f_bias"]: WeightSpec((H,), init=("uniform", 1.0, 6.0), full_precision=True)}

    def load(self, tensors):
        self._load_base(tensors)
        n = self.names
        self.w_gates = torch.cat([tensors[n["i"]], tensors[n["f"]]], dim=0).contiguous()
        self.b_gates = torch.cat([tensors[n["i_bias"]], tensors[n["f_bias"]]]).to(torch.float32).contiguous()
        self.head_weight = tensors[n["norm"]].to(torch.float32).contiguous()

    def forward(self, h, ctx: StepContext, cache_view, residual, writes_cache: bool = True):
        H, dk, dv = self.H, self.dk, self.dv
        rows = linear.linear(h, self.w_in, self.runtime.act_dtype)
        pre = ops.small_proj(h, self.w_gates)         # the gates enter the recurrence: a 32-bit product of their own
        raw, enm = ops.linear_scan(rows, 0, H * dk, 2 * H * dk, cache_view, ctx.cu_rows, ctx.slots, ctx.tok_pos, ctx.B,
                                   H, dk, dv, q_scale=dk ** -0.5, gates=(pre, self.b_gates, self.cap), single=ctx.decode)
        g_off = 2 * H * dk + H * dv
        out = ops.head_norm_gate(raw, dv, self.eps, self.runtime.act_dtype, exp_neg_m=enm, weight=self.head_weight,
                                 gate=rows[:, g_off:g_off + H * dv], act="sigmoid")
        return self._finish(out, residual)


@register_part("mixer", "channel_decay")
class ChannelDecay(_MatrixStateMixer):
    def __init__(self, runtime: Runtime, hidden_size: int, n_heads: int, key_dim: int, value_dim: int, tau: float,
                 eps: float, rank: int | None = None, names: dict | None = None):
        """rank: the inner size of the decays' two products; None: whatever the stored tensors have."""
        super().__init__(runtime, hidden_size, n_heads, key_dim, value_dim, eps,
                         {"norm": "norm", "a1": "a1", "a2": "a2", "a2_bias": "a2.b", **(names or {})})
        if not tau > 0 or (rank is not None and rank < 1):
            raise ValueError(f"channel_decay: tau {tau} must be positive and the rank {rank} at least 1")
        self.tau, self.rank = float(tau), int(rank) if rank is not None else -1
        self.w_a1 = self.w_a2 = self.b_a2 = self.head_weight = None

    def cache_need(self):
        return StateNeed((self.H, self.dk, self.dv), torch.float32)

    def weights(self):
        n, H = self.names, self.H
        return {**self._base_weights(),
                n["norm"]: WeightSpec((self.dv,), init="gain", full_precision=True),
                n["a1"]: WeightSpec((self.rank, self.D)), n["a2"]: WeightSpec((H * self.dk, self.rank)),
                n["a2_bias"]: WeightSpec((H * self.dk,), init=("uniform", 0.0, 4.0), full_precision=True)}

    def load(self, tensors):
        self._load_base(tensors)
        n = self.names
        self.w_a1, self.w_a2 = linear.LinearWeight(tensors[n["a1"]]), tensors[n["a2"]].contiguous()
        if self.w_a1.N != self.w_a2.shape[1]:
            raise ValueError(f"channel_decay: {n['a1']} has {self.w_a1.N} rows, {n['a2']} {self.w_a2.shape[1]} columns")
        self.b_a2 = tensors[n["a2_bias"]].to(torch.float32).contiguous()
        self.head_weight = tensors[n["norm"]].to(torch.float32).repeat(self.H).contiguous()     # one weight for every head

    def forward(self, h, ctx: StepContext, cache_view, residual, writes_cache: bool = True):
        H, dk, dv = self.H, self.dk, self.dv
        rows = linear.linear(h, self.w_in, self.runtime.act_dtype)
        # The decays enter the recurrence: the first of their two products (over the layer's width) runs as the layer's
        # other products do and hands on its 32-bit sums unrounded; the second (over the small inner size) is a 32-bit
        # product, so that nothing between the first product's sums and the decay itself is rounded.
        pre = ops.gemm_plain(linear.linear(h, self.w_a1, torch.float32), self.w_a2, torch.float32)
        raw, _ = ops.linear_scan(rows, 0, H * dk, 2 * H * dk, cache_view, ctx.cu_rows, ctx.slots, ctx.tok_pos, ctx.B,
                                 H, dk, dv, q_scale=dk ** -0.5, channel_decay=(pre, self.b_a2, self.tau), single=ctx.decode)
        g_off = 2 * H * dk + H * dv
        out = ops.head_norm_gate(raw, dv, self.eps, self.runtime.act_dtype, weight=self.head_weight,
                                 gate=rows[:, g_off:g_off + H * dv], act="silu")
        return self._finish(out, residual)
