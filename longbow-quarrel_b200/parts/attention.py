"""Grouped-query causal attention over the cache.

Order of work as in the reference's block (internal/device/metal.go:1377-1435):
q, k, v projections without bias; position encoding on q and k; k and v stored in
the cache at the token's position; for each query head h the keys of kv head
h // (H / Hkv) from `start` to the token's own position, scores q.k * scale,
softmax, weighted sum of v (internal/device/kernels.metal:657-766); output
projection added to the residual stream.  `window` w restricts the keys to the
last w positions (start = p - w + 1, internal/device/kernels.metal:676).

The three projections are one matrix product over the concatenated weight
[(H + 2 Hkv) hd, D]; rotation and cache write are one kernel.

Options that other designs use, each off by default: `bias` (q, k and v projections
with a bias each); `value_dim` (values of another size than queries and keys); a
position part that rotates only the first dimensions of a head; `sink` (a learned
number per head whose exponential is one more term of the softmax denominator, with
no key and no value: p_j = exp(s_j) / (exp(sink) + sum exp(s_j'))); `gate` ("sigmoid":
the heads' outputs times sigmoid(W_g h) before the output projection); and
`own_kv=False` (the layer has no keys and values: it reads the cache entry that
another layer writes, with its own queries); `softcap` c (score <- c tanh(score / c) after the
scale); `keep_first` n (with a window, the first n positions of a sequence stay visible, at their own
positions, when the window has moved past them); `value_norm_eps` (each value head is divided by its
root mean square, sqrt(mean(v^2) + eps), before it is cached); a position part with interleaved pairs
(the rows of the query and key projections are reordered at load, `parts.rope.pair_order`); and
`cache_window` / `cache_keep_first`, what the cache entry keeps when layers that read it see further
than the layer that writes it (default: the layer's own window and kept positions); `sink="one"` (the
denominator's one more term is exp(0) = 1 for every head, no tensor); `gate="sigmoid_head"` (one gate per
head, W_g of H rows: every value of a head times sigmoid of the head's number); `qk_norm` "head" (q and k each
divided by its root mean square per head, sqrt(mean(x^2) + norm_eps), no weight) or "all" (one norm over the whole
query projection and one over the whole key projection, each with a weight of that size), in 32-bit on the
products' 32-bit sums, ahead of the rotation; `q_temp` (coef, every): the queries times
1 + coef ln(floor((p + 1) / every) + 1) at position p; `chunk` n (instead of a window): position i sees j <= i
only in its own block of n positions, floor(i / n) = floor(j / n), and the cache gives back the pages below it.
"""
from __future__ import annotations

import torch

from ..kernels import attention as attention_kernels
from ..kernels import linear, ops
from ..weights.spec import WeightSpec
from .base import KVNeed, Mixer, Runtime, StepContext
from .registry import make_part, register_part
from .rope import pair_order
from .spec import PartSpec

DEFAULT_NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight"}


@register_part("mixer", "attention")
class Attention(Mixer):
    graph_safe = True
    folds_norm = True
    returns_branch = True

    @property
    def kernel_libraries(self):
        """The tensor-core attention kernels, built with the model's other libraries before its first step."""
        return ("attn_decode", "attn_prefill", "attn_prefill_tc") if self.runtime.dtype == torch.bfloat16 else ()

    def __init__(self, runtime: Runtime, hidden_size: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 scale: float, position: PartSpec | None = None, window: int | None = None,
                 own_kv: bool = True, names: dict | None = None, value_dim: int | None = None, bias: bool = False,
                 sink: bool = False, gate: str | None = None, softcap: float | None = None, keep_first: int = 0,
                 value_norm_eps: float | None = None, cache_window: int | None | str = "own",
                 cache_keep_first: int | None = None, qk_norm: str | None = None, norm_eps: float = 0.0,
                 q_temp: tuple | None = None, chunk: int | None = None):
        if n_heads % n_kv_heads:
            raise ValueError(f"attention: {n_heads} heads are not a multiple of {n_kv_heads} kv heads")
        if (head_dim % 2 and position is not None) or not 1 <= head_dim <= 256:
            # Pairs of the rotation need an even size; the plain kernels hold a head in 256 threads' registers.
            # Which of the faster kernels take a head size is each kernel's own rule (kernels/attention.py).
            raise ValueError(f"attention: head_dim {head_dim} must be at most 256, and even where it is rotated")
        self.runtime = runtime
        self.D, self.H, self.Hkv, self.hd = hidden_size, n_heads, n_kv_heads, head_dim
        self.scale, self.window, self.own_kv = float(scale), window, own_kv
        self.vd = head_dim if value_dim is None else int(value_dim)
        if not 1 <= self.vd <= 256:
            raise ValueError(f"attention: value_dim {self.vd} must be at most 256")
        if gate not in (None, "sigmoid", "sigmoid_head"):
            raise ValueError(f"attention: gate {gate!r} is not supported (supported: 'sigmoid', 'sigmoid_head')")
        if qk_norm not in (None, "head", "all"):
            raise ValueError(f"attention: qk_norm {qk_norm!r} is not supported (supported: 'head', 'all')")
        if chunk is not None and (window is not None or int(chunk) < 1):
            raise ValueError("attention: blocks of positions (chunk >= 1) or a window, not both")
        if q_temp is not None and not int(q_temp[1]) > 0:
            raise ValueError("attention: q_temp is (coef, every) with every >= 1")
        self.bias, self.sink, self.gate = bool(bias), bool(sink), gate
        self.sink_learned = self.sink and sink != "one"
        self.gate_per_head = gate == "sigmoid_head"
        self.qk_norm, self.norm_eps = qk_norm, float(norm_eps)
        self.q_temp = (float(q_temp[0]), int(q_temp[1])) if q_temp is not None else None
        self.chunk = int(chunk) if chunk is not None else None
        self.norm_w = None
        self.softcap = float(softcap) if softcap else None
        self.keep_first = int(keep_first or 0) if window is not None else 0
        self.value_norm_eps = None if value_norm_eps is None else float(value_norm_eps)
        self.cache_window = window if cache_window == "own" else cache_window
        self.cache_keep_first = self.keep_first if cache_keep_first is None else int(cache_keep_first)
        if self.cache_window is not None and (window is None or window > self.cache_window or self.keep_first > self.cache_keep_first):
            raise ValueError("attention: the cache entry must keep at least what the layer itself sees")
        self.names = {**DEFAULT_NAMES, **(names or {})}
        for key in ("q", "k", "v"):
            self.names.setdefault(key + "_bias", self.names[key].replace(".weight", "") + ".bias")
        self.names.setdefault("sink", "sinks")
        self.names.setdefault("g", "g_proj.weight")
        self.names.setdefault("q_norm", "q_norm.weight")
        self.names.setdefault("k_norm", "k_norm.weight")
        self.position = make_part("position", position, runtime) if position is not None else None
        self.rot = getattr(self.position, "rotary_dims", head_dim) if self.position is not None else 0
        # The kernels that fuse rotation and cache write into the projections, and the tensor-core attention
        # kernels, know the plain form only; every option above takes the general kernels.
        self.general = self.bias or self.sink or self.gate is not None or self.vd != head_dim or \
            (self.position is not None and self.rot != head_dim) or self.softcap is not None or self.keep_first > 0 or \
            self.value_norm_eps is not None or self.qk_norm is not None or self.q_temp is not None or self.chunk is not None
        self.b_qkv = self.sinks = None
        self.w_qkv: linear.LinearWeight | None = None
        self.w_o: linear.LinearWeight | None = None

    def cache_need(self):
        return KVNeed(self.Hkv, self.hd, self.cache_window, self.vd if self.vd != self.hd else None,
                      keep_first=self.cache_keep_first if self.cache_window is not None else 0, chunk=self.chunk)

    def step_needs(self):
        return attention_kernels.step_needs(self.runtime.act_dtype, self.hd, self.H, self.Hkv, self.window,
                                            self.runtime.device, keep_first=self.keep_first, chunk=self.chunk)

    def weights(self):
        n = self.names
        out = {n["q"]: WeightSpec((self.H * self.hd, self.D)), n["o"]: WeightSpec((self.D, self.H * self.vd))}
        if self.own_kv:
            out[n["k"]] = WeightSpec((self.Hkv * self.hd, self.D))
            out[n["v"]] = WeightSpec((self.Hkv * self.vd, self.D))
        if self.bias:
            out[n["q_bias"]] = WeightSpec((self.H * self.hd,), init="small", full_precision=True)
            if self.own_kv:
                out[n["k_bias"]] = WeightSpec((self.Hkv * self.hd,), init="small", full_precision=True)
                out[n["v_bias"]] = WeightSpec((self.Hkv * self.vd,), init="small", full_precision=True)
        if self.sink_learned:
            out[n["sink"]] = WeightSpec((self.H,), init=("uniform", 0.0, 4.0), full_precision=True)
        if self.gate is not None:
            out[n["g"]] = WeightSpec((self.H if self.gate_per_head else self.H * self.vd, self.D))
        if self.qk_norm == "all":
            out[n["q_norm"]] = WeightSpec((self.H * self.hd,), init="gain", full_precision=True)
            if self.own_kv:
                out[n["k_norm"]] = WeightSpec((self.Hkv * self.hd,), init="gain", full_precision=True)
        if self.position is not None:
            out.update(self.position.weights())        # a position encoding may have tensors of its own
        return out

    def _reordered(self, w: torch.Tensor, heads: int) -> torch.Tensor:
        """Rows (or entries) of a query or key projection in the order in which the kernels' half-split pairs are
        the position part's interleaved ones."""
        if not getattr(self.position, "interleaved", False):
            return w
        order = torch.tensor(pair_order(self.hd, self.rot), device=w.device)
        return w.reshape(heads, self.hd, *w.shape[1:])[:, order].reshape(w.shape).contiguous()

    def load(self, tensors):
        n = self.names
        tensors = dict(tensors)
        for key, heads in (("q", self.H), ("k", self.Hkv)):
            for name in (n[key], n[key + "_bias"], n[key + "_norm"]):
                if name in tensors and (key == "q" or self.own_kv):
                    tensors[name] = self._reordered(tensors[name], heads)
        rows = [tensors[n["q"]]] + ([tensors[n["k"]], tensors[n["v"]]] if self.own_kv else [])
        if self.gate is not None:
            rows.append(tensors[n["g"]])               # the gate's rows ride in the same product, after q, k and v
        if len({r.dtype for r in rows}) > 1:
            rows = [r.to(torch.float32) for r in rows]
        self.w_qkv = linear.LinearWeight(torch.cat(rows, dim=0))
        if self.bias:
            keys = ["q_bias"] + (["k_bias", "v_bias"] if self.own_kv else [])
            self.b_qkv = torch.cat([tensors[n[k]].to(torch.float32) for k in keys]).contiguous()
        if self.sink:
            self.sinks = tensors[n["sink"]].to(torch.float32).contiguous() if self.sink_learned else \
                torch.zeros(self.H, dtype=torch.float32, device=self.runtime.device)
        if self.qk_norm == "all":
            keys = ["q_norm"] + (["k_norm"] if self.own_kv else [])
            self.norm_w = torch.cat([tensors[n[k]].to(torch.float32) for k in keys]).contiguous()
        self.w_o = linear.LinearWeight(tensors[n["o"]])
        if self.position is not None and self.position.weights():
            self.position.load({name: tensors[name] for name in self.position.weights()})

    def _forward_general(self, h, ctx: StepContext, cache_view, residual, store: bool):
        """The layer with any of its options: one product for q, k, v and the gate; biases, rotation of
        the rotated dimensions and the cache write in one kernel; attention with the sink in the
        denominator and the gate on the way out; the output projection."""
        H, G, hd, vd = self.H, self.Hkv, self.hd, self.vd
        act = self.runtime.act_dtype
        # With biases (or norms of q and k) the product hands on its 32-bit sums: bias, norm and rotation meet them
        # before anything is rounded, as if they were done inside the product.
        wide = (self.bias or self.qk_norm is not None) and act != torch.float32
        rows = linear.linear(h, self.w_qkv, torch.float32 if wide else act)
        q = torch.empty((rows.shape[0], H * hd), dtype=act, device=rows.device) if wide else rows
        tables = self.position.tables() if self.position is not None else None
        if self.position is not None and tables is None:
            raise ValueError("attention: a position part without tables cannot be combined with the layer's options")
        cos, sin = tables if tables is not None else (None, None)
        v_off = (H + G) * hd
        ops.rope_partial(rows, self.b_qkv, cos, sin, self.rot if tables is not None else 0, ctx.tok_pos, ctx.tok_seq,
                         ctx.slots, cache_view.page_table if store else None, cache_view.k_pages if store else None,
                         cache_view.v_pages if store else None, H + (G if self.own_kv else 0), H, G, hd, vd, v_off,
                         cache_view.page_size, qout=q if wide else None, v_unit_eps=self.value_norm_eps,
                         unit_norm=self.qk_norm, norm_weight=self.norm_w, norm_eps=self.norm_eps, q_temp=self.q_temp)
        g_off = H * hd + (G * (hd + vd) if self.own_kv else 0)
        gate = rows[:, g_off:g_off + (H if self.gate_per_head else H * vd)] if self.gate is not None else None
        out = attention_kernels.attention(q, cache_view, ctx, H, G, hd, self.scale, self.window,
                                          next_w=self.w_o.tensor, vd=vd, sink=self.sinks, gate=gate, softcap=self.softcap,
                                          keep_first=self.keep_first, chunk=self.chunk, gate_per_head=self.gate_per_head)
        return self._project(out, residual, None)

    def forward(self, h, ctx: StepContext, cache_view, residual, writes_cache: bool = True, emit=None):
        store = self.own_kv and writes_cache
        if self.own_kv and not store:
            raise ValueError("attention: a layer with its own k and v must write its cache entry")
        if self.general:
            return self._forward_general(h, ctx, cache_view, residual, store)
        tables = self.position.tables() if self.position is not None else None
        fused = (store and h.dtype == torch.bfloat16 and self.w_qkv.tensor.dtype == torch.bfloat16 and self.D % 8 == 0
                 and self.hd % 16 == 0 and cache_view.k_pages.dtype == torch.bfloat16 and (self.position is None or tables is not None))
        few = h.shape[0] <= 16 and ops.streams_through_registers(h.shape[0], self.w_qkv.N)
        if fused and (few or (self.hd in (64, 128) and not isinstance(h, ops.NormedRows))):
            # Projection, rotation and cache write are one kernel (for few tokens the one that streams the
            # weights through registers, else the tcgen05 one).
            cos, sin = tables if tables is not None else (None, None)
            linear.note(self.w_qkv)
            qkv_kernel = ops.gemm_skinny_qkv if few else ops.gemm_tc_qkv
            q = qkv_kernel(h, self.w_qkv.tensor, cos, sin, ctx.tok_pos, ctx.tok_seq, ctx.slots,
                           cache_view.page_table, cache_view.k_pages, cache_view.v_pages, self.H, self.Hkv,
                           self.hd, cache_view.page_size)
            out = attention_kernels.attention(q, cache_view, ctx, self.H, self.Hkv, self.hd, self.scale, self.window,
                                              next_w=self.w_o.tensor)
            return self._project(out, residual, emit)
        qkv = linear.linear(h, self.w_qkv, self.runtime.act_dtype)
        if self.position is not None and tables is None:
            q = qkv[:, :self.H * self.hd].unflatten(1, (self.H, self.hd))
            k = qkv[:, self.H * self.hd:(self.H + self.Hkv) * self.hd].unflatten(1, (self.Hkv, self.hd)) \
                if self.own_kv else None
            self.position.apply(q, k, ctx.tok_pos)
        cos, sin = tables if tables is not None else (None, None)
        if not self.own_kv:
            ops.rope_kv_write(qkv, cos, sin, ctx.tok_pos, ctx.tok_seq, ctx.slots, None, None, None,
                              self.H, self.Hkv, self.hd, cache_view.page_size)
        else:
            if not store:
                raise ValueError("attention: a layer with its own k and v must write its cache entry")
            ops.rope_kv_write(qkv, cos, sin, ctx.tok_pos, ctx.tok_seq, ctx.slots, cache_view.page_table,
                              cache_view.k_pages, cache_view.v_pages, self.H, self.Hkv, self.hd, cache_view.page_size)
        out = attention_kernels.attention(qkv, cache_view, ctx, self.H, self.Hkv, self.hd, self.scale, self.window,
                                          next_w=self.w_o.tensor)
        return self._project(out, residual, emit)

    def _project(self, out, residual, emit):
        """Output projection added into the residual; with `emit`, the next norm's rows (or None).  Without a
        residual the projection itself comes back, as float32 (a block that norms the branch before adding it)."""
        if residual is None:
            return linear.linear(out, self.w_o, torch.float32)
        if emit is None:
            linear.linear(out, self.w_o, self.runtime.act_dtype, residual=residual)
            return None
        return linear.linear(out, self.w_o, self.runtime.act_dtype, residual=residual, emit=emit)[1]
