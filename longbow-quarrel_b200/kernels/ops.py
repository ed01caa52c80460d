"""Python faces of the CUDA kernels.

Every function takes torch tensors that live on the GPU, checks what the kernel
cannot check itself, and launches on torch's current stream.  There is no
fallback: a tensor on the CPU, or a library that cannot be built, is an error.
"""
from __future__ import annotations

import os
from ctypes import c_float, c_int, c_long, c_longlong, c_void_p

import torch

from . import build

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}


class KernelError(RuntimeError):
    pass


def dtype_code(t: torch.Tensor | torch.dtype) -> int:
    dt = t if isinstance(t, torch.dtype) else t.dtype
    try:
        return _CODES[dt]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16, not {dt}") from None


def _p(t: torch.Tensor | None):
    if t is None:
        return c_void_p(0)
    if not t.is_cuda:
        raise KernelError("the kernels run on the GPU only: got a tensor on " + str(t.device))
    return c_void_p(t.data_ptr())


def _stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


_launches = 0
_by_name: dict[str, int] = {}


def launch_count() -> int:
    """Kernels launched so far by this process (replays of a captured step count the
    kernels the capture recorded)."""
    return _launches


def launches_by_name() -> dict[str, int]:
    """How often each launcher has run so far (a copy): which kernels a piece of work went through."""
    return dict(_by_name)


def add_launches(n: int, by_name: dict[str, int] | None = None, sign: int = 1) -> None:
    """Count `n` kernels that were recorded or replayed rather than launched here; `by_name` says which."""
    global _launches
    _launches += n
    for name, k in (by_name or {}).items():
        _by_name[name] = _by_name.get(name, 0) + sign * k


def launches_since(before: dict[str, int]) -> dict[str, int]:
    return {name: k - before.get(name, 0) for name, k in _by_name.items() if k != before.get(name, 0)}


def _check(code: int, what: str, kernels: int = 1, variant: str | None = None) -> None:
    """`variant` names the path inside the launcher that the sizes chose (counted beside the launcher)."""
    global _launches
    if code == 0:
        _launches += kernels
        _by_name[what] = _by_name.get(what, 0) + 1
        if variant:
            _by_name[variant] = _by_name.get(variant, 0) + 1
        return
    reason = {-1: "unsupported dtype", -2: "unsupported size", -3: "CUDA driver entry point not found",
              -4: "scratch too small"}.get(code, f"CUDA error {code}")
    raise KernelError(f"{what}: {reason}")


_declared: set[tuple[str, str]] = set()


# Libraries whose kernels wait on barriers with a time limit, and what their status codes mean.
_WATCHED = {"gemm_tc": {1: "the TMA producer waited for a free stage", 2: "the product issuer waited for a free accumulator",
                        3: "the product issuer waited for a stage's copies", 4: "the epilogue waited for an accumulator"},
            "gemm_pair": {1: "a TMA producer waited for a free stage", 2: "the product issuer waited for a free accumulator",
                          3: "the product issuer waited for a stage's copies", 4: "an epilogue waited for an accumulator"},
            "attn_prefill_tc": {}}
_status_words: dict[str, object] = {}


def _watch(lib: str, handle) -> None:
    """Set up the library's status word in mapped host memory (once; not while a stream is being captured,
    since the set-up copies a pointer to the device)."""
    if lib in _status_words or torch.cuda.is_current_stream_capturing():
        return
    from ctypes import POINTER
    fn = getattr(handle, f"lq_{lib}_status_word")
    fn.restype = POINTER(c_int)
    fn.argtypes = []
    _status_words[lib] = fn()


def check_status() -> None:
    """Raise if a bounded wait inside a tensor-core kernel gave up since the last check.  It reads words
    in host memory that such a kernel writes through, so it costs no CUDA call and sees everything that
    ran before the host's last synchronisation: call it where the host has just waited for results."""
    for lib, word in _status_words.items():
        if word and word[0]:
            code = int(word[0])
            word[0] = 0
            why = _WATCHED[lib].get(code, "a wait on a barrier")
            raise KernelError(f"{lib}: {why} for two seconds and gave up (code {code}); the step's results are not valid")


def _fn(lib: str, name: str, argtypes):
    handle = build.load(lib)
    if lib in _WATCHED:
        _watch(lib, handle)
    fn = getattr(handle, name)
    if (lib, name) not in _declared:
        fn.argtypes = argtypes
        fn.restype = c_int
        _declared.add((lib, name))
    return fn


def _contig(t: torch.Tensor, what: str) -> torch.Tensor:
    if not t.is_contiguous():
        raise KernelError(f"{what} must be contiguous")
    return t


def prepare(dtype: torch.dtype, verbose: bool = True, extra: tuple = ()) -> None:
    """Build and load the libraries a model of this dtype uses, before the first step.  extra: libraries
    that parts of the model name beyond the common ones (`Part.kernel_libraries`)."""
    from concurrent.futures import ThreadPoolExecutor
    names = ["plain_kernels", *extra] + (["gemm_skinny", "gemm_tc", "gemm_pair"] if dtype == torch.bfloat16 else [])
    names = list(dict.fromkeys(names))
    with ThreadPoolExecutor(max_workers=len(names)) as pool:
        list(pool.map(build.build, names))
    for name in names:
        build.load(name)


# ------------------------------------------------------------------ plain kernels

def embedding(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """out[t] = table[tokens[t]] as float32 (the residual stream starts in 32-bit)."""
    V, D = table.shape
    T = tokens.numel()
    if out is None:
        out = torch.empty((T, D), dtype=torch.float32, device=table.device)
    fn = _fn("plain_kernels", "lq_embedding", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(_p(_contig(table, "table")), dtype_code(table), _p(tokens), _p(out), T, D, V, _stream()), "embedding")
    return out


def embedding_pairs(table: torch.Tensor, pairs: torch.Tensor, buckets: int, mul_prev: int, mul_cur: int, tokens, tok_pos,
                    tok_seq, slots, cu_rows, last: torch.Tensor, B: int) -> torch.Tensor:
    """out[t] = table[tok_t] + pairs[(tok_(t-1) * mul_prev + tok_t * mul_cur) mod buckets] as float32; pairs[buckets] for a
    sequence's first token.  `last` (int32 [slots]) holds each live sequence's last token between steps: read for a
    step's first row, written with the step's last token afterwards."""
    V, D = table.shape
    T = tokens.numel()
    if pairs.shape != (buckets + 1, D) or pairs.dtype != table.dtype or last.dtype != torch.int32:
        raise KernelError(f"embedding_pairs: the second table must be [{buckets + 1}, {D}] of the first one's dtype, the state int32")
    out = torch.empty((T, D), dtype=torch.float32, device=table.device)
    fn = _fn("plain_kernels", "lq_embedding_pairs", [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                     c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_longlong, c_longlong,
                                                     c_void_p])
    _check(fn(_p(_contig(table, "table")), _p(_contig(pairs, "pairs")), dtype_code(table), _p(tokens), _p(tok_pos), _p(tok_seq),
              _p(slots), _p(cu_rows), _p(last), _p(out), T, B, D, V, int(buckets), int(mul_prev), int(mul_cur), _stream()),
           "embedding_pairs", kernels=2)
    return out


def causal_conv(h: torch.Tensor, w: torch.Tensor, state: torch.Tensor | None, tok_seq, slots, cu_rows, B: int,
                add_input: bool = True, w_by_taps: torch.Tensor | None = None) -> torch.Tensor:
    """out[t] = (h[t] +) sum_j w[:, j] h[t - taps + 1 + j] over each sequence's own rows, per channel; w float32 [D, taps].
    state float32 [slots, taps - 1, D]: the rows ahead of a step's first row (zero at a sequence's start), moved on
    by the step's rows afterwards.  w_by_taps: the same weight as contiguous float32 [taps, D]; with it, rows whose
    channels come in whole 16-byte pieces take the kernel that makes 16 bytes of channels a thread (the same sums)."""
    T, D = h.shape
    taps = w.shape[1]
    if w.dtype != torch.float32 or w.shape[0] != D or not w.is_contiguous():
        raise KernelError("causal_conv: the taps must be contiguous float32 [D, taps]")
    if w_by_taps is not None and (w_by_taps.dtype != torch.float32 or tuple(w_by_taps.shape) != (taps, D) or not w_by_taps.is_contiguous()):
        raise KernelError("causal_conv: the weight by taps must be contiguous float32 [taps, D]")
    if taps > 1 and (state is None or state.dtype != torch.float32 or tuple(state.shape[1:]) != (taps - 1, D) or not state.is_contiguous()):
        raise KernelError(f"causal_conv: the state must be contiguous float32 [slots, {taps - 1}, {D}]")
    out = torch.empty_like(h)
    fn = _fn("plain_kernels", "lq_causal_conv_by_taps", [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                         c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(_p(_contig(h, "h")), _p(out), dtype_code(h), _p(w), _p(w_by_taps), _p(state), _p(tok_seq), _p(slots), _p(cu_rows), T, B,
              D, taps, int(add_input), _stream()), "causal_conv", kernels=2 if taps > 1 else 1)
    return out


def add_scaled(x: torch.Tensor, y: torch.Tensor, m: float) -> torch.Tensor:
    """x += m * y, both float32 of one shape (a branch that joins the stream with a multiplier)."""
    if x.dtype != torch.float32 or y.dtype != torch.float32 or x.shape != y.shape or not x.is_contiguous() or not y.is_contiguous():
        raise KernelError("add_scaled: two contiguous float32 tensors of one shape")
    fn = _fn("plain_kernels", "lq_add_scaled", [c_void_p, c_void_p, c_float, c_longlong, c_void_p])
    _check(fn(_p(x), _p(y), float(m), x.numel(), _stream()), "add_scaled")
    return x


def add_scaled_norm(x: torch.Tensor, y: torch.Tensor, m: float, gain: torch.Tensor, eps: float, out_dtype: torch.dtype) -> torch.Tensor:
    """x += m * y in place (float32 [T, D] both), and the rows of the RMS norm that reads x next, x / rms(x) * gain in
    out_dtype: add_scaled and rmsnorm in one pass over the stream, with their sums in the same order."""
    T, D = x.shape
    if x.dtype != torch.float32 or y.dtype != torch.float32 or x.shape != y.shape or not x.is_contiguous() or not y.is_contiguous():
        raise KernelError("add_scaled_norm: contiguous float32 tensors of one shape")
    if gain.dtype != torch.float32 or gain.numel() != D or not gain.is_contiguous():
        raise KernelError("add_scaled_norm: the gain must be contiguous float32 [D]")
    out = torch.empty((T, D), dtype=out_dtype, device=x.device)
    fn = _fn("plain_kernels", "lq_add_scaled_norm", [c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int, c_int, c_float,
                                                     c_void_p])
    _check(fn(_p(x), _p(y), float(m), _p(gain), _p(out), dtype_code(out_dtype), T, D, float(eps), _stream()), "add_scaled_norm")
    return out


def rmsnorm(x: torch.Tensor, gain: torch.Tensor, eps: float, out_dtype: torch.dtype,
            rows: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """RMS norm of rows of the float32 stream x [T, D]; `rows` (int32) picks rows."""
    if x.dtype != torch.float32 or gain.dtype != torch.float32:
        raise KernelError("rmsnorm reads a float32 stream and float32 gains")
    D = x.shape[-1]
    n = x.shape[0] if rows is None else rows.numel()
    if out is None:
        out = torch.empty((n, D), dtype=out_dtype, device=x.device)
    fn = _fn("plain_kernels", "lq_rmsnorm", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p])
    _check(fn(_p(_contig(x, "x")), _p(gain), _p(rows), _p(out), dtype_code(out_dtype), n, D, float(eps), _stream()), "rmsnorm")
    return out


def layernorm(x: torch.Tensor, gain: torch.Tensor, bias: torch.Tensor | None, eps: float, out_dtype: torch.dtype,
              rows: torch.Tensor | None = None, add: tuple = ()) -> torch.Tensor:
    """Layer norm of rows of the float32 stream x [T, D]: (x - mean) / sqrt(var + eps) * gain + bias, var the mean of the
    squared deviations, all in 32-bit; `rows` (int32) picks rows.  add = ((y, m), ...) (one or two float32 [T, D]): the
    stream first takes x += m * y for each, in place, in the same pass."""
    if x.dtype != torch.float32 or gain.dtype != torch.float32 or (bias is not None and bias.dtype != torch.float32):
        raise KernelError("layernorm reads a float32 stream, float32 gains and biases")
    D = x.shape[-1]
    n = x.shape[0] if rows is None else rows.numel()
    if len(add) > 2 or (add and rows is not None):
        raise KernelError("layernorm: at most two branches join the stream, and only when every row is normed")
    for y, _ in add:
        if y.dtype != torch.float32 or y.shape != x.shape or not y.is_contiguous():
            raise KernelError("layernorm: a branch must be contiguous float32 of the stream's shape")
    (y1, m1), (y2, m2) = (tuple(add) + ((None, 0.0), (None, 0.0)))[:2]
    out = torch.empty((n, D), dtype=out_dtype, device=x.device)
    fn = _fn("plain_kernels", "lq_layernorm", [c_void_p, c_void_p, c_float, c_void_p, c_float, c_void_p, c_void_p, c_void_p,
                                               c_void_p, c_int, c_int, c_int, c_float, c_void_p])
    _check(fn(_p(_contig(x, "x")), _p(y1), float(m1), _p(y2), float(m2), _p(gain), _p(bias), _p(rows), _p(out),
              dtype_code(out_dtype), n, D, float(eps), _stream()), "layernorm")
    return out


def side_by_side(a: torch.Tensor, b: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """[a, b] along the columns, in out_dtype, from two contiguous float32 [T, D]: the input of a product that reads two streams."""
    if a.dtype != torch.float32 or b.dtype != torch.float32 or a.shape != b.shape or not a.is_contiguous() or not b.is_contiguous():
        raise KernelError("side_by_side: two contiguous float32 tensors of one shape")
    T, D = a.shape
    out = torch.empty((T, 2 * D), dtype=out_dtype, device=a.device)
    fn = _fn("plain_kernels", "lq_side_by_side", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(_p(a), _p(b), _p(out), dtype_code(out_dtype), T, D, _stream()), "side_by_side")
    return out


def gemm_plain(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, residual: torch.Tensor | None = None,
               out: torch.Tensor | None = None) -> torch.Tensor:
    """a [M, K] . w [N, K]^T (+ residual) on the CUDA cores, every product in float32."""
    M, K = a.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelError(f"linear: input width {K} does not match weight width {K2}")
    if residual is not None:
        if residual.dtype != torch.float32 or tuple(residual.shape) != (M, N):
            raise KernelError("linear: residual must be float32 [M, N]")
        if out is None:
            out = residual
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    fn = _fn("plain_kernels", "lq_gemm_plain", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p,
                                                c_int, c_int, c_int, c_void_p])
    _check(fn(_p(_contig(a, "a")), dtype_code(a), _p(_contig(w, "w")), dtype_code(w), _p(out), dtype_code(out),
              _p(residual), M, N, K, _stream()), "linear")
    return out


def _check_tables(what: str, cos, sin, hd: int, tok_pos=None) -> None:
    """The fused q/k/v epilogues read cos/sin at [position, head_dim / 2]: tables of another width (a part
    that rotates only some of a head's dimensions) would be read across rows."""
    if cos is None and sin is None:
        return
    if cos is None or sin is None:
        raise KernelError(f"{what}: cos and sin tables come together")
    for t in (cos, sin):
        if t.dtype != torch.float32 or t.dim() != 2 or t.shape[1] != hd // 2 or not t.is_contiguous():
            raise KernelError(f"{what}: cos/sin tables must be contiguous float32 [positions, head_dim / 2 = {hd // 2}], "
                              f"found {tuple(t.shape)} {t.dtype}")
    if cos.shape != sin.shape:
        raise KernelError(f"{what}: cos {tuple(cos.shape)} and sin {tuple(sin.shape)} differ")


def rope_kv_write(qkv: torch.Tensor, cos: torch.Tensor | None, sin: torch.Tensor | None, tok_pos, tok_seq, slots,
                  page_table: torch.Tensor | None, k_pages: torch.Tensor | None, v_pages: torch.Tensor | None,
                  H: int, Hkv: int, hd: int, page_size: int) -> None:
    """Rotate q and k of every token in place and store k, v into the cache pages."""
    T = qkv.shape[0]
    has_kv = k_pages is not None
    width = (H + (2 * Hkv if has_kv else 0)) * hd
    if qkv.shape[1] != width:
        raise KernelError(f"rope: qkv rows are {qkv.shape[1]} wide, expected {width}")
    if has_kv and (k_pages.dtype != qkv.dtype or v_pages.dtype != qkv.dtype):
        raise KernelError("rope: the cache and the activations must have one dtype")
    _check_tables("rope", cos, sin, hd)
    fn = _fn("plain_kernels", "lq_rope_kv_write", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                   c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                                   c_int, c_int, c_void_p])
    _check(fn(_p(_contig(qkv, "qkv")), dtype_code(qkv), _p(cos), _p(sin), _p(tok_pos), _p(tok_seq), _p(slots),
              _p(page_table), page_table.stride(0) if page_table is not None else 0, _p(k_pages), _p(v_pages),
              T, H, Hkv, hd, page_size, int(has_kv), _stream()), "rope_kv_write")


def attention_plain(q: torch.Tensor, k_pages, v_pages, page_table, tok_pos, tok_seq, slots, H: int, Hkv: int,
                    hd: int, page_size: int, scale: float, window: int | None,
                    out: torch.Tensor | None = None, vd: int | None = None, sink: torch.Tensor | None = None,
                    gate: torch.Tensor | None = None, softcap: float | None = None, keep_first: int = 0,
                    chunk: int | None = None, gate_per_head: bool = False) -> torch.Tensor:
    """Causal attention of every token over its own sequence's cache; q is the left
    H*hd columns of a [T, q_stride] buffer.  softcap c: score <- c tanh(score / c) after the scale.  keep_first: with a
    window, the sequence's first keep_first positions stay visible when the window has moved past them.  vd: size of a value head (default hd).  sink: float32 [H], one
    more term exp(sink) in each head's softmax denominator.  gate: a [T, H*vd] view (rows may be strided) whose
    sigmoid multiplies the output; with gate_per_head a [T, H] view, one number for all values of a head.
    chunk n (instead of a window): a position sees only its own block of n positions."""
    T = q.shape[0]
    vd = vd or hd
    if hd > 256 or vd > 256:
        raise KernelError(f"attention: head sizes {hd}, {vd} exceed 256")
    if sink is not None and (sink.dtype != torch.float32 or sink.numel() != H):
        raise KernelError("attention: sink must be float32 [H]")
    if gate is not None and (gate.dtype not in (q.dtype, torch.float32) or gate.stride(1) != 1
                             or gate.shape != (T, H if gate_per_head else H * vd)):
        raise KernelError("attention: the gate must be [T, H * vd] (or [T, H]) of the queries' dtype or float32, with unit column stride")
    if out is None:
        out = torch.empty((T, H * vd), dtype=q.dtype, device=q.device)
    fn = _fn("plain_kernels", "lq_attention_plain", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                                     c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                                     c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_float, c_int,
                                                     c_int, c_void_p])
    _check(fn(_p(q), q.stride(0), dtype_code(q), _p(k_pages), _p(v_pages), _p(page_table), page_table.stride(0),
              _p(tok_pos), _p(tok_seq), _p(slots), _p(out), T, H, Hkv, hd, page_size, float(scale),
              span(window, chunk), vd, _p(sink), _p(gate), gate.stride(0) if gate is not None else 0,
              dtype_code(gate) if gate is not None else F32, float(softcap or 0.0), int(keep_first or 0),
              int(bool(gate_per_head and gate is not None)), _stream()), "attention")
    return out


def span(window: int | None, chunk: int | None = None) -> int:
    """A mask as the one integer the attention kernels take: a sliding window of w positions as w, blocks of n
    positions (a position sees its own block only) as -n, every earlier position as 0."""
    if chunk:
        if window:
            raise KernelError("attention: a window or blocks of positions, not both")
        return -int(chunk)
    return int(window or 0)


def swiglu(gu: torch.Tensor, block: int = 0, out: torch.Tensor | None = None) -> torch.Tensor:
    """gu [T, 2F] -> up * silu(gate) [T, F].  block 0: gate columns, then up columns;
    block b: b gate columns, b up columns, alternating."""
    T, F2 = gu.shape
    F = F2 // 2
    if out is None:
        out = torch.empty((T, F), dtype=gu.dtype, device=gu.device)
    fn = _fn("plain_kernels", "lq_swiglu", [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(_p(_contig(gu, "gu")), _p(out), dtype_code(gu), T, F, block, _stream()), "swiglu")
    return out


def clear_page_tails(k_pages: torch.Tensor, v_pages: torch.Tensor, items: list[tuple[int, int]]) -> None:
    """Zero the rows [first, page_size) of the pages in `items` = [(page, first)], in every entry and kv
    head of the pools k_pages, v_pages [entries, pages, kv heads, page_size, head_dim]."""
    from ctypes import c_int as _int
    if v_pages.shape != k_pages.shape:
        # Values of another size than the keys: each pool on its own.
        if v_pages.shape[:4] != k_pages.shape[:4] or v_pages.dtype != k_pages.dtype:
            raise KernelError("clear_page_tails: keys and values must agree in all but the head size")
        clear_page_tails(k_pages, k_pages, items)
        clear_page_tails(v_pages, v_pages, items)
        return
    E, P, Hkv, page_size, hd = k_pages.shape
    if v_pages.dtype != k_pages.dtype:
        raise KernelError("clear_page_tails: keys and values must have one dtype")
    n = len(items)
    pages = (_int * n)(*[int(p) for p, _ in items])
    first = (_int * n)(*[int(f) for _, f in items])
    from ctypes import POINTER
    fn = _fn("plain_kernels", "lq_clear_page_tails", [c_void_p, c_void_p, c_int, POINTER(c_int), POINTER(c_int), c_int,
                                                      c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(_p(_contig(k_pages, "k_pages")), _p(_contig(v_pages, "v_pages")), dtype_code(k_pages), pages, first, n,
              E, P, Hkv, page_size, hd, _stream()), "clear_page_tails", -(-n // 120))


def rmsnorm_add(y: torch.Tensor, gain: torch.Tensor, eps: float, x: torch.Tensor, next_norm: tuple | None = None,
                out_dtype: torch.dtype | None = None) -> torch.Tensor | None:
    """x += y / rms(y) * gain, row by row, in place (x, y float32 [T, D]): a branch joins the stream after
    its own norm.  next_norm = (gain, eps) of the norm that reads the stream next: its rows
    x / rms(x) * gain are made by the same kernel and returned in out_dtype."""
    if x.dtype != torch.float32 or y.dtype != torch.float32 or gain.dtype != torch.float32 or x.shape != y.shape:
        raise KernelError("rmsnorm_add reads float32 rows of one shape and float32 gains")
    T, D = x.shape
    h = next_gain = None
    next_eps = 0.0
    if next_norm is not None:
        next_gain, next_eps = next_norm
        if next_gain.dtype != torch.float32 or next_gain.numel() != D:
            raise KernelError("rmsnorm_add: the next norm's gain must be float32 [D]")
        h = torch.empty((T, D), dtype=out_dtype, device=x.device)
    fn = _fn("plain_kernels", "lq_rmsnorm_add", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                                 c_float, c_float, c_void_p])
    _check(fn(_p(_contig(y, "y")), _p(gain), _p(_contig(x, "x")), _p(next_gain), _p(h),
              dtype_code(out_dtype) if h is not None else F32, T, D, float(eps), float(next_eps), _stream()), "rmsnorm_add")
    return h


def rope_partial(buf: torch.Tensor, bias: torch.Tensor | None, cos, sin, rot: int, tok_pos, tok_seq, slots,
                 page_table, k_pages, v_pages, n_rot: int, k_first: int, Hkv: int, hd: int, vd: int, v_off: int,
                 page_size: int, qout: torch.Tensor | None = None, v_unit_eps: float | None = None,
                 unit_norm: str | None = None, norm_weight: torch.Tensor | None = None, norm_eps: float = 0.0,
                 q_temp: tuple | None = None) -> None:
    """Biases, then rotation of the first `rot` dimensions, for each of the n_rot heads at the left of buf's rows;
    heads below k_first (queries) go to `qout` [T, k_first * hd] (default: back in place), heads k_first.. into
    k_pages and the values at column v_off into v_pages where a cache is given.  bias: float32 over buf's
    columns, or None; cos/sin: float32 [positions, rot / 2].  buf may be float32 while qout and the cache are
    bfloat16 (a product's 32-bit sums, rounded once, after bias and rotation).  v_unit_eps: each value head is divided by
    its root mean square, sqrt(mean(v^2) + v_unit_eps), before it is stored.  unit_norm (32-bit, after the bias and ahead
    of the rotation): "head", every one of the n_rot heads over its own root mean square sqrt(mean(x^2) + norm_eps);
    "all", the queries over the root mean square of all of them together and the keys likewise, times norm_weight
    (float32 over the n_rot * hd columns).  q_temp = (coef, every): the queries times 1 + coef ln(floor((p + 1) / every) + 1)."""
    T = buf.shape[0]
    if buf.stride(1) != 1:
        raise KernelError("rope_partial: rows must be contiguous")
    if qout is None:
        qout = buf
    elif qout.shape[0] != T or qout.shape[1] < k_first * hd or qout.stride(1) != 1:
        raise KernelError("rope_partial: qout must be [T, >= k_first * hd] with unit column stride")
    if rot:
        for t in (cos, sin):
            if t is None or t.dtype != torch.float32 or t.dim() != 2 or t.shape[1] != rot // 2 or not t.is_contiguous():
                raise KernelError(f"rope_partial: cos/sin tables must be contiguous float32 [positions, {rot // 2}]")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() < (v_off + Hkv * vd if k_pages is not None else n_rot * hd)):
        raise KernelError("rope_partial: the bias must be float32 over the rows' columns")
    if k_pages is not None and (k_pages.dtype != qout.dtype or v_pages.dtype != qout.dtype):
        raise KernelError("rope_partial: the cache and the queries must have one dtype")
    if unit_norm not in (None, "head", "all"):
        raise KernelError(f"rope_partial: unit_norm {unit_norm!r} is not one of None, 'head', 'all'")
    mode = {None: 0, "head": 1, "all": 2}[unit_norm]
    if norm_weight is not None and (mode != 2 or norm_weight.dtype != torch.float32 or norm_weight.numel() != n_rot * hd
                                    or not norm_weight.is_contiguous()):
        raise KernelError("rope_partial: the norm's weight goes with unit_norm 'all' and is contiguous float32 over the heads' columns")
    if q_temp is not None and not int(q_temp[1]) > 0:
        raise KernelError("rope_partial: the query temperature's step must be positive")
    fn = _fn("plain_kernels", "lq_rope_partial", [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                                  c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                                  c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                                  c_int, c_void_p, c_float, c_float, c_int, c_void_p])
    _check(fn(_p(buf), dtype_code(buf), buf.stride(0), _p(qout), dtype_code(qout), qout.stride(0), _p(bias), _p(cos), _p(sin),
              int(rot), _p(tok_pos), _p(tok_seq), _p(slots), _p(page_table),
              page_table.stride(0) if page_table is not None else 0, _p(k_pages), _p(v_pages),
              T, n_rot, k_first, Hkv, hd, vd, v_off, page_size, int(v_unit_eps is not None), float(v_unit_eps or 0.0),
              mode, _p(norm_weight), float(norm_eps), float(q_temp[0]) if q_temp else 0.0, int(q_temp[1]) if q_temp else 0,
              _stream()), "rope_partial")


ACTIVATIONS = {"relu2": 0, "gelu_tanh": 1, "silu": 2, "relu": 3, "gelu": 4}


def activation(x: torch.Tensor, kind: str, out: torch.Tensor | None = None) -> torch.Tensor:
    """act(x) element by element, computed in float32: relu2 (the square of relu), gelu_tanh, silu, relu, gelu (the erf form)."""
    if kind not in ACTIVATIONS:
        raise KernelError(f"activation {kind!r} is not one of {', '.join(ACTIVATIONS)}")
    if out is None:
        out = torch.empty_like(x)
    fn = _fn("plain_kernels", "lq_activation", [c_void_p, c_void_p, c_int, c_long, c_int, c_void_p])
    _check(fn(_p(_contig(x, "x")), _p(out), dtype_code(x), x.numel(), ACTIVATIONS[kind], _stream()), "activation")
    return out


def softcap(x: torch.Tensor, cap: float) -> torch.Tensor:
    """x <- cap * tanh(x / cap) in place (float32)."""
    if x.dtype != torch.float32:
        raise KernelError("softcap works on float32 logits")
    fn = _fn("plain_kernels", "lq_softcap", [c_void_p, c_long, c_float, c_void_p])
    _check(fn(_p(_contig(x, "x")), x.numel(), float(cap), _stream()), "softcap")
    return x


def gate_mul(x: torch.Tensor, gate: torch.Tensor, act: str = "sigmoid", group: int = 1) -> torch.Tensor:
    """x *= act(gate) in place; x [rows, cols] contiguous, gate a [rows, cols / group] view whose rows may be strided:
    one gate for every `group` neighbouring columns (group = a head's size: one number per head)."""
    rows, cols = x.shape
    if group < 1 or cols % group or gate.dtype not in (x.dtype, torch.float32) or tuple(gate.shape) != (rows, cols // group) \
            or gate.stride(1) != 1:
        raise KernelError("gate_mul: the gate must be [rows, cols / group] of x's dtype or float32, with unit column stride")
    fn = _fn("plain_kernels", "lq_gate_mul", [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(_p(_contig(x, "x")), _p(gate), gate.stride(0), dtype_code(x), dtype_code(gate), rows, cols, GATES[act], int(group),
              _stream()), "gate_mul")
    return x


def gated_act(gu: torch.Tensor, bias: torch.Tensor | None, kind: str, out_dtype: torch.dtype) -> torch.Tensor:
    """gu [T, 2F] (gate columns, then up columns) -> act(gate + b_gate) * (up + b_up) [T, F]; bias float32 [2F] or None."""
    T, F2 = gu.shape
    F = F2 // 2
    if kind not in ACTIVATIONS:
        raise KernelError(f"activation {kind!r} is not one of {', '.join(ACTIVATIONS)}")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != F2):
        raise KernelError("gated_act: the bias must be float32 [2F]")
    out = torch.empty((T, F), dtype=out_dtype, device=gu.device)
    fn = _fn("plain_kernels", "lq_gated_act", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(_p(_contig(gu, "gu")), dtype_code(gu), _p(bias), _p(out), dtype_code(out), T, F, ACTIVATIONS[kind], _stream()), "gated_act")
    return out


def add_bias(x: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """x[t, :] += bias in place (float32 rows of the stream, float32 bias)."""
    if x.dtype != torch.float32 or bias.dtype != torch.float32 or bias.numel() != x.shape[1]:
        raise KernelError("add_bias works on float32 rows with a float32 bias of their width")
    fn = _fn("plain_kernels", "lq_add_bias", [c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check(fn(_p(_contig(x, "x")), _p(bias), x.shape[0], x.shape[1], _stream()), "add_bias")
    return x


# ------------------------------------------------------------------ attention over a latent cache
def latent_kv_store(rows: torch.Tensor, c_off: int, r_off: int, gain: torch.Tensor, eps: float, cos, sin, rot: int, tok_pos,
                    tok_seq, slots, page_table, pages: torch.Tensor, R: int, dr: int, page_size: int) -> None:
    """For every row: the latent (columns c_off .. c_off + R) over its root mean square times `gain`, and the shared key
    part (columns r_off .. r_off + dr) with its first `rot` dimensions rotated by the row's position, stored as one row
    [R + dr] of the row's cache page (pages [pages, page_size, R + dr])."""
    if rows.stride(1) != 1 or gain.dtype != torch.float32 or gain.numel() != R:
        raise KernelError("latent_kv_store: rows with unit column stride and a float32 gain [R]")
    if pages.shape[-1] != R + dr or not pages.is_contiguous():
        raise KernelError(f"latent_kv_store: cache rows must be {R + dr} wide")
    if rot:
        for t in (cos, sin):
            if t is None or t.dtype != torch.float32 or t.dim() != 2 or t.shape[1] != rot // 2 or not t.is_contiguous():
                raise KernelError(f"latent_kv_store: cos/sin tables must be contiguous float32 [positions, {rot // 2}]")
    fn = _fn("latent_attn", "lq_latent_kv_store", [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p, c_void_p,
                                                   c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int,
                                                   c_int, c_int, c_int, c_void_p])
    _check(fn(_p(rows), dtype_code(rows), rows.stride(0), c_off, r_off, _p(gain), float(eps), _p(cos), _p(sin), int(rot),
              _p(tok_pos), _p(tok_seq), _p(slots), _p(page_table), page_table.stride(0), _p(pages), dtype_code(pages),
              rows.shape[0], R, dr, page_size, _stream()), "latent_kv_store")


def rope_tail(src: torch.Tensor, src_head: int, src_off: int, out: torch.Tensor, out_head: int, out_off: int, cos, sin,
              rot: int, tok_pos, H: int, n: int) -> None:
    """The n columns at src_off of each of the H heads (src_head wide) of src's rows, their first `rot` dimensions rotated
    by the row's position, written to out (float32) at out_off of each head (out_head wide)."""
    if src.stride(1) != 1 or out.stride(1) != 1 or out.dtype != torch.float32:
        raise KernelError("rope_tail: unit column strides and a float32 output")
    fn = _fn("latent_attn", "lq_rope_tail", [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_int, c_void_p,
                                             c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(_p(src), dtype_code(src), src.stride(0), src_head, src_off, _p(out), out.stride(0), out_head, out_off, _p(cos),
              _p(sin), int(rot), _p(tok_pos), src.shape[0], H, n, _stream()), "rope_tail")


def head_matmul(src: torch.Tensor, src_head: int, src_off: int, w: torch.Tensor, out: torch.Tensor, out_head: int,
                out_off: int) -> torch.Tensor:
    """out[t, h * out_head + out_off + n] = sum_k src[t, h * src_head + src_off + k] * w[h, k, n] for w [H, K, N]: one small
    matrix per head, float32 sums over k in rising order."""
    H, K, N = w.shape
    if src.stride(1) != 1 or out.stride(1) != 1 or not w.is_contiguous():
        raise KernelError("head_matmul: unit column strides and a contiguous weight [H, K, N]")
    fn = _fn("latent_attn", "lq_head_matmul", [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_int,
                                               c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(_p(src), dtype_code(src), src.stride(0), src_head, src_off, _p(w), dtype_code(w), _p(out), dtype_code(out),
              out.stride(0), out_head, out_off, src.shape[0], H, K, N, _stream()), "head_matmul")
    return out


def latent_attention(q: torch.Tensor, pages: torch.Tensor, page_table, tok_pos, tok_seq, slots, H: int, R: int, page_size: int,
                     scale: float, window: int | None, splits: int = 1) -> torch.Tensor:
    """Causal attention of every row's H wide queries q [T, H, Dk] (float32) over the latent rows of its sequence's cache
    (pages [pages, page_size, Dk]): scores over all Dk numbers, values the rows' first R numbers.  Returns float32
    [T, H, R].  splits: slices that each row's keys are cut into (merged by a second kernel)."""
    T, Hq, Dk = q.shape
    if q.dtype != torch.float32 or not q.is_contiguous() or Hq != H or pages.shape[-1] != Dk or not pages.is_contiguous():
        raise KernelError("latent_attention: contiguous float32 queries [T, H, Dk] and cache rows of Dk numbers")
    if R > 1024:
        raise KernelError(f"latent_attention: a latent of {R} numbers exceeds 1024")
    out = torch.empty((T, H, R), dtype=torch.float32, device=q.device)
    part_o = part_ml = None
    if splits > 1:
        part_o = torch.empty((T, H, splits, R), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((T, H, splits, 2), dtype=torch.float32, device=q.device)
    fn = _fn("latent_attn", "lq_latent_attention", [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                                    c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                                                    c_int, c_int, c_void_p])
    _check(fn(_p(q), _p(pages), dtype_code(pages), _p(page_table), page_table.stride(0), _p(tok_pos), _p(tok_seq), _p(slots),
              _p(out), _p(part_o), _p(part_ml), T, H, R, Dk, page_size, float(scale), int(window or 0), int(splits), _stream()),
           "latent_attention", 2 if splits > 1 else 1, "latent_attention:slices" if splits > 1 else None)
    return out


def latent_tc_tokens(H: int) -> int:
    """Tokens of one block of latent_attention_tc for H heads: as many as fit, with all their heads, into its 64 rows."""
    return 1 if H >= 64 else 64 // H


def latent_attention_tc_takes(pages: torch.Tensor, page_size: int) -> bool:
    """Whether the tensor-core kernel serves this cache: bfloat16 rows of a multiple of 8 numbers, pages of a multiple of 32."""
    return pages.dtype == torch.bfloat16 and pages.shape[-1] % 8 == 0 and page_size % 32 == 0


def latent_attention_tc(q: torch.Tensor, pages: torch.Tensor, page_table, slots, H: int, R: int, page_size: int, scale: float,
                        window: int | None, blocks: tuple | None = None, tok_pos=None, tok_seq=None, splits: int = 1,
                        out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """latent_attention on the tensor cores (mma.sync, bfloat16 cache rows).  blocks = (sequence, first row, tokens, first
    position) int32 tensors, one entry per block of at most latent_tc_tokens(H) consecutive tokens of one sequence, for
    a step with prompts; without it every row is its own block (tok_pos, tok_seq) and its keys may be cut into `splits`.
    Returns [T, H, R] in out_dtype (float32 or bfloat16)."""
    T, Hq, Dk = q.shape
    if q.dtype != torch.float32 or not q.is_contiguous() or Hq != H or pages.shape[-1] != Dk or not pages.is_contiguous():
        raise KernelError("latent_attention_tc: contiguous float32 queries [T, H, Dk] and cache rows of Dk numbers")
    if not latent_attention_tc_takes(pages, page_size):
        raise KernelError("latent_attention_tc takes bfloat16 cache rows of a multiple of 8 numbers in pages of a multiple of 32")
    out = torch.empty((T, H, R), dtype=out_dtype, device=q.device)
    part_o = part_ml = None
    if blocks is not None:
        splits = 1
    if splits > 1:
        part_o = torch.empty((T, H, splits, R), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((T, H, splits, 2), dtype=torch.float32, device=q.device)
    qb = blocks if blocks is not None else (None, None, None, None)
    fn = _fn("latent_attn_tc", "lq_latent_attention_tc", [c_void_p, c_void_p, c_void_p, c_int] + [c_void_p] * 8 + [c_int, c_void_p, c_void_p]
             + [c_int] * 6 + [c_float, c_int, c_int, c_void_p])
    _check(fn(_p(q), _p(pages), _p(page_table), page_table.stride(0), _p(slots), _p(qb[0]), _p(qb[1]), _p(qb[2]), _p(qb[3]),
              _p(tok_pos), _p(tok_seq), _p(out), dtype_code(out), _p(part_o), _p(part_ml), qb[0].numel() if blocks is not None else T, T, H, R, Dk,
              page_size, float(scale), int(window or 0), int(splits), _stream()),
           "latent_attention_tc", 2 if splits > 1 else 1, "latent_attention_tc:slices" if splits > 1 else None)
    return out


# ------------------------------------------------------------------ many small products in one launch
def grouped_gemm_takes(a: torch.Tensor, w: torch.Tensor, a_group_stride: int = 0) -> bool:
    """Whether grouped_gemm serves these operands: bfloat16, rows and groups that start on 16-byte boundaries."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[-1] % 8 == 0 and a.stride(0) % 8 == 0
            and a_group_stride % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def grouped_gemm(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, a_group_stride: int = 0, o_group_stride: int = 0,
                 listed: tuple | None = None, a_div: int = 1, act: str | None = None) -> torch.Tensor:
    """out[row, group g's columns] = act(a[row, group g's columns] . w[g]^T) for w [G, N, K] on the tensor cores.
    Without `listed` every group takes all rows of a, its K columns starting at g * a_group_stride, and writes its N
    columns at g * o_group_stride of out's rows (one small matrix per head).  listed = (rows, group_off, tile_off) as
    `group_rows` makes them: group g owns rows[group_off[g] : group_off[g + 1]]; it reads row rows[r] // a_div of a
    and writes row rows[r] of out (routed experts)."""
    G, N, K = w.shape
    if a.stride(1) != 1 or out.stride(1) != 1 or not w.is_contiguous() or not grouped_gemm_takes(a, w, a_group_stride):
        raise KernelError("grouped_gemm: bfloat16 operands with unit column strides, rows and groups on 16-byte boundaries")
    rows, group_off, tile_off = listed if listed is not None else (None, None, None)
    fn = _fn("grouped_gemm", "lq_grouped_gemm", [c_void_p, c_long, c_long, c_int, c_void_p, c_long, c_void_p, c_int, c_long, c_long,
                                                 c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(_p(a), a.stride(0), a_group_stride, a_div, _p(w), N * K, _p(out), dtype_code(out), out.stride(0), o_group_stride,
              _p(rows), _p(group_off), _p(tile_off), rows.numel() if rows is not None else 0, G, a.shape[0], N, K, MOE_ACTS[act],
              _stream()), "grouped_gemm", 1, "grouped_gemm:listed" if listed is not None else "grouped_gemm:uniform")
    return out


def group_rows(ids: torch.Tensor, G: int) -> tuple:
    """ids int32 [n], each in [0, G) -> (rows [n]: the indices 0 .. n-1 group by group, group_off [G + 1], tile_off [G + 1]),
    made on the device."""
    n = ids.numel()
    rows = torch.empty(n, dtype=torch.int32, device=ids.device)
    group_off = torch.empty(G + 1, dtype=torch.int32, device=ids.device)
    tile_off = torch.empty(G + 1, dtype=torch.int32, device=ids.device)
    fn = _fn("grouped_gemm", "lq_group_rows", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(fn(_p(_contig(ids, "ids")), n, G, _p(rows), _p(group_off), _p(tile_off), _stream()), "group_rows")
    return rows, group_off, tile_off


GROUP_TILE = 128       # rows of a tile of gemm_tc: the padded order gives every group whole tiles


def group_rows_padded(ids: torch.Tensor, G: int) -> tuple:
    """ids int32 [n] -> (src [cap], dst [n], tile_group [cap / 128]) on the device: the indices group by group with
    every group padded to whole tiles of 128 places (src: the index at each place, -1 for padding; dst: the place of
    each index; tile_group: each tile's group, -1 behind the last).  An index whose id is G or above (a group without
    rows of its own) takes no place: its dst is -1."""
    n = ids.numel()
    cap = (-(-n // GROUP_TILE) + G) * GROUP_TILE
    src = torch.empty(cap, dtype=torch.int32, device=ids.device)
    dst = torch.empty(n, dtype=torch.int32, device=ids.device)
    tile_group = torch.empty(cap // GROUP_TILE, dtype=torch.int32, device=ids.device)
    fn = _fn("grouped_gemm", "lq_group_rows_padded", [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(fn(_p(_contig(ids, "ids")), n, G, GROUP_TILE, cap, _p(src), _p(dst), _p(tile_group), _stream()), "group_rows_padded")
    return src, dst, tile_group


def gather_rows(a: torch.Tensor, src: torch.Tensor, div: int = 1) -> torch.Tensor:
    """out[p] = a[src[p] // div] (zeros where src[p] < 0); rows of a multiple of 16 bytes."""
    row_bytes = a.shape[1] * a.element_size()
    if not a.is_contiguous() or row_bytes % 16:
        raise KernelError("gather_rows: contiguous rows of a multiple of 16 bytes")
    out = torch.empty((src.numel(), a.shape[1]), dtype=a.dtype, device=a.device)
    fn = _fn("grouped_gemm", "lq_gather_rows", [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p])
    _check(fn(_p(a), _p(src), div, _p(out), src.numel(), row_bytes, _stream()), "gather_rows")
    return out


def gemm_tc_grouped(a: torch.Tensor, w: torch.Tensor, tile_group: torch.Tensor, out_dtype: torch.dtype,
                    swiglu: bool = False) -> torch.Tensor:
    """a [M, K] (M a multiple of 128, its row tiles each of one group) times w [G, N, K]: row tile i is multiplied with
    w[tile_group[i]] on the tcgen05 tensor cores (tiles with group -1 are left out and their rows of the result are not
    written).  Returns [M, N] in out_dtype (bfloat16 or float32).  swiglu: every group's rows are 8 gate rows and 8 up
    rows by turns (`linear.interleave_gate_up`), and what comes back is silu(gate) * up, [M, N / 2] bfloat16."""
    M, K = a.shape
    G, N, K2 = w.shape
    if swiglu and (N % 16 or out_dtype != torch.bfloat16):
        raise KernelError("gemm_tc_grouped: the gated form takes 16 rows of weight at a time and hands on bfloat16")
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or K2 != K or K % 8 or M % GROUP_TILE or not a.is_contiguous() \
            or not w.is_contiguous() or tile_group.numel() != M // GROUP_TILE:
        raise KernelError("gemm_tc_grouped: contiguous bfloat16 operands, K a multiple of 8, whole row tiles with a group each")
    out = torch.empty((M, N // 2 if swiglu else N), dtype=out_dtype, device=a.device)
    fn = _fn("gemm_tc", "lq_gemm_tc_grouped", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(fn(_p(a), _p(w), _p(out), 2 if swiglu else int(out_dtype == torch.float32), M, N, K, G, _p(tile_group), _stream()),
           "gemm_tc_grouped")
    return out


def moe_combine(y: torch.Tensor, weights: torch.Tensor, x: torch.Tensor, accumulate: bool = True,
                shared: torch.Tensor | None = None, shared_gate: torch.Tensor | None = None,
                place: torch.Tensor | None = None, ids: torch.Tensor | None = None, E: int = 0,
                h: torch.Tensor | None = None, shared_scale: float = 1.0) -> torch.Tensor:
    """x[t] (+)= sum_j weights[t, j] y[t * top + j] (+ shared_scale * sigmoid(shared_gate[t]) * shared[t]); y float32
    [T * top, D].  place int32 [T * top]: the row of y that holds pair t * top + j (y then has any number of rows).
    ids int32 [T, top] with E and h (bfloat16 [T, D]): a pair whose id is E or above has no row in y and adds
    weights[t, j] * h[t] instead (an expert that passes its input on)."""
    T, top = weights.shape
    D = y.shape[1]
    if y.dtype != torch.float32 or not y.is_contiguous() or tuple(x.shape) != (T, D) or (place is None and y.shape[0] != T * top):
        raise KernelError("moe_combine: float32 rows [T * top, D] and [T, D]")
    if ids is not None and (h is None or h.dtype != torch.bfloat16 or tuple(h.shape) != (T, D) or not h.is_contiguous()
                            or ids.dtype != torch.int32 or ids.numel() != T * top):
        raise KernelError("moe_combine: ids int32 [T, top] come with the experts' input, contiguous bfloat16 [T, D]")
    fn = _fn("grouped_gemm", "lq_moe_combine_more", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int,
                                                     c_int, c_int, c_void_p, c_int, c_void_p, c_float, c_void_p])
    _check(fn(_p(y), _p(place), _p(_contig(weights, "weights")), _p(shared), _p(shared_gate),
              shared_gate.stride(0) if shared_gate is not None else 0, _p(_contig(x, "x")), int(accumulate), T, top, D,
              _p(_contig(ids, "ids")) if ids is not None else None, int(E), _p(h) if ids is not None else None,
              float(shared_scale), _stream()), "moe_combine")
    return x


# ------------------------------------------------------------------ routed feed-forward
MOE_ACTS = {None: 0, "gelu": 1, "gelu_tanh": 2, "silu": 3, "relu": 4}


SCORE_FNS = {"sigmoid": 0, "softmax": 1}
GROUP_RULES = {"top2": 0, "max": 1}


def moe_route(z: torch.Tensor, E: int, groups: int, keep: int, top: int, scale: float, score: str = "sigmoid",
              correction: torch.Tensor | None = None, group_rule: str = "top2", normalize: bool = True):
    """Router logits z float32 [T, >= E] (the first E columns) -> (ids int32 [T, top], weights float32 [T, top]).
    Scores s: sigmoid, or softmax over the E logits.  The choice is made by s + correction (float32 [E], optional):
    the `keep` best of `groups` equal groups of neighbouring experts, a group scored by the sum of its two best
    choice scores ("top2") or by its best ("max"); of their experts the `top` best.  weights = the chosen s (over
    their sum with `normalize`) times `scale`."""
    T = z.shape[0]
    if z.dtype != torch.float32 or z.stride(1) != 1 or z.shape[1] < E:
        raise KernelError("moe_route: float32 logits with unit column stride")
    if correction is not None and (correction.dtype != torch.float32 or correction.numel() != E or not correction.is_contiguous()):
        raise KernelError("moe_route: the correction must be contiguous float32 [E]")
    ids = torch.empty((T, top), dtype=torch.int32, device=z.device)
    weights = torch.empty((T, top), dtype=torch.float32, device=z.device)
    fn = _fn("moe", "lq_moe_route", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                                     c_void_p, c_int, c_int, c_void_p])
    _check(fn(_p(z), z.stride(0), _p(ids), _p(weights), T, E, groups, keep, top, float(scale), SCORE_FNS[score], _p(correction),
              GROUP_RULES[group_rule], int(normalize), _stream()), "moe_route")
    return ids, weights


def moe_up(h: torch.Tensor, w_up: torch.Tensor, ids: torch.Tensor, act: str | None, gated: bool = False,
           block: int = 0) -> torch.Tensor:
    """u[t, j] = act(w_up[ids[t, j]] h[t]) for w_up [E, F, D]; returns [T, top, F] in h's dtype.  gated: w_up is
    [E, 2F, D], an expert's F gate rows ahead of its F up rows (or, with `block` b, b gate rows and b up rows by turns),
    and u = act(gate rows . h) * (up rows . h).  Chosen experts numbered E and above (identity experts) have no rows;
    their u is left unwritten."""
    T, D = h.shape
    E, F, D2 = w_up.shape
    if gated:
        F //= 2
    if D2 != D or w_up.dtype != h.dtype or not w_up.is_contiguous():
        raise KernelError("moe_up: a contiguous weight [E, F, D] of the rows' dtype")
    top = ids.shape[1]
    u = torch.empty((T, top, F), dtype=h.dtype, device=h.device)
    fn = _fn("moe", "lq_moe_up_rows", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                       c_int, c_void_p])
    _check(fn(_p(_contig(h, "h")), _p(w_up), _p(ids), _p(u), dtype_code(h), T, top, D, F, MOE_ACTS[act], int(gated), E, int(block),
              _stream()), "moe_up")
    return u


def moe_down(u: torch.Tensor, w_down: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, x: torch.Tensor,
             accumulate: bool = True, shared: torch.Tensor | None = None, shared_gate: torch.Tensor | None = None,
             h: torch.Tensor | None = None, shared_scale: float = 1.0) -> torch.Tensor:
    """x[t] (+)= sum_j weights[t, j] w_down[ids[t, j]] u[t, j] (+ shared_scale * sigmoid(shared_gate[t]) * shared[t])
    for w_down [E, D, F]; x float32 [T, D]; shared float32 [T, D]; shared_gate float32 [T] (may be a strided column;
    None: the shared rows are added as they are).  h [T, D] (u's dtype): the experts' input, which a chosen expert
    numbered E or above (an identity expert) passes on times its weight."""
    T, top, F = u.shape
    E, D, F2 = w_down.shape
    if F2 != F or w_down.dtype != u.dtype or not w_down.is_contiguous() or x.dtype != torch.float32 or tuple(x.shape) != (T, D):
        raise KernelError("moe_down: a contiguous weight [E, D, F] of u's dtype and float32 rows [T, D]")
    if shared is not None and (shared.dtype != torch.float32 or tuple(shared.shape) != (T, D) or not shared.is_contiguous()):
        raise KernelError("moe_down: the shared rows must be contiguous float32 [T, D]")
    if shared_gate is not None and (shared_gate.dtype != torch.float32 or shared_gate.numel() != T):
        raise KernelError("moe_down: the shared gate must be float32 [T]")
    if h is not None and (h.dtype != u.dtype or tuple(h.shape) != (T, D) or not h.is_contiguous()):
        raise KernelError("moe_down: the experts' input must be contiguous [T, D] of u's dtype")
    fn = _fn("moe", "lq_moe_down", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int,
                                    c_int, c_int, c_int, c_int, c_void_p, c_int, c_float, c_void_p])
    _check(fn(_p(_contig(u, "u")), _p(w_down), _p(ids), _p(weights), _p(shared), _p(shared_gate),
              shared_gate.stride(0) if shared_gate is not None else 0, _p(_contig(x, "x")), int(accumulate), dtype_code(u),
              T, top, D, F, _p(h), E if h is not None else (1 << 30), float(shared_scale), _stream()), "moe_down")
    return x


# ------------------------------------------------------------------ mixers with a matrix state per head
def linear_scan(qkv: torch.Tensor, q_off: int, k_off: int, v_off: int, state: torch.Tensor, cu_rows, slots, tok_pos,
                B: int, H: int, dk: int, dv: int, q_scale: float = 1.0, k_scale: float = 1.0,
                decay: torch.Tensor | None = None, gates: tuple | None = None, rot: tuple | None = None,
                single: bool = False, in_act: str | None = None, channel_decay: tuple | None = None):
    """S_t = a_t S_(t-1) + b_t k_t v_t^T, o_t = S_t^T q_t for the rows of B sequences (rows cu_rows[b] ..
    cu_rows[b+1] of qkv belong to the sequence in slot slots[b]), from and into `state` (float32
    [slots, H, dk (+1), dv (+1)]).  decay: float32 [H] (a_t fixed, b_t = 1).  gates = (pre [rows, 2H] float32,
    bias [2H] float32, cap): exponential input gate and sigmoid forget gate with a running maximum; the state then
    has one more row (the maximum) and one more column (the normaliser).  rot = (cos, sin, dims): q and k are
    rotated as they are read.  single: every sequence brings exactly one token (the kernel then streams the
    state once, without staging chunks of tokens).  in_act "silu": q, k and v each pass through silu, in float32, as
    they are read.  channel_decay = (pre, bias, tau): a decay for every key channel and token instead of one per head,
    a_t[h, r] = sigmoid(pre[t, h * dk + r] + bias[h * dk + r])^(1 / tau), the rows of the state that belong to channel r
    decaying by it; pre is a float32 [rows, H * dk] view (rows may be strided), bias float32 [H * dk] or None.
    Returns the raw outputs float32 [rows, H, dv (+1)] and, with gates, exp(-maximum) float32 [rows, H]."""
    rows = qkv.shape[0]
    mlstm = gates is not None
    dvx, dkx = dv + int(mlstm), dk + int(mlstm)
    if state.dtype != torch.float32 or tuple(state.shape[1:]) != (H, dkx, dvx) or not state.is_contiguous():
        raise KernelError(f"linear_scan: the state must be contiguous float32 [slots, {H}, {dkx}, {dvx}]")
    if qkv.stride(1) != 1:
        raise KernelError("linear_scan: rows must be contiguous")
    if (decay is not None) + (gates is not None) + (channel_decay is not None) != 1:
        raise KernelError("linear_scan takes a fixed decay, gates or channel decays: one of them")
    d_pre, d_bias, tau = channel_decay if channel_decay is not None else (None, None, 1.0)
    if d_pre is not None and (d_pre.dtype != torch.float32 or tuple(d_pre.shape) != (rows, H * dk) or d_pre.stride(1) != 1
                              or (d_bias is not None and (d_bias.dtype != torch.float32 or d_bias.numel() != H * dk))
                              or not tau > 0):
        raise KernelError("linear_scan: channel decays are float32 [rows, H * dk] with a float32 bias [H * dk] and tau > 0")
    if dk > 256:
        raise KernelError(f"linear_scan: key size {dk} exceeds 256")
    out = torch.empty((rows, H, dvx), dtype=torch.float32, device=qkv.device)
    enm = torch.empty((rows, H), dtype=torch.float32, device=qkv.device) if mlstm else None
    pre, bias, cap = gates if mlstm else (None, None, 0.0)
    if mlstm and (pre.dtype != torch.float32 or tuple(pre.shape) != (rows, 2 * H) or not pre.is_contiguous()
                  or bias.dtype != torch.float32 or bias.numel() != 2 * H):
        raise KernelError("linear_scan: gates are float32 [rows, 2H] with a float32 bias [2H]")
    if decay is not None and (decay.dtype != torch.float32 or decay.numel() != H):
        raise KernelError("linear_scan: decay must be float32 [H]")
    cos, sin, dims = rot if rot is not None else (None, None, 0)
    fn = _fn("recurrent", "lq_linear_scan", [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int,
                                             c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_float, c_float, c_void_p,
                                             c_long, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                             c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_float, c_void_p])
    _check(fn(_p(qkv), dtype_code(qkv), qkv.stride(0), q_off, k_off, v_off, _p(cos), _p(sin), int(dims), _p(tok_pos),
              _p(pre), _p(bias), float(cap), _p(decay), float(q_scale), float(k_scale), _p(state), state.stride(0),
              _p(cu_rows), _p(slots), _p(out), _p(enm), B, H, dk, dv, int(mlstm), int(single and rows == B),
              {None: 0, "silu": 1}[in_act], _p(d_pre), d_pre.stride(0) if d_pre is not None else 0, _p(d_bias), 1.0 / float(tau),
              _stream()),
           "linear_scan", 1, "linear_scan:single" if single and rows == B else None)
    return out, enm


def small_proj(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x [rows, K] . w [N, K]^T in float32 for a weight of few rows (gates): every product and sum in 32-bit,
    the order of sums fixed by K alone."""
    rows, K = x.shape
    if w.shape[1] != K:
        raise KernelError(f"small_proj: input width {K} does not match weight width {w.shape[1]}")
    if 16 * K > 200 * 1024:
        return gemm_plain(x, w, torch.float32)          # rows too wide for the kernel's shared memory: the tiled product
    out = torch.empty((rows, w.shape[0]), dtype=torch.float32, device=x.device)
    fn = _fn("recurrent", "lq_small_proj", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(_p(_contig(x, "x")), dtype_code(x), _p(_contig(w, "w")), dtype_code(w), _p(out), rows, w.shape[0], K, _stream()),
           "small_proj")
    return out


GATES = {None: 0, "sigmoid": 1, "silu": 2}


def head_norm_gate(raw: torch.Tensor, dv: int, eps: float, out_dtype: torch.dtype, exp_neg_m: torch.Tensor | None = None,
                   weight: torch.Tensor | None = None, gate: torch.Tensor | None = None, act: str | None = None) -> torch.Tensor:
    """raw float32 [rows, H, dvx] -> [rows, H * dv]: each head over its root mean square (after division by
    max(|raw[.., dv]|, exp_neg_m) + 1e-6 where exp_neg_m is given), times weight [H * dv], times act(gate)."""
    rows, H, dvx = raw.shape
    if act is not None and (gate is None or gate.dtype != out_dtype or gate.shape != (rows, H * dv) or gate.stride(1) != 1):
        raise KernelError("head_norm_gate: the gate must be [rows, H * dv] of the output's dtype with unit column stride")
    if weight is not None and (weight.dtype != torch.float32 or weight.numel() != H * dv):
        raise KernelError("head_norm_gate: the weight must be float32 [H * dv]")
    out = torch.empty((rows, H * dv), dtype=out_dtype, device=raw.device)
    fn = _fn("recurrent", "lq_head_norm_gate", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p,
                                                c_int, c_int, c_int, c_int, c_float, c_void_p])
    _check(fn(_p(_contig(raw, "raw")), dvx, _p(exp_neg_m), _p(weight), _p(gate), gate.stride(0) if gate is not None else 0,
              GATES[act], _p(out), dtype_code(out_dtype), rows, H, dv, float(eps), _stream()), "head_norm_gate")
    return out


# ------------------------------------------------------------------ bfloat16 tensor-core kernels
EPI_BF16, EPI_F32, EPI_RESID, EPI_SWIGLU = 0, 1, 2, 3
SKINNY_MAX_ROWS = 64          # most rows gemm_skinny takes
SKINNY_BEST_ROWS = int(os.environ.get("LQ_SKINNY_BEST_ROWS", "16"))         # up to here streaming W through registers beats the TMA-fed tcgen05 kernel in a step

_sm_counts: dict = {}


def sm_count(device=None) -> int:
    """Multiprocessors of the device (the current one by default)."""
    index = torch.cuda.current_device() if device is None else (torch.device(device).index or 0)
    if index not in _sm_counts:
        _sm_counts[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return _sm_counts[index]


def streams_through_registers(M: int, N: int) -> bool:
    """Whether a product of M rows with a weight of N rows goes to gemm_skinny rather than gemm_tc: up to 16 rows.
    Timed alone at 16 rows gemm_tc is the faster kernel for every weight but the square output projection
    ([28672, 4096]: 48 us against 54; the head [128256, 4096]: 167 against 211), yet a whole model runs no
    faster with it (8B shape, 16 rows, context 2,048: 4.47 ms a step with gemm_tc for every product, 4.40 with
    gemm_skinny), and 15 % slower when only the products of more than one wave of blocks take it, as the single
    timings suggest (6.11 against 5.43 ms at context 4,096): its blocks fill a multiprocessor, so nothing of the
    kernel after it overlaps with it.  From 17 rows on gemm_tc wins (17 rows: 4.50 against 5.69 ms)."""
    return M <= SKINNY_BEST_ROWS


class NormedRows:
    """Rows of an RMS norm whose 1 / rms is still to be applied, as the residual epilogue of
    gemm_skinny leaves them: `data` = residual * gain in bfloat16 [M, width]; `sums` float32
    [M, blocks], each row's sum of squares cut into column blocks; `eps` of the norm.  A product
    that reads them multiplies its result by 1 / sqrt(sum(sums) / width + eps)."""

    __slots__ = ("data", "sums", "eps")

    def __init__(self, data: torch.Tensor, sums: torch.Tensor, eps: float):
        self.data, self.sums, self.eps = data, sums, float(eps)

    @property
    def shape(self):
        return self.data.shape

    @property
    def dtype(self):
        return self.data.dtype

    def finish(self) -> torch.Tensor:
        """The normalised rows themselves (for an operation that cannot take them unfinished)."""
        scale = torch.rsqrt(self.sums.sum(dim=1, keepdim=True) / self.data.shape[1] + self.eps)
        return (self.data.to(torch.float32) * scale).to(self.data.dtype)


def _norm_in(a):
    """(tensor, sums pointer, blocks, 1 / width, eps) of plain or unfinished rows."""
    if isinstance(a, NormedRows):
        if a.sums.dtype != torch.float32 or a.sums.shape[0] != a.data.shape[0] or not a.sums.is_contiguous():
            raise KernelError("unfinished rows: sums must be contiguous float32 [rows, blocks]")
        return a.data, _p(a.sums), a.sums.shape[1], 1.0 / a.data.shape[1], a.eps
    return a, None, 0, 0.0, 0.0


PREFETCH_BYTES = int(float(os.environ.get("LQ_PREFETCH_MB", "8")) * (1 << 20))   # of the weights read next; 0: none


# The same, asked by the decode attention, which leaves HBM a third idle: all of a 34 MB output projection
# (measured: a decode step 0.8 % shorter than with 8 MB).
PREFETCH_BYTES_ATTN = int(float(os.environ.get("LQ_PREFETCH_ATTN_MB", "48")) * (1 << 20))


def _next(next_w, limit=None):
    """(pointer, bytes) of the piece of the next weights to ask into L2."""
    limit = PREFETCH_BYTES if limit is None else limit
    if next_w is None or limit <= 0:
        return None, 0
    return _p(next_w), min(limit, next_w.numel() * next_w.element_size())


def gemm_skinny(a, w: torch.Tensor, epi: int, residual: torch.Tensor | None = None,
                out: torch.Tensor | None = None, emit: tuple | None = None, next_w: torch.Tensor | None = None):
    """a [M <= 64, K] . w [N, K]^T, both bfloat16, streaming w once from memory.
    epi: EPI_BF16 / EPI_F32 store; EPI_RESID adds into the float32 `residual` in place;
    EPI_SWIGLU reads w as alternating blocks of 8 gate and 8 up rows and stores
    up * silu(gate) [M, N / 2].
    `a` may be NormedRows.  emit = (gain [N] float32, eps), with EPI_RESID only: also returns what the
    RMS norm with that gain makes of the new residual, as NormedRows: (residual, rows).
    next_w: the weights that the stream reads after these; their first bytes are asked into L2."""
    a, in_sums, in_blocks, in_inv, in_eps = _norm_in(a)
    M, K = a.shape
    N = w.shape[0]
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_skinny takes bfloat16 inputs")
    if w.shape[1] != K:
        raise KernelError(f"linear: input width {K} does not match weight width {w.shape[1]}")
    if M > SKINNY_MAX_ROWS or K % 8:
        raise KernelError(f"gemm_skinny: {M} rows (at most {SKINNY_MAX_ROWS}) and width {K} (a multiple of 8)")
    if epi == EPI_RESID:
        if residual is None or residual.dtype != torch.float32 or tuple(residual.shape) != (M, N):
            raise KernelError("linear: residual must be float32 [M, N]")
        out = residual
    elif out is None:
        shape = (M, N // 2) if epi == EPI_SWIGLU else (M, N)
        out = torch.empty(shape, dtype=torch.float32 if epi == EPI_F32 else torch.bfloat16, device=a.device)
    rows = None
    gain = None
    if emit is not None:
        gain, eps = emit
        if epi != EPI_RESID or gain.dtype != torch.float32 or gain.numel() != N:
            raise KernelError("gemm_skinny: rows for the next norm come with EPI_RESID and a float32 gain [N]")
        rows = NormedRows(torch.empty((M, N), dtype=torch.bfloat16, device=a.device),
                          torch.empty((M, -(-N // 16)), dtype=torch.float32, device=a.device), eps)
    fn = _fn("gemm_skinny", "lq_gemm_skinny", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                               c_void_p, c_int, c_float, c_float, c_void_p, c_void_p, c_void_p, c_void_p,
                                               c_long, c_void_p])
    next_p, next_n = _next(next_w)
    _check(fn(_p(_contig(a, "a")), _p(_contig(w, "w")), _p(out), _p(residual), M, N, K, epi, in_sums, in_blocks, in_inv,
              in_eps, _p(gain), _p(rows.data) if rows else None, _p(rows.sums) if rows else None, next_p, next_n,
              _stream()), "gemm_skinny", 1, f"gemm_skinny:rows{-(-M // 8) * 8}" + (":norm_in" if in_blocks else "")
           + (":norm_out" if rows else ""))
    return (out, rows) if emit is not None else out


def gemm_skinny_qkv(a, w: torch.Tensor, cos, sin, tok_pos, tok_seq, slots, page_table, k_pages, v_pages,
                    H: int, Hkv: int, hd: int, page_size: int, out: torch.Tensor | None = None,
                    next_w: torch.Tensor | None = None) -> torch.Tensor:
    """The q/k/v projection of at most 16 tokens with rotation and cache write in its epilogue:
    returns the rotated q [M, H*hd]; the rotated k and v are stored in each token's cache page.
    `a` may be NormedRows."""
    a, in_sums, in_blocks, in_inv, in_eps = _norm_in(a)
    M, K = a.shape
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or k_pages.dtype != torch.bfloat16:
        raise KernelError("gemm_skinny_qkv takes bfloat16 inputs and cache")
    if tuple(w.shape) != ((H + 2 * Hkv) * hd, K):
        raise KernelError(f"gemm_skinny_qkv: weight shape {tuple(w.shape)} is not [(H + 2 Hkv) hd, K]")
    if M > SKINNY_BEST_ROWS or K % 8 or hd % 16:
        raise KernelError(f"gemm_skinny_qkv: {M} rows (at most 16), width {K} (multiple of 8), head_dim {hd} (multiple of 16)")
    _check_tables("gemm_skinny_qkv", cos, sin, hd)
    if out is None:
        out = torch.empty((M, H * hd), dtype=torch.bfloat16, device=a.device)
    fn = _fn("gemm_skinny", "lq_gemm_skinny_qkv", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                                   c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                                                   c_int, c_int, c_void_p, c_int, c_float, c_float, c_void_p, c_long,
                                                   c_void_p])
    next_p, next_n = _next(next_w)
    _check(fn(_p(_contig(a, "a")), _p(_contig(w, "w")), _p(out), M, K, _p(cos), _p(sin), _p(tok_pos), _p(tok_seq),
              _p(slots), _p(page_table), page_table.stride(0), _p(k_pages), _p(v_pages), H, Hkv, hd, page_size,
              in_sums, in_blocks, in_inv, in_eps, next_p, next_n, _stream()), "gemm_skinny_qkv", 1,
           f"gemm_skinny_qkv:rows{-(-M // 8) * 8}" + (":norm_in" if in_blocks else ""))
    return out


USE_PAIRS = True        # many rows: products on pairs of SMs (tcgen05 cta_group::2) where gemm_pair takes the sizes


def gemm_pair_takes(M: int, N: int, K: int) -> bool:
    """Whether the product of these sizes runs on pairs of SMs (256 x 256 tiles fill the pairs at least once)."""
    return USE_PAIRS and bool(_fn("gemm_pair", "lq_gemm_pair_takes", [c_int, c_int, c_int])(M, N, K))


def gemm_pair_status() -> int:
    fn = build.load("gemm_pair").lq_gemm_pair_status
    fn.restype = c_int
    return int(fn())


def _gemm_tc_scratch_floats(M: int, N: int, K: int) -> int:
    fn = build.load("gemm_tc").lq_gemm_tc_scratch_floats
    fn.argtypes, fn.restype = [c_int, c_int, c_int], c_long
    return int(fn(M, N, K))


def gemm_tc(a: torch.Tensor, w: torch.Tensor, epi: int, residual: torch.Tensor | None = None,
            out: torch.Tensor | None = None) -> torch.Tensor:
    """a [M, K] . w [N, K]^T on the tcgen05 tensor cores (TMA-fed, float32 accumulation in
    tensor memory), with the epilogues of gemm_skinny.  For many rows; with few tiles (few rows
    and a narrow weight) the contraction is cut into ranges that a second kernel adds."""
    M, K = a.shape
    N = w.shape[0]
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_tc takes bfloat16 inputs")
    if w.shape[1] != K:
        raise KernelError(f"linear: input width {K} does not match weight width {w.shape[1]}")
    if K % 8:
        raise KernelError(f"gemm_tc: width {K} must be a multiple of 8 (16-byte rows for TMA)")
    if epi == EPI_RESID:
        if residual is None or residual.dtype != torch.float32 or tuple(residual.shape) != (M, N):
            raise KernelError("linear: residual must be float32 [M, N]")
        out = residual
    elif out is None:
        shape = (M, N // 2) if epi == EPI_SWIGLU else (M, N)
        out = torch.empty(shape, dtype=torch.float32 if epi == EPI_F32 else torch.bfloat16, device=a.device)
    out_cols = N // 2 if epi == EPI_SWIGLU else N
    if (gemm_pair_takes(M, N, K) and out.is_contiguous() and out.data_ptr() % 16 == 0
            and (out_cols * out.element_size()) % 16 == 0 and a.is_contiguous() and w.is_contiguous()):
        # Many rows: tiles of 256 x 256 on pairs of SMs, the output leaving by TMA.
        fn = _fn("gemm_pair", "lq_gemm_pair", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
        _check(fn(_p(a), _p(w), _p(out), _p(residual), M, N, K, epi, _stream()), "gemm_pair")
        return out
    # Few tiles (few rows, narrow weight): the kernel cuts the contraction into ranges and adds them afterwards.
    splits = int(_fn("gemm_tc", "lq_gemm_tc_splits", [c_int, c_int, c_int])(M, N, K))
    scratch = torch.empty(_gemm_tc_scratch_floats(M, N, K), dtype=torch.float32, device=a.device) if splits > 1 else None
    fn = _fn("gemm_tc", "lq_gemm_tc", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                                       c_void_p])
    _check(fn(_p(_contig(a, "a")), _p(_contig(w, "w")), _p(out), _p(residual), M, N, K, epi, _p(scratch), _stream()),
           "gemm_tc", 2 if splits > 1 else 1, "gemm_tc:split_k" if splits > 1 else ("gemm_tc:few_rows" if M <= 64 else None))
    return out


def gemm_tc_qkv(a: torch.Tensor, w: torch.Tensor, cos, sin, tok_pos, tok_seq, slots, page_table, k_pages, v_pages,
                H: int, Hkv: int, hd: int, page_size: int, out: torch.Tensor | None = None) -> torch.Tensor:
    """The q/k/v projection of many rows (or of 17 and more decoded tokens) with rotation and cache
    write in its epilogue, on the tcgen05 kernel: returns the rotated q [M, H*hd]; the rotated k and v
    are stored in each row's cache page.  head_dim 64 or 128."""
    M, K = a.shape
    N = (H + 2 * Hkv) * hd
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or k_pages.dtype != torch.bfloat16:
        raise KernelError("gemm_tc_qkv takes bfloat16 inputs and cache")
    if tuple(w.shape) != (N, K):
        raise KernelError(f"gemm_tc_qkv: weight shape {tuple(w.shape)} is not [(H + 2 Hkv) hd, K]")
    if K % 8 or hd not in (64, 128):
        raise KernelError(f"gemm_tc_qkv: width {K} (multiple of 8), head_dim {hd} (64 or 128)")
    _check_tables("gemm_tc_qkv", cos, sin, hd)
    if out is None:
        out = torch.empty((M, H * hd), dtype=torch.bfloat16, device=a.device)
    if gemm_pair_takes(M, N, K) and a.is_contiguous() and w.is_contiguous():
        fn = _fn("gemm_pair", "lq_gemm_pair_qkv", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                                   c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                                                   c_int, c_int, c_void_p])
        _check(fn(_p(a), _p(w), _p(out), M, K, _p(cos), _p(sin), _p(tok_pos), _p(tok_seq), _p(slots), _p(page_table),
                  page_table.stride(0), _p(k_pages), _p(v_pages), H, Hkv, hd, page_size, _stream()), "gemm_pair_qkv")
        return out
    splits = int(_fn("gemm_tc", "lq_gemm_tc_splits", [c_int, c_int, c_int])(M, N, K))
    scratch = torch.empty(_gemm_tc_scratch_floats(M, N, K), dtype=torch.float32, device=a.device) if splits > 1 else None
    fn = _fn("gemm_tc", "lq_gemm_tc_qkv", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                           c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
                                           c_int, c_void_p, c_void_p])
    _check(fn(_p(_contig(a, "a")), _p(_contig(w, "w")), _p(out), M, K, _p(cos), _p(sin), _p(tok_pos), _p(tok_seq),
              _p(slots), _p(page_table), page_table.stride(0), _p(k_pages), _p(v_pages), H, Hkv, hd, page_size,
              _p(scratch), _stream()), "gemm_tc_qkv", 2 if splits > 1 else 1,
           "gemm_tc_qkv:split_k" if splits > 1 else ("gemm_tc_qkv:few_rows" if M <= 64 else None))
    return out


def gemm_tc_status() -> int:
    """0, or the code of a wait inside gemm_tc that gave up (after a synchronize)."""
    fn = build.load("gemm_tc").lq_gemm_tc_status
    fn.restype = c_int
    return int(fn())


def _check_sink(sink, H: int):
    if sink is not None and (sink.dtype != torch.float32 or sink.numel() != H or not sink.is_contiguous()):
        raise KernelError("attention: sink must be contiguous float32 [H]")


def attn_prefill(q: torch.Tensor, k_pages, v_pages, page_table, slots, kv_len, query_blocks, H: int, Hkv: int, hd: int,
                 page_size: int, scale: float, window: int | None, out: torch.Tensor | None = None,
                 sink: torch.Tensor | None = None, softcap: float | None = None, keep_first: int = 0) -> torch.Tensor:
    """Causal attention of blocks of query rows over the paged bfloat16 cache (flash style:
    tensor-core products, online softmax in float32).  query_blocks = (sequence, first row,
    rows, first position) int32 tensors, one entry for each block of at most 64 rows.  softcap c: score <-
    c tanh(score / c) after the scale; keep_first n (with a window): a row's first n keys stay visible.  window: as `span`
    makes it (w positions; -n for blocks of n positions; 0 or None for all)."""
    T = q.shape[0]
    if q.dtype != torch.bfloat16 or k_pages.dtype != torch.bfloat16:
        raise KernelError("attn_prefill takes bfloat16 queries and cache")
    if hd % 16 or hd > 128 or page_size != 64:
        raise KernelError(f"attn_prefill: head_dim {hd} (multiple of 16, at most 128), page size {page_size} (64)")
    if out is None:
        out = torch.empty((T, H * hd), dtype=torch.bfloat16, device=q.device)
    qb_seq, qb_row, qb_rows, qb_pos = query_blocks
    fn = _fn("attn_prefill", "lq_attn_prefill_capped", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                                        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                                        c_int, c_int, c_float, c_int, c_void_p, c_float, c_int, c_void_p])
    _check_sink(sink, H)
    _check(fn(_p(q), q.stride(0), _p(k_pages), _p(v_pages), _p(page_table), page_table.stride(0), _p(slots), _p(kv_len),
              _p(qb_seq), _p(qb_row), _p(qb_rows), _p(qb_pos), _p(out), qb_seq.numel(), H, Hkv, hd, page_size,
              float(scale), int(window or 0), _p(sink), float(softcap or 0.0), int(keep_first if window else 0), _stream()),
           "attn_prefill")
    return out


def attn_prefill_tc(q: torch.Tensor, k_pages, v_pages, page_table, slots, kv_len, query_blocks128, H: int, Hkv: int,
                    hd: int, page_size: int, scale: float, window: int | None,
                    out: torch.Tensor | None = None, sink: torch.Tensor | None = None, softcap: float | None = None,
                    keep_first: int = 0) -> torch.Tensor:
    """attn_prefill on the tcgen05 tensor cores (TMA-fed, S and O in tensor memory): blocks of at
    most 128 query rows, head_dim 64 or 128, pages of 64 keys, a cache that is finite everywhere.  softcap and
    keep_first as in attn_prefill.  window: as `span` makes it (w positions; -n for blocks of n positions; 0 or None for all)."""
    T = q.shape[0]
    if q.dtype != torch.bfloat16 or k_pages.dtype != torch.bfloat16:
        raise KernelError("attn_prefill_tc takes bfloat16 queries and cache")
    if hd not in (64, 128) or page_size != 64:
        raise KernelError(f"attn_prefill_tc: head_dim {hd} (64 or 128) and page size {page_size} (64)")
    if out is None:
        out = torch.empty((T, H * hd), dtype=torch.bfloat16, device=q.device)
    qb_seq, qb_row, qb_rows, qb_pos = query_blocks128
    fn = _fn("attn_prefill_tc", "lq_attn_prefill_tc_capped",
             [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
              c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_float, c_int, c_void_p])
    _check_sink(sink, H)
    _check(fn(_p(q), q.stride(0), T, _p(_contig(k_pages, "k_pages")), _p(_contig(v_pages, "v_pages")), k_pages.shape[0],
              _p(page_table), page_table.stride(0), _p(slots), _p(kv_len), _p(qb_seq), _p(qb_row), _p(qb_rows), _p(qb_pos),
              _p(out), qb_seq.numel(), H, Hkv, hd, page_size, float(scale), int(window or 0), _p(sink), float(softcap or 0.0),
              int(keep_first if window else 0), _stream()), "attn_prefill_tc")
    return out


def attn_prefill_tc_status() -> int:
    fn = build.load("attn_prefill_tc").lq_attn_prefill_tc_status
    fn.restype = c_int
    return int(fn())


def attn_decode(q: torch.Tensor, k_pages, v_pages, page_table, tok_pos, tok_seq, slots, H: int, Hkv: int, hd: int,
                page_size: int, scale: float, window: int | None, n_splits: int,
                out: torch.Tensor | None = None, scratch: tuple | None = None,
                next_w: torch.Tensor | None = None, early_loads: bool = False,
                work: torch.Tensor | None = None, teams: int = 0, sink: torch.Tensor | None = None,
                softcap: float | None = None, keep_first: int = 0) -> torch.Tensor:
    """Attention of single query rows over the paged bfloat16 cache, the keys of each
    sequence cut into n_splits slices that are merged afterwards.  With `work` (int32: teams + 1 offsets,
    then (token, first tile, last tile + 1, part, parts) per segment) the grid is `teams` blocks per kv
    head and row tile, each walking the segments between its offset and the next, and n_splits is the most
    parts any token has; the list must cover every tile of every token once (the kernel trusts it).  next_w: the weights that the
    stream reads after this; their first bytes are asked into L2 as the blocks finish.
    early_loads: of the keys and values a row reads, only those at its own position can have been
    written by the kernel ahead on the stream (a decode step: one new token per sequence); the kernel
    then requests the others without waiting for that kernel.  softcap c: score <- c tanh(score / c) after the
    scale.  keep_first n (with a window): a token's first n keys stay visible once its window has moved past them;
    the tiles that a work list counts are then the kept tiles ahead of the window and after them the window's.
    window: as `span` makes it (w positions; -n for blocks of n positions, whose tiles a work list counts from the
    block's first; 0 or None for all)."""
    T = q.shape[0]
    if q.dtype != torch.bfloat16 or k_pages.dtype != torch.bfloat16:
        raise KernelError("attn_decode takes bfloat16 queries and cache")
    if hd % 16 or hd > 128:
        raise KernelError(f"attn_decode: head_dim {hd} must be a multiple of 16 and at most 128")
    if out is None:
        out = torch.empty((T, H * hd), dtype=torch.bfloat16, device=q.device)
    part_o = part_ml = None
    if n_splits > 1:
        if scratch is None:
            scratch = (torch.empty(T * H * n_splits * hd, dtype=torch.float32, device=q.device),
                       torch.empty(T * H * n_splits * 2, dtype=torch.float32, device=q.device))
        part_o, part_ml = scratch
        if part_o.numel() < T * H * n_splits * hd or part_ml.numel() < T * H * n_splits * 2:
            raise KernelError("attn_decode: scratch too small")
    counters = None
    if n_splits > 1:
        n_counters = T * Hkv * -(-(H // Hkv) // 16)
        counters = _attn_counters(q.device)
        if n_counters > counters.numel():
            if work is not None:
                raise KernelError("attn_decode: more (token, kv head) pairs than counters for a work list")
            counters = None          # more (token, kv head) pairs than counters: merge with the second kernel
    if work is not None and (work.dtype != torch.int32 or not work.is_contiguous() or teams < 1
                             or work.numel() < teams + 1 + 5 * T):
        raise KernelError("attn_decode: the work list must be int32 with teams + 1 offsets and at least a segment per token")
    _check_sink(sink, H)
    fn = _fn("attn_decode", "lq_attn_decode_capped", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                                      c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                                      c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_int,
                                                      c_void_p, c_long, c_int, c_void_p, c_float, c_int, c_void_p])
    next_p, next_n = _next(next_w, PREFETCH_BYTES_ATTN)
    _check(fn(_p(q), q.stride(0), _p(k_pages), _p(v_pages), _p(page_table), page_table.stride(0), _p(tok_pos),
              _p(tok_seq), _p(slots), _p(part_o), _p(part_ml), _p(counters), _p(out), T, H, Hkv, hd, page_size,
              float(scale), int(window or 0), n_splits, _p(work), int(teams), next_p, next_n, int(early_loads), _p(sink),
              float(softcap or 0.0), int(keep_first if window else 0), _stream()),
           "attn_decode", 2 if n_splits > 1 and counters is None else 1,
           "attn_decode:teams" if work is not None else "attn_decode:one_slice" if n_splits == 1 else "attn_decode:slices")
    return out


_counters: dict = {}


def _attn_counters(device) -> torch.Tensor:
    """The counters by which the last block of a (token, kv head) finds out that it is the last:
    zero between calls (the kernel resets what it used), one buffer per device."""
    key = (device.type, device.index)
    if key not in _counters:
        _counters[key] = torch.zeros(1 << 16, dtype=torch.int32, device=device)
    return _counters[key]
