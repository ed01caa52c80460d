"""Plain, slow Lavutar decoder: the oracle that the engine tests of this design compare with.

Whole sequences, no cache, no batching, one function for each mechanism, float64 by
default, a loop over positions for every attention row, every recurrent step and every
routed token.  It shares no code with the product: config.json is read as a plain dict,
safetensors with its own few lines, and every formula is written out here.

The design, in this file's notation (h: what a mixer or feed-forward reads, x: the residual
stream, e: the embedding's output, t: a position counted from 0):

  embedding     e_t = E[tok_t]
  norm(x; g, b) (x - mean(x)) / sqrt(mean((x - mean(x))^2) + eps) * g + b
  layer         x += mixer(norm1(x));  x += ffn(norm2(x))   (ffn may be absent)
  order         layers start .. stop - 1 run `times` times in a row with the same weights; ahead of the first
                layer of every such pass  x <- W_in [x; e]
  attention     grouped queries, values of their own size.  Options: the first r dimensions of q and k rotated
                in pairs (i, i + r/2) with frequencies blended between f_i and f_i / factor, cos and sin times
                0.1 ln(factor) + 1; q and k over their root mean square per head (no weight) or over the whole
                projection (with a weight); q times 1 + c ln(floor((t + 1) / n) + 1); scores times a given
                scale, then cap tanh(score / cap); position t sees j <= t, or only j > t - w (window), or only
                j in t's block of w positions (chunk); softmax whose denominator may hold one more term, 1 or
                exp(s_head); the heads times sigmoid(W_g h), one gate per value or one per head; W_o
  gated linear  S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T (q_t dim^-1/2), a_t = sigmoid(W_a2 W_a1 h + b)^(1/tau)
  attention     per key channel; each head's o over its root mean square times a weight shared by the heads, times
                silu(W_g h); W_o
  parallel      l * attention(h) + r * gated linear attention(h)
  dense ffn     W_down (gelu_tanh(W_gate h) * (W_up h))
  routed ffn    the `top` largest router logits choose the experts, their softmax (over the chosen alone) weighs
                them; experts W_down (silu(W_gate h) * (W_up h))
  output        final norm, logits = W_head x
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch

_ST = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "I32": torch.int32, "I64": torch.int64,
       "F64": torch.float64}


def read_safetensors(path) -> dict[str, torch.Tensor]:
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        dt = _ST[info["dtype"]]
        t = torch.frombuffer(bytearray(raw[8 + n + lo:8 + n + hi]), dtype=dt) if hi > lo else torch.empty(0, dtype=dt)
        out[name] = t.reshape(info["shape"]).clone()
    return out


def load_folder(folder):
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), read_safetensors(folder / "model.safetensors")


# --------------------------------------------------------------------------- small pieces

_STORAGE = None        # set by forward(storage=...): the dtype in which activations are kept between operations


def _st(x: torch.Tensor) -> torch.Tensor:
    """What a tensor looks like after it was stored in the storage dtype between two operations."""
    return x if _STORAGE is None else x.to(_STORAGE).to(x.dtype)


def layer_norm(x: torch.Tensor, g: torch.Tensor, b: torch.Tensor, eps: float) -> torch.Tensor:
    mean = x.mean(dim=-1, keepdim=True)
    var = ((x - mean) ** 2).mean(dim=-1, keepdim=True)
    return _st((x - mean) / torch.sqrt(var + eps) * g + b)


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def sigmoid(z: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-z))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * sigmoid(z)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def blended_frequencies(rot: dict) -> tuple[torch.Tensor, float]:
    """Frequencies of the rotated pairs and the factor on cos and sin."""
    dims, base = rot["dims"], float(rot["base"])
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
    s = rot.get("scaling")
    if not s:
        return f, 1.0
    factor, original = float(s["factor"]), float(s["original"])

    def turn(t):
        return dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(base))
    lo = max(math.floor(turn(float(s["fast"]))), 0)
    hi = min(math.ceil(turn(float(s["slow"]))), dims - 1)
    ramp = torch.tensor([min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(dims // 2)], dtype=torch.float64)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_halves(x: torch.Tensor, pos: int, rot: dict) -> torch.Tensor:
    """x [heads, dim] at position pos: pairs (i, i + dims/2) of the first dims dimensions turn by pos * f_i."""
    f, mag = blended_frequencies(rot)
    dims = rot["dims"]
    a = (pos * f).to(x.dtype)
    c, s = torch.cos(a) * mag, torch.sin(a) * mag
    u, v = x[:, :dims // 2], x[:, dims // 2:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[:, dims:]], dim=1)


def visible(i: int, j: int, m: dict, kind: str) -> bool:
    if j > i:
        return False
    size = (m.get("mask") or {}).get("size")
    if size is None:
        return True
    if kind == "attention_2":
        return i // size == j // size          # blocks counted from the sequence's first position
    return i - j < size


# --------------------------------------------------------------------------- attention in its three forms

def queries_keys_values(h: torch.Tensor, w: dict, m: dict, eps: float, kind: str):
    """q [T, H, dim], k [T, G, dim], v [T, G, vdim] as the scores read them."""
    T = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = h @ w["q"].T, h @ w["k"].T, h @ w["v"].T
    if kind == "attention_2":                               # one norm over the whole projection, with a weight
        q = unit_rms(q, eps) * w["q.norm"]
        k = unit_rms(k, eps) * w["k.norm"]
    q, k, v = q.reshape(T, H, dim), k.reshape(T, G, dim), _st(v).reshape(T, G, vdim)
    if kind == "left":                                      # per head, no weight
        q, k = unit_rms(q, eps), unit_rms(k, eps)
        qt = m.get("q_temp")
        if qt:
            for t in range(T):
                q[t] = q[t] * (1.0 + qt["coef"] * math.log(math.floor((t + 1) / qt["every"]) + 1.0))
    if m.get("rot"):
        q = torch.stack([rotate_halves(q[t], t, m["rot"]) for t in range(T)])
        k = torch.stack([rotate_halves(k[t], t, m["rot"]) for t in range(T)])
    return _st(q), _st(k), v


def attention(h: torch.Tensor, w: dict, m: dict, eps: float, kind: str) -> torch.Tensor:
    """kind: "attention" (rotation, window, one more 1 in the denominator), "attention_2" (whole-projection norms, capped
    scores, chunks, a learned term in the denominator, a gate per head), "left" (per-head norms, query temperature,
    all earlier positions, a gate per value)."""
    T = h.shape[0]
    H, G, vdim = m["heads"], m["kv_heads"], m["vdim"]
    q, k, v = queries_keys_values(h, w, m, eps, kind)
    cap = m.get("softcap")
    out = torch.zeros(T, H, vdim, dtype=h.dtype)
    for t in range(T):
        keys = [j for j in range(t + 1) if visible(t, j, m, kind)]
        for head in range(H):
            g = head // (H // G)
            s = torch.stack([q[t, head] @ k[j, g] for j in keys]) * m["scale"]
            if cap:
                s = cap * torch.tanh(s / cap)
            extra = None
            if kind == "attention":
                extra = torch.zeros((), dtype=h.dtype)
            elif kind == "attention_2":
                extra = w["sink"][head]
            top = s.max() if extra is None else torch.maximum(s.max(), extra)
            e = torch.exp(s - top)
            den = e.sum() + (torch.exp(extra - top) if extra is not None else 0.0)
            p = e / den
            out[t, head] = sum(p[n] * v[j, g] for n, j in enumerate(keys))
    if kind == "left":
        out = out * sigmoid(h @ w["g"].T).reshape(T, H, vdim)
    elif kind == "attention_2":
        out = out * sigmoid(h @ w["g"].T).reshape(T, H, 1)
    return _st(out.reshape(T, H * vdim)) @ w["o"].T


# --------------------------------------------------------------------------- gated linear attention

def channel_decays(h: torch.Tensor, w: dict, m: dict) -> torch.Tensor:
    """a_t [T, heads, dim]: sigmoid(z)^(1/tau), z = W_a2 (W_a1 h) + b."""
    z = (h @ w["a1"].T) @ w["a2"].T + w["a2.b"]
    log_a = -torch.log1p(torch.exp(-z)) / m["tau"]             # log sigmoid(z) / tau
    return torch.exp(log_a).reshape(h.shape[0], m["heads"], m["dim"])


def gated_linear_attention(h: torch.Tensor, w: dict, m: dict, eps: float, state: list | None = None) -> torch.Tensor:
    T = h.shape[0]
    H, dim, vdim = m["heads"], m["dim"], m["vdim"]
    q = _st(h @ w["q"].T).reshape(T, H, dim) * dim ** -0.5
    k = _st(h @ w["k"].T).reshape(T, H, dim)
    v = _st(h @ w["v"].T).reshape(T, H, vdim)
    a = channel_decays(h, w, m)
    S = torch.zeros(H, dim, vdim, dtype=h.dtype)
    o = torch.zeros(T, H, vdim, dtype=h.dtype)
    for t in range(T):
        for head in range(H):
            S[head] = a[t, head][:, None] * S[head] + k[t, head][:, None] * v[t, head][None, :]
            o[t, head] = S[head].T @ q[t, head]
    if state is not None:
        state.append(S)
    o = unit_rms(o, eps) * w["norm"]
    o = o.reshape(T, H * vdim) * silu(_st(h @ w["g"].T))
    return _st(o) @ w["o"].T


def parallel_mixer(h: torch.Tensor, w: dict, m: dict, eps: float) -> torch.Tensor:
    left = attention(h, _sub(w, "left."), m["left"], eps, "left")
    right = gated_linear_attention(h, _sub(w, "right."), m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


# --------------------------------------------------------------------------- feed-forward

def dense_ffn(h: torch.Tensor, w: dict) -> torch.Tensor:
    return _st(gelu_tanh(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def route(z: torch.Tensor, top: int):
    """Chosen experts (largest logits first; the lower number wins a tie) and their weights."""
    order = sorted(range(z.numel()), key=lambda e: (-float(z[e]), e))[:top]
    chosen = z[order]
    p = torch.exp(chosen - chosen.max())
    return order, p / p.sum()


def choice_margin(z: torch.Tensor, top: int) -> float:
    """How far the last chosen logit lies above the first that is not."""
    s = torch.sort(z, descending=True).values
    return float(s[top - 1] - s[top]) if z.numel() > top else math.inf


def routed_ffn(h: torch.Tensor, w: dict, mlp: dict, margins: list | None = None) -> torch.Tensor:
    top = mlp["router"]["top"]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        z = w["router"] @ h[t]
        if margins is not None:
            margins.append(choice_margin(z, top))
        experts, weights = route(z, top)
        for e, p in zip(experts, weights):
            u = _st(silu(w[f"e{e}.gate"] @ h[t]) * (w[f"e{e}.up"] @ h[t]))
            out[t] += p * (w[f"e{e}.down"] @ u)
    return out


# --------------------------------------------------------------------------- the model

def _sub(weights: dict, prefix: str, dtype=None) -> dict:
    return {n[len(prefix):]: (t if dtype is None else t.to(dtype)) for n, t in weights.items() if n.startswith(prefix)}


def layer_order(cfg: dict) -> list[tuple[int, bool]]:
    """(layer, whether W_in comes right ahead of it) for every run of a layer."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    lo, hi, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, False) for i in range(lo)]
    for _ in range(times):
        runs += [(i, i == lo) for i in range(lo, hi)]
    return runs + [(i, False) for i in range(hi, n)]


def forward(cfg: dict, weights: dict, tokens, dtype=torch.float64, storage=None, layers_out: list | None = None,
            margins: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence.  storage: the dtype activations are kept in between operations (None: dtype).
    layers_out: receives the residual stream after every run of a layer."""
    global _STORAGE
    _STORAGE = storage
    try:
        eps = cfg["norm"]["eps"]
        W = {n: t.to(dtype) for n, t in weights.items()}
        e = W["embed"][torch.tensor(list(tokens))]
        x = e.clone()
        for i, reenter in layer_order(cfg):
            layer, w = cfg["layers"][i], _sub(W, f"l{i}.")
            if reenter:
                x = torch.cat([_st(x), e], dim=1) @ W["loop.in"].T
            h = layer_norm(x, w["norm1"], w["norm1.b"], eps)
            mix = _sub(w, "mix.")
            if layer["type"] == "parallel":
                x = x + parallel_mixer(h, mix, layer["mixer"], eps)
            else:
                x = x + attention(h, mix, layer["mixer"], eps, layer["type"])
            if layer.get("mlp"):
                h = layer_norm(x, w["norm2"], w["norm2.b"], eps)
                mlp = _sub(w, "mlp.")
                x = x + (dense_ffn(h, mlp) if layer["mlp"]["kind"] == "dense" else routed_ffn(h, mlp, layer["mlp"], margins))
            if layers_out is not None:
                layers_out.append(x.clone())
        return layer_norm(x, W["final.norm"], W["final.norm.b"], eps) @ W["head"].T
    finally:
        _STORAGE = None


def greedy(cfg: dict, weights: dict, prompt, n_new: int) -> list[int]:
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(forward(cfg, weights, toks)[-1].argmax()))
    return toks[len(prompt):]
