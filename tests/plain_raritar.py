"""Plain, slow Raritar decoder: the oracle that the engine tests of this design compare with.

Whole sequences, no cache, no batching, one function for each mechanism, float64 by
default, a loop over positions for every attention row and every routed token.  It
shares no code with the product: config.json is read as a plain dict, safetensors with
its own few lines, and every formula is written out here.

The design, in this file's notation (h: what a mixer or feed-forward reads, x: the residual
stream, t: a position counted from 0, m: the residual multiplier):

  embedding     x_t = E[tok_t] + B[(tok_(t-1) * a + tok_t * b) mod n]; B's last row (number n) for t = 0
  norm(x; g)    x / sqrt(mean(x^2) + eps) * g, g one number
  layer         h = norm1(x);  h <- h + conv(h);  x += m * mixer(h);  x += m * ffn(norm2(x))   (ffn may be absent)
  conv(h)_t     sum_j c[:, j] * h_(t - taps + 1 + j), rows before the sequence's start are zero
  attention     grouped queries; interleaved pairs (2i, 2i + 1) of the first r dimensions rotated by t * f_i, the
                frequencies rescaled by wavelength; each value head divided by its root mean square; scores
                times a given scale, then c * tanh(score / c); position t sees j <= t with t - j < window or
                j < kept; softmax; W_o.  A layer may read another layer's keys and values with its own queries.
  routed ffn    softmax router; choice by score + correction among the experts of the best groups (a group's
                score: its best choice score); weights are the plain scores of the chosen, not renormalised;
                experts W_down (silu(W_gate h) * (W_up h)); the last router outputs are identity experts (h itself);
                a shared expert of the same form for every token, times sigmoid(w_sg . h)
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
    """An activation as the engine would keep it between two operations."""
    return x if _STORAGE is None else x.to(_STORAGE).to(x.dtype)


def scalar_norm(x: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * g


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def embed(tokens, table: torch.Tensor, bigram: torch.Tensor | None, hashing: dict | None) -> torch.Tensor:
    if hashing is None:
        return torch.stack([table[int(tok)] for tok in tokens])
    n, a, b = int(hashing["buckets"]), int(hashing["mul_prev"]), int(hashing["mul_cur"])
    rows = []
    for t, tok in enumerate(tokens):
        row = n if t == 0 else (int(tokens[t - 1]) * a + int(tok) * b) % n
        rows.append(table[int(tok)] + bigram[row])
    return torch.stack(rows)


def causal_conv(h: torch.Tensor, c: torch.Tensor) -> torch.Tensor:
    """conv(h)_t = sum_j c[:, j] * h_(t - taps + 1 + j); c is [width, taps]."""
    T, taps = h.shape[0], c.shape[1]
    out = torch.zeros_like(h)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += c[:, j] * h[s]
    return out


def scaled_frequencies(dims: int, base: float, scaling: dict | None) -> torch.Tensor:
    f = torch.tensor([float(base) ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
    if not scaling:
        return f
    factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    out = []
    for fi in f.tolist():
        wave = 2.0 * math.pi / fi
        if wave < original / high:
            out.append(fi)
        elif wave > original / low:
            out.append(fi / factor)
        else:
            s = (original / wave - low) / (high - low)
            out.append((1.0 - s) * fi / factor + s * fi)
    return torch.tensor(out, dtype=torch.float64)


def rotate_pairs(x: torch.Tensor, pos: int, freqs: torch.Tensor) -> torch.Tensor:
    """x [..., d]: the pairs (2i, 2i + 1) for i < len(freqs) turned by pos * f_i; the rest unchanged."""
    out = x.clone()
    ang = (pos * freqs).to(x.dtype)
    cos, sin = torch.cos(ang), torch.sin(ang)
    r = 2 * len(freqs)
    u, v = x[..., 0:r:2], x[..., 1:r:2]
    out[..., 0:r:2] = u * cos - v * sin
    out[..., 1:r:2] = v * cos + u * sin
    return out


def visible(i: int, j: int, mask: dict | None) -> bool:
    if j > i:
        return False
    if not mask:
        return True
    return i - j < int(mask["size"]) or j < int(mask.get("keep_first", 0))


def keys_and_values(h: torch.Tensor, w: dict, m: dict, eps: float):
    """Rotated keys [T, G, dim] and normed values [T, G, vdim] of a layer that has projections of its own."""
    T = h.shape[0]
    G, dim, vdim = int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    rot = m.get("rot")
    freqs = scaled_frequencies(int(rot["dims"]), float(rot["base"]), rot.get("scaling")) if rot and int(rot["dims"]) else None
    k = _st(h @ w["k"].T).reshape(T, G, dim)
    v = _st(h @ w["v"].T).reshape(T, G, vdim)
    if freqs is not None:
        k = torch.stack([rotate_pairs(k[t], t, freqs) for t in range(T)])
    return _st(k), _st(unit_rms(v, eps))


def attention(h: torch.Tensor, w: dict, m: dict, eps: float, kv=None) -> torch.Tensor:
    """kv: (keys, values) of the layer whose cache this layer reads; None: its own."""
    T = h.shape[0]
    H, G, dim, vdim = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    rot = m.get("rot")
    freqs = scaled_frequencies(int(rot["dims"]), float(rot["base"]), rot.get("scaling")) if rot and int(rot["dims"]) else None
    k, v = kv if kv is not None else keys_and_values(h, w, m, eps)
    q = _st(h @ w["q"].T).reshape(T, H, dim)
    if freqs is not None:
        q = _st(torch.stack([rotate_pairs(q[t], t, freqs) for t in range(T)]))
    scale, cap = float(m["scale"]), m.get("softcap")
    out = torch.zeros(T, H, vdim, dtype=h.dtype)
    for i in range(T):
        js = [j for j in range(i + 1) if visible(i, j, m.get("mask"))]
        for hh in range(H):
            g = hh // (H // G)
            s = (k[js, g] @ q[i, hh]) * scale
            if cap:
                s = float(cap) * torch.tanh(s / float(cap))
            p = torch.softmax(s, dim=0)
            out[i, hh] = p @ v[js, g]
    return _st(out.reshape(T, H * vdim)) @ w["o"].T


def gated_expert(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    return _st(silu(h @ gate.T) * (h @ up.T)) @ down.T


def route(scores: torch.Tensor, correction: torch.Tensor, router: dict):
    """scores [n] (softmax over real and identity experts together).  Returns the chosen indices, best first."""
    n, top = scores.shape[0], int(router["top"])
    groups = router.get("groups") or {"count": 1, "keep": 1}
    count, keep = int(groups["count"]), int(groups["keep"])
    per = n // count
    choice = scores + correction
    group_score = [max(float(choice[g * per + i]) for i in range(per)) for g in range(count)]
    kept = sorted(range(count), key=lambda g: (-group_score[g], g))[:keep]
    allowed = [e for e in range(n) if e // per in kept]
    allowed.sort(key=lambda e: (-float(choice[e]), e))
    return allowed[:top]


def choice_margin(scores: torch.Tensor, correction: torch.Tensor, router: dict) -> float:
    """How far the choice is from tipping: the smallest gap between something taken and something left, over the
    kept groups' edge and the chosen experts' edge."""
    n, top = scores.shape[0], int(router["top"])
    groups = router.get("groups") or {"count": 1, "keep": 1}
    count, keep = int(groups["count"]), int(groups["keep"])
    per = n // count
    choice = (scores + correction).tolist()
    gs = sorted((max(choice[g * per:(g + 1) * per]) for g in range(count)), reverse=True)
    margin = gs[keep - 1] - gs[keep] if keep < count else math.inf
    picked = route(scores, correction, router)
    kept = {e // per for e in picked} | {g for g in range(count) if max(choice[g * per:(g + 1) * per]) >= gs[keep - 1]}
    rest = [choice[e] for e in range(n) if e // per in kept and e not in picked]
    if rest:
        margin = min(margin, min(choice[e] for e in picked) - max(rest))
    return margin


def routed_ffn(h: torch.Tensor, w: dict, mlp: dict, margins: list | None = None) -> torch.Tensor:
    router = mlp["router"]
    n_real, n_id = int(router["experts"]), int(router.get("identity", 0))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        z = h[t] @ w["router"].T
        s = torch.softmax(z, dim=0)
        corr = w["correction"].to(h.dtype) if "correction" in w else torch.zeros_like(s)
        if margins is not None:
            margins.append(choice_margin(s, corr, router))
        for e in route(s, corr, router):
            if e >= n_real:
                out[t] += s[e] * h[t]
            else:
                out[t] += s[e] * gated_expert(h[t], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"])
        if mlp.get("shared"):
            g = torch.sigmoid((h[t] * w["shared.sg"][0]).sum())
            out[t] += g * gated_expert(h[t], w["shared.gate"], w["shared.up"], w["shared.down"])
    assert n_real + n_id == w["router"].shape[0]
    return out


# --------------------------------------------------------------------------- the model

def _sub(weights: dict, prefix: str, dtype) -> dict:
    return {k[len(prefix):]: v.to(dtype) for k, v in weights.items() if k.startswith(prefix)}


def forward(cfg: dict, weights: dict, tokens, dtype=torch.float64, storage=None, layers_out: list | None = None,
            margins: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.  `storage`: keep activations between operations in that dtype (what
    a reduced-precision engine does) while everything else stays in `dtype`; the distance of such a run from the
    exact one is the yardstick for the engine's own distance.  layers_out: the stream after every layer.  margins:
    every routed token's choice margin, layer after layer."""
    global _STORAGE
    _STORAGE = storage
    try:
        eps, m = float(cfg["norm"]["eps"]), float(cfg.get("residual_mult", 1.0))
        hashing = (cfg.get("embedding") or {}).get("bigram")
        x = embed(tokens, weights["embed"].to(dtype), weights["bigram"].to(dtype) if hashing else None, hashing)
        kv = {}
        for i, layer in enumerate(cfg["layers"]):
            pre = f"l{i}."
            h = _st(scalar_norm(x, weights[pre + "norm1"].to(dtype), eps))
            if pre + "canon1" in weights:
                h = _st(h + causal_conv(h, weights[pre + "canon1"].to(dtype)))
            mix, wm = layer["mixer"], _sub(weights, pre + "mix.", dtype)
            if layer["type"] != "attention":
                raise ValueError(f"layer {i}: unknown mixer {layer['type']!r}")
            if mix.get("kv_from") is None:
                kv[i] = keys_and_values(h, wm, mix, eps)
                y = attention(h, wm, mix, eps, kv[i])
            else:
                y = attention(h, wm, mix, eps, kv[int(mix["kv_from"])])
            x = x + m * y
            if layer.get("mlp") is not None:
                h = _st(scalar_norm(x, weights[pre + "norm2"].to(dtype), eps))
                x = x + m * routed_ffn(h, _sub(weights, pre + "mlp.", dtype), layer["mlp"], margins)
            if layers_out is not None:
                layers_out.append(x.clone())
        h = _st(scalar_norm(x, weights["final.norm"].to(dtype), eps))
        return h @ weights["head"].to(dtype).T
    finally:
        _STORAGE = None


def greedy(cfg: dict, weights: dict, prompt, n_new: int) -> list[int]:
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(forward(cfg, weights, toks)[-1].argmax()))
    return toks[len(prompt):]
