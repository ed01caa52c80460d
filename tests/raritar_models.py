"""Small Raritar configurations and model folders with random weights, for the tests of this design.

The configurations differ from each other in every size and option: windows of 5, 20, 33, 64 and 100 tokens and no
window; kept first positions of 0, 1, 3, 5, 64 and 70 (fewer and more than a window, exactly a page, more than a page);
rotation of all and of a part of a head, with and without rescaled frequencies (ranges that leave all, some and none
of the frequencies alone); values wider and narrower than keys; one and several key heads; caps and none; layers that
read the keys and values of another layer through a longer and a shorter window than its own; convolutions of 1 to 5
taps and none; pair-hash embeddings with small and large multipliers and none; branch multipliers of 0.25 to 1.5 and
none; routers with 0 to 3 identity outputs, 1 to 4 groups of which some or all are kept, 1 to 4 experts per token, with
and without a shared expert; layers without a feed-forward; a width that is no multiple of 8.
"""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch

import plain_raritar


def attn(heads, kv_heads, dim, vdim, window=None, keep=0, rot=None, scale=None, cap=None, kv_from=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5 if scale is None else scale}
    if window is not None:
        m["mask"] = {"size": window, "keep_first": keep}
    if rot is not None:
        m["rot"] = rot
    if cap is not None:
        m["softcap"] = cap
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": mlp}


def moe(experts, top, ff, identity=0, groups=None, shared=None):
    router = {"experts": experts, "top": top, "identity": identity}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    out = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


def model(width, vocab, layers, eps=1e-5, mult=None, taps=None, bigram=None):
    out = {"architecture": "Raritar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if mult is not None:
        out["residual_mult"] = mult
    if taps is not None:
        out["canon"] = {"taps": taps}
    if bigram is not None:
        out["embedding"] = {"bigram": {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}}
    return out


SCALED_A = {"dims": 8, "base": 10000.0, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}}
SCALED_B = {"dims": 48, "base": 5e5, "scaling": {"factor": 16.0, "low": 2.0, "high": 8.0, "original": 256}}
ROT_ALL = {"dims": 32, "base": 300.0}
MOE_A = moe(6, 3, 32, identity=2, groups=(4, 2), shared=48)
MOE_W = moe(13, 4, 48, identity=3, groups=(4, 3), shared=64)

CONFIGS = {
    # every option at once; layer 2 reads layer 0's keys through a longer window (100 against 33) and keeps fewer first
    # positions, layer 4 reads layer 1's (no window) through a window of 20
    "mixed": model(64, 200, [
        attn(4, 2, 16, 24, window=33, keep=5, rot=SCALED_A, scale=0.3, cap=20.0, mlp=MOE_A),
        attn(2, 1, 32, 32, rot=ROT_ALL, mlp=None),
        attn(6, 2, 16, 24, window=100, keep=2, rot=SCALED_A, scale=0.2, cap=8.0, kv_from=0, mlp=moe(4, 1, 40)),
        attn(3, 3, 8, 8, window=5, keep=0, mlp=moe(5, 2, 24, identity=1, groups=(2, 2))),
        attn(2, 1, 32, 32, window=20, keep=3, rot=ROT_ALL, cap=30.0, kv_from=1, mlp=MOE_A),
    ], eps=1e-6, mult=0.7, taps=3, bigram=(97, 5, 3)),
    # one head, a width that is no multiple of 8, no multiplier, no convolution, no second table: the layers whose
    # norms fold into the products on either side
    "odd": model(100, 131, [
        attn(1, 1, 12, 20, window=7, keep=1, rot={"dims": 8, "base": 300.0}, mlp=moe(3, 3, 24, shared=16)),
        attn(1, 1, 12, 20, rot={"dims": 12, "base": 50.0}, cap=5.0, mlp=None),
        attn(5, 1, 12, 20, window=64, keep=70, rot={"dims": 12, "base": 50.0}, kv_from=1, mlp=moe(2, 1, 16, identity=2, groups=(2, 1))),
    ]),
    # sizes near those of real layers, small: heads of 64 and 128 that the tensor-core kernels take, a window and kept
    # positions of exactly one page, sixteen router outputs in four groups
    "wide": model(128, 300, [
        attn(8, 2, 64, 64, window=64, keep=64, rot=SCALED_B, scale=0.11, cap=30.0, mlp=MOE_W),
        attn(2, 1, 128, 128, window=100, keep=3, rot={"dims": 64, "base": 1e4}, cap=50.0, mlp=MOE_W),
        attn(4, 2, 64, 64, window=40, keep=70, rot=SCALED_B, scale=0.2, kv_from=0, mlp=MOE_W),
    ], mult=0.5, taps=4, bigram=(2039, 1000003, 999983)),
    # each mechanism behind as little else as the design allows
    "only_attention": model(48, 90, [attn(4, 2, 16, 16, window=20, keep=3, rot={"dims": 8, "base": 100.0, "scaling": {
        "factor": 2.0, "low": 1.0, "high": 2.0, "original": 32}}, scale=0.4, cap=10.0)]),
    "only_attention_full": model(48, 90, [attn(2, 2, 16, 8, rot={"dims": 4, "base": 50.0}, cap=3.0)]),
    "only_attention_bare": model(48, 90, [attn(2, 1, 16, 16, window=20, keep=3, scale=1.0)]),
    "only_shared_keys": model(40, 70, [attn(2, 1, 8, 12, window=9, keep=2, rot={"dims": 8, "base": 20.0}),
                                       attn(4, 1, 8, 12, window=30, keep=0, rot={"dims": 8, "base": 20.0}, cap=4.0, kv_from=0)]),
    "only_conv": model(40, 70, [attn(1, 1, 8, 8)], taps=5),
    "only_conv_one_tap": model(40, 70, [attn(1, 1, 8, 8)], taps=1, mult=1.5),
    "only_pairs": model(40, 70, [attn(1, 1, 8, 8)], bigram=(7, 1, 1)),
    "only_multiplier": model(40, 70, [attn(1, 1, 8, 8, mlp=moe(2, 1, 8))], mult=0.25),
    "only_moe": model(40, 70, [attn(1, 1, 8, 8, mlp=moe(7, 2, 16, identity=1, groups=(4, 1), shared=24))]),
    "only_moe_plain": model(40, 70, [attn(1, 1, 8, 8, mlp=moe(5, 2, 16))]),
    "only_moe_identity": model(40, 70, [attn(1, 1, 8, 8, mlp=moe(1, 4, 16, identity=3, groups=(2, 2)))], mult=0.5),
}


def random_config(rng) -> dict:
    """A configuration drawn by `rng` (a random.Random): 2 to 6 layers, each with its own head counts, head sizes (also ones
    that no tensor-core kernel takes), value size, window, kept positions, rotation, cap and scale, or on an earlier layer's
    keys and values; routers with any mix of real and identity outputs, groups and choices; any taps, hashing and multiplier."""
    width, vocab = rng.choice([64, 96, 128, 192, 320]), rng.choice([257, 500, 1000])
    layers: list = []
    for _ in range(rng.randint(2, 6)):
        own = [j for j, layer in enumerate(layers) if "kv_from" not in layer["mixer"]]
        if own and rng.random() < 0.35:
            kv_from = rng.choice(own)
            src = layers[kv_from]["mixer"]
            kv, dim, vdim, rot = src["kv_heads"], src["dim"], src["vdim"], src.get("rot")
            heads = kv * rng.choice([1, 2, 4])
        else:
            kv_from = None
            heads = rng.choice([1, 2, 4, 6, 8])
            kv = rng.choice([k for k in (1, 2, 3, 4, 8) if heads % k == 0])
            dim = rng.choice([16, 32, 48, 64, 64, 80, 96, 128])
            vdim = rng.choice([dim, dim, dim, dim // 2, dim + 16])
            rotated = rng.choice([0, dim // 2 // 2 * 2, dim])
            rot = None
            if rotated:
                rot = {"dims": rotated, "base": rng.choice([100.0, 10000.0, 5e5])}
                if rng.random() < 0.6:
                    rot["scaling"] = {"factor": rng.choice([2.0, 8.0, 32.0]), "low": 1.0, "high": rng.choice([2.0, 4.0]),
                                      "original": rng.choice([16, 64, 1024])}
        window = rng.choice([None, 8, 24, 44, 64, 100])
        mlp = None
        if rng.random() < 0.8:
            groups, per = rng.choice([1, 2, 4]), rng.choice([1, 2, 3, 4])
            identity = min(rng.choice([0, 0, 1, 2, 4]), groups * per - 1)
            kept = rng.randint(1, groups)
            mlp = moe(groups * per - identity, rng.randint(1, min(kept * per, 4)), rng.choice([16, 24, 40, 64]), identity=identity,
                      groups=(groups, kept) if groups > 1 else None, shared=rng.choice([None, 32, 96]))
        layers.append(attn(heads, kv, dim, vdim, window=window, keep=rng.choice([0, 1, 4, 9, 64]) if window else 0, rot=rot,
                           scale=rng.choice([dim ** -0.5, 0.1, 0.2]), cap=rng.choice([None, 10.0, 30.0]), kv_from=kv_from, mlp=mlp))
    return model(width, vocab, layers, eps=rng.choice([1e-5, 1e-6]), mult=rng.choice([None, 0.5, 0.7, 1.3]),
                 taps=rng.choice([None, 2, 3, 4]),
                 bigram=rng.choice([None, (rng.choice([97, 509, 4099]), rng.randint(1, 100), rng.randint(1, 100))]))


def make_folder(tmp, name, seed: int = 0, std: float = 0.1, gain_std: float = 0.2, dtype=torch.bfloat16) -> Path:
    """A model folder with random weights, written by the framework's random-weights mode."""
    import longbow_quarrel_b200  # noqa: F401
    from longbow_quarrel_b200 import architectures  # noqa: F401
    from longbow_quarrel_b200.config import architecture_of
    from longbow_quarrel_b200.engine.model import Model
    from longbow_quarrel_b200.parts.base import Runtime
    from longbow_quarrel_b200.weights import write_random_model
    data = CONFIGS[name] if isinstance(name, str) else name
    arch = architecture_of(data)
    cfg = arch.config_from_dict(data)
    table = Model(arch.describe(cfg), Runtime(torch.device("cpu"), torch.float32, 64)).weight_table()
    label = name if isinstance(name, str) else "custom"
    return write_random_model(Path(tmp) / f"raritar_{label}_{seed}", cfg.to_dict(), table, seed, dtype, std, gain_std)


def tokens(n: int, vocab: int, seed: int) -> list[int]:
    return [int(t) for t in np.random.default_rng(seed).integers(0, vocab, size=n)]


def row_errors(got: np.ndarray, ref: np.ndarray) -> np.ndarray:
    """Per row: root mean square of the difference over the root mean square of the reference row."""
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert np.isfinite(got).all(), "non-finite logits"
    return np.sqrt(((got - ref) ** 2).mean(-1)) / np.maximum(np.sqrt((ref ** 2).mean(-1)), 1e-30)


F32_TOL = 2e-5        # the floor of every float32 bound, per row


def bound(dtype: str, cfg: dict, weights: dict, toks, exact: np.ndarray) -> float:
    """What a row may differ by from the float64 plain implementation, measured on the request itself: three times
    what the plain implementation moves by when it runs in float32 (at least 2e-5), or when it keeps its
    activations in bfloat16.  Both take the request's worst row."""
    if dtype == "float32":
        single = plain_raritar.forward(cfg, weights, toks, dtype=torch.float32).numpy()
        return max(F32_TOL, 3.0 * float(row_errors(single, exact).max()))
    stored = plain_raritar.forward(cfg, weights, toks, storage=torch.bfloat16).numpy()
    return 3.0 * float(row_errors(stored, exact).max())


def load(folder):
    return json.loads((Path(folder) / "config.json").read_text()), plain_raritar.read_safetensors(Path(folder) / "model.safetensors")


CLOSE_CALL = 0.004     # in score (a softmax over a few outputs): rounding in bfloat16 moves a router's scores by less


def firm_rows(dtype: str, cfg: dict, weights: dict, toks) -> np.ndarray:
    """Which positions' logits a bfloat16 run can be held to: those where no router's choice is a close call.  Where two
    experts (or two groups) score within CLOSE_CALL of each other at the edge of the choice, rounding decides which
    one is taken, and the row that follows is another row; both are right.  float32: every position."""
    firm = np.ones(len(toks), dtype=bool)
    if dtype != "float32":
        margins: list = []
        plain_raritar.forward(cfg, weights, toks, margins=margins)
        per_layer = np.asarray(margins, dtype=np.float64).reshape(-1, len(toks)) if margins else np.zeros((0, len(toks)))
        for m in per_layer:
            firm &= m >= CLOSE_CALL
    return firm
