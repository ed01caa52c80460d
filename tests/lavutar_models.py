"""Small Lavutar configurations and model folders with random weights, for the tests of this design.

The configurations differ from each other in every size and option: windows of 5, 20, 40, 64 and 100 positions and
none; blocks of 1, 7, 24, 64, 70 and 100 positions and none; rotation of all and of a part of a head, with and without
blended frequencies (ramps that cover all, some and none of the pairs); values wider and narrower than keys; one and
several key heads in every kind of attention; caps and none; query temperatures that step every 3, 16 and 50
positions and none; decayed heads of 8 to 80 key channels with 1 to 3 heads, tau of 1 to 16 and inner sizes of 1 to 8;
side scales of 0.25 to 1.5; gated feed-forwards, experts of which 1, some or all are chosen, and layers without a
feed-forward; repeated stretches from the first layer, in the middle and to the last, once, twice and three times,
and none; widths and head sizes that are no multiples of 8.
"""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch

import plain_lavutar


def attn(heads, kv_heads, dim, vdim, window=None, rot=None, scale=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5 if scale is None else scale}
    if window is not None:
        m["mask"] = {"size": window}
    if rot is not None:
        m["rot"] = rot
    return {"type": "attention", "mixer": m, "mlp": mlp}


def attn2(heads, kv_heads, dim, vdim, block=None, cap=None, scale=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5 if scale is None else scale}
    if block is not None:
        m["mask"] = {"size": block}
    if cap is not None:
        m["softcap"] = cap
    return {"type": "attention_2", "mixer": m, "mlp": mlp}


def parallel(left, right, left_scale=1.0, right_scale=1.0, mlp=None):
    """left: (heads, kv_heads, dim, vdim, scale, (coef, every) | None); right: (heads, dim, vdim, tau, rank)."""
    h, g, dim, vdim, scale, temp = left
    lm = {"heads": h, "kv_heads": g, "dim": dim, "vdim": vdim, "scale": dim ** -0.5 if scale is None else scale}
    if temp is not None:
        lm["q_temp"] = {"coef": temp[0], "every": temp[1]}
    rh, rdim, rvdim, tau, rank = right
    return {"type": "parallel", "mlp": mlp,
            "mixer": {"left": lm, "right": {"heads": rh, "dim": rdim, "vdim": rvdim, "tau": tau, "rank": rank},
                      "left_scale": left_scale, "right_scale": right_scale}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def model(width, vocab, layers, eps=1e-5, loop=None):
    out = {"architecture": "Lavutar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if loop is not None:
        out["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return out


ROT_PART = {"dims": 8, "base": 10000.0, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}}
ROT_WIDE = {"dims": 48, "base": 5e5, "scaling": {"factor": 16.0, "original": 256, "fast": 32.0, "slow": 2.0}}
ROT_ALL = {"dims": 32, "base": 300.0}
ROT_64 = {"dims": 64, "base": 20000.0, "scaling": {"factor": 2.0, "original": 128, "fast": 16.0, "slow": 1.0}}

CONFIGS = {
    # one mechanism each
    "only_attention": model(48, 120, [attn(4, 2, 16, 24, window=20, rot=ROT_PART, scale=0.3, mlp=dense(64))]),
    "only_attention_bare": model(32, 90, [attn(2, 1, 32, 32, window=None, rot=None, mlp=None)]),
    "only_attention_tensor": model(64, 150, [attn(4, 2, 64, 64, window=40, rot=ROT_64, mlp=dense(48))]),
    "only_attention_2": model(40, 110, [attn2(4, 2, 32, 16, block=24, cap=30.0, scale=0.2, mlp=dense(56))]),
    "only_attention_2_tensor": model(64, 130, [attn2(2, 1, 64, 64, block=70, cap=None, mlp=None)]),
    "only_attention_2_open": model(40, 100, [attn2(3, 3, 24, 40, block=None, cap=8.0, mlp=None)]),
    "only_parallel": model(64, 140, [parallel((2, 1, 64, 64, None, (0.4, 16)), (2, 48, 32, 8.0, 4), 0.8, 0.5, mlp=dense(40))]),
    "only_parallel_odd": model(36, 100, [parallel((3, 3, 24, 40, 0.25, None), (3, 80, 40, 2.0, 5), 1.5, 0.25, mlp=None)]),
    "only_parallel_small": model(32, 80, [parallel((4, 2, 8, 8, None, (1.0, 3)), (1, 8, 72, 1.0, 1), 0.5, 1.25, mlp=None)]),
    "only_moe": model(32, 90, [attn(2, 1, 16, 16, mlp=moe(8, 2, 24))]),
    "only_moe_all": model(32, 90, [attn(2, 2, 16, 16, mlp=moe(3, 3, 20))]),
    "only_moe_one": model(32, 90, [attn(2, 2, 16, 16, mlp=moe(5, 1, 16))]),
    "only_loop": model(32, 90, [attn(2, 1, 16, 16, window=30, mlp=dense(40)), attn2(2, 2, 16, 8, block=7, mlp=None)], loop=(0, 2, 3)),
    "only_loop_once": model(32, 90, [attn(2, 1, 16, 16, mlp=None), attn(2, 1, 16, 16, mlp=dense(24)), attn(2, 1, 16, 16, mlp=None)],
                            loop=(1, 2, 1)),
    # whole models
    "mixed": model(64, 200, [
        attn2(4, 1, 32, 16, block=64, cap=20.0, mlp=dense(96)),
        parallel((2, 2, 32, 48, 0.2, (0.3, 50)), (2, 24, 40, 16.0, 8), 0.7, 0.6, mlp=moe(6, 2, 32)),
        attn(4, 2, 32, 32, window=40, rot=ROT_PART, scale=0.15, mlp=dense(72)),
        attn2(2, 2, 64, 64, block=100, cap=50.0, scale=0.1, mlp=moe(4, 3, 24)),
        attn(2, 1, 64, 64, window=100, rot=ROT_WIDE, mlp=moe(6, 2, 32))], loop=(1, 4, 2)),
    "odd": model(44, 131, [
        parallel((3, 1, 20, 12, None, (0.5, 16)), (2, 36, 20, 4.0, 3), 1.0, 1.0, mlp=dense(50)),
        attn(3, 3, 12, 20, window=5, rot={"dims": 4, "base": 50.0}, mlp=None),
        attn2(5, 1, 12, 12, block=1, cap=None, mlp=moe(3, 2, 12)),
        attn2(2, 2, 20, 28, block=7, cap=5.0, mlp=dense(36))], eps=1e-6, loop=(2, 4, 3)),
    "wide": model(128, 300, [
        attn(4, 1, 128, 128, window=64, rot={"dims": 128, "base": 1e4}, mlp=dense(160)),
        parallel((4, 2, 64, 64, None, (0.2, 50)), (2, 64, 64, 16.0, 8), 0.9, 0.4, mlp=moe(8, 3, 64)),
        attn2(4, 2, 64, 64, block=100, cap=30.0, mlp=dense(128))], loop=(0, 2, 2)),
}


def random_config(rng) -> dict:
    """A configuration whose sizes and options nobody chose."""
    width = rng.choice([24, 40, 56, 64, 72])

    def ffn():
        kind = rng.choice(["dense", "moe", None])
        if kind == "dense":
            return dense(rng.choice([24, 40, 64]))
        if kind == "moe":
            experts = rng.randint(2, 7)
            return moe(experts, rng.randint(1, experts), rng.choice([8, 12, 24, 32]))
        return None

    def heads():
        g = rng.randint(1, 3)
        return g * rng.randint(1, 3), g

    layers = []
    for _ in range(rng.randint(2, 5)):
        kind = rng.choice(["attention", "attention_2", "parallel"])
        h, g = heads()
        dim = rng.choice([8, 16, 24, 32, 64])
        vdim = rng.choice([dim, dim, 8, 24, 40])
        scale = rng.choice([None, 0.1, 0.25])
        if kind == "attention":
            rot = None
            if rng.random() < 0.8:
                rot = {"dims": rng.choice([d for d in (2, 4, 8, 16, dim) if d <= dim]), "base": rng.choice([100.0, 1e4, 5e5])}
                if rng.random() < 0.6:
                    rot["scaling"] = {"factor": rng.choice([2.0, 4.0, 8.0]), "original": rng.choice([32, 64, 256]),
                                      "fast": rng.choice([4.0, 16.0, 32.0]), "slow": rng.choice([0.5, 1.0, 2.0])}
            layers.append(attn(h, g, dim, vdim, window=rng.choice([None, 3, 17, 50, 64, 90]), rot=rot, scale=scale, mlp=ffn()))
        elif kind == "attention_2":
            layers.append(attn2(h, g, dim, vdim, block=rng.choice([None, 2, 9, 33, 64, 80]), cap=rng.choice([None, 10.0, 40.0]),
                                scale=scale, mlp=ffn()))
        else:
            temp = rng.choice([None, (rng.choice([0.2, 0.6]), rng.choice([4, 20, 64]))])
            right = (rng.randint(1, 3), rng.choice([8, 16, 40, 72]), rng.choice([8, 24, 48]), rng.choice([1.0, 4.0, 16.0]), rng.randint(1, 8))
            layers.append(parallel((h, g, dim, vdim, scale, temp), right, rng.choice([0.5, 0.8, 1.0]), rng.choice([0.3, 0.5, 1.2]), mlp=ffn()))
    loop = None
    if rng.random() < 0.7:
        lo = rng.randint(0, len(layers) - 1)
        loop = (lo, rng.randint(lo + 1, len(layers)), rng.randint(1, 3))
    return model(width, rng.choice([77, 128, 200]), layers, eps=rng.choice([1e-5, 1e-6]), loop=loop)


def make_folder(tmp, name, seed: int = 0, std: float = 0.1, gain_std: float = 0.2, dtype=torch.bfloat16, keep_rank: bool = True) -> Path:
    """A model folder with random weights, written by the framework's random-weights mode.  keep_rank False: config.json
    does not say the inner size of the decays' products (it is then read from the tensors' shapes)."""
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
    folder = write_random_model(Path(tmp) / f"lavutar_{label}_{seed}", cfg.to_dict(), table, seed, dtype, std, gain_std)
    if not keep_rank:
        data = json.loads((folder / "config.json").read_text())
        for layer in data["layers"]:
            if layer["type"] == "parallel":
                layer["mixer"]["right"].pop("rank", None)
        (folder / "config.json").write_text(json.dumps(data, indent=2))
    return folder


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
        single = plain_lavutar.forward(cfg, weights, toks, dtype=torch.float32).numpy()
        return max(F32_TOL, 3.0 * float(row_errors(single, exact).max()))
    stored = plain_lavutar.forward(cfg, weights, toks, storage=torch.bfloat16).numpy()
    return 3.0 * float(row_errors(stored, exact).max())


def load(folder):
    return json.loads((Path(folder) / "config.json").read_text()), plain_lavutar.read_safetensors(Path(folder) / "model.safetensors")


CLOSE_CALL = 0.02      # in router logits: rounding in bfloat16 moves a router's logits by less


def firm_rows(dtype: str, cfg: dict, weights: dict, toks) -> np.ndarray:
    """Which positions' logits a bfloat16 run can be held to: those where no router's choice is a close call.  Where the
    last chosen expert's logit and the first that is not chosen lie within CLOSE_CALL of each other, rounding decides
    which one is taken, and the row that follows is another row; both are right.  float32: every position."""
    firm = np.ones(len(toks), dtype=bool)
    if dtype != "float32":
        margins: list = []
        plain_lavutar.forward(cfg, weights, toks, margins=margins)
        per_layer = np.asarray(margins, dtype=np.float64).reshape(-1, len(toks)) if margins else np.zeros((0, len(toks)))
        # The other row is a key and a value for the positions after it: where a window or a block is short it weighs as
        # much as a fifth of what they see, so the rows within reach of a close call through such a layer are left out as
        # well (through longer windows and blocks it is one key among many).
        spans = [m.get("mask", {}).get("size") for layer in cfg["layers"] for m in [layer["mixer"]] if isinstance(m.get("mask"), dict)]
        reach = max([s for s in spans if s < 16], default=0)
        for m in per_layer:
            for p in np.nonzero(m < CLOSE_CALL)[0]:
                firm[p:p + reach + 1] = False
    return firm
