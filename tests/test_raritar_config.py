"""Raritar without a GPU: the typed configuration and its errors, the model as data (which storage each part asks
for, which cache entry a layer reads), the weight table, the rotation tables with rescaled frequencies, the order of
reordered pairs, the decode kernel's work list with kept tiles, and the plain implementation against itself."""
import copy
import math

import numpy as np
import pytest
import torch

import plain_raritar
from raritar_models import CONFIGS, load, make_folder, row_errors, tokens


def _arch(data):
    import longbow_quarrel_b200  # noqa: F401
    from longbow_quarrel_b200 import architectures  # noqa: F401
    from longbow_quarrel_b200.config import architecture_of
    arch = architecture_of(data)
    return arch, arch.config_from_dict(data)


def test_configuration_round_trip_and_description():
    from longbow_quarrel_b200.parts.base import KVNeed, Runtime, StateNeed
    from longbow_quarrel_b200.engine.model import Model
    arch, cfg = _arch(CONFIGS["mixed"])
    assert arch.name == "Raritar"
    assert _arch(cfg.to_dict())[1] == cfg
    assert cfg.layers[0].rot.factor == 4.0 and cfg.layers[1].rot.factor is None and cfg.layers[3].rot is None
    assert cfg.layers[1].mlp is None and cfg.layers[1].window is None and cfg.layers[1].softcap is None
    assert (cfg.layers[0].window, cfg.layers[0].keep_first, cfg.layers[2].kv_from, cfg.layers[4].kv_from) == (33, 5, 0, 1)
    r = cfg.layers[0].mlp.router
    assert (r.experts, r.identity, r.groups, r.keep, r.top) == (6, 2, 4, 2, 3) and cfg.layers[2].mlp.router.groups == 1
    assert (cfg.taps, cfg.residual_mult, cfg.bigram.buckets, cfg.bigram.mul_prev, cfg.bigram.mul_cur) == (3, 0.7, 97, 5, 3)
    spec = arch.describe(cfg)
    assert [(e.layer, e.cache, e.writes_cache) for e in spec.schedule] == \
        [(0, 0, True), (1, 1, True), (2, 0, False), (3, 3, True), (4, 1, False)]
    model = Model(spec, Runtime(torch.device("cpu"), torch.float32, 128))
    needs = model.cache_needs()
    # Entry 0 keeps what its furthest reader sees (layer 2's window of 100, layer 0's five first positions); entry 1 keeps
    # everything because layer 1 itself has no window; values of another size than keys get a pool of their own size.
    assert needs[0] == KVNeed(2, 16, 100, 24, keep_first=5) and needs[1] == KVNeed(1, 32, None, None)
    assert needs[3] == KVNeed(3, 8, 5, None)
    states = sorted((k, v) for k, v in needs.items() if isinstance(v, StateNeed))
    assert len(states) == 1 + 5 and all(v.shape == (2, 64) for _, v in states[1:])       # the last token, and taps - 1 rows a layer
    table = model.weight_table()
    assert table["embed"].shape == (200, 64) and table["bigram"].shape == (98, 64) and table["head"].shape == (200, 64)
    assert table["l0.norm1"].shape == () and table["final.norm"].shape == () and table["l0.canon1"].shape == (64, 3)
    assert table["l0.mix.q"].shape == (64, 64) and table["l0.mix.k"].shape == (32, 64) and table["l0.mix.v"].shape == (48, 64)
    assert table["l0.mix.o"].shape == (64, 96) and table["l2.mix.q"].shape == (96, 64) and table["l2.mix.o"].shape == (64, 144)
    assert "l2.mix.k" not in table and "l2.mix.v" not in table and "l4.mix.k" not in table
    assert table["l0.mlp.router"].shape == (8, 64) and table["l0.mlp.correction"].shape == (8,)
    assert table["l0.mlp.e5.gate"].shape == (32, 64) and table["l0.mlp.e5.down"].shape == (64, 32) and "l0.mlp.e6.up" not in table
    assert table["l0.mlp.shared.gate"].shape == (48, 64) and table["l0.mlp.shared.sg"].shape == (1, 64)
    assert "l1.norm2" not in table and "l1.mlp.router" not in table and "l2.mlp.shared.up" not in table


def test_absent_keys_leave_their_mechanism_out():
    """A model without the second table, the convolution, the multiplier, masks, caps and rotation is plain
    grouped-query attention; its layers then take the products that fold the norms."""
    from longbow_quarrel_b200.parts.base import Runtime
    from longbow_quarrel_b200.engine.model import Model
    arch, cfg = _arch(CONFIGS["odd"])
    assert cfg.taps is None and cfg.bigram is None and cfg.residual_mult == 1.0
    model = Model(arch.describe(cfg), Runtime(torch.device("cpu"), torch.float32, 128))
    table = model.weight_table()
    assert "bigram" not in table and "l0.canon1" not in table
    assert all(block.folds_norm for block in model.blocks)
    arch, cfg = _arch(CONFIGS["only_conv_one_tap"])
    model = Model(arch.describe(cfg), Runtime(torch.device("cpu"), torch.float32, 128))
    assert model.weight_table()["l0.canon1"].shape == (40, 1) and not model.blocks[0].folds_norm
    assert not [v for v in model.cache_needs().values() if type(v).__name__ == "StateNeed"]      # one tap needs no earlier row


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "at most"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("low"), "low"),
    (lambda c: c["layers"][0]["mixer"].pop("heads"), "heads"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "size"),
    (lambda c: c["layers"][2].update(type="lightning"), "not one of"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "earlier"),
    (lambda c: c["layers"][4]["mixer"].update(kv_from=2), "of its own"),
    (lambda c: c["layers"][2]["mixer"].update(dim=8), "must equal"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "not supported"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(identity=1), "equal"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "top"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(keep=5), "kept"),
    (lambda c: c["layers"][0]["mlp"].pop("expert"), "expert"),
    (lambda c: c["embedding"]["bigram"].pop("mul_cur"), "mul_cur"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.update(layers=[]), "layers"),
])
def test_configuration_errors_name_the_key(change, word):
    from longbow_quarrel_b200.config import ConfigError
    data = copy.deepcopy(CONFIGS["mixed"])
    change(data)
    with pytest.raises(ConfigError, match=word):
        _arch(data)


@pytest.mark.parametrize("dims,base,scaling", [
    (8, 10000.0, {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}),        # some frequencies kept, some blended, some divided
    (48, 5e5, {"factor": 16.0, "low": 2.0, "high": 8.0, "original": 256}),
    (16, 100.0, {"factor": 2.0, "low": 1.0, "high": 4.0, "original": 1e6}),        # every wavelength is short: all kept
    (6, 5e5, {"factor": 3.0, "low": 1.0, "high": 2.0, "original": 4}),             # every wavelength is long: all divided
    (12, 300.0, None),
])
def test_rotation_tables_follow_the_rescaled_frequencies(dims, base, scaling):
    """The framework's tables against the frequencies written out here, wavelength by wavelength."""
    from longbow_quarrel_b200.parts.base import Runtime
    from longbow_quarrel_b200.parts.registry import make_part
    from longbow_quarrel_b200.parts.rope import WavelengthScaling
    from longbow_quarrel_b200.parts.spec import PartSpec
    sc = WavelengthScaling(scaling["factor"], scaling["low"], scaling["high"], scaling["original"]) if scaling else None
    part = make_part("position", PartSpec("rope", {"head_dim": dims + 4, "theta": base, "rotary_dims": dims, "scaling": sc,
                                                   "layout": "interleaved"}), Runtime(torch.device("cpu"), torch.float32, 200))
    cos, sin = part.tables()
    want = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling:
            wave, orig = 2.0 * math.pi / f, scaling["original"]
            if wave > orig / scaling["low"]:
                f = f / scaling["factor"]
            elif wave >= orig / scaling["high"]:
                s = (orig / wave - scaling["low"]) / (scaling["high"] - scaling["low"])
                f = (1.0 - s) * f / scaling["factor"] + s * f
        want.append(f)
    freqs = torch.tensor(want, dtype=torch.float64)
    assert (plain_raritar.scaled_frequencies(dims, base, scaling) - freqs).abs().max() < 1e-15
    pos = torch.arange(200, dtype=torch.float64)[:, None]
    assert cos.shape == (200, dims // 2)
    assert (cos.double() - torch.cos(pos * freqs)).abs().max() < 1e-6
    assert (sin.double() - torch.sin(pos * freqs)).abs().max() < 1e-6


@pytest.mark.parametrize("hd,rot", [(16, 8), (12, 12), (64, 32), (8, 0), (10, 2)])
def test_reordered_rows_turn_interleaved_pairs_into_halves(hd, rot):
    """Rows of a query projection in the order `pair_order` gives: rotating the halves (i, i + rot / 2) of the
    reordered head and scoring it against an equally reordered key gives the score of the interleaved pairs."""
    from longbow_quarrel_b200.parts.rope import pair_order
    order = pair_order(hd, rot)
    assert sorted(order) == list(range(hd)) and order[rot:] == list(range(rot, hd))
    g = torch.Generator().manual_seed(hd * 100 + rot)
    q, k = torch.randn(hd, generator=g, dtype=torch.float64), torch.randn(hd, generator=g, dtype=torch.float64)
    freqs = torch.tensor([3.0 ** -i for i in range(rot // 2)], dtype=torch.float64)

    def halves(x, pos):
        out = x.clone()
        c, s = torch.cos(pos * freqs), torch.sin(pos * freqs)
        a, b = x[:rot // 2], x[rot // 2:rot]
        out[:rot // 2], out[rot // 2:rot] = a * c - b * s, b * c + a * s
        return out
    want = plain_raritar.rotate_pairs(q, 7, freqs) @ plain_raritar.rotate_pairs(k, 3, freqs)
    got = halves(q[order], 7) @ halves(k[order], 3)
    assert abs(float(want - got)) < 1e-12


def test_routing_of_the_plain_implementation():
    """Scores chosen so that each rule shows: the correction moves the choice but not the weights; a group is scored
    by its best member; an expert outside the kept groups is not chosen although its choice score is the third
    best; negative choice scores inside a kept group still beat everything outside it."""
    router = {"experts": 5, "identity": 1, "top": 2, "groups": {"count": 3, "keep": 2}}
    s = torch.tensor([0.30, 0.02, 0.25, 0.05, 0.20, 0.18], dtype=torch.float64)
    none = torch.zeros(6, dtype=torch.float64)
    assert plain_raritar.route(s, none, router) == [0, 2]
    corr = torch.tensor([0.0, 0.0, -0.2, 0.0, 0.0, 0.1], dtype=torch.float64)       # groups score 0.30, 0.05, 0.28
    assert plain_raritar.route(s, corr, router) == [0, 5]
    assert plain_raritar.route(s, corr, {**router, "top": 4}) == [0, 5, 4, 1]
    low = torch.tensor([-1.0, -1.0, -0.9, -2.0, -3.0, -3.0], dtype=torch.float64)    # groups score -0.70, -0.65, -2.80
    assert plain_raritar.route(s, low, {**router, "top": 3}) == [2, 0, 1]
    assert plain_raritar.choice_margin(s, none, router) == pytest.approx(0.05)      # groups 0.30, 0.25, 0.20; experts 0.25 against 0.05
    h = torch.tensor([[1.0, -2.0]], dtype=torch.float64)
    w = {"router": torch.tensor([[0.0, 0.0], [5.0, 0.0]], dtype=torch.float64)}
    y = plain_raritar.routed_ffn(h, w, {"router": {"experts": 0, "identity": 2, "top": 1}})
    assert torch.allclose(y, h * torch.softmax(torch.tensor([0.0, 5.0], dtype=torch.float64), 0)[1])


def test_the_work_list_of_single_tokens_counts_kept_tiles():
    from longbow_quarrel_b200.kernels.attention import cut_decode_work
    pos = [0, 15, 16, 100, 1000, 5000]
    for window, keep in ((0, 0), (64, 0), (64, 5), (64, 16), (64, 40), (300, 700)):
        work = cut_decode_work(pos, window, teams=24, keep_first=keep)
        segs = work[25:].reshape(-1, 5)[:work[24]]
        for b, p in enumerate(pos):
            first = (p - window + 1) // 16 if window and p >= window else 0
            counted = p // 16 + 1 - first + (min(-(-keep // 16), first) if window else 0)
            mine = sorted((int(s[1]), int(s[2])) for s in segs if s[0] == b)
            assert mine[0][0] == 0 and mine[-1][1] == counted and all(a[1] == c[0] for a, c in zip(mine, mine[1:])), (window, keep, p)


def test_plain_implementation_agrees_with_itself(tmp_path):
    """A prefix's logits do not depend on what follows; float32 stays close to float64; in a model of attention alone
    (window 20, three kept positions, nothing else that looks back) a token beyond the window no longer changes a later
    position unless it is one of the kept first, while one inside the window does."""
    folder = make_folder(tmp_path, "mixed", seed=1)
    cfg, weights = load(folder)
    toks = tokens(60, cfg["vocab"], 2)
    full = plain_raritar.forward(cfg, weights, toks).numpy()
    part = plain_raritar.forward(cfg, weights, toks[:17]).numpy()
    assert row_errors(part, full[:17]).max() < 1e-12
    single = plain_raritar.forward(cfg, weights, toks, dtype=torch.float32).numpy()
    assert row_errors(single, full).max() < 1e-4
    stored = plain_raritar.forward(cfg, weights, toks, storage=torch.bfloat16).numpy()
    assert 1e-4 < row_errors(stored, full).max() < 0.1
    layers: list = []
    plain_raritar.forward(cfg, weights, toks, layers_out=layers)
    assert len(layers) == 5 and layers[0].shape == (60, 64)
    assert plain_raritar.greedy(cfg, weights, toks[:5], 3) == plain_raritar.greedy(cfg, weights, toks[:5], 3)
    folder = make_folder(tmp_path, "only_attention_bare", seed=2)
    cfg, weights = load(folder)
    toks = tokens(40, cfg["vocab"], 3)
    base = plain_raritar.forward(cfg, weights, toks).numpy()
    for changed, same in ((0, False), (2, False), (3, True), (10, True), (19, True), (20, False), (39, False)):   # 39 sees 0..2 and 20..39
        other = list(toks)
        other[changed] = (other[changed] + 1) % cfg["vocab"]
        moved = row_errors(plain_raritar.forward(cfg, weights, other).numpy()[39:], base[39:]).max()
        assert (moved < 1e-12) == same, (changed, moved)
