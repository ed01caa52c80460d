"""The Lavutar design without a GPU: configuration, the model as data, cache needs, the weight table, page
bookkeeping for blocks of positions, the decode work list for blocks, and the plain implementation against itself."""
import json
import math

import numpy as np
import pytest
import torch

import plain_lavutar
from lavutar_models import CONFIGS, attn, attn2, dense, make_folder, model, moe, parallel, random_config, tokens

import longbow_quarrel_b200  # noqa: F401
from longbow_quarrel_b200 import architectures  # noqa: F401
from longbow_quarrel_b200.cache import Cache
from longbow_quarrel_b200.config import ConfigError, architecture_of
from longbow_quarrel_b200.config.lavutar import LavutarConfig
from longbow_quarrel_b200.engine.model import Model
from longbow_quarrel_b200.kernels.attention import cut_decode_work, DECODE_TILE
from longbow_quarrel_b200.parts.base import KVNeed, Runtime, SeveralNeeds, StateNeed


def _model(data, dtype=torch.float32):
    arch = architecture_of(data)
    cfg = arch.config_from_dict(data)
    return cfg, arch.describe(cfg), Model(arch.describe(cfg), Runtime(torch.device("cpu"), dtype, 256))


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_a_configuration_survives_the_round_trip(name):
    cfg = LavutarConfig.from_dict(CONFIGS[name])
    again = LavutarConfig.from_dict(json.loads(json.dumps(cfg.to_dict())))
    assert again == cfg


def test_repeated_layers_run_in_order_each_run_with_a_cache_entry_of_its_own():
    cfg, spec, m = _model(CONFIGS["mixed"])
    assert [i for i, _ in cfg.runs()] == [0, 1, 2, 3, 1, 2, 3, 4]
    assert [first for _, first in cfg.runs()] == [False, True, False, False, True, False, False, False]
    mix = len(cfg.layers)                                     # the block that mixes the stream with the embedding's rows
    assert [e.layer for e in spec.schedule] == [0, mix, 1, 2, 3, mix, 1, 2, 3, 4]
    assert len({e.cache for e in spec.schedule}) == len(spec.schedule)
    needs = m.cache_needs()
    assert needs[1] is None and needs[5] is None              # the mixing block keeps nothing
    assert needs[0] == KVNeed(1, 32, None, 16, chunk=64)
    assert needs[2] == needs[6] == SeveralNeeds((KVNeed(2, 32, None, 48), StateNeed((2, 24, 40), torch.float32)))
    assert needs[3] == needs[7] == KVNeed(2, 32, 40, None)
    assert needs[9] == KVNeed(1, 64, 100, None)
    once = _model(CONFIGS["only_loop_once"])[1]
    assert [e.layer for e in once.schedule] == [0, 3, 1, 2]
    none = _model(CONFIGS["only_moe"])[1]
    assert [e.layer for e in none.schedule] == [0] and len(none.layers) == 1


def test_the_weight_table_names_every_tensor_of_the_design():
    cfg, spec, m = _model(CONFIGS["mixed"])
    table = m.weight_table()
    assert table["loop.in"].shape == (64, 128) and table["embed"].shape == (200, 64) and table["head"].shape == (200, 64)
    for name in ("norm1", "norm1.b", "norm2", "norm2.b"):
        assert table["l0." + name].shape == (64,)
    assert table["final.norm.b"].shape == (64,)
    assert table["l0.mix.q.norm"].shape == (4 * 32,) and table["l0.mix.k.norm"].shape == (32,)
    assert table["l0.mix.g"].shape == (4, 64) and table["l0.mix.sink"].shape == (4,) and table["l0.mix.o"].shape == (64, 4 * 16)
    assert table["l1.mix.left.g"].shape == (2 * 48, 64) and table["l1.mix.left.v"].shape == (2 * 48, 64)
    assert table["l1.mix.right.a1"].shape == (8, 64) and table["l1.mix.right.a2"].shape == (48, 8)
    assert table["l1.mix.right.a2.b"].shape == (48,) and table["l1.mix.right.norm"].shape == (40,)
    assert table["l1.mlp.router"].shape == (6, 64) and table["l1.mlp.e5.gate"].shape == (32, 64)
    assert "l2.mix.g" not in table and "l2.mix.sink" not in table and "l2.mix.q.norm" not in table
    assert "l1.mix.left.sink" not in table and "l1.mix.left.q.norm" not in table


def test_the_inner_size_of_the_decay_products_may_come_from_the_tensors():
    data = json.loads(json.dumps(CONFIGS["only_parallel"]))
    del data["layers"][0]["mixer"]["right"]["rank"]
    table = _model(data)[2].weight_table()
    assert table["l0.mix.right.a1"].shape == (-1, 64) and table["l0.mix.right.a2"].shape == (96, -1)
    from longbow_quarrel_b200.weights.loader import _fits
    assert _fits((7, 64), (-1, 64)) and not _fits((7, 63), (-1, 64)) and not _fits((64,), (-1, 64))
    from longbow_quarrel_b200.weights import random_weights
    with pytest.raises(ValueError, match="leaves a size open"):
        random_weights(table, 0)


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].update(type="attention_3"), "type"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3, kv_heads=2), "multiple"),
    (lambda c: c["layers"][0]["mixer"].pop("dim"), "dim"),
    (lambda c: c["layers"][0]["mixer"].update(softcap=-1.0), "softcap"),
    (lambda c: c["layers"][0]["mixer"].update(mask={"size": 0}), "size"),
    (lambda c: c["layers"][1]["mixer"].pop("right"), "right"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(tau=0.0), "tau"),
    (lambda c: c["layers"][1]["mixer"]["left"].update(q_temp={"coef": 0.1, "every": 0}), "every"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=7), "top"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=7), "dims"),
    (lambda c: c["layers"][2]["mixer"]["rot"]["scaling"].pop("fast"), "fast"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["loop"].update(start=3, stop=3), "loop"),
    (lambda c: c["loop"].update(times=0), "times"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "kind"),
])
def test_configuration_errors_name_the_key(change, message):
    data = json.loads(json.dumps(CONFIGS["mixed"]))
    change(data)
    with pytest.raises(ConfigError, match=message):
        LavutarConfig.from_dict(data)


def test_absent_keys_leave_their_mechanism_out():
    data = model(32, 50, [{"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 16}, "mlp": None},
                          {"type": "attention_2", "mixer": {"heads": 2, "kv_heads": 2, "dim": 8}, "mlp": None},
                          {"type": "parallel", "mlp": None,
                           "mixer": {"left": {"heads": 1, "kv_heads": 1, "dim": 8}, "right": {"heads": 1, "dim": 8, "tau": 2.0}}}])
    cfg = LavutarConfig.from_dict(data)
    a, b, c = cfg.layers
    assert a.attn.span is None and a.attn.rot is None and a.attn.vdim == 16 and a.attn.scale == 0.25
    assert b.attn.span is None and b.attn.softcap is None
    assert c.attn.temp_coef is None and c.left_scale == 1.0 and c.right_scale == 1.0 and c.right.rank is None and c.right.vdim == 8
    assert cfg.loop is None and [i for i, _ in cfg.runs()] == [0, 1, 2]


def test_pages_below_a_sequence_s_block_go_back():
    """A group for blocks of 100 positions on pages of 64: once position 100 is next, page 0 (positions 0..63) goes
    back; page 1 holds positions 100..127 and stays; at 200, pages 1 and 2 go back (page 3 holds 200..)."""
    c = Cache({0: KVNeed(1, 8, None, chunk=100)}, max_tokens=640, max_context=640, dtype=torch.float32, device="cpu", max_slots=2)
    g = c.kv_groups[0]
    s = c.alloc_slot()
    c.reserve(s, 99)
    c.commit(s, 99)
    assert g.pages_in_use() == 2
    c.reserve_one_each([s])
    c.commit_one_each([s])                 # 100 tokens: the next position starts the second block
    assert g.pages_in_use() == 1 and g.table[s, 0] == -1 and g.table[s, 1] != -1
    c.reserve(s, 101)
    c.commit(s, 101)                       # 201 tokens: positions 200.. lie on page 3
    assert [int(p != -1) for p in g.table[s, :5]] == [0, 0, 0, 1, 0]
    for _ in range(99):
        c.reserve_one_each([s])
        c.commit_one_each([s])             # 300 tokens, one by one
    assert [int(p != -1) for p in g.table[s, :6]] == [0, 0, 0, 0, 1, 0]
    c.free_slot(s)
    assert g.pages_in_use() == 0


def test_a_layer_of_two_sides_keeps_pages_and_a_state_under_one_entry():
    need = SeveralNeeds((KVNeed(1, 8, None), StateNeed((2, 4, 4), torch.float32)))
    c = Cache({0: need, 1: need, 2: KVNeed(1, 8, 20)}, max_tokens=256, max_context=256, dtype=torch.float32, device="cpu", max_slots=2)
    assert len(c.groups) == 2 and len(c.kv_groups) == 2 and len(c.state_groups) == 1
    kv, state = c.view(0)
    assert state.shape == (2, 2, 4, 4) and kv.k_pages.shape[-1] == 8 and c.view(1)[1].data_ptr() != state.data_ptr()
    s = c.alloc_slot()
    state[s].fill_(3.0)
    c.reserve(s, 70)
    c.commit(s, 70)
    assert c.pages_in_use() == 2 + 2           # two pages in each of the two kv groups
    c.free_slot(s)
    assert c.pages_in_use() == 0
    assert c.alloc_slot() == s and float(c.view(0)[1][s].abs().sum()) == 0.0     # the state starts from zero again


def test_the_decode_work_list_starts_at_the_block_of_the_token():
    pos = np.array([0, 99, 100, 199, 250, 1023])
    teams = 40
    work = cut_decode_work(pos, 0, teams, chunk=100)
    seg = work[teams + 1:].reshape(-1, 5)
    seg = seg[:work[teams]]
    for tok, p in enumerate(pos):
        first = (p - p % 100) // DECODE_TILE
        tiles = p // DECODE_TILE + 1 - first
        mine = seg[seg[:, 0] == tok]
        covered = sorted((int(lo), int(hi)) for lo, hi in mine[:, 1:3])
        assert covered[0][0] == 0 and covered[-1][1] == tiles
        assert all(a[1] == b[0] for a, b in zip(covered, covered[1:]))


# ------------------------------------------------------------------ the plain implementation against itself

def test_plain_blocks_windows_and_the_state_behave_as_the_design_says(tmp_path):
    folder = make_folder(tmp_path, "only_attention_2", seed=1, std=0.3)
    cfg, weights = json.loads((folder / "config.json").read_text()), plain_lavutar.read_safetensors(folder / "model.safetensors")
    base = tokens(60, cfg["vocab"], 2)
    ref = plain_lavutar.forward(cfg, weights, base)
    odd = list(base)
    odd[23] = (odd[23] + 1) % cfg["vocab"]                  # the last position of the first block of 24
    out = plain_lavutar.forward(cfg, weights, odd)
    assert float((out[23] - ref[23]).abs().max()) > 1e-6
    assert float((out[24:] - ref[24:]).abs().max()) == 0.0   # the next block sees nothing of it
    assert float((out[:23] - ref[:23]).abs().max()) == 0.0

    folder = make_folder(tmp_path, "only_attention", seed=1, std=0.3)
    cfg, weights = json.loads((folder / "config.json").read_text()), plain_lavutar.read_safetensors(folder / "model.safetensors")
    ref = plain_lavutar.forward(cfg, weights, base)
    odd = list(base)
    odd[10] = (odd[10] + 1) % cfg["vocab"]
    out = plain_lavutar.forward(cfg, weights, odd)
    assert float((out[29] - ref[29]).abs().max()) > 1e-6    # window 20: position 29 is the last that sees position 10
    assert float((out[30:] - ref[30:]).abs().max()) == 0.0

    folder = make_folder(tmp_path, "only_parallel", seed=1, std=0.3)
    cfg, weights = json.loads((folder / "config.json").read_text()), plain_lavutar.read_safetensors(folder / "model.safetensors")
    ref = plain_lavutar.forward(cfg, weights, base)
    odd = list(base)
    odd[0] = (odd[0] + 1) % cfg["vocab"]
    out = plain_lavutar.forward(cfg, weights, odd)
    assert float((out[59] - ref[59]).abs().max()) > 1e-9    # nothing ever hides the first position from this layer


def test_plain_mechanisms_one_by_one():
    torch.manual_seed(0)
    x = torch.randn(5, 12, dtype=torch.float64)
    g, b = torch.randn(12, dtype=torch.float64), torch.randn(12, dtype=torch.float64)
    y = plain_lavutar.layer_norm(x, g, b, 1e-5)
    assert torch.allclose(y, torch.nn.functional.layer_norm(x, (12,), g, b, 1e-5), atol=1e-12)
    # frequencies: without scaling the plain ones; with a ramp from 0 to the last pair a blend that ends at f / factor
    rot = {"dims": 8, "base": 100.0}
    f, mag = plain_lavutar.blended_frequencies(rot)
    assert mag == 1.0 and torch.allclose(f, torch.tensor([100.0 ** (-2 * i / 8) for i in range(4)], dtype=torch.float64))
    f2, mag2 = plain_lavutar.blended_frequencies({**rot, "scaling": {"factor": 4.0, "original": 64, "fast": 1e9, "slow": 1e-9}})
    assert math.isclose(mag2, 0.1 * math.log(4.0) + 1.0) and float(f2[0]) == float(f[0]) and float(f2[3]) < float(f[3])
    # routing: the largest logits, the lower number first on a tie, weights that sum to one
    experts, w = plain_lavutar.route(torch.tensor([0.1, 2.0, -1.0, 2.0, 0.5], dtype=torch.float64), 3)
    assert experts == [1, 3, 4] and math.isclose(float(w.sum()), 1.0) and float(w[0]) == float(w[1]) > float(w[2])
    # a decay of exactly one keeps the state; with the state carried over, two halves give what the whole gives
    m = {"heads": 1, "dim": 4, "vdim": 3, "tau": 2.0}
    w = {k: torch.randn(s, dtype=torch.float64) for k, s in
         {"q": (4, 6), "k": (4, 6), "v": (3, 6), "g": (3, 6), "o": (6, 3), "a1": (2, 6), "a2": (4, 2), "a2.b": (4,), "norm": (3,)}.items()}
    h = torch.randn(7, 6, dtype=torch.float64)
    a = plain_lavutar.channel_decays(h, w, m)
    z = (h @ w["a1"].T) @ w["a2"].T + w["a2.b"]
    assert torch.allclose(a.reshape(7, 4), torch.sigmoid(z) ** 0.5, atol=1e-12)
    state: list = []
    plain_lavutar.gated_linear_attention(h, w, m, 1e-5, state)
    S = torch.zeros(4, 3, dtype=torch.float64)
    for t in range(7):
        S = a[t, 0][:, None] * S + (w["k"] @ h[t])[:, None] * (w["v"] @ h[t])[None, :]
    assert torch.allclose(state[0][0], S, atol=1e-12)


def test_a_configuration_drawn_at_random_runs_plain(tmp_path):
    import random
    for seed in (1, 2, 3):
        data = random_config(random.Random(seed))
        folder = make_folder(tmp_path, data, seed=seed)
        cfg, weights = json.loads((folder / "config.json").read_text()), plain_lavutar.read_safetensors(folder / "model.safetensors")
        toks = tokens(20, cfg["vocab"], seed)
        layers: list = []
        out = plain_lavutar.forward(cfg, weights, toks, layers_out=layers)
        assert out.shape == (20, cfg["vocab"]) and torch.isfinite(out).all()
        assert len(layers) == len(plain_lavutar.layer_order(cfg))
