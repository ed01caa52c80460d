"""The Lavutar design through the engine: every mechanism alone and together, every way of cutting and batching
requests, slots and pages used again, decoding until windows and blocks have passed over decoded tokens, the edges
of windows and blocks made visible by one odd token, repeated layers, generation through the entry point and the
command line -- each against the plain implementation (tests/plain_lavutar.py)."""
import json
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_lavutar
from lavutar_models import CONFIGS, bound, firm_rows, load, make_folder, random_config, row_errors, tokens
from trace_tools import ROOT, Trace, run_trace, split, trace_batches, trace_chunked, trace_last_one_by_one, trace_mixed, trace_whole

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]


def _engine(folder, dtype, **kw):
    from longbow_quarrel_b200.engine import Engine
    return Engine.from_pretrained(folder, dtype=dtype, **kw)


_memo: dict = {}


def _plain(folder, toks):
    """The plain implementation's logits for a request (kept: every cut of a request is compared with the same rows)."""
    key = (str(folder), tuple(toks))
    if key not in _memo:
        cfg, weights = load(folder)
        _memo[key] = {"plain": (cfg, weights, plain_lavutar.forward(cfg, weights, toks).numpy())}
    return _memo[key]["plain"]


def _yard(folder, toks, dtype):
    """(bound, firm rows) of a request in a precision, measured once."""
    cfg, weights, ref = _plain(folder, toks)
    entry = _memo[(str(folder), tuple(toks))]
    if dtype not in entry:
        entry[dtype] = (bound(dtype, cfg, weights, toks, ref), firm_rows(dtype, cfg, weights, toks))
    return entry[dtype]


def _check(got: dict, requests: dict, folder, dtype: str, what: str):
    """float32: every row within its request's bound.  bfloat16: no row beyond one and a half times the bound and at
    most one row in fifty beyond the bound itself, over the rows where no router's choice is a close call."""
    over = total = 0
    for rid, toks in requests.items():
        cfg, weights, ref = _plain(folder, toks)
        tol, firm = _yard(folder, toks, dtype)
        keys = [k for k in got if k[0] == rid]
        assert keys, f"{what}: nothing came back for {rid}"
        for _, pos in keys:
            if not firm[pos]:
                continue
            err = float(row_errors(got[(rid, pos)], ref[pos]))
            hard = tol if dtype == "float32" else 1.5 * tol
            assert err < hard, f"{what}: request {rid} position {pos} of {len(toks)}: error {err:.3g}, bound {hard:.3g}"
            over += err >= tol
            total += 1
    assert total > 0 and over <= 0.02 * total, f"{what}: {over} of {total} rows over their bound"


# ------------------------------------------------------------------ each mechanism alone

ALONE = [name for name in sorted(CONFIGS) if name.startswith("only_")]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ALONE)
def test_one_layer_of_each_kind_whole_and_token_by_token(tmp_path, name, dtype):
    """A model of one mechanism: the whole prompt in one step (its first tokens included), and the same tokens one by one
    from the first (133 steps: across two page borders and, for the windows and blocks, far past them; replayed from a
    captured step)."""
    folder = make_folder(tmp_path, name, seed=3, keep_rank=False)
    toks = tokens(133, CONFIGS[name]["vocab"], 5)
    cfg, weights, ref = _plain(folder, toks)
    tol = bound(dtype, cfg, weights, toks, ref)
    firm = firm_rows(dtype, cfg, weights, toks)
    assert firm.sum() > 60
    eng = _engine(folder, dtype, max_tokens=512)
    s = eng.new_sequence()
    whole = eng.step([(s, toks)], [list(range(len(toks)))]).cpu().numpy()
    eng.end_sequence(s)
    assert row_errors(whole, ref)[firm].max() < tol
    s = eng.new_sequence()
    single = np.stack([eng.step([(s, [t])], [[0]]).cpu().numpy()[0] for t in toks])
    eng.end_sequence(s)
    assert row_errors(single, ref)[firm].max() < tol
    assert row_errors(single, whole)[firm].max() < tol
    eng.close()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["only_attention_bare_window", "only_attention_2_open_block"])
def test_windows_and_blocks_decide_when_one_token_outweighs_all_others(tmp_path, name, dtype):
    """One layer of attention and nothing else that looks back, in a prompt of one odd token among copies of another.
    With a window of 4 an odd token at position 30 changes the logits up to position 33 and not at all from 34 on; with
    blocks of 4 an odd token at position 30 changes the logits up to position 31 (the last of its block) and none from
    32 on, an odd token at position 31 changes its own row alone, and one at position 28 (the block's first) the whole
    block -- in a prompt, with the edge among decoded tokens, and with everything after the odd token decoded."""
    data = json.loads(json.dumps(CONFIGS["only_attention_bare" if "bare" in name else "only_attention_2_open"]))
    data["layers"][0]["mixer"]["mask"] = {"size": 4}
    data["layers"][0]["mixer"]["scale"] = 0.02          # a flat softmax: every visible key weighs about the same, so one odd key shows
    folder = make_folder(tmp_path, data, seed=9, std=0.5)
    cfg, weights = load(folder)
    base = [7] * 70
    ref_base = plain_lavutar.forward(cfg, weights, base).numpy()
    eng = _engine(folder, dtype, max_tokens=256)
    cases = [(30, 33)] if "bare" in name else [(30, 31), (31, 31), (28, 31)]
    for at, inside in cases:
        outside = inside + 1
        odd = list(base)
        odd[at] = 55
        ref_odd = plain_lavutar.forward(cfg, weights, odd).numpy()
        assert row_errors(ref_odd[inside], ref_base[inside]) > 1e-3
        assert row_errors(ref_odd[outside:], ref_base[outside:]).max() < 1e-12
        tol = bound(dtype, cfg, weights, odd, ref_odd)
        for cut in (70, max(at + 1, inside - 3), at + 1):
            s = eng.new_sequence()
            rows = [eng.step([(s, odd[:cut])], [list(range(cut))]).cpu().numpy()]
            rows += [eng.step([(s, [t])], [[0]]).cpu().numpy() for t in odd[cut:]]
            eng.end_sequence(s)
            got = np.concatenate(rows)
            assert row_errors(got, ref_odd).max() < tol, (at, cut)
            assert row_errors(got[inside], ref_base[inside]) > 2 * tol, (at, cut)
            assert row_errors(got[outside:], ref_base[outside:]).max() < tol, (at, cut)
    eng.close()


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_first_token_lasts_in_the_state_and_the_far_key_is_found(tmp_path, dtype):
    """A layer of two sides whose decays are all but one (a large bias): the first token of 300 still changes the last
    position's logits through the state, whole and with the last 200 tokens decoded; and in the same model the softmax side
    sees every earlier position, so an odd first token among copies shows at position 299."""
    folder = make_folder(tmp_path, "only_parallel", seed=4, std=0.5)
    cfg, weights = load(folder)
    weights["l0.mix.right.a2.b"] = torch.full_like(weights["l0.mix.right.a2.b"], 12.0)
    from longbow_quarrel_b200.weights import write_safetensors
    write_safetensors(folder / "model.safetensors", weights, {"format": "pt"})
    base = [3] * 300
    odd = [11] + base[1:]
    ref_base, ref_odd = plain_lavutar.forward(cfg, weights, base).numpy(), plain_lavutar.forward(cfg, weights, odd).numpy()
    tol = bound(dtype, cfg, weights, odd, ref_odd)
    # One token among three hundred moves the last row by a few per cent: hundreds of times the float32 bound, and
    # about as much as rounding to bfloat16 does, so only the float32 run can show that it was found.
    sharp = row_errors(ref_odd[299], ref_base[299]) > 20 * tol
    assert sharp == (dtype == "float32")
    eng = _engine(folder, dtype, max_tokens=512)
    for cut in (300, 100):
        s = eng.new_sequence()
        rows = [eng.step([(s, odd[:cut])], [list(range(cut))]).cpu().numpy()]
        rows += [eng.step([(s, [t])], [[0]]).cpu().numpy() for t in odd[cut:]]
        eng.end_sequence(s)
        got = np.concatenate(rows)
        assert row_errors(got, ref_odd).max() < tol, cut
        assert not sharp or row_errors(got[299], ref_base[299]) > 10 * tol, cut
    eng.close()


# ------------------------------------------------------------------ whole models, every cut, through the replay program

LENGTHS = {"r0": 70, "r1": 33, "r2": 140, "r3": 65, "r4": 64, "r5": 34, "r6": 129}
PROMPTS = {"r0": 7, "r1": 1, "r2": 100, "r3": 2, "r4": 63, "r5": 20, "r6": 65}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "odd", "wide"])
def test_every_cut_of_every_request_matches_plain(tmp_path, name, dtype):
    """Whole; the last 32 tokens one by one; batches of three unequal requests that go on together, the shorter
    ending earlier, the next batch in the slots and pages given back; portions of 2, 3, 59, 1, 64 and 7 tokens;
    steps that mix portions with single tokens.  One call of the replay program runs them one after the other."""
    folder = make_folder(tmp_path, name, seed=11, keep_rank=False)
    vocab = CONFIGS[name]["vocab"]
    requests = {rid: tokens(n, vocab, 100 + i) for i, (rid, n) in enumerate(LENGTHS.items())}
    tr = Trace()
    tr.extend(trace_whole(requests), "whole:")
    tr.extend(trace_last_one_by_one(requests), "tail:")
    tr.extend(trace_batches(requests, PROMPTS, width=3), "batched:")
    tr.extend(trace_chunked(requests, [2, 3, 59, 1, 64, 7]), "portions:")
    tr.extend(trace_mixed(requests, PROMPTS, [5, 1, 2, 1, 17]), "mixed:")
    got = run_trace(folder, dtype, tr, tmp_path / "out")
    cuts = {p: split(got, p + ":") for p in ("whole", "tail", "batched", "portions", "mixed")}
    for what, rows in cuts.items():
        assert len(rows) == (33 * len(requests) if what == "tail" else sum(LENGTHS.values())), what
        _check(rows, requests, folder, dtype, what)
    if dtype == "float32":
        for rid, toks in requests.items():
            tol, _ = _yard(folder, toks, dtype)
            for what in ("tail", "batched", "portions", "mixed"):
                for (r, pos), row in cuts[what].items():
                    if r == rid:
                        err = float(row_errors(row, cuts["whole"][(r, pos)]))
                        assert err < 2 * tol, f"{what} against whole: {rid} position {pos}: {err:.3g}, bound {2 * tol:.3g}"


@pytest.mark.parametrize("seed", [3, 12, 29])
def test_configurations_drawn_at_random_match_plain(tmp_path, seed):
    """Sizes and options that nobody chose: whole, the last 30 tokens one by one and an unequal batch, in both precisions."""
    import random
    rng = random.Random(seed)
    folder = make_folder(tmp_path, random_config(rng), seed=seed, std=rng.choice([0.1, 0.2]))
    cfg, _ = load(folder)
    requests = {rid: tokens(n, cfg["vocab"], 50 * seed + i) for i, (rid, n) in enumerate({"a": 150, "b": 70, "c": 33}.items())}
    tr = Trace()
    tr.extend(trace_whole(requests), "whole:")
    tr.extend(trace_last_one_by_one(requests, n_last=30), "tail:")
    tr.extend(trace_batches(requests, {"a": 110, "b": 40, "c": 3}, width=3), "batched:")
    for dtype in DTYPES:
        got = run_trace(folder, dtype, tr, tmp_path / ("out_" + dtype))
        for what in ("whole", "tail", "batched"):
            _check(split(got, what + ":"), requests, folder, dtype, f"seed {seed} {dtype} {what}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_stream_after_every_run_of_a_layer_matches_plain(tmp_path, dtype):
    """The residual stream after each run of a layer (a repeated layer counts every time), for a prompt that is longer
    than every window and block, and for the same prompt cut into portions."""
    folder = make_folder(tmp_path, "mixed", seed=13)
    toks = tokens(150, CONFIGS["mixed"]["vocab"], 17)
    cfg, weights = load(folder)
    exact: list = []
    plain_lavutar.forward(cfg, weights, toks, layers_out=exact)
    other: list = []
    if dtype == "float32":
        plain_lavutar.forward(cfg, weights, toks, dtype=torch.float32, layers_out=other)
    else:
        plain_lavutar.forward(cfg, weights, toks, storage=torch.bfloat16, layers_out=other)
    firm = firm_rows(dtype, cfg, weights, toks)
    eng = _engine(folder, dtype, max_tokens=512)
    for portions in ([150], [64, 1, 2, 83]):
        seen: dict = {}
        eng.model.probe = lambda i, x, ctx: seen.setdefault(i, []).append(x.detach().float().cpu().clone())
        s = eng.new_sequence()
        at = 0
        for n in portions:
            eng.step([(s, toks[at:at + n])], [[n - 1]])
            at += n
        eng.end_sequence(s)
        eng.model.probe = None
        runs = [i for i in sorted(seen) if i >= 0]             # the schedule's places at which a layer ran
        assert len(runs) == len(exact) == 8
        for n, i in enumerate(runs):
            got = torch.cat(seen[i]).numpy()
            yard = max(1e-5, 3.0 * float(row_errors(other[n].numpy(), exact[n].numpy())[firm].max()))
            assert row_errors(got, exact[n].numpy())[firm].max() < yard, (portions, n)
    eng.close()


# ------------------------------------------------------------------ slots and pages used again, long decoding

@pytest.mark.parametrize("dtype", DTYPES)
def test_a_slot_that_is_used_again_starts_from_nothing(tmp_path, dtype):
    """One slot and just enough pages: each request runs in what the one before it gave back, so a state or a page that
    outlived its request would show in the next one's first tokens."""
    folder = make_folder(tmp_path, "mixed", seed=21)
    eng = _engine(folder, dtype, max_tokens=192, max_batch=1)
    for i, n in enumerate([150, 3, 130, 66]):
        toks = tokens(n, CONFIGS["mixed"]["vocab"], 300 + i)
        s = eng.new_sequence()
        assert s == 0
        cut = max(1, n - 40)
        rows = [eng.step([(s, toks[:cut])], [list(range(cut))]).cpu().numpy()]
        rows += [eng.step([(s, [t])], [[0]]).cpu().numpy() for t in toks[cut:]]
        eng.end_sequence(s)
        _check({(i, p): row for p, row in enumerate(np.concatenate(rows))}, {i: toks}, folder, dtype, f"request {i}")
    assert eng.cache.pages_in_use() == 0
    eng.close()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_from_the_first_token(tmp_path, dtype):
    """260 single-token steps of three sequences side by side (captured once, replayed): the windows of 40 and 100 and the
    blocks of 64 and 100 pass wholly over decoded tokens, their pages go back and come to other sequences, and the states
    are carried over hundreds of steps."""
    folder = make_folder(tmp_path, "mixed", seed=31)
    vocab = CONFIGS["mixed"]["vocab"]
    seqs = [tokens(260, vocab, 40), tokens(260, vocab, 41), tokens(150, vocab, 42)]
    eng = _engine(folder, dtype, max_tokens=3 * 320)
    slots = [eng.new_sequence() for _ in seqs]
    last = {}
    for t in range(260):
        live = [i for i, q in enumerate(seqs) if t < len(q)]
        out = eng.step([(slots[i], [seqs[i][t]]) for i in live], [[0]] * len(live)).cpu().numpy()
        for row, i in zip(out, live):
            last[(i, t)] = row
        for i in live:
            if t == len(seqs[i]) - 1:
                eng.end_sequence(slots[i])
    for i, q in enumerate(seqs):
        cfg, weights, ref = _plain(folder, q)
        tol = bound(dtype, cfg, weights, q, ref)
        firm = firm_rows(dtype, cfg, weights, q)
        errs = np.array([float(row_errors(last[(i, t)], ref[t])) for t in range(len(q))])
        assert firm[100:].sum() > 20 and errs[firm].max() < tol, (i, int(np.argmax(np.where(firm, errs, 0))), errs[firm].max(), tol)
    eng.close()


# ------------------------------------------------------------------ generation through the entry point and the command line

def _greedy_matches(folder, prompt, new, dtype):
    cfg, weights = load(folder)
    seq = list(prompt)
    for tok in new:
        logits = plain_lavutar.forward(cfg, weights, seq)[-1].numpy()
        best = int(np.argmax(logits))
        gap = (logits[best] - logits[tok]) / np.sqrt((logits ** 2).mean())
        # Where a router's choice at this position is a close call, a bfloat16 run may take the other expert and
        # so another token; the test goes on from the token that was generated.
        if firm_rows(dtype, cfg, weights, seq)[-1]:
            assert tok == best or (dtype == "bfloat16" and gap < 5e-2), (dtype, len(seq), tok, best, gap)
        seq.append(tok)


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_scheduler(tmp_path, dtype):
    """Engine.generate: unequal prompts in batches of three (the second batch in the first one's slots), greedy."""
    from longbow_quarrel_b200.sampling import SamplingParams
    folder = make_folder(tmp_path, "mixed", seed=41)
    vocab = CONFIGS["mixed"]["vocab"]
    prompts = [tokens(n, vocab, 500 + i) for i, n in enumerate([9, 1, 70, 2, 64])]
    eng = _engine(folder, dtype, max_tokens=3 * 128, max_batch=3)
    out = eng.generate(prompts, max_new_tokens=10, sampling=SamplingParams(temperature=0.0), stop_ids=[], batch_size=3)
    assert [len(o) for o in out] == [10] * 5
    for prompt, new in zip(prompts, out):
        _greedy_matches(folder, prompt, new, dtype)
    eng.close()


def test_the_command_line_generates_with_a_lavutar_folder(tmp_path):
    folder = make_folder(tmp_path, "odd", seed=51, keep_rank=False)
    prompt = tokens(12, CONFIGS["odd"]["vocab"], 7)
    proc = subprocess.run([str(ROOT / "bin" / "quarrel"), "-model", str(folder), "-prompt-ids", ",".join(map(str, prompt)),
                           "-n", "6", "-temp", "0", "-penalty", "1.0", "-dtype", "float32", "-output", "json"],
                          capture_output=True, text=True, timeout=600, env={**__import__("os").environ, "LQ_PYTHON": sys.executable})
    assert proc.returncode == 0, proc.stderr[-3000:]
    new = json.loads(proc.stdout.strip().splitlines()[-1])["output"][0]
    assert len(new) == 6
    _greedy_matches(folder, prompt, new, "float32")


def test_random_weights_from_a_configuration_and_the_kernels_that_served_it():
    """Engine.from_config builds the design from a dict with config.json's keys; in bfloat16 a prompt of seven hundred
    tokens and decoded tokens go through the design's kernels: attention on the tensor cores (tcgen05 for the prompt,
    the split kernel with its work list for single tokens) for the layers whose values are as wide as their keys, the scan
    in both of its forms, the layer norm that takes the two sides' branches, the experts of the prompt as row tiles of
    tcgen05 products and those of the decoded tokens through the streaming kernels."""
    from longbow_quarrel_b200.engine import Engine
    from longbow_quarrel_b200.kernels import ops
    from longbow_quarrel_b200.sampling import SamplingParams
    eng = Engine.from_config(CONFIGS["wide"], seed=3, max_tokens=2048, max_batch=2)
    before = ops.launches_by_name()
    out = eng.generate([[t % 300 for t in range(1, 701)], [4]], max_new_tokens=5, sampling=SamplingParams(temperature=0.0), stop_ids=[])
    ran = ops.launches_since(before)
    assert [len(o) for o in out] == [5, 5]
    for kernel in ("layernorm", "side_by_side", "rope_partial", "attn_prefill_tc", "attn_decode:teams", "linear_scan",
                   "linear_scan:single", "head_norm_gate", "small_proj", "moe_route", "group_rows_padded", "gather_rows",
                   "gemm_tc_grouped", "moe_combine", "moe_up", "moe_down", "gate_mul", "gated_act"):
        assert ran.get(kernel, 0) >= 1, (kernel, ran)
    assert ran.get("attention", 0) == 0, ran            # the plain attention kernel served no layer
    eng.close()
