"""The kernels that the Raritar design added or widened, each alone against a float64 restatement of its own
operation written here: attention with capped scores and kept first positions in all four attention kernels
(window edges, the kept positions' edge, pages that the cache has taken back, values of another size than keys),
the pair-hash embedding and the causal convolution with their per-sequence state, rotation of reordered pairs with
the value norm and the cache write, the softmax router with correction, groups and identity outputs, and the gated
experts' streaming products."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
BF16_ULP = 2.0 ** -8


def _ops():
    from longbow_quarrel_b200.kernels import ops
    return ops


def _i32(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


def _rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).to(DEV)


def _close(got, ref, tol, rel=0.0):
    got, ref = got.float().cpu().double(), ref.float().cpu().double()
    assert torch.isfinite(got).all()
    rms = ref.pow(2).mean().sqrt().clamp_min(1e-30)
    err = float((((got - ref).abs() - rel * ref.abs()) / rms).max())
    assert err < tol, err
    return err


def _close_on_average(got, ref, tol):
    """Rows that went through two roundings to bfloat16 on their way: the error's root mean square within `tol` of the
    reference's, and no single element further off than ten times that."""
    got, ref = got.float().cpu().double(), ref.float().cpu().double()
    assert torch.isfinite(got).all()
    rms = ref.pow(2).mean().sqrt().clamp_min(1e-30)
    assert float((got - ref).pow(2).mean().sqrt() / rms) < tol and float((got - ref).abs().max() / rms) < 10 * tol


# ------------------------------------------------------------------ a paged cache as a windowed sequence leaves it

class Cache:
    """Random keys [n, G, hd] and values [n, G, vd] of sequences of given lengths in shuffled pages.  `first_query`
    gives, per sequence, the lowest position that asks in the call: the pages that lie wholly below its window, and
    do not hold kept first positions, are taken back (their table entry is -1, their memory poisoned), as the cache
    manager does when a window has passed them."""

    def __init__(self, lens, G, hd, vd, dtype, seed, window=None, keep=0, first_query=None, page=64, poison=float("nan")):
        rng = np.random.default_rng(seed)
        self.lens, self.G, self.hd, self.vd, self.page = lens, G, hd, vd, page
        pages_per = [-(-n // page) for n in lens]
        n_pages = sum(pages_per) + 3
        perm = rng.permutation(n_pages)
        self.k = [_rand((n, G, hd), dtype, seed * 100 + i) for i, n in enumerate(lens)]
        self.v = [_rand((n, G, vd), dtype, seed * 100 + 50 + i) for i, n in enumerate(lens)]
        self.k_pages = torch.full((n_pages, G, page, hd), poison, dtype=dtype, device=DEV)
        self.v_pages = torch.full((n_pages, G, page, vd), poison, dtype=dtype, device=DEV)
        n_slots = len(lens) + 2
        self.slot_of = [int(s) for s in rng.permutation(n_slots)[:len(lens)]]
        table = np.full((n_slots, max(pages_per) + 1), -1, dtype=np.int32)
        nxt = 0
        for i, n in enumerate(lens):
            lowest = 0
            if window and first_query is not None:
                lowest = max(0, first_query[i] - window + 1) // page
            kept_pages = -(-keep // page) if window else 0
            for p in range(pages_per[i]):
                pg = int(perm[nxt]); nxt += 1
                if kept_pages <= p < lowest:
                    continue                                  # taken back: no entry, poisoned memory
                table[self.slot_of[i], p] = pg
                lo, hi = p * page, min(n, (p + 1) * page)
                self.k_pages[pg, :, :hi - lo] = self.k[i][lo:hi].transpose(0, 1)
                self.v_pages[pg, :, :hi - lo] = self.v[i][lo:hi].transpose(0, 1)
        self.table = torch.from_numpy(table).to(DEV)
        self.slots = _i32(self.slot_of)

    def plant(self, seq, pos, key):
        """Replace the key at a position (all key heads)."""
        pg = int(self.table[self.slot_of[seq], pos // self.page])
        assert pg >= 0
        self.k_pages[pg, :, pos % self.page] = key
        self.k[seq][pos, :] = key

    def reference(self, q, tok_seq, tok_pos, H, scale, window, keep, cap):
        """q [T, H, hd]: softmax(cap tanh(q.k scale / cap)) over the keys j <= p with p - j < window or j < keep."""
        out = torch.empty((q.shape[0], H, self.vd), dtype=torch.float64)
        per = H // self.G
        for r in range(q.shape[0]):
            s, p = tok_seq[r], tok_pos[r]
            js = [j for j in range(p + 1) if not window or p - j < window or j < keep]
            k, v = self.k[s][js].double().cpu(), self.v[s][js].double().cpu()
            for h in range(H):
                sc = (k[:, h // per] @ q[r, h].double().cpu()) * scale
                if cap:
                    sc = cap * torch.tanh(sc / cap)
                out[r, h] = torch.softmax(sc, 0) @ v[:, h // per]
        return out

    def tol(self, ref):
        vmax = max(float(v.float().abs().max()) for v in self.v)
        return 2.0 ** -8 * vmax / float(ref.pow(2).mean().sqrt())


# ------------------------------------------------------------------ capped, windowed attention with kept first positions

# H, G, hd, vd, window, kept first positions, cap
GENERAL = [(6, 2, 48, 40, 37, 5, 30.0),        # values narrower than keys
           (4, 4, 16, 24, 20, 33, None),       # more kept positions than the window is long; no cap
           (8, 1, 128, 128, 64, 64, 50.0),     # window and kept positions of exactly one page
           (2, 1, 256, 64, None, 0, 10.0),     # no window: a cap alone
           (3, 3, 10, 6, 1, 1, 2.0),           # a window of one token
           (4, 1, 64, 64, 40, 130, 20.0)]      # kept positions over three pages


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,hd,vd,window,keep,cap", GENERAL)
def test_plain_attention_caps_scores_and_keeps_first_positions(dtype, H, G, hd, vd, window, keep, cap):
    """Tokens at the first position, around the kept positions' edge, around the window's edge, where the window just
    leaves the kept positions behind, at page borders and far along, in one call."""
    ops = _ops()
    w, k = window or 50, keep
    lens = [400, 1, 200]
    case = Cache(lens, G, hd, vd, dtype, seed=2)
    pos0 = sorted({0, max(k - 1, 0), k, w - 1, w, w + k - 1, w + k, 63, 64, 127, 128, 399} - {-1})
    tok_seq = [0] * len(pos0) + [1, 2, 2]
    tok_pos = pos0 + [0, 199, min(w + k, 198)]
    q = _rand((len(tok_seq), H * hd + 16), dtype, 70)
    scale = 0.7 * hd ** -0.5
    out = ops.attention_plain(q, case.k_pages, case.v_pages, case.table, _i32(tok_pos), _i32(tok_seq), case.slots, H, G, hd,
                              case.page, scale, window, vd=vd, softcap=cap, keep_first=keep)
    ref = case.reference(q[:, :H * hd].reshape(-1, H, hd), tok_seq, tok_pos, H, scale, window, keep, cap)
    _close(out.reshape(-1, H, vd), ref, 3e-6 if dtype == torch.float32 else 1e-2)


# H, G, hd, window, kept first positions, cap: what the tensor-core kernels take (values as wide as keys)
FUSED = [(8, 2, 128, 100, 6, 50.0),
         (6, 2, 48, 37, 20, None),
         (4, 4, 16, 16, 16, 5.0),
         (40, 2, 64, 100, 70, 30.0),
         (3, 1, 32, None, 0, 8.0),
         (4, 1, 64, 44, 1, 45.0),
         (2, 2, 64, 33, 300, 12.0)]           # every key of the short sequences is a kept one


@pytest.mark.parametrize("H,G,hd,window,keep,cap", FUSED)
@pytest.mark.parametrize("n_splits", [1, 3])
def test_decode_attention_caps_scores_and_keeps_first_positions(H, G, hd, window, keep, cap, n_splits):
    """One token per sequence at its end; the pages between the kept ones and the window are gone."""
    ops = _ops()
    lens = [300, 1, 77, 64, 17, 1500, 33]
    tok_pos = [n - 1 for n in lens]
    case = Cache(lens, G, hd, hd, torch.bfloat16, seed=3, window=window, keep=keep, first_query=tok_pos)
    tok_seq = list(range(len(lens)))
    q = _rand((len(lens), (H + 2 * G) * hd), torch.bfloat16, 71)
    scale = 0.9 * hd ** -0.5
    ref = case.reference(q[:, :H * hd].reshape(-1, H, hd), tok_seq, tok_pos, H, scale, window, keep, cap)
    for early in (False, True):
        out = ops.attn_decode(q, case.k_pages, case.v_pages, case.table, _i32(tok_pos), _i32(tok_seq), case.slots, H, G, hd,
                              case.page, scale, window, n_splits, early_loads=early, softcap=cap, keep_first=keep)
        _close(out.reshape(-1, H, hd), ref, case.tol(ref), BF16_ULP)


@pytest.mark.parametrize("H,G,hd,window,keep,cap", FUSED)
@pytest.mark.parametrize("teams", [7, 40])
def test_decode_attention_with_a_work_list_counts_the_kept_tiles(H, G, hd, window, keep, cap, teams):
    """The balanced work list cuts each token's tiles, the kept ones ahead of the window's, into parts."""
    ops = _ops()
    from longbow_quarrel_b200.kernels.attention import MAX_SPLITS, cut_decode_work
    lens = [300, 1, 77, 64, 17, 1500, 33]
    tok_pos = [n - 1 for n in lens]
    case = Cache(lens, G, hd, hd, torch.bfloat16, seed=4, window=window, keep=keep, first_query=tok_pos)
    tok_seq = list(range(len(lens)))
    q = _rand((len(lens), (H + 2 * G) * hd), torch.bfloat16, 72)
    scale = hd ** -0.5
    ref = case.reference(q[:, :H * hd].reshape(-1, H, hd), tok_seq, tok_pos, H, scale, window, keep, cap)
    work = cut_decode_work(tok_pos, int(window or 0), teams, keep_first=keep)
    segs = work[teams + 1:].reshape(-1, 5)[:work[teams]]
    for b, p in enumerate(tok_pos):          # the parts of a token cover its counted tiles once
        first = max(0, p - window + 1) // 16 if window and p >= window else 0
        counted = p // 16 + 1 - first + (min(-(-keep // 16), first) if window else 0)
        mine = sorted((int(s[1]), int(s[2])) for s in segs if s[0] == b)
        assert mine[0][0] == 0 and mine[-1][1] == counted and all(a[1] == c[0] for a, c in zip(mine, mine[1:]))
    out = ops.attn_decode(q, case.k_pages, case.v_pages, case.table, _i32(tok_pos), _i32(tok_seq), case.slots, H, G, hd,
                          case.page, scale, window, min(MAX_SPLITS, teams), early_loads=True, work=_i32(work.tolist()),
                          teams=teams, softcap=cap, keep_first=keep)
    _close(out.reshape(-1, H, hd), ref, case.tol(ref), BF16_ULP)


def _blocks(new, past, rows):
    out, row = [], 0
    for b, (n, p) in enumerate(zip(new, past)):
        for r in range(0, n, rows):
            out.append((b, row + r, min(rows, n - r), p + r))
        row += n
    arr = np.asarray(out, dtype=np.int32)
    return tuple(torch.from_numpy(np.ascontiguousarray(arr[:, i])).to(DEV) for i in range(4))


@pytest.mark.parametrize("H,G,hd,window,keep,cap", FUSED)
def test_prompt_attention_caps_scores_and_keeps_first_positions(H, G, hd, window, keep, cap):
    """Three sequences in one call: one whole from its first token, one single token, one that goes on after 270 cached
    tokens (the pages that its window has passed are gone, the kept ones are not)."""
    ops = _ops()
    lens, new, past = [300, 1, 400], [300, 1, 130], [0, 0, 270]
    case = Cache(lens, G, hd, hd, torch.bfloat16, seed=5, window=window, keep=keep, first_query=past)
    tok_seq = [b for b, n in enumerate(new) for _ in range(n)]
    tok_pos = [p + i for n, p in zip(new, past) for i in range(n)]
    q = _rand((sum(new), (H + 2 * G) * hd), torch.bfloat16, 73)
    scale = 1.1 * hd ** -0.5
    out = ops.attn_prefill(q, case.k_pages, case.v_pages, case.table, case.slots, _i32(lens), _blocks(new, past, 64), H, G, hd,
                           64, scale, window, softcap=cap, keep_first=keep)
    ref = case.reference(q[:, :H * hd].reshape(-1, H, hd), tok_seq, tok_pos, H, scale, window, keep, cap)
    _close(out.reshape(-1, H, hd), ref, case.tol(ref), BF16_ULP)


@pytest.mark.parametrize("hd", [128, 64])
@pytest.mark.parametrize("H,G,window,keep,cap", [(8, 2, None, 0, 50.0), (4, 4, 100, 6, 30.0), (2, 1, 300, 130, None),
                                                 (4, 1, 40, 200, 20.0), (2, 2, 128, 128, 9.0)])
def test_tensor_core_prompt_attention_caps_scores_and_keeps_first_positions(H, G, window, keep, cap, hd):
    """The tcgen05 kernel, whose key tiles are two pages wide: a kept tile's second page may be one that was taken back."""
    ops = _ops()
    lens, new, past = [700, 1, 530], [700, 1, 260], [0, 0, 270]
    case = Cache(lens, G, hd, hd, torch.bfloat16, seed=6, window=window, keep=keep, first_query=past, poison=3.0e38)
    tok_seq = [b for b, n in enumerate(new) for _ in range(n)]
    tok_pos = [p + i for n, p in zip(new, past) for i in range(n)]
    q = _rand((sum(new), (H + 2 * G) * hd), torch.bfloat16, 74)
    scale = hd ** -0.5
    out = ops.attn_prefill_tc(q, case.k_pages, case.v_pages, case.table, case.slots, _i32(lens), _blocks(new, past, 128), H, G,
                              hd, 64, scale, window, softcap=cap, keep_first=keep)
    torch.cuda.synchronize()
    assert ops.attn_prefill_tc_status() == 0
    ref = case.reference(q[:, :H * hd].reshape(-1, H, hd), tok_seq, tok_pos, H, scale, window, keep, cap)
    _close(out.reshape(-1, H, hd), ref, case.tol(ref), BF16_ULP)


def _attend(kernel, case, q, n, hd, scale, window, keep, cap):
    """All n positions of sequence 0 as one prompt (or, for the decode kernel, the rows asked for, one token each)."""
    ops = _ops()
    args = (case.k_pages, case.v_pages, case.table)
    if kernel == "plain":
        return ops.attention_plain(q, *args, _i32(list(range(n))), _i32([0] * n), case.slots, 1, 1, hd, 64, scale, window,
                                   softcap=cap, keep_first=keep)
    if kernel == "decode":
        return torch.cat([ops.attn_decode(q[p:p + 1], *args, _i32([p]), _i32([0]), case.slots, 1, 1, hd, 64, scale, window, 2,
                                          softcap=cap, keep_first=keep) for p in range(n)])
    if kernel == "mma":
        return ops.attn_prefill(q, *args, case.slots, _i32([n]), _blocks([n], [0], 64), 1, 1, hd, 64, scale, window,
                                softcap=cap, keep_first=keep)
    return ops.attn_prefill_tc(q, *args, case.slots, _i32([n]), _blocks([n], [0], 128), 1, 1, hd, 64, scale, window,
                               softcap=cap, keep_first=keep)


@pytest.mark.parametrize("kernel", ["plain", "decode", "mma", "tc"])
def test_one_key_that_outweighs_all_others_shows_every_edge(kernel):
    """Keys are made to stand out for one query each: the last kept position and the first one that is not kept, seen from
    far along; the last key inside the window and the first one outside.  A row whose planted key is visible returns that
    key's value; a row whose planted key is hidden does not."""
    hd, n, W, K = 64, 400, 50, 6
    case = Cache([n], 1, hd, hd, torch.bfloat16, seed=7, poison=3.0e38 if kernel == "tc" else float("nan"))
    q = _rand((n, hd), torch.bfloat16, 75)
    plants = {(K - 1, 399): True, (K, 390): False, (300, 349): True, (250, 300): False, (0, 200): True}
    for (key_pos, row) in plants:
        qh = q[row].float()
        case.plant(0, key_pos, (qh / qh.norm() * 40.0).to(torch.bfloat16))
    out = _attend(kernel, case, q, n, hd, 0.125, W, K, 30.0)
    for (key_pos, row), seen in plants.items():
        gap = float((out[row].float() - case.v[0][key_pos, 0].float()).abs().max())
        assert (gap < 0.05) == seen, (key_pos, row, gap)
    ref = case.reference(q.reshape(n, 1, hd), [0] * n, list(range(n)), 1, 0.125, W, K, 30.0)
    _close(out.reshape(n, 1, hd), ref, 2 * case.tol(ref), BF16_ULP)


@pytest.mark.parametrize("kernel", ["plain", "decode", "mma", "tc"])
def test_two_keys_far_above_the_cap_share_the_weight(kernel):
    """Two planted keys score 150 and 300 before the cap of 10: capped, both score 10 and the row is the mean of their
    values; without the cap the larger one would take everything."""
    hd, n = 64, 200
    case = Cache([n], 1, hd, hd, torch.bfloat16, seed=8, poison=3.0e38 if kernel == "tc" else float("nan"))
    q = _rand((n, hd), torch.bfloat16, 76, scale=0.1)
    qh = q[n - 1].float()
    unit = qh / qh.norm() / float(qh.norm())
    case.plant(0, 20, (unit * 150.0).to(torch.bfloat16))
    case.plant(0, 150, (unit * 300.0).to(torch.bfloat16))
    capped = _attend(kernel, case, q, n, hd, 1.0, None, 0, 10.0)[n - 1].float()
    free = _attend(kernel, case, q, n, hd, 1.0, None, 0, None)[n - 1].float()
    v1, v2 = case.v[0][20, 0].float(), case.v[0][150, 0].float()
    others = (n - 2) * math.exp(1.0 - 10.0)                  # what all other keys together can weigh against e^10 each
    assert float((capped - (v1 + v2) / 2).abs().max()) < 0.03 + others * 4
    assert float((free - v2).abs().max()) < 0.03


# ------------------------------------------------------------------ embedding by pairs, convolution: state between steps

def _step_lists(rows_per_seq, past, slots):
    """tok_pos, tok_seq, cu_rows of a step in which sequence b brings rows_per_seq[b] rows after past[b] tokens."""
    tok_pos = [p + i for n, p in zip(rows_per_seq, past) for i in range(n)]
    tok_seq = [b for b, n in enumerate(rows_per_seq) for _ in range(n)]
    cu = [0] + list(np.cumsum(rows_per_seq))
    return _i32(tok_pos), _i32(tok_seq), _i32(cu), _i32(slots)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("buckets,a,b", [(1019, 37, 11), (7, 1, 1), (50, 0, 3), (64, 1000003, 999983)])
def test_pair_embedding_remembers_each_sequences_last_token(dtype, buckets, a, b):
    """Three sequences in slots 4, 0 and 2 over three steps of unequal portions (one of them a single token): the row
    of the second table comes from the token before, which for a step's first row is the one the state holds; a
    sequence's first token takes the table's last row whatever an earlier owner of its slot left in the state."""
    ops = _ops()
    V, D = 300, 24
    table, pairs = _rand((V, D), dtype, 1), _rand((buckets + 1, D), dtype, 2)
    rng = np.random.default_rng(3)
    seqs = [rng.integers(0, V, size=n).tolist() for n in (9, 4, 12)]
    slots = [4, 0, 2]
    last = torch.full((6,), 123, dtype=torch.int32, device=DEV)           # what earlier owners left behind
    done = [0, 0, 0]
    for portions in ([3, 1, 7], [5, 1, 1], [1, 2, 4]):
        tok_pos, tok_seq, cu, sl = _step_lists(portions, done, slots)
        toks = [t for s, d, n in zip(seqs, done, portions) for t in s[d:d + n]]
        out = ops.embedding_pairs(table, pairs, buckets, a, b, _i32(toks), tok_pos, tok_seq, sl, cu, last, 3)
        want = []
        for s, d, n in zip(seqs, done, portions):
            for i in range(d, d + n):
                row = buckets if i == 0 else (s[i - 1] * a + s[i] * b) % buckets
                want.append(table[s[i]].double() + pairs[row].double())
        _close(out, torch.stack(want), 1e-6)
        done = [d + n for d, n in zip(done, portions)]
        assert [int(last[s]) for s in slots] == [s[d - 1] for s, d in zip(seqs, done)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps,add", [(4, True), (2, True), (7, False), (1, True)])
@pytest.mark.parametrize("D,by_taps", [(40, True), (40, False), (42, True), (2056, True)])   # 16-byte pieces of channels (with the
# weight by taps) and one channel a thread; a width without whole pieces; more than a block of threads covers
def test_causal_convolution_carries_its_last_rows_between_steps(dtype, taps, add, D, by_taps):
    """Portions of 1, 2, 3 and more rows (shorter and longer than the taps) of three sequences against the convolution of
    each whole sequence; the state of a slot's earlier owner is not read at a sequence's start."""
    ops = _ops()
    w = _rand((D, taps), torch.float32, 5, scale=0.5)
    lens = [11, 6, 17]
    hs = [_rand((n, D), dtype, 10 + i) for i, n in enumerate(lens)]
    slots = [1, 3, 0]
    state = torch.full((5, max(taps - 1, 1), D), 77.0, dtype=torch.float32, device=DEV)[:, :taps - 1].contiguous() if taps > 1 else None
    done, got = [0, 0, 0], [[], [], []]
    for portions in ([1, 2, 3], [2, 1, 1], [5, 3, 9], [3, 0, 4]):
        live = [i for i, n in enumerate(portions) if n]
        tok_pos, tok_seq, cu, sl = _step_lists([portions[i] for i in live], [done[i] for i in live], [slots[i] for i in live])
        h = torch.cat([hs[i][done[i]:done[i] + portions[i]] for i in live])
        if done[live[0]] == 0 and state is not None:
            # The engine zeroes a slot's state when a sequence starts in it; here the kernel is given the positions.
            for i in live:
                state[slots[i]] = 0
        out = ops.causal_conv(h, w, state, tok_seq, sl, cu, len(live), add, w_by_taps=w.t().contiguous() if by_taps else None)
        at = 0
        for i in live:
            got[i].append(out[at:at + portions[i]])
            at += portions[i]
            done[i] += portions[i]
    for i, n in enumerate(lens):
        h = hs[i].double().cpu()
        ref = h.clone() if add else torch.zeros_like(h)
        for t in range(n):
            for j in range(taps):
                s = t - taps + 1 + j
                if s >= 0:
                    ref[t] += w[:, j].double().cpu() * h[s]
        _close(torch.cat(got[i]), ref, 2e-6 if dtype == torch.float32 else 1e-6, 0.0 if dtype == torch.float32 else BF16_ULP)


# ------------------------------------------------------------------ rotation of a part of a head, value norm, cache write

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,hd,vd,rot,eps", [(4, 2, 16, 24, 8, 1e-5), (1, 1, 12, 20, 12, 1e-6), (3, 3, 8, 8, 0, 1e-2),
                                               (8, 2, 64, 64, 48, 1e-5)])
def test_rotation_value_norm_and_cache_write(dtype, H, G, hd, vd, rot, eps):
    """Rows [q | k | v] of three sequences at scattered positions: the first `rot` dimensions of every query and key head
    are rotated as halves (i, i + rot / 2) by the token's position, the rest pass; every value head is divided by its root
    mean square; keys and values land in their pages at the token's place, and nothing else in the cache moves."""
    ops = _ops()
    page, n_pos = 64, 200
    tok_seq, tok_pos = [0, 0, 0, 1, 2, 2], [0, 63, 64, 5, 130, 199]
    slots = [2, 0, 1]
    T, width = len(tok_pos), (H + G) * hd + G * vd
    rows = _rand((T, width), dtype, 20)
    freqs = torch.tensor([50.0 ** (-2.0 * i / max(rot, 2)) for i in range(rot // 2)], dtype=torch.float64)
    ang = torch.arange(n_pos, dtype=torch.float64)[:, None] * freqs
    cos, sin = torch.cos(ang).float().to(DEV).contiguous(), torch.sin(ang).float().to(DEV).contiguous()
    table = torch.full((3, 4), -1, dtype=torch.int32)
    nxt = 0
    for s, p in zip(tok_seq, tok_pos):
        if table[slots[s], p // page] < 0:
            table[slots[s], p // page] = nxt
            nxt += 1
    table = table.to(DEV)
    k_pages = torch.full((nxt, G, page, hd), 9.0, dtype=dtype, device=DEV)
    v_pages = torch.full((nxt, G, page, vd), 9.0, dtype=dtype, device=DEV)
    src = rows.double().cpu()
    buf = rows.clone()
    ops.rope_partial(buf, None, cos if rot else None, sin if rot else None, rot, _i32(tok_pos), _i32(tok_seq), _i32(slots), table,
                     k_pages, v_pages, H + G, H, G, hd, vd, (H + G) * hd, page, v_unit_eps=eps)
    tol, rel = (2e-6, 0.0) if dtype == torch.float32 else (1e-6, BF16_ULP)
    written = 0
    for r, (s, p) in enumerate(zip(tok_seq, tok_pos)):
        heads = src[r, :(H + G) * hd].reshape(H + G, hd).clone()
        a, b = heads[:, :rot // 2].clone(), heads[:, rot // 2:rot].clone()
        c, sn = torch.cos(ang[p]), torch.sin(ang[p])
        heads[:, :rot // 2], heads[:, rot // 2:rot] = a * c - b * sn, b * c + a * sn
        _close(buf[r, :H * hd].reshape(H, hd), heads[:H], tol, rel)
        pg = int(table[slots[s], p // page])
        _close(k_pages[pg, :, p % page], heads[H:], tol, rel)
        v = src[r, (H + G) * hd:].reshape(G, vd)
        _close(v_pages[pg, :, p % page], v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps), tol, rel)
        written += 1
    assert int((k_pages != 9.0).any(-1).sum()) <= written * G and int((v_pages != 9.0).any(-1).sum()) <= written * G


# ------------------------------------------------------------------ the router

def _route_ref(z, corr, groups, keep, top):
    """Softmax scores; the choice by score + correction inside the `keep` groups whose best choice score is largest;
    the weights are the chosen plain scores.  Returns (chosen, weights, margin to the nearest other outcome)."""
    s = torch.softmax(z.double(), 0)
    c = (s + corr.double()).tolist()
    n = len(c)
    per = n // groups
    gs = [max(c[g * per:(g + 1) * per]) for g in range(groups)]
    order = sorted(range(groups), key=lambda g: (-gs[g], g))
    kept = set(order[:keep])
    allowed = sorted((e for e in range(n) if e // per in kept), key=lambda e: (-c[e], e))
    margin = gs[order[keep - 1]] - gs[order[keep]] if keep < groups else math.inf
    if len(allowed) > top:
        margin = min(margin, c[allowed[top - 1]] - c[allowed[top]])
    return allowed[:top], [float(s[e]) for e in allowed[:top]], margin


@pytest.mark.parametrize("n,groups,keep,top", [(12, 4, 3, 4), (8, 4, 2, 3), (6, 1, 1, 2), (16, 4, 1, 4), (4, 2, 2, 4), (5, 5, 2, 1),
                                               (64, 8, 4, 8)])
def test_router_softmax_correction_and_groups_by_their_best_member(n, groups, keep, top):
    """300 tokens: the chosen set equals the float64 rule wherever that rule's decision is not a close call; the weights are
    the plain softmax scores times the scale, in the order of the choice scores; corrections include negative ones large
    enough that every choice score of some kept group is below zero."""
    ops = _ops()
    T = 300
    z = _rand((T, n + 1), torch.float32, 30, scale=2.0)                 # one more column rides along, as the shared gate does
    corr = _rand((n,), torch.float32, 31, scale=0.3) - 0.4
    ids, weights = ops.moe_route(z, n, groups, keep, top, 0.5, score="softmax", correction=corr, group_rule="max", normalize=False)
    ids, weights = ids.cpu(), weights.cpu()
    firm = 0
    for t in range(T):
        chosen, w, margin = _route_ref(z[t, :n].cpu(), corr.cpu(), groups, keep, top)
        if margin < 1e-5:
            continue
        firm += 1
        assert ids[t].tolist() == chosen, (t, ids[t].tolist(), chosen)
        assert np.allclose(weights[t].numpy(), 0.5 * np.asarray(w), rtol=2e-6, atol=1e-9)
    assert firm > 250
    plain_ids, plain_w = ops.moe_route(z, n, groups, keep, top, 1.0, score="softmax", group_rule="max", normalize=False)
    for t in range(0, T, 7):
        chosen, w, margin = _route_ref(z[t, :n].cpu(), torch.zeros(n), groups, keep, top)
        if margin >= 1e-5:
            assert plain_ids[t].tolist() == chosen and np.allclose(plain_w[t].cpu().numpy(), w, rtol=2e-6)


# ------------------------------------------------------------------ gated experts, identity experts, the multiplier

def _experts_ref(h, w_up, w_down, ids, weights, E, shared, zs, shared_scale):
    """float64: sum over the chosen of weight * (W_down (silu(W_gate h) * (W_up h))), or weight * h for an identity
    expert; plus shared_scale * sigmoid(zs) * shared."""
    T, D = h.shape
    F = w_up.shape[1] // 2
    out = torch.zeros((T, D), dtype=torch.float64)
    for t in range(T):
        x = h[t].double().cpu()
        for e, w in zip(ids[t].tolist(), weights[t].tolist()):
            if e >= E:
                out[t] += w * x
                continue
            gu = w_up[e].double().cpu() @ x
            u = torch.nn.functional.silu(gu[:F]) * gu[F:]
            u = u.to(h.dtype).double()                                    # the products hand their rows on in the rows' dtype
            out[t] += w * (w_down[e].double().cpu() @ u)
        if shared is not None:
            out[t] += shared_scale * torch.sigmoid(zs[t].double().cpu()) * shared[t].double().cpu()
    return out


def _expert_case(T, D, F, E, identity, top, dtype, seed):
    rng = np.random.default_rng(seed)
    h = _rand((T, D), dtype, seed)
    w_up = _rand((E, 2 * F, D), dtype, seed + 1, scale=D ** -0.5)
    w_down = _rand((E, D, F), dtype, seed + 2, scale=F ** -0.5)
    ids = torch.tensor(np.stack([rng.permutation(E + identity)[:top] for _ in range(T)]), dtype=torch.int32, device=DEV)
    weights = torch.rand((T, top), device=DEV, dtype=torch.float32) * 0.5
    shared = _rand((T, D), torch.float32, seed + 3)
    zs = _rand((T, 3), torch.float32, seed + 4)[:, 1]                     # a strided column, as the router's product leaves it
    return h, w_up, w_down, ids, weights, shared, zs


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,D,F,E,identity,top", [(1, 64, 32, 6, 2, 3), (5, 40, 16, 1, 3, 4), (16, 128, 48, 13, 3, 4), (3, 100, 24, 3, 0, 3)])
def test_streamed_gated_experts_pass_identity_inputs_on(dtype, T, D, F, E, identity, top):
    ops = _ops()
    h, w_up, w_down, ids, weights, shared, zs = _expert_case(T, D, F, E, identity, top, dtype, 40)
    ref = _experts_ref(h, w_up, w_down, ids, weights, E, shared, zs, 0.7)
    x0 = _rand((T, D), torch.float32, 49)
    u = ops.moe_up(h, w_up, ids, "silu", gated=True)
    if F % 8 == 0:          # the same rows with gate and up by turns in blocks of 8: the same u
        from longbow_quarrel_b200.kernels.linear import interleave_gate_up
        turns = torch.stack([interleave_gate_up(w[:F], w[F:]) for w in w_up])
        real = (ids < E).cpu()
        assert torch.equal(ops.moe_up(h, turns, ids, "silu", gated=True, block=8).cpu()[real], u.cpu()[real])
    for accumulate in (False, True):
        x = x0.clone()
        ops.moe_down(u, w_down, ids, weights, x, accumulate=accumulate, shared=shared, shared_gate=zs,
                     h=h if identity else None, shared_scale=0.7)
        want = ref + (x0.double().cpu() if accumulate else 0.0)
        _close(x, want, 5e-6 if dtype == torch.float32 else 4e-3)


@pytest.mark.parametrize("T,D,F,E,identity,top", [(700, 128, 48, 13, 3, 4), (300, 64, 32, 6, 2, 3), (520, 256, 64, 2, 2, 1)])
def test_grouped_gated_experts_leave_identity_pairs_out_of_the_products(T, D, F, E, identity, top):
    """A prompt's (token, choice) pairs through both grouped forms -- row tiles of the tcgen05 product padded per expert,
    and the listed mma.sync product -- against float64: pairs that chose an identity output take no place in the padded
    order, have no tile, and come back as the token's own input times the weight."""
    ops = _ops()
    h, w_up, w_down, ids, weights, shared, zs = _expert_case(T, D, F, E, identity, top, torch.bfloat16, 50)
    ref = _experts_ref(h, w_up, w_down, ids, weights, E, shared, zs, 0.5)
    more = dict(ids=ids, E=E, h=h) if identity else {}
    src, dst, tile_group = ops.group_rows_padded(ids.view(-1), E)
    flat, place = ids.view(-1).cpu(), dst.cpu()
    assert ((place < 0) == (flat >= E)).all() and len(set(place[place >= 0].tolist())) == int((flat < E).sum())
    groups = tile_group.cpu()
    assert all(int(groups[int(p) // 128]) == int(e) for p, e in zip(place.tolist(), flat.tolist()) if p >= 0)
    from longbow_quarrel_b200.kernels.linear import interleave_gate_up
    turns = torch.stack([interleave_gate_up(w[:F], w[F:]) for w in w_up])
    u = ops.gemm_tc_grouped(ops.gather_rows(h, src, top), turns, tile_group, h.dtype, swiglu=True)     # silu(gate) * up in the epilogue
    assert tuple(u.shape) == (src.numel(), F)
    y = ops.gemm_tc_grouped(u, w_down, tile_group, torch.float32)
    torch.cuda.synchronize()
    assert ops.gemm_tc_status() == 0
    out = ops.moe_combine(y, weights, torch.empty((T, D), dtype=torch.float32, device=DEV), accumulate=False, shared=shared,
                          shared_gate=zs, place=dst, shared_scale=0.5, **more)
    _close_on_average(out, ref, 4e-3)
    listed = ops.group_rows(ids.view(-1), E + identity)
    u = torch.empty((T * top, 2 * F), dtype=h.dtype, device=DEV)
    ops.grouped_gemm(h, w_up, u, listed=listed, a_div=top)
    y = torch.full((T * top, D), float("nan"), dtype=torch.float32, device=DEV)
    ops.grouped_gemm(ops.gated_act(u, None, "silu", h.dtype), w_down, y, listed=listed)
    x0 = _rand((T, D), torch.float32, 59)
    out = ops.moe_combine(y, weights, x0.clone(), accumulate=True, shared=shared, shared_gate=zs, shared_scale=0.5, **more)
    _close_on_average(out, ref + x0.double().cpu(), 4e-3)


# ------------------------------------------------------------------ a branch joins the stream, and the next norm, in one kernel

@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,D", [(5, 64), (3, 100), (2, 42), (4, 2048), (1, 8192 + 4)])
def test_scaled_add_and_norm_in_one_pass_equal_the_two_kernels(out_dtype, T, D):
    """x += m y and the rows of the norm that follows: bit for bit what add_scaled and rmsnorm give one after the other
    (widths by float4 pieces, not, and wider than the kernel's registers hold), and close to float64."""
    ops = _ops()
    x, y, gain = _rand((T, D), torch.float32, 60), _rand((T, D), torch.float32, 61), _rand((D,), torch.float32, 62) + 1.0
    two = x.clone()
    ops.add_scaled(two, y, 0.7)
    rows_two = ops.rmsnorm(two, gain, 1e-5, out_dtype)
    one = x.clone()
    rows_one = ops.add_scaled_norm(one, y, 0.7, gain, 1e-5, out_dtype)
    assert torch.equal(one, two) and torch.equal(rows_one, rows_two)
    ref = x.double().cpu() + 0.7 * y.double().cpu()
    _close(one, ref, 1e-6)
    want = ref / torch.sqrt((ref * ref).mean(-1, keepdim=True) + 1e-5) * gain.double().cpu()
    _close(rows_one, want, 3e-6 if out_dtype == torch.float32 else 1e-6, 0.0 if out_dtype == torch.float32 else BF16_ULP)
