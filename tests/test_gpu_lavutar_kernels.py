"""The kernels that the Lavutar design added or widened, each alone against a float64 restatement of its own operation
written here: layer norm (alone, on chosen rows, with branches joining the stream in the same pass), the two streams
side by side, unit norms of q and k (per head and over the whole projection) with the query temperature ahead of the
rotation and the cache write, gates of one number per head, attention over blocks of positions in all four attention
kernels (block edges, page borders, pages that the cache has taken back, a far key inside a long block), and the
matrix-state scan with a decay for every key channel (whole, in pieces, token by token, decays of exactly one)."""
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


# ------------------------------------------------------------------ layer norm, two streams side by side, gates per head

@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D", [1, 44, 192, 1000, 4100])
def test_layer_norm_alone_on_rows_and_with_branches(out_dtype, D):
    ops = _ops()
    T = 9
    x = _rand((T, D), torch.float32, 1, 3.0) + 5.0            # a mean far from zero: the deviations are taken from it
    g, b = _rand((D,), torch.float32, 2) + 1.0, _rand((D,), torch.float32, 3)
    eps = 1e-5
    ref = torch.nn.functional.layer_norm(x.double().cpu(), (D,), g.double().cpu(), b.double().cpu(), eps)
    tol = 3e-6 if out_dtype == torch.float32 else 1.5 * BF16_ULP
    rel = 0.0 if out_dtype == torch.float32 else BF16_ULP
    _close(ops.layernorm(x, g, b, eps, out_dtype), ref, tol, rel)
    rows = [7, 0, 3]
    _close(ops.layernorm(x, g, b, eps, out_dtype, rows=_i32(rows)), ref[rows], tol, rel)
    y1, y2 = _rand((T, D), torch.float32, 4), _rand((T, D), torch.float32, 5)
    for add in (((y1, 0.8),), ((y1, 0.8), (y2, -0.5))):
        xs = x.clone()
        want = x.double().cpu() + sum(m * y.double().cpu() for y, m in add)
        out = ops.layernorm(xs, g, b, eps, out_dtype, add=add)
        _close(xs, want, 1e-6)                               # the stream took the branches
        _close(out, torch.nn.functional.layer_norm(want, (D,), g.double().cpu(), b.double().cpu(), eps), tol, rel)


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_two_streams_side_by_side(out_dtype):
    ops = _ops()
    a, b = _rand((5, 36), torch.float32, 1), _rand((5, 36), torch.float32, 2)
    out = ops.side_by_side(a, b, out_dtype)
    assert out.shape == (5, 72) and torch.equal(out, torch.cat([a, b], dim=1).to(out_dtype))


@pytest.mark.parametrize("dtype,gdtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16), (torch.bfloat16, torch.float32)])
def test_a_gate_of_one_number_per_head(dtype, gdtype):
    ops = _ops()
    rows, H, vd = 7, 3, 20
    x = _rand((rows, H * vd), dtype, 1)
    wide = _rand((rows, 50), gdtype, 2)
    gate = wide[:, 11:11 + H]                                 # rows are strided
    ref = x.double().cpu().reshape(rows, H, vd) * torch.sigmoid(gate.double().cpu())[:, :, None]
    out = ops.gate_mul(x.clone(), gate, "sigmoid", group=vd)
    _close(out.reshape(rows, H, vd), ref, 1e-6 if dtype == torch.float32 else BF16_ULP, BF16_ULP if dtype != torch.float32 else 0.0)


# ------------------------------------------------------------------ unit norms of q and k, query temperature, rotation, cache write

@pytest.mark.parametrize("mode", ["head", "all"])
@pytest.mark.parametrize("in_dtype,out_dtype", [(torch.float32, torch.float32), (torch.float32, torch.bfloat16)])
@pytest.mark.parametrize("H,G,hd,vd,rot,temp", [(4, 2, 16, 24, 8, (0.3, 4)), (3, 1, 64, 64, 0, None), (2, 2, 10, 6, 0, (1.5, 1)),
                                                (8, 1, 32, 16, 32, None)])
def test_unit_norms_and_query_temperature_ahead_of_rotation_and_cache_write(mode, in_dtype, out_dtype, H, G, hd, vd, rot, temp):
    ops = _ops()
    page, eps = 64, 1e-5
    tok_pos = [0, 1, 63, 64, 3, 130, 7]
    tok_seq = [0, 0, 0, 0, 1, 1, 1]
    slots = [2, 0]
    T = len(tok_pos)
    width = (H + G) * hd + G * vd + 5
    buf = _rand((T, width), in_dtype, 1, 2.0)
    half = rot // 2
    cos = torch.rand((200, max(half, 1)), device=DEV) if rot else None
    sin = torch.rand((200, max(half, 1)), device=DEV) if rot else None
    w = (_rand(((H + G) * hd,), torch.float32, 2) + 1.0) if mode == "all" else None
    table = torch.tensor([[5, 1, 3], [-1, -1, -1], [0, 2, 4]], dtype=torch.int32, device=DEV)
    k_pages = torch.zeros((6, G, page, hd), dtype=out_dtype, device=DEV)
    v_pages = torch.zeros((6, G, page, vd), dtype=out_dtype, device=DEV)
    q_out = torch.zeros((T, H * hd), dtype=out_dtype, device=DEV)
    src = buf.clone()
    ops.rope_partial(buf, None, cos, sin, rot, _i32(tok_pos), _i32(tok_seq), _i32(slots), table, k_pages, v_pages, H + G, H, G, hd,
                     vd, (H + G) * hd, page, qout=q_out, unit_norm=mode, norm_weight=w, norm_eps=eps, q_temp=temp)
    x = src.double().cpu()
    heads = x[:, :(H + G) * hd].reshape(T, H + G, hd)
    if mode == "head":
        heads = heads / torch.sqrt((heads ** 2).mean(-1, keepdim=True) + eps)
    else:
        q, k = x[:, :H * hd], x[:, H * hd:(H + G) * hd]
        q = q / torch.sqrt((q ** 2).mean(-1, keepdim=True) + eps) * w[:H * hd].double().cpu()
        k = k / torch.sqrt((k ** 2).mean(-1, keepdim=True) + eps) * w[H * hd:].double().cpu()
        heads = torch.cat([q, k], dim=1).reshape(T, H + G, hd)
    if temp is not None:
        mult = torch.tensor([1.0 + temp[0] * math.log((p + 1) // temp[1] + 1.0) for p in tok_pos], dtype=torch.float64)
        heads[:, :H] = heads[:, :H] * mult[:, None, None]
    if rot:
        c = cos.double().cpu()[tok_pos][:, None, :half]
        s = sin.double().cpu()[tok_pos][:, None, :half]
        u, v = heads[..., :half].clone(), heads[..., half:rot].clone()
        heads[..., :half], heads[..., half:rot] = u * c - v * s, v * c + u * s
    tol, rel = (3e-6, 0.0) if out_dtype == torch.float32 else (BF16_ULP, BF16_ULP)
    _close(q_out.reshape(T, H, hd), heads[:, :H], tol, rel)
    for r, (p, b) in enumerate(zip(tok_pos, tok_seq)):
        pg = int(table[slots[b], p // page])
        _close(k_pages[pg, :, p % page], heads[r, H:], tol, rel)
        _close(v_pages[pg, :, p % page], x[r, (H + G) * hd:(H + G) * hd + G * vd].reshape(G, vd), tol, rel)


# ------------------------------------------------------------------ a paged cache as a sequence with blocks leaves it

class Pages:
    """Random keys [n, G, hd] and values [n, G, vd] of sequences of given lengths in shuffled pages.  `first_query` gives,
    per sequence, the lowest position that asks in the call: the pages that lie wholly below the first key that position
    sees are taken back (their table entry is -1, their memory poisoned), as the cache manager does."""

    def __init__(self, lens, G, hd, vd, dtype, seed, block=None, first_query=None, page=64, poison=float("nan")):
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
            if block and first_query is not None:
                lowest = (first_query[i] - first_query[i] % block) // page
            for p in range(pages_per[i]):
                pg = int(perm[nxt]); nxt += 1
                if p < lowest:
                    continue                                  # taken back: no entry, poisoned memory
                table[self.slot_of[i], p] = pg
                lo, hi = p * page, min(n, (p + 1) * page)
                self.k_pages[pg, :, :hi - lo] = self.k[i][lo:hi].transpose(0, 1)
                self.v_pages[pg, :, :hi - lo] = self.v[i][lo:hi].transpose(0, 1)
                if poison == poison:                          # a finite poison: rows beyond the sequence's end are zero, as the cache leaves them
                    self.k_pages[pg, :, hi - lo:] = 0
                    self.v_pages[pg, :, hi - lo:] = 0
        self.table = torch.from_numpy(table).to(DEV)
        self.slots = _i32(self.slot_of)

    def plant(self, seq, pos, key):
        pg = int(self.table[self.slot_of[seq], pos // self.page])
        assert pg >= 0
        self.k_pages[pg, :, pos % self.page] = key
        self.k[seq][pos, :] = key

    def reference(self, q, tok_seq, tok_pos, H, scale, block, cap=None, sink=None):
        """q [T, H, hd]: softmax (with exp(sink_h) in the denominator) over the keys j <= p of p's block."""
        out = torch.empty((q.shape[0], H, self.vd), dtype=torch.float64)
        per = H // self.G
        for r in range(q.shape[0]):
            s, p = tok_seq[r], tok_pos[r]
            js = [j for j in range(p + 1) if not block or j // block == p // block]
            k, v = self.k[s][js].double().cpu(), self.v[s][js].double().cpu()
            for h in range(H):
                sc = (k[:, h // per] @ q[r, h].double().cpu()) * scale
                if cap:
                    sc = cap * torch.tanh(sc / cap)
                if sink is not None:
                    sc = torch.cat([sc, sink[h:h + 1].double().cpu()])
                    out[r, h] = torch.softmax(sc, 0)[:-1] @ v[:, h // per]
                else:
                    out[r, h] = torch.softmax(sc, 0) @ v[:, h // per]
        return out

    def tol(self, ref):
        vmax = max(float(v.float().abs().max()) for v in self.v)
        return 2.0 ** -8 * vmax / float(ref.pow(2).mean().sqrt())


def _blocks(new, past, rows):
    out, row = [], 0
    for b, (n, p) in enumerate(zip(new, past)):
        for r in range(0, n, rows):
            out.append((b, row + r, min(rows, n - r), p + r))
        row += n
    arr = np.asarray(out, dtype=np.int32)
    return tuple(torch.from_numpy(np.ascontiguousarray(arr[:, i])).to(DEV) for i in range(4))


# H, G, hd, vd, block, cap
GENERAL = [(6, 2, 48, 40, 37, 30.0), (4, 4, 16, 24, 64, None), (8, 1, 64, 32, 100, 50.0), (3, 3, 10, 6, 1, 2.0), (2, 1, 256, 64, 200, None),
           (5, 5, 7, 9, 13, None)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,hd,vd,block,cap", GENERAL)
def test_plain_attention_over_blocks_with_a_sink_and_a_gate_per_head(dtype, H, G, hd, vd, block, cap):
    """Tokens at the first position, at the last position of a block and the first of the next, at page borders and far
    along, in one call; a learned term in the denominator and one gate per head."""
    ops = _ops()
    lens = [400, 1, 200]
    case = Pages(lens, G, hd, vd, dtype, seed=2)
    pos0 = sorted({0, block - 1, block, 2 * block - 1, 2 * block, 63, 64, 127, 128, 399, 399 - 399 % block} & set(range(400)))
    tok_seq = [0] * len(pos0) + [1, 2, 2]
    tok_pos = pos0 + [0, 199, min(block, 198)]
    q = _rand((len(tok_seq), H * hd + 16), dtype, 70)
    gate = _rand((len(tok_seq), H + 3), dtype, 71)[:, 1:1 + H]
    sink = _rand((H,), torch.float32, 72)
    scale = 0.7 * hd ** -0.5
    out = ops.attention_plain(q, case.k_pages, case.v_pages, case.table, _i32(tok_pos), _i32(tok_seq), case.slots, H, G, hd,
                              case.page, scale, None, vd=vd, softcap=cap, chunk=block, sink=sink, gate=gate, gate_per_head=True)
    ref = case.reference(q[:, :H * hd].reshape(-1, H, hd), tok_seq, tok_pos, H, scale, block, cap, sink)
    ref = ref * torch.sigmoid(gate.double().cpu())[:, :, None]
    if dtype == torch.float32:
        _close(out.reshape(-1, H, vd), ref, 3e-6)
    else:
        _close(out.reshape(-1, H, vd), ref, 1e-2, BF16_ULP)      # beyond the rounding of each output to bfloat16


# H, G, hd, block, cap: what the tensor-core kernels take (values as wide as keys)
FUSED = [(8, 2, 128, 100, 50.0), (6, 2, 48, 37, None), (4, 4, 16, 16, 5.0), (12, 2, 64, 200, 30.0), (3, 1, 32, 1, None),
         (4, 1, 64, 70, None), (2, 2, 64, 64, 12.0), (2, 1, 64, 1000, None)]


@pytest.mark.parametrize("H,G,hd,block,cap", FUSED)
@pytest.mark.parametrize("n_splits", [1, 3])
def test_decode_attention_over_blocks(H, G, hd, block, cap, n_splits):
    """One token per sequence at its end; the pages below its block are gone."""
    ops = _ops()
    lens = [300, 1, 77, 64, 17, 1500, 33, 201, 200]
    tok_pos = [n - 1 for n in lens]
    case = Pages(lens, G, hd, hd, torch.bfloat16, seed=3, block=block, first_query=tok_pos)
    tok_seq = list(range(len(lens)))
    q = _rand((len(lens), (H + 2 * G) * hd), torch.bfloat16, 71)
    sink = _rand((H,), torch.float32, 73)
    scale = 0.9 * hd ** -0.5
    ref = case.reference(q[:, :H * hd].reshape(-1, H, hd), tok_seq, tok_pos, H, scale, block, cap, sink)
    for early in (False, True):
        out = ops.attn_decode(q, case.k_pages, case.v_pages, case.table, _i32(tok_pos), _i32(tok_seq), case.slots, H, G, hd,
                              case.page, scale, ops.span(None, block), n_splits, early_loads=early, softcap=cap, sink=sink)
        _close(out.reshape(-1, H, hd), ref, case.tol(ref), BF16_ULP)


@pytest.mark.parametrize("H,G,hd,block,cap", FUSED)
@pytest.mark.parametrize("teams", [9, 40])
def test_decode_attention_over_blocks_from_a_work_list(H, G, hd, block, cap, teams):
    ops = _ops()
    from longbow_quarrel_b200.kernels.attention import MAX_SPLITS, cut_decode_work
    lens = [300, 1, 77, 64, 17, 1500, 33, 201, 200]
    tok_pos = [n - 1 for n in lens]
    case = Pages(lens, G, hd, hd, torch.bfloat16, seed=4, block=block, first_query=tok_pos)
    tok_seq = list(range(len(lens)))
    q = _rand((len(lens), (H + 2 * G) * hd), torch.bfloat16, 72)
    scale = hd ** -0.5
    ref = case.reference(q[:, :H * hd].reshape(-1, H, hd), tok_seq, tok_pos, H, scale, block, cap)
    work = cut_decode_work(tok_pos, 0, teams, chunk=block)
    out = ops.attn_decode(q, case.k_pages, case.v_pages, case.table, _i32(tok_pos), _i32(tok_seq), case.slots, H, G, hd,
                          case.page, scale, ops.span(None, block), min(MAX_SPLITS, teams), early_loads=True, work=_i32(work.tolist()),
                          teams=teams, softcap=cap)
    _close(out.reshape(-1, H, hd), ref, case.tol(ref), BF16_ULP)


@pytest.mark.parametrize("H,G,hd,block,cap", FUSED)
def test_prompt_attention_over_blocks(H, G, hd, block, cap):
    """Three sequences in one call: one whole from its first token, one single token, one that goes on after 270 cached
    tokens (the pages below the block of its first new position are gone)."""
    ops = _ops()
    lens, new, past = [300, 1, 400], [300, 1, 130], [0, 0, 270]
    case = Pages(lens, G, hd, hd, torch.bfloat16, seed=5, block=block, first_query=past)
    tok_seq = [b for b, n in enumerate(new) for _ in range(n)]
    tok_pos = [p + i for n, p in zip(new, past) for i in range(n)]
    q = _rand((sum(new), (H + 2 * G) * hd), torch.bfloat16, 73)
    sink = _rand((H,), torch.float32, 74)
    scale = 1.1 * hd ** -0.5
    out = ops.attn_prefill(q, case.k_pages, case.v_pages, case.table, case.slots, _i32(lens), _blocks(new, past, 64), H, G, hd,
                           64, scale, ops.span(None, block), softcap=cap, sink=sink)
    ref = case.reference(q[:, :H * hd].reshape(-1, H, hd), tok_seq, tok_pos, H, scale, block, cap, sink)
    _close(out.reshape(-1, H, hd), ref, case.tol(ref), BF16_ULP)


@pytest.mark.parametrize("hd", [128, 64])
@pytest.mark.parametrize("H,G,block,cap", [(8, 2, 100, 50.0), (4, 4, 64, None), (2, 1, 300, 30.0), (4, 1, 37, None), (2, 2, 128, 9.0), (2, 1, 1, None)])
def test_tensor_core_prompt_attention_over_blocks(H, G, block, cap, hd):
    """The tcgen05 kernel, whose key tiles are whole pages: a block that starts inside a page, rows of one query tile in
    two and more blocks, tiles that lie wholly in an earlier block for every row."""
    ops = _ops()
    lens, new, past = [700, 1, 530], [700, 1, 260], [0, 0, 270]
    case = Pages(lens, G, hd, hd, torch.bfloat16, seed=6, block=block, first_query=past, poison=3.0e38)
    tok_seq = [b for b, n in enumerate(new) for _ in range(n)]
    tok_pos = [p + i for n, p in zip(new, past) for i in range(n)]
    q = _rand((sum(new), (H + 2 * G) * hd), torch.bfloat16, 74)
    sink = _rand((H,), torch.float32, 75)
    scale = hd ** -0.5
    out = ops.attn_prefill_tc(q, case.k_pages, case.v_pages, case.table, case.slots, _i32(lens), _blocks(new, past, 128), H, G,
                              hd, 64, scale, ops.span(None, block), softcap=cap, sink=sink)
    torch.cuda.synchronize()
    assert ops.attn_prefill_tc_status() == 0
    ref = case.reference(q[:, :H * hd].reshape(-1, H, hd), tok_seq, tok_pos, H, scale, block, cap, sink)
    _close(out.reshape(-1, H, hd), ref, case.tol(ref), BF16_ULP)


def _attend(kernel, case, q, n, hd, scale, block):
    """All n positions of sequence 0 as one prompt (or, for the decode kernel, the rows one token each)."""
    ops = _ops()
    args = (case.k_pages, case.v_pages, case.table)
    mask = ops.span(None, block)
    if kernel == "plain":
        return ops.attention_plain(q, *args, _i32(list(range(n))), _i32([0] * n), case.slots, 1, 1, hd, 64, scale, None, chunk=block)
    if kernel == "decode":
        return torch.cat([ops.attn_decode(q[p:p + 1], *args, _i32([p]), _i32([0]), case.slots, 1, 1, hd, 64, scale, mask, 2)
                          for p in range(n)])
    if kernel == "mma":
        return ops.attn_prefill(q, *args, case.slots, _i32([n]), _blocks([n], [0], 64), 1, 1, hd, 64, scale, mask)
    return ops.attn_prefill_tc(q, *args, case.slots, _i32([n]), _blocks([n], [0], 128), 1, 1, hd, 64, scale, mask)


@pytest.mark.parametrize("kernel", ["plain", "decode", "mma", "tc"])
@pytest.mark.parametrize("block", [150, 1000])
def test_one_key_that_outweighs_all_others_shows_the_blocks_edges(kernel, block):
    """Keys are made to stand out for one query each: the first key of the query's own block (seen, also from the block's
    last position) and the last key of the block before (hidden); a key hundreds of positions back inside a long block."""
    hd, n = 64, 460
    case = Pages([n], 1, hd, hd, torch.bfloat16, seed=7, poison=3.0e38 if kernel == "tc" else float("nan"))
    q = _rand((n, hd), torch.bfloat16, 75)
    if block == 150:
        plants = {(150, 299): True, (149, 290): False, (450, 459): True, (449, 451): False, (0, 149): True, (300, 300): True, (299, 310): False}
    else:
        plants = {(3, 459): True, (0, 200): True, (390, 391): True}
    for (key_pos, row) in plants:
        qh = q[row].float()
        case.plant(0, key_pos, (qh / qh.norm() * 40.0).to(torch.bfloat16))
    out = _attend(kernel, case, q, n, hd, 0.125, block)
    for (key_pos, row), seen in plants.items():
        gap = float((out[row].float() - case.v[0][key_pos, 0].float()).abs().max())
        assert (gap < 0.05) == seen, (key_pos, row, gap)
    ref = case.reference(q.reshape(n, 1, hd), [0] * n, list(range(n)), 1, 0.125, block)
    _close(out.reshape(n, 1, hd), ref, 2 * case.tol(ref), BF16_ULP)


@pytest.mark.parametrize("kernel", ["plain", "decode", "mma", "tc"])
def test_a_sink_that_outweighs_every_key_empties_the_head(kernel):
    """Two heads on one key head, 300 keys in blocks of 100: the first head's term in the denominator is e^30 times what its
    keys weigh, so its output is next to nothing at every position; the second head's is e^-30 of it and changes nothing."""
    ops = _ops()
    hd, n, block, H = 64, 300, 100, 2
    case = Pages([n], 1, hd, hd, torch.bfloat16, seed=9, poison=3.0e38 if kernel == "tc" else float("nan"))
    q = _rand((n, H * hd), torch.bfloat16, 77)
    sink = torch.tensor([30.0, -30.0], dtype=torch.float32, device=DEV)
    args = (case.k_pages, case.v_pages, case.table)
    mask = ops.span(None, block)
    if kernel == "plain":
        out = ops.attention_plain(q, *args, _i32(list(range(n))), _i32([0] * n), case.slots, H, 1, hd, 64, 0.05, None, chunk=block, sink=sink)
    elif kernel == "decode":
        rows = [0, 1, 99, 100, 199, 299]
        out = torch.zeros((n, H * hd), dtype=torch.bfloat16, device=DEV)
        for p in rows:
            out[p] = ops.attn_decode(q[p:p + 1], *args, _i32([p]), _i32([0]), case.slots, H, 1, hd, 64, 0.05, mask, 2, sink=sink)[0]
    elif kernel == "mma":
        out = ops.attn_prefill(q, *args, case.slots, _i32([n]), _blocks([n], [0], 64), H, 1, hd, 64, 0.05, mask, sink=sink)
    else:
        out = ops.attn_prefill_tc(q, *args, case.slots, _i32([n]), _blocks([n], [0], 128), H, 1, hd, 64, 0.05, mask, sink=sink)
    ref = case.reference(q.reshape(n, H, hd), [0] * n, list(range(n)), H, 0.05, block)          # without any sink
    rows = [0, 1, 99, 100, 199, 299] if kernel == "decode" else list(range(n))
    got = out.reshape(n, H, hd)[rows].float().cpu()
    assert float(got[:, 0].abs().max()) < 1e-6                                                  # emptied
    _close(got[:, 1], ref[rows][:, 1], 2 * case.tol(ref), BF16_ULP)                             # untouched


# ------------------------------------------------------------------ the scan with a decay for every key channel

def _scan_reference(q, k, v, pre, bias, tau, H, dk, dv, state):
    """float64, token by token; state [H, dk, dv] is advanced in place."""
    T = q.shape[0]
    a = torch.exp(torch.nn.functional.logsigmoid(pre + bias) / tau).reshape(T, H, dk)
    out = torch.zeros(T, H, dv, dtype=torch.float64)
    for t in range(T):
        for h in range(H):
            state[h] = a[t, h][:, None] * state[h] + k[t, h][:, None] * v[t, h][None, :]
            out[t, h] = state[h].T @ (q[t, h] * dk ** -0.5)
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,dk,dv,tau", [(2, 48, 64, 16.0), (1, 8, 72, 1.0), (3, 80, 40, 2.0), (2, 130, 24, 4.0), (1, 256, 16, 8.0)])
def test_channel_decay_scan_whole_in_pieces_and_token_by_token(dtype, H, dk, dv, tau):
    """Three sequences of 70, 1 and 37 tokens in slots 3, 0 and 4: whole in one step; in portions of unequal sizes; and one
    token per sequence and step (the streaming form); each against the float64 recurrence, and the states they leave."""
    ops = _ops()
    lens, slots = [70, 1, 37], [3, 0, 4]
    width = 2 * H * dk + 2 * H * dv
    rows = [_rand((n, width), dtype, 10 + i) for i, n in enumerate(lens)]
    pres = [_rand((n, H * dk + 4), torch.float32, 20 + i, 2.0) for i, n in enumerate(lens)]
    bias = _rand((H * dk,), torch.float32, 30) + 2.0
    refs, finals = [], []
    for r, p in zip(rows, pres):
        x = r.double().cpu()
        st = torch.zeros(H, dk, dv, dtype=torch.float64)
        refs.append(_scan_reference(x[:, :H * dk].reshape(-1, H, dk), x[:, H * dk:2 * H * dk].reshape(-1, H, dk),
                                    x[:, 2 * H * dk:2 * H * dk + H * dv].reshape(-1, H, dv), p[:, 2:2 + H * dk].double().cpu(),
                                    bias.double().cpu(), tau, H, dk, dv, st))
        finals.append(st)
    tol = 2e-5 if dtype == torch.float32 else 2e-5      # q, k, v enter as stored; everything else is 32-bit in both
    for cuts in ([[70], [1], [37]], [[2, 31, 1, 36], [1], [17, 16, 3, 1]], "single"):
        state = torch.full((6, H, dk, dv), 7.0, dtype=torch.float32, device=DEV)
        for s in slots:
            state[s].zero_()
        done = [0, 0, 0]
        got = [[], [], []]
        if cuts == "single":
            steps = [[1 if t < n else 0 for n in lens] for t in range(max(lens))]
        else:
            steps = [[c[i] if i < len(c) else 0 for c in cuts] for i in range(max(len(c) for c in cuts))]
        for step in steps:
            live = [b for b, n in enumerate(step) if n]
            x = torch.cat([rows[b][done[b]:done[b] + step[b]] for b in live])
            pre = torch.cat([pres[b][done[b]:done[b] + step[b]] for b in live])[:, 2:2 + H * dk]
            cu = [0] + list(np.cumsum([step[b] for b in live]))
            pos = [done[b] + i for b in live for i in range(step[b])]
            out, _ = ops.linear_scan(x, 0, H * dk, 2 * H * dk, state, _i32(cu), _i32([slots[b] for b in live]), _i32(pos), len(live),
                                     H, dk, dv, q_scale=dk ** -0.5, channel_decay=(pre, bias, tau), single=cuts == "single")
            for j, b in enumerate(live):
                got[b].append(out[cu[j]:cu[j + 1]])
                done[b] += step[b]
        for b in range(3):
            _close(torch.cat(got[b]), refs[b], tol)
            _close(state[slots[b]], finals[b], tol)
        assert float(state[1].min()) == 7.0 and float(state[5].max()) == 7.0       # other slots are left alone


@pytest.mark.parametrize("single", [False, True])
def test_a_decay_of_exactly_one_keeps_the_first_token_for_good(single):
    """With a huge bias every decay is exactly one: after 300 tokens whose keys are orthogonal to the query but for the
    first one, the output is still the first token's value; with a strongly negative bias on one head it is gone."""
    ops = _ops()
    H, dk, dv, T = 2, 16, 8, 300
    x = torch.zeros((T, 2 * H * dk + 2 * H * dv), dtype=torch.float32, device=DEV)
    q = torch.zeros(H, dk); q[:, 0] = 4.0
    x[:, :H * dk] = q.reshape(-1).to(DEV)                                 # every query looks along channel 0
    x[0, H * dk:2 * H * dk] = q.reshape(-1).to(DEV) / 4.0                 # only the first key has a part along it
    x[1:, H * dk + 1:2 * H * dk:dk] = 1.0                                 # the others lie along channel 1
    v = _rand((T, H * dv), torch.float32, 3)
    x[:, 2 * H * dk:2 * H * dk + H * dv] = v
    pre = torch.zeros((T, H * dk), dtype=torch.float32, device=DEV)
    bias = torch.full((H * dk,), 60.0, dtype=torch.float32, device=DEV)
    bias[dk:] = -3.0                                                      # the second head forgets
    state = torch.zeros((1, H, dk, dv), dtype=torch.float32, device=DEV)
    if single:
        outs = [ops.linear_scan(x[t:t + 1], 0, H * dk, 2 * H * dk, state, _i32([0, 1]), _i32([0]), _i32([t]), 1, H, dk, dv,
                                q_scale=dk ** -0.5, channel_decay=(pre[t:t + 1], bias, 2.0), single=True)[0] for t in range(T)]
        out = torch.cat(outs)
    else:
        out, _ = ops.linear_scan(x, 0, H * dk, 2 * H * dk, state, _i32([0, T]), _i32([0]), _i32(list(range(T))), 1, H, dk, dv,
                                 q_scale=dk ** -0.5, channel_decay=(pre, bias, 2.0))
    want = v[0].reshape(H, dv) * (4.0 * 1.0 * dk ** -0.5)
    assert float((out[T - 1, 0] - want[0]).abs().max()) < 1e-5
    assert float(out[T - 1, 1].abs().max()) < 1e-6 * float(want[1].abs().max())
