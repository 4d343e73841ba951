"""Each CUDA kernel alone against the plain implementation, at sizes other than the engine's.

float32 kernels must equal the plain implementation (reproducible exp) bit for bit.
bfloat16 kernels are compared with the plain float32 result of the same bfloat16 inputs,
within the tolerances stated beside each test.
"""
import numpy as np
import pytest
import torch

import plain_llama as P

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _ops(dtype):
    from bitwise_b200.kernels.ops import get_ops
    return get_ops(dtype)


def _bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def assert_same_bits(got, want, what):
    got = np.asarray(got, dtype=np.float32)
    want = np.asarray(want, dtype=np.float32)
    bad = _bits(got) != _bits(want)
    assert not bad.any(), (f"{what}: {int(bad.sum())} of {bad.size} values differ in bits; max abs diff "
                           f"{np.abs(got - want).max():.3e}; first at {np.argwhere(bad)[0].tolist()}")


def t(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV).to(dtype)


def rnd(rng, *shape, scale=1.0):
    return (rng.standard_normal(shape) * scale).astype(np.float32)


# ----------------------------------------------------------------------------------------
# float32: bit equality

@pytest.mark.parametrize("n,width", [(1, 16), (5, 100), (9, 257), (3, 2048)])
def test_f32_rmsnorm(n, width):
    rng = np.random.default_rng(width)
    x, w = rnd(rng, n, width), (1 + 0.1 * rnd(rng, width)).astype(np.float32)
    out = torch.empty(n, width, device=DEV)
    _ops("float32").rmsnorm(t(x), t(w), 1e-5, out)
    assert_same_bits(out.cpu().numpy(), P.rmsnorm(x, w, 1e-5), "rmsnorm")
    rows = np.array([n - 1, 0], dtype=np.int32)
    out2 = torch.empty(2, width, device=DEV)
    _ops("float32").rmsnorm(t(x), t(w), 1e-6, out2, rows=torch.from_numpy(rows).to(DEV))
    assert_same_bits(out2.cpu().numpy(), P.rmsnorm(x[rows], w, 1e-6), "rmsnorm with gathered rows")


@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (1, 100, 33), (7, 15, 16), (17, 64, 172), (70, 130, 96), (16, 65, 600)])
def test_f32_linear(m, n, k):
    rng = np.random.default_rng(m * 1000 + n + k)
    x, w = rnd(rng, m, k), rnd(rng, n, k, scale=0.1)
    out = torch.empty(m, n, device=DEV)
    _ops("float32").linear(t(x), t(w), out)
    want = P.linear(x, w)
    assert_same_bits(out.cpu().numpy(), want, "linear")
    res = rnd(rng, m, n)
    acc = t(res).clone()
    _ops("float32").linear(t(x), t(w), acc, residual=acc)
    assert_same_bits(acc.cpu().numpy(), (res + want).astype(np.float32), "linear with residual in place")


@pytest.mark.parametrize("m", [1, 3, 8, 9, 16])
def test_f32_linear_of_few_rows_every_tile_width_gives_the_chain(m):
    """Products of up to 16 rows whose k is a multiple of 32 stream the weights through tiles of
    16, 32, 64 or 128 columns (one to eight outputs per lane); the width is chosen for speed and
    every one must give the plain chain's bits: widths that cut the matrix's edge, a single
    line of k, stages that end before their last line, and more tiles than blocks."""
    rng = np.random.default_rng(40 + m)
    ops = _ops("float32")
    try:
        for n, k in ((1, 32), (50, 96), (333, 416), (200, 1056), (40000, 64)):
            x, w = rnd(rng, m, k), rnd(rng, n, k, scale=0.1)
            want = P.linear(x, w)
            res = rnd(rng, m, n)
            for width in (0, 16, 32, 64, 128):
                for stages in (0, 2):
                    ops.force_rows_plan(width, stages)
                    out = torch.empty(m, n, device=DEV)
                    ops.linear(t(x), t(w), out)
                    assert_same_bits(out.cpu().numpy(), want, f"[{m}x{k}] x [{n}x{k}], tiles of {width}, {stages} stages")
                    acc = t(res).clone()
                    ops.linear(t(x), t(w), acc, residual=acc)
                    assert_same_bits(acc.cpu().numpy(), (res + want).astype(np.float32),
                                     f"[{m}x{k}] x [{n}x{k}] with residual, tiles of {width}")
    finally:
        ops.force_rows_plan(0, 0)
    assert not ops.device_failure(), "a kernel gave up a bounded wait"


def test_f32_linear_row_alone_equals_row_in_batch():
    rng = np.random.default_rng(5)
    x, w = rnd(rng, 50, 200), rnd(rng, 77, 200)
    ops = _ops("float32")
    full = torch.empty(50, 77, device=DEV)
    ops.linear(t(x), t(w), full)
    for r in (0, 13, 49):
        one = torch.empty(1, 77, device=DEV)
        ops.linear(t(x[r:r + 1]), t(w), one)
        assert_same_bits(one.cpu().numpy(), full[r:r + 1].cpu().numpy(), f"row {r}")


def test_f32_swiglu():
    rng = np.random.default_rng(2)
    gu = rnd(rng, 9, 2 * 172, scale=3.0)
    gu[0, :4] = [-100.0, 100.0, 0.0, -87.5]
    out = torch.empty(9, 172, device=DEV)
    _ops("float32").swiglu(t(gu), out)
    assert_same_bits(out.cpu().numpy(), P.swiglu(gu, 172, exp="det"), "swiglu")


def _paged(rng, lens, kv_heads, hd, page, dtype=np.float32, spare=3):
    """A scrambled paged cache for sequences of the given lengths: (k, v, table, per-seq k/v)."""
    blocks = [(n + page - 1) // page for n in lens]
    total = sum(blocks) + spare
    perm = rng.permutation(total)
    table = np.zeros((len(lens), max(blocks)), dtype=np.int32)
    k = rnd(rng, total, kv_heads, page, hd)
    v = rnd(rng, total, kv_heads, page, hd)
    at = 0
    seq_k, seq_v = [], []
    for s, nb in enumerate(blocks):
        table[s, :nb] = perm[at:at + nb]
        at += nb
        kk = np.concatenate([k[b] for b in table[s, :nb]], axis=1)[:, :lens[s]]  # [kvh, len, hd]
        vv = np.concatenate([v[b] for b in table[s, :nb]], axis=1)[:, :lens[s]]
        seq_k.append(np.transpose(kk, (1, 0, 2)))
        seq_v.append(np.transpose(vv, (1, 0, 2)))
    return k, v, table, seq_k, seq_v


@pytest.mark.parametrize("heads,kv_heads,hd,page,window", [(4, 2, 16, 16, 0), (3, 1, 32, 8, 0), (5, 5, 48, 16, 0),
                                                           (4, 2, 16, 16, 7), (6, 2, 64, 32, 40)])
def test_f32_attention(heads, kv_heads, hd, page, window):
    rng = np.random.default_rng(heads * 100 + hd + window)
    lens = [37, 1, 70]
    k, v, table, seq_k, seq_v = _paged(rng, lens, kv_heads, hd, page)
    # rows: for every sequence a few query positions, batched together
    rows = [(0, 36), (0, 5), (1, 0), (2, 69), (2, 68), (2, 16), (2, 15)]
    q = rnd(rng, len(rows), heads, hd)
    qkv = np.zeros((len(rows), (heads + 2 * kv_heads) * hd), dtype=np.float32)
    qkv[:, :heads * hd] = q.reshape(len(rows), -1)
    out = torch.empty(len(rows), heads * hd, device=DEV)
    ops = _ops("float32")
    ops.attention(t(qkv), t(k), t(v), torch.from_numpy(table).to(DEV),
                  torch.tensor([r[0] for r in rows], dtype=torch.int32, device=DEV),
                  torch.tensor([r[1] for r in rows], dtype=torch.int32, device=DEV), out, heads, kv_heads, hd,
                  window, max(r[1] for r in rows) + 1, 1.0 / np.sqrt(np.float32(hd)).item())
    got = out.cpu().numpy().reshape(len(rows), heads, hd)
    for i, (s, p) in enumerate(rows):
        # plain attention of the whole prefix with the query placed at position p
        T = p + 1
        qq = np.zeros((T, heads, hd), dtype=np.float32)
        qq[p] = q[i]
        want = P.attention(qq, seq_k[s][:T], seq_v[s][:T], exp="det", window=window)[p]
        assert_same_bits(got[i], want, f"attention row {i} (seq {s}, pos {p})")


def test_f32_rope_and_cache_write():
    rng = np.random.default_rng(3)
    heads, kv_heads, hd, page = 3, 1, 32, 8
    from bitwise_b200.parts.rope import RotaryEncoding
    rot = RotaryEncoding(hd, 500000.0, None, positions=64)
    cos, sin = rot.rotary_tables(DEV)
    pos = np.array([0, 1, 17, 63, 9], dtype=np.int32)
    seq = np.array([0, 0, 1, 1, 2], dtype=np.int32)
    table = np.array([[5, 0, 0, 0, 0, 0, 0, 0], [1, 2, 3, 4, 6, 7, 8, 9], [10, 11, 0, 0, 0, 0, 0, 0]], dtype=np.int32)
    qkv = rnd(rng, 5, (heads + 2 * kv_heads) * hd)
    k = torch.zeros(12, kv_heads, page, hd, device=DEV)
    v = torch.zeros(12, kv_heads, page, hd, device=DEV)
    buf = t(qkv).clone()
    _ops("float32").rope_cache(buf, t(pos, torch.int32), t(seq, torch.int32), cos, sin, t(table, torch.int32), k, v,
                               heads, kv_heads, hd)
    inv = P.rope_inv_freq(hd, 500000.0)
    want_q = P.rope(qkv[:, :heads * hd].reshape(5, heads, hd), pos, inv)
    want_k = P.rope(qkv[:, heads * hd:(heads + kv_heads) * hd].reshape(5, kv_heads, hd), pos, inv)
    assert_same_bits(buf.cpu().numpy()[:, :heads * hd].reshape(5, heads, hd), want_q, "rotated q")
    kc, vc = k.cpu().numpy(), v.cpu().numpy()
    for r in range(5):
        blk, slot = table[seq[r], pos[r] // page], pos[r] % page
        assert_same_bits(kc[blk, :, slot], want_k[r], f"cached k of row {r}")
        assert_same_bits(vc[blk, :, slot], qkv[r, (heads + kv_heads) * hd:].reshape(kv_heads, hd), f"cached v of row {r}")
    assert int((kc != 0).any(axis=(1, 3)).sum()) == 5, "keys were written to other slots too"


def test_embed_rows_both_table_dtypes():
    rng = np.random.default_rng(4)
    table = rnd(rng, 50, 72)
    toks = np.array([3, 49, 0, 3], dtype=np.int32)
    out = torch.empty(4, 72, device=DEV)
    _ops("float32").embed_rows(t(table), t(toks, torch.int32), out)
    assert_same_bits(out.cpu().numpy(), table[toks], "embed float32")
    tb = P.bf16_round(table)
    _ops("float32").embed_rows(t(tb, torch.bfloat16), t(toks, torch.int32), out)
    assert_same_bits(out.cpu().numpy(), tb[toks], "embed bfloat16 table")


def test_sample_rows_greedy_and_temperature():
    rng = np.random.default_rng(6)
    vocab = 1003  # no power of two, not a multiple of the block size
    logits = rnd(rng, 6, vocab, scale=2.0)
    logits[0, 17] = logits[0, 900] = 50.0  # tie: the first maximum wins
    temps = np.array([0.0, 0.8, 1.3, 0.0, 0.05, 2.0], dtype=np.float32)
    us = np.array([0.3, 0.999999, 0.0, 0.5, 0.41, 0.73], dtype=np.float64)
    out = torch.empty(6, dtype=torch.int32, device=DEV)
    _ops("float32").sample_rows(t(logits), t(temps), torch.from_numpy(us).to(DEV), out)
    got = out.cpu().numpy()
    for r in range(6):
        want = P.argmax_row(logits[r]) if temps[r] <= 0 else P.sample_row(logits[r], temps[r], us[r], exp="det")
        assert got[r] == want, f"row {r}: sampled {got[r]}, plain sampler says {want}"
    assert got[0] == 17


def test_fingerprint_rows():
    rng = np.random.default_rng(7)
    for vocab in (256, 385):
        logits = rnd(rng, 3, vocab)
        state = torch.full((5,), 0, dtype=torch.int64, device=DEV)
        seed = 1469598103934665603
        state[:] = seed
        slot = torch.tensor([4, 0, 2], dtype=torch.int32, device=DEV)
        ops = _ops("float32")
        ops.fingerprint_rows(t(logits), slot, state)
        ops.fingerprint_rows(t(logits[::-1].copy()), slot, state)
        got = [int(x) & ((1 << 64) - 1) for x in state.cpu().numpy()]
        for i, s in enumerate([4, 0, 2]):
            want = P.fingerprint(P.fingerprint(seed, logits[i]), logits[::-1][i])
            assert got[s] == want


# ----------------------------------------------------------------------------------------
# bfloat16

def bf(a):
    return P.bf16_round(np.asarray(a, dtype=np.float32))


@pytest.mark.parametrize("m,n,k", [(1, 64, 64), (5, 100, 96), (64, 344, 64), (65, 130, 172), (200, 256, 1100),
                                   (8, 2048, 2048), (33, 72, 520), (65, 64, 64), (130, 100, 96), (200, 256, 1104),
                                   (300, 2112, 2048), (1000, 136, 520), (8, 2048, 8192), (20, 1000, 4100),
                                   (5, 48, 2064), (70, 2304, 6152), (260, 96, 4104)])
def test_bf16_linear(m, n, k):
    """Tolerance: float32 accumulation of exact bfloat16 products; the result may differ from
    the float64 sum by accumulation rounding only: 1e-4 of the largest output (float32 out),
    plus one bfloat16 rounding (2^-8 relative) when the output is bfloat16."""
    rng = np.random.default_rng(m + n + k)
    x, w = bf(rnd(rng, m, k)), bf(rnd(rng, n, k, scale=0.1))
    want = x.astype(np.float64) @ w.astype(np.float64).T
    ops = _ops("bfloat16")
    out32 = torch.empty(m, n, device=DEV)
    ops.linear(t(x, torch.bfloat16), t(w, torch.bfloat16), out32)
    assert np.abs(out32.cpu().numpy() - want).max() <= 1e-4 * np.abs(want).max()
    out16 = torch.empty(m, n, device=DEV, dtype=torch.bfloat16)
    ops.linear(t(x, torch.bfloat16), t(w, torch.bfloat16), out16)
    got = out16.float().cpu().numpy()
    assert (np.abs(got - want) <= 2.0 ** -8 * np.abs(want) + 1e-4 * np.abs(want).max()).all()
    res = rnd(rng, m, n)
    acc = t(res).clone()
    ops.linear(t(x, torch.bfloat16), t(w, torch.bfloat16), acc, residual=acc)
    assert np.abs(acc.cpu().numpy() - (res + want)).max() <= 1e-4 * np.abs(want).max() + 1e-6
    assert not ops.device_failure(), "a kernel gave up a bounded wait"


def test_bf16_linear_row_bits_do_not_depend_on_the_batch():
    """The summation order is the same for every batch size: a row gives the same bits
    alone, in a small batch (narrow tiles, split along k where k is long and n small) and in
    a large one (one block or a pair of blocks walks k)."""
    rng = np.random.default_rng(8)
    for n, k in ((96, 2048), (2048, 1536), (64, 200), (2048, 8192), (136, 4104), (6144, 2048)):
        x, w = bf(rnd(rng, 200, k)), bf(rnd(rng, n, k, scale=0.05))
        ops = _ops("bfloat16")
        full = torch.empty(200, n, device=DEV)
        ops.linear(t(x, torch.bfloat16), t(w, torch.bfloat16), full)
        for rows in ((0, 1), (3, 11), (0, 64), (100, 165), (7, 136)):
            part = torch.empty(rows[1] - rows[0], n, device=DEV)
            ops.linear(t(x[rows[0]:rows[1]], torch.bfloat16), t(w, torch.bfloat16), part)
            assert_same_bits(part.cpu().numpy(), full[rows[0]:rows[1]].cpu().numpy(), f"rows {rows} of [{n}x{k}]")


def test_bf16_linear_tensor_core_generations_agree_bit_for_bit():
    """The tcgen05 kernel (whole and split mode) and the legacy mma.sync tile implement the
    same summation order: equal bits for the same rows."""
    rng = np.random.default_rng(14)
    ops = _ops("bfloat16")
    for m, n, k in ((8, 2048, 2048), (1, 6144, 2048), (64, 2048, 8192), (100, 320, 1536), (128, 16384, 512),
                    (300, 200, 1032), (17, 136, 520), (3, 1000, 4104), (128, 2304, 6152), (16, 6144, 4096),
                    (40, 96, 2056), (300, 200, 4104), (8, 4096, 14336)):
        x, w = bf(rnd(rng, m, k)), bf(rnd(rng, n, k, scale=0.05))
        res = rnd(rng, m, n)
        a, b = t(res).clone(), t(res).clone()
        ops.linear(t(x, torch.bfloat16), t(w, torch.bfloat16), a, residual=a)
        ops.linear(t(x, torch.bfloat16), t(w, torch.bfloat16), b, residual=b, legacy=True)
        assert_same_bits(a.cpu().numpy(), b.cpu().numpy(), f"[{m}x{k}] x [{n}x{k}]")
        want = res + x.astype(np.float64) @ w.astype(np.float64).T
        assert np.abs(a.cpu().numpy() - want).max() <= 1e-4 * np.abs(want).max()
    assert not ops.device_failure()


def test_bf16_linear_every_plan_of_a_small_batch_gives_the_same_bits():
    """A small batch may run whole (one block walks k) or split along k, on tiles 16 .. 128
    or 256 columns wide: the plan is chosen for speed and must not change a bit."""
    rng = np.random.default_rng(16)
    ops = _ops("bfloat16")
    for m, n, k in ((8, 2048, 2048), (1, 6144, 1536), (40, 1000, 4104), (128, 520, 1032), (17, 136, 520)):
        x, w = bf(rnd(rng, m, k)), bf(rnd(rng, n, k, scale=0.05))
        res = rnd(rng, m, n)
        want = t(res).clone()
        ops.linear(t(x, torch.bfloat16), t(w, torch.bfloat16), want, residual=want, legacy=True)
        try:
            for mode in (1, 2):
                for width in (16, 48, 112, 128, 256):
                    ops.force_linear_plan(width, mode)
                    got = t(res).clone()
                    ops.linear(t(x, torch.bfloat16), t(w, torch.bfloat16), got, residual=got)
                    assert_same_bits(got.cpu().numpy(), want.cpu().numpy(),
                                     f"mode {mode} width {width} [{m}x{k}] x [{n}x{k}]")
                    got16 = torch.empty(m, n, device=DEV, dtype=torch.bfloat16)
                    ops.linear(t(x, torch.bfloat16), t(w, torch.bfloat16), got16)
                    ref16 = torch.empty(m, n, device=DEV, dtype=torch.bfloat16)
                    ops.force_linear_plan(0, 0)
                    ops.linear(t(x, torch.bfloat16), t(w, torch.bfloat16), ref16, legacy=True)
                    assert torch.equal(got16.view(torch.int16), ref16.view(torch.int16))
        finally:
            ops.force_linear_plan(0, 0)
    assert not ops.device_failure()


def test_bf16_linear_two_blocks_per_tile_give_the_same_bits():
    """Large batches run on pairs of thread blocks that share a 256 x 256 tile (cta_group::2);
    the same product with one block per tile, and the legacy kernel, give equal bits. Sizes:
    a second block with no rows, with one row, partial tiles in both directions, many tiles
    per pair, k with a partial chunk."""
    rng = np.random.default_rng(15)
    ops = _ops("bfloat16")
    for m, n, k in ((129, 256, 64), (257, 264, 520), (256, 512, 2048), (600, 520, 1032), (2047, 2048, 576),
                    (1500, 6144, 512), (385, 136, 4104)):
        x, w = bf(rnd(rng, m, k)), bf(rnd(rng, n, k, scale=0.05))
        res = rnd(rng, m, n)
        a, b, c = t(res).clone(), t(res).clone(), t(res).clone()
        before = ops.pair_tiles(True)
        try:
            ops.linear(t(x, torch.bfloat16), t(w, torch.bfloat16), a, residual=a)
            ops.pair_tiles(False)
            ops.linear(t(x, torch.bfloat16), t(w, torch.bfloat16), b, residual=b)
        finally:
            ops.pair_tiles(before)
        assert_same_bits(a.cpu().numpy(), b.cpu().numpy(), f"pair vs single [{m}x{k}] x [{n}x{k}]")
        if m * n * k < 2e9:
            ops.linear(t(x, torch.bfloat16), t(w, torch.bfloat16), c, residual=c, legacy=True)
            assert_same_bits(a.cpu().numpy(), c.cpu().numpy(), f"pair vs legacy [{m}x{k}] x [{n}x{k}]")
        want = res + x.astype(np.float64) @ w.astype(np.float64).T
        assert np.abs(a.cpu().numpy() - want).max() <= 1e-4 * np.abs(want).max()
    assert not ops.device_failure()


def test_bf16_linear_few_rows_kernel_gives_the_same_bits():
    """Steps of up to 16 rows run their products on the streaming kernel (a warp per 8 columns
    and chunk, chunk sums added inside the kernel, clusters of blocks when k is long). Same bits
    as the tcgen05 kernel, for every output kind: bfloat16, float32 with residual, float32
    without. Sizes: one chunk, a partial chunk, 4 / 8 / 16 / 28 chunks (clusters of 1, 2, 4, 8),
    columns that are no multiple of 8 or 16, 1 .. 16 rows."""
    rng = np.random.default_rng(21)
    ops = _ops("bfloat16")
    for m, n, k in ((1, 64, 64), (8, 2048, 2048), (3, 100, 200), (5, 1000, 520), (8, 2048, 8192), (2, 77, 4104),
                    (9, 6144, 2048), (16, 136, 4096), (13, 1001, 8192), (8, 512, 14336), (16, 264, 14336),
                    (7, 49152 // 8, 2048)):
        x, w = bf(rnd(rng, m, k)), bf(rnd(rng, n, k, scale=0.05))
        res = rnd(rng, m, n)
        outs = {}
        for on in (True, False):
            before = ops.rows_path(on)
            try:
                a = t(res).clone()
                ops.linear(t(x, torch.bfloat16), t(w, torch.bfloat16), a, residual=a)
                b = torch.empty(m, n, device=DEV)
                ops.linear(t(x, torch.bfloat16), t(w, torch.bfloat16), b)
                c = torch.empty(m, n, device=DEV, dtype=torch.bfloat16)
                ops.linear(t(x, torch.bfloat16), t(w, torch.bfloat16), c)
                outs[on] = (a.cpu().numpy(), b.cpu().numpy(), c.view(torch.int16).cpu().numpy())
            finally:
                ops.rows_path(before)
        for got, want, what in zip(outs[True], outs[False], ("residual", "float32", "bfloat16")):
            assert_same_bits(got, want, f"{what} [{m}x{k}] x [{n}x{k}]")
        exact = res + x.astype(np.float64) @ w.astype(np.float64).T
        assert np.abs(outs[True][0] - exact).max() <= 1e-4 * np.abs(exact).max()
    assert not ops.device_failure()


def test_bf16_linear_swiglu_fused_equals_product_then_swiglu():
    """The gate/up product with SwiGLU in the same kernel (interleaved weights) gives the bits
    of the plain product followed by the SwiGLU kernel, on every path: few rows (streaming
    kernel), a small batch (tcgen05, whole or split) and a large one."""
    rng = np.random.default_rng(22)
    ops = _ops("bfloat16")
    for m, inter, k in ((1, 128, 64), (8, 8192, 2048), (5, 192, 520), (16, 2560, 960), (12, 256, 4104),
                        (40, 1024, 2048), (300, 512, 1032)):
        x = bf(rnd(rng, m, k))
        gate, up = bf(rnd(rng, inter, k, scale=0.05)), bf(rnd(rng, inter, k, scale=0.05))
        gu = torch.empty(m, 2 * inter, device=DEV, dtype=torch.bfloat16)
        ops.linear(t(x, torch.bfloat16), t(np.concatenate([gate, up]), torch.bfloat16), gu)
        want = torch.empty(m, inter, device=DEV, dtype=torch.bfloat16)
        ops.swiglu(gu, want)
        wi = ops.interleave_gate_up(t(gate, torch.bfloat16), t(up, torch.bfloat16))
        for on in (True, False):
            before = ops.rows_path(on)
            try:
                got = torch.empty(m, inter, device=DEV, dtype=torch.bfloat16)
                ops.linear_swiglu(t(x, torch.bfloat16), wi, got)
            finally:
                ops.rows_path(before)
            assert torch.equal(got.view(torch.int16), want.view(torch.int16)), f"rows path {on} [{m}x{k}] x [{2 * inter}x{k}]"
    assert not ops.device_failure()


def test_bf16_qkv_product_that_rotates_and_stores_equals_product_then_rope():
    """Steps of few rows: the fused q/k/v projection rotates q and k and writes k and v into
    their pages in its own epilogue. Same bits as the product followed by the rotation
    kernel: rotated q, and every byte of both caches; also without tables (no rotation) and
    for a run that only reads a cache (nothing stored)."""
    rng = np.random.default_rng(24)
    ops = _ops("bfloat16")
    from bitwise_b200.parts.rope import RotaryEncoding
    for m, width, heads, kv_heads, hd, page in ((8, 2048, 32, 32, 64, 16), (1, 960, 15, 5, 64, 16), (13, 512, 4, 2, 128, 32),
                                                (5, 192, 6, 3, 16, 8), (16, 1024, 8, 1, 48, 16)):
        assert ops.fuses_rope(m, width, heads, kv_heads, hd), (m, width, heads, kv_heads, hd)
        n = (heads + 2 * kv_heads) * hd
        x, w = bf(rnd(rng, m, width)), bf(rnd(rng, n, width, scale=0.05))
        cos, sin = RotaryEncoding(hd, 10000.0, None, positions=256).rotary_tables(DEV)
        pos = rng.integers(0, 250, m).astype(np.int32)
        seq = np.arange(m, dtype=np.int32)
        pages = m * (256 // page) + 2
        table = rng.permutation(pages)[:m * (256 // page)].reshape(m, -1).astype(np.int32)
        for tables, write in (((cos, sin), True), ((None, None), True), ((cos, sin), False)):
            outs = []
            for fused in (False, True):
                k = torch.full((pages, kv_heads, page, hd), 0.5, device=DEV, dtype=torch.bfloat16)
                v = torch.full((pages, kv_heads, page, hd), -0.25, device=DEV, dtype=torch.bfloat16)
                qkv = torch.zeros(m, n, device=DEV, dtype=torch.bfloat16)
                args = (t(pos, torch.int32), t(seq, torch.int32), tables[0], tables[1], t(table, torch.int32), k, v,
                        heads, kv_heads, hd)
                if fused:
                    ops.linear_rope_cache(t(x, torch.bfloat16), t(w, torch.bfloat16), qkv, *args, write_kv=write)
                else:
                    ops.linear(t(x, torch.bfloat16), t(w, torch.bfloat16), qkv)
                    ops.rope_cache(qkv, *args, write_kv=write)
                outs.append((qkv[:, :heads * hd].float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy()))
            for got, want, what in zip(outs[1], outs[0], ("q", "key cache", "value cache")):
                assert_same_bits(got, want, f"{what}: {heads}/{kv_heads} heads of {hd}, {m} rows, rotate "
                                            f"{tables[0] is not None}, store {write}")
    assert not ops.fuses_rope(40, 2048, 32, 32, 64)
    assert not ops.device_failure()


def test_bf16_rmsnorm_and_swiglu():
    """Tolerance: one bfloat16 rounding of a float32 result (2^-8 relative) plus 1e-6 absolute."""
    rng = np.random.default_rng(9)
    x, w = rnd(rng, 7, 960), (1 + 0.1 * rnd(rng, 960)).astype(np.float32)
    out = torch.empty(7, 960, device=DEV, dtype=torch.bfloat16)
    ops = _ops("bfloat16")
    ops.rmsnorm(t(x), t(w), 1e-5, out)
    want = P.rmsnorm(x, w, 1e-5)
    assert (np.abs(out.float().cpu().numpy() - want) <= 2.0 ** -8 * np.abs(want) + 1e-6).all()
    gu = bf(rnd(rng, 5, 2 * 172, scale=2.0))
    h = torch.empty(5, 172, device=DEV, dtype=torch.bfloat16)
    ops.swiglu(t(gu, torch.bfloat16), h)
    want = P.swiglu(gu, 172, exp="det")
    assert (np.abs(h.float().cpu().numpy() - want) <= 2.0 ** -8 * np.abs(want) + 1e-6).all()


def _run_bf16_attention(q, rows_by_seq, k, v, table, heads, kv_heads, hd, window):
    return _run_attention("bfloat16", q, rows_by_seq, k, v, table, heads, kv_heads, hd, window)


def _run_attention(dtype, q, rows_by_seq, k, v, table, heads, kv_heads, hd, window):
    """rows_by_seq: list of (first position, count) per sequence; q: [rows, heads, hd] (bfloat16 values
    for the serving kernels)."""
    ops = _ops(dtype)
    td = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    n = q.shape[0]
    qkv = np.zeros((n, (heads + 2 * kv_heads) * hd), dtype=np.float32)
    qkv[:, :heads * hd] = q.reshape(n, -1)

    class Batch:
        pass
    b = Batch()
    seq_row0, seq_pos0, r = [], [], 0
    pos, row_seq = [], []
    for s, (p0, cnt) in enumerate(rows_by_seq):
        seq_row0.append(r)
        seq_pos0.append(p0)
        pos += list(range(p0, p0 + cnt))
        row_seq += [s] * cnt
        r += cnt
    seq_row0.append(r)
    I = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
    b.seq_row0, b.seq_pos0 = I(seq_row0), I(seq_pos0)

    def query_tiles(rows):  # tiles of at most `rows` query rows of one sequence, as the stepper builds them
        tiles = []
        for s, (p0, cnt) in enumerate(rows_by_seq):
            for a in range(0, cnt, rows):
                tiles.append((s, seq_row0[s] + a, min(rows, cnt - a)))
        return I([x[0] for x in tiles]), I([x[1] for x in tiles]), I([x[2] for x in tiles]), len(tiles)
    b.query_tiles = query_tiles
    b.tile_sets = {rows: None for rows in ops.attention_tile_heights(heads, kv_heads, hd)}  # heights on offer
    out = torch.empty(n, heads * hd, device=DEV, dtype=td)
    ops.attention(t(qkv, td), t(k, td), t(v, td), I(table), I(row_seq), I(pos),
                  out, heads, kv_heads, hd, window, max(pos) + 1, 1.0 / np.sqrt(np.float32(hd)).item(), batch=b)
    return out.float().cpu().numpy().reshape(n, heads, hd), pos, row_seq


@pytest.mark.parametrize("heads,kv_heads,hd,page,window", [(4, 2, 16, 16, 0), (3, 1, 32, 8, 0), (5, 5, 48, 16, 0),
                                                           (8, 2, 64, 64, 0), (2, 2, 128, 32, 0), (6, 2, 64, 16, 50),
                                                           (4, 4, 80, 16, 0), (2, 1, 256, 16, 0), (4, 2, 96, 4, 21)])
def test_f32_attention_in_tiles_of_rows(heads, kv_heads, hd, page, window):
    """Prompt portions on the 32-bit path run as tiles of up to 16 query rows that share their
    keys, and single rows as two kernels (scores by many blocks, then the chains): both equal the
    plain attention bit for bit, for whole prompts, late portions, first tokens and decoded rows,
    alone and side by side in one step."""
    rng = np.random.default_rng(heads * 100 + hd + window)
    lens = [150, 1, 70, 200, 333]
    k, v, table, seq_k, seq_v = _paged(rng, lens, kv_heads, hd, page)
    for rows_by_seq in ([(0, 150), (0, 1), (69, 1), (130, 70), (300, 33)],   # a step of portions and single rows
                        [(149, 1), (0, 1), (69, 1), (199, 1), (332, 1)]):    # a step of single rows
        n = sum(c for _, c in rows_by_seq)
        q = rnd(rng, n, heads, hd)
        got, pos, row_seq = _run_attention("float32", q, rows_by_seq, k, v, table, heads, kv_heads, hd, window)
        r = 0
        for s, (p0, cnt) in enumerate(rows_by_seq):
            T = p0 + cnt
            qq = np.zeros((T, heads, hd), dtype=np.float32)
            qq[p0:] = q[r:r + cnt]
            want = P.attention(qq, seq_k[s][:T], seq_v[s][:T], exp="det", window=window)[p0:]
            assert_same_bits(got[r:r + cnt], want, f"sequence {s} rows {p0}..{T - 1}")
            r += cnt


@pytest.mark.parametrize("heads,kv_heads,hd,page", [(8, 2, 64, 16), (8, 8, 16, 16), (4, 4, 48, 8), (8, 4, 128, 4), (6, 2, 96, 64)])
def test_f32_attention_of_many_single_rows_by_pages(heads, kv_heads, hd, page):
    """A decode step with (row, head) pairs enough for every SM takes the form that brings the
    values page by page: same bits as the plain attention, at context lengths on and beside the
    edges of pages and of tiles of 64 keys."""
    rng = np.random.default_rng(heads + hd + page)
    lens = [1, 2, 15, 16, 17, 63, 64, 65, 127, 128, 129, 200, 255, 256, 257, 300, 64 * 5, 64 * 5 + 1, 333, 31, 33, 48,
            100, 191, 192, 193, 7, 70, 140, 210, 280, 350, 420, 21, 42, 84, 168, 336]
    assert len(lens) * heads >= 148
    k, v, table, seq_k, seq_v = _paged(rng, lens, kv_heads, hd, page)
    rows_by_seq = [(n - 1, 1) for n in lens]
    q = rnd(rng, len(lens), heads, hd)
    got, _, _ = _run_attention("float32", q, rows_by_seq, k, v, table, heads, kv_heads, hd, 0)
    for s, n in enumerate(lens):
        qq = np.zeros((n, heads, hd), dtype=np.float32)
        qq[n - 1] = q[s]
        want = P.attention(qq, seq_k[s], seq_v[s], exp="det")[n - 1]
        assert_same_bits(got[s], want, f"sequence {s} of {n} keys")
    assert not _ops("float32").device_failure()


def test_f32_attention_finds_a_far_key_and_the_window_edge():
    """One key among hundreds carries the weight (its score stands out), once far back and once
    just inside or just outside the window: random inputs would hide a wrong key range."""
    heads, kv_heads, hd, page, L = 2, 1, 64, 16, 600
    rng = np.random.default_rng(4)
    for far, window, inside in ((3, 0, True), (L - 100, 100, True), (L - 101, 100, False), (L - 17, 0, True)):
        k, v, table, seq_k, seq_v = _paged(rng, [L], kv_heads, hd, page)
        q = rnd(rng, 16, heads, hd) * 0.1
        blk, slot = table[0, far // page], far % page
        k[blk, 0, slot] = 160.0 * q[15, 0] / np.linalg.norm(q[15, 0])   # stands out for the last row, head 0
        v[blk, 0, slot] = 100.0
        seq_k[0][far] = k[blk, 0, slot]
        seq_v[0][far] = v[blk, 0, slot]
        got, _, _ = _run_attention("float32", q, [(L - 16, 16)], k, v, table, heads, kv_heads, hd, window)
        qq = np.zeros((L, heads, hd), dtype=np.float32)
        qq[L - 16:] = q
        want = P.attention(qq, seq_k[0], seq_v[0], exp="det", window=window)[L - 16:]
        assert_same_bits(got, want, f"far key {far}, window {window}")
        assert (np.abs(want[15, 0]).max() > 50.0) == inside


@pytest.mark.parametrize("heads,kv_heads,hd,page,window", [(4, 2, 16, 16, 0), (3, 1, 32, 8, 0), (5, 5, 48, 16, 0),
                                                           (8, 2, 64, 64, 0), (2, 2, 128, 32, 0), (6, 2, 64, 16, 50),
                                                           (4, 4, 80, 16, 0)])
def test_bf16_attention(heads, kv_heads, hd, page, window):
    """Against plain attention of the same bfloat16 q, k, v with the softmax weights rounded
    to bfloat16 before the value product.  Tolerance: the output is one bfloat16 rounding
    (2^-8 relative) of a sum whose weights carry a bfloat16 rounding each relative to a
    running instead of the final maximum: 2^-7 of the largest |v| of the sequence."""
    rng = np.random.default_rng(heads * 100 + hd + window)
    lens = [150, 1, 70, 200]
    k, v, table, seq_k, seq_v = _paged(rng, lens, kv_heads, hd, page)
    k, v = bf(k), bf(v)
    seq_k, seq_v = [bf(a) for a in seq_k], [bf(a) for a in seq_v]
    rows_by_seq = [(0, 150), (0, 1), (69, 1), (130, 70)]  # a whole prompt, a first token, a decode, a late portion
    n = sum(c for _, c in rows_by_seq)
    q = bf(rnd(rng, n, heads, hd))
    got, pos, row_seq = _run_bf16_attention(q, rows_by_seq, k, v, table, heads, kv_heads, hd, window)
    r = 0
    for s, (p0, cnt) in enumerate(rows_by_seq):
        T = p0 + cnt
        qq = np.zeros((T, heads, hd), dtype=np.float32)
        qq[p0:] = q[r:r + cnt]
        want = P.attention(qq, seq_k[s][:T], seq_v[s][:T], exp="det", window=window, round_bf16=True)[p0:]
        tol = 2.0 ** -7 * np.abs(seq_v[s]).max()
        err = np.abs(got[r:r + cnt] - want).max()
        assert err <= tol, f"sequence {s}: max error {err:.4f} > {tol:.4f}"
        r += cnt


def test_bf16_attention_finds_a_far_key_and_the_window_edge():
    """One key among hundreds is made to stand out by scaling it along the query: the output
    must be that key's value.  With a window that ends one position after it, it must vanish."""
    rng = np.random.default_rng(11)
    heads, kv_heads, hd, page = 2, 1, 64, 16
    L = 500
    k, v, table, seq_k, seq_v = _paged(rng, [L], kv_heads, hd, page)
    k, v = bf(k * 0.1), bf(v)
    q = bf(rnd(rng, 1, heads, hd))
    far = 3  # the far key's position
    blk, slot = table[0, far // page], far % page
    k[blk, 0, slot] = bf(q[0, 0] * 4.0)  # score ~ 4 |q|^2 / 8 = about 32 above the rest
    got, _, _ = _run_bf16_attention(q, [(L - 1, 1)], k, v, table, heads, kv_heads, hd, 0)
    assert np.abs(got[0, 0] - v[blk, 0, slot]).max() < 2e-2, "head 0 should return the far key's value"
    window = L - 1 - far  # keys far+1 .. L-1: the far key is just outside
    got_w, _, _ = _run_bf16_attention(q, [(L - 1, 1)], k, v, table, heads, kv_heads, hd, window)
    assert np.abs(got_w[0, 0] - v[blk, 0, slot]).max() > 0.3, "the far key must be outside the window"
    got_in, _, _ = _run_bf16_attention(q, [(L - 1, 1)], k, v, table, heads, kv_heads, hd, window + 1)
    assert np.abs(got_in[0, 0] - v[blk, 0, slot]).max() < 2e-2, "one more position and it is inside"


def test_bf16_attention_row_bits_do_not_depend_on_the_tile():
    """A query row gives the same bits alone (a decode step) and inside a long portion."""
    rng = np.random.default_rng(12)
    heads, kv_heads, hd, page = 4, 2, 64, 16
    k, v, table, _, _ = _paged(rng, [300], kv_heads, hd, page)
    k, v = bf(k), bf(v)
    q = bf(rnd(rng, 300, heads, hd))
    full, _, _ = _run_bf16_attention(q, [(0, 300)], k, v, table, heads, kv_heads, hd, 0)
    for p in (0, 63, 64, 255, 299):
        one, _, _ = _run_bf16_attention(q[p:p + 1], [(p, 1)], k, v, table, heads, kv_heads, hd, 0)
        assert_same_bits(one[0], full[p], f"position {p}")
    part, _, _ = _run_bf16_attention(q[100:171], [(100, 71)], k, v, table, heads, kv_heads, hd, 0)
    assert_same_bits(part, full[100:171], "portion 100..170")


def test_bf16_attention_decode_rows_split_over_chunks_give_the_same_bits():
    """Decode rows of long contexts run one chunk of 256 keys per thread block plus a merge
    kernel; prefill portions walk the chunks inside one block.  Same order, same bits; also
    with a window, and for several sequences of different lengths in one step."""
    rng = np.random.default_rng(15)
    for heads, kv_heads, hd, page, window in ((4, 2, 64, 16, 0), (3, 3, 32, 16, 300), (8, 2, 128, 32, 0)):
        lens = [700, 257, 1030]
        k, v, table, _, _ = _paged(rng, lens, kv_heads, hd, page)
        k, v = bf(k), bf(v)
        qs = [bf(rnd(rng, n, heads, hd)) for n in lens]
        for s, n in enumerate(lens):
            tab = table[s:s + 1]
            full, _, _ = _run_bf16_attention(qs[s], [(0, n)], k, v, tab, heads, kv_heads, hd, window)
            for p in (n - 1, 256, 255, 600 if n > 600 else 100):
                one, _, _ = _run_bf16_attention(qs[s][p:p + 1], [(p, 1)], k, v, tab, heads, kv_heads, hd, window)
                assert_same_bits(one[0], full[p], f"heads {heads}/{kv_heads} hd {hd} window {window} seq {s} pos {p}")
        # all three sequences decode together
        q3 = np.stack([qs[s][lens[s] - 1] for s in range(3)])
        got, _, _ = _run_bf16_attention(q3, [(lens[s] - 1, 1) for s in range(3)], k, v, table, heads, kv_heads, hd, window)
        for s in range(3):
            alone, _, _ = _run_bf16_attention(q3[s:s + 1], [(lens[s] - 1, 1)], k, v, table[s:s + 1], heads, kv_heads, hd, window)
            assert_same_bits(got[s], alone[0], f"sequence {s} in a batch of three")


def test_bf16_attention_streaming_decode_kernel_gives_the_same_bits():
    """Head size 64: decode steps read the cache through a persistent kernel whose warps keep
    rings of key tiles filled by TMA (a page of a head per copy), or, with few rows, through a
    block per key tile that gets its tile as TMA boxes. Same bits as the kernel that gives every
    key tile a block of its own and copies with cp.async: groups of 1 .. 16 heads, pages of
    8 .. 64 keys, a window, sequences of very different lengths in one step (one shorter than a
    tile)."""
    rng = np.random.default_rng(17)
    ops = _ops("bfloat16")
    hd = 64
    for heads, kv_heads, page, window in ((4, 4, 16, 0), (8, 2, 16, 0), (3, 1, 8, 0), (4, 2, 64, 200), (16, 1, 32, 0),
                                          (6, 3, 16, 0)):
        lens = [700, 40, 1030, 129, 64]
        k, v, table, _, _ = _paged(rng, lens, kv_heads, hd, page)
        k, v = bf(k), bf(v)
        q = bf(rnd(rng, len(lens), heads, hd))
        rows = [(n - 1, 1) for n in lens]
        outs = {}
        for mode in (2, 1, 0):  # persistent blocks; a block per key tile fed by TMA boxes (5 rows); cp.async blocks
            before = ops.stream_attention(hd, mode)
            try:
                outs[mode], _, _ = _run_bf16_attention(q, rows, k, v, table, heads, kv_heads, hd, window)
            finally:
                ops.stream_attention(hd, before)
        assert_same_bits(outs[2], outs[0], f"streaming: heads {heads}/{kv_heads} page {page} window {window}")
        assert_same_bits(outs[1], outs[0], f"a block per tile with TMA boxes: heads {heads}/{kv_heads} page {page} window {window}")
    assert not ops.device_failure()


def test_bf16_attention_tensor_core_generations_agree_bit_for_bit():
    """The tcgen05 prefill kernel (head sizes 64 and 128) and the mma.sync kernels give the same
    bits: whole prompts, late portions, with a window, grouped heads, several sequences in a step."""
    rng = np.random.default_rng(16)
    ops = _ops("bfloat16")
    for hd, heads, kv_heads, page, window in ((64, 4, 4, 16, 0), (64, 8, 2, 16, 0), (64, 2, 1, 32, 0), (64, 4, 2, 64, 90),
                                              (64, 16, 2, 16, 0), (128, 4, 1, 16, 0), (128, 2, 2, 32, 0), (128, 8, 2, 16, 75),
                                              (128, 3, 1, 8, 0)):
        lib = ops._attention_lib(hd)
        rows_tc = lib.bw_bf16_attention_tc_tile_rows(heads, kv_heads, hd, page, (heads + 2 * kv_heads) * hd)
        assert (rows_tc > 0) == (128 % (heads // kv_heads) == 0), "the tcgen05 kernel takes groups that divide 128"
        lens = [333, 70, 129]
        k, v, table, _, _ = _paged(rng, lens, kv_heads, hd, page)
        k, v = bf(k), bf(v)
        rows_by_seq = [(0, 333), (10, 60), (100, 29)]
        n = sum(c for _, c in rows_by_seq)
        q = bf(rnd(rng, n, heads, hd))
        new, _, _ = _run_bf16_attention(q, rows_by_seq, k, v, table, heads, kv_heads, hd, window)
        ops.legacy_attention = True
        try:
            old, _, _ = _run_bf16_attention(q, rows_by_seq, k, v, table, heads, kv_heads, hd, window)
        finally:
            ops.legacy_attention = False
        assert_same_bits(new, old, f"head size {hd} heads {heads}/{kv_heads} page {page} window {window}")
    assert not ops.device_failure()


def test_bf16_rope_and_cache_write():
    rng = np.random.default_rng(13)
    heads, kv_heads, hd, page = 4, 2, 16, 16
    from bitwise_b200.parts.rope import RotaryEncoding
    rot = RotaryEncoding(hd, 10000.0, None, positions=40)
    cos, sin = rot.rotary_tables(DEV)
    pos = np.array([0, 39, 16], dtype=np.int32)
    seq = np.array([0, 0, 1], dtype=np.int32)
    table = np.array([[2, 0, 1], [3, 4, 0]], dtype=np.int32)
    qkv = bf(rnd(rng, 3, (heads + 2 * kv_heads) * hd))
    k = torch.zeros(5, kv_heads, page, hd, device=DEV, dtype=torch.bfloat16)
    v = torch.zeros_like(k)
    buf = t(qkv, torch.bfloat16).clone()
    _ops("bfloat16").rope_cache(buf, t(pos, torch.int32), t(seq, torch.int32), cos, sin, t(table, torch.int32), k, v,
                                heads, kv_heads, hd)
    inv = P.rope_inv_freq(hd, 10000.0)
    want_q = bf(P.rope(qkv[:, :heads * hd].reshape(3, heads, hd), pos, inv))
    want_k = bf(P.rope(qkv[:, heads * hd:(heads + kv_heads) * hd].reshape(3, kv_heads, hd), pos, inv))
    got_q = buf.float().cpu().numpy()[:, :heads * hd].reshape(3, heads, hd)
    # the kernel may fuse the two products of a rotation: at most one bfloat16 step apart
    assert (np.abs(got_q - want_q) <= 2.0 ** -7 * np.abs(want_q) + 1e-6).all()
    kc = k.float().cpu().numpy()
    for r in range(3):
        blk, slot = table[seq[r], pos[r] // page], pos[r] % page
        assert (np.abs(kc[blk, :, slot] - want_k[r]) <= 2.0 ** -7 * np.abs(want_k[r]) + 1e-6).all()


def test_a_bounded_wait_that_runs_out_raises_the_failure_word_once():
    """No wait in the kernels is endless: a thread that polls a barrier gives up after a limit,
    raises the library's failure word, and the kernel returns.  The check kernel runs the
    kernels' own wait helper on a barrier on which nothing ever arrives, with a limit of a few
    thousand polls: it must come back, the word must read raised exactly once, and the device
    must go on computing right results (nothing faulted, nothing hung)."""
    ops = _ops("bfloat16")
    assert not ops.device_failure()
    assert ops.selftest_bounded_wait(polls=5000) == 2       # the wait gave up and said so
    assert ops.device_failure() is True                      # raised ...
    assert ops.device_failure() is False                     # ... once
    # through the asynchronous route that the engine uses
    assert ops.selftest_bounded_wait(polls=3000) == 2
    ops.failure_poll()
    torch.cuda.synchronize()
    assert ops.failure_seen() is True and ops.failure_seen() is False
    ops.failure_poll()
    torch.cuda.synchronize()
    assert ops.failure_seen() is False
    g = torch.Generator(device=DEV).manual_seed(5)
    x = torch.randn(8, 1024, device=DEV, generator=g).to(torch.bfloat16)
    w = (torch.randn(256, 1024, device=DEV, generator=g) * 0.05).to(torch.bfloat16)
    y = torch.empty(8, 256, device=DEV)
    ops.linear(x, w, y)
    ref = x.double() @ w.double().t()
    assert float((y.double() - ref).abs().max()) <= 1e-3 * float(ref.abs().max())
    assert not ops.device_failure()
