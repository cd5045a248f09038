"""GPU parity, through the C ABI: the f16 matrix products (mm_run, mm_run2, mm_tokens, mm_group) against a float64
sum over the same f16-rounded operands, within the reference's own bound (tests/gpu/test_mm_gpu.hip:328-343:
(cols / 16 + 20) 2^-24 sum |w16 x16|), and the batch invariance the reference asserts: a token's results are the
same bits whatever it is batched with and wherever in the batch."""
import numpy as np
import pytest
import torch

from helpers import ptr, same_bits, sync, to_dev
from libosmos_b200 import synth
from oracle.oracle import TYPES

pytestmark = pytest.mark.gpu
ALL = sorted(set(TYPES) - {"F32", "BF16"})  # (the block types: an unquantized matrix has no f16 product here)


def _x16(lib, dev, x, cols):
    """x's rows as the library's tiled f16 (mm_x16)"""
    n = x.shape[0]
    buf = torch.zeros(((n + 15) // 16 * 16) * cols, dtype=torch.float16, device=dev)
    flag = torch.zeros(1, dtype=torch.int32, device=dev)
    assert lib.mm_x16(ptr(to_dev(x, dev)), x.shape[1], n, cols, ptr(buf), ptr(flag), None)
    sync()
    assert int(flag.item()) == 0
    return buf


def _exact(oracle, tid, w, rows, cols, x):
    """(float64 sums, magnitude sums) over the operands as the kernel sees them: both rounded to f16"""
    with np.errstate(over="ignore"):
        w16 = oracle.dequant(tid, w, rows * cols).reshape(rows, cols).astype(np.float16).astype(np.float64)
    x16 = x[:, :cols].astype(np.float16).astype(np.float64)
    return x16 @ w16.T, np.abs(x16) @ np.abs(w16.T)


def _within(got, exact, mag, cols):
    return np.all(np.abs(got - exact) <= (cols / 16 + 20) * 2.0 ** -24 * mag + 1e-30)


@pytest.mark.parametrize("name", ALL)
def test_mm_run_bound_and_batch_invariance(lib, dev, oracle, name):
    tid = TYPES[name]
    rows, cols, n = 144, 512, 37  # a second, partial tile of rows; tokens not a whole tile
    rng = synth.rng_for(51, tid)
    w = synth.random_tensor(tid, rows, cols, rng)
    x = rng.standard_normal((n, cols)).astype(np.float32)
    exact, mag = _exact(oracle, tid, w, rows, cols, x)
    wd = to_dev(w, dev)
    y = torch.full((n, rows + 2), -7.0, dtype=torch.float32, device=dev)
    lib.mm_status()
    assert lib.mm_known(tid) and lib.mm_fits(tid, rows, cols)
    assert lib.mm_run(tid, ptr(wd), rows, cols, ptr(_x16(lib, dev, x, cols)), n, ptr(y), rows + 2, None)
    sync()
    got = y.cpu().numpy()
    assert (got[:, rows:] == -7.0).all() and _within(got[:, :rows], exact, mag, cols)
    # the same tokens in another order and another count: each token's bits unchanged
    order = np.array([5, 36, 0, 17])
    y2 = torch.empty((len(order), rows), dtype=torch.float32, device=dev)
    assert lib.mm_run(tid, ptr(wd), rows, cols, ptr(_x16(lib, dev, x[order], cols)), len(order), ptr(y2), rows, None)
    sync()
    assert same_bits(y2.cpu().numpy(), got[order, :rows])
    assert lib.mm_status() == 0


@pytest.mark.parametrize("name", ["Q4_K", "Q8_0", "IQ3_XXS"])
def test_mm_run_many_tokens(lib, dev, oracle, name):
    """more than one block of 512 tokens, several row tiles, a longer K"""
    tid = TYPES[name]
    rows, cols, n = 384, 2048, 600
    rng = synth.rng_for(52, tid)
    w = synth.random_tensor(tid, rows, cols, rng)
    x = rng.standard_normal((n, cols)).astype(np.float32)
    exact, mag = _exact(oracle, tid, w, rows, cols, x)
    wd, xb = to_dev(w, dev), _x16(lib, dev, x, cols)
    y = torch.empty((n, rows), dtype=torch.float32, device=dev)
    assert lib.mm_run(tid, ptr(wd), rows, cols, ptr(xb), n, ptr(y), rows, None)
    sync()
    got = y.cpu().numpy()
    assert _within(got, exact, mag, cols)
    one = torch.empty((1, rows), dtype=torch.float32, device=dev)
    for t in (0, 511, 512, 599):  # a token alone: the bits it has in the batch
        assert lib.mm_run(tid, ptr(wd), rows, cols, ptr(_x16(lib, dev, x[t:t + 1], cols)), 1, ptr(one), rows, None)
        sync()
        assert same_bits(one.cpu().numpy()[0], got[t])
    assert lib.mm_status() == 0


def test_mm_run2_tokens_and_scales(lib, dev, oracle):
    tid = TYPES["Q4_K"]
    rows0, rows1, cols, n = 128, 48, 256, 19
    rng = synth.rng_for(53)
    w0, w1 = synth.random_tensor(tid, rows0, cols, rng), synth.random_tensor(tid, rows1, cols, rng)
    x = rng.standard_normal((n, cols + 8)).astype(np.float32)
    d0, d1, xd = to_dev(w0, dev), to_dev(w1, dev), to_dev(x, dev)
    xb = _x16(lib, dev, np.ascontiguousarray(x[:, :cols]), cols)
    ya, yb = torch.empty((n, rows0), device=dev), torch.empty((n, rows1), device=dev)
    assert lib.mm_run(tid, ptr(d0), rows0, cols, ptr(xb), n, ptr(ya), rows0, None)
    assert lib.mm_run(tid, ptr(d1), rows1, cols, ptr(xb), n, ptr(yb), rows1, None)
    y0, y1 = torch.empty_like(ya), torch.empty_like(yb)
    assert lib.mm_run2(tid, ptr(d0), rows0, ptr(y0), rows0, ptr(d1), rows1, ptr(y1), rows1, cols, ptr(xb), n, None)
    sync()
    assert same_bits(y0.cpu().numpy(), ya.cpu().numpy()) and same_bits(y1.cpu().numpy(), yb.cpu().numpy())
    # mm_tokens from F32 x (its own x16), and the scaled form: one F32 multiply of the same sums
    scratch = torch.zeros(32 * cols, dtype=torch.float16, device=dev)
    flag = torch.zeros(1, dtype=torch.int32, device=dev)
    t0, t1 = torch.empty_like(ya), torch.empty_like(yb)
    assert lib.mm_tokens(tid, ptr(d0), rows0, ptr(t0), rows0, ptr(d1), rows1, ptr(t1), rows1, cols, ptr(xd), cols + 8, n,
                         ptr(scratch), ptr(flag), False, None)
    sync()
    assert same_bits(t0.cpu().numpy(), ya.cpu().numpy()) and same_bits(t1.cpu().numpy(), yb.cpu().numpy())
    assert lib.mm_tokens_scaled(tid, ptr(d0), rows0, ptr(t0), rows0, 0.75, None, 0, None, 0, 1.0, cols, ptr(xd), cols + 8, n,
                                ptr(scratch), ptr(flag), False, None)
    sync()
    assert same_bits(t0.cpu().numpy(), ya.cpu().numpy() * np.float32(0.75)) and int(flag.item()) == 0
    assert not lib.mm_run(tid, ptr(d0), rows0 + 8, cols, ptr(xb), n, ptr(ya), rows0 + 8, None)  # rows not whole tiles
    assert not lib.mm_run(tid, ptr(d0), rows0, cols + 64, ptr(xb), n, ptr(ya), rows0, None)  # cols not whole slabs
    assert not lib.mm_run(tid, ptr(d0), rows0, cols, ptr(xb), 2049, ptr(ya), rows0, None)
    assert not lib.mm_run2(tid, ptr(d0), rows0, ptr(y0), rows0, None, rows1, ptr(y1), rows1, cols, ptr(xb), n, None)


def test_mm_group_entries(lib, dev, oracle):
    """experts, each on its own gathered tokens: the bits mm_run gives each token"""
    tid = TYPES["IQ3_XXS"]
    rows, cols, n_mat = 64, 512, 3
    cnt = [20, 0, 130]
    rng = synth.rng_for(54)
    mats = [synth.random_tensor(tid, rows, cols, rng) for _ in range(n_mat)]
    xs = [rng.standard_normal((max(c, 1), cols)).astype(np.float32) for c in cnt]
    devs = [to_dev(m, dev) for m in mats]
    # each matrix's tokens gathered into whole tiles of one x16 (rows cols long), one after another
    tiles = [(c + 15) // 16 for c in cnt]
    slots = sum(tiles) * 16
    idx = np.full(slots, -1, np.int32)
    allx = np.concatenate(xs)
    first, at, xoff, yoff = 0, 0, [], []
    for m in range(n_mat):
        idx[at:at + cnt[m]] = first + np.arange(cnt[m])
        xoff.append(at * cols), yoff.append(at * rows)
        first, at = first + xs[m].shape[0], at + tiles[m] * 16
    x16 = torch.zeros(slots * cols, dtype=torch.float16, device=dev)
    flag = torch.zeros(1, dtype=torch.int32, device=dev)
    assert lib.mm_x16_rows(ptr(to_dev(allx, dev)), cols, ptr(to_dev(idx, dev)), slots, cols, ptr(x16), ptr(flag), None)
    y = torch.full((slots, rows), -3.0, dtype=torch.float32, device=dev)
    table = torch.tensor([d.data_ptr() for d in devs], dtype=torch.int64, device=dev)
    assert lib.mm_group(tid, ptr(table), ptr(to_dev(np.array(cnt, np.int32), dev)), n_mat, 130, rows, cols, ptr(x16),
                        ptr(to_dev(np.array(xoff, np.uint32), dev)), cols, ptr(y), ptr(to_dev(np.array(yoff, np.uint32), dev)),
                        rows, None)
    sync()
    got = y.cpu().numpy()
    at = 0
    for m in range(n_mat):
        if cnt[m]:
            alone = torch.empty((cnt[m], rows), dtype=torch.float32, device=dev)
            assert lib.mm_run(tid, ptr(devs[m]), rows, cols, ptr(_x16(lib, dev, xs[m][:cnt[m]], cols)), cnt[m], ptr(alone), rows, None)
            sync()
            assert same_bits(got[at:at + cnt[m]], alone.cpu().numpy())
        assert (got[at + cnt[m]:at + tiles[m] * 16] == -3.0).all()
        at += tiles[m] * 16
    assert lib.mm_status() == 0


def _tiled16(buf, n, cols):
    """the tiled f16 activations (16 x 16 tiles, mm_x16_at) back as rows: [n][cols] float16"""
    t16 = (n + 15) // 16
    a = buf.cpu().numpy()[: t16 * 16 * cols].reshape(t16, cols // 16, 16, 16)  # [token tile][col tile][token][col]
    return a.transpose(0, 2, 1, 3).reshape(t16 * 16, cols)[:n]


@pytest.mark.parametrize("name", ["Q8_0", "Q4_K", "IQ4_NL"])
def test_mm_run_silu(lib, dev, oracle, name):
    """mm_run_silu = mm_run, then y = silu(y scale) and its f16 for the next product, in one launch (the reference's
    test: tests/gpu/test_mm_gpu.hip:252-283 - 1, 16 and 64 tokens, and its refusals)"""
    tid = TYPES[name]
    rows, cols, scale = 320, 512, 0.25
    rng = synth.rng_for(57, tid)
    w = synth.random_tensor(tid, rows, cols, rng)
    wd = to_dev(w, dev)
    for n in (1, 16, 37, 64):
        x = rng.standard_normal((n, cols)).astype(np.float32) * 4.0
        if n == 37:
            x[5] *= 3.0e4  # one token past f16's range after the silu: the flag must be raised
        xb = _x16(lib, dev, np.clip(x, -6.0e4, 6.0e4), cols)
        y0 = torch.empty((n, rows), dtype=torch.float32, device=dev)
        assert lib.mm_run(tid, ptr(wd), rows, cols, ptr(xb), n, ptr(y0), rows, None)
        y = torch.full((n, rows + 3), -7.0, dtype=torch.float32, device=dev)
        out16 = torch.full((((n + 15) // 16) * 16 * rows,), 9.0, dtype=torch.float16, device=dev)
        flag = torch.zeros(1, dtype=torch.int32, device=dev)
        lib.mm_status()
        assert lib.mm_run_silu(tid, ptr(wd), rows, cols, ptr(xb), n, ptr(y), rows + 3, scale, ptr(out16), ptr(flag), None)
        sync()
        assert lib.mm_status() == 0
        got = y.cpu().numpy()
        u = y0.cpu().numpy() * np.float32(scale)  # (one F32 product, as the kernel rounds it)
        with np.errstate(over="ignore"):
            want = u.astype(np.float64) / (1.0 + np.exp(-u.astype(np.float64)))
        assert (got[:, rows:] == -7.0).all()
        # (where expf(-u) passes F32's range the expression gives -0: an absolute 1e-35 covers that band of u near -89)
        assert np.all(np.abs(got[:, :rows] - want) <= 3e-6 * np.abs(want) + 1e-35)
        with np.errstate(over="ignore"):
            assert same_bits(_tiled16(out16, n, rows), got[:, :rows].astype(np.float16))  # the f16 of the same F32 values
        assert int(flag.item()) == int(bool((np.abs(got[:, :rows]) > 65504.0).any()))
        if n == 37:
            assert int(flag.item()) == 1
    assert not lib.mm_run_silu(tid, ptr(wd), rows, cols, ptr(xb), 65, ptr(y), rows, scale, ptr(out16), ptr(flag), None)
    assert not lib.mm_run_silu(tid, ptr(wd), rows, cols, ptr(xb), 1, ptr(y), rows, scale, ptr(xb), ptr(flag), None)  # its own x16
    assert not lib.mm_run_silu(tid, ptr(wd), rows, cols, ptr(xb), 1, ptr(y), rows, scale, None, ptr(flag), None)
    assert not lib.mm_run_silu(tid, ptr(wd), rows, cols, ptr(xb), 1, ptr(y), rows, scale, ptr(out16), None, None)
    assert not lib.mm_run_silu(tid, ptr(wd), rows, cols + 64, ptr(xb), 1, ptr(y), rows, scale, ptr(out16), ptr(flag), None)


@pytest.mark.parametrize("hc,dim,cols,counts", [(4, 2560, 384, (1, 5, 16, 17, 37, 64, 100, 2048)), (2, 64, 128, (3, 33)),
                                                 (3, 48, 128, (40,)), (8, 80, 256, (130,)), (1, 144, 128, (7,))])
def test_mm_run_gated_mean(lib, dev, oracle, hc, dim, cols, counts):
    """mm_run_gated_mean = mm_run of the hc dim rows, then out[t][d] = (sum over s in order of xn[t][s][d]
    sigmoid(up[t][s dim + d])) / hc and its f16, the up never stored (the reference's test:
    tests/gpu/test_gated_mean_gpu.hip - its stream counts, token counts, overflow case and refusals)"""
    tid = TYPES["Q8_0"]
    rows = hc * dim
    rng = synth.rng_for(58, hc * 1000 + dim)
    w = synth.random_tensor(tid, rows, cols, rng)
    wd = to_dev(w, dev)
    for n in counts:
        x = rng.standard_normal((n, cols)).astype(np.float32)
        xn = rng.standard_normal((n, hc, dim)).astype(np.float32)
        if n > 3:
            xn[2, 0, 5] = 1.0e30  # one token's mean past f16's range: the flag set
        xb, xnd = _x16(lib, dev, x, cols), to_dev(xn, dev)
        up = torch.empty((n, rows), dtype=torch.float32, device=dev)
        assert lib.mm_run(tid, ptr(wd), rows, cols, ptr(xb), n, ptr(up), rows, None)
        out = torch.full((n, dim), -7.0, dtype=torch.float32, device=dev)
        row0 = 16
        out16 = torch.full(((row0 + n + 15) // 16 * 16 * dim,), 9.0, dtype=torch.float16, device=dev)
        flag = torch.zeros(1, dtype=torch.int32, device=dev)
        lib.mm_status()
        assert lib.mm_run_gated_mean(tid, ptr(wd), hc, dim, cols, ptr(xb), n, ptr(xnd), ptr(out), ptr(out16), row0, ptr(flag), None)
        sync()
        assert lib.mm_status() == 0
        got = out.cpu().numpy()
        g = up.cpu().numpy().reshape(n, hc, dim).astype(np.float64)
        terms = xn.astype(np.float64) / (1.0 + np.exp(-g))
        want, mag = terms.sum(axis=1) / hc, np.abs(terms).sum(axis=1) / hc
        assert np.all(np.abs(got - want) <= 3e-6 * mag + 1e-37)
        rows16 = _tiled16(out16, row0 + n, dim)
        with np.errstate(over="ignore"):
            assert same_bits(rows16[row0:], got.astype(np.float16))
        assert (rows16[:row0] == np.float16(9.0)).all()  # (the rows before row0 are someone else's)
        assert int(flag.item()) == (1 if n > 3 else 0)
        # without the f16 copy: the same F32 bits
        out2 = torch.empty_like(out)
        assert lib.mm_run_gated_mean(tid, ptr(wd), hc, dim, cols, ptr(xb), n, ptr(xnd), ptr(out2), None, 0, None, None)
        sync()
        assert same_bits(out2.cpu().numpy(), got)
    f = ptr(out)
    assert not lib.mm_run_gated_mean(tid, ptr(wd), hc, dim, cols, ptr(xb), 8, ptr(xnd), f, ptr(xb), 0, ptr(flag), None)  # out16 = x16
    assert not lib.mm_run_gated_mean(tid, ptr(wd), hc, dim, cols, ptr(xb), 8, ptr(xnd), f, ptr(out16), 0, None, None)  # no flag
    assert not lib.mm_run_gated_mean(tid, ptr(wd), 9, dim, cols, ptr(xb), 8, ptr(xnd), f, None, 0, None, None)
    assert not lib.mm_run_gated_mean(tid, ptr(wd), hc, dim + 8, cols, ptr(xb), 8, ptr(xnd), f, None, 0, None, None)  # dim not 16s
    assert not lib.mm_run_gated_mean(tid, ptr(wd), hc, dim, cols, ptr(xb), 2049, ptr(xnd), f, None, 0, None, None)
