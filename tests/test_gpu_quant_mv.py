"""GPU parity, through the C ABI: block decoders and the F32-activation matvec family against the CPU oracle and
the committed golden vectors. Bit-exact everywhere."""
import os

import numpy as np
import pytest
import torch

from helpers import pointer_table, ptr, same_bits, sync, to_dev
from libosmos_b200 import synth
from oracle.oracle import BLOCK, LANE_TYPES, TYPES

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
ALL = sorted(TYPES)


@pytest.mark.parametrize("name", sorted(set(TYPES) - {"Q2_0", "MXFP8"}))  # (those two: no gguf-py decoder, the oracle below)
def test_dequant_golden(lib, dev, name):
    g = np.load(os.path.join(GOLD, "dequant.npz"))
    raw, want = g[name + "_raw"], g[name + "_values"]
    src, dst = to_dev(raw, dev), torch.empty(want.size, dtype=torch.float32, device=dev)
    assert lib.quant_dequant(TYPES[name], ptr(src), want.size, ptr(dst), None)
    sync()
    assert same_bits(dst.cpu().numpy(), want)
    h = torch.empty(want.size, dtype=torch.float16, device=dev)
    assert lib.quant_dequant_f16(TYPES[name], ptr(src), want.size, ptr(h), None)
    sync()
    with np.errstate(over="ignore"):
        want16 = want.astype(np.float16)
    assert np.array_equal(h.cpu().numpy().view(np.uint16), want16.view(np.uint16))


@pytest.mark.parametrize("name", ALL)
def test_dequant_large_vs_oracle(lib, dev, oracle, name):
    tid = TYPES[name]
    values = BLOCK[tid][0] * 3000 + (0 if BLOCK[tid][0] == 256 else BLOCK[tid][0] * 5)
    if BLOCK[tid][0] == 1:
        values = 8 * 3001  # the unquantized types go 8 values at a time
    raw = synth.random_blocks(tid, values // BLOCK[tid][0], synth.rng_for(11, tid))
    want = oracle.dequant(tid, raw, values)
    dst = torch.full((values + 8,), -7.0, dtype=torch.float32, device=dev)
    assert lib.quant_dequant(tid, ptr(to_dev(raw, dev)), values, ptr(dst), None)
    sync()
    got = dst.cpu().numpy()
    assert same_bits(got[:values], want) and (got[values:] == -7.0).all()
    assert not lib.quant_dequant(tid, ptr(dst), values + 1, ptr(dst), None)


def _mv_case(tid, rows, cols, ntok, key):
    rng = synth.rng_for(12, tid, rows, cols, key)
    w = synth.random_tensor(tid, rows, cols, rng)
    x = rng.standard_normal((ntok, cols)).astype(np.float32)
    return w, x


@pytest.mark.parametrize("name", ALL)
def test_mv_run_bits_and_batch_invariance(lib, dev, oracle, name):
    tid = TYPES[name]
    rows, cols = 37, 1024 if BLOCK[tid][0] == 256 else 1088  # an odd row count; a row's last lanes take one chunk fewer
    w, x = _mv_case(tid, rows, cols, 8, 0)
    want = oracle.mv_rows(tid, w, rows, cols, x)
    wd, xd = to_dev(w, dev), to_dev(x, dev)
    y = torch.full((8, rows), np.nan, dtype=torch.float32, device=dev)
    assert lib.mv_run(tid, ptr(wd), rows, cols, ptr(xd), 8, ptr(y), None)
    sync()
    assert same_bits(y.cpu().numpy(), want)
    for n in (1, 2, 3, 5, 7):  # every count the same bits for each token (schedule invariance)
        y2 = torch.full((n, rows), np.nan, dtype=torch.float32, device=dev)
        assert lib.mv_run(tid, ptr(wd), rows, cols, ptr(xd), n, ptr(y2), None)
        sync()
        assert same_bits(y2.cpu().numpy(), want[:n])
    y1 = torch.empty((1, rows), dtype=torch.float32, device=dev)
    for t in (0, 4, 7):  # each token alone
        assert lib.mv_run(tid, ptr(wd), rows, cols, ptr(xd[t]), 1, ptr(y1), None)
        sync()
        assert same_bits(y1.cpu().numpy()[0], want[t])


@pytest.mark.parametrize("name", ALL)
def test_mv_staged_kernel_same_bits(lib, dev, oracle, name):
    """the kernel that stages rows through shared memory against the generic one and the oracle"""
    tid = TYPES[name]
    rows, cols = 203, 2048
    w, x = _mv_case(tid, rows, cols, 8, 1)
    want = oracle.mv_rows(tid, w, rows, cols, x)
    wd, xd = to_dev(w, dev), to_dev(x, dev)
    lib.mv_status()
    try:
        for n in (1, 2, 3, 8):
            got = []
            for staged in (1, 0):
                lib.mv_set_staged(staged)
                y = torch.full((n, rows), np.nan, dtype=torch.float32, device=dev)
                assert lib.mv_run(tid, ptr(wd), rows, cols, ptr(xd), n, ptr(y), None)
                sync()
                got.append(y.cpu().numpy())
            assert same_bits(got[0], got[1]) and same_bits(got[0], want[:n])
    finally:
        lib.mv_set_staged(1)
    assert lib.mv_status() == 0


@pytest.mark.parametrize("name", ["Q4_0", "Q8_0", "IQ3_XXS", "Q4_K"])
def test_mv_staged_row_pairs(lib, dev, oracle, name):
    """a matrix tall enough that a warp sums two rows at once; an odd row count leaves the last unit one row"""
    tid = TYPES[name]
    rows, cols = 8 * 16 * 160 + 3, 512
    w, x = _mv_case(tid, rows, cols, 8, 2)
    want = oracle.mv_rows(tid, w, rows, cols, x)
    wd, xd = to_dev(w, dev), to_dev(x, dev)
    lib.mv_status()
    for n in (1, 2, 3, 4, 7, 8):
        y = torch.full((n, rows), np.nan, dtype=torch.float32, device=dev)
        assert lib.mv_run(tid, ptr(wd), rows, cols, ptr(xd), n, ptr(y), None)
        sync()
        assert same_bits(y.cpu().numpy(), want[:n])
    assert lib.mv_status() == 0


@pytest.mark.parametrize("name", ["Q4_0", "IQ3_XXS", "Q4_K", "MXFP4"])
def test_mv_strided_many_tokens(lib, dev, oracle, name):
    tid = TYPES[name]
    rows, cols, ntok, xs, ys = 19, 512, 77, 520, 24
    rng = synth.rng_for(13, tid)
    w = synth.random_tensor(tid, rows, cols, rng)
    x = rng.standard_normal((ntok, xs)).astype(np.float32)
    want = oracle.mv_rows(tid, w, rows, cols, np.ascontiguousarray(x[:, :cols]))
    y = torch.full((ntok, ys), -3.0, dtype=torch.float32, device=dev)
    assert lib.mv_strided(tid, ptr(to_dev(w, dev)), rows, cols, ptr(to_dev(x, dev)), xs, ntok, ptr(y), ys, None)
    sync()
    got = y.cpu().numpy()
    assert same_bits(got[:, :rows], want) and (got[:, rows:] == -3.0).all()


@pytest.mark.parametrize("name,cols,ntok", [("Q4_K", 7168, 8), ("Q4_K", 7168, 5), ("Q8_0", 14336, 7), ("IQ1_M", 16384, 4)])
def test_mv_long_rows_in_passes(lib, dev, oracle, name, cols, ntok):
    """rows so long that the staged kernel cannot hold every token's x: the tokens go a few a pass, with the bits of the
    generic kernel and the oracle"""
    tid = TYPES[name]
    rows, xs, ys = 150, cols + 8, 152
    rng = synth.rng_for(14, tid, cols)
    w = synth.random_tensor(tid, rows, cols, rng)
    x = rng.standard_normal((ntok, xs)).astype(np.float32)
    want = oracle.mv_rows(tid, w, rows, cols, np.ascontiguousarray(x[:, :cols]))
    wd, xd = to_dev(w, dev), to_dev(x, dev)
    lib.mv_status()
    for staged in (1, 0):
        lib.mv_set_staged(staged)
        y = torch.full((ntok, ys), -3.0, dtype=torch.float32, device=dev)
        assert lib.mv_strided(tid, ptr(wd), rows, cols, ptr(xd), xs, ntok, ptr(y), ys, None)
        sync()
        got = y.cpu().numpy()
        assert same_bits(got[:, :rows], want) and (got[:, rows:] == -3.0).all(), "staged" if staged else "generic"
    lib.mv_set_staged(1)
    assert lib.mv_status() == 0


@pytest.mark.parametrize("name", LANE_TYPES)
def test_mv_matches_reference_cpu_golden(lib, dev, name):
    g = np.load(os.path.join(GOLD, "lane_%s.npz" % name))
    for cols in (512, 768, 4096):
        w, x, want = g["w_%d" % cols], g["x_%d" % cols], g["ymv_%d" % cols]
        y = torch.empty(want.shape, dtype=torch.float32, device=dev)
        assert lib.mv_run(TYPES[name], ptr(to_dev(w, dev)), 10, cols, ptr(to_dev(x, dev)), x.shape[0], ptr(y), None)
        sync()
        assert same_bits(y.cpu().numpy(), want)


@pytest.mark.parametrize("name", ["IQ3_XXS", "IQ1_M", "Q8_0", "MXFP4"])
def test_mv_group_and_group_tok(lib, dev, oracle, name):
    tid = TYPES[name]
    rows, cols, n_mat = 24, 512, 5
    rng = synth.rng_for(14, tid)
    mats = [synth.random_tensor(tid, rows, cols, rng) for _ in range(n_mat)]
    pool = to_dev(np.concatenate(mats), dev)
    nbytes = mats[0].size
    table = pointer_table(pool, [m * nbytes for m in range(n_mat)], dev)
    # mv_group: matrix m on vector m / 2
    x = rng.standard_normal((3, cols)).astype(np.float32)
    y = torch.empty((n_mat, rows), dtype=torch.float32, device=dev)
    assert lib.mv_group(tid, ptr(table), n_mat, rows, cols, ptr(to_dev(x, dev)), cols, 2, ptr(y), None)
    sync()
    got = y.cpu().numpy()
    for m in range(n_mat):
        assert same_bits(got[m], oracle.mv_rows(tid, mats[m], rows, cols, x[m // 2:m // 2 + 1])[0])
    # mv_group_tok: entries of 1..8 rows, one skipped (count 0), rows xs apart, outputs untouched elsewhere
    cnt = np.array([3, 0, 8, 1, 5], dtype=np.int32)
    xrow = np.array([0, 3, 3, 11, 12], dtype=np.int32)
    total, xs, ys = 17, cols + 8, rows + 4
    xx = rng.standard_normal((total + 8, xs)).astype(np.float32)
    yy = torch.full((total + 8, ys), -5.0, dtype=torch.float32, device=dev)
    assert lib.mv_group_tok(tid, ptr(table), ptr(to_dev(cnt, dev)), ptr(to_dev(xrow, dev)), n_mat, 8, rows, cols,
                            ptr(to_dev(xx, dev)), xs, ptr(yy), ys, None)
    sync()
    got = yy.cpu().numpy()
    want = np.full_like(got, -5.0)
    for m in range(n_mat):
        for t in range(cnt[m]):
            r = xrow[m] + t
            want[r, :rows] = oracle.mv_rows(tid, mats[m], rows, cols, np.ascontiguousarray(xx[r:r + 1, :cols]))[0]
    assert same_bits(got, want)


@pytest.mark.parametrize("name,rows,cols", [("MXFP4", 96, 4096), ("MXFP4", 64, 1536), ("Q4_K", 80, 2048), ("IQ1_M", 48, 7168),
                                             ("Q8_0", 40, 1024), ("IQ3_XXS", 32, 2048), ("Q4_0", 33, 2048)])
def test_mv_grouped_on_the_staged_kernel(lib, dev, oracle, name, rows, cols):
    """mv_group_tok / mv_group where the staged kernel takes the shape (whole 256-value stretches, rows of whole 16 bytes):
    entries of every count 0 .. 8 in their count classes, the generic kernel's bits and the oracle's"""
    tid = TYPES[name]
    rng = synth.rng_for(15, tid, rows)
    cnt = np.array([1, 3, 0, 8, 2, 1, 5, 4, 7, 1, 6, 2], dtype=np.int32)
    n_mat = cnt.size
    mats = [synth.random_tensor(tid, rows, cols, rng) for _ in range(n_mat)]
    nbytes = mats[0].size
    assert nbytes % 16 == 0
    pool = to_dev(np.concatenate(mats), dev)
    table = pointer_table(pool, [m * nbytes for m in range(n_mat)], dev)
    xrow = np.concatenate([[0], np.cumsum(cnt)[:-1]]).astype(np.int32)
    total, xs, ys = int(cnt.sum()), cols + 8, rows + 4
    xx = rng.standard_normal((total, xs)).astype(np.float32)
    xd, cd, rd = to_dev(xx, dev), to_dev(cnt, dev), to_dev(xrow, dev)
    outs = []
    for staged in (1, 0):
        lib.mv_set_staged(staged)
        yy = torch.full((total, ys), -5.0, dtype=torch.float32, device=dev)
        assert lib.mv_group_tok(tid, ptr(table), ptr(cd), ptr(rd), n_mat, 8, rows, cols, ptr(xd), xs, ptr(yy), ys, None)
        sync()
        outs.append(yy.cpu().numpy())
    lib.mv_set_staged(1)
    assert lib.mv_status() == 0
    assert same_bits(outs[0], outs[1])
    want = np.full_like(outs[0], -5.0)
    for m in range(n_mat):
        if cnt[m]:
            r0 = xrow[m]
            want[r0:r0 + cnt[m], :rows] = oracle.mv_rows(tid, mats[m], rows, cols, np.ascontiguousarray(xx[r0:r0 + cnt[m], :cols]))
    assert same_bits(outs[0], want)
    # a call whose max_cnt is below an entry's count serves the entry's first max_cnt tokens, as the generic kernel does
    for staged in (1, 0):
        lib.mv_set_staged(staged)
        yy = torch.full((total, ys), -5.0, dtype=torch.float32, device=dev)
        assert lib.mv_group_tok(tid, ptr(table), ptr(cd), ptr(rd), n_mat, 2, rows, cols, ptr(xd), xs, ptr(yy), ys, None)
        sync()
        outs.append(yy.cpu().numpy())
    lib.mv_set_staged(1)
    assert same_bits(outs[2], outs[3])
    # mv_group: matrix m on vector m / 3
    x = rng.standard_normal((4, cols)).astype(np.float32)
    y = torch.empty((n_mat, rows), dtype=torch.float32, device=dev)
    assert lib.mv_group(tid, ptr(table), n_mat, rows, cols, ptr(to_dev(x, dev)), cols, 3, ptr(y), None)
    sync()
    got = y.cpu().numpy()
    for m in range(n_mat):
        assert same_bits(got[m], oracle.mv_rows(tid, mats[m], rows, cols, x[m // 3:m // 3 + 1])[0])
    assert lib.mv_status() == 0
