"""GPU parity, through the C ABI: the int8 lane (q8_round, q8_group_tok, q8_gate_up, q8_run) against the reference's
CPU lane (golden vectors) and the oracle. Bit-exact: bytes, scales, integer dots, F32 sums, activations."""
import os

import numpy as np
import pytest
import torch

from helpers import pointer_table, ptr, same_bits, sync, to_dev
from libosmos_b200 import synth
from oracle.oracle import LANE_TYPES, TYPES

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _round(lib, dev, x, fn="q8_round", xs=None):
    rows, cols = x.shape[0], x.shape[1] if xs is None else xs[0]
    stride = x.shape[1]
    q = torch.zeros((rows, cols), dtype=torch.int8, device=dev)
    d = torch.zeros((rows, cols // 32), dtype=torch.float32, device=dev)
    assert getattr(lib, fn)(ptr(to_dev(x, dev)), rows, cols, stride, ptr(q), ptr(d), None)
    sync()
    return q, d


@pytest.mark.parametrize("name", LANE_TYPES)
def test_lane_matches_reference_cpu_golden(lib, dev, name):
    g = np.load(os.path.join(GOLD, "lane_%s.npz" % name))
    tid = TYPES[name]
    for cols in (512, 768, 4096):
        w, x = g["w_%d" % cols], g["x_%d" % cols]
        q, d = _round(lib, dev, x)
        assert np.array_equal(q.cpu().numpy(), g["q_%d" % cols]) and same_bits(d.cpu().numpy(), g["d_%d" % cols])
        n = x.shape[0]
        y = torch.empty((n, 10), dtype=torch.float32, device=dev)
        assert lib.q8_run(tid, ptr(to_dev(w, dev)), 10, cols, ptr(q), ptr(d), n, ptr(y), 10, None)
        sync()
        assert same_bits(y.cpu().numpy(), g["y_%d" % cols])


def test_round_strided_and_special_blocks(lib, dev, oracle):
    rng = synth.rng_for(21)
    x = (rng.standard_normal((11, 96 + 32)) * 3).astype(np.float32)
    x[0, :32] = 0.0
    x[1, 32:64] = 0.0
    x[1, 37] = -2.5
    q, d = _round(lib, dev, x, xs=(96,))
    wq, wd = oracle.q8_round(np.ascontiguousarray(x[:, :96]))
    assert np.array_equal(q.cpu().numpy(), wq) and same_bits(d.cpu().numpy(), wd)
    assert d[0, 0].item() == 0.0 and q[1, 37].item() == -127
    q0, d0 = _round(lib, dev, x, fn="q8_0_round", xs=(96,))
    wq0, wd0 = oracle.q8_round(np.ascontiguousarray(x[:, :96]), ggml_q8_0=True)
    assert np.array_equal(q0.cpu().numpy(), wq0) and same_bits(d0.cpu().numpy(), wd0)


def _tables(dev, mats, cnt, xrow):
    pool = to_dev(np.concatenate(mats), dev)
    table = pointer_table(pool, [m * mats[0].size for m in range(len(mats))], dev)
    return pool, table, to_dev(np.asarray(cnt, dtype=np.int32), dev), to_dev(np.asarray(xrow, dtype=np.int32), dev)


@pytest.mark.parametrize("name", LANE_TYPES)
@pytest.mark.parametrize("cols", [512, 4096])
def test_group_tok_and_gate_up(lib, dev, oracle, name, cols):
    tid = TYPES[name]
    rows, n_mat = 21, 4
    rng = synth.rng_for(22, tid, cols)
    gate = [synth.random_tensor(tid, rows, cols, rng) for _ in range(n_mat)]
    up = [synth.random_tensor(tid, rows, cols, rng) for _ in range(n_mat)]
    cnt, xrow = [2, 8, 1, 5], [0, 2, 10, 11]
    total, n_tok = 16, 6
    x = rng.standard_normal((n_tok, cols)).astype(np.float32)
    xin = rng.integers(0, n_tok, size=total + 8).astype(np.int32)      # each row's token
    win = rng.permutation(total + 8).astype(np.int32)                  # each row's weight slot
    scale = rng.uniform(0.05, 0.5, size=total + 8).astype(np.float32)
    lim = 1.5
    wq, wd = oracle.q8_round(x)
    q, d = to_dev(wq, dev), to_dev(wd, dev)
    pg, tg, cd, xd_ = _tables(dev, gate, cnt, xrow)
    pu, tu, _, _ = _tables(dev, up, cnt, xrow)
    ys = rows + 3
    yg = torch.full((total + 8, ys), -9.0, dtype=torch.float32, device=dev)
    yu = torch.full((total + 8, ys), -9.0, dtype=torch.float32, device=dev)
    xin_d = to_dev(xin, dev)
    assert lib.q8_group_tok(tid, ptr(tg), ptr(cd), ptr(xd_), ptr(xin_d), n_mat, 8, rows, cols, ptr(q), ptr(d), ptr(yg), ys, None)
    assert lib.q8_group_tok(tid, ptr(tu), ptr(cd), ptr(xd_), ptr(xin_d), n_mat, 8, rows, cols, ptr(q), ptr(d), ptr(yu), ys, None)
    sync()
    want_g, want_u = np.full((total + 8, ys), -9.0, np.float32), np.full((total + 8, ys), -9.0, np.float32)
    for m in range(n_mat):
        for t in range(cnt[m]):
            r = xrow[m] + t
            tok = xin[r]
            want_g[r, :rows] = oracle.q8_rows(tid, gate[m], rows, cols, wq[tok:tok + 1], wd[tok:tok + 1])[0]
            want_u[r, :rows] = oracle.q8_rows(tid, up[m], rows, cols, wq[tok:tok + 1], wd[tok:tok + 1])[0]
    assert same_bits(yg.cpu().numpy(), want_g) and same_bits(yu.cpu().numpy(), want_u)
    # the fusion = the two sums then the lane's activation, bit for bit; weights by `win`
    h = torch.full((total + 8, ys), -9.0, dtype=torch.float32, device=dev)
    assert lib.q8_gate_up(tid, ptr(tg), ptr(tu), ptr(cd), ptr(xd_), ptr(xin_d), ptr(to_dev(win, dev)), n_mat, 8, rows,
                          cols, ptr(q), ptr(d), ptr(to_dev(scale, dev)), lim, ptr(h), ys, None)
    sync()
    want_h = np.full((total + 8, ys), -9.0, np.float32)
    for m in range(n_mat):
        for t in range(cnt[m]):
            r = xrow[m] + t
            want_h[r, :rows] = oracle.swiglu_lane(want_g[r:r + 1, :rows], want_u[r:r + 1, :rows], lim, scale[win[r]:win[r] + 1])[0]
    assert same_bits(h.cpu().numpy(), want_h)
    # and through ops_swiglu_lane on the GPU's own sums
    gg = yg[:total, :rows].contiguous()
    uu = yu[:total, :rows].contiguous()
    live = np.zeros(total, dtype=bool)
    for m in range(n_mat):
        live[xrow[m]:xrow[m] + cnt[m]] = True
    sc_rows = to_dev(scale[win[:total]], dev)
    hh = torch.empty_like(gg)
    assert lib.ops_swiglu_lane(ptr(gg), ptr(uu), rows, lim, ptr(sc_rows), total, ptr(hh), None)
    sync()
    assert same_bits(hh.cpu().numpy()[live], h.cpu().numpy()[:total, :rows][live])
    # a token's bits do not depend on max_cnt or on its neighbours: entry 2 (one row) alone at max_cnt 1
    y1 = torch.full((total + 8, ys), -9.0, dtype=torch.float32, device=dev)
    assert lib.q8_group_tok(tid, ptr(tg[2:]), ptr(cd[2:]), ptr(xd_[2:]), ptr(xin_d), 1, 1, rows, cols, ptr(q), ptr(d), ptr(y1), ys, None)
    sync()
    assert same_bits(y1.cpu().numpy()[10, :rows], want_g[10, :rows])


@pytest.mark.parametrize("name", ["Q4_0", "Q8_0"])
@pytest.mark.parametrize("cols", [2048, 4096])
def test_q8_run_plain_blocks(lib, dev, oracle, name, cols):
    """the extension of the lane order to one-scale blocks: bit-equal to the oracle's restatement, whose integer dots
    are checked against plain integer arithmetic and whose result is within rounding of a double sum"""
    tid = TYPES[name]
    rows, ntok = 50, 11
    rng = synth.rng_for(23, tid, cols)
    w = synth.random_tensor(tid, rows, cols, rng)
    x = rng.standard_normal((ntok, cols)).astype(np.float32)
    for ggml in (False, True):
        wq, wd = oracle.q8_round(x, ggml_q8_0=ggml)
        want = oracle.q8_rows(tid, w, rows, cols, wq, wd)
        y = torch.empty((ntok, rows), dtype=torch.float32, device=dev)
        assert lib.q8_run(tid, ptr(to_dev(w, dev)), rows, cols, ptr(to_dev(wq, dev)), ptr(to_dev(wd, dev)), ntok, ptr(y), rows, None)
        sync()
        assert same_bits(y.cpu().numpy(), want)
        # against exact arithmetic over the same quantized operands
        wv = oracle.dequant(tid, w, rows * cols).reshape(rows, cols).astype(np.float64)
        xv = (wq.astype(np.float64).reshape(ntok, cols // 32, 32) * wd.astype(np.float64)[:, :, None]).reshape(ntok, cols)
        exact = xv @ wv.T
        mag = np.abs(xv) @ np.abs(wv.T)
        assert np.all(np.abs(want - exact) <= (cols / 32 / (32 if cols >= 4096 else 16) + 8) * 2.0 ** -24 * mag)
    # integer block dots of a row: the oracle's against numpy's
    dots = oracle.q8_block_dots(tid, w[:w.size // rows], cols, wq[0])
    blk = w[:w.size // rows].reshape(cols // 32, -1)
    if name == "Q4_0":
        codes = np.concatenate([(blk[:, 2:] & 0x0F).astype(np.int64) - 8, (blk[:, 2:] >> 4).astype(np.int64) - 8], axis=1)
    else:
        codes = blk[:, 2:].view(np.int8).astype(np.int64)
    xi = wq[0].astype(np.int64).reshape(cols // 32, 32)
    assert np.array_equal(dots.reshape(-1, 2).sum(1), (codes * xi).sum(1))


ALL_LANE = list(LANE_TYPES)


@pytest.mark.parametrize("name", ALL_LANE)
@pytest.mark.parametrize("cols,rows", [(512, 136), (512, 160), (512, 128), (1024, 32), (1024, 256), (2048, 64), (2048, 512),
                                       (4096, 24), (7168, 16), (8192, 8), (24576, 8)])
def test_staged_kernel_matches_generic_and_oracle(lib, dev, oracle, name, cols, rows):
    """shapes the staged (bulk-copy) kernel takes: its bits are the generic kernel's and the oracle's, for every count
    1..8, with token and weight indirection, a skipped entry, and rows that leave the last tile partial (at 24576
    columns eight tokens' rows pass the generic kernel's shared memory: it takes an entry's tokens four at a time)"""
    tid = TYPES[name]
    n_mat = 6
    rng = synth.rng_for(24, tid, cols)
    gate = [synth.random_tensor(tid, rows, cols, rng) for _ in range(n_mat)]
    up = [synth.random_tensor(tid, rows, cols, rng) for _ in range(n_mat)]
    cnt, xrow = [1, 8, 0, 3, 2, 5], [0, 1, 9, 9, 12, 14]
    total, n_tok = 19, 7
    x = rng.standard_normal((n_tok, cols)).astype(np.float32)
    xin = rng.integers(0, n_tok, size=total).astype(np.int32)
    win = rng.permutation(total).astype(np.int32)
    scale = rng.uniform(0.05, 0.5, size=total).astype(np.float32)
    wq, wd = oracle.q8_round(x)
    q, d = to_dev(wq, dev), to_dev(wd, dev)
    pg, tg, cd, xd_ = _tables(dev, gate, cnt, xrow)
    pu, tu, _, _ = _tables(dev, up, cnt, xrow)
    xin_d, win_d, sc_d = to_dev(xin, dev), to_dev(win, dev), to_dev(scale, dev)
    ys, lim = rows + 5, 2.0
    results = []
    for staged in (2, 0, 1):  # the tile-staging kernel, the generic one, the warp-ring one (where it takes the type)
        lib.q8_set_staged(staged)
        yg = torch.full((total, ys), -9.0, dtype=torch.float32, device=dev)
        h = torch.full((total, ys), -9.0, dtype=torch.float32, device=dev)
        assert lib.q8_group_tok(tid, ptr(tg), ptr(cd), ptr(xd_), ptr(xin_d), n_mat, 8, rows, cols, ptr(q), ptr(d), ptr(yg), ys, None)
        assert lib.q8_gate_up(tid, ptr(tg), ptr(tu), ptr(cd), ptr(xd_), ptr(xin_d), ptr(win_d), n_mat, 8, rows, cols,
                              ptr(q), ptr(d), ptr(sc_d), lim, ptr(h), ys, None)
        sync()
        results.append((yg.cpu().numpy(), h.cpu().numpy()))
    lib.q8_set_staged(1)
    assert lib.q8_status() == 0
    want_g, want_h = np.full((total, ys), -9.0, np.float32), np.full((total, ys), -9.0, np.float32)
    for m in range(n_mat):
        for t in range(cnt[m]):
            r = xrow[m] + t
            tok = xin[r]
            g_ = oracle.q8_rows(tid, gate[m], rows, cols, wq[tok:tok + 1], wd[tok:tok + 1])
            u_ = oracle.q8_rows(tid, up[m], rows, cols, wq[tok:tok + 1], wd[tok:tok + 1])
            want_g[r, :rows] = g_[0]
            want_h[r, :rows] = oracle.swiglu_lane(g_, u_, lim, scale[win[r]:win[r] + 1])[0]
    assert same_bits(results[1][0], want_g) and same_bits(results[1][1], want_h), "generic kernel"
    assert same_bits(results[0][0], want_g) and same_bits(results[0][1], want_h), "staged kernel"
    assert same_bits(results[2][0], want_g) and same_bits(results[2][1], want_h), "warp-ring kernel"


@pytest.mark.parametrize("name", ["Q4_0", "Q8_0", "IQ3_XXS", "IQ1_M"])
@pytest.mark.parametrize("cols,rows,ntok", [(2048, 96, 1), (4096, 40, 5), (256, 8, 8)])
def test_staged_dense_matches_generic_and_oracle(lib, dev, oracle, name, cols, rows, ntok):
    tid = TYPES[name]
    rng = synth.rng_for(25, tid, cols)
    w = synth.random_tensor(tid, rows, cols, rng)
    x = rng.standard_normal((ntok, cols)).astype(np.float32)
    wq, wd = oracle.q8_round(x)
    want = oracle.q8_rows(tid, w, rows, cols, wq, wd)
    wdv, q, d = to_dev(w, dev), to_dev(wq, dev), to_dev(wd, dev)
    for staged in (1, 0):
        lib.q8_set_staged(staged)
        y = torch.full((ntok, rows + 2), -4.0, dtype=torch.float32, device=dev)
        assert lib.q8_run(tid, ptr(wdv), rows, cols, ptr(q), ptr(d), ntok, ptr(y), rows + 2, None)
        sync()
        got = y.cpu().numpy()
        assert same_bits(got[:, :rows], want) and (got[:, rows:] == -4.0).all(), "staged" if staged else "generic"
    lib.q8_set_staged(1)
    assert lib.q8_status() == 0


PLAIN_SHAPES = [(2048, 99, 1), (2048, 77, 2), (4096, 45, 1), (4096, 33, 2), (8192, 19, 1), (1024, 20, 2), (768, 21, 1),
                (512, 37891 + 16 * 148 * 2, 1)]


@pytest.mark.parametrize("name", ["Q4_0", "Q8_0"])
@pytest.mark.parametrize("cols,rows,ntok", PLAIN_SHAPES)
def test_plain_dense_kernel_same_bits(lib, dev, oracle, name, cols, rows, ntok):
    """q8_run's kernel for one-scale blocks and one or two tokens (x in registers, rows through a ring a warp)
    against the generic kernel and the oracle; the last shape is tall enough for slots of several row groups"""
    tid = TYPES[name]
    rng = synth.rng_for(27, tid, cols, rows)
    w = synth.random_tensor(tid, rows, cols, rng)
    x = rng.standard_normal((ntok, cols)).astype(np.float32)
    wq, wd = oracle.q8_round(x)
    want = oracle.q8_rows(tid, w, rows, cols, wq, wd)
    wdv, q, d = to_dev(w, dev), to_dev(wq, dev), to_dev(wd, dev)
    lib.q8_status()
    for staged in (1, 0):
        lib.q8_set_staged(staged)
        y = torch.full((ntok, rows + 2), -4.0, dtype=torch.float32, device=dev)
        assert lib.q8_run(tid, ptr(wdv), rows, cols, ptr(q), ptr(d), ntok, ptr(y), rows + 2, None)
        sync()
        got = y.cpu().numpy()
        assert same_bits(got[:, :rows], want) and (got[:, rows:] == -4.0).all(), "staged" if staged else "generic"
    lib.q8_set_staged(1)
    assert lib.q8_status() == 0


def test_staged_refuses_misaligned_matrix_without_faulting(lib, dev, oracle):
    """a matrix table entry that is not 16-byte aligned: the staged kernel records it and leaves (no fault, the
    context stays usable); the generic kernel takes the same call"""
    tid, rows, cols = TYPES["IQ3_XXS"], 64, 2048
    rng = synth.rng_for(26)
    w = synth.random_tensor(tid, rows, cols, rng)
    pool = torch.zeros(w.size + 64, dtype=torch.uint8, device=dev)
    pool[2:2 + w.size] = to_dev(w, dev)
    table = torch.tensor([pool.data_ptr() + 2], dtype=torch.int64, device=dev)
    x = rng.standard_normal((1, cols)).astype(np.float32)
    wq, wd = oracle.q8_round(x)
    q, d = to_dev(wq, dev), to_dev(wd, dev)
    one, zero = to_dev(np.array([1], np.int32), dev), to_dev(np.array([0], np.int32), dev)
    y = torch.zeros((1, rows), dtype=torch.float32, device=dev)
    lib.q8_set_staged(1)
    assert lib.q8_group_tok(tid, ptr(table), ptr(one), ptr(zero), None, 1, 1, rows, cols, ptr(q), ptr(d), ptr(y), rows, None)
    sync()
    assert lib.q8_status() & 2
    lib.q8_set_staged(0)
    assert lib.q8_group_tok(tid, ptr(table), ptr(one), ptr(zero), None, 1, 1, rows, cols, ptr(q), ptr(d), ptr(y), rows, None)
    sync()
    lib.q8_set_staged(1)
    assert same_bits(y.cpu().numpy(), oracle.q8_rows(tid, w, rows, cols, wq, wd))
