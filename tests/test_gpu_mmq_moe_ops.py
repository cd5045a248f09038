"""GPU parity, through the C ABI: Q4_K x int8 (mmq), routing and expert tables, activations, combine, the lane's
device-built tables and whole expert FFN, the MX roundings and the bounded host-flag wait."""
import os

import numpy as np
import pytest
import torch

from helpers import pointer_table, ptr, same_bits, sync, to_dev
from libosmos_b200 import api, synth
from oracle.oracle import TYPES

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


# ---- mmq ----------------------------------------------------------------------------------------------------------
def test_mmq_x8_rows(lib, dev, oracle):
    rng = synth.rng_for(31)
    cols, xs = 512, 520
    x = rng.standard_normal((9, xs)).astype(np.float32)
    x[2, 64:96] = 0.0
    idx = np.array([3, -1, 2, 8, 0, 0, 5, 1, 7, 4, 6, 2, -1, 3, 1, 0, 8, 2, 5], dtype=np.int32)  # 19 slots: two tiles
    w8, wdx, wsx = oracle.mmq_x8_rows(x, idx, cols)
    tiles = (idx.size + 15) // 16
    x8 = torch.zeros(tiles * 16 * cols, dtype=torch.int8, device=dev)
    dx = torch.zeros(tiles * 16 * (cols // 32), dtype=torch.float32, device=dev)
    sx = torch.zeros_like(dx)
    assert lib.mmq_x8_rows(ptr(to_dev(x, dev)), xs, ptr(to_dev(idx, dev)), idx.size, cols, ptr(x8), ptr(dx), ptr(sx), None)
    sync()
    assert np.array_equal(x8.cpu().numpy(), w8)
    assert same_bits(dx.cpu().numpy(), wdx) and same_bits(sx.cpu().numpy(), wsx)


@pytest.mark.parametrize("cnts", [[1], [16], [37, 5], [64, 1, 20]])
def test_mmq_group_bits(lib, dev, oracle, cnts):
    rows, cols, ys = 48, 1024, 56
    rng = synth.rng_for(32, len(cnts), cnts[0])
    mats = [synth.random_tensor(12, rows, cols, rng) for _ in cnts]
    n_tok = max(cnts)
    x = rng.standard_normal((n_tok, cols)).astype(np.float32)
    # matrix m's tokens are the first cnt[m] rows of x, in slots soff[m] ..
    soff, idx = [], []
    for c in cnts:
        soff.append(len(idx))
        idx += list(range(c)) + [-1] * ((16 - c % 16) % 16)
    idx = np.array(idx, dtype=np.int32)
    w8, wdx, wsx = oracle.mmq_x8_rows(x, idx, cols)
    yoff, total = [], 0
    for c in cnts:
        yoff.append(total * ys)
        total += c
    y = torch.full((total + 4, ys), -11.0, dtype=torch.float32, device=dev)
    pool = to_dev(np.concatenate(mats), dev)
    table = pointer_table(pool, [m * mats[0].size for m in range(len(mats))], dev)
    assert lib.mmq_group(12, ptr(table), ptr(to_dev(np.array(cnts, np.int32), dev)), len(cnts), max(cnts), rows, cols,
                         ptr(to_dev(w8, dev)), ptr(to_dev(wdx, dev)), ptr(to_dev(wsx, dev)),
                         ptr(to_dev(np.array(soff, np.uint32).view(np.int32), dev)), ptr(y),
                         ptr(to_dev(np.array(yoff, np.uint32).view(np.int32), dev)), ys, None)
    sync()
    got = y.cpu().numpy()
    want = np.full_like(got, -11.0)  # canary: nothing outside the live outputs is written
    r0 = 0
    for m, c in enumerate(cnts):
        want[r0:r0 + c, :rows] = oracle.mmq_rows(mats[m], rows, cols, w8, wdx, wsx, soff[m], c)
        r0 += c
    assert same_bits(got, want)


@pytest.mark.parametrize("rows,cols,cnts", [(128, 256, [16]), (128, 512, [1, 37]), (256, 768, [130, 5, 64]),
                                            (128, 2048, [300]), (384, 1024, [129])])
def test_mmq_tensor_kernel_matches_generic_and_oracle(lib, dev, oracle, rows, cols, cnts):
    """rows in 128s: mmq_group runs the tcgen05 kernel; its bits are the generic kernel's and the oracle's (K shorter
    than four partitions, several token tiles, several matrices with their own slots and outputs, canary rows)"""
    ys = rows + 8
    rng = synth.rng_for(41, rows, cols, len(cnts))
    mats = [synth.random_tensor(12, rows, cols, rng) for _ in cnts]
    x = rng.standard_normal((max(cnts), cols)).astype(np.float32)
    soff, idx = [], []
    for c in cnts:
        soff.append(len(idx))
        idx += list(range(c)) + [-1] * ((16 - c % 16) % 16)
    w8, wdx, wsx = oracle.mmq_x8_rows(x, np.array(idx, np.int32), cols)
    yoff, total = [], 0
    for c in cnts:
        yoff.append(total * ys)
        total += c
    pool = to_dev(np.concatenate(mats), dev)
    table = pointer_table(pool, [m * mats[0].size for m in range(len(mats))], dev)
    args = (ptr(to_dev(np.array(cnts, np.int32), dev)), len(cnts), max(cnts), rows, cols, ptr(to_dev(w8, dev)),
            ptr(to_dev(wdx, dev)), ptr(to_dev(wsx, dev)), ptr(to_dev(np.array(soff, np.uint32).view(np.int32), dev)))
    yo = ptr(to_dev(np.array(yoff, np.uint32).view(np.int32), dev))
    want = np.full((total + 4, ys), -11.0, np.float32)
    r0 = 0
    for m, c in enumerate(cnts):
        want[r0:r0 + c, :rows] = oracle.mmq_rows(mats[m], rows, cols, w8, wdx, wsx, soff[m], c)
        r0 += c
    for tensor in (1, 0):
        lib.mmq_set_tensor(tensor)
        y = torch.full((total + 4, ys), -11.0, dtype=torch.float32, device=dev)
        assert lib.mmq_group(12, ptr(table), *args, ptr(y), yo, ys, None)
        sync()
        assert same_bits(y.cpu().numpy(), want), "tensor-core kernel" if tensor else "generic kernel"
    lib.mmq_set_tensor(1)
    assert lib.mmq_status() == 0


# ---- routing and tables -------------------------------------------------------------------------------------------
def _softmax_topk(logits, k):
    l = logits.astype(np.float64)
    p = np.exp(l - l.max(1, keepdims=True))
    p /= p.sum(1, keepdims=True)
    order = np.argsort(-p, axis=1, kind="stable")[:, :k]
    pk = np.take_along_axis(p, order, 1)
    return order, pk / np.maximum(pk.sum(1, keepdims=True), 2.0 ** -14)


@pytest.mark.parametrize("n_exp,k,n_tok", [(512, 10, 64), (256, 8, 3), (60, 32, 2), (1024, 1, 5)])
def test_route(lib, dev, n_exp, k, n_tok):
    rng = synth.rng_for(33, n_exp, k)
    logits = rng.standard_normal((n_tok, n_exp)).astype(np.float32)
    ids = torch.empty((n_tok, k), dtype=torch.int32, device=dev)
    w = torch.empty((n_tok, k), dtype=torch.float32, device=dev)
    rows = torch.empty((n_tok, k), dtype=torch.int32, device=dev)
    assert lib.q4x_route(ptr(to_dev(logits, dev)), n_tok, n_exp, k, ptr(ids), ptr(w), ptr(rows), None)
    sync()
    want_ids, want_w = _softmax_topk(logits, k)
    assert np.array_equal(ids.cpu().numpy(), want_ids)
    assert np.allclose(w.cpu().numpy(), want_w, rtol=2e-6, atol=0)
    assert np.array_equal(rows.cpu().numpy(), np.repeat(np.arange(n_tok), k).reshape(n_tok, k))


def test_route_ties_and_nan(lib, dev):
    logits = np.zeros((2, 64), dtype=np.float32)          # all equal: the lowest ids, in order
    logits[1, 5] = np.nan                                  # a NaN poisons the softmax: still k distinct ids below n
    ids = torch.empty((2, 4), dtype=torch.int32, device=dev)
    w = torch.empty((2, 4), dtype=torch.float32, device=dev)
    rows = torch.empty((2, 4), dtype=torch.int32, device=dev)
    assert lib.q4x_route(ptr(to_dev(logits, dev)), 2, 64, 4, ptr(ids), ptr(w), ptr(rows), None)
    sync()
    got = ids.cpu().numpy()
    assert list(got[0]) == [0, 1, 2, 3] and np.allclose(w.cpu().numpy()[0], 0.25)
    assert len(set(got[1])) == 4 and got[1].min() >= 0 and got[1].max() < 64


def _tiles_reference(ids, k, n_exp, dim, ff, bounds, bytes_):
    """the tables by a host stable sort (the reference's own check: tests/gpu/test_q4x_moe_gpu.hip:68-83)"""
    n = ids.size
    order = np.argsort(ids, kind="stable")
    where = np.empty(n, np.int32)
    where[order] = np.arange(n)
    count = np.bincount(ids, minlength=n_exp)
    place0 = np.concatenate([[0], np.cumsum(count)[:-1]])
    slots_e = (count + 15) // 16 * 16
    slot0 = np.concatenate([[0], np.cumsum(slots_e)[:-1]])
    gidx = np.full(bounds.slots, -1, np.int32)
    hidx = np.full(bounds.slots, -1, np.int32)
    for i in order:
        e = ids[i]
        s = slot0[e] + where[i] - place0[e]
        gidx[s], hidx[s] = i // k, where[i]
    run_of = lambda c: 0 if c <= 16 else 1 if c <= 32 else 2 if c <= 64 else 3
    ent = {r: [] for r in range(4)}
    for e in range(n_exp):
        c = count[e]
        for part in range((c + 127) // 128):
            m = min(c - part * 128, 128)
            ent[run_of(m)].append((m, (slot0[e] + part * 128) * dim, (slot0[e] + part * 128) * ff,
                                   (place0[e] + part * 128) * ff, (place0[e] + part * 128) * dim, e))
    cnt = np.zeros(bounds.entries, np.int32)
    xg, xd, yg, yd = (np.zeros(bounds.entries, np.uint32) for _ in range(4))
    pe = np.full(bounds.entries, -1, np.int64)
    for r in range(4):
        for i, (m, a, b, c_, d_, e) in enumerate(ent[r]):
            at = bounds.first[r] + i
            cnt[at], xg[at], xd[at], yg[at], yd[at], pe[at] = m, a, b, c_, d_, e
    return where, gidx, hidx, cnt, xg, xd, yg, yd, pe


@pytest.mark.parametrize("n_tok,k,n_exp", [(3, 10, 512), (64, 10, 512), (256, 10, 64), (700, 4, 16)])
def test_expert_tiles(lib, dev, n_tok, k, n_exp):
    rng = synth.rng_for(34, n_tok, n_exp)
    n, dim, ff = n_tok * k, 2048, 512
    ids = np.stack([rng.permutation(n_exp)[:k] for _ in range(n_tok)]).astype(np.int32).reshape(-1)
    if n_exp == 16:
        ids[:300] = 3  # an expert past 128 tokens: several entries
    b = api.Q4xExpertBounds()
    lib.q4x_expert_bounds(n, n_exp, b)
    bytes_ = [1000, 2000, 3000]
    t = api.Q4xExpertTiles()
    bufs = {}
    for j in range(3):
        t.base[j], t.bytes[j], t.tab[j] = 0x100000 * (j + 1), bytes_[j], None
        bufs["ptr%d" % j] = torch.zeros(b.entries, dtype=torch.int64, device=dev)
        t.ptr[j] = ptr(bufs["ptr%d" % j])
    for name, size, dt in (("cnt", b.entries, torch.int32), ("gidx", b.slots, torch.int32), ("hidx", b.slots, torch.int32),
                           ("xg", b.entries, torch.int32), ("yg", b.entries, torch.int32), ("xd", b.entries, torch.int32),
                           ("yd", b.entries, torch.int32), ("where", n, torch.int32), ("off", 3 * n_exp, torch.int32)):
        bufs[name] = torch.full((size,), 77, dtype=dt, device=dev)
        setattr(t, name, ptr(bufs[name]))
    assert lib.q4x_expert_tiles(ptr(to_dev(ids, dev)), n, k, n_exp, dim, ff, t, None)
    sync()
    where, gidx, hidx, cnt, xg, xd, yg, yd, pe = _tiles_reference(ids, k, n_exp, dim, ff, b, bytes_)
    assert np.array_equal(bufs["where"].cpu().numpy(), where)
    assert np.array_equal(bufs["gidx"].cpu().numpy(), gidx) and np.array_equal(bufs["hidx"].cpu().numpy(), hidx)
    assert np.array_equal(bufs["cnt"].cpu().numpy(), cnt)
    live = cnt > 0
    for name, want in (("xg", xg), ("xd", xd), ("yg", yg), ("yd", yd)):
        assert np.array_equal(bufs[name].cpu().numpy().view(np.uint32)[live], want[live])
    for j in range(3):
        assert np.array_equal(bufs["ptr%d" % j].cpu().numpy()[live], 0x100000 * (j + 1) + pe[live] * bytes_[j])


def test_swiglu_and_moe_sum(lib, dev):
    rng = synth.rng_for(35)
    n_tok, k, dim = 7, 4, 36
    g = rng.standard_normal(300).astype(np.float32) * 3
    u = rng.standard_normal(300).astype(np.float32)
    y = torch.empty(300, dtype=torch.float32, device=dev)
    assert lib.q4x_swiglu(ptr(to_dev(g, dev)), ptr(to_dev(u, dev)), 300, ptr(y), None, None)
    sync()
    want = (g.astype(np.float64) / (1 + np.exp(-g.astype(np.float64)))) * u
    assert np.allclose(y.cpu().numpy(), want, rtol=3e-6, atol=1e-30)
    yy = rng.standard_normal((n_tok * k, dim)).astype(np.float32)
    where = rng.permutation(n_tok * k).astype(np.int32)
    w = rng.uniform(0, 1, n_tok * k).astype(np.float32)
    shared = rng.standard_normal((n_tok, dim)).astype(np.float32)
    logit = rng.standard_normal(n_tok).astype(np.float32)
    for off in (0, 1):  # the 16-byte path and the scalar one (an unaligned output)
        out = torch.empty(n_tok * dim + 1, dtype=torch.float32, device=dev)
        o = out[off:off + n_tok * dim]
        assert lib.q4x_moe_sum(ptr(to_dev(yy, dev)), ptr(to_dev(where, dev)), ptr(to_dev(w, dev)), n_tok, k, dim,
                               ptr(to_dev(shared, dev)), ptr(to_dev(logit, dev)), ptr(o), None)
        sync()
        got = o.cpu().numpy().reshape(n_tok, dim)
        gate = (1 / (1 + np.exp(-logit.astype(np.float64)))).astype(np.float32)
        acc = np.zeros((n_tok, dim), np.float32)
        for j in range(k):  # pick order, each product and sum rounded to F32
            acc = (acc + yy[where.reshape(n_tok, k)[:, j]] * w.reshape(n_tok, k)[:, j:j + 1]).astype(np.float32)
        want = acc + shared * gate[:, None]
        assert np.allclose(got, want, rtol=1e-6, atol=1e-6)
        if off == 0:
            first = got.copy()
        else:
            assert same_bits(first, got)  # both paths: the same operations, the same bits


def test_swiglu_side_and_swiglu_rows(lib, dev, oracle):
    """q4x_swiglu's f16 side output and q4x_swiglu_rows: the bits mm_x16 / mm_x16_rows make of q4x_swiglu's F32 output"""
    rng = synth.rng_for(38)
    rows, ff = 21, 48
    g = (rng.standard_normal((rows, ff)) * 3).astype(np.float32)
    u = rng.standard_normal((rows, ff)).astype(np.float32)
    g[3, 5], u[3, 5] = 90.0, 1.0e4  # past f16's range: the overflow flag
    gd, ud = to_dev(g, dev), to_dev(u, dev)
    y = torch.empty((rows, ff), dtype=torch.float32, device=dev)
    row0, padded = 16, 48
    side16 = torch.zeros(padded * ff, dtype=torch.float16, device=dev)
    over = torch.zeros(1, dtype=torch.int32, device=dev)
    side = api.Q4xX16(side16.data_ptr(), over.data_ptr(), ff, row0)
    assert lib.q4x_swiglu(ptr(gd), ptr(ud), rows * ff, ptr(y), side, None)
    sync()
    yh = y.cpu().numpy()
    want16, want_over = oracle.x16_rows(np.concatenate([np.zeros((row0, ff), np.float32), yh, np.zeros((padded - row0 - rows, ff), np.float32)]), padded, ff)
    assert np.array_equal(side16.cpu().numpy().view(np.uint16), want16) and int(over.item()) == 1 == want_over
    # the rows form: slots name rows of g / u, -1 a pad slot of zeros
    idx = np.array([4, -1, 0, 20, 7, 7, -1, 2, 9, 11, 13, 1, 19, 18, 17, 16, 15, -1, 3], dtype=np.int32)
    slots = 32
    full = np.concatenate([idx, -np.ones(slots - idx.size, np.int32)])
    x16 = torch.full((slots * ff,), 5.0, dtype=torch.float16, device=dev)
    over.zero_()
    assert lib.q4x_swiglu_rows(ptr(gd), ptr(ud), ff, ptr(to_dev(full, dev)), slots, ptr(x16), ptr(over), None)
    sync()
    want16, want_over = oracle.x16_rows(yh, slots, ff, idx=full)
    assert np.array_equal(x16.cpu().numpy().view(np.uint16), want16) and int(over.item()) == want_over == 1
    assert not lib.q4x_swiglu_rows(ptr(gd), ptr(ud), 40, ptr(to_dev(full, dev)), slots, ptr(x16), ptr(over), None)
    assert not lib.q4x_swiglu_rows(ptr(gd), ptr(ud), ff, 0, slots, ptr(x16), ptr(over), None)


# ---- lane ops ---------------------------------------------------------------------------------------------------------
def test_swiglu_lane_and_gathers(lib, dev, oracle):
    rng = synth.rng_for(36)
    n_tok, n = 9, 40
    g = (rng.standard_normal((n_tok, n)) * 6).astype(np.float32)
    u = (rng.standard_normal((n_tok, n)) * 6).astype(np.float32)
    scale = rng.uniform(0.1, 1, n_tok).astype(np.float32)
    h = torch.empty((n_tok, n), dtype=torch.float32, device=dev)
    assert lib.ops_swiglu_lane(ptr(to_dev(g, dev)), ptr(to_dev(u, dev)), n, 7.0, ptr(to_dev(scale, dev)), n_tok, ptr(h), None)
    sync()
    assert same_bits(h.cpu().numpy(), oracle.swiglu_lane(g, u, 7.0, scale))
    h2 = torch.empty((n_tok, n), dtype=torch.float32, device=dev)
    assert lib.ops_swiglu(ptr(to_dev(g, dev)), ptr(to_dev(u, dev)), n, 7.0, ptr(to_dev(scale, dev)), n_tok, ptr(h2), None)
    sync()
    assert np.allclose(h2.cpu().numpy(), h.cpu().numpy(), rtol=2e-6, atol=1e-12)
    src = rng.standard_normal((20, 24)).astype(np.float32)
    idx = rng.integers(0, 20, size=12).astype(np.int32)
    dst = torch.empty((12, 24), dtype=torch.float32, device=dev)
    assert lib.ops_gather_rows(ptr(dst), ptr(to_dev(src, dev)), ptr(to_dev(idx, dev)), 12, 24, None)
    add = rng.standard_normal((4, 24)).astype(np.float32)
    y = torch.empty((4, 24), dtype=torch.float32, device=dev)
    y2 = torch.empty((4, 24), dtype=torch.float32, device=dev)
    assert lib.ops_gather_sum(ptr(y), ptr(to_dev(src, dev)), ptr(to_dev(idx, dev)), 3, 4, 24, None)
    assert lib.ops_gather_sum_add(ptr(y2), ptr(to_dev(src, dev)), ptr(to_dev(idx, dev)), 3, 4, 24, ptr(to_dev(add, dev)), None)
    cp = torch.zeros((20, 24), dtype=torch.float32, device=dev)
    rows = np.array([4, 9, 17], dtype=np.int32)
    assert lib.ops_copy_rows(ptr(cp), ptr(to_dev(src, dev)), ptr(to_dev(rows, dev)), 3, 24, None)
    sync()
    assert same_bits(dst.cpu().numpy(), src[idx])
    assert same_bits(y.cpu().numpy(), oracle.gather_sum(src, idx, 3))
    assert same_bits(y2.cpu().numpy(), oracle.gather_sum(src, idx, 3, add))
    want = np.zeros_like(src)
    want[rows] = src[rows]
    assert same_bits(cp.cpu().numpy(), want)


@pytest.mark.parametrize("score", [0, 1])
def test_ops_router(lib, dev, score):
    rng = synth.rng_for(37, score)
    n_tok, n_exp, k = 5, 256, 8
    logits = rng.standard_normal((n_tok, n_exp)).astype(np.float32) * 2
    bias = (rng.standard_normal(n_exp) * 0.1).astype(np.float32)
    idx = torch.empty((n_tok, k), dtype=torch.int32, device=dev)
    w = torch.empty((n_tok, k), dtype=torch.float32, device=dev)
    assert lib.ops_router_scored(ptr(to_dev(logits, dev)), ptr(to_dev(bias, dev)), n_exp, k, 2.5, score, n_tok, ptr(idx), ptr(w), None)
    sync()
    l = logits.astype(np.float64)
    sc = 1 / (1 + np.exp(-l)) if score == 1 else np.sqrt(np.log1p(np.exp(l)))
    key = (sc.astype(np.float32) + bias).astype(np.float32)
    order = np.argsort(-key, axis=1, kind="stable")[:, :k]
    got = idx.cpu().numpy()
    # picks: exact unless two keys are within float rounding of each other
    srt = -np.sort(-key, axis=1)
    if np.min(srt[:, :k] - srt[:, 1:k + 1]) > 1e-6:
        assert np.array_equal(got, order)
    pk = np.take_along_axis(sc, got.astype(np.int64), 1)
    assert np.allclose(w.cpu().numpy(), pk / (pk.sum(1, keepdims=True) + 1e-20) * 2.5, rtol=3e-6)


def test_mx_rounding(lib, dev, oracle):
    rng = synth.rng_for(38)
    dim = 128
    x = (rng.standard_normal((6, dim)) * np.exp(rng.standard_normal((6, 1)) * 3)).astype(np.float32)
    x[0, :32] = 0.0
    for block, e4m3 in ((32, False), (16, True)):
        want, wp = oracle.fp4_round(x, block=block, e4m3_scale=e4m3, dim=dim)
        xd = to_dev(x.reshape(-1), dev).clone()
        packed = torch.zeros(wp.size, dtype=torch.uint8, device=dev)
        assert lib.ops_fp4_round(ptr(xd), x.size, block, e4m3, ptr(packed), dim, None)
        sync()
        assert same_bits(xd.cpu().numpy(), want) and np.array_equal(packed.cpu().numpy(), wp)
    want, wp = oracle.fp8_round(x, dim=dim)
    xd = to_dev(x.reshape(-1), dev).clone()
    packed = torch.zeros(wp.size, dtype=torch.uint8, device=dev)
    assert lib.ops_fp8_round(ptr(xd), x.size, ptr(packed), dim, None)
    sync()
    assert same_bits(xd.cpu().numpy(), want) and np.array_equal(packed.cpu().numpy(), wp)


def test_ops_wait_is_bounded(lib, dev):
    """a posted value lets the stream through; a value nothing posts runs into the bound and raises the status bit -
    the context stays usable (no trap, no endless spin)"""
    flag = torch.zeros(1, dtype=torch.int32).pin_memory()
    flag[0] = 5
    dptr = flag.data_ptr()  # pinned host memory is device-addressable at the same address under unified addressing
    assert lib.ops_wait_status() == 0
    assert lib.ops_wait(dptr, 5, None)
    sync()
    assert lib.ops_wait_status() == 0
    flag[0] = -2147483643        # 0x80000005: the poster's failure mark still releases the wait
    assert lib.ops_wait(dptr, 5, None)
    sync()
    assert lib.ops_wait_status() == 0
    lib.ops_wait_set_limit_ms(50)
    assert lib.ops_wait(dptr, 6, None)
    sync()
    assert lib.ops_wait_status() == 1 and lib.ops_wait_status() == 0
    lib.ops_wait_set_limit_ms(2000)
    y = torch.ones(4, device=dev) * 2
    assert float(y.sum().item()) == 8.0


# ---- the lane's tables and the whole expert FFN -----------------------------------------------------------------------------
def _lane_setup(lib, dev, name, n_tok, k, n_exp, dim, ff, key):
    tid = TYPES[name]
    rng = synth.rng_for(39, tid, key)
    per = [synth.tensor_bytes(tid, ff, dim), synth.tensor_bytes(tid, ff, dim), synth.tensor_bytes(tid, dim, ff)]
    tensors = [synth.random_tensor(tid, n_exp * (ff if j < 2 else dim), dim if j < 2 else ff, rng) for j in range(3)]
    dev_tensors = [to_dev(t, dev) for t in tensors]
    layer = api.LaneLayer(tid, tid, dim, ff, n_exp, k, 7.0, api.LaneExperts())
    for j in range(3):
        layer.experts.base[j], layer.experts.bytes[j], layer.experts.tab[j] = ptr(dev_tensors[j]), per[j], None
    nbytes = lib.lane_scratch_bytes(layer, n_tok)
    mem = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
    scratch = api.LaneScratch()
    assert lib.lane_scratch_bind(layer, n_tok, ptr(mem), nbytes, scratch)
    return tid, rng, per, tensors, dev_tensors, layer, scratch, mem


@pytest.mark.parametrize("name,n_tok,k,n_exp", [("IQ3_XXS", 12, 4, 16), ("IQ1_M", 5, 3, 8), ("IQ2_XXS", 40, 2, 4)])
def test_lane_ffn_matches_oracle(lib, dev, oracle, name, n_tok, k, n_exp):
    dim, ff = 512, 256
    tid, rng, per, tensors, dev_tensors, layer, scratch, mem = _lane_setup(lib, dev, name, n_tok, k, n_exp, dim, ff, n_tok)
    x = rng.standard_normal((n_tok, dim)).astype(np.float32)
    ids = np.stack([rng.permutation(n_exp)[:k] for _ in range(n_tok)]).astype(np.int32)
    wts = rng.uniform(0.05, 0.5, size=(n_tok, k)).astype(np.float32)
    add = rng.standard_normal((n_tok, dim)).astype(np.float32)
    out = torch.empty((n_tok, dim), dtype=torch.float32, device=dev)
    assert lib.lane_ffn(layer, scratch, ptr(to_dev(x, dev)), ptr(to_dev(ids, dev)), ptr(to_dev(wts, dev)), n_tok,
                        ptr(to_dev(add, dev)), ptr(out), None)
    sync()
    # the oracle: every pick's row through its expert, then each token's rows added in ascending expert id, then add
    want = np.zeros((n_tok, dim), np.float32)
    for t in range(n_tok):
        acc = np.zeros(dim, np.float32)
        for j in np.argsort(ids[t], kind="stable"):
            e = ids[t, j]
            parts = [tensors[m][e * per[m]:(e + 1) * per[m]] for m in range(3)]
            y = oracle.lane_expert(tid, tid, parts[0], parts[1], parts[2], dim, ff, 7.0, x[t:t + 1], wts[t, j:j + 1])
            acc = (acc + y[0]).astype(np.float32)
        want[t] = acc + add[t]
    assert same_bits(out.cpu().numpy(), want)


def test_lane_ffn_matches_reference_cpu_golden(lib, dev):
    """the reference's own cpu_lane_submit output (tests/golden/ffn.npz) for three experts of 1, 3 and 2 rows: here
    each row is a token with one pick"""
    g = np.load(os.path.join(GOLD, "ffn.npz"))
    dim, ff, lim = int(g["dim"]), int(g["ff"]), float(g["lim"])
    for name in ("IQ3_XXS", "IQ1_M"):
        tid = TYPES[name]
        counts = g[name + "_counts"]
        x, scale, want = g[name + "_x"], g[name + "_scale"], g[name + "_y"]
        n_tok = x.shape[0]
        tensors = [np.concatenate([g["%s_%s%d" % (name, part, e)] for e in range(len(counts))]) for part in ("gate", "up", "down")]
        dev_tensors = [to_dev(t, dev) for t in tensors]
        layer = api.LaneLayer(tid, tid, dim, ff, len(counts), 1, lim, api.LaneExperts())
        for j in range(3):
            layer.experts.base[j], layer.experts.bytes[j] = ptr(dev_tensors[j]), tensors[j].size // len(counts)
        nbytes = lib.lane_scratch_bytes(layer, n_tok)
        mem = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
        scratch = api.LaneScratch()
        assert lib.lane_scratch_bind(layer, n_tok, ptr(mem), nbytes, scratch)
        ids = np.repeat(np.arange(len(counts)), counts).astype(np.int32)
        out = torch.empty((n_tok, dim), dtype=torch.float32, device=dev)
        assert lib.lane_ffn(layer, scratch, ptr(to_dev(x, dev)), ptr(to_dev(ids, dev)), ptr(to_dev(scale, dev)), n_tok,
                            None, ptr(out), None)
        sync()
        # a single row summed from 0: 0 + y = y, the reference's bits
        assert same_bits(out.cpu().numpy(), want)


def test_lane_tables_large_step(lib, dev):
    """more picks than the table kernel places itself (the second kernel's path), and an expert range (another
    rank's experts have no rows here)"""
    n_tok, k, n_exp = 600, 4, 32
    rng = synth.rng_for(40)
    ids = np.stack([rng.permutation(n_exp)[:k] for _ in range(n_tok)]).astype(np.int32).reshape(-1)
    n = ids.size
    for e0, e1 in ((0, n_exp), (8, 20)):
        ents = lib.lane_max_entries(n, n_exp)
        t = api.LaneTables()
        bufs = {}
        for j in range(3):
            bufs["w%d" % j] = torch.zeros(ents, dtype=torch.int64, device=dev)
            t.w[j] = ptr(bufs["w%d" % j])
        for name, size in (("cnt", ents), ("xrow", ents), ("tok", n), ("pair", n), ("row_of", n), ("order", n),
                           ("off", 2 * n_exp), ("counts", 2)):
            bufs[name] = torch.full((size,), -7, dtype=torch.int32, device=dev)
            setattr(t, name, ptr(bufs[name]))
        t.max_entries = ents
        ex = api.LaneExperts()
        for j in range(3):
            ex.base[j], ex.bytes[j] = 0x1000000 * (j + 1), 4096 * (j + 1)
        assert lib.lane_tables(ptr(to_dev(ids, dev)), n, k, n_exp, e0, e1, ex, t, None)
        sync()
        own = (ids >= e0) & (ids < e1)
        order = [i for i in np.argsort(ids, kind="stable") if own[i]]
        rows = len(order)
        live, nrows = bufs["counts"].cpu().numpy()
        assert nrows == rows
        assert np.array_equal(bufs["pair"].cpu().numpy()[:rows], np.array(order, np.int32))
        assert np.array_equal(bufs["tok"].cpu().numpy()[:rows], np.array(order, np.int32) // k)
        row_of = np.full(n, -1, np.int32)
        row_of[order] = np.arange(rows)
        assert np.array_equal(bufs["row_of"].cpu().numpy(), row_of)
        cnt, xrow = bufs["cnt"].cpu().numpy(), bufs["xrow"].cpu().numpy()
        want_cnt, want_xrow, want_e = [], [], []
        r = 0
        for e in range(e0, e1):
            c = int((ids == e).sum())
            for part in range((c + 7) // 8):
                want_cnt.append(min(8, c - 8 * part)), want_xrow.append(r + 8 * part), want_e.append(e)
            r += c
        assert live == len(want_cnt) and list(cnt[:live]) == want_cnt and list(xrow[:live]) == want_xrow
        assert not cnt[live:].any()
        for j in range(3):
            assert list(bufs["w%d" % j].cpu().numpy()[:live]) == [0x1000000 * (j + 1) + e * 4096 * (j + 1) for e in want_e]
        got_order = bufs["order"].cpu().numpy().reshape(n_tok, k)
        ro = row_of.reshape(n_tok, k).astype(np.int64)
        ro[ro < 0] = 1 << 40
        want_order = np.sort(ro, axis=1)
        want_order[want_order == 1 << 40] = -1
        assert np.array_equal(got_order, want_order.astype(np.int32))
