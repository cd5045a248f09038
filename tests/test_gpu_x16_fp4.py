"""GPU parity, through the C ABI: the tiled f16 activation layout (mm_x16, mm_x16_rows, mm_x16_heads) and NVFP4's own
matvec (mv_fp4, mv_fp4_tok) against the CPU oracle. Bit-exact; the matvec also within its rounding bound of a
float64 sum over the same values (the reference's own check: tests/gpu/test_mv_fp4_tok_gpu.hip:97-112)."""
import numpy as np
import pytest
import torch

from helpers import ptr, same_bits, sync, to_dev
from libosmos_b200 import synth
from oracle.oracle import TYPES

pytestmark = pytest.mark.gpu
NVFP4 = TYPES["NVFP4"]


def _tiled(dev, slots, cols, heads=1):
    padded = (slots + 15) // 16 * 16
    return torch.full((heads * padded * cols,), 0x7BFF, dtype=torch.int16, device=dev)  # (a non-zero fill)


@pytest.mark.parametrize("n,cols,pad", [(1, 64, 0), (16, 128, 8), (37, 1040, 4), (5, 48, 1), (2048, 32, 0)])
def test_mm_x16_bits_layout_and_padding(lib, dev, oracle, n, cols, pad):
    rng = synth.rng_for(31, n, cols)
    xs = cols + pad  # pad 1: rows not 16-byte aligned, the single-load path
    x = (rng.standard_normal((n, xs)) * 40).astype(np.float32)
    want, over = oracle.x16_rows(x, n, cols)
    assert over == 0
    out, flag = _tiled(dev, n, cols), torch.zeros(1, dtype=torch.int32, device=dev)
    assert lib.mm_x16(ptr(to_dev(x, dev)), xs, n, cols, ptr(out), ptr(flag), None)
    sync()
    assert np.array_equal(out.cpu().numpy().view(np.uint16), want) and int(flag.item()) == 0
    # the layout function the header gives is the one the kernel wrote with
    t, c = n - 1, cols - 3
    at = (t // 16) * 16 * cols + (c // 16) * 256 + (t % 16) * 16 + c % 16
    assert want[at] == np.float32(x[t, c]).astype(np.float16).view(np.uint16)


@pytest.mark.parametrize("bad", [70000.0, -1e9, float("nan"), float("inf")])
def test_mm_x16_overflow_flag(lib, dev, oracle, bad):
    x = np.zeros((3, 64), np.float32)
    x[1, 17] = bad
    want, over = oracle.x16_rows(x, 3, 64)
    assert over == 1
    out, flag = _tiled(dev, 3, 64), torch.zeros(1, dtype=torch.int32, device=dev)
    assert lib.mm_x16(ptr(to_dev(x, dev)), 64, 3, 64, ptr(out), ptr(flag), None)
    sync()
    got = out.cpu().numpy().view(np.uint16)
    assert int(flag.item()) == 1
    if np.isnan(bad):  # a NaN stays a NaN (its payload is the converter's own; the step is refused anyway)
        at = np.flatnonzero(got != want)
        assert at.size == 1 and np.isnan(got[at].view(np.float16)[0]) and np.isnan(want[at].view(np.float16)[0])
    else:
        assert np.array_equal(got, want)
    x[1, 17] = 65504.0  # the largest f16 is not an overflow
    flag.zero_()
    assert lib.mm_x16(ptr(to_dev(x, dev)), 64, 3, 64, ptr(out), ptr(flag), None)
    sync()
    assert int(flag.item()) == 0


def test_mm_x16_rows_gathers_and_zeroes(lib, dev, oracle):
    rng = synth.rng_for(32)
    rows, cols, xs, slots = 23, 272, 280, 41
    x = rng.standard_normal((rows, xs)).astype(np.float32)
    idx = rng.integers(-1, rows, size=slots).astype(np.int32)
    idx[[0, 7, 40]] = -1
    want, over = oracle.x16_rows(x, slots, cols, idx)
    out, flag = _tiled(dev, slots, cols), torch.zeros(1, dtype=torch.int32, device=dev)
    assert lib.mm_x16_rows(ptr(to_dev(x, dev)), xs, ptr(to_dev(idx, dev)), slots, cols, ptr(out), ptr(flag), None)
    sync()
    assert np.array_equal(out.cpu().numpy().view(np.uint16), want) and int(flag.item()) == over == 0
    assert not lib.mm_x16_rows(ptr(out), xs - 1, ptr(out), slots, cols, ptr(out), ptr(flag), None)  # xs not whole float4s


def test_mm_x16_heads_is_mm_x16_a_head(lib, dev, oracle):
    rng = synth.rng_for(33)
    n, heads, hs, cols = 21, 3, 96, 80
    xs = heads * hs
    x = rng.standard_normal((n, xs)).astype(np.float32)
    out, flag = _tiled(dev, n, cols, heads), torch.zeros(1, dtype=torch.int32, device=dev)
    assert lib.mm_x16_heads(ptr(to_dev(x, dev)), xs, n, heads, hs, cols, ptr(out), ptr(flag), None)
    sync()
    got = out.cpu().numpy().view(np.uint16).reshape(heads, -1)
    for h in range(heads):
        want, _ = oracle.x16_rows(np.ascontiguousarray(x[:, h * hs:h * hs + cols]), n, cols)
        assert np.array_equal(got[h], want)


def _table(tensors, dev):
    """device table of the tensors' addresses"""
    return torch.tensor([t.data_ptr() for t in tensors], dtype=torch.int64, device=dev)


def _fp4_case(rows, cols, ntok, key):
    rng = synth.rng_for(34, rows, cols, key)
    w = synth.random_tensor(NVFP4, rows, cols, rng)
    x = rng.standard_normal((ntok, cols + 4)).astype(np.float32)
    return w, x


def _f64_bound_ok(oracle, w, rows, cols, x, y):
    wv = oracle.dequant(NVFP4, w, rows * cols).reshape(rows, cols).astype(np.float64)
    xv = x[:, :cols].astype(np.float64)
    exact, mag = xv @ wv.T, np.abs(xv) @ np.abs(wv.T)
    return np.all(np.abs(y - exact) <= cols * 6e-8 * (mag + 1e-30))


@pytest.mark.parametrize("rows,cols", [(50, 320), (33, 2112), (16, 6144)])
def test_mv_fp4_bits_and_token_invariance(lib, dev, oracle, rows, cols):
    w, x = _fp4_case(rows, cols, 4, 0)
    scale = 0.37
    want = oracle.mv_fp4_rows(w, rows, cols, x, 32, scale)
    assert _f64_bound_ok(oracle, w, rows, cols, x, want / np.float32(scale))
    wd, xd = to_dev(w, dev), to_dev(x, dev)
    for n in (4, 3, 2, 1):
        y = torch.full((n, rows + 3), -2.0, dtype=torch.float32, device=dev)
        assert lib.mv_fp4(ptr(wd), rows, cols, ptr(xd), cols + 4, n, ptr(y), rows + 3, scale, None)
        sync()
        got = y.cpu().numpy()
        assert same_bits(got[:, :rows], want[:n]) and (got[:, rows:] == -2.0).all()
    assert not lib.mv_fp4(ptr(wd), rows, cols, ptr(xd), cols + 4, 5, ptr(xd), rows, scale, None)
    assert not lib.mv_fp4(ptr(wd), rows, cols + 32, ptr(xd), cols + 4, 1, ptr(xd), rows, scale, None)


@pytest.mark.parametrize("cols,lanes", [(1536, 8), (3072, 16), (6144, 32), (64, 8)])
def test_mv_fp4_tok_entries(lib, dev, oracle, cols, lanes):
    rows, n_mat = 40, 6
    rng = synth.rng_for(35, cols)
    mats = [synth.random_tensor(NVFP4, rows, cols, rng) for _ in range(n_mat)]
    cnt, xrow = [1, 4, 0, 3, 2, 4], [0, 1, 5, 5, 8, 10]
    total = 14
    x = rng.standard_normal((total + 4, cols)).astype(np.float32)
    xd = to_dev(x, dev)
    devs = [to_dev(m, dev) for m in mats]
    table = _table(devs, dev)
    y = torch.full((total, rows), -5.0, dtype=torch.float32, device=dev)
    assert lib.mv_fp4_tok(ptr(table), ptr(to_dev(np.array(cnt, np.int32), dev)), ptr(to_dev(np.array(xrow, np.int32), dev)),
                          n_mat, rows, cols, ptr(xd), cols, ptr(y), rows, None)
    sync()
    got = y.cpu().numpy()
    want = np.full((total, rows), -5.0, np.float32)
    for m in range(n_mat):
        if cnt[m]:
            want[xrow[m]:xrow[m] + cnt[m]] = oracle.mv_fp4_rows(mats[m], rows, cols, x[xrow[m]:xrow[m] + cnt[m]], lanes)
    assert same_bits(got, want)
    # each token alone, an entry of its own: the same bits (a step's split does not change a token's sums)
    p1, c1, r1 = [], [], []
    for m in range(n_mat):
        for t in range(cnt[m]):
            p1.append(devs[m]), c1.append(1), r1.append(xrow[m] + t)
    y1 = torch.full((total, rows), -5.0, dtype=torch.float32, device=dev)
    assert lib.mv_fp4_tok(ptr(_table(p1, dev)), ptr(to_dev(np.array(c1, np.int32), dev)),
                          ptr(to_dev(np.array(r1, np.int32), dev)), len(p1), rows, cols, ptr(xd), cols, ptr(y1), rows, None)
    sync()
    assert same_bits(y1.cpu().numpy(), got)
    assert not lib.mv_fp4_tok(None, None, None, 1, 16, 64, None, 64, None, 16, None)


def _attn_case(n, heads, head_dim, rope_dim, seed, pos_zero=False):
    rng = synth.rng_for(33, n, heads, head_dim, rope_dim, seed)
    cols = heads * head_dim
    x = (rng.standard_normal((n, cols)) * 3).astype(np.float32)
    freqs = (10000.0 ** (-np.arange(max(rope_dim // 2, 1)) / max(rope_dim // 2, 1))).astype(np.float32)
    pos = np.zeros(n, np.int32) if pos_zero else rng.integers(0, 4000, n).astype(np.int32)
    return x, cols, freqs, pos


def _run_attn(lib, dev, x, n, cols, head_dim, rope_dim, freqs, pos):
    out, flag = _tiled(dev, n, cols), torch.zeros(1, dtype=torch.int32, device=dev)
    assert lib.mm_x16_attn(ptr(to_dev(x, dev)), x.shape[1], n, cols, head_dim, rope_dim, ptr(to_dev(freqs, dev)),
                           ptr(to_dev(pos, dev)), ptr(out), ptr(flag), None)
    sync()
    return out.cpu().numpy().view(np.uint16), int(flag.item())


@pytest.mark.parametrize("n,heads,head_dim,rope_dim,pos_zero", [(5, 2, 64, 0, False), (16, 3, 128, 64, True), (37, 2, 192, 64, True)])
def test_mm_x16_attn_exact_cases(lib, dev, oracle, n, heads, head_dim, rope_dim, pos_zero):
    """no rotation, or a rotation by angle 0 (cos 1, sin 0 in every library): the oracle's bits"""
    x, cols, freqs, pos = _attn_case(n, heads, head_dim, rope_dim, 1, pos_zero)
    want, over = oracle.x16_attn(x, n, cols, head_dim, rope_dim, freqs, pos)
    got, flag = _run_attn(lib, dev, x, n, cols, head_dim, rope_dim, freqs, pos)
    assert np.array_equal(got, want) and flag == over == 0


def test_mm_x16_attn_rotated(lib, dev, oracle):
    """general positions: the device's cosine and sine may differ from the host library's in the last place, which moves
    a value across an E4M3 rounding boundary now and then - by one step at most, in well under 1 % of the values"""
    n, heads, head_dim, rope_dim = 50, 4, 128, 64
    x, cols, freqs, pos = _attn_case(n, heads, head_dim, rope_dim, 2)
    want, over = oracle.x16_attn(x, n, cols, head_dim, rope_dim, freqs, pos)
    got, flag = _run_attn(lib, dev, x, n, cols, head_dim, rope_dim, freqs, pos)
    assert flag == over == 0
    g, w = got.view(np.float16).astype(np.float64), want.view(np.float16).astype(np.float64)
    off = g != w
    assert off.mean() < 0.01
    assert (np.abs(g - w)[off] <= 0.126 * np.maximum(np.abs(w[off]), 2.0 ** -6)).all()
    # the part of every head that is not rotated has the oracle's bits everywhere
    keep = np.zeros((64, cols), bool)
    keep[:, [c for c in range(cols) if c % head_dim < head_dim - rope_dim]] = True
    idx = [(t // 16) * 16 * cols + (c // 16) * 256 + (t % 16) * 16 + c % 16 for t in range(n) for c in range(cols) if keep[t, c]]
    assert np.array_equal(got[idx], want[idx])
    assert not got[[(48 // 16) * 16 * cols + (c // 16) * 256 + (t % 16) * 16 + c % 16 for t in range(50, 64) for c in range(cols)]].any()


def test_mm_x16_attn_refusals(lib, dev):
    a = torch.zeros(4096, dtype=torch.float32, device=dev)
    f = torch.zeros(1, dtype=torch.int32, device=dev)
    args = lambda n, cols, hd, rd, xs=None: (ptr(a), xs or cols, n, cols, hd, rd, ptr(a), ptr(f), ptr(a), ptr(f), None)
    assert not lib.mm_x16_attn(*args(0, 128, 64, 32)) and not lib.mm_x16_attn(*args(2049, 128, 64, 32))
    assert not lib.mm_x16_attn(*args(2, 128, 48, 0)) and not lib.mm_x16_attn(*args(2, 128, 64, 48))
    assert not lib.mm_x16_attn(*args(2, 128, 64, 33)) and not lib.mm_x16_attn(*args(2, 128, 64, 96))
    assert not lib.mm_x16_attn(*args(2, 192, 128, 64)) and not lib.mm_x16_attn(*args(2, 128, 64, 32, xs=64))
