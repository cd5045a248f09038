"""GPU parity, through the C ABI: the W4A4 product's activation quantization (mm_fp4_act, mm_fp4_quant) - the bytes of
the CPU oracle, bit for bit - and the product mm_fp4 within the reference's own bound: a relative error below 1e-5
against float64 sums over the quantized operands (tests/gpu/test_mm_fp4_gpu.hip:129-153 in the reference)."""
import numpy as np
import pytest
import torch

from helpers import ptr, sync, to_dev
from libosmos_b200 import synth
from oracle.oracle import TYPES

pytestmark = pytest.mark.gpu
NVFP4 = TYPES["NVFP4"]


def _bf16_bits(x):
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def _quant(lib, dev, x, cols, gs, seed=0, bf16=False, gs_on_device=False):
    n, xs = x.shape
    q = torch.full((n, cols // 2), 0xA5, dtype=torch.uint8, device=dev)
    sc = torch.full((n, cols // 16), 0xA5, dtype=torch.uint8, device=dev)
    xd = to_dev(x, dev)
    gd = to_dev(np.array([gs], np.float32), dev) if gs_on_device else None
    if seed == 0 and not bf16 and not gs_on_device:
        assert lib.mm_fp4_act(ptr(xd), xs, n, cols, gs, ptr(q), ptr(sc), None)
    else:
        assert lib.mm_fp4_quant(ptr(xd), int(bf16), xs, n, cols, 0.0 if gs_on_device else gs, ptr(gd) if gd is not None else None,
                                seed, ptr(q), ptr(sc), None)
    sync()
    return q.cpu().numpy(), sc.cpu().numpy()


@pytest.mark.parametrize("n,cols,pad,gs", [(1, 64, 0, 0.05), (33, 256, 0, 0.05), (7, 192, 3, 1.0), (64, 4096, 0, 0.013),
                                           (5, 128, 4, 1e-4), (3, 64, 0, 3e4)])
def test_fp4_act_bytes(lib, dev, oracle, n, cols, pad, gs):
    assert lib.mm_fp4_ok()
    rng = synth.rng_for(71, n, cols, pad)
    x = (rng.standard_normal((n, cols + pad)) * gs * 6.0).astype(np.float32)
    x[0, :16] = 0.0            # a group of zeros: scale code 0, codes 0
    x[n - 1, 16:32] *= 1e4     # past the largest scale: the scale saturates at 448, the codes at +-6
    x[0, 40] = -0.0
    wq, wsc = oracle.fp4_act(x, cols, gs)
    q, sc = _quant(lib, dev, x, cols, gs)
    assert np.array_equal(sc, wsc) and np.array_equal(q, wq)
    assert wsc[0, 0] == 0 and not wq[0, :8].any() and wsc[n - 1, 1] == 0x7E


def test_fp4_act_every_tie_and_boundary(lib, dev, oracle):
    """values at and next to every rounding boundary of the code grid, under a scale of exactly 1"""
    edges = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 0.5, 1, 1.5, 2, 3, 4, 6], np.float32)
    vals = np.concatenate([edges, np.nextafter(edges, np.float32(0)), np.nextafter(edges, np.float32(9))])
    vals = np.concatenate([vals, -vals])
    groups = []
    for v in vals:  # a group whose amax is 6 (scale code of 1.0 under gs = 1), the value under test beside it
        g = np.zeros(16, np.float32)
        g[0], g[5] = 6.0, v
        groups.append(g)
    while len(groups) % 4:
        groups.append(np.zeros(16, np.float32))
    x = np.concatenate(groups).reshape(1, -1)
    cols = x.shape[1]
    wq, wsc = oracle.fp4_act(x, cols, 1.0)
    q, sc = _quant(lib, dev, x, cols, 1.0)
    assert np.array_equal(sc, wsc) and np.array_equal(q, wq)
    assert (wsc[0, :len(vals)] == 0x38).all()  # 1.0


def test_fp4_act_scale_codes_sweep(lib, dev, oracle):
    """every scale code is produced and agrees: amax swept over E4M3's whole range, subnormals and saturation too"""
    amax = np.concatenate([np.geomspace(1e-4, 5000, 4096), 6.0 * np.arange(0, 18) * 2.0 ** -9]).astype(np.float32)
    while amax.size % 4:
        amax = np.append(amax, np.float32(1))
    x = np.zeros((1, amax.size * 16), np.float32)
    x[0, 3::16] = amax
    x[0, 7::16] = -amax * 0.37
    wq, wsc = oracle.fp4_act(x, x.shape[1], 1.0)
    q, sc = _quant(lib, dev, x, x.shape[1], 1.0)
    assert np.array_equal(sc, wsc) and np.array_equal(q, wq)
    assert len(np.unique(wsc)) > 100


@pytest.mark.parametrize("seed,on_device", [(12345, False), (1, False), (977, True)])
def test_fp4_quant_bf16_and_stochastic(lib, dev, oracle, seed, on_device):
    n, cols, gs = 19, 320, 0.05
    rng = synth.rng_for(72, seed)
    xf = (rng.standard_normal((n, cols)) * gs * 6.0).astype(np.float32)
    xb = _bf16_bits(xf)
    for bf16, x in ((False, xf), (True, xb)):
        # a scale read on the device salts the seed with the scale's bits (never 0)
        eff = ((seed ^ (int(np.float32(gs).view(np.uint32)) * 0x9E3779B1 & 0xFFFFFFFF)) | 1) if on_device else seed
        wq, wsc = oracle.fp4_act(x, cols, gs, seed=eff, bf16=bf16)
        q, sc = _quant(lib, dev, x, cols, gs, seed=seed, bf16=bf16, gs_on_device=on_device)
        assert np.array_equal(sc, wsc) and np.array_equal(q, wq)
    nq, _ = oracle.fp4_act(xf, cols, gs)
    assert not np.array_equal(nq, wq)  # (the stochastic codes are not the nearest ones)


@pytest.mark.parametrize("rows,cols,n", [(128, 128, 1), (256, 512, 37), (144, 1024, 130), (1024, 2048, 300)])
def test_mm_fp4_product(lib, dev, oracle, rows, cols, n):
    rng = synth.rng_for(73, rows, cols, n)
    gs, wscale = 0.05, 0.7
    w = synth.random_tensor(NVFP4, rows, cols, rng)
    x = (rng.standard_normal((n, cols)) * gs * 6.0).astype(np.float32)
    q, sc = oracle.fp4_act(x, cols, gs)
    want, mag = oracle.fp4_mm(w, rows, cols, q, sc, scale=wscale * gs)
    y = torch.full((n, rows), float("nan"), dtype=torch.float32, device=dev)
    qd, sd = to_dev(q, dev), to_dev(sc, dev)
    assert lib.mm_fp4(ptr(to_dev(w, dev)), rows, cols, ptr(qd), ptr(sd), n, wscale * gs, ptr(y), rows, None)
    sync()
    assert lib.mm_status() == 0
    got = y.cpu().numpy().astype(np.float64)
    rel = np.sqrt(((got - want) ** 2).sum() / (want ** 2).sum())
    assert rel < 1e-5, rel  # the reference's bound
    # and element by element: exact products, F32 additions (a bound of (cols / 16 + 20) half-ulps of the magnitudes)
    assert (np.abs(got - want) <= (cols / 16 + 20) * 2.0 ** -24 * mag + 1e-30).all()


def test_mm_fp4_past_one_x16_and_batch_invariance(lib, dev, oracle):
    """more tokens than one tiled x16 holds; a token's sums are the same bits alone and in the batch"""
    rows, cols, n = 128, 128, 2048 + 77
    rng = synth.rng_for(74)
    w = synth.random_tensor(NVFP4, rows, cols, rng)
    x = rng.standard_normal((n, cols)).astype(np.float32)
    q, sc = oracle.fp4_act(x, cols, 0.2)
    wd, qd, sd = to_dev(w, dev), to_dev(q, dev), to_dev(sc, dev)
    y = torch.full((n, rows), float("nan"), dtype=torch.float32, device=dev)
    assert lib.mm_fp4(ptr(wd), rows, cols, ptr(qd), ptr(sd), n, 1.0, ptr(y), rows, None)
    sync()
    got = y.cpu().numpy()
    want, mag = oracle.fp4_mm(w, rows, cols, q[-80:], sc[-80:])
    assert (np.abs(got[-80:] - want) <= (cols / 16 + 20) * 2.0 ** -24 * mag).all()
    for t in (0, 2047, 2048, n - 1):
        y1 = torch.zeros((1, rows), dtype=torch.float32, device=dev)
        assert lib.mm_fp4(ptr(wd), rows, cols, ptr(qd[t:t + 1].contiguous()), ptr(sd[t:t + 1].contiguous()), 1, 1.0, ptr(y1), rows, None)
        sync()
        assert np.array_equal(y1.cpu().numpy()[0].view(np.uint32), got[t].view(np.uint32))


def test_mm_fp4_refusals(lib, dev):
    a = torch.zeros(4096, dtype=torch.uint8, device=dev)
    y = torch.zeros(4096, dtype=torch.float32, device=dev)
    assert not lib.mm_fp4(ptr(a), 128, 96, ptr(a), ptr(a), 1, 1.0, ptr(y), 128, None)    # cols not in 128s
    assert not lib.mm_fp4(ptr(a), 120, 128, ptr(a), ptr(a), 1, 1.0, ptr(y), 128, None)   # rows not in 16s
    assert not lib.mm_fp4(ptr(a), 128, 128, ptr(a), ptr(a), 0, 1.0, ptr(y), 128, None)   # no tokens
    assert not lib.mm_fp4(ptr(a), 128, 128, ptr(a), ptr(a), 2, 1.0, ptr(y), 64, None)    # ys shorter than a row
    assert not lib.mm_fp4_act(ptr(y), 96, 1, 96, 1.0, ptr(a), ptr(a), None)              # cols not in 64s
    assert not lib.mm_fp4_act(ptr(y), 64, 1, 64, 0.0, ptr(a), ptr(a), None)              # a scale not above 0
    assert not lib.mm_fp4_act(ptr(y), 32, 2, 64, 1.0, ptr(a), ptr(a), None)              # xs shorter than a row


# ---- the block-scaled FP4 tensor-core route ------------------------------------------------------------------------------
@pytest.mark.parametrize("rows,cols,n", [(128, 256, 1), (128, 256, 16), (128, 512, 129), (256, 1024, 256), (384, 2048, 700)])
def test_mm_fp4_tensor_route(lib, dev, oracle, rows, cols, n):
    """mm_fp4 on tcgen05.mma kind::mxf4nvf4 (whole 128-row tiles, 256-value steps) against float64 sums over the quantized
    operands, and against the f16 route; scale bytes with a sign bit and the byte 0x7F (ggml: ignored, zero) among them"""
    rng = synth.rng_for(75, rows, cols, n)
    gs, wscale = 0.05, 0.7
    w = synth.random_tensor(NVFP4, rows, cols, rng).reshape(-1, 36)
    w[3::17, 1] |= 0x80   # a sign bit on a scale: read without it
    w[5::23, 2] = 0x7F    # the byte ggml reads as zero
    w = w.reshape(-1)
    x = (rng.standard_normal((n, cols)) * gs * 6.0).astype(np.float32)
    q, sc = oracle.fp4_act(x, cols, gs)
    want, mag = oracle.fp4_mm(w, rows, cols, q, sc, scale=wscale * gs)
    wd, qd, sd = to_dev(w, dev), to_dev(q, dev), to_dev(sc, dev)
    outs = []
    for tensor in (1, 0):
        lib.mm_fp4_set_tensor(tensor)
        y = torch.full((n, rows), float("nan"), dtype=torch.float32, device=dev)
        assert lib.mm_fp4(ptr(wd), rows, cols, ptr(qd), ptr(sd), n, wscale * gs, ptr(y), rows, None)
        assert lib.mm_fp4_last_route() == tensor
        sync()
        outs.append(y.cpu().numpy().astype(np.float64))
    lib.mm_fp4_set_tensor(1)
    assert lib.mm_status() == 0
    for got in outs:
        assert (np.abs(got - want) <= (cols / 16 + 20) * 2.0 ** -24 * mag + 1e-30).all()
        assert np.sqrt(((got - want) ** 2).sum() / (want ** 2).sum()) < 1e-5
    # a token's sums do not depend on the tokens beside it
    for t in sorted({0, n // 2, n - 1}):
        y1 = torch.zeros((1, rows), dtype=torch.float32, device=dev)
        assert lib.mm_fp4(ptr(wd), rows, cols, ptr(qd[t:t + 1].contiguous()), ptr(sd[t:t + 1].contiguous()), 1, wscale * gs, ptr(y1), rows, None)
        sync()
        assert np.array_equal(y1.cpu().numpy()[0].astype(np.float64), outs[0][t])


@pytest.mark.parametrize("rows,cols,n", [(128, 512, 1), (128, 512, 40), (256, 1536, 300), (384, 4096, 64)])
def test_mm_mxfp4(lib, dev, oracle, rows, cols, n):
    """MXFP4 weights x MXFP4 activations on tcgen05.mma kind::mxf4: the activations rounded by ops_fp4_round (its packed
    rows feed the product as they are), against float64 sums over the quantized operands"""
    tid = TYPES["MXFP4"]
    rng = synth.rng_for(76, rows, cols, n)
    w = synth.random_tensor(tid, rows, cols, rng)
    x = (rng.standard_normal((n, cols)) * 3.0).astype(np.float32)
    xr, packed = oracle.fp4_round(x, 32, False, cols)  # the rounded values and the packed codes + scales
    xd = to_dev(x.reshape(-1), dev)
    pk = torch.zeros(n * (cols // 2 + cols // 32), dtype=torch.uint8, device=dev)
    assert lib.ops_fp4_round(ptr(xd), n * cols, 32, False, ptr(pk), cols, None)
    sync()
    assert np.array_equal(pk.cpu().numpy(), packed)
    wf = oracle.dequant(tid, w, rows * cols).reshape(rows, cols).astype(np.float64)
    xq = xr.reshape(n, cols).astype(np.float64)
    want, mag = 0.5 * (xq @ wf.T), 0.5 * (np.abs(xq) @ np.abs(wf).T)
    y = torch.full((n, rows), float("nan"), dtype=torch.float32, device=dev)
    assert lib.mm_mxfp4(ptr(to_dev(w, dev)), rows, cols, ptr(pk), n, 0.5, ptr(y), rows, None)
    sync()
    assert lib.mm_status() == 0
    got = y.cpu().numpy().astype(np.float64)
    assert (np.abs(got - want) <= (cols / 16 + 20) * 2.0 ** -24 * mag + 1e-30).all()
    assert not lib.mm_mxfp4(ptr(pk), 128, 256, ptr(pk), 1, 1.0, ptr(y), 128, None)  # cols not whole 512s
    assert not lib.mm_mxfp4(ptr(pk), 64, 512, ptr(pk), 1, 1.0, ptr(y), 64, None)    # rows not whole 128s
