"""The CPU oracle against the committed golden vectors (no GPU): gguf-py's values for every block decoder, and the
reference's own CPU lane outputs for the int8 lane, the F32 matvec and the expert FFN."""
import os

import numpy as np
import pytest

from oracle.oracle import BLOCK, LANE_TYPES, TYPES, Reference

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


OWN_TYPES = ("Q2_0", "MXFP8")  # the reference's own ids 42 and 43: gguf-py has no decoder for them


@pytest.mark.parametrize("name", sorted(set(TYPES) - set(OWN_TYPES)))
def test_decoder_matches_gguf_py(oracle, name):
    g = np.load(os.path.join(GOLD, "dequant.npz"))
    raw, want = g[name + "_raw"], g[name + "_values"]
    got = oracle.dequant(TYPES[name], raw, raw.shape[0] * BLOCK[TYPES[name]][0])
    assert got is not None
    assert np.array_equal(_bits(got), _bits(want))


def test_own_types_match_their_definitions(oracle):
    """Q2_0: an F16 scale times (2-bit code - 1); MXFP8: 2^(e - 127) times an E4M3 value - written out here in numpy,
    the E4M3 values taken from torch's float8_e4m3fn: independent of the oracle's C"""
    import torch
    from libosmos_b200 import synth
    raw = synth.random_blocks(TYPES["Q2_0"], 40, synth.rng_for(111))
    d = raw[:, :2].copy().view(np.float16).astype(np.float32)  # [40, 1]
    codes = (raw[:, 2:, None] >> (2 * np.arange(4, dtype=np.uint8))) & 3  # [40, 16, 4]: value 4 b + i of byte b
    want = (d * (codes.reshape(40, 64).astype(np.float32) - 1.0)).astype(np.float32)
    got = oracle.dequant(TYPES["Q2_0"], raw, 40 * 64)
    assert np.array_equal(_bits(got), _bits(want.reshape(-1)))
    raw = synth.random_blocks(TYPES["MXFP8"], 40, synth.rng_for(112))
    raw[:, 0] = np.arange(40) * 6  # exponents from the subnormal end up
    vals = torch.from_numpy(raw[:, 1:].copy()).view(torch.float8_e4m3fn).to(torch.float32).numpy()
    want = (np.ldexp(np.float32(1.0), raw[:, :1].astype(np.int32) - 127).astype(np.float32) * vals).astype(np.float32)
    got = oracle.dequant(TYPES["MXFP8"], raw, 40 * 32)
    assert np.array_equal(_bits(got), _bits(want.reshape(-1)))


@pytest.mark.parametrize("name", LANE_TYPES)
def test_lane_matches_reference_cpu(oracle, name):
    g = np.load(os.path.join(GOLD, "lane_%s.npz" % name))
    tid = TYPES[name]
    for cols in (512, 768, 4096):
        w, x = g["w_%d" % cols], g["x_%d" % cols]
        q, d = oracle.q8_round(x)
        assert np.array_equal(q, g["q_%d" % cols]) and np.array_equal(_bits(d), _bits(g["d_%d" % cols]))
        y = oracle.q8_rows(tid, w, 10, cols, q, d)
        assert np.array_equal(_bits(y), _bits(g["y_%d" % cols])), "int8 lane sums differ from the reference's"
        ymv = oracle.mv_rows(tid, w, 10, cols, x)
        assert np.array_equal(_bits(ymv), _bits(g["ymv_%d" % cols])), "F32 matvec sums differ from the reference's"


def test_round_special_blocks(oracle):
    # the reference's own assertions (tests/test_cpu_q8.c:191-197): zeros give d 0 / q 0, a lone -2.5 gives -127
    x = np.zeros((1, 64), dtype=np.float32)
    x[0, 37] = -2.5
    q, d = oracle.q8_round(x)
    assert d[0, 0] == 0.0 and not q[0, :32].any() and q[0, 37] == -127 and d[0, 1] == np.float32(2.5) / np.float32(127)


@pytest.mark.parametrize("name", ["IQ3_XXS", "IQ1_M"])
def test_expert_ffn_matches_reference_cpu(oracle, name):
    g = np.load(os.path.join(GOLD, "ffn.npz"))
    dim, ff, lim = int(g["dim"]), int(g["ff"]), float(g["lim"])
    tid = TYPES[name]
    x, scale, want = g[name + "_x"], g[name + "_scale"], g[name + "_y"]
    row0 = 0
    for e, c in enumerate(g[name + "_counts"]):
        y = oracle.lane_expert(tid, tid, g["%s_gate%d" % (name, e)], g["%s_up%d" % (name, e)],
                               g["%s_down%d" % (name, e)], dim, ff, lim, x[row0:row0 + c], scale[row0:row0 + c])
        assert np.array_equal(_bits(y), _bits(want[row0:row0 + c]))
        row0 += c


def test_lane_exp_is_close_to_exp(oracle):
    x = np.linspace(-20, 20, 4001).astype(np.float32)
    got = oracle.lane_exp(x).astype(np.float64)
    assert np.max(np.abs(got / np.exp(x.astype(np.float64)) - 1)) < 5e-7


@pytest.mark.skipif(not Reference.available(), reason="the reference's CPU lane is not built here or lacks AVX-512 VNNI")
@pytest.mark.parametrize("name", LANE_TYPES)
def test_oracle_matches_reference_live(oracle, name):
    """fresh random inputs every type, straight against the reference's compiled CPU code"""
    from libosmos_b200 import synth
    ref = Reference()
    tid = TYPES[name]
    for cols in (256, 1024, 5120):
        rng = synth.rng_for(7, tid, cols)
        w = synth.random_tensor(tid, 6, cols, rng)
        x = rng.standard_normal((9, cols)).astype(np.float32)
        q, d = oracle.q8_round(x)
        q2, d2 = ref.q8_round(x)
        assert np.array_equal(q, q2) and np.array_equal(_bits(d), _bits(d2))
        assert np.array_equal(_bits(oracle.q8_rows(tid, w, 6, cols, q, d)), _bits(ref.q8_rows(tid, w, 6, cols, q, d)))
        assert np.array_equal(_bits(oracle.mv_rows(tid, w, 6, cols, x)), _bits(ref.mv_rows(tid, w, 6, cols, x)))


def test_mmq_oracle_integer_dots_and_bound(oracle):
    """the Q4_K x int8 restatement: its group dots are the plain integer dots, and its F32 result stays within the
    reference test's error bound of a double sum over the same quantized operands (tests/gpu/test_mmq_gpu.hip:207-233)"""
    from libosmos_b200 import synth
    rows, cols, n = 16, 512, 5
    rng = synth.rng_for(8)
    w = synth.random_tensor(12, rows, cols, rng)
    x = rng.standard_normal((n, cols)).astype(np.float32)
    idx = np.arange(n, dtype=np.int32)
    x8, dx, sx = oracle.mmq_x8_rows(x, idx, cols)
    y, ints = oracle.mmq_rows(w, rows, cols, x8, dx, sx, 0, n, want_ints=True)
    wv = oracle.dequant(12, w, rows * cols).reshape(rows, cols).astype(np.float64)
    groups = cols // 32
    blk = w.reshape(rows, cols // 256, 144)
    for t in range(n):
        xq = np.array([[x8[oracle.lib.orc_mmq_x8_at(t, c, cols)] for c in range(cols)]], dtype=np.int64)[0]
        dxt = np.array([dx[oracle.lib.orc_mmq_dx_at(t, g, groups)] for g in range(groups)], dtype=np.float64)
        xdq = xq.reshape(groups, 32) * dxt[:, None]
        want = wv @ xdq.reshape(-1)
        mag = np.abs(wv) @ np.abs(xdq.reshape(-1))
        assert np.all(np.abs(y[t] - want) <= 64 * 2.0 ** -24 * mag + 1e-30)
        # integer dots: nibbles against x8
        for r in (0, 7, 15):
            for g in (0, 5, groups - 1):
                b, gi = g // 8, g % 8
                nib = (blk[r, b, 16 + (gi // 2) * 32:16 + (gi // 2) * 32 + 32] >> (4 * (gi % 2))) & 0x0F
                assert ints[r, t, g] == int(nib.astype(np.int64) @ xq[g * 32:(g + 1) * 32])


def test_x16_layout_and_rounding_against_numpy(oracle):
    """the tiled f16 layout (kernels/mm.h:47-49 in the reference) and nearest-even rounding, against numpy's float16"""
    rng = np.random.default_rng(5)
    n, cols = 21, 48
    x = (rng.standard_normal((n, cols + 4)) * 100).astype(np.float32)
    idx = rng.integers(-1, n, size=n).astype(np.int32)
    for use_idx in (None, idx):
        got, over = oracle.x16_rows(x, n, cols, use_idx)
        assert over == 0 and got.size == 32 * cols
        for t in range(32):
            r = -1 if t >= n else (t if use_idx is None else int(use_idx[t]))
            row = x[r, :cols].astype(np.float16).view(np.uint16) if r >= 0 else np.zeros(cols, np.uint16)
            for c in range(cols):
                assert got[(t // 16) * 16 * cols + (c // 16) * 256 + (t % 16) * 16 + c % 16] == row[c]
    x[3, 5] = 65520.0  # rounds past the largest f16
    assert oracle.x16_rows(x, n, cols)[1] == 1


def test_mv_fp4_order_against_float64(oracle):
    """NVFP4's own matvec order (kernels/mv_fp4.hip in the reference): every product exact, so the result is within
    cols roundings of the float64 sum (the reference's bound, tests/gpu/test_mv_fp4_tok_gpu.hip:110)"""
    from libosmos_b200 import synth
    tid = TYPES["NVFP4"]
    for cols, lanes in ((1536, 8), (3072, 16), (6144, 32)):
        rows = 12
        w = synth.random_tensor(tid, rows, cols, synth.rng_for(41, cols))
        x = np.random.default_rng(cols).standard_normal((3, cols)).astype(np.float32)
        y = oracle.mv_fp4_rows(w, rows, cols, x, lanes)
        wv = oracle.dequant(tid, w, rows * cols).reshape(rows, cols).astype(np.float64)
        exact, mag = x.astype(np.float64) @ wv.T, np.abs(x.astype(np.float64)) @ np.abs(wv.T)
        assert np.all(np.abs(y - exact) <= cols * 6e-8 * (mag + 1e-30))
        # a token's sums do not depend on the tokens beside it
        assert np.array_equal(oracle.mv_fp4_rows(w, rows, cols, x[1:2], lanes).view(np.uint32), y[1:2].view(np.uint32))
        scaled = oracle.mv_fp4_rows(w, rows, cols, x, lanes, 0.25)
        assert np.array_equal(scaled, y * np.float32(0.25))


def _e4m3_table():
    """the values of E4M3's codes 0 .. 0x7E, from the format's definition (4 exponent bits, bias 7, 3 mantissa bits)"""
    c = np.arange(0x7F)
    e, m = c >> 3, c & 7
    return np.where(e > 0, (1 + m / 8.0) * 2.0 ** (e - 7.0), m * 2.0 ** -9)


def test_fp4_act_codes_against_nearest_value_search(oracle):
    """the oracle's NVFP4 activation quantization (kernels/mm_fp4.hip:23-104 in the reference) pinned against an
    independent statement of the same rule: the scale is the E4M3 value nearest amax / 6 / gs (a tie to the even code,
    at most 448), a code the grid point nearest v / scale (a tie to the even index)"""
    rng = np.random.default_rng(2024)
    n, cols, gs = 24, 256, 0.05
    x = (rng.standard_normal((n, cols)) * gs * 6).astype(np.float32)
    x[0, :16] = 0
    x[1, :16] *= 1e5
    x[2, 16:32] *= 1e-4
    q, sc = oracle.fp4_act(x, cols, gs)
    table = _e4m3_table()
    grid = np.array([0, .5, 1, 1.5, 2, 3, 4, 6])
    for t in range(n):
        for b in range(cols // 16):
            v = x[t, 16 * b:16 * b + 16]
            target = min(float(np.float32(np.float32(np.abs(v).max() / np.float32(6.0)) / np.float32(gs))), 448.0)
            d = np.abs(table - target)
            best = np.flatnonzero(d == d.min())
            code = best[0] if best.size == 1 else [k for k in best if k % 2 == 0][0]
            assert sc[t, b] == code, (t, b, target)
            sf = np.float32(np.float32(table[code]) * np.float32(gs))
            for j in range(16):
                a = float(np.clip(np.float32(v[j]) / sf, -6, 6)) if sf > 0 else 0.0
                dd = np.abs(grid - abs(a))
                bi = np.flatnonzero(dd == dd.min())
                i = bi[0] if bi.size == 1 else [k for k in bi if k % 2 == 0][0]
                want = (8 if a < 0 and i else 0) | i
                got = (q[t, (16 * b + j) // 2] >> (4 * (j & 1))) & 15
                assert got == want, (t, b, j, a)


def test_fp4_act_stochastic_is_unbiased_and_seeded(oracle):
    x = np.full((1, 64 * 512), 0.8, np.float32)
    x[0, ::16] = 6.0  # every group's scale is 1
    q1, _ = oracle.fp4_act(x, x.shape[1], 1.0, seed=7)
    q2, _ = oracle.fp4_act(x, x.shape[1], 1.0, seed=7)
    q3, _ = oracle.fp4_act(x, x.shape[1], 1.0, seed=8)
    assert np.array_equal(q1, q2) and not np.array_equal(q1, q3)
    codes = np.stack([q1 & 15, q1 >> 4], -1).reshape(-1)
    codes = codes[np.arange(codes.size) % 16 != 0]
    assert set(np.unique(codes)) == {1, 2}  # 0.5 or 1.0
    up = (codes == 2).mean()   # 0.8 lies 0.6 of the way from 0.5 to 1
    assert abs(up - 0.6) < 0.01


def test_fp4_mm_sums(oracle):
    """the float64 sums over the quantized operands equal the dequantized weights times the decoded activations"""
    from libosmos_b200 import synth
    tid = TYPES["NVFP4"]
    rows, cols, n = 16, 256, 5
    w = synth.random_tensor(tid, rows, cols, synth.rng_for(43))
    x = np.random.default_rng(5).standard_normal((n, cols)).astype(np.float32)
    q, sc = oracle.fp4_act(x, cols, 0.2)
    y, mag = oracle.fp4_mm(w, rows, cols, q, sc, scale=0.5)
    wv = oracle.dequant(tid, w, rows * cols).reshape(rows, cols).astype(np.float64)
    grid = np.array([0, .5, 1, 1.5, 2, 3, 4, 6])
    codes = np.stack([q & 15, q >> 4], -1).reshape(n, cols)
    xv = np.where(codes & 8, -1.0, 1.0) * grid[codes & 7] * np.repeat(_e4m3_table()[sc], 16, axis=1)
    assert np.allclose(y, 0.5 * xv @ wv.T, rtol=1e-12, atol=1e-300) and (mag >= np.abs(y)).all()
    # the quantized activations stay close to x under its scale: |x - xq gs| <= the step of the group's scale
    assert np.abs(xv * 0.2 - x).max() < 0.2 * np.abs(x).max()


def test_x16_attn_against_numpy(oracle):
    """mm_x16_attn's restatement against the same steps taken with numpy: rotate, round 32 at a time, tile"""
    n, heads, head_dim, rope_dim = 6, 2, 64, 32
    cols = heads * head_dim
    rng = np.random.default_rng(9)
    x = (rng.standard_normal((n, cols)) * 2).astype(np.float32)
    freqs = (100.0 ** (-np.arange(rope_dim // 2) / (rope_dim // 2))).astype(np.float32)
    pos = rng.integers(0, 50, n).astype(np.int32)
    got, over = oracle.x16_attn(x, n, cols, head_dim, rope_dim, freqs, pos)
    assert over == 0
    v = x.copy().reshape(n, heads, head_dim)
    ang = pos[:, None].astype(np.float32) * freqs[None, :]
    cs, sn = np.cos(ang.astype(np.float64)), np.sin(ang.astype(np.float64))
    a, b = v[:, :, head_dim - rope_dim::2].astype(np.float64), v[:, :, head_dim - rope_dim + 1::2].astype(np.float64)
    v[:, :, head_dim - rope_dim::2] = a * cs[:, None, :] + b * sn[:, None, :]
    v[:, :, head_dim - rope_dim + 1::2] = b * cs[:, None, :] - a * sn[:, None, :]
    want = oracle.fp8_round(v.reshape(-1))[0].reshape(n, cols)
    tiled = got.view(np.float16).astype(np.float32)
    back = np.zeros((16, cols), np.float32)
    for t in range(16):
        for c in range(cols):
            back[t, c] = tiled[(t // 16) * 16 * cols + (c // 16) * 256 + (t % 16) * 16 + c % 16]
    assert not back[n:].any()
    # the unrotated part is exactly the FP8 rounding of x; the rotated part agrees with the float64 rotation to one
    # E4M3 step (the F32 rotation rounds differently in the last place)
    keep = (np.arange(cols) % head_dim) < head_dim - rope_dim
    ref16 = want.astype(np.float16).astype(np.float32)
    assert np.array_equal(back[:n][:, keep], ref16[:, keep])
    assert (np.abs(back[:n] - ref16) <= 0.126 * np.maximum(np.abs(ref16), 2.0 ** -6)).all()
    assert (back[:n] != ref16).mean() < 0.02
