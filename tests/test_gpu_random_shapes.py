"""GPU parity over seeded random shapes: every fast kernel (the per-warp rings, the thread-a-row kernel, the
tile-staging kernel) against the generic kernel of the same entry point, bit for bit - the fixed-shape tests pin the
kernels to the oracle, this one walks the shape space between them (row counts that leave partial tiles and slots,
every lane width, 1..8 tokens, entries of 0..8 tokens)."""
import numpy as np
import pytest
import torch

from libosmos_b200 import synth
from oracle.oracle import LANE_TYPES, TYPES

pytestmark = pytest.mark.gpu
COLS = [256, 512, 768, 1024, 1536, 2048, 2304, 4096, 5120, 7168, 8192]


def _same(a, b):
    return np.array_equal(a.view(np.uint32), b.view(np.uint32))


@pytest.mark.parametrize("seed", [11, 12, 13])
def test_dense_entry_points(lib, dev, seed):
    rng = np.random.default_rng(seed)
    names = sorted(TYPES)
    try:
        for it in range(40):
            name = names[int(rng.integers(len(names)))]
            tid = TYPES[name]
            cols, rows, ntok = int(rng.choice(COLS)), int(rng.integers(1, 300)), int(rng.integers(1, 9))
            w = torch.from_numpy(synth.random_tensor(tid, rows, cols, synth.rng_for(seed, it, tid))).to(dev)
            x = torch.randn(ntok, cols, device=dev, generator=torch.Generator(device=dev).manual_seed(seed * 1000 + it))
            got = []
            for mode in (1, 0):
                lib.mv_set_staged(mode)
                y = torch.full((ntok, rows), float("nan"), device=dev)
                assert lib.mv_run(tid, w.data_ptr(), rows, cols, x.data_ptr(), ntok, y.data_ptr(), None)
                torch.cuda.synchronize()
                got.append(y.cpu().numpy())
            assert _same(got[0], got[1]), ("mv_run", name, rows, cols, ntok)
            if name in LANE_TYPES or name in ("Q4_0", "Q8_0"):
                q = torch.zeros(ntok, cols, dtype=torch.int8, device=dev)
                d = torch.zeros(ntok, cols // 32, device=dev)
                assert lib.q8_round(x.data_ptr(), ntok, cols, cols, q.data_ptr(), d.data_ptr(), None)
                got = []
                for mode in (1, 2, 0):
                    lib.q8_set_staged(mode)
                    y = torch.full((ntok, rows), float("nan"), device=dev)
                    assert lib.q8_run(tid, w.data_ptr(), rows, cols, q.data_ptr(), d.data_ptr(), ntok, y.data_ptr(), rows, None)
                    torch.cuda.synchronize()
                    got.append(y.cpu().numpy())
                assert _same(got[0], got[2]) and _same(got[1], got[2]), ("q8_run", name, rows, cols, ntok)
    finally:
        lib.mv_set_staged(1), lib.q8_set_staged(1)
    assert lib.q8_status() == 0 and lib.mv_status() == 0


@pytest.mark.parametrize("seed", [21, 22])
def test_grouped_entry_points(lib, dev, seed):
    rng = np.random.default_rng(seed)
    try:
        for it in range(24):
            name = LANE_TYPES[int(rng.integers(len(LANE_TYPES)))]
            tid = TYPES[name]
            cols, rows = int(rng.choice(COLS)), int(rng.choice([8, 16, 24, 32, 64, 96, 128]))
            n_mat, n_tok = int(rng.integers(1, 6)), 7
            mats = [torch.from_numpy(synth.random_tensor(tid, rows, cols, synth.rng_for(seed, it, tid, m))).to(dev)
                    for m in range(2 * n_mat)]
            cnt = rng.integers(0, 9, size=n_mat).astype(np.int32)
            xrow = np.concatenate([[0], np.cumsum(cnt)[:-1]]).astype(np.int32)
            total = int(cnt.sum()) + 8
            x = torch.randn(n_tok, cols, device=dev, generator=torch.Generator(device=dev).manual_seed(seed * 1000 + it))
            q = torch.zeros(n_tok, cols, dtype=torch.int8, device=dev)
            d = torch.zeros(n_tok, cols // 32, device=dev)
            assert lib.q8_round(x.data_ptr(), n_tok, cols, cols, q.data_ptr(), d.data_ptr(), None)
            xin = torch.from_numpy(rng.integers(0, n_tok, size=total).astype(np.int32)).to(dev)
            win = torch.from_numpy(rng.permutation(total).astype(np.int32)).to(dev)
            scale = torch.from_numpy(rng.uniform(0.05, 1.0, size=total).astype(np.float32)).to(dev)
            tg = torch.tensor([m.data_ptr() for m in mats[:n_mat]], dtype=torch.int64, device=dev)
            tu = torch.tensor([m.data_ptr() for m in mats[n_mat:]], dtype=torch.int64, device=dev)
            cd, xd = torch.from_numpy(cnt).to(dev), torch.from_numpy(xrow).to(dev)
            got = []
            for mode in (1, 2, 0):
                lib.q8_set_staged(mode)
                yg = torch.full((total, rows), -9.0, device=dev)
                h = torch.full((total, rows), -9.0, device=dev)
                assert lib.q8_group_tok(tid, tg.data_ptr(), cd.data_ptr(), xd.data_ptr(), xin.data_ptr(), n_mat, 8, rows, cols,
                                        q.data_ptr(), d.data_ptr(), yg.data_ptr(), rows, None)
                assert lib.q8_gate_up(tid, tg.data_ptr(), tu.data_ptr(), cd.data_ptr(), xd.data_ptr(), xin.data_ptr(),
                                      win.data_ptr(), n_mat, 8, rows, cols, q.data_ptr(), d.data_ptr(), scale.data_ptr(), 2.0,
                                      h.data_ptr(), rows, None)
                torch.cuda.synchronize()
                got.append((yg.cpu().numpy(), h.cpu().numpy()))
            for k in (0, 1):
                assert _same(got[0][k], got[2][k]) and _same(got[1][k], got[2][k]), (name, rows, cols, list(cnt), k)
    finally:
        lib.q8_set_staged(1)
    assert lib.q8_status() == 0
