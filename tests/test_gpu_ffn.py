"""The host drivers of a layer's feed-forward parts (include/osmos_b200/ffn.h), through the C ABI:
lane_ffn_f32 bit-equal to the CPU oracle (the F32 matvec's order, the lane's activation, the ordered sum); shared_ffn and
q4x_moe, whose products run on the f16 tensor cores, stage by stage within the reference test's bound of a float64 sum
over the f16-rounded operands ((cols / 16 + 20) 2^-24 sum |w16 x16|, tests/gpu/test_mm_gpu.hip:328-343)."""
import numpy as np
import pytest
import torch

from helpers import ptr, same_bits, sync, to_dev
from libosmos_b200 import api, synth, workloads

pytestmark = pytest.mark.gpu


def _scratch(lib, dev, bytes_fn, bind_fn, layer, max_tok, struct):
    n = bytes_fn(layer, max_tok)
    assert n
    mem = torch.zeros(n + 256, dtype=torch.uint8, device=dev)
    base = (mem.data_ptr() + 255) // 256 * 256
    s = struct()
    assert bind_fn(layer, max_tok, base, n, s)
    return s, mem


def _f64_bound(x, w, cols):
    x16, w16 = x.astype(np.float16).astype(np.float64), w.astype(np.float16).astype(np.float64)
    return x16 @ w16.T, (cols / 16 + 20) * 2.0 ** -24 * (np.abs(x16) @ np.abs(w16).T)


@pytest.mark.parametrize("name,dim,ff", [("MXFP4", 1024, 512), ("Q4_K", 512, 256), ("IQ3_XXS", 512, 512)])
def test_lane_ffn_f32(lib, dev, oracle, name, dim, ff):
    tid = synth.TYPE_ID[name]
    cfg = dict(name="f32lane", type=name, n_exp=12, k=3, n_tok=9, dim=dim, ff=ff, sigma=0.01, lim=7.0)
    host = workloads.moe_layer_host(cfg)
    per = workloads.moe_expert_bytes(cfg)
    dw = [to_dev(h, dev) for h in host]
    L = api.LaneLayer(tid, tid, dim, ff, cfg["n_exp"], cfg["k"], cfg["lim"], api.LaneExperts())
    for j in range(3):
        L.experts.base[j], L.experts.bytes[j] = dw[j].data_ptr(), per[j]
    s, keep = _scratch(lib, dev, lib.lane_f32_scratch_bytes, lib.lane_f32_scratch_bind, L, cfg["n_tok"], api.LaneScratchF32)
    x, logits = workloads.moe_inputs_host(cfg, 3)
    ids, wts = workloads.softmax_topk(logits, cfg["k"])
    add = synth.rng_for(61).standard_normal((cfg["n_tok"], dim)).astype(np.float32)
    out = torch.empty((cfg["n_tok"], dim), dtype=torch.float32, device=dev)
    for with_add in (False, True):
        assert lib.lane_ffn_f32(L, s, ptr(to_dev(x, dev)), ptr(to_dev(ids, dev)), ptr(to_dev(wts, dev)), cfg["n_tok"],
                                ptr(to_dev(add, dev)) if with_add else None, ptr(out), None)
        sync()
        want = np.zeros((cfg["n_tok"], dim), np.float32)
        for t in range(cfg["n_tok"]):
            acc = np.zeros(dim, np.float32)
            for j in np.argsort(ids[t], kind="stable"):
                e = int(ids[t, j])
                p = [host[m][e * per[m]:(e + 1) * per[m]] for m in range(3)]
                g = oracle.mv_rows(tid, p[0], ff, dim, x[t:t + 1])
                u = oracle.mv_rows(tid, p[1], ff, dim, x[t:t + 1])
                h = oracle.swiglu_lane(g, u, cfg["lim"], wts[t, j:j + 1])
                acc = (acc + oracle.mv_rows(tid, p[2], dim, ff, h)[0]).astype(np.float32)
            want[t] = (acc + add[t]).astype(np.float32) if with_add else acc
        assert same_bits(out.cpu().numpy(), want)
    assert lib.mv_status() == 0
    assert not lib.lane_ffn_f32(L, s, ptr(out), ptr(out), ptr(out), cfg["n_tok"] + 1, None, ptr(out), None)
    bad = api.LaneLayer.from_buffer_copy(L)
    bad.type_gu = 0
    assert not lib.lane_ffn_f32(bad, s, ptr(out), ptr(out), ptr(out), 1, None, ptr(out), None)


@pytest.mark.parametrize("name,n", [("Q4_K", 5), ("Q4_K", 40), ("MXFP4", 17)])
def test_shared_ffn(lib, dev, oracle, name, n):
    tid = synth.TYPE_ID[name]
    dim, ff, lim = 512, 256, 5.0
    rng = synth.rng_for(62, tid, n)
    w = [synth.random_tensor(tid, r, c, rng, 0.02) for r, c in ((ff, dim), (ff, dim), (dim, ff))]
    dw = [to_dev(a, dev) for a in w]
    e = api.SharedExpert(tid, tid, dim, ff, lim, dw[0].data_ptr(), dw[1].data_ptr(), dw[2].data_ptr())
    s, keep = _scratch(lib, dev, lib.shared_scratch_bytes, lib.shared_scratch_bind, e, 64, api.SharedScratch)
    x = rng.standard_normal((n, dim)).astype(np.float32)
    y = torch.empty((n, dim), dtype=torch.float32, device=dev)
    assert lib.shared_ffn(e, s, ptr(to_dev(x, dev)), n, ptr(y), None)
    sync()
    wf = [oracle.dequant(tid, a, r * c).reshape(r, c) for a, (r, c) in zip(w, ((ff, dim), (ff, dim), (dim, ff)))]
    g = torch.empty((n, ff), dtype=torch.float32, device=dev)
    u, h = torch.empty_like(g), torch.empty_like(g)
    for dst, src in ((g, s.g), (u, s.u), (h, s.h)):  # the stages, out of the caller's scratch
        assert lib.ops_gather_rows(ptr(dst), src, ptr(to_dev(np.arange(n, dtype=np.int32), dev)), n, ff, None)
    sync()
    gh, uh, hh = g.cpu().numpy(), u.cpu().numpy(), h.cpu().numpy()
    matvec = n <= 8  # a decode step's few tokens go through the F32 matvec: the oracle's bits
    for got, wmat, raw in ((gh, wf[0], w[0]), (uh, wf[1], w[1])):
        if matvec:
            assert same_bits(got, oracle.mv_rows(tid, raw, ff, dim, x))
        else:
            ref, bound = _f64_bound(x, wmat, dim)
            assert (np.abs(got - ref) <= bound).all()
    gv, uv = np.minimum(gh.astype(np.float64), lim), np.clip(uh.astype(np.float64), -lim, lim)
    assert np.allclose(hh, gv / (1 + np.exp(-gv)) * uv, rtol=3e-6, atol=1e-30)
    if matvec:
        assert same_bits(y.cpu().numpy(), oracle.mv_rows(tid, w[2], dim, ff, hh))
    else:
        ref, bound = _f64_bound(hh, wf[2], ff)
        assert (np.abs(y.cpu().numpy() - ref) <= bound).all()
    assert lib.mm_status() == 0
    assert not lib.shared_ffn(e, s, ptr(y), 65, ptr(y), None)


@pytest.mark.parametrize("name,n_tok", [("MXFP4", 40), ("Q4_K", 300)])
def test_q4x_moe(lib, dev, oracle, name, n_tok):
    tid = synth.TYPE_ID[name]
    # (block scales small enough that the activations stay inside f16's range, as a model's do)
    cfg = dict(name="q4xmoe", type=name, n_exp=8, k=2, n_tok=n_tok, dim=512, ff=256, sigma=0.02 if name == "MXFP4" else 0.0015, lim=1e30)
    dim, ff, k, n_exp = cfg["dim"], cfg["ff"], cfg["k"], cfg["n_exp"]
    host = workloads.moe_layer_host(cfg)
    per = workloads.moe_expert_bytes(cfg)
    dw = [to_dev(hh, dev) for hh in host]
    L = api.Q4xMoeLayer()
    L.dim, L.ff, L.n_exp, L.k = dim, ff, n_exp, k
    for j in range(3):
        L.type[j], L.base[j], L.bytes[j] = tid, dw[j].data_ptr(), per[j]
    s, keep = _scratch(lib, dev, lib.q4x_moe_scratch_bytes, lib.q4x_moe_scratch_bind, L, n_tok, api.Q4xMoeScratch)
    x, logits = workloads.moe_inputs_host(cfg, 4)
    rng = synth.rng_for(63)
    shared = rng.standard_normal((n_tok, dim)).astype(np.float32)
    slog = rng.standard_normal(n_tok).astype(np.float32)
    out = torch.empty((n_tok, dim), dtype=torch.float32, device=dev)
    assert lib.q4x_moe(L, s, ptr(to_dev(x, dev)), ptr(to_dev(logits, dev)), ptr(to_dev(shared, dev)), ptr(to_dev(slog, dev)),
                       n_tok, ptr(out), None)
    sync()
    picks = n_tok * k

    def fetch(p, rows, cols):
        dst = torch.empty((rows, cols), dtype=torch.float32, device=dev)
        assert lib.ops_gather_rows(ptr(dst), p, ptr(to_dev(np.arange(rows, dtype=np.int32), dev)), rows, cols, None)
        sync()
        return dst.cpu().numpy()

    ids_w = fetch(s.w, 1, picks)[0]
    ids = np.frombuffer(fetch(s.ids, 1, picks).tobytes(), np.int32)
    where = np.frombuffer(fetch(s.where, 1, picks).tobytes(), np.int32)
    want_ids, want_w = workloads.softmax_topk(logits, k)
    assert np.array_equal(ids.reshape(n_tok, k), want_ids) and np.allclose(ids_w.reshape(n_tok, k), want_w, rtol=1e-5)
    # places: the picks stably sorted by expert
    assert np.array_equal(np.argsort(np.argsort(ids, kind="stable"), kind="stable"), where)
    ga, up, y = fetch(s.ga, picks, ff), fetch(s.up, picks, ff), fetch(s.y, picks, dim)
    wf = [[oracle.dequant(tid, host[m][e * per[m]:(e + 1) * per[m]], per_rows * per_cols).reshape(per_rows, per_cols)
           for e in range(n_exp)] for m, (per_rows, per_cols) in enumerate(((ff, dim), (ff, dim), (dim, ff)))]
    for i in range(picks):
        e, t, r = int(ids[i]), i // k, int(where[i])
        for got, wmat in ((ga[r], wf[0][e]), (up[r], wf[1][e])):
            ref, bound = _f64_bound(x[t:t + 1], wmat, dim)
            assert (np.abs(got - ref[0]) <= bound[0]).all()
        g64 = ga[r].astype(np.float64)
        h = (g64 / (1 + np.exp(-g64)) * up[r]).astype(np.float32)
        ref, bound = _f64_bound(h[None], wf[2][e], ff)
        # (the activation's last bit may differ from the device's before it is rounded to f16: one f16 step in a value
        # moves a sum by at most 2^-11 |h w|)
        slack = 2.0 ** -10 * (np.abs(h.astype(np.float64))[None] @ np.abs(wf[2][e].astype(np.float64)).T)
        assert (np.abs(y[r] - ref[0]) <= bound[0] + slack[0]).all()
    gate = 1 / (1 + np.exp(-slog.astype(np.float64)))
    want, mag = np.zeros((n_tok, dim)), np.zeros((n_tok, dim))
    for i in range(picks):
        want[i // k] += y[where[i]].astype(np.float64) * ids_w[i]
        mag[i // k] += np.abs(y[where[i]].astype(np.float64) * ids_w[i])
    want += shared * gate[:, None]
    mag += np.abs(shared * gate[:, None])
    # (F32 products and sums in pick order: a few roundings of the terms' magnitudes, whatever cancels)
    assert (np.abs(out.cpu().numpy() - want) <= 1e-6 * mag + 1e-30).all()
    assert lib.mm_status() == 0 and np.frombuffer(fetch(s.overflow, 1, 1).tobytes(), np.int32)[0] == 0
    assert not lib.q4x_moe(L, s, ptr(out), ptr(out), ptr(out), ptr(out), n_tok + 1, ptr(out), None)
