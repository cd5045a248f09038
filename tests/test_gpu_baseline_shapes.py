"""Parity at the exact shapes of the benchmark configurations (the kernels the benchmark times, at the sizes it times
them), each against the CPU checker:
  config 1 - Q4_0 6144 x 2048, one token: q8_run after q8_round and after q8_0_round, and mv_run, every row;
  config 2 - Q4_K 4096 x 4096 over 512 tokens: mmq_group bit-equal and mm_run within the reference test's bound, on 256
             sampled rows x all tokens;
  config 3 - the IQ3_XXS layer, all 64 tokens of step 0, against the reference's own cpu_lane_submit where its library
             is present (else the scalar restatement) - the counterpart of the reference's tests/gpu/test_cpu_lane_gpu.hip
             (CPU and GPU bit-equal at model shapes).
"""
import numpy as np
import pytest
import torch

import bench
from helpers import ptr, same_bits, sync, to_dev
from libosmos_b200 import ep, synth, workloads

pytestmark = pytest.mark.gpu


def test_config1_q4_0_decode_matvec(lib, dev, oracle):
    cfg = workloads.MV_Q4_0
    tid, rows, cols = synth.TYPE_ID[cfg["type"]], cfg["rows"], cfg["cols"]
    rng = synth.rng_for(401)
    w = synth.random_tensor(tid, rows, cols, rng, cfg["sigma"])
    x = rng.standard_normal((1, cols)).astype(np.float32)
    wd, xd = to_dev(w, dev), to_dev(x, dev)
    q = torch.zeros((1, cols), dtype=torch.int8, device=dev)
    d = torch.zeros((1, cols // 32), dtype=torch.float32, device=dev)
    y = torch.empty((1, rows), dtype=torch.float32, device=dev)
    for ggml, rounder in ((False, lib.q8_round), (True, lib.q8_0_round)):
        assert rounder(ptr(xd), 1, cols, cols, ptr(q), ptr(d), None)
        y.fill_(-3.0)
        assert lib.q8_run(tid, ptr(wd), rows, cols, ptr(q), ptr(d), 1, ptr(y), rows, None)
        sync()
        qh, dh = oracle.q8_round(x, ggml_q8_0=ggml)
        assert np.array_equal(q.cpu().numpy(), qh) and same_bits(d.cpu().numpy(), dh)
        assert same_bits(y.cpu().numpy(), oracle.q8_rows(tid, w, rows, cols, qh, dh))
    y.fill_(-3.0)
    assert lib.mv_run(tid, ptr(wd), rows, cols, ptr(xd), 1, ptr(y), None)
    sync()
    assert same_bits(y.cpu().numpy(), oracle.mv_rows(tid, w, rows, cols, x))
    assert lib.q8_status() == 0 and lib.mv_status() == 0


def test_config2_q4_k_prefill(lib, dev, oracle):
    cfg = workloads.MM_Q4_K
    tid, rows, cols, tokens = synth.TYPE_ID[cfg["type"]], cfg["rows"], cfg["cols"], cfg["tokens"]
    rng = synth.rng_for(402)
    w = synth.random_tensor(tid, rows, cols, rng, cfg["sigma"])
    x = rng.standard_normal((tokens, cols)).astype(np.float32)
    pick = np.sort(rng.choice(rows, 256, replace=False))
    rb = w.size // rows
    wsel = np.ascontiguousarray(w.reshape(rows, rb)[pick]).reshape(-1)
    wd, xd = to_dev(w, dev), to_dev(x, dev)
    y = torch.zeros((tokens, rows), dtype=torch.float32, device=dev)
    # the int8 product: bit-equal
    idx = torch.arange(tokens, dtype=torch.int32, device=dev)
    x8 = torch.zeros(tokens * cols, dtype=torch.int8, device=dev)
    dx = torch.zeros(tokens * cols // 32, dtype=torch.float32, device=dev)
    sx = torch.zeros_like(dx)
    assert lib.mmq_x8_rows(ptr(xd), cols, ptr(idx), tokens, cols, ptr(x8), ptr(dx), ptr(sx), None)
    tab = torch.tensor([wd.data_ptr()], dtype=torch.int64, device=dev)
    cnt = torch.tensor([tokens], dtype=torch.int32, device=dev)
    zero = torch.zeros(1, dtype=torch.int32, device=dev)
    assert lib.mmq_group(tid, ptr(tab), ptr(cnt), 1, tokens, rows, cols, ptr(x8), ptr(dx), ptr(sx), ptr(zero), ptr(y), ptr(zero), rows, None)
    sync()
    hx8, hdx, hsx = oracle.mmq_x8_rows(x, np.arange(tokens, dtype=np.int32), cols)
    assert np.array_equal(x8.cpu().numpy(), hx8) and same_bits(dx.cpu().numpy(), hdx) and same_bits(sx.cpu().numpy(), hsx)
    want = oracle.mmq_rows(wsel, len(pick), cols, hx8, hdx, hsx, 0, tokens)
    assert same_bits(y.cpu().numpy()[:, pick], want)
    # the f16 product: within the reference test's bound of a float64 sum over the f16-rounded operands
    x16 = torch.zeros(tokens * cols, dtype=torch.float16, device=dev)
    flag = torch.zeros(1, dtype=torch.int32, device=dev)
    y.zero_()
    assert lib.mm_x16(ptr(xd), cols, tokens, cols, ptr(x16), ptr(flag), None)
    assert lib.mm_run(tid, ptr(wd), rows, cols, ptr(x16), tokens, ptr(y), rows, None)
    sync()
    wf = oracle.dequant(tid, wsel, len(pick) * cols).reshape(len(pick), cols)
    w16, h16 = wf.astype(np.float16).astype(np.float64), x.astype(np.float16).astype(np.float64)
    ref = h16 @ w16.T
    bound = (cols / 16 + 20) * 2.0 ** -24 * (np.abs(h16) @ np.abs(w16).T)
    assert (np.abs(y.cpu().numpy()[:, pick].astype(np.float64) - ref) <= bound).all()
    assert int(flag.item()) == 0 and lib.mm_status() == 0 and lib.mmq_status() == 0


def test_config3_moe_layer_all_tokens(lib, dev):
    cfg = workloads.MOE_IQ3
    host = workloads.moe_layer_host(cfg)
    layer = ep.EpMoeLane(lib, cfg, dev, 0, 1, host_tensors=host)
    x, logits = workloads.moe_inputs_host(cfg, 0)
    out = torch.empty((cfg["n_tok"], cfg["dim"]), dtype=torch.float32, device=dev)
    layer.step(to_dev(x, dev), to_dev(logits, dev), out, 0, torch.cuda.current_stream().cuda_stream)
    sync()
    ids, wts = layer.last_picks()
    want_ids, want_wts = workloads.softmax_topk(logits, cfg["k"])
    assert np.array_equal(ids, want_ids) and np.allclose(wts, want_wts, rtol=1e-5, atol=0)
    arm = bench.CpuArm(cfg, host)  # the reference's CPU lane where its library is present
    assert same_bits(out.cpu().numpy(), arm.layer(x, ids, wts))
    assert lib.ep_wait_status() == 0 and lib.q8_status() == 0
    layer.close()


@pytest.mark.parametrize("world", [2, 8])
def test_config2_rows_split_among_ranks_have_the_whole_products_bits(lib, dev, world):
    """the prefill product with its rows split among `world` ranks (each emulated here in turn): the slices side by side
    are the whole product bit for bit, whatever block width a slice's smaller grid makes the kernel choose"""
    from libosmos_b200 import shard
    cfg = workloads.MM_Q4_K
    tid, rows, cols, tokens = synth.TYPE_ID[cfg["type"]], cfg["rows"], cfg["cols"], cfg["tokens"]
    w = synth.random_tensor(tid, rows, cols, synth.rng_for(402), cfg["sigma"])
    x = torch.from_numpy(synth.rng_for(403).standard_normal((tokens, cols)).astype(np.float32)).to(dev)
    whole = shard.DenseRows(lib, dev, tid, rows, cols, w, 0, 1, max_tok=tokens)
    want = torch.zeros((tokens, rows), dtype=torch.float32, device=dev)
    whole.step(x, tokens, want, 0, None)
    for rank in range(world):
        part = shard.DenseRows(lib, dev, tid, rows, cols, w, rank, world, max_tok=tokens)
        y = torch.full((tokens, part.rows), -3.0, dtype=torch.float32, device=dev)
        part.step(x, tokens, y, 0, None)
        sync()
        assert np.array_equal(y.cpu().numpy().view(np.uint32), want[:, part.r0:part.r1].cpu().numpy().view(np.uint32)), rank
    assert lib.mmq_status() == 0
