"""The fused expert-parallel step on one GPU.

One rank: `ep_layer_step` is the single-GPU layer (every flag is already there when its wait runs) and must have the
bits of the unfused layer (q4x_route + lane_ffn); the same step captured in a CUDA graph and replayed must repeat them.

Two and four ranks EMULATED on the one GPU: each rank has its own plan, step counter, scratch and exchange buffer, all
on this device, and each plan's `peer` table names all of them. The ranks' stages are queued on one stream in an order in
which every producer comes before its consumers (all ranks' stage 1, then all ranks' stage 2, ...), so a wait's flag is
always set when the waiting kernel runs - no kernel ever spins on a kernel of the same GPU. This checks what one rank
cannot: the token-major dispatch placement by home rank, the row homes, the per-sender flags and the step parity, with
the outputs' bits equal to the single-GPU layer. (Two real GPUs: tests/test_gpu_ep_peer.py.)
"""
import numpy as np
import pytest
import torch

from libosmos_b200 import api, ep, runner, workloads

pytestmark = pytest.mark.gpu

# (the fused step runs on the warp-ring / thread-a-row kernels only: rows of 512 columns or more)
SMALL = dict(name="moe_small", type="IQ3_XXS", n_exp=16, k=4, n_tok=24, dim=512, ff=512, sigma=0.005, lim=1.0e30)
WIDE = dict(name="moe_wide", type="IQ1_M", n_exp=32, k=6, n_tok=16, dim=2048, ff=1024, sigma=0.005, lim=7.0)


def _bits(t):
    return t.cpu().numpy().view(np.uint32)


@pytest.mark.parametrize("cfg", [SMALL, WIDE], ids=["small", "wide"])
@pytest.mark.parametrize("transport", ["peer", "nccl"])
def test_one_rank_step_has_the_unfused_layers_bits(lib, dev, cfg, transport):
    host = workloads.moe_layer_host(cfg)
    plain = runner.MoeLane(lib, cfg, dev, host_tensors=host)
    layer = ep.EpMoeLane(lib, cfg, dev, 0, 1, host_tensors=host, transport=transport)
    stream = torch.cuda.current_stream().cuda_stream
    want = torch.empty((cfg["n_tok"], cfg["dim"]), dtype=torch.float32, device=dev)
    got = torch.empty_like(want)
    for step in range(3):  # both halves of the exchange buffers, and a reuse
        x, logits = workloads.moe_inputs_host(cfg, step)
        xd, ld = torch.from_numpy(x).to(dev), torch.from_numpy(logits).to(dev)
        plain.step(xd, ld, want, cfg["n_tok"], 0, stream)
        got.fill_(-7.0)
        layer.step(xd, ld, got, 0, stream)
        torch.cuda.synchronize()
        assert np.array_equal(_bits(got), _bits(want))
        ids, wts = layer.last_picks()
        assert np.array_equal(ids.reshape(-1), plain.ids.cpu().numpy()) and np.array_equal(wts.reshape(-1), plain.wts.cpu().numpy())
    assert lib.ep_wait_status() == 0 and lib.q8_status() == 0
    layer.close()


def test_one_rank_step_with_add_and_in_a_graph(lib, dev):
    cfg = SMALL
    host = workloads.moe_layer_host(cfg)
    layer = ep.EpMoeLane(lib, cfg, dev, 0, 1, host_tensors=host)
    x, logits = workloads.moe_inputs_host(cfg, 5)
    xd, ld = torch.from_numpy(x).to(dev), torch.from_numpy(logits).to(dev)
    add = torch.randn((cfg["n_tok"], cfg["dim"]), device=dev)
    base = torch.empty_like(add)
    out = torch.empty_like(add)
    stream = torch.cuda.current_stream().cuda_stream
    layer.step(xd, ld, base, 0, stream)
    layer.step(xd, ld, out, 0, stream, add=add)
    torch.cuda.synchronize()
    assert np.array_equal(_bits(out), _bits(base + add))  # one rounded addition a value, after the rows' sum
    # the step's launches do not change from step to step (the step number lives on the device): captured once,
    # replayed on either parity
    side, g = torch.cuda.Stream(), torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        layer.step(xd, ld, out, 0, side.cuda_stream)
    for _ in range(3):
        out.fill_(3.0)
        g.replay()
        torch.cuda.synchronize()
        assert np.array_equal(_bits(out), _bits(base))
    assert lib.ep_wait_status() == 0 and lib.q8_status() == 0
    layer.close()


@pytest.mark.parametrize("world", [2, 4])
def test_emulated_ranks_have_the_single_gpu_bits(lib, dev, world):
    cfg = SMALL
    n_tok, k, dim = cfg["n_tok"], cfg["k"], cfg["dim"]
    T = n_tok // world
    host = workloads.moe_layer_host(cfg)
    plain = runner.MoeLane(lib, cfg, dev, host_tensors=host)
    lay = api.EpLayout()
    assert lib.ep_layout(world, n_tok, k, dim, lay)
    bufs = [torch.zeros(lay.bytes + 256, dtype=torch.uint8, device=dev) for _ in range(world)]
    base = [(b.data_ptr() + 255) // 256 * 256 for b in bufs]
    ranks = []
    for r in range(world):
        e0, e1 = ep.expert_range(r, world, cfg["n_exp"])
        local = runner.MoeLane(lib, cfg, dev, max_tok=n_tok, host_tensors=host, expert_range=(e0, e1))
        sync = torch.zeros(4, dtype=torch.int32, device=dev)
        rows = torch.zeros(2 * n_tok * k, dtype=torch.int64, device=dev)
        p = api.EpPlan()
        p.rank, p.n_ranks, p.n_tok, p.expert0, p.expert1, p.lay = r, world, n_tok, e0, e1, lay
        for q in range(world):
            p.peer[q] = base[q]
        p.sync, p.rows, p.layer, p.scratch = sync.data_ptr(), rows.data_ptr(), local.layers[0], local.scratch
        assert lib.ep_plan_ok(p)
        ranks.append((p, local, sync, rows))
    stream = torch.cuda.current_stream().cuda_stream
    want = torch.empty((n_tok, dim), dtype=torch.float32, device=dev)
    got = torch.empty_like(want)
    for step in range(3):
        x, logits = workloads.moe_inputs_host(cfg, 10 + step)
        xd, ld = torch.from_numpy(x).to(dev), torch.from_numpy(logits).to(dev)
        plain.step(xd, ld, want, n_tok, 0, stream)
        got.fill_(-7.0)
        torch.cuda.synchronize()
        # stage by stage over all ranks: every producer is queued before its consumers
        for p, _, _, _ in ranks:
            t0 = p.rank * T
            assert lib.ep_route_round_push(p, xd[t0:t0 + T].data_ptr(), ld[t0:t0 + T].data_ptr(), stream)
        for p, _, _, _ in ranks:
            assert lib.ep_lane_tables(p, stream)
        for p, _, _, _ in ranks:
            assert lib.ep_gate_up(p, stream)
        for p, local, _, _ in ranks:
            s, L = p.scratch, p.layer
            assert lib.q8_round(s.hh, n_tok * k, L.ff, L.ff, s.hq, s.hqd, stream)
        for p, _, _, _ in ranks:
            assert lib.ep_down_push(p, stream)
        for p, _, _, _ in ranks:
            t0 = p.rank * T
            assert lib.ep_combine_wait(p, None, got[t0:t0 + T].data_ptr(), stream)
        torch.cuda.synchronize()
        assert lib.ep_wait_status() == 0 and lib.q8_status() == 0
        assert np.array_equal(_bits(got), _bits(want)), "step %d" % step
        for p, _, sync, _ in ranks:
            assert int(sync[0].item()) == step + 1 and int(sync[1].item()) == 0 and int(sync[2].item()) == 0


def test_plan_refusals(lib, dev):
    cfg = SMALL
    layer = ep.EpMoeLane(lib, cfg, dev, 0, 1)
    p = layer.plans[0]
    x = torch.zeros((cfg["n_tok"], cfg["dim"]), device=dev)
    l = torch.zeros((cfg["n_tok"], cfg["n_exp"]), device=dev)
    assert not lib.ep_layer_step(p, None, l.data_ptr(), None, x.data_ptr(), None)
    assert not lib.ep_layer_step(p, x.data_ptr(), l.data_ptr(), None, x.data_ptr() + 4, None)  # out not 16-byte aligned
    bad = api.EpPlan.from_buffer_copy(p)
    bad.n_tok = cfg["n_tok"] + 1
    assert not lib.ep_plan_ok(bad)
    bad = api.EpPlan.from_buffer_copy(p)
    bad.expert1 = cfg["n_exp"] + 1
    assert not lib.ep_plan_ok(bad)
    bad = api.EpPlan.from_buffer_copy(p)
    bad.layer.type_gu = 12  # Q4_K is not a lane type
    assert not lib.ep_plan_ok(bad)
    lay = api.EpLayout()
    assert not lib.ep_layout(3, 64, 10, 2048, lay) and not lib.ep_layout(17, 68, 10, 2048, lay) and not lib.ep_layout(2, 64, 33, 2048, lay)
    layer.close()


@pytest.mark.parametrize("n_tok,k", [(1, 8), (2, 3), (1, 1)])
def test_one_rank_step_of_very_few_tokens(lib, dev, n_tok, k):
    """a decode step of one or two tokens: fewer picks than experts, entries of one token, a single block in the
    per-token kernels"""
    cfg = dict(name="moe_tiny", type="IQ1_M", n_exp=32, k=k, n_tok=n_tok, dim=4096, ff=1024, sigma=0.01, lim=10.0,
               router="sqrt_softplus", route_scale=2.5)
    host = workloads.moe_layer_host(cfg)
    layer = ep.EpMoeLane(lib, cfg, dev, 0, 1, host_tensors=host)
    stream = torch.cuda.current_stream().cuda_stream
    got = torch.empty((n_tok, cfg["dim"]), dtype=torch.float32, device=dev)
    from oracle.oracle import Oracle
    orc = Oracle()
    for step in range(2):
        x, logits = workloads.moe_inputs_host(cfg, 20 + step)
        layer.step(torch.from_numpy(x).to(dev), torch.from_numpy(logits).to(dev), got, 0, stream)
        torch.cuda.synchronize()
        ids, wts = layer.last_picks()
        want_ids, want_w = workloads.route_host(cfg, logits)
        assert np.array_equal(ids, want_ids) and np.allclose(wts, want_w, rtol=1e-5, atol=0)
        want = runner.moe_oracle(orc, cfg, host, x, ids, wts)
        assert np.array_equal(_bits(got), want.view(np.uint32))
    assert lib.ep_wait_status() == 0 and lib.q8_status() == 0
    layer.close()
