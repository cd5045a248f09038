"""The expert-parallel step's protocol on CPU: 2 and 4 `gloo` ranks run the same sharding, slot and ordering rules as
libosmos_b200/ep.py (its index functions are the ones used here) with the CPU oracle standing in for the kernels, and
the combined result must equal the single-rank layer bit for bit."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from libosmos_b200 import ep, runner, synth, workloads

CFG = dict(workloads.MOE_IQ3, name="ep_test", n_exp=8, k=3, n_tok=8, dim=256, ff=256)  # (both divide by 2 and 4 ranks)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, result_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle.oracle import Oracle
    orc = Oracle()
    cfg = CFG
    k, dim, ff, n_tok = cfg["k"], cfg["dim"], cfg["ff"], cfg["n_tok"]
    host = workloads.moe_layer_host(cfg)
    per = workloads.moe_expert_bytes(cfg)
    x, logits = workloads.moe_inputs_host(cfg, 0)
    t0, t1 = ep.home_tokens(rank, world, n_tok)
    T = t1 - t0
    e0, e1 = ep.expert_range(rank, world, cfg["n_exp"])
    # 1. route and round the home tokens
    ids_home, wts_home = workloads.softmax_topk(logits[t0:t1], k)
    q_home, d_home = orc.q8_round(x[t0:t1])
    # 2. dispatch: all-gather
    def gather(a):
        parts = [torch.zeros_like(torch.from_numpy(a)) for _ in range(world)]
        dist.all_gather(parts, torch.from_numpy(np.ascontiguousarray(a)))
        return np.concatenate([p.numpy() for p in parts])
    ids, wts, q, d = gather(ids_home), gather(wts_home), gather(q_home), gather(d_home)
    # 3. the rows of the owned experts, sorted by (expert, pick)
    flat = ids.reshape(-1)
    order = [i for i in np.argsort(flat, kind="stable") if e0 <= flat[i] < e1]
    tid = synth.TYPE_ID[cfg["type"]]
    # 4. each row goes straight to its token's home rank: row (t % T) * k + j of that rank's receive block
    contrib = np.zeros((world, T * k, dim), np.float32)  # what this rank stores into each home's block
    for i in order:
        e, t = int(flat[i]), i // k
        parts = [host[m][e * per[m]:(e + 1) * per[m]] for m in range(3)]
        g = orc.q8_rows(tid, parts[0], ff, dim, q[t:t + 1], d[t:t + 1])
        u = orc.q8_rows(tid, parts[1], ff, dim, q[t:t + 1], d[t:t + 1])
        h = orc.swiglu_lane(g, u, cfg["lim"], wts.reshape(-1)[i:i + 1])
        hq, hd = orc.q8_round(h)
        y = orc.q8_rows(tid, parts[2], dim, ff, hq, hd)
        home, row = ep.recv_row(i, k, T)
        contrib[home, row] = y[0]
    # 5. the stores of all ranks land in the homes' blocks: every row has exactly one writer, so the block is the sum
    blocks = [torch.zeros(world, T * k, dim) for _ in range(world)]
    dist.all_gather(blocks, torch.from_numpy(contrib))
    recv = sum(b.numpy()[rank] for b in blocks)
    # 6. each home token's rows in ascending expert id
    out = np.zeros((T, dim), np.float32)
    for t in range(T):
        acc = np.zeros(dim, np.float32)
        for j in np.argsort(ids_home[t], kind="stable"):
            acc = (acc + recv[t * k + j]).astype(np.float32)
        out[t] = acc
    outs = [torch.zeros(T, dim) for _ in range(world)]
    dist.all_gather(outs, torch.from_numpy(out))
    if rank == 0:
        full = np.concatenate([o.numpy() for o in outs])
        all_ids, all_wts = workloads.softmax_topk(logits, k)
        want = runner.moe_oracle(orc, cfg, host, x, all_ids, all_wts)
        np.save(result_path, np.array([np.array_equal(full.view(np.uint32), want.view(np.uint32))]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_ranks_equal_one_rank(tmp_path, world):
    result = str(tmp_path / "ok.npy")
    mp.spawn(_rank_main, args=(world, _free_port(), result), nprocs=world, join=True)
    assert bool(np.load(result)[0])


def test_sharding_rules():
    assert ep.expert_range(3, 8, 512) == (192, 256) and ep.home_tokens(7, 8, 64) == (56, 64)
    # every pick lands in a distinct slot, grouped by its token's home
    k, T, world = 10, 8, 8
    slots = [ep.send_slot(i, k, T) for i in range(world * T * k)]
    assert sorted(slots) == list(range(world * T * k))
    assert all(ep.send_slot(i, k, T) // (T * k) == (i // k) // T for i in range(world * T * k))


def test_recv_rows_are_distinct_per_home():
    k, T, world = 10, 8, 8
    seen = set()
    for i in range(world * T * k):
        home, row = ep.recv_row(i, k, T)
        assert home == (i // k) // T and 0 <= row < T * k and (home, row) not in seen
        seen.add((home, row))


def test_exchange_buffer_layout_regions_do_not_overlap():
    """the exchange buffer every rank maps (ep_layout, host code of the library): two flag arrays, two halves of the
    token-major dispatch arrays, two halves of the home rows - nothing overlapping, everything 256-byte aligned"""
    import libosmos_b200
    from libosmos_b200 import api
    lib = libosmos_b200.load()
    for world, n_tok, k, dim in ((1, 64, 10, 2048), (2, 64, 10, 2048), (8, 64, 10, 2048), (16, 32, 8, 7168)):
        lay = api.EpLayout()
        assert lib.ep_layout(world, n_tok, k, dim, lay)
        picks, T = n_tok * k, n_tok // world
        spans = [(lay.flags_dispatch, world * 4), (lay.flags_combine, world * 4)]
        for h in range(2):
            spans += [(lay.ids[h], picks * 4), (lay.weights[h], picks * 4), (lay.q[h], n_tok * dim), (lay.d[h], n_tok * dim // 32 * 4),
                      (lay.recv[h], T * k * dim * 4)]
        spans.sort()
        for (a, n), (b, _) in zip(spans, spans[1:]):
            assert a + n <= b
        assert spans[-1][0] + spans[-1][1] <= lay.bytes and all(a % 256 == 0 for a, _ in spans)
        # the halves are the same distance apart for every array the lane kernels read by parity
        assert lay.q[1] - lay.q[0] == lay.d[1] - lay.d[0] == lay.ids[1] - lay.ids[0] == lay.weights[1] - lay.weights[0]


def test_row_ranges_cover_a_matrix_in_whole_tiles():
    """dense projections across GPUs: every row in exactly one rank's slice, slices in whole 128-row tiles"""
    from libosmos_b200 import shard
    for rows in (128, 512, 4096, 17408):
        for world in (1, 2, 3, 4, 8):
            got = [shard.row_range(r, world, rows) for r in range(world)]
            assert got[0][0] == 0 and got[-1][1] == rows
            assert all(a[1] == b[0] for a, b in zip(got, got[1:]))
            assert all(r0 % 128 == 0 and r1 % 128 == 0 and r1 >= r0 for r0, r1 in got)
            sizes = [r1 - r0 for r0, r1 in got]
            assert max(sizes) - min(sizes) <= 128
    with pytest.raises(ValueError):
        shard.row_range(0, 2, 100)
