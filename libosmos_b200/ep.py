"""Expert-parallel MoE layer across the GPUs of one box: one process per GPU, `torch.distributed` (NCCL) for the two
exchanges, every computation a call into libosmos_b200.so (include/osmos_b200/ep.h describes the step).

Sharding: rank r owns experts [r * E / N, (r + 1) * E / N) and is home to tokens [r * T, (r + 1) * T), T = tokens / N.
Dispatch = all-gather of each rank's routed, int8-rounded home tokens (with top-k >= N nearly every rank needs every
token, so the dispatch all-to-all degenerates to an all-gather of 2.4 KB a token); combine = all-to-all of the
computed rows back to the tokens' homes, where each token's rows are added in ascending expert id - the single-GPU
order, so the output bits do not depend on N.

Two transports for the exchanges: "peer" (the default) - the library's own kernels store into the peers' mapped
buffers over NVLink and release per-sender flags (ep_push, ep_scatter_rows_peer, ep_wait); "nccl" - all-gather and
all-to-all through torch.distributed. Same bits either way.
"""
import ctypes as C
import json

import numpy as np
import torch

from . import api, runner, synth, workloads


def expert_range(rank, world, n_exp):
    per = n_exp // world
    return rank * per, (rank + 1) * per


def home_tokens(rank, world, n_tok):
    per = n_tok // world
    return rank * per, (rank + 1) * per


def send_slot(pick, k, tokens_per_rank):
    """where pick i's row goes in the combine's send buffer (row index; blocks of tokens_per_rank * k rows a home)"""
    t, j = pick // k, pick % k
    return (t // tokens_per_rank) * tokens_per_rank * k + (t % tokens_per_rank) * k + j


def peer_layout(world, seg_bytes, block_bytes):
    """byte offsets inside a rank's exchange buffer: the two flag arrays (dispatch, combine; a word a sender), the two
    halves of gathered segments (a segment a sender), the two halves of received row blocks (a block a sender); and
    the buffer's size. Every region starts on 256 bytes."""
    up = lambda v: (v + 255) // 256 * 256
    off_flag = [0, 256]
    off_seg = [512 + p * up(world * seg_bytes) for p in range(2)]
    base_recv = 512 + 2 * up(world * seg_bytes)
    off_recv = [base_recv + p * up(world * block_bytes) for p in range(2)]
    return off_flag, off_seg, off_recv, base_recv + 2 * up(world * block_bytes)


class PeerBuffers:
    """Every rank's exchange buffer, mapped into this process: [dispatch flags][combine flags][2 halves of gathered
    segments][2 halves of received rows]; and the device tables of addresses the pushing kernels take."""

    def __init__(self, lib, dist, dev, rank, world, seg_bytes, block_bytes):
        self.lib, self.rank, self.world = lib, rank, world
        self.off_flag, self.off_seg, self.off_recv, total = peer_layout(world, seg_bytes, block_bytes)
        # Every rank takes every step of the set-up whether or not its own part worked, and the ranks then agree on the
        # outcome: either all of them hold all the mappings or all of them raise (and the caller takes NCCL) - a rank
        # that left alone would leave the others waiting in the next collective.
        mine, handle = C.c_void_p(), (C.c_uint8 * 64)()
        failed = None if lib.ep_peer_alloc(total, C.byref(mine), handle) else "ep_peer_alloc failed"
        self.mine = mine.value if failed is None else None
        all_handles = torch.empty(world * 64, dtype=torch.uint8, device=dev)
        dist.all_gather_into_tensor(all_handles, torch.tensor(list(handle), dtype=torch.uint8, device=dev))
        ok = torch.tensor([int(failed is None)], dtype=torch.int32, device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        all_handles = all_handles.cpu().numpy().reshape(world, 64)
        self.base = [None] * world
        if int(ok.item()):
            for r in range(world):
                if r == rank:
                    self.base[r] = self.mine
                    continue
                p = C.c_void_p()
                h = (C.c_uint8 * 64)(*[int(b) for b in all_handles[r]])
                if not lib.ep_peer_open(h, C.byref(p)):
                    failed = "ep_peer_open failed for rank %d" % r
                    break
                self.base[r] = p.value
        else:
            failed = failed or "ep_peer_alloc failed on another rank"
        ok = torch.tensor([int(failed is None)], dtype=torch.int32, device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if not int(ok.item()):
            for r, b in enumerate(self.base):
                if r != rank and b is not None:
                    lib.ep_peer_close(b)
            dist.barrier()  # nobody's buffer is freed while a peer still maps it
            if self.mine is not None:
                lib.ep_peer_free(self.mine)
            raise RuntimeError(failed or "a peer could not map the exchange buffers")
        tbl = lambda f: torch.tensor([f(r) for r in range(world)], dtype=torch.int64, device=dev)
        # where this rank's piece goes in rank r's buffer, and the flag this rank owns there
        self.dst_seg = [tbl(lambda r, p=p: self.base[r] + self.off_seg[p] + rank * seg_bytes) for p in range(2)]
        self.dst_recv = [tbl(lambda r, p=p: self.base[r] + self.off_recv[p] + rank * block_bytes) for p in range(2)]
        self.flag = [tbl(lambda r, i=i: self.base[r] + self.off_flag[i] + rank * 4) for i in range(2)]
        self.counters = torch.zeros(2, dtype=torch.int32, device=dev)
        dist.barrier()  # every rank has mapped every buffer before anyone stores into one

    def close(self, dist):
        torch.cuda.synchronize()
        dist.barrier()
        for r, b in enumerate(self.base):
            if r != self.rank:
                self.lib.ep_peer_close(b)
        dist.barrier()
        self.lib.ep_peer_free(self.mine)


class EpMoeLane:
    def __init__(self, lib, cfg, dev, rank, world, copies=1, host_tensors=None, transport="peer"):
        import torch.distributed as dist
        self.dist = dist
        self.lib, self.cfg, self.dev, self.rank, self.world = lib, cfg, dev, rank, world
        assert cfg["n_exp"] % world == 0 and cfg["n_tok"] % world == 0
        self.e0, self.e1 = expert_range(rank, world, cfg["n_exp"])
        self.T = cfg["n_tok"] // world
        self.k, self.dim, self.ff, self.n_exp, self.n_tok = cfg["k"], cfg["dim"], cfg["ff"], cfg["n_exp"], cfg["n_tok"]
        self.local = runner.MoeLane(lib, cfg, dev, copies=copies, max_tok=cfg["n_tok"], host_tensors=host_tensors,
                                    expert_range=(self.e0, self.e1))
        self.seg = api.EpSegment()
        lib.ep_segment(self.T, self.k, self.dim, self.seg)
        self.segment = torch.zeros(self.seg.bytes, dtype=torch.uint8, device=dev)
        self.gathered = torch.zeros(self.seg.bytes * world, dtype=torch.uint8, device=dev)
        picks = self.n_tok * self.k
        self.ids_all = torch.zeros(picks, dtype=torch.int32, device=dev)
        self.wts_all = torch.zeros(picks, dtype=torch.float32, device=dev)
        self.q_all = torch.zeros((self.n_tok, self.dim), dtype=torch.int8, device=dev)
        self.d_all = torch.zeros((self.n_tok, self.dim // 32), dtype=torch.float32, device=dev)
        self.rows = torch.zeros(self.T * self.k, dtype=torch.int32, device=dev)
        self.send = torch.zeros((world, self.T * self.k, self.dim), dtype=torch.float32, device=dev)
        self.recv = torch.zeros_like(self.send)
        self.transport, self.step_no = transport, 0
        self.peer = None
        if transport == "peer":
            self.peer = PeerBuffers(lib, dist, dev, rank, world, self.seg.bytes, self.T * self.k * self.dim * 4)
            # route, round, push, wait, unpack, tables, gate_up, round, down, scatter, wait, combine
            self.kernels_per_step = 12
        else:
            self.kernels_per_step = 9  # route, round, unpack, tables, gate_up, round, down, scatter, combine

    def close(self):
        if self.peer:
            self.peer.close(self.dist)
            self.peer = None

    def step(self, x_home, logits_home, out_home, copy=0, stream=0, events=None):
        """x_home [T, dim], logits_home [T, n_exp], out_home [T, dim]: this rank's tokens; all on this GPU.
        events: a pair of CUDA events recorded around this rank's expert kernels (tables, gate + up, round, down)"""
        lib, s, base = self.lib, self.seg, self.segment.data_ptr()
        T, k = self.T, self.k
        ok = lib.q4x_route(logits_home.data_ptr(), T, self.n_exp, k, base + s.ids, base + s.weights, self.rows.data_ptr(), stream)
        ok = ok and lib.q8_round(x_home.data_ptr(), T, self.dim, self.dim, base + s.q, base + s.d, stream)
        if not ok:
            raise RuntimeError("libosmos_b200 refused a call (route / round)")
        self.step_no += 1
        P, n, half = self.peer, self.step_no, self.step_no & 1
        if P:
            ok = lib.ep_push(base, s.bytes, P.dst_seg[half].data_ptr(), P.flag[0].data_ptr(), self.world, n,
                             P.counters.data_ptr(), stream)
            ok = ok and lib.ep_wait(P.mine + P.off_flag[0], self.world, n, stream)
            gathered = P.mine + P.off_seg[half]
        else:
            self.dist.all_gather_into_tensor(self.gathered, self.segment)
            gathered = self.gathered.data_ptr()
        L = self.local
        ok = ok and lib.ep_unpack(gathered, self.world, T, k, self.dim, self.ids_all.data_ptr(),
                                  self.wts_all.data_ptr(), self.q_all.data_ptr(), self.d_all.data_ptr(), stream)
        if events:
            events[0].record()
        ok = ok and lib.lane_ffn_rows(L.layers[copy % len(L.layers)], L.scratch, self.q_all.data_ptr(), self.d_all.data_ptr(),
                                      self.ids_all.data_ptr(), self.wts_all.data_ptr(), self.n_tok, self.e0, self.e1, stream)
        if events:
            events[1].record()
        if P:
            ok = ok and lib.ep_scatter_rows_peer(L.scratch.ye, L.scratch.tab.row_of, self.n_tok * k, k, T, self.dim,
                                                 P.dst_recv[half].data_ptr(), P.flag[1].data_ptr(), self.world, n,
                                                 P.counters.data_ptr() + 4, stream)
            ok = ok and lib.ep_wait(P.mine + P.off_flag[1], self.world, n, stream)
            recv = P.mine + P.off_recv[half]
        else:
            ok = ok and lib.ep_scatter_rows(L.scratch.ye, L.scratch.tab.row_of, self.n_tok * k, k, T, self.dim,
                                            self.send.data_ptr(), stream)
        if not ok:
            raise RuntimeError("libosmos_b200 refused a call (unpack / experts / scatter)")
        if not P:
            self.dist.all_to_all_single(self.recv, self.send)
            recv = self.recv.data_ptr()
        if not lib.ep_combine(recv, base + s.ids, T, k, self.n_exp // self.world, self.dim, None,
                              out_home.data_ptr(), stream):
            raise RuntimeError("libosmos_b200 refused a call (combine)")


def run_bench(args, rank, world, dev, metric, unit, ClockSampler, measured_peaks):
    import torch.distributed as dist

    import libosmos_b200
    lib = libosmos_b200.load()
    cfg = workloads.MOE_IQ3
    n_tok, dim, k = cfg["n_tok"], cfg["dim"], cfg["k"]
    host = workloads.moe_layer_host(cfg)
    copies = 4
    import os
    transport = os.environ.get("OSMOS_EP_TRANSPORT", "peer")
    try:
        layer = EpMoeLane(lib, cfg, dev, rank, world, copies=copies, host_tensors=host, transport=transport)
    except RuntimeError as e:  # the peers' memory could not be mapped here: the exchanges go through NCCL
        if transport != "peer":
            raise
        transport = "nccl (peer mapping unavailable: %s)" % e
        layer = EpMoeLane(lib, cfg, dev, rank, world, copies=copies, host_tensors=host, transport="nccl")
    t0, t1 = home_tokens(rank, world, n_tok)
    n_inputs = 8
    hx, hl = zip(*[workloads.moe_inputs_host(cfg, s) for s in range(n_inputs)])
    dx = [torch.from_numpy(np.ascontiguousarray(a[t0:t1])).to(dev) for a in hx]
    dl = [torch.from_numpy(np.ascontiguousarray(a[t0:t1])).to(dev) for a in hl]
    px = [torch.from_numpy(np.ascontiguousarray(a[t0:t1])).pin_memory() for a in hx]
    pl = [torch.from_numpy(np.ascontiguousarray(a[t0:t1])).pin_memory() for a in hl]
    out = torch.empty((t1 - t0, dim), dtype=torch.float32, device=dev)
    stream = torch.cuda.current_stream().cuda_stream

    # parity first: this rank's first home token against the CPU oracle (same bits as on one GPU)
    from oracle.oracle import Oracle
    layer.step(dx[0], dl[0], out, 0, stream)
    torch.cuda.synchronize()
    ids, wts = workloads.softmax_topk(hl[0][t0:t0 + 1], k)
    got_ids = layer.segment[layer.seg.ids:layer.seg.ids + 4 * k].view(torch.int32).cpu().numpy()
    want = runner.moe_oracle(Oracle(), cfg, host, hx[0][t0:t0 + 1], got_ids.reshape(1, k),
                             layer.segment[layer.seg.weights:layer.seg.weights + 4 * k].view(torch.float32).cpu().numpy().reshape(1, k))
    ok = np.array_equal(got_ids, ids.reshape(-1)) and np.array_equal(out.cpu().numpy()[:1].view(np.uint32), want.view(np.uint32))
    flag = torch.tensor([0 if ok else 1], device=dev)
    dist.all_reduce(flag)
    if int(flag.item()):
        raise SystemExit("bench: the expert-parallel layer's output differs from the CPU oracle's bits on some rank")

    def timed(fn, steps, drain=None):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.barrier()
        torch.cuda.synchronize()
        e0.record()
        for s in range(steps):
            fn(s)
        if drain:
            drain()
        e1.record()
        torch.cuda.synchronize()
        dist.barrier()
        t = torch.tensor([e0.elapsed_time(e1) / 1e3], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def resident(s):
        layer.step(dx[s % n_inputs], dl[s % n_inputs], out, s % copies, stream)

    # end to end: this rank's tokens come from pinned host memory and its output goes back, the copies on their own
    # streams and double-buffered so that they overlap the neighbouring steps' compute (events order a buffer's copy,
    # its use and its reuse); all of it inside the timed region
    cin, cout = torch.cuda.Stream(), torch.cuda.Stream()
    main = torch.cuda.current_stream()
    bx, bl = [torch.empty_like(dx[0]) for _ in range(2)], [torch.empty_like(dl[0]) for _ in range(2)]
    bo = [torch.empty_like(out) for _ in range(2)]
    bp = [torch.empty((t1 - t0, dim), dtype=torch.float32).pin_memory() for _ in range(2)]
    in_ready = [torch.cuda.Event() for _ in range(2)]
    used = [torch.cuda.Event() for _ in range(2)]
    out_done = [torch.cuda.Event() for _ in range(2)]
    for e in used + out_done:
        e.record(main)

    def end_to_end(s):
        b = s & 1
        cin.wait_event(used[b])
        with torch.cuda.stream(cin):
            bx[b].copy_(px[s % n_inputs], non_blocking=True)
            bl[b].copy_(pl[s % n_inputs], non_blocking=True)
            in_ready[b].record(cin)
        main.wait_event(in_ready[b])
        main.wait_event(out_done[b])
        layer.step(bx[b], bl[b], bo[b], s % copies, stream)
        used[b].record(main)
        cout.wait_event(used[b])
        with torch.cuda.stream(cout):
            bp[b].copy_(bo[b], non_blocking=True)
            out_done[b].record(cout)

    def e2e_drain():
        main.wait_stream(cin), main.wait_stream(cout)

    for s in range(args.warmup):
        resident(s), end_to_end(s)
    with ClockSampler(dev.index) as clocks:
        t_res = timed(resident, args.steps)
        t_e2e = timed(end_to_end, args.steps, e2e_drain)
        # rank 0's expert kernels alone (tables, gate + up + activation, round, down), by events inside the step
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
        for s, pair in enumerate(evs):
            layer.step(dx[s % n_inputs], dl[s % n_inputs], out, s % copies, stream, events=pair)
        torch.cuda.synchronize()
        dist.barrier()
    if rank == 0:
        per = workloads.moe_expert_bytes(cfg)
        k_ms = [a.elapsed_time(b) for a, b in evs]
        e0, e1 = expert_range(rank, world, cfg["n_exp"])
        alg = []
        for s in range(args.steps):
            picked = np.unique(workloads.softmax_topk(hl[s % n_inputs], k)[0])
            alg.append(int(((picked >= e0) & (picked < e1)).sum()) * sum(per))
        achieved = float(np.sum(alg) / (np.sum(k_ms) * 1e-3) / 1e9)
        peak, peak_kind = measured_peaks()
        line = {"metric": metric, "value": n_tok * args.steps / t_res, "unit": unit, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": 1e3 * t_res / args.steps, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "int8xint8->f32", "data": "synthetic",
                "config": {"workload": cfg["name"], "tokens": n_tok, "experts": cfg["n_exp"], "top_k": k, "hidden": dim,
                           "expert_ff": cfg["ff"], "format": cfg["type"],
                           "parallelism": "ep%d: experts in contiguous ranges, tokens by home rank, all-gather dispatch, all-to-all combine" % world,
                           "transport": transport,
                           "cold_cache": "%d copies of each rank's %d MB of expert weights cycled" % (copies, sum(per) * cfg["n_exp"] // world // 1000000)},
                "e2e": {"value": n_tok * args.steps / t_e2e, "unit": unit,
                        "h2d_bytes_per_step": int((px[0].numel() + pl[0].numel()) * 4 * world),
                        "d2h_bytes_per_step": int(bp[0].numel() * 4 * world)},
                "gpu_launches": layer.kernels_per_step * args.steps * world,
                "roofline": {"bound": "hbm", "kernel": "rank 0's expert kernels of a step (lane tables, q8_gate_up, q8_round, q8_group_tok)",
                             "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind,
                             "traffic": None, "algorithmic_bytes_per_launch": float(np.mean(alg)),
                             "us_per_launch": float(np.mean(k_ms) * 1e3)},
                "cpu_baseline": None, "clocks": clocks.summary()}
        print(json.dumps(line), flush=True)
    if lib.ep_wait_status():
        raise SystemExit("bench: a wait on a peer's flag ran out on rank %d" % rank)
    layer.close()
    dist.barrier()
    dist.destroy_process_group()
