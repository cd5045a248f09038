"""Expert-parallel MoE layer across the GPUs of one box: one process per GPU, every computation a call into
libosmos_b200.so (include/osmos_b200/ep.h describes the step). This module is set-up only: it allocates the exchange
buffers, lets the ranks map each other's (CUDA IPC handles passed through `torch.distributed`), fills the C plan, and
then a step is ONE call, `ep_layer_step`.

Sharding: rank r owns experts [r * E / N, (r + 1) * E / N) and is home to tokens [r * T, (r + 1) * T), T = tokens / N.
Dispatch: each rank routes and rounds its home tokens and stores the result into every rank's buffer (with top-k >= N
nearly every rank needs every token, so the dispatch all-to-all degenerates to an all-gather of 2.4 KB a token).
Combine: the down projection stores each computed row straight into its token's home rank, where each token's rows are
added in ascending expert id - the single-GPU order, so the output bits do not depend on N. With one rank the same
step runs on the rank's own buffer (no mapping, no process group): that is the single-GPU layer.

A second transport, "nccl", keeps the exchanges in the collective library (all-gather + all-to-all through
torch.distributed) with the library's unfused kernels around them; it is the fallback when the peers' memory cannot
be mapped. Same bits either way.
"""
import ctypes as C

import torch

from . import api, runner, synth, workloads

ROUTERS = {"softmax": 0, "sqrt_softplus": 1, "sigmoid": 2}


def expert_range(rank, world, n_exp):
    per = n_exp // world
    return rank * per, (rank + 1) * per


def home_tokens(rank, world, n_tok):
    per = n_tok // world
    return rank * per, (rank + 1) * per


def send_slot(pick, k, tokens_per_rank):
    """where pick i's row goes in the nccl transport's send buffer (row index; blocks of tokens_per_rank * k rows a home)"""
    t, j = pick // k, pick % k
    return (t // tokens_per_rank) * tokens_per_rank * k + (t % tokens_per_rank) * k + j


def recv_row(pick, k, tokens_per_rank):
    """(home rank, row) of pick i's result in the fused step: row (t % T) * k + j of the home rank's receive block"""
    t, j = pick // k, pick % k
    return t // tokens_per_rank, (t % tokens_per_rank) * k + j


class PeerBuffers:
    """Every rank's exchange buffer (`nbytes`, zeroed) mapped into this process: base[r] is rank r's, base[rank] ours."""

    def __init__(self, lib, dist, dev, rank, world, nbytes):
        self.lib, self.rank, self.world, self.dist = lib, rank, world, dist
        if world == 1:  # nothing to map: plain device memory
            self.own = torch.zeros(nbytes + 256, dtype=torch.uint8, device=dev)
            self.mine = (self.own.data_ptr() + 255) // 256 * 256
            self.base = [self.mine]
            return
        # Every rank takes every step of the set-up whether or not its own part worked, and the ranks then agree on the
        # outcome: either all of them hold all the mappings or all of them raise (and the caller takes NCCL) - a rank
        # that left alone would leave the others waiting in the next collective.
        mine, handle = C.c_void_p(), (C.c_uint8 * 64)()
        failed = None if lib.ep_peer_alloc(nbytes, C.byref(mine), handle) else "ep_peer_alloc failed"
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
        dist.barrier()  # every rank has mapped every buffer before anyone stores into one

    def close(self):
        torch.cuda.synchronize()
        if self.world == 1:
            return
        self.dist.barrier()
        for r, b in enumerate(self.base):
            if r != self.rank:
                self.lib.ep_peer_close(b)
        self.dist.barrier()
        self.lib.ep_peer_free(self.mine)


class EpMoeLane:
    """The layer on this rank. transport "peer": the fused step (one C call); "nccl": the unfused kernels around
    torch.distributed's all-gather and all-to-all."""

    def __init__(self, lib, cfg, dev, rank=0, world=1, copies=1, host_tensors=None, transport="peer", dist=None):
        self.dist = dist
        self.lib, self.cfg, self.dev, self.rank, self.world = lib, cfg, dev, rank, world
        assert cfg["n_exp"] % world == 0 and cfg["n_tok"] % world == 0
        assert world == 1 or dist is not None
        self.e0, self.e1 = expert_range(rank, world, cfg["n_exp"])
        self.T = cfg["n_tok"] // world
        self.k, self.dim, self.ff, self.n_exp, self.n_tok = cfg["k"], cfg["dim"], cfg["ff"], cfg["n_exp"], cfg["n_tok"]
        self.local = runner.MoeLane(lib, cfg, dev, copies=copies, max_tok=cfg["n_tok"], host_tensors=host_tensors,
                                    expert_range=(self.e0, self.e1))
        self.transport, self.peer = transport, None
        picks = self.n_tok * self.k
        self.shared = None
        if cfg.get("shared"):  # a dense expert on every home token, its output added after the routed experts' sum
            sh = cfg["shared"]
            self.shared_w = [torch.from_numpy(a).to(dev) for a in workloads.shared_expert_host(cfg)]
            tid = synth.TYPE_ID[sh["type"]]
            self.shared = api.SharedExpert(tid, tid, self.dim, sh["ff"], sh["lim"], *[t.data_ptr() for t in self.shared_w])
            nbytes = lib.shared_scratch_bytes(self.shared, self.T)
            assert nbytes, "shared_scratch_bytes refused the shared expert"
            self.shared_mem = torch.zeros(nbytes + 256, dtype=torch.uint8, device=dev)
            self.shared_scratch = api.SharedScratch()
            assert lib.shared_scratch_bind(self.shared, self.T, (self.shared_mem.data_ptr() + 255) // 256 * 256, nbytes,
                                           self.shared_scratch)
            self.sye = torch.zeros((self.T, self.dim), dtype=torch.float32, device=dev)
        if transport == "peer":
            lay = api.EpLayout()
            assert lib.ep_layout(world, self.n_tok, self.k, self.dim, lay), "ep_layout refused the shape"
            self.lay = lay
            self.peer = PeerBuffers(lib, dist, dev, rank, world, lay.bytes)
            self.sync = torch.zeros(4, dtype=torch.int32, device=dev)
            self.rows = torch.zeros(2 * picks, dtype=torch.int64, device=dev)  # (the rows' homes, then their weights)
            self.plans = []
            router = ROUTERS[cfg.get("router", "softmax")]
            if router:  # (one tensor for all the plans, alive as long as they are)
                self.route_bias = torch.from_numpy(workloads.route_bias_host(cfg)).to(dev)
            for layer in self.local.layers:
                p = api.EpPlan()
                p.rank, p.n_ranks, p.n_tok, p.expert0, p.expert1, p.lay = rank, world, self.n_tok, self.e0, self.e1, lay
                for r in range(world):
                    p.peer[r] = self.peer.base[r]
                p.sync, p.rows, p.layer, p.scratch = self.sync.data_ptr(), self.rows.data_ptr(), layer, self.local.scratch
                p.router = router
                if router:
                    p.route_bias, p.route_scale = self.route_bias.data_ptr(), cfg["route_scale"]
                if not lib.ep_plan_ok(p):
                    self.peer.close()
                    raise RuntimeError("the fused step does not take this layer")
                self.plans.append(p)
            # route+round+push, wait+tables, gate_up, round, down+push, wait+combine (+ the shared expert's x16,
            # gate, up, activation, x16, down - or, for a decode step's few tokens, its three matvecs and the activation)
            self.kernels_per_step = 6 + (0 if self.shared is None else 4 if self.T <= 8 else 6)
            torch.cuda.synchronize()
            return
        # ---- nccl transport: the unfused kernels ----
        self.seg = api.EpSegment()
        lib.ep_segment(self.T, self.k, self.dim, self.seg)
        self.segment = torch.zeros(self.seg.bytes, dtype=torch.uint8, device=dev)
        self.gathered = torch.zeros(self.seg.bytes * world, dtype=torch.uint8, device=dev)
        self.ids_all = torch.zeros(picks, dtype=torch.int32, device=dev)
        self.wts_all = torch.zeros(picks, dtype=torch.float32, device=dev)
        self.q_all = torch.zeros((self.n_tok, self.dim), dtype=torch.int8, device=dev)
        self.d_all = torch.zeros((self.n_tok, self.dim // 32), dtype=torch.float32, device=dev)
        self.route_rows = torch.zeros(self.T * self.k, dtype=torch.int32, device=dev)
        self.send = torch.zeros((world, self.T * self.k, self.dim), dtype=torch.float32, device=dev)
        self.recv = torch.zeros_like(self.send)
        self.kernels_per_step = 9  # route, round, unpack, tables, gate_up, round, down, scatter, combine

    def close(self):
        if self.peer:
            self.peer.close()
            self.peer = None

    def last_picks(self):
        """(ids, weights) of this rank's home tokens in the last step, as numpy [T, k] (synchronizes)"""
        torch.cuda.synchronize()
        if self.transport == "peer":
            import numpy as np
            ids = np.zeros((self.T, self.k), np.int32)
            wts = np.zeros((self.T, self.k), np.float32)
            assert self.lib.ep_last_picks(self.plans[0], ids.ctypes.data, wts.ctypes.data)
            return ids, wts
        s = self.seg
        ids = self.segment[s.ids:s.ids + 4 * self.T * self.k].view(torch.int32).cpu().numpy().reshape(self.T, self.k)
        wts = self.segment[s.weights:s.weights + 4 * self.T * self.k].view(torch.float32).cpu().numpy().reshape(self.T, self.k)
        return ids, wts

    def step(self, x_home, logits_home, out_home, copy=0, stream=0, add=None, shared=True):
        """x_home [T, dim], logits_home [T, n_exp], out_home [T, dim]: this rank's tokens; all on this GPU. A layer with
        a shared expert runs it first on the home tokens (shared False: the routed experts alone)."""
        if self.shared is not None and shared:
            assert add is None
            if not self.lib.shared_ffn(self.shared, self.shared_scratch, x_home.data_ptr(), self.T, self.sye.data_ptr(), stream):
                raise RuntimeError("libosmos_b200 refused shared_ffn")
            add = self.sye
        if self.transport == "peer":
            if not self.lib.ep_layer_step(self.plans[copy % len(self.plans)], x_home.data_ptr(), logits_home.data_ptr(),
                                          add.data_ptr() if add is not None else None, out_home.data_ptr(), stream):
                raise RuntimeError("libosmos_b200 refused ep_layer_step")
            return
        self._step_nccl(x_home, logits_home, out_home, copy, stream, add)

    def step_phases(self, x_home, logits_home, out_home, copy, stream, events):
        """the fused step with its stages queued one by one and a CUDA event recorded after each (events: 7, the first
        recorded before the first stage): dispatch / wait + tables / gate_up / round / down + push / wait + combine"""
        lib, p = self.lib, self.plans[copy % len(self.plans)]
        L, s = p.layer, p.scratch
        picks = self.n_tok * self.k
        add = None
        if self.shared is not None:  # (before the first event: the stages are the routed experts')
            if not lib.shared_ffn(self.shared, self.shared_scratch, x_home.data_ptr(), self.T, self.sye.data_ptr(), stream):
                raise RuntimeError("libosmos_b200 refused shared_ffn")
            add = self.sye.data_ptr()
        events[0].record()
        ok = lib.ep_route_round_push(p, x_home.data_ptr(), logits_home.data_ptr(), stream)
        events[1].record()
        ok = ok and lib.ep_lane_tables(p, stream)
        events[2].record()
        ok = ok and lib.ep_gate_up(p, stream)
        events[3].record()
        ok = ok and lib.q8_round(s.hh, picks, L.ff, L.ff, s.hq, s.hqd, stream)
        events[4].record()
        ok = ok and lib.ep_down_push(p, stream)
        events[5].record()
        ok = ok and lib.ep_combine_wait(p, add, out_home.data_ptr(), stream)
        events[6].record()
        if not ok:
            raise RuntimeError("libosmos_b200 refused a stage of the fused step")

    def _step_nccl(self, x_home, logits_home, out_home, copy, stream, add):
        lib, s, base = self.lib, self.seg, self.segment.data_ptr()
        T, k = self.T, self.k
        ok = lib.q4x_route(logits_home.data_ptr(), T, self.n_exp, k, base + s.ids, base + s.weights,
                           self.route_rows.data_ptr(), stream)
        ok = ok and lib.q8_round(x_home.data_ptr(), T, self.dim, self.dim, base + s.q, base + s.d, stream)
        if not ok:
            raise RuntimeError("libosmos_b200 refused a call (route / round)")
        if self.world > 1:
            self.dist.all_gather_into_tensor(self.gathered, self.segment)
            gathered = self.gathered.data_ptr()
        else:
            gathered = base
        L = self.local
        ok = lib.ep_unpack(gathered, self.world, T, k, self.dim, self.ids_all.data_ptr(), self.wts_all.data_ptr(),
                           self.q_all.data_ptr(), self.d_all.data_ptr(), stream)
        ok = ok and lib.lane_ffn_rows(L.layers[copy % len(L.layers)], L.scratch, self.q_all.data_ptr(), self.d_all.data_ptr(),
                                      self.ids_all.data_ptr(), self.wts_all.data_ptr(), self.n_tok, self.e0, self.e1, stream)
        ok = ok and lib.ep_scatter_rows(L.scratch.ye, L.scratch.tab.row_of, self.n_tok * k, k, T, self.dim,
                                        self.send.data_ptr(), stream)
        if not ok:
            raise RuntimeError("libosmos_b200 refused a call (unpack / experts / scatter)")
        if self.world > 1:
            self.dist.all_to_all_single(self.recv, self.send)
            recv = self.recv.data_ptr()
        else:
            recv = self.send.data_ptr()
        if not lib.ep_combine(recv, base + s.ids, T, k, self.n_exp // self.world, self.dim,
                              add.data_ptr() if add is not None else None, out_home.data_ptr(), stream):
            raise RuntimeError("libosmos_b200 refused a call (combine)")
