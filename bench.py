#!/usr/bin/env python
"""Benchmark of the quantized-weight matrix path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]
    python bench.py --kernel OP TYPE ROWS COLS [--tokens T] [--plain L] [--generic]    # one kernel alone

Default workload (config.workload): the Qwen-style MoE FFN layer in IQ3_XXS - 512 experts, 64 tokens routed top-10,
hidden 2048, expert width 512 - run as the int8 lane: softmax router, activations rounded to int8 per 32, fused gate +
up + activation over the picked experts, the activations rounded again, down, each token's rows summed in ascending
expert id. A step is one pass of the layer over one 64-token batch; successive steps use successive cold copies of
the layer's weights (a model's next layer), so no step finds its weights in L2. On N GPUs the layer runs
expert-parallel (libosmos_b200/ep.py): the same 64 tokens, experts and home tokens split over the ranks.

Prints ONE JSON line: tokens/s through the layer (value: inputs resident in HBM; e2e: pinned host buffers in, host
buffer out, through the C ABI), the dominant kernel's weight-GB/s against the measured HBM peak (roofline), a
per-stage breakdown, and the reference's own CPU lane on this host's cores beside it (cpu_baseline).
`--impl reference` times only that CPU path. Every figure is preceded, in the same run, by a bit-for-bit check of the
GPU result against the CPU checker.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC, UNIT = "moe_layer_tokens_per_s", "tokens/s"
REGIONS = 5  # timed regions of exactly --steps steps each; value is their median


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def measured_tflops():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["bf16_tflops"]), "measured"
    except Exception:
        return 1590.0, "fallback"


class ClockSampler:
    """nvidia-smi's SM clock and throttle reasons sampled while the timed regions run"""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.index, self.lines, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "50"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=lambda: [self.lines.append(l) for l in self.proc.stdout], daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        for l in self.lines:
            f = [x.strip() for x in l.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[1])), mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons), "samples": len(sm)}


def dist_env():
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    return rank, world, int(os.environ.get("LOCAL_RANK", str(rank)))


def workload_config(cfg):
    """the workload's description: the same keys in both arms"""
    c = {"workload": cfg["name"], "tokens": cfg["n_tok"], "experts": cfg["n_exp"], "top_k": cfg["k"],
         "hidden": cfg["dim"], "expert_ff": cfg["ff"], "format": cfg["type"]}
    if cfg.get("router"):
        c["router"] = cfg["router"]
    if cfg.get("shared"):
        c["shared_expert"] = "%s, ff %d" % (cfg["shared"]["type"], cfg["shared"]["ff"])
    if cfg.get("path"):
        c["path"] = {"f32_lane": "F32 activations, an expert read once for its tokens (mv_group_tok)",
                     "f16_group": "f16 activations, grouped tensor-core product (mm_group)"}[cfg["path"]]
    return c


# ---------------------------------------------------------------------------------------------------------------------
# the CPU checker and the reference arm: the reference's CPU lane (oracle/_ref, its sources compiled unmodified) or,
# where that library is missing or this CPU lacks its AVX-512 VNNI kernels, this repository's scalar restatement
# ---------------------------------------------------------------------------------------------------------------------
def lane_rows_of(cfg, x, ids, wts):
    """a step's rows by (expert, pick) - the lane's layout, a row an expert's copy of its token's input: the rows'
    inputs and routed weights, the experts' (id, first row, count), and each row's pick"""
    flat = ids.reshape(-1)
    order = np.argsort(flat, kind="stable")
    xr = np.ascontiguousarray(x[order // cfg["k"]])
    sc = np.ascontiguousarray(wts.reshape(-1)[order])
    experts, r = [], 0
    for e in np.unique(flat):
        c = int((flat == e).sum())
        experts.append((int(e), r, c))
        r += c
    return xr, sc, experts, order


def cpu_step_inputs(cfg, step):
    from libosmos_b200 import workloads
    x, logits = workloads.moe_inputs_host(cfg, step)
    ids, wts = workloads.route_host(cfg, logits)
    return lane_rows_of(cfg, x, ids, wts)


class CpuArm:
    def __init__(self, cfg, host_tensors, threads=None, pin=True):
        from libosmos_b200 import synth, workloads
        from oracle.oracle import Oracle, Reference
        self.cfg, self.host = cfg, host_tensors
        self.tid = synth.TYPE_ID[cfg["type"]]
        self.per = workloads.moe_expert_bytes(cfg)
        avail = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
        self.kind = "reference" if Reference.available() else "port"
        self.pinned = []
        if self.kind == "reference":
            self.ref = Reference()
            self.threads = max(1, min(64, threads or avail))
            self.pool, self.pinned = self.ref.lane_pool(self.threads, cfg["n_tok"] * cfg["k"], cfg["dim"], cfg["ff"], pin)
            if not self.pool:
                self.kind = "port"
        if self.kind == "port":
            self.oracle, self.threads = Oracle(), 1

    def parts(self, e):
        return [self.host[m][e * self.per[m]:(e + 1) * self.per[m]] for m in range(3)]

    def job(self, xr, sc, experts):
        cfg = self.cfg
        ex = [tuple(self.parts(e)) + (r0, c) for e, r0, c in experts]
        return self.ref.lane_job(self.tid, self.tid, cfg["dim"], cfg["ff"], cfg["lim"], xr, sc, ex)

    def rows(self, xr, sc, experts, limit_rows=None):
        """one step's expert FFN rows on the CPU; returns (seconds, rows done, y). The reference's job is built before
        the clock starts."""
        cfg = self.cfg
        if self.kind == "reference":
            job = self.job(xr, sc, experts)
            t0 = time.perf_counter()
            ok = job.run(self.pool)
            dt = time.perf_counter() - t0
            assert ok, "the reference's cpu_lane refused or failed the job"
            return dt, xr.shape[0], job.y
        done, t0 = 0, time.perf_counter()
        y = np.zeros((xr.shape[0], cfg["dim"]), np.float32)
        for e, r0, c in experts:
            p = self.parts(e)
            y[r0:r0 + c] = self.oracle.lane_expert(self.tid, self.tid, p[0], p[1], p[2], cfg["dim"], cfg["ff"], cfg["lim"],
                                                   xr[r0:r0 + c], sc[r0:r0 + c])
            done += c
            if limit_rows and done >= limit_rows:
                break
        return time.perf_counter() - t0, done, y

    def layer(self, x, ids, wts):
        """the whole layer's output for tokens x with the given picks: the rows, then each token's rows added in
        ascending expert id (the checker of the GPU step)"""
        cfg = self.cfg
        xr, sc, experts, order = lane_rows_of(cfg, x, ids, wts)
        _, done, y = self.rows(xr, sc, experts)
        assert done == xr.shape[0]
        out = np.zeros((x.shape[0], cfg["dim"]), np.float32)
        tok = order // cfg["k"]
        for r in range(xr.shape[0]):  # rows ascend with the expert id
            out[tok[r]] = (out[tok[r]] + y[r]).astype(np.float32)
        return out

    def shared_seconds(self):
        """a step's shared expert on this CPU: the scalar restatement's F32 matvec (not reference code: the reference has
        no CPU path for the shared expert's type), its rows split over as many threads as the lane uses, timed on one
        token and scaled to the step's tokens"""
        cfg = self.cfg
        if not cfg.get("shared"):
            return 0.0
        from concurrent.futures import ThreadPoolExecutor

        from libosmos_b200 import synth, workloads
        from oracle.oracle import Oracle
        sh, orc = cfg["shared"], Oracle()
        tid = synth.TYPE_ID[sh["type"]]
        w = workloads.shared_expert_host(cfg)
        x = np.ones((1, cfg["dim"]), np.float32)

        def product(mat, rows, cols, v, pool):
            rb = mat.size // rows
            cuts = np.linspace(0, rows, self.threads + 1).astype(int)
            parts = pool.map(lambda i: orc.mv_rows(tid, mat[cuts[i] * rb:cuts[i + 1] * rb], int(cuts[i + 1] - cuts[i]), cols, v),
                             [i for i in range(self.threads) if cuts[i + 1] > cuts[i]])
            return np.concatenate(list(parts), axis=1)

        with ThreadPoolExecutor(self.threads) as pool:
            t0 = time.perf_counter()
            g = product(w[0], sh["ff"], cfg["dim"], x, pool)
            product(w[1], sh["ff"], cfg["dim"], x, pool)
            product(w[2], cfg["dim"], sh["ff"], g, pool)
            return (time.perf_counter() - t0) * cfg["n_tok"]

    def timed(self, steps, warmup, first_step=0):
        """tokens/s over `steps` steps after `warmup`; each step's job is built outside its clock"""
        cfg, limit = self.cfg, (None if self.kind == "reference" else 24)
        times, rows = [], 0
        for s in range(warmup + steps):
            xr, sc, experts, _ = cpu_step_inputs(cfg, first_step + s)
            dt, done, _ = self.rows(xr, sc, experts, limit)
            if s >= warmup:
                times.append(dt), (rows := rows + done)
        sample = ("%d full steps of %d tokens (%d expert rows each) after %d warm-up" % (steps, cfg["n_tok"], cfg["n_tok"] * cfg["k"], warmup)
                  if limit is None else "the first %d expert rows of %d steps, scaled to tokens" % (limit, steps))
        shared = self.shared_seconds()
        if shared:
            sample += "; + the shared expert by the scalar restatement on the same threads (one token timed, scaled to the step: %.1f ms a step)" % (1e3 * shared)
        per_step = sum(times) / len(times) * (cfg["n_tok"] * cfg["k"] / (rows / len(times))) + shared
        return cfg["n_tok"] / per_step, 1e3 * per_step, sample


def port_tokens_per_s(cfg, host, per):
    """the CPU figure of a workload the reference has no CPU path for (its experts' type is not a CPU lane type): this
    repository's scalar restatement of the F32 matvec on ONE pick's three matrices, scaled to the step's picks"""
    from libosmos_b200 import synth
    from oracle.oracle import Oracle
    orc, tid = Oracle(), synth.TYPE_ID[cfg["type"]]
    x = np.ones((1, cfg["dim"]), np.float32)
    p = [host[m][:per[m]] for m in range(3)]
    t0 = time.perf_counter()
    g = orc.mv_rows(tid, p[0], cfg["ff"], cfg["dim"], x)
    orc.mv_rows(tid, p[1], cfg["ff"], cfg["dim"], x)
    orc.mv_rows(tid, p[2], cfg["dim"], cfg["ff"], g)
    dt = (time.perf_counter() - t0) * cfg["n_tok"] * cfg["k"]
    return cfg["n_tok"] / dt, 1e3 * dt, "one pick's gate, up and down by the scalar restatement (1 thread), scaled to the step's %d picks" % (cfg["n_tok"] * cfg["k"])


def run_reference(args):
    from libosmos_b200 import workloads
    rank, world, _ = dist_env()
    if rank != 0:
        return
    cfg = workloads.BY_NAME[args.workload]
    if cfg.get("path") == "dense_rows":  # the product's scalar restatement on a sample of rows, scaled to the matrix
        from libosmos_b200 import synth
        from oracle.oracle import Oracle
        orc = Oracle()
        tid, rows, cols, n_tok = synth.TYPE_ID[cfg["type"]], cfg["rows"], cfg["cols"], cfg["tokens"]
        w = synth.random_tensor(tid, rows, cols, synth.rng_for(2, tid, rows), cfg["sigma"])
        x = synth.rng_for(8, n_tok, 0).standard_normal((n_tok, cols)).astype(np.float32)
        sample_rows, times = 8, []
        for _ in range(max(1, min(args.steps, 5))):
            t0 = time.perf_counter()
            hx8, hdx, hsx = orc.mmq_x8_rows(x, np.arange(n_tok, dtype=np.int32), cols)
            orc.mmq_rows(np.ascontiguousarray(w.reshape(rows, -1)[:sample_rows]).reshape(-1), sample_rows, cols, hx8, hdx, hsx, 0, n_tok)
            times.append(time.perf_counter() - t0)
        sec = float(np.median(times)) * rows / sample_rows
        sample = "%d rows x all tokens through the scalar restatement, scaled to %d rows" % (sample_rows, rows)
        line = {"impl": "reference", "metric": "prefill_tokens_per_s", "value": n_tok / sec, "unit": "tokens/s", "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * sec, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "int8xint8->f32", "data": "synthetic",
                "config": {"workload": cfg["name"], "format": cfg["type"], "rows": rows, "cols": cols, "tokens": n_tok},
                "cpu_baseline": {"value": n_tok / sec, "unit": "tokens/s", "cores": 1, "kind": "port", "sample": sample},
                "e2e": {"value": n_tok / sec, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line), flush=True)
        return
    if cfg.get("path"):
        per = workloads.moe_expert_bytes(cfg)
        tok_s, ms, sample = port_tokens_per_s(cfg, workloads.moe_layer_host(cfg, expert_range=(0, 1)), per)
        line = {"impl": "reference", "metric": METRIC, "value": tok_s, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "f32", "data": "synthetic", "config": workload_config(cfg),
                "cpu_baseline": {"value": tok_s, "unit": UNIT, "cores": 1, "kind": "port", "sample": sample},
                "e2e": {"value": tok_s, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line), flush=True)
        return
    host = workloads.moe_layer_host(cfg)
    arm = CpuArm(cfg, host)
    tok_s, ms, sample = arm.timed(args.steps, args.warmup)
    one = None
    if arm.kind == "reference":  # the single-thread figure beside it
        one_arm = CpuArm(cfg, host, threads=1)
        one = one_arm.timed(max(1, min(3, args.steps)), 1)[0]
    line = {"impl": "reference", "metric": METRIC, "value": tok_s, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "int8xint8->f32", "data": "synthetic",
            "config": workload_config(cfg),
            "cpu_baseline": {"value": tok_s, "unit": UNIT, "cores": arm.threads, "kind": arm.kind, "sample": sample,
                             "pinned_cpus": arm.pinned, "one_thread_value": one},
            "e2e": {"value": tok_s, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------------------------------
def run_ours(args):
    import torch

    import libosmos_b200
    from libosmos_b200 import ep, workloads
    rank, world, local = dist_env()
    assert world == args.gpus or world == 1, "launch N ranks for --gpus N"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    lib = libosmos_b200.load()
    cfg = workloads.BY_NAME[args.workload]
    if cfg.get("path") == "dense_rows":  # the prefill product, rows split among the ranks
        run_dense_rows(args, cfg, lib, dev, rank, world, dist)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return
    if cfg.get("path"):  # the experts over F32 activations, or through the grouped f16 product: one GPU
        return run_f32_or_f16(args, cfg, lib, dev)
    n_tok, dim, k = cfg["n_tok"], cfg["dim"], cfg["k"]
    if n_tok % world:
        raise SystemExit("bench: %d tokens do not split over %d ranks" % (n_tok, world))
    host = workloads.moe_layer_host(cfg)
    per = workloads.moe_expert_bytes(cfg)
    # cold weights every step: copies of the layer cycled (a large layer's step touches far more than L2 by itself)
    copies = 4 if sum(per) * cfg["n_exp"] // world < (3 << 30) // 2 else 2
    transport = os.environ.get("OSMOS_EP_TRANSPORT", "peer")
    try:
        layer = ep.EpMoeLane(lib, cfg, dev, rank, world, copies=copies, host_tensors=host, transport=transport, dist=dist)
    except RuntimeError as e:  # the peers' memory could not be mapped here: the exchanges go through NCCL
        if transport != "peer" or world == 1:
            raise
        transport = "nccl (peer mapping unavailable: %s)" % e
        layer = ep.EpMoeLane(lib, cfg, dev, rank, world, copies=copies, host_tensors=host, transport="nccl", dist=dist)
    fused = layer.transport == "peer"
    t0, t1 = ep.home_tokens(rank, world, n_tok)
    T = t1 - t0
    n_inputs = 8
    hx, hl = zip(*[workloads.moe_inputs_host(cfg, s) for s in range(n_inputs)])
    dx = [torch.from_numpy(np.ascontiguousarray(a[t0:t1])).to(dev) for a in hx]
    dl = [torch.from_numpy(np.ascontiguousarray(a[t0:t1])).to(dev) for a in hl]
    px = [torch.from_numpy(np.ascontiguousarray(a[t0:t1])).pin_memory() for a in hx]
    pl = [torch.from_numpy(np.ascontiguousarray(a[t0:t1])).pin_memory() for a in hl]
    out = torch.empty((T, dim), dtype=torch.float32, device=dev)
    stream = torch.cuda.current_stream().cuda_stream

    def all_ok(ok):
        if world == 1:
            return ok
        flag = torch.tensor([0 if ok else 1], device=dev)
        dist.all_reduce(flag)
        return int(flag.item()) == 0

    # parity first: EVERY home token of step 0 against the CPU checker's bits (the reference's own CPU lane where it
    # runs, else the scalar restatement), with the picks the GPU made (checked equal to a double-precision softmax)
    layer.step(dx[0], dl[0], out, 0, stream, shared=False)
    torch.cuda.synchronize()
    got_ids, got_wts = layer.last_picks()
    arm = CpuArm(cfg, host)
    ok = workloads.router_check(cfg, hl[0][t0:t1], got_ids, got_wts)
    if not ok:
        sys.stderr.write("bench: rank %d: the router's picks or weights differ from the double-precision router (first token: picks %r weights %r)\n"
                         % (rank, got_ids[0].tolist(), got_wts[0].tolist()))
    want = arm.layer(hx[0][t0:t1], got_ids, got_wts)
    routed = out.cpu().numpy().copy()
    if not np.array_equal(routed.view(np.uint32), want.view(np.uint32)):
        bad = np.argwhere(routed.view(np.uint32) != want.view(np.uint32))
        sys.stderr.write("bench: rank %d: %d of %d values of the routed experts' sum differ from the CPU checker's bits (first at token %d "
                         "column %d: %r against %r)\n" % (rank, len(bad), routed.size, bad[0][0], bad[0][1], routed[tuple(bad[0])], want[tuple(bad[0])]))
        ok = False
    parity = "all %d home tokens of step 0 on every rank, the routed experts' sum bit-equal to the %s" % (
        T, "reference's cpu_lane_submit" if arm.kind == "reference" else "scalar restatement of the reference's CPU lane")
    if ok and cfg.get("shared"):
        # the shared expert runs on the f16 tensor cores (more than 8 home tokens) or through the F32 matvec: either way its
        # sums are held to a bound around a float64 sum over the f16-rounded operands, on this rank's first tokens
        from libosmos_b200 import synth
        from oracle.oracle import Oracle
        layer.step(dx[0], dl[0], out, 0, stream)
        torch.cuda.synchronize()
        sh, orc, ns = cfg["shared"], Oracle(), min(T, 2)
        tid = synth.TYPE_ID[sh["type"]]
        wf = [orc.dequant(tid, a, r * c).reshape(r, c).astype(np.float16).astype(np.float64) for a, (r, c) in
              zip(workloads.shared_expert_host(cfg), ((sh["ff"], dim), (sh["ff"], dim), (dim, sh["ff"])))]
        x16 = hx[0][t0:t0 + ns].astype(np.float16).astype(np.float64)
        g, u = np.minimum(x16 @ wf[0].T, sh["lim"]), np.clip(x16 @ wf[1].T, -sh["lim"], sh["lim"])
        h16 = (g / (1 + np.exp(-g)) * u).astype(np.float16).astype(np.float64)
        ref = h16 @ wf[2].T
        mag = np.abs(h16) @ np.abs(wf[2]).T
        diff = out.cpu().numpy()[:ns].astype(np.float64) - routed[:ns]
        ok = bool((np.abs(diff - ref) <= 2.0 ** -9 * mag + 1e-6 * np.abs(routed[:ns])).all())
        if not ok:
            sys.stderr.write("bench: rank %d: the shared expert's output is outside its bound (worst %.3e of its magnitude sum)\n"
                             % (rank, float((np.abs(diff - ref) / (mag + 1e-30)).max())))
        parity += "; the shared expert's output (%s) within 2^-9 sum |h w| of a float64 model over f16-rounded operands (%d tokens)" % (
            "F32 matvec: a decode step's tokens" if T <= 8 else "f16 tensor-core product", ns)
    if not all_ok(ok):
        raise SystemExit("bench: the GPU layer's output differs from the CPU checker on some rank - not timing a wrong result")
    distinct = [np.unique(workloads.route_host(cfg, l)[0]) for l in hl]

    def barrier():
        if world > 1:
            dist.barrier()

    def timed(fn, steps, drain=None):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        torch.cuda.synchronize()
        e0.record()
        for s in range(steps):
            fn(s)
        if drain:
            drain()  # the side streams' last copies are inside the timed region
        e1.record()
        torch.cuda.synchronize()
        barrier()
        t = e0.elapsed_time(e1) / 1e3
        if world > 1:
            tt = torch.tensor([t], device=dev)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            t = float(tt.item())
        return t

    def resident(s):
        layer.step(dx[s % n_inputs], dl[s % n_inputs], out, s % copies, stream)

    # end to end: every step's inputs come from pinned host memory and its output goes back to it, the copies on
    # their own streams so that step s + 1's inputs and step s - 1's output move while step s computes (two buffers
    # of each; events order a buffer's copy, its use and its reuse); all of it inside the timed region
    cin, cout = torch.cuda.Stream(), torch.cuda.Stream()
    main = torch.cuda.current_stream()
    bx = [torch.empty_like(dx[0]) for _ in range(2)]
    bl = [torch.empty_like(dl[0]) for _ in range(2)]
    bo = [torch.empty_like(out) for _ in range(2)]
    bp = [torch.empty((T, dim), dtype=torch.float32).pin_memory() for _ in range(2)]
    in_ready = [torch.cuda.Event() for _ in range(2)]
    used = [torch.cuda.Event() for _ in range(2)]
    out_done = [torch.cuda.Event() for _ in range(2)]
    for e in used + out_done:
        e.record(main)

    def end_to_end(s):
        b = s & 1
        cin.wait_event(used[b])  # the step that last read these input buffers is done
        with torch.cuda.stream(cin):
            bx[b].copy_(px[s % n_inputs], non_blocking=True)
            bl[b].copy_(pl[s % n_inputs], non_blocking=True)
            in_ready[b].record(cin)
        main.wait_event(in_ready[b])
        main.wait_event(out_done[b])  # the last output in bo[b] has reached the host
        layer.step(bx[b], bl[b], bo[b], s % copies, stream)
        used[b].record(main)
        cout.wait_event(used[b])
        with torch.cuda.stream(cout):
            bp[b].copy_(bo[b], non_blocking=True)
            out_done[b].record(cout)

    def e2e_drain():
        main.wait_stream(cin), main.wait_stream(cout)

    if args.profile:  # for a profiler: the checked step, then W + K plain steps on the stream, nothing timed or printed
        for s in range(args.warmup + args.steps):
            resident(s)
        torch.cuda.synchronize()
        if lib.ep_wait_status() or lib.q8_status():
            raise SystemExit("bench: a bounded wait ran out on rank %d" % rank)
        layer.close()
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return
    for s in range(args.warmup):
        resident(s), end_to_end(s)
    # the resident step as a user of the C ABI would run a decode loop: captured once per (input, weight copy) pair in
    # a CUDA graph and replayed - the same launches (the fused step keeps its step number on the device, so a captured
    # step is valid for every replay), without the host's launch gaps
    graphs = []
    if fused:
        torch.cuda.synchronize()
        barrier()
        side = torch.cuda.Stream()
        for s in range(n_inputs):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                layer.step(dx[s], dl[s], out, s % copies, side.cuda_stream)
            graphs.append(g)
        torch.cuda.synchronize()
        barrier()

    def resident_graph(s):
        graphs[s % n_inputs].replay()

    best = resident_graph if graphs else resident
    if graphs:
        for s in range(args.warmup):
            resident_graph(s)
        torch.cuda.synchronize()
        layer.step(dx[1], dl[1], out, 1 % copies, stream)
        torch.cuda.synchronize()
        plain_bits = out.cpu().numpy().view(np.uint32).copy()
        resident_graph(1)
        torch.cuda.synchronize()
        if not all_ok(np.array_equal(plain_bits, out.cpu().numpy().view(np.uint32))):
            raise SystemExit("bench: the graph-replayed step differs from the stream-launched one")
    with ClockSampler(local) as clocks:
        # about a second of the same steps first, so that the clock sampler sees the GPU under this load (the same
        # count on every rank: a rank's steps pair with its peers')
        n_warm = int(min(20000, max(args.steps, 1.0 / (timed(best, args.steps) / args.steps))))
        for s in range(n_warm):
            best(s)
            if s % 256 == 255:
                torch.cuda.synchronize()
        torch.cuda.synchronize()
        t_regions = [timed(best, args.steps) for _ in range(REGIONS)]
        t_stream = [timed(resident, args.steps) for _ in range(REGIONS)]
        t_e2e = [timed(end_to_end, args.steps, e2e_drain) for _ in range(REGIONS)]
        # the stages of a step by events inside the step (fused transport), max over ranks of each stage's mean
        stage_names = ["route+round+dispatch", "wait+tables", "gate_up", "round", "down+push", "wait+combine"]
        stage_ms = None
        if fused:
            n_ev = min(args.steps, 50)
            evs = [[torch.cuda.Event(enable_timing=True) for _ in range(7)] for _ in range(n_ev)]
            barrier()
            torch.cuda.synchronize()
            for s, e in enumerate(evs):
                layer.step_phases(dx[s % n_inputs], dl[s % n_inputs], out, s % copies, stream, e)
            torch.cuda.synchronize()
            stage = np.array([[e[i].elapsed_time(e[i + 1]) for i in range(6)] for e in evs])
            stage_ms = stage.mean(axis=0)
            if world > 1:
                tt = torch.tensor(stage_ms, device=dev)
                dist.all_reduce(tt, op=dist.ReduceOp.MAX)
                stage_ms = tt.cpu().numpy()
    t_res, t_str, t_ee = float(np.median(t_regions)), float(np.median(t_stream)), float(np.median(t_e2e))
    if lib.ep_wait_status() or lib.q8_status():
        raise SystemExit("bench: a bounded wait ran out on rank %d" % rank)
    if rank == 0:
        e0, e1 = ep.expert_range(rank, world, cfg["n_exp"])
        peak, peak_kind = measured_peaks()
        roof = {"bound": "hbm", "peak": peak, "unit": "GB/s", "peak_kind": peak_kind}
        if fused:
            # rank 0's gate + up + activation kernel: the distinct experts of the steps it was timed on, that it owns
            alg = [int(((distinct[s % n_inputs] >= e0) & (distinct[s % n_inputs] < e1)).sum()) * (per[0] + per[1])
                   for s in range(len(evs))]
            k_ms = stage[:, 2]
            achieved = float(np.sum(alg) / (np.sum(k_ms) * 1e-3) / 1e9)
            roof.update({"kernel": "q8_gate_up (lane_ring_kernel, %s, fused gate + up + activation) on rank 0" % cfg["type"],
                         "achieved": achieved, "frac": achieved / peak,
                         "traffic": 296292352 if (world == 1 and cfg["name"] == workloads.MOE_IQ3["name"]) else None,
                         "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one launch, profiles/lane_ring_rows_iq3xxs_moe.md"
                         if (world == 1 and cfg["name"] == workloads.MOE_IQ3["name"]) else None,
                         "algorithmic_bytes_per_launch": float(np.mean(alg)), "us_per_launch": float(np.mean(k_ms) * 1e3)})
        cpu = None
        try:
            tok_s, _, sample = arm.timed(5 if arm.kind == "reference" else 1, 1)
            cpu = {"value": tok_s, "unit": UNIT, "cores": arm.threads, "kind": arm.kind, "sample": sample}
        except Exception as e:  # the baseline is reported, never required
            cpu = {"value": None, "unit": UNIT, "cores": 0, "kind": "unavailable", "sample": str(e)[:120]}
        line = {"metric": METRIC, "value": n_tok * args.steps / t_res, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": 1e3 * t_res / args.steps, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "int8xint8->f32", "data": "synthetic", "config": workload_config(cfg),
                "run": {"parallelism": "1 gpu" if world == 1 else
                        "ep%d: experts in contiguous ranges, tokens by home rank; dispatch and combine by peer stores from the producing kernels" % world,
                        "transport": transport if world > 1 else "none",
                        "launch": ("value: CUDA graph replay, one graph a (input, weight copy) pair" if graphs else "value: launched on the stream")
                                  + "; the same steps launched on the stream take %.4f ms" % (1e3 * t_str / args.steps),
                        "cold_cache": "%d copies of each rank's %d MB of expert weights cycled; a step touches ~%d MB in all (> 126 MB L2 at 1 GPU)"
                                      % (copies, sum(per) * cfg["n_exp"] // world // 1000000,
                                         int(np.mean([len(d) for d in distinct])) * sum(per) // 1000000),
                        "timing": "median of %d regions of exactly %d steps, CUDA events, max over ranks" % (REGIONS, args.steps),
                        "regions_ms_per_step": [1e3 * t / args.steps for t in t_regions],
                        "parity": parity},
                "e2e": {"value": n_tok * args.steps / t_ee, "unit": UNIT,
                        "h2d_bytes_per_step": int((px[0].numel() + pl[0].numel()) * 4 * world),
                        "d2h_bytes_per_step": int(bp[0].numel() * 4 * world)},
                "gpu_launches": layer.kernels_per_step * args.steps * world,
                "roofline": roof,
                "stages_ms": None if stage_ms is None else dict(zip(stage_names, [float(v) for v in stage_ms])),
                "cpu_baseline": cpu, "clocks": clocks.summary()}
        if world == 1 and cfg["name"] == workloads.MOE_IQ3["name"]:
            try:
                line["matvec"] = matvec_leg(lib, dev, peak)
            except Exception as e:  # a second figure beside the headline: reported, never required
                line["matvec"] = {"unavailable": str(e)[:160]}
            try:
                line["prefill"] = prefill_leg(lib, dev)
            except Exception as e:
                line["prefill"] = {"unavailable": str(e)[:160]}
        print(json.dumps(line), flush=True)
    layer.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_dense_rows(args, cfg, lib, dev, rank, world, dist):
    """The prefill product of a dense projection with its output rows split among the GPUs: Q4_K W[rows x cols] over the
    tokens, every rank rounding all the tokens to int8 (the activations are not split) and multiplying its slice of
    whole 128-row tiles - no collective on the data path, a rank's columns of y stay with it. Before timing every rank
    compares its slice's sampled rows x all tokens with the CPU checker's bits. A step = mmq_x8_rows + mmq_group on a
    cold copy of the slice; value = tokens through the whole matrix a second (max over ranks); strong scaling."""
    import torch

    from libosmos_b200 import shard, synth
    from oracle.oracle import Oracle
    orc = Oracle()
    tid, rows, cols, n_tok = synth.TYPE_ID[cfg["type"]], cfg["rows"], cfg["cols"], cfg["tokens"]
    w = synth.random_tensor(tid, rows, cols, synth.rng_for(2, tid, rows), cfg["sigma"])
    nb_all = int(w.size)
    r0, r1 = shard.row_range(rank, world, rows)
    mine = r1 - r0
    copies = max(2, int((160 << 20) // max(1, nb_all * mine // rows)) + 1)  # more than the 126 MB L2 cycled
    copies = min(copies, 256)
    layer = shard.DenseRows(lib, dev, tid, rows, cols, w, rank, world, copies=copies, max_tok=n_tok)
    n_inputs = 4
    hx = [synth.rng_for(8, n_tok, s).standard_normal((n_tok, cols)).astype(np.float32) for s in range(n_inputs)]
    dx = [torch.from_numpy(a).to(dev) for a in hx]
    px = [torch.from_numpy(a).pin_memory() for a in hx]
    y = torch.zeros((n_tok, max(mine, 1)), dtype=torch.float32, device=dev)
    pout = torch.empty((n_tok, max(mine, 1)), dtype=torch.float32).pin_memory()
    stream = torch.cuda.current_stream().cuda_stream

    def all_ok(ok):
        if world == 1:
            return ok
        flag = torch.tensor([0 if ok else 1], device=dev)
        dist.all_reduce(flag)
        return int(flag.item()) == 0

    layer.step(dx[0], n_tok, y, 0, stream)
    torch.cuda.synchronize()
    ok = True
    if mine:
        pick = np.sort(synth.rng_for(7, rank).choice(mine, min(mine, 64), replace=False))
        rb = nb_all // rows
        wsel = np.ascontiguousarray(w.reshape(rows, rb)[r0 + pick]).reshape(-1)
        hx8, hdx, hsx = orc.mmq_x8_rows(hx[0], np.arange(n_tok, dtype=np.int32), cols)
        want = orc.mmq_rows(wsel, len(pick), cols, hx8, hdx, hsx, 0, n_tok)
        ok = bool(np.array_equal(y.cpu().numpy()[:, pick].view(np.uint32), want.view(np.uint32)))
        if not ok:
            sys.stderr.write("bench: rank %d: its slice's rows differ from the CPU checker's bits\n" % rank)
    if not all_ok(ok):
        raise SystemExit("bench: a slice of the product differs from the CPU checker - not timing a wrong result")

    def timed(fn, steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0.record()
        for s in range(steps):
            fn(s)
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / 1e3], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def resident(s):
        layer.step(dx[s % n_inputs], n_tok, y, s, stream)

    bx = torch.empty_like(dx[0])

    def end_to_end(s):  # the tokens from pinned host memory in, this rank's columns out, every step
        bx.copy_(px[s % n_inputs], non_blocking=True)
        layer.step(bx, n_tok, y, s, stream)
        pout.copy_(y, non_blocking=True)

    for s in range(max(args.warmup, 3)):
        resident(s), end_to_end(s)
    with ClockSampler(dev.index) as clocks:
        n_warm = int(min(5000, max(args.steps, 0.5 / (timed(resident, args.steps) / args.steps))))
        for s in range(n_warm):
            resident(s)
        t_regions = [timed(resident, args.steps) for _ in range(REGIONS)]
        t_e2e = [timed(end_to_end, args.steps) for _ in range(REGIONS)]
        # the product alone, by events around each launch of the slice's kernel (the roofline's kernel)
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(32)]
        for s, (a, b) in enumerate(ev):
            lib.mmq_x8_rows(dx[0].data_ptr(), cols, layer.idx.data_ptr(), n_tok, cols, layer.x8.data_ptr(), layer.dx.data_ptr(),
                            layer.sx.data_ptr(), stream)
            a.record()
            if mine:
                lib.mmq_group(tid, layer.tabs[s % copies].data_ptr(), layer.cnt.data_ptr(), 1, n_tok, mine, cols, layer.x8.data_ptr(),
                              layer.dx.data_ptr(), layer.sx.data_ptr(), layer.zero.data_ptr(), y.data_ptr(), layer.zero.data_ptr(), mine, stream)
            b.record()
        torch.cuda.synchronize()
        us_kernel = float(np.median([a.elapsed_time(b) for a, b in ev[4:]])) * 1e3
    t_res, t_ee = float(np.median(t_regions)), float(np.median(t_e2e))
    if lib.mmq_status():
        raise SystemExit("bench: a bounded wait ran out")
    if rank != 0:
        return
    tf_peak, kind = measured_tflops()
    ops = 2.0 * mine * cols * n_tok
    # the CPU arm: the scalar restatement of the product on a sample of rows, scaled to the matrix
    t0 = time.perf_counter()
    sample_rows = 8
    hx8, hdx, hsx = orc.mmq_x8_rows(hx[0], np.arange(n_tok, dtype=np.int32), cols)
    orc.mmq_rows(np.ascontiguousarray(w.reshape(rows, nb_all // rows)[:sample_rows]).reshape(-1), sample_rows, cols, hx8, hdx, hsx, 0, n_tok)
    cpu_s = (time.perf_counter() - t0) * rows / sample_rows
    line = {"metric": "prefill_tokens_per_s", "value": n_tok * args.steps / t_res, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": 1e3 * t_res / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "int8xint8->f32", "data": "synthetic",
            "config": {"workload": cfg["name"], "format": cfg["type"], "rows": rows, "cols": cols, "tokens": n_tok},
            "run": {"parallelism": "rows%d: a rank a slice of whole 128-row tiles (rank 0: rows %d-%d), every rank rounds all the tokens; no collective" % (world, r0, r1),
                    "cold_cache": "%d copies of the slice's %.1f MB cycled" % (copies, nb_all * mine / rows / 1e6),
                    "timing": "median of %d regions of exactly %d steps, CUDA events, max over ranks; launched on the stream" % (REGIONS, args.steps),
                    "regions_ms_per_step": [1e3 * t / args.steps for t in t_regions],
                    "parity": "every rank: 64 sampled rows of its slice x all tokens bit-equal to the CPU checker (mmq_rows)"},
            "e2e": {"value": n_tok * args.steps / t_ee, "unit": "tokens/s", "h2d_bytes_per_step": int(px[0].numel() * 4),
                    "d2h_bytes_per_step": int(pout.numel() * 4)},
            "gpu_launches": 2 * args.steps,
            "roofline": {"bound": "tensor", "kernel": "mmq_group (q4k_tc_kernel) on rank 0's slice", "achieved": ops / us_kernel / 1e6,
                         "peak": 2 * tf_peak, "unit": "TOP/s", "frac": ops / us_kernel / 1e6 / (2 * tf_peak),
                         "peak_kind": "nominal: twice the %s bf16 burst (no int8 peak measured)" % kind, "traffic": None,
                         "us_per_launch": us_kernel, "algorithmic_ops_per_launch": ops},
            "cpu_baseline": {"value": n_tok / cpu_s, "unit": "tokens/s", "cores": 1, "kind": "port",
                             "sample": "%d rows x all tokens through the scalar restatement, scaled to %d rows" % (sample_rows, rows)},
            "clocks": clocks.summary()}
    print(json.dumps(line), flush=True)


def run_f32_or_f16(args, cfg, lib, dev):
    """The MXFP4 experts (128 of them, top-4) on one GPU: 32 tokens through the F32 lane (q4x_route + lane_ffn_f32: an
    expert read once for its tokens by mv_group_tok - the reference's decode path for a type without an int8 form), or
    2048 tokens through the grouped f16 tensor-core product (q4x_moe). Same contract as the default workload's line."""
    import torch

    from libosmos_b200 import api, synth, workloads
    from oracle.oracle import Oracle
    if dist_env()[1] > 1:
        raise SystemExit("bench: workload %s runs on one GPU" % cfg["name"])
    tid, n_tok, dim, ff, k, n_exp = synth.TYPE_ID[cfg["type"]], cfg["n_tok"], cfg["dim"], cfg["ff"], cfg["k"], cfg["n_exp"]
    picks = n_tok * k
    host = workloads.moe_layer_host(cfg)
    per = workloads.moe_expert_bytes(cfg)
    copies = 2
    first = [torch.from_numpy(h).to(dev) for h in host]
    weights = [first] + [[t.clone() for t in first] for _ in range(copies - 1)]
    f32 = cfg["path"] == "f32_lane"
    layers = []
    for w in weights:
        if f32:
            L = api.LaneLayer(tid, tid, dim, ff, n_exp, k, cfg["lim"], api.LaneExperts())
            for j in range(3):
                L.experts.base[j], L.experts.bytes[j] = w[j].data_ptr(), per[j]
        else:
            L = api.Q4xMoeLayer()
            L.dim, L.ff, L.n_exp, L.k = dim, ff, n_exp, k
            for j in range(3):
                L.type[j], L.base[j], L.bytes[j] = tid, w[j].data_ptr(), per[j]
        layers.append(L)
    if f32:
        nbytes, scratch = lib.lane_f32_scratch_bytes(layers[0], n_tok), api.LaneScratchF32()
        bind = lib.lane_f32_scratch_bind
    else:
        nbytes, scratch = lib.q4x_moe_scratch_bytes(layers[0], n_tok), api.Q4xMoeScratch()
        bind = lib.q4x_moe_scratch_bind
    assert nbytes, "the driver refused the layer"
    mem = torch.zeros(nbytes + 256, dtype=torch.uint8, device=dev)
    assert bind(layers[0], n_tok, (mem.data_ptr() + 255) // 256 * 256, nbytes, scratch)
    ids = torch.zeros(picks, dtype=torch.int32, device=dev)
    wts = torch.zeros(picks, dtype=torch.float32, device=dev)
    rows = torch.zeros(picks, dtype=torch.int32, device=dev)
    zeros = torch.zeros((n_tok, dim), dtype=torch.float32, device=dev)  # q4x_moe's shared-expert term: none here
    zlog = torch.zeros(n_tok, dtype=torch.float32, device=dev)
    n_inputs = 8 if f32 else 4
    hx, hl = zip(*[workloads.moe_inputs_host(cfg, s) for s in range(n_inputs)])
    dx = [torch.from_numpy(a).to(dev) for a in hx]
    dl = [torch.from_numpy(a).to(dev) for a in hl]
    px = [torch.from_numpy(a).pin_memory() for a in hx]
    pl = [torch.from_numpy(a).pin_memory() for a in hl]
    out = torch.empty((n_tok, dim), dtype=torch.float32, device=dev)
    pout = torch.empty((n_tok, dim), dtype=torch.float32).pin_memory()
    stream = torch.cuda.current_stream().cuda_stream

    def step(x, logits, o, copy, st):
        L = layers[copy % copies]
        if f32:
            ok = lib.q4x_route(logits.data_ptr(), n_tok, n_exp, k, ids.data_ptr(), wts.data_ptr(), rows.data_ptr(), st) and \
                lib.lane_ffn_f32(L, scratch, x.data_ptr(), ids.data_ptr(), wts.data_ptr(), n_tok, None, o.data_ptr(), st)
        else:
            ok = lib.q4x_moe(L, scratch, x.data_ptr(), logits.data_ptr(), zeros.data_ptr(), zlog.data_ptr(), n_tok, o.data_ptr(), st)
        if not ok:
            raise RuntimeError("libosmos_b200 refused a call of the step")

    # parity first, on the step's first tokens
    orc = Oracle()
    step(dx[0], dl[0], out, 0, stream)
    torch.cuda.synchronize()
    want_ids, want_w = workloads.softmax_topk(hl[0], k)
    ns = 8 if f32 else 4
    got = out.cpu().numpy()[:ns]
    if f32:
        gi, gw = ids.cpu().numpy().reshape(n_tok, k), wts.cpu().numpy().reshape(n_tok, k)
        ok = np.array_equal(gi, want_ids) and np.allclose(gw, want_w, rtol=1e-5, atol=0)
        want = np.zeros((ns, dim), np.float32)
        for t in range(ns):
            acc = np.zeros(dim, np.float32)
            for j in np.argsort(gi[t], kind="stable"):
                e = int(gi[t, j])
                p = [host[m][e * per[m]:(e + 1) * per[m]] for m in range(3)]
                g = orc.mv_rows(tid, p[0], ff, dim, hx[0][t:t + 1])
                u = orc.mv_rows(tid, p[1], ff, dim, hx[0][t:t + 1])
                acc = (acc + orc.mv_rows(tid, p[2], dim, ff, orc.swiglu_lane(g, u, cfg["lim"], gw[t, j:j + 1]))[0]).astype(np.float32)
            want[t] = acc
        ok = ok and np.array_equal(got.view(np.uint32), want.view(np.uint32))
        parity = "the first %d tokens of step 0 bit-equal to the CPU checker (the F32 matvec's order, the lane's activation)" % ns
    else:
        ref = np.zeros((ns, dim))
        for t in range(ns):
            x16 = hx[0][t].astype(np.float16).astype(np.float64)
            for j in range(k):
                e = int(want_ids[t, j])
                wf = [orc.dequant(tid, host[m][e * per[m]:(e + 1) * per[m]], r * c).reshape(r, c).astype(np.float64)
                      for m, (r, c) in enumerate(((ff, dim), (ff, dim), (dim, ff)))]
                g, u = wf[0] @ x16, wf[1] @ x16
                h16 = (g / (1 + np.exp(-g)) * u).astype(np.float16).astype(np.float64)
                ref[t] += float(want_w[t, j]) * (wf[2] @ h16)
        err = np.abs(got - ref).max() / np.abs(ref).max()
        ok = bool(err < 1e-3)
        parity = "the first %d tokens of step 0 within 1e-3 (of the largest value) of a float64 model over f16-rounded activations: %.2e" % (ns, err)
    if not ok:
        raise SystemExit("bench: the GPU layer's output fails its check against the CPU checker - not timing a wrong result")
    distinct = [len(np.unique(workloads.softmax_topk(l, k)[0])) for l in hl]

    def timed(fn, steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for s in range(steps):
            fn(s)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / 1e3

    def resident(s):
        step(dx[s % n_inputs], dl[s % n_inputs], out, s, stream)

    bx, bl = torch.empty_like(dx[0]), torch.empty_like(dl[0])

    def end_to_end(s):  # host buffers in, host buffer out, every step
        bx.copy_(px[s % n_inputs], non_blocking=True)
        bl.copy_(pl[s % n_inputs], non_blocking=True)
        step(bx, bl, out, s, stream)
        pout.copy_(out, non_blocking=True)

    for s in range(args.warmup):
        resident(s), end_to_end(s)
    torch.cuda.synchronize()
    graphs, side = [], torch.cuda.Stream()
    for s in range(n_inputs):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            step(dx[s], dl[s], out, s, side.cuda_stream)
        graphs.append(g)

    def resident_graph(s):
        graphs[s % n_inputs].replay()

    with ClockSampler(dev.index) as clocks:
        n_warm = int(min(20000, max(args.steps, 1.0 / (timed(resident_graph, args.steps) / args.steps))))
        for s in range(n_warm):
            resident_graph(s)
        torch.cuda.synchronize()
        t_regions = [timed(resident_graph, args.steps) for _ in range(REGIONS)]
        t_stream = [timed(resident, args.steps) for _ in range(REGIONS)]
        t_e2e = [timed(end_to_end, args.steps) for _ in range(REGIONS)]
    t_res, t_str, t_ee = float(np.median(t_regions)), float(np.median(t_stream)), float(np.median(t_e2e))
    if lib.mv_status() or lib.mm_status():
        raise SystemExit("bench: a bounded wait ran out")
    peak, peak_kind = measured_peaks()
    alg = float(np.mean(distinct)) * sum(per)
    achieved = alg / (t_res / args.steps) / 1e9
    roof = {"bound": "hbm", "kernel": "the whole step (its three expert products: %s)" % ("mv_group_tok x 3" if f32 else "mm_group x 3"),
            "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind, "traffic": None,
            "algorithmic_bytes_per_launch": alg, "us_per_launch": 1e6 * t_res / args.steps}
    if not f32:
        tf, kind = measured_tflops()
        flops = 2.0 * 3 * ff * dim * picks
        roof["tensor"] = {"tflops": flops / (t_res / args.steps) / 1e12, "peak_tflops": tf, "peak_kind": kind + " bf16 burst",
                          "frac": flops / (t_res / args.steps) / 1e12 / tf}
    cpu_tok_s, _, sample = port_tokens_per_s(cfg, host, per)
    line = {"metric": METRIC, "value": n_tok * args.steps / t_res, "unit": UNIT, "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1e3 * t_res / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32" if f32 else "f16xf16->f32", "data": "synthetic", "config": workload_config(cfg),
            "run": {"parallelism": "1 gpu", "launch": "value: CUDA graph replay; the same steps launched on the stream take %.4f ms" % (1e3 * t_str / args.steps),
                    "cold_cache": "%d copies of the layer's %d MB of expert weights cycled; a step touches ~%d MB" % (copies, sum(per) * n_exp // 1000000, int(alg) // 1000000),
                    "timing": "median of %d regions of exactly %d steps, CUDA events" % (REGIONS, args.steps),
                    "regions_ms_per_step": [1e3 * t / args.steps for t in t_regions], "parity": parity,
                    "inputs": "activations are bf16 values held as F32 (the conversion is exact)"},
            "e2e": {"value": n_tok * args.steps / t_ee, "unit": UNIT, "h2d_bytes_per_step": int((px[0].numel() + pl[0].numel()) * 4),
                    "d2h_bytes_per_step": int(pout.numel() * 4)},
            "gpu_launches": (10 if f32 else 13) * args.steps, "roofline": roof,
            "cpu_baseline": {"value": cpu_tok_s, "unit": UNIT, "cores": 1, "kind": "port", "sample": sample},
            "clocks": clocks.summary()}
    print(json.dumps(line), flush=True)


def graph_time(fn, n=64, reps=5):
    """device microseconds a launch: n launches (fn(i, stream)) captured in one CUDA graph, replayed reps times"""
    import torch
    for i in range(3):
        assert fn(i, None), "the library refused the call"
    torch.cuda.synchronize()
    g, st = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    with torch.cuda.graph(g, stream=st):
        for i in range(n):
            assert fn(i, st.cuda_stream)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (n * reps)


def matvec_leg(lib, dev, peak):
    """The decode matvec's weight-GB/s, the second figure beside the headline: the reference's dense decode matrix (Q4_0
    6144 x 2048, 7 MB: a launch is latency-bound), the same rows eight times over, and a 302 MB matrix (131072 x 4096:
    what a launch reaches once its start and end no longer count), each through the int8 lane form (q8_run: x rounded
    once by q8_round) and the F32 form in the reference's order (mv_run). Each case's first launch is compared with the
    CPU checker's bits (a sample of rows for the large matrices) before anything is timed. 64 launches on successive
    cold copies (more than 1 GiB cycled) captured in one CUDA graph, replayed; device time a launch."""
    import torch

    from libosmos_b200 import synth
    from oracle.oracle import Oracle
    orc = Oracle()
    tid = synth.TYPE_ID["Q4_0"]
    out = {"format": "Q4_0", "tokens": 1, "timing": "64 launches on successive copies (> 1 GiB cycled) in a CUDA graph, replayed 5 times",
           "parity": "first launch of every case bit-equal to the CPU checker (all rows at 6144, 4096 sampled rows above)",
           "cases": []}
    for rows, cols in ((6144, 2048), (49152, 2048), (131072, 4096)):
        w = synth.random_tensor(tid, rows, cols, synth.rng_for(1, tid, rows))
        nb = int(w.size)
        copies = max(2, int(1.1 * 2 ** 30 // nb) + 1)
        pool = torch.from_numpy(w).to(dev).repeat(copies)
        xh = synth.rng_for(5, rows).standard_normal((1, cols)).astype(np.float32)
        x = torch.from_numpy(xh).to(dev)
        q = torch.zeros(1, cols, dtype=torch.int8, device=dev)
        d = torch.zeros(1, cols // 32, device=dev)
        y = torch.empty(1, rows, device=dev)
        assert lib.q8_round(x.data_ptr(), 1, cols, cols, q.data_ptr(), d.data_ptr(), None)
        calls = {
            "q8_run": lambda i, st: lib.q8_run(tid, pool.data_ptr() + (i % copies) * nb, rows, cols, q.data_ptr(),
                                               d.data_ptr(), 1, y.data_ptr(), rows, st),
            "mv_run": lambda i, st: lib.mv_run(tid, pool.data_ptr() + (i % copies) * nb, rows, cols, x.data_ptr(), 1,
                                               y.data_ptr(), st),
        }
        # the checker's rows: all of a small matrix, else a seeded sample
        pick = np.arange(rows) if rows <= 8192 else np.sort(synth.rng_for(6, rows).choice(rows, 4096, replace=False))
        rb = nb // rows
        wsel = np.ascontiguousarray(w.reshape(rows, rb)[pick]).reshape(-1)
        qh, dh = orc.q8_round(xh)
        want = {"q8_run": orc.q8_rows(tid, wsel, len(pick), cols, qh, dh), "mv_run": orc.mv_rows(tid, wsel, len(pick), cols, xh)}
        case = {"rows": rows, "cols": cols, "weight_bytes": nb}
        for name, fn in calls.items():
            y.zero_()
            assert fn(1, None)
            torch.cuda.synchronize()
            if not np.array_equal(y.cpu().numpy()[:, pick].view(np.uint32), want[name].view(np.uint32)):
                raise SystemExit("bench: %s at %dx%d differs from the CPU checker's bits" % (name, rows, cols))
            us = graph_time(fn)
            case[name] = {"us_per_launch": us, "weight_gbs": nb / us / 1e3, "frac_of_hbm_peak": nb / us / 1e3 / peak}
        out["cases"].append(case)
        del pool
    if lib.q8_status() or lib.mv_status():
        raise SystemExit("bench: a staged matvec kernel reported a copy that never landed")
    return out


def prefill_leg(lib, dev):
    """The prefill product beside the headline: a Q4_K 4096 x 4096 matrix over 512 tokens through the int8 product in
    the reference's order of sums (mmq_group, bit-exact) and through the f16 product (mm_run), and the f16 product
    again at 2048 tokens. Before timing, mmq_group's output is compared bit for bit with the CPU checker on 256 sampled
    rows x all tokens, and mm_run's with a double-precision sum over the f16-rounded operands on the same rows, within
    the reference test's bound. Activations converted once, outside the timed launches; 64 launches on successive cold
    copies of the matrix in one CUDA graph, replayed; device time a launch. The int8 fraction is of twice the measured
    bf16 burst (the nominal ratio of the int8 to the bf16 tensor rate; no int8 peak is measured here)."""
    import torch

    from libosmos_b200 import synth
    from oracle.oracle import Oracle
    orc = Oracle()
    tf_peak, kind = measured_tflops()
    tid, rows, cols = synth.TYPE_ID["Q4_K"], 4096, 4096
    w = synth.random_tensor(tid, rows, cols, synth.rng_for(2, tid, rows))
    nb = int(w.size)
    copies = 24  # 226 MB cycled: more than the 126 MB L2
    pool = torch.from_numpy(w).to(dev).repeat(copies)
    pick = np.sort(synth.rng_for(7).choice(rows, 256, replace=False))
    rb = nb // rows
    wsel = np.ascontiguousarray(w.reshape(rows, rb)[pick]).reshape(-1)
    wf = orc.dequant(tid, wsel, len(pick) * cols).reshape(len(pick), cols)
    out = {"format": "Q4_K", "rows": rows, "cols": cols, "peak_tflops": tf_peak, "peak_kind": kind,
           "int8_peak_tops": 2 * tf_peak, "int8_peak_kind": "nominal: twice the %s bf16 burst" % kind,
           "parity": "mmq_group bit-equal to the CPU checker, mm_run within (cols/16+20) 2^-24 sum|w16 x16| of a float64 sum, 256 sampled rows x all tokens",
           "cases": []}
    for op, tokens in (("mmq_group", 512), ("mm_run", 512), ("mm_run", 2048)):
        n16 = (tokens + 15) // 16 * 16
        xh = synth.rng_for(8, tokens).standard_normal((tokens, cols)).astype(np.float32)
        x = torch.from_numpy(xh).to(dev)
        y = torch.zeros(tokens, rows, device=dev)
        if op == "mm_run":
            x16 = torch.zeros(n16 * cols, dtype=torch.float16, device=dev)
            flag = torch.zeros(1, dtype=torch.int32, device=dev)
            assert lib.mm_x16(x.data_ptr(), cols, tokens, cols, x16.data_ptr(), flag.data_ptr(), None)
            fn = lambda i, st: lib.mm_run(tid, pool.data_ptr() + (i % copies) * nb, rows, cols, x16.data_ptr(), tokens,
                                          y.data_ptr(), rows, st)
        else:
            idx = torch.arange(tokens, dtype=torch.int32, device=dev)
            x8 = torch.zeros(n16 * cols, dtype=torch.int8, device=dev)
            dx = torch.zeros(n16 * cols // 32, device=dev)
            sx = torch.zeros_like(dx)
            assert lib.mmq_x8_rows(x.data_ptr(), cols, idx.data_ptr(), tokens, cols, x8.data_ptr(), dx.data_ptr(),
                                   sx.data_ptr(), None)
            tabs = [torch.tensor([pool.data_ptr() + c * nb], dtype=torch.int64, device=dev) for c in range(copies)]
            cnt = torch.tensor([tokens], dtype=torch.int32, device=dev)
            zero = torch.zeros(1, dtype=torch.int32, device=dev)
            fn = lambda i, st: lib.mmq_group(tid, tabs[i % copies].data_ptr(), cnt.data_ptr(), 1, tokens, rows, cols,
                                             x8.data_ptr(), dx.data_ptr(), sx.data_ptr(), zero.data_ptr(), y.data_ptr(),
                                             zero.data_ptr(), rows, st)
        assert fn(1, None)
        torch.cuda.synchronize()
        got = y.cpu().numpy()[:, pick]
        if op == "mmq_group":
            hx8, hdx, hsx = orc.mmq_x8_rows(xh, np.arange(tokens, dtype=np.int32), cols)
            want = orc.mmq_rows(wsel, len(pick), cols, hx8, hdx, hsx, 0, tokens)
            good = np.array_equal(got.view(np.uint32), want.view(np.uint32))
        else:
            w16 = wf.astype(np.float16).astype(np.float64)
            h16 = xh.astype(np.float16).astype(np.float64)
            want = h16 @ w16.T
            bound = (cols / 16 + 20) * 2.0 ** -24 * (np.abs(h16) @ np.abs(w16).T)
            good = bool((np.abs(got.astype(np.float64) - want) <= bound).all())
        if not good:
            raise SystemExit("bench: %s at %d tokens fails its check against the CPU checker" % (op, tokens))
        us = graph_time(fn)
        tf = 2.0 * rows * cols * tokens / us / 1e6
        case = {"op": op, "tokens": tokens, "us_per_launch": us, "tflops": tf, "tokens_per_s": tokens / us * 1e6}
        if op == "mmq_group":
            case["frac_of_int8_peak"], case["peak_kind"] = tf / (2 * tf_peak), out["int8_peak_kind"]
        else:
            case["frac_of_bf16_peak"] = tf / tf_peak
        out["cases"].append(case)
    if lib.mm_status() or lib.mmq_status():
        raise SystemExit("bench: a tensor-core product reported a wait that ran out")
    return out


# ---------------------------------------------------------------------------------------------------------------------
# one kernel alone (the per-kernel counterpart of the step; the reference keeps such sweeps under tools/bench/)
# ---------------------------------------------------------------------------------------------------------------------
def run_kernel(args):
    """python bench.py --kernel q8_run Q4_0 49152 2048              one token, graph-timed
       python bench.py --kernel mv_run Q8_0 6144 2048 --tokens 2
       python bench.py --kernel q8_run Q4_0 49152 2048 --plain 4    four plain launches, nothing timed (for a profiler)
       python bench.py --kernel mm_run Q4_K 4096 4096 --tokens 512  the f16 prefill product (x16 made once)
       python bench.py --kernel mm_fp4 NVFP4 17408 5120 --tokens 2048   W4A4: quantization + product a launch
       python bench.py --kernel mm_fp4_only NVFP4 17408 5120 --tokens 2048   the product alone (--generic: the f16 route)
       python bench.py --kernel mm_mxfp4 MXFP4 16384 4096 --tokens 2048  W4A4 on MXFP4: rounding + product a launch
       python bench.py --kernel mmq_group Q4_K 4096 4096 --tokens 512   the int8 prefill product (x8 made once)
    64 launches on successive cold copies of the matrix (more than 1 GiB cycled) in one CUDA graph, replayed 5 times."""
    import torch

    import libosmos_b200
    from libosmos_b200 import synth
    op, tname, rows, cols = args.kernel[0], args.kernel[1], int(args.kernel[2]), int(args.kernel[3])
    lib = libosmos_b200.load()
    dev = torch.device("cuda", 0)
    tid = synth.TYPE_ID[tname]
    tokens = args.tokens
    w = synth.random_tensor(tid, rows, cols, synth.rng_for(1, tid, rows))
    nb = int(w.size)
    copies = 4 if args.plain else max(2, int(1.1 * 2 ** 30 // nb) + 1)
    pool = torch.from_numpy(w).to(dev).repeat(copies)
    x = torch.randn(tokens, cols, device=dev, generator=torch.Generator(device=dev).manual_seed(1017))
    q = torch.zeros(tokens, cols, dtype=torch.int8, device=dev)
    d = torch.zeros(tokens, cols // 32, device=dev)
    y = torch.empty(tokens, rows, device=dev)
    if args.generic:
        lib.mv_set_staged(0), lib.q8_set_staged(0)
    assert lib.q8_round(x.data_ptr(), tokens, cols, cols, q.data_ptr(), d.data_ptr(), None)
    flops = None
    if op == "mm_fp4":  # the W4A4 step: the activations' quantization and the product (TYPE must be NVFP4)
        flops = 2.0 * rows * cols * tokens
        xq = torch.zeros(tokens, cols // 2, dtype=torch.uint8, device=dev)
        xsc = torch.zeros(tokens, cols // 16, dtype=torch.uint8, device=dev)
        fn = lambda i, st: (lib.mm_fp4_act(x.data_ptr(), cols, tokens, cols, 0.5, xq.data_ptr(), xsc.data_ptr(), st)
                            and lib.mm_fp4(pool.data_ptr() + (i % copies) * nb, rows, cols, xq.data_ptr(),
                                           xsc.data_ptr(), tokens, 1.0, y.data_ptr(), rows, st))
    elif op == "mm_mxfp4":  # W4A4 on MXFP4 (TYPE must be MXFP4): the activations' rounding and the product a launch
        flops = 2.0 * rows * cols * tokens
        pk = torch.zeros(tokens * (cols // 2 + cols // 32), dtype=torch.uint8, device=dev)
        xr = x.clone()
        fn = lambda i, st: (lib.ops_fp4_round(xr.data_ptr(), tokens * cols, 32, False, pk.data_ptr(), cols, st)
                            and lib.mm_mxfp4(pool.data_ptr() + (i % copies) * nb, rows, cols, pk.data_ptr(), tokens, 1.0,
                                             y.data_ptr(), rows, st))
    elif op == "mm_mxfp4_only":  # the MXFP4 W4A4 product alone: the activations rounded once, outside
        flops = 2.0 * rows * cols * tokens
        pk = torch.zeros(tokens * (cols // 2 + cols // 32), dtype=torch.uint8, device=dev)
        assert lib.ops_fp4_round(x.clone().data_ptr(), tokens * cols, 32, False, pk.data_ptr(), cols, None)
        fn = lambda i, st: lib.mm_mxfp4(pool.data_ptr() + (i % copies) * nb, rows, cols, pk.data_ptr(), tokens, 1.0,
                                        y.data_ptr(), rows, st)
    elif op == "mm_fp4_only":  # the W4A4 product alone (TYPE NVFP4): the activations quantized once, outside
        flops = 2.0 * rows * cols * tokens
        xq = torch.zeros(tokens, cols // 2, dtype=torch.uint8, device=dev)
        xsc = torch.zeros(tokens, cols // 16, dtype=torch.uint8, device=dev)
        assert lib.mm_fp4_act(x.data_ptr(), cols, tokens, cols, 0.5, xq.data_ptr(), xsc.data_ptr(), None)
        if args.generic:
            lib.mm_fp4_set_tensor(0)
        fn = lambda i, st: lib.mm_fp4(pool.data_ptr() + (i % copies) * nb, rows, cols, xq.data_ptr(), xsc.data_ptr(), tokens,
                                      1.0, y.data_ptr(), rows, st)
    elif op in ("mm_run", "mmq_group"):
        n16 = (tokens + 15) // 16 * 16
        flops = 2.0 * rows * cols * tokens
        if op == "mm_run":
            x16 = torch.zeros(n16 * cols, dtype=torch.float16, device=dev)
            flag = torch.zeros(1, dtype=torch.int32, device=dev)
            assert lib.mm_x16(x.data_ptr(), cols, tokens, cols, x16.data_ptr(), flag.data_ptr(), None)
            fn = lambda i, st: lib.mm_run(tid, pool.data_ptr() + (i % copies) * nb, rows, cols, x16.data_ptr(),
                                          tokens, y.data_ptr(), rows, st)
        else:
            idx = torch.arange(tokens, dtype=torch.int32, device=dev)
            x8 = torch.zeros(n16 * cols, dtype=torch.int8, device=dev)
            dx = torch.zeros(n16 * cols // 32, device=dev)
            sx = torch.zeros_like(dx)
            assert lib.mmq_x8_rows(x.data_ptr(), cols, idx.data_ptr(), tokens, cols, x8.data_ptr(), dx.data_ptr(), sx.data_ptr(), None)
            tabs = [torch.tensor([pool.data_ptr() + c * nb], dtype=torch.int64, device=dev) for c in range(copies)]
            cnt = torch.tensor([tokens], dtype=torch.int32, device=dev)
            zero = torch.zeros(1, dtype=torch.int32, device=dev)
            fn = lambda i, st: lib.mmq_group(tid, tabs[i % copies].data_ptr(), cnt.data_ptr(), 1, tokens, rows, cols,
                                             x8.data_ptr(), dx.data_ptr(), sx.data_ptr(), zero.data_ptr(), y.data_ptr(),
                                             zero.data_ptr(), rows, st)
    elif op == "q8_run":
        fn = lambda i, st: lib.q8_run(tid, pool.data_ptr() + (i % copies) * nb, rows, cols, q.data_ptr(), d.data_ptr(),
                                      tokens, y.data_ptr(), rows, st)
    elif op == "mv_run":
        fn = lambda i, st: lib.mv_run(tid, pool.data_ptr() + (i % copies) * nb, rows, cols, x.data_ptr(), tokens, y.data_ptr(), st)
    else:
        raise SystemExit("unknown kernel %r" % op)
    if args.plain:
        for i in range(args.plain):
            if not fn(i, None):
                raise SystemExit("the library refused the call")
        torch.cuda.synchronize()
        print("%d launches, status %d" % (args.plain, lib.q8_status() | lib.mv_status() | lib.mm_status() | lib.mmq_status()))
        return
    us = graph_time(fn)
    print(json.dumps({"op": op, "type": tname, "rows": rows, "cols": cols, "tokens": tokens,
                      "kernels": "generic" if args.generic else "default", "us_per_launch": us, "weight_bytes": nb,
                      "weight_gbs": nb / us / 1e3, "tflops": None if flops is None else flops / us / 1e6,
                      "status": lib.q8_status() | lib.mv_status() | lib.mm_status() | lib.mmq_status()}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="moe_iq3xxs_512e_top10")
    ap.add_argument("--kernel", nargs=4, metavar=("OP", "TYPE", "ROWS", "COLS"), help="time one kernel alone")
    ap.add_argument("--tokens", type=int, default=1)
    ap.add_argument("--plain", type=int, default=0, help="--kernel: this many plain launches on 4 copies instead of timing")
    ap.add_argument("--generic", action="store_true", help="--kernel: the generic kernels")
    ap.add_argument("--profile", action="store_true",
                    help="for a profiler: the parity-checked step, then warmup + steps plain steps on the stream; nothing is timed")
    args = ap.parse_args()
    if args.kernel:
        return run_kernel(args)
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
