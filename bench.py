#!/usr/bin/env python
"""Benchmark of the quantized-weight matrix path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (config.workload): the Qwen-style MoE FFN layer in IQ3_XXS - 512 experts, 64 tokens routed top-10, hidden
2048, expert width 512 - run as the int8 lane: softmax router, activations rounded to int8 per 32, fused gate + up +
activation over the picked experts, the activations rounded again, down, each token's rows summed in ascending
expert id. A step is one pass of the layer over one 64-token batch; successive steps use successive cold copies of
the layer's weights (a model's next layer), 616 MB each, so no step finds its weights in L2.

Prints ONE JSON line: tokens/s through the layer (value: inputs resident in HBM; e2e: host buffers in, host
buffer out through the C ABI), the dominant kernel's weight-GB/s against the measured HBM peak (roofline), and the
reference's own CPU lane on this host's cores beside it (cpu_baseline). `--impl reference` times only that CPU
path.
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


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi's SM clock and throttle reasons sampled while the timed region runs"""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.index, self.lines, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
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


# ---------------------------------------------------------------------------------------------------------------------
# the reference arm: the reference's CPU lane (oracle/_ref, its sources compiled unmodified) or, where that library
# is missing or this CPU lacks its AVX-512 VNNI kernels, this repository's scalar restatement of it
# ---------------------------------------------------------------------------------------------------------------------
def cpu_step_inputs(cfg, step):
    from libosmos_b200 import workloads
    x, logits = workloads.moe_inputs_host(cfg, step)
    ids, wts = workloads.softmax_topk(logits, cfg["k"])
    # rows by (expert, pick): the lane's layout (a row an expert's copy of its token's input)
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


class CpuArm:
    def __init__(self, cfg, host_tensors, threads=None):
        from libosmos_b200 import synth, workloads
        from oracle.oracle import Oracle, Reference
        self.cfg, self.host = cfg, host_tensors
        self.tid = synth.TYPE_ID[cfg["type"]]
        self.per = workloads.moe_expert_bytes(cfg)
        self.cores = os.cpu_count() or 1
        self.kind = "reference" if Reference.available() else "port"
        if self.kind == "reference":
            self.ref = Reference()
            self.threads = min(64, threads or self.cores)
            self.pool = self.ref.lib.cpu_lane_create(self.threads, None, cfg["n_tok"] * cfg["k"], cfg["dim"], cfg["ff"])
            if not self.pool:
                self.kind = "port"
        if self.kind == "port":
            self.oracle, self.threads = Oracle(), 1

    def parts(self, e):
        return [self.host[m][e * self.per[m]:(e + 1) * self.per[m]] for m in range(3)]

    def run(self, xr, sc, experts, limit_rows=None):
        """one step's expert FFN rows on the CPU; returns (seconds, rows done, y)"""
        cfg = self.cfg
        if self.kind == "reference":
            ex = [tuple(self.parts(e)) + (r0, c) for e, r0, c in experts]
            t0 = time.perf_counter()
            y = self.ref.lane_ffn(self.threads, self.tid, self.tid, cfg["dim"], cfg["ff"], cfg["lim"], xr, sc, ex, pool=self.pool)
            dt = time.perf_counter() - t0
            assert y is not None, "the reference's cpu_lane refused the job"
            return dt, xr.shape[0], y
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


def run_reference(args):
    from libosmos_b200 import workloads
    rank, world, _ = dist_env()
    if rank != 0:
        return
    cfg = workloads.MOE_IQ3
    arm = CpuArm(cfg, workloads.moe_layer_host(cfg))
    limit = None if arm.kind == "reference" else 24  # the scalar port: a bounded sample of a step's rows
    times, rows = [], 0
    for s in range(args.warmup + args.steps):
        xr, sc, experts, _ = cpu_step_inputs(cfg, s)
        dt, done, _ = arm.run(xr, sc, experts, limit)
        if s >= args.warmup:
            times.append(dt), (rows := rows + done)
    tok_s = rows / cfg["k"] / sum(times)
    sample = ("full steps of %d tokens (%d expert rows each)" % (cfg["n_tok"], cfg["n_tok"] * cfg["k"])
              if limit is None else "the first %d expert rows of each step, scaled to tokens" % limit)
    line = {"impl": "reference", "metric": METRIC, "value": tok_s, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1e3 * sum(times) / len(times), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "int8xint8->f32", "data": "synthetic",
            "config": {"workload": cfg["name"], "tokens": cfg["n_tok"], "experts": cfg["n_exp"], "top_k": cfg["k"],
                       "hidden": cfg["dim"], "expert_ff": cfg["ff"], "format": cfg["type"]},
            "cpu_baseline": {"value": tok_s, "unit": UNIT, "cores": arm.threads, "kind": arm.kind, "sample": sample},
            "e2e": {"value": tok_s, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------------------------------
def run_ours(args):
    import torch

    import libosmos_b200
    from libosmos_b200 import runner, workloads
    rank, world, local = dist_env()
    assert world == args.gpus or world == 1, "launch N ranks for --gpus N"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
        from libosmos_b200 import ep
        return ep.run_bench(args, rank, world, dev, METRIC, UNIT, ClockSampler, measured_peaks)

    lib = libosmos_b200.load()
    cfg = workloads.MOE_IQ3
    n_tok, dim = cfg["n_tok"], cfg["dim"]
    host = workloads.moe_layer_host(cfg)
    copies = 4
    layer = runner.MoeLane(lib, cfg, dev, copies=copies, host_tensors=host)
    n_inputs = 8
    hx, hl = zip(*[workloads.moe_inputs_host(cfg, s) for s in range(n_inputs)])
    dx = [torch.from_numpy(a).to(dev) for a in hx]
    dl = [torch.from_numpy(a).to(dev) for a in hl]
    px = [torch.from_numpy(a).pin_memory() for a in hx]
    pl = [torch.from_numpy(a).pin_memory() for a in hl]
    out = torch.empty((n_tok, dim), dtype=torch.float32, device=dev)
    stream = torch.cuda.current_stream().cuda_stream

    # parity first: step 0 against the CPU oracle on a few tokens (the GPU tests hold the rest)
    from oracle.oracle import Oracle
    layer.step(dx[0], dl[0], out, n_tok, 0, stream)
    torch.cuda.synchronize()
    ids = layer.ids.cpu().numpy().reshape(n_tok, cfg["k"])
    wts = layer.wts.cpu().numpy().reshape(n_tok, cfg["k"])
    want = runner.moe_oracle(Oracle(), cfg, host, hx[0][:2], ids[:2], wts[:2])
    got = out.cpu().numpy()[:2]
    if not np.array_equal(got.view(np.uint32), want.view(np.uint32)):
        raise SystemExit("bench: the GPU layer's output differs from the CPU oracle's bits - not timing a wrong result")
    distinct = [len(np.unique(workloads.softmax_topk(l, cfg["k"])[0])) for l in hl]

    def timed(fn, steps, drain=None):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for s in range(steps):
            fn(s)
        if drain:
            drain()  # the side streams' last copies are inside the timed region
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / 1e3

    def resident(s):
        layer.step(dx[s % n_inputs], dl[s % n_inputs], out, n_tok, s % copies, stream)

    # end to end: every step's inputs come from pinned host memory and its output goes back to it, the copies on
    # their own streams so that step s + 1's inputs and step s - 1's output move while step s computes (two buffers
    # of each; events order a buffer's copy, its use and its reuse)
    cin, cout = torch.cuda.Stream(), torch.cuda.Stream()
    main = torch.cuda.current_stream()
    bx = [torch.empty_like(dx[0]) for _ in range(2)]
    bl = [torch.empty_like(dl[0]) for _ in range(2)]
    bo = [torch.empty_like(out) for _ in range(2)]
    bp = [torch.empty((n_tok, dim), dtype=torch.float32).pin_memory() for _ in range(2)]
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
        layer.step(bx[b], bl[b], bo[b], n_tok, s % copies, stream)
        used[b].record(main)
        cout.wait_event(used[b])
        with torch.cuda.stream(cout):
            bp[b].copy_(bo[b], non_blocking=True)
            out_done[b].record(cout)

    def e2e_drain():
        main.wait_stream(cin), main.wait_stream(cout)

    for s in range(args.warmup):
        resident(s), end_to_end(s)
    # the resident step as a user of the C ABI would run a decode loop: captured once per (input, weight copy) pair in
    # a CUDA graph and replayed - the same seven launches, without the host's launch gaps
    torch.cuda.synchronize()
    graphs, side = [], torch.cuda.Stream()
    for s in range(n_inputs):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            layer.step(dx[s], dl[s], out, n_tok, s % copies, side.cuda_stream)
        graphs.append(g)

    def resident_graph(s):
        graphs[s % n_inputs].replay()

    for s in range(args.warmup):
        resident_graph(s)
    torch.cuda.synchronize()
    layer.step(dx[1], dl[1], out, n_tok, 1 % copies, stream)
    torch.cuda.synchronize()
    plain_bits = out.cpu().numpy().view(np.uint32).copy()
    resident_graph(1)
    torch.cuda.synchronize()
    if not np.array_equal(plain_bits, out.cpu().numpy().view(np.uint32)):
        raise SystemExit("bench: the graph-replayed step differs from the stream-launched one")
    with ClockSampler(local) as clocks:
        t_res = timed(resident_graph, args.steps)
        t_res_stream = timed(resident, args.steps)
        t_e2e = timed(end_to_end, args.steps, e2e_drain)
        # the dominant kernel alone: events around q8_gate_up inside the same step
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
        torch.cuda.synchronize()
        for s, (a, b) in enumerate(evs):
            layer.step_timed_gate_up(dx[s % n_inputs], dl[s % n_inputs], out, n_tok, s % copies, a, b, stream)
        torch.cuda.synchronize()
    k_ms = [a.elapsed_time(b) for a, b in evs]
    per = workloads.moe_expert_bytes(cfg)
    alg = [distinct[s % n_inputs] * (per[0] + per[1]) for s in range(args.steps)]
    achieved = float(np.sum(alg) / (np.sum(k_ms) * 1e-3) / 1e9)
    peak, peak_kind = measured_peaks()

    # the CPU baseline beside it: the reference's CPU lane on this host, one to three steps
    cpu = None
    try:
        arm = CpuArm(cfg, host)
        limit = None if arm.kind == "reference" else 24
        tt, rows = 0.0, 0
        for s in range(3 if arm.kind == "reference" else 1):
            xr, sc, experts, _ = cpu_step_inputs(cfg, s)
            dt, done, _ = arm.run(xr, sc, experts, limit)
            if s or arm.kind != "reference":
                tt, rows = tt + dt, rows + done
        cpu = {"value": rows / cfg["k"] / tt, "unit": UNIT, "cores": arm.threads, "kind": arm.kind,
               "sample": "2 full 64-token steps after 1 warm-up" if limit is None else "24 expert rows of one step, scaled"}
    except Exception as e:  # the baseline is reported, never required
        cpu = {"value": None, "unit": UNIT, "cores": 0, "kind": "unavailable", "sample": str(e)[:120]}

    line = {"metric": METRIC, "value": n_tok * args.steps / t_res, "unit": UNIT, "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1e3 * t_res / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "int8xint8->f32", "data": "synthetic",
            "config": {"workload": cfg["name"], "tokens": n_tok, "experts": cfg["n_exp"], "top_k": cfg["k"], "hidden": dim,
                       "expert_ff": cfg["ff"], "format": cfg["type"], "parallelism": "1 gpu",
                       "launch": "value: CUDA graph replay, one graph a (input, weight copy) pair; the same steps launched "
                                 "on the stream take %.4f ms" % (1e3 * t_res_stream / args.steps),
                       "cold_cache": "%d copies of the layer's 616 MB of weights cycled; each step touches ~%d MB > 126 MB L2"
                                     % (copies, int(np.mean(distinct)) * sum(per) // 1000000)},
            "e2e": {"value": n_tok * args.steps / t_e2e, "unit": UNIT,
                    "h2d_bytes_per_step": int(px[0].numel() * 4 + pl[0].numel() * 4), "d2h_bytes_per_step": int(bp[0].numel() * 4)},
            "gpu_launches": layer.kernels_per_step * args.steps,
            "roofline": {"bound": "hbm", "kernel": "q8_gate_up (lane_ring_kernel, IQ3_XXS, fused gate + up + activation)",
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind,
                         "traffic": 296433152, "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one launch "
                         "(step 6's experts: 291.8 MB + 4.7 MB), profiles/lane_ring_rows_iq3xxs_moe.md",
                         "algorithmic_bytes_per_launch": float(np.mean(alg)),
                         "us_per_launch": float(np.mean(k_ms) * 1e3)},
            "cpu_baseline": cpu, "clocks": clocks.summary()}
    try:
        line["matvec"] = matvec_leg(lib, dev, peak)
    except Exception as e:  # a second figure beside the headline: reported, never required
        line["matvec"] = {"unavailable": str(e)[:160]}
    try:
        line["prefill"] = prefill_leg(lib, dev)
    except Exception as e:
        line["prefill"] = {"unavailable": str(e)[:160]}
    print(json.dumps(line), flush=True)


def matvec_leg(lib, dev, peak):
    """The decode matvec's weight-GB/s, the second figure beside the headline: the reference's dense decode matrix (Q4_0
    6144 x 2048, 7 MB: a launch is latency-bound), the same rows eight times over, and a 302 MB matrix (131072 x 4096:
    what a launch reaches once its start and end no longer count), each through the int8 lane
    form (q8_run: x rounded once by q8_round) and the F32 form in the reference's order (mv_run). 64 launches on
    successive cold copies (more than 1 GiB cycled) captured in one CUDA graph, replayed; device time a launch."""
    import torch

    from libosmos_b200 import synth
    tid = synth.TYPE_ID["Q4_0"]
    out = {"format": "Q4_0", "tokens": 1, "timing": "64 launches on successive copies (> 1 GiB cycled) in a CUDA graph, replayed 5 times",
           "cases": []}
    for rows, cols in ((6144, 2048), (49152, 2048), (131072, 4096)):
        w = synth.random_tensor(tid, rows, cols, synth.rng_for(1, tid, rows))
        nb = int(w.size)
        copies = max(2, int(1.1 * 2 ** 30 // nb) + 1)
        pool = torch.from_numpy(w).to(dev).repeat(copies)
        x = torch.randn(1, cols, device=dev)
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
        case = {"rows": rows, "cols": cols, "weight_bytes": nb}
        for name, fn in calls.items():
            for i in range(3):
                assert fn(i, None)
            torch.cuda.synchronize()
            n, reps = 64, 5
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
            us = e0.elapsed_time(e1) * 1e3 / (n * reps)
            case[name] = {"us_per_launch": us, "weight_gbs": nb / us / 1e3, "frac_of_hbm_peak": nb / us / 1e3 / peak}
        out["cases"].append(case)
        del pool
    if lib.q8_status() or lib.mv_status():
        raise SystemExit("bench: a staged matvec kernel reported a copy that never landed")
    return out


def prefill_leg(lib, dev):
    """The prefill product beside the headline: a Q4_K 4096 x 4096 matrix over 512 tokens through the
    int8 product in the reference's order of sums (mmq_group, bit-exact) and through the f16 product (mm_run), and
    the f16 product again at 2048 tokens. Activations converted once, outside the timed launches; 64 launches on
    successive cold copies of the matrix in one CUDA graph, replayed; device time a launch; the fraction is of the
    measured bf16 burst peak."""
    import torch

    from libosmos_b200 import synth
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            tf_peak, kind = float(json.load(f)["bf16_tflops"]), "measured"
    except Exception:
        tf_peak, kind = 1590.0, "fallback"
    tid, rows, cols = synth.TYPE_ID["Q4_K"], 4096, 4096
    w = synth.random_tensor(tid, rows, cols, synth.rng_for(2, tid, rows))
    nb = int(w.size)
    copies = 24  # 226 MB cycled: more than the 126 MB L2
    pool = torch.from_numpy(w).to(dev).repeat(copies)
    out = {"format": "Q4_K", "rows": rows, "cols": cols, "peak_tflops": tf_peak, "peak_kind": kind, "cases": []}
    for op, tokens in (("mmq_group", 512), ("mm_run", 512), ("mm_run", 2048)):
        n16 = (tokens + 15) // 16 * 16
        x = torch.randn(tokens, cols, device=dev)
        y = torch.empty(tokens, rows, device=dev)
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
        for i in range(3):
            assert fn(i, None)
        torch.cuda.synchronize()
        n, reps = 64, 5
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
        us = e0.elapsed_time(e1) * 1e3 / (n * reps)
        tf = 2.0 * rows * cols * tokens / us / 1e6
        out["cases"].append({"op": op, "tokens": tokens, "us_per_launch": us, "tflops": tf, "frac_of_bf16_peak": tf / tf_peak,
                             "tokens_per_s": tokens / us * 1e6})
    if lib.mm_status() or lib.mmq_status():
        raise SystemExit("bench: a tensor-core product reported a wait that ran out")
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
