"""Time one dense matvec entry point on a seeded synthetic matrix: the per-kernel counterpart of bench.py (the
reference keeps such sweeps under tools/bench/).

    python -m libosmos_b200.kbench q8_run Q4_0 49152 2048            # one token, graph-timed
    python -m libosmos_b200.kbench mv_run Q8_0 6144 2048 --tokens 2
    python -m libosmos_b200.kbench q8_run Q4_0 49152 2048 --plain 4  # four plain launches, nothing timed (for a profiler)
    python -m libosmos_b200.kbench mm_run Q4_K 4096 4096 --tokens 512  # the f16 prefill product (x16 made once)
    python -m libosmos_b200.kbench mm_fp4 NVFP4 17408 5120 --tokens 2048  # W4A4: quantization + product a launch
    python -m libosmos_b200.kbench mmq_group Q4_K 4096 4096 --tokens 512  # the int8 prefill product (x8 made once)

Timing: 64 launches on successive cold copies of the matrix (more than 1 GiB cycled, so every launch reads HBM)
captured in one CUDA graph and replayed 5 times; CUDA events around the replays; device time a launch.
"""
import argparse
import json

import numpy as np
import torch

import libosmos_b200
from libosmos_b200 import synth


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("op", choices=["mv_run", "q8_run", "mm_run", "mmq_group", "mm_fp4"])
    ap.add_argument("type")
    ap.add_argument("rows", type=int)
    ap.add_argument("cols", type=int)
    ap.add_argument("--tokens", type=int, default=1)
    ap.add_argument("--plain", type=int, default=0, help="this many plain launches on 4 copies instead of timing")
    ap.add_argument("--generic", action="store_true", help="the generic kernels (mv_set_staged(0), q8_set_staged(0))")
    args = ap.parse_args()
    lib = libosmos_b200.load()
    dev = torch.device("cuda", 0)
    tid = synth.TYPE_ID[args.type]
    w = synth.random_tensor(tid, args.rows, args.cols, synth.rng_for(1, tid, args.rows))
    nb = int(w.size)
    copies = 4 if args.plain else max(2, int(1.1 * 2 ** 30 // nb) + 1)
    pool = torch.from_numpy(w).to(dev).repeat(copies)
    x = torch.randn(args.tokens, args.cols, device=dev, generator=torch.Generator(device=dev).manual_seed(1017))
    q = torch.zeros(args.tokens, args.cols, dtype=torch.int8, device=dev)
    d = torch.zeros(args.tokens, args.cols // 32, device=dev)
    y = torch.empty(args.tokens, args.rows, device=dev)
    if args.generic:
        lib.mv_set_staged(0), lib.q8_set_staged(0)
    assert lib.q8_round(x.data_ptr(), args.tokens, args.cols, args.cols, q.data_ptr(), d.data_ptr(), None)
    flops = None
    if args.op == "mm_fp4":  # the W4A4 step: the activations' quantization and the product (TYPE must be NVFP4)
        flops = 2.0 * args.rows * args.cols * args.tokens
        xq = torch.zeros(args.tokens, args.cols // 2, dtype=torch.uint8, device=dev)
        xsc = torch.zeros(args.tokens, args.cols // 16, dtype=torch.uint8, device=dev)
        fn = lambda i, st: (lib.mm_fp4_act(x.data_ptr(), args.cols, args.tokens, args.cols, 0.5, xq.data_ptr(), xsc.data_ptr(), st)
                            and lib.mm_fp4(pool.data_ptr() + (i % copies) * nb, args.rows, args.cols, xq.data_ptr(),
                                           xsc.data_ptr(), args.tokens, 1.0, y.data_ptr(), args.rows, st))
    elif args.op in ("mm_run", "mmq_group"):
        n16 = (args.tokens + 15) // 16 * 16
        flops = 2.0 * args.rows * args.cols * args.tokens
        if args.op == "mm_run":
            x16 = torch.zeros(n16 * args.cols, dtype=torch.float16, device=dev)
            flag = torch.zeros(1, dtype=torch.int32, device=dev)
            assert lib.mm_x16(x.data_ptr(), args.cols, args.tokens, args.cols, x16.data_ptr(), flag.data_ptr(), None)
            fn = lambda i, st: lib.mm_run(tid, pool.data_ptr() + (i % copies) * nb, args.rows, args.cols, x16.data_ptr(),
                                          args.tokens, y.data_ptr(), args.rows, st)
        else:
            idx = torch.arange(args.tokens, dtype=torch.int32, device=dev)
            x8 = torch.zeros(n16 * args.cols, dtype=torch.int8, device=dev)
            dx = torch.zeros(n16 * args.cols // 32, device=dev)
            sx = torch.zeros_like(dx)
            assert lib.mmq_x8_rows(x.data_ptr(), args.cols, idx.data_ptr(), args.tokens, args.cols, x8.data_ptr(),
                                   dx.data_ptr(), sx.data_ptr(), None)
            tabs = [torch.tensor([pool.data_ptr() + c * nb], dtype=torch.int64, device=dev) for c in range(copies)]
            cnt = torch.tensor([args.tokens], dtype=torch.int32, device=dev)
            zero = torch.zeros(1, dtype=torch.int32, device=dev)
            fn = lambda i, st: lib.mmq_group(tid, tabs[i % copies].data_ptr(), cnt.data_ptr(), 1, args.tokens, args.rows,
                                             args.cols, x8.data_ptr(), dx.data_ptr(), sx.data_ptr(), zero.data_ptr(),
                                             y.data_ptr(), zero.data_ptr(), args.rows, st)
    elif args.op == "q8_run":
        fn = lambda i, st: lib.q8_run(tid, pool.data_ptr() + (i % copies) * nb, args.rows, args.cols, q.data_ptr(),
                                      d.data_ptr(), args.tokens, y.data_ptr(), args.rows, st)
    else:
        fn = lambda i, st: lib.mv_run(tid, pool.data_ptr() + (i % copies) * nb, args.rows, args.cols, x.data_ptr(),
                                      args.tokens, y.data_ptr(), st)
    for i in range(max(args.plain, 3)):
        if not fn(i, None):
            raise SystemExit("the library refused the call")
    torch.cuda.synchronize()
    status = lib.q8_status() | lib.mv_status() | lib.mm_status() | lib.mmq_status()
    if args.plain:
        print("%d launches, status %d" % (args.plain, status))
        return
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
    print(json.dumps({"op": args.op, "type": args.type, "rows": args.rows, "cols": args.cols, "tokens": args.tokens,
                      "kernels": "generic" if args.generic else "default", "us_per_launch": us,
                      "weight_bytes": nb, "weight_gbs": nb / us / 1e3, "tflops": None if flops is None else flops / us / 1e6,
                      "status": status | lib.q8_status() | lib.mv_status() | lib.mm_status() | lib.mmq_status()}))


if __name__ == "__main__":
    main()
