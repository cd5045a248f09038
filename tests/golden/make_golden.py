"""Generate the committed golden vectors. Run where the reference tree is mounted and gguf-py is installed:

    python tests/golden/make_golden.py [reference-tree]

Writes (numpy .npz, a few hundred KB in all):
  dequant.npz   - for every block type: 48 random blocks (every scale/exponent byte random too) and the F32 values
                  gguf-py's dequantize gives for them. Third-party ground truth for the decoders: gguf %s.
  lane_<T>.npz  - for each of the reference's int8 lane types: random weights at 16- and 32-lane widths, F32 inputs
                  (with an all-zero block and a lone -2.5), and what the reference's own CPU lane, compiled
                  unmodified from src/cpu/{q8,expert,lane}.c, returns: cpu_q8_round's bytes and scales,
                  cpu_q8_rows' sums, cpu_mv_rows' sums.
  ffn.npz       - one small expert FFN job through the reference's cpu_lane_submit (4 threads): inputs and outputs.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))

import gguf  # noqa: E402
from gguf import quants as Q  # noqa: E402

from libosmos_b200 import synth  # noqa: E402
from oracle import oracle as orc  # noqa: E402

GG = gguf.GGMLQuantizationType
GG_TYPE = {2: GG.Q4_0, 8: GG.Q8_0, 10: GG.Q2_K, 12: GG.Q4_K, 16: GG.IQ2_XXS, 17: GG.IQ2_XS, 18: GG.IQ3_XXS,
           19: GG.IQ1_S, 22: GG.IQ2_S, 29: GG.IQ1_M, 39: GG.MXFP4, 40: GG.NVFP4, 7: GG.Q5_1, 11: GG.Q3_K, 13: GG.Q5_K,
           14: GG.Q6_K, 20: GG.IQ4_NL, 23: GG.IQ4_XS, 0: GG.F32, 30: GG.BF16}
# (Q2_0 and MXFP8 are the reference's own ids 42 and 43: gguf-py has no decoder for them, so they have no third-party
# golden - the oracle's restatement of kernels/quant.h:252-256, 308-311 stands alone for those two)


def dequant_golden():
    out = {}
    for name, tid in orc.TYPES.items():
        if tid not in GG_TYPE:
            continue
        rng = synth.rng_for(101, tid)
        raw = synth.random_blocks(tid, 48, rng)
        if tid == 39:
            raw[:, 0] = rng.integers(0, 256, size=48)
        if tid == 40:
            raw[:, 0:4] = rng.integers(0, 256, size=(48, 4))
        if tid == 0:  # (the unquantized types: what the bytes are, no decoder to speak of)
            vals = raw.reshape(-1).view(np.float32)
        elif tid == 30:
            vals = (raw.reshape(-1).view(np.uint16).astype(np.uint32) << 16).view(np.float32)
        else:
            vals = Q.dequantize(raw, GG_TYPE[tid]).astype(np.float32).reshape(-1)
        out[name + "_raw"] = raw
        out[name + "_values"] = vals
    np.savez_compressed(os.path.join(HERE, "dequant.npz"), gguf_version=gguf.__version__ if hasattr(gguf, "__version__") else "?", **out)


def lane_golden(ref):
    for name in orc.LANE_TYPES:
        tid = orc.TYPES[name]
        out = {}
        for cols in (512, 768, 4096):
            rows, ntok = 10, 5
            rng = synth.rng_for(102, tid, cols)
            w = synth.random_tensor(tid, rows, cols, rng)
            x = (rng.standard_normal((ntok, cols)) * 1.5).astype(np.float32)
            x[0, :32] = 0.0
            x[1, 32:64] = 0.0
            x[1, 37] = -2.5
            q, d = ref.q8_round(x)
            assert d[0, 0] == 0.0 and q[1, 37] == -127
            y = ref.q8_rows(tid, w, rows, cols, q, d)
            ymv = ref.mv_rows(tid, w, rows, cols, x)
            assert y is not None and ymv is not None
            out.update({"w_%d" % cols: w, "x_%d" % cols: x, "q_%d" % cols: q, "d_%d" % cols: d, "y_%d" % cols: y,
                        "ymv_%d" % cols: ymv})
        np.savez_compressed(os.path.join(HERE, "lane_%s.npz" % name), **out)


def ffn_golden(ref):
    dim, ff, lim = 512, 256, 7.0
    out = {}
    for name in ("IQ3_XXS", "IQ1_M"):
        tid = orc.TYPES[name]
        rng = synth.rng_for(103, tid)
        counts = [1, 3, 2]
        n_rows = sum(counts)
        x = rng.standard_normal((n_rows, dim)).astype(np.float32)
        scale = rng.uniform(0.05, 0.4, size=n_rows).astype(np.float32)
        experts, row0 = [], 0
        for e, c in enumerate(counts):
            g = synth.random_tensor(tid, ff, dim, rng)
            u = synth.random_tensor(tid, ff, dim, rng)
            dn = synth.random_tensor(tid, dim, ff, rng)
            experts.append((g, u, dn, row0, c))
            out["%s_gate%d" % (name, e)], out["%s_up%d" % (name, e)], out["%s_down%d" % (name, e)] = g, u, dn
            row0 += c
        y = ref.lane_ffn(4, tid, tid, dim, ff, lim, x, scale, experts)
        assert y is not None
        out[name + "_x"], out[name + "_scale"], out[name + "_y"] = x, scale, y
        out[name + "_counts"] = np.array(counts, dtype=np.int32)
    out["dim"], out["ff"], out["lim"] = dim, ff, np.float32(lim)
    np.savez_compressed(os.path.join(HERE, "ffn.npz"), **out)


if __name__ == "__main__":
    tree = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("OSMOS_REF")
    if not tree or not os.path.isdir(os.path.join(tree, "src", "cpu")):
        raise SystemExit("make_golden.py: pass the reference tree (argument or $OSMOS_REF)")
    orc.build(tree)
    ref = orc.Reference()
    assert ref.lib.cpu_q8_ready(), "this CPU lacks AVX-512 VNNI: the reference's int8 lane refuses"
    dequant_golden()
    lane_golden(ref)
    ffn_golden(ref)
    print("golden vectors written to", HERE)
