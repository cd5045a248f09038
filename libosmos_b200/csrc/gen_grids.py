"""Write the IQ codebook tables the kernels and the CPU oracle share.

The tables are not typed in anywhere in this repository: they are read out of the
installed ``gguf`` package (llama.cpp's gguf-py, the ground truth for GGUF block
values) and written to a generated header that is kept out of version control.

    python libosmos_b200/csrc/gen_grids.py <out.h>

Each grid row is packed little-endian, value j in byte j, as signed bytes:
IQ2 grids hold 8, 25, 43; IQ3_XXS holds 4..62 (four values a row); IQ1 holds -1, 0, 1.
The same role as the reference's tools/gen_grids.py:9-41.
"""
import sys

import numpy as np
from gguf import quants as Q


def _rows(cls):
    cls.init_grid()
    g = cls.grid.reshape(cls.grid_shape).astype(np.int8)
    assert g.shape[1] in (4, 8), g.shape
    return [int.from_bytes(r.tobytes(), "little") for r in g], g.shape[1]


def _emit(out, name, ctype, vals, fmt, per_line):
    out.append("static OSMOS_TABLE %s %s[%d] = {" % (ctype, name, len(vals)))
    for i in range(0, len(vals), per_line):
        out.append("  " + ", ".join(fmt % v for v in vals[i:i + per_line]) + ",")
    out.append("};")
    out.append("")


def render():
    out = [
        "/* generated from the installed gguf package by gen_grids.py - not tracked, do not edit */",
        "#ifndef OSMOS_B200_GRIDS_H",
        "#define OSMOS_B200_GRIDS_H",
        "#include <stdint.h>",
        "#if defined(__CUDACC__)",
        "#define OSMOS_TABLE __device__ const",
        "#else",
        "#define OSMOS_TABLE const",
        "#endif",
        "",
    ]
    for name, cls in (("osmos_grid_iq2xxs", Q.IQ2_XXS), ("osmos_grid_iq2xs", Q.IQ2_XS),
                      ("osmos_grid_iq2s", Q.IQ2_S), ("osmos_grid_iq1s", Q.IQ1_S),
                      ("osmos_grid_iq3xxs", Q.IQ3_XXS)):
        vals, width = _rows(cls)
        if width == 8:
            _emit(out, name, "uint64_t", vals, "0x%016xull", 4)
        else:
            _emit(out, name, "uint32_t", vals, "0x%08xu", 8)
    _emit(out, "osmos_ksigns", "uint8_t", [int(v) for v in Q.IQ2_XXS.ksigns], "0x%02x", 16)
    _emit(out, "osmos_iq4nl_values", "int8_t", [int(v) for v in Q.IQ4_NL.kvalues], "%d", 16)
    _emit(out, "osmos_e2m1_doubled", "int8_t", [int(v) for v in Q.MXFP4.kvalues], "%d", 16)
    # the two 16-entry code tables once more as four words each (entry i the byte i % 4 of word i / 4): constants a
    # byte permute can index
    for name, vals in (("OSMOS_IQ4NL_WORDS", Q.IQ4_NL.kvalues), ("OSMOS_E2M1_WORDS", Q.MXFP4.kvalues)):
        b = bytes(int(v) & 0xFF for v in vals)
        out.append("#define %s %s" % (name, ", ".join("0x%08xu" % int.from_bytes(b[i:i + 4], "little") for i in range(0, 16, 4))))
    out.append("")
    assert Q.IQ1_M.grid_hex == Q.IQ1_S.grid_hex and float(Q.IQ1_S.delta) == 0.125
    out.append("#endif")
    return "\n".join(out) + "\n"


if __name__ == "__main__":
    text = render()
    if len(sys.argv) > 1:
        with open(sys.argv[1], "w") as f:
            f.write(text)
    else:
        sys.stdout.write(text)
