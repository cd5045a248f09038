"""The C-ABI boundary without a GPU: the library loads, exports every function the headers declare, the ctypes
signatures cover them all, and the refusals that are decided before any launch return false."""
import ctypes as C
import os
import re

import libosmos_b200
from libosmos_b200 import api

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
INC = os.path.join(ROOT, "include", "osmos_b200")


def declared_functions():
    names = set()
    for f in sorted(os.listdir(INC)):
        text = open(os.path.join(INC, f)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        text = re.sub(r"static inline[^{;]*\{.*?\n\}", "", text, flags=re.S)  # inline helpers are not exports
        for m in re.finditer(r"^\s*(?:const\s+)?(?:bool|void|int|uint32_t|uint64_t|OsmosQTypeInfo\s*\*|Gguf\w*\s*\*)\s*\*?\s*(\w+)\s*\(",
                             text, flags=re.M):
            names.add(m.group(1))
    return names


def test_library_exports_every_declared_function(lib):
    names = declared_functions()
    assert len(names) >= 40, names
    dll = C.CDLL(lib.path)
    missing = [n for n in sorted(names) if not hasattr(dll, n)]
    assert not missing, "declared in include/osmos_b200 but not exported: %s" % missing
    unbound = [n for n in sorted(names) if n not in api.SIGNATURES]
    assert not unbound, "no ctypes signature for: %s" % unbound


def test_library_leaves_none_of_its_own_symbols_undefined(lib):
    """a source file dropped from the build while another still calls into it links (a shared library may have
    undefined symbols) and only fails when the call is made: every undefined symbol must be somebody else's"""
    import shutil
    import subprocess
    if not shutil.which("nm"):
        import pytest
        pytest.skip("no nm")
    out = subprocess.run(["nm", "-D", "--undefined-only", lib.path], capture_output=True, text=True, check=True).stdout
    ours = [line for line in out.splitlines() if "osmos" in line]
    assert not ours, ours


def test_missing_library_fails_loudly(tmp_path):
    try:
        api.Lib(str(tmp_path / "nope.so"))
    except RuntimeError as e:
        assert "no fallback" in str(e)
    else:
        raise AssertionError("loading a missing library must raise")


def test_type_table(lib):
    want = {2: (32, 18), 8: (32, 34), 10: (256, 84), 12: (256, 144), 16: (256, 66), 17: (256, 74), 18: (256, 98),
            19: (256, 50), 22: (256, 82), 29: (256, 56), 39: (32, 17), 40: (64, 36)}
    for tid, (values, nbytes) in want.items():
        row = lib.qtype_info(tid).contents
        assert (row.values, row.bytes) == (values, nbytes)
        assert lib.quant_known(tid)
        assert lib.qtype_tensor_bytes(tid, 3, values * 5) == 3 * 5 * nbytes
    assert not lib.qtype_info(3) and not lib.quant_known(3) and not lib.quant_known(0)
    assert lib.qtype_tensor_bytes(18, 4, 100) == 0
    assert lib.mmq_known(12) and not lib.mmq_known(18)


def test_refusals_decided_on_the_host(lib):
    x = 0x1000  # a non-NULL stand-in: a refused call never touches it
    # mv: unknown type, ragged cols, token limits, strides (reference: include/osmos/gpu/mv.h:38-62)
    assert not lib.mv_run(3, x, 16, 256, x, 1, x, None)
    assert not lib.mv_run(18, x, 16, 100, x, 1, x, None)
    assert not lib.mv_run(18, x, 16, 256, x, 0, x, None)
    assert not lib.mv_run(18, x, 16, 256, x, 9, x, None)
    assert not lib.mv_strided(18, x, 16, 256, x, 252, 1, x, 16, None)
    assert not lib.mv_strided(18, x, 16, 256, x, 128, 2, x, 16, None)
    assert not lib.mv_group(18, x, 0, 16, 256, x, 0, 1, x, None)
    assert not lib.mv_group(18, x, 4, 16, 256, x, 0, 0, x, None)
    assert not lib.mv_group(18, x, 65536, 16, 256, x, 0, 1, x, None)
    assert not lib.mv_group_tok(18, x, x, x, 4, 9, 16, 256, x, 256, x, 16, None)
    assert not lib.mv_group_tok(18, x, x, x, 4, 0, 16, 256, x, 256, x, 16, None)
    assert not lib.mv_group_tok(18, x, x, x, 4, 2, 16, 256, x, 128, x, 16, None)
    # x16 and NVFP4's matvec (reference: kernels/mm.hip:469, 611; kernels/mv_fp4.hip:303, 326)
    assert not lib.mm_x16(8, 64, 0, 64, 8, 8, None) and not lib.mm_x16(8, 64, 2049, 64, 8, 8, None)
    assert not lib.mm_x16(8, 64, 2, 72, 8, 8, None) and not lib.mm_x16(8, 32, 2, 64, 8, 8, None)
    assert not lib.mm_x16_rows(16, 66, 8, 4, 64, 8, 8, None) and not lib.mm_x16_rows(8, 64, 8, 4, 64, 8, 8, None)
    assert not lib.mm_x16_heads(16, 64, 4, 3, 32, 16, 16, 8, None)  # the last head reaches past a row
    assert not lib.mm_x16_attn(16, 128, 2, 128, 48, 0, 16, 16, 16, 16, None) and not lib.mm_x16_attn(16, 128, 2, 128, 64, 33, 16, 16, 16, 16, None)
    assert not lib.mv_fp4(16, 8, 64, 16, 64, 0, 16, 8, 1.0, None) and not lib.mv_fp4(16, 8, 96, 16, 96, 1, 16, 8, 1.0, None)
    assert not lib.mv_fp4_tok(16, 16, 16, 0, 8, 64, 16, 64, 16, 8, None)
    assert not lib.mv_fp4_tok(16, 16, 16, 1, 8, 64, 16, 66, 16, 8, None)
    # W4A4 (reference: kernels/mm_fp4.hip:412-445): no device here, so every call is refused
    assert not lib.mm_fp4_ok()
    assert [lib.mm_col_tiles(12, n) for n in (1, 128, 129, 256, 257, 2048)] == [1, 1, 2, 2, 4, 4] and lib.mm_col_tiles(99, 5) == 0
    assert not lib.mm_fp4_act(16, 64, 1, 64, 1.0, 16, 16, None) and not lib.mm_fp4_quant(16, 1, 64, 1, 64, 1.0, None, 3, 16, 16, None)
    assert not lib.mm_fp4(16, 128, 128, 16, 16, 1, 1.0, 16, 128, None)
    # the peer transport's launches (set-up calls need a GPU and are not made here)
    assert not lib.ep_push(16, 24, 16, 16, 2, 1, 16, None) and not lib.ep_push(16, 32, 16, 16, 17, 1, 16, None)
    assert not lib.ep_wait(16, 0, 1, None) and not lib.ep_wait(None, 2, 1, None)
    assert not lib.ep_scatter_rows_peer(16, 16, 4, 2, 2, 6, 16, 16, 2, 1, 16, None)
    # q8 (reference: include/osmos/gpu/q8.h:26-44; tests/test_cpu_q8.c:226-229)
    assert not lib.q8_round(x, 1, 48, 48, x, x, None)
    assert not lib.q8_round(x, 1, 64, 32, x, x, None)
    assert not lib.q8_round(x, 0, 32, 32, x, x, None)
    assert not lib.q8_group_tok(13, x, x, x, None, 1, 1, 16, 256, x, x, x, 16, None)  # Q5_K: not a lane type
    assert not lib.q8_group_tok(2, x, x, x, None, 1, 1, 16, 256, x, x, x, 16, None)   # Q4_0: q8_run only
    assert not lib.q8_group_tok(16, x, x, x, None, 1, 1, 16, 128, x, x, x, 16, None)
    assert not lib.q8_group_tok(16, x, x, x, None, 1, 9, 16, 256, x, x, x, 16, None)
    assert not lib.q8_group_tok(16, x, x, x, None, 0, 1, 16, 256, x, x, x, 16, None)
    assert not lib.q8_gate_up(16, x, x, x, x, None, None, 1, 1, 16, 256, x, x, None, 7.0, x, 16, None)  # no scale
    assert not lib.q8_gate_up(16, x, x, x, x, None, None, 1, 1, 16, 256, x, x, x, 7.0, x, 8, None)      # hs < rows
    assert not lib.q8_run(12, x, 16, 256, x, x, 1, x, 16, None)  # Q4_K has no lane order
    assert not lib.q8_run(2, x, 16, 48, x, x, 1, x, 16, None)
    # mmq (reference: tests/gpu/test_mmq_gpu.hip:256-261)
    assert not lib.mmq_group(18, x, x, 1, 1, 16, 256, x, x, x, x, x, x, 16, None)
    assert not lib.mmq_group(12, x, x, 1, 1, 24, 256, x, x, x, x, x, x, 24, None)
    assert not lib.mmq_group(12, x, x, 1, 1, 16, 128, x, x, x, x, x, x, 16, None)
    assert not lib.mmq_group(12, x, x, 1, 1, 16, 256, x, x, x, x, x, x, 8, None)
    assert not lib.mmq_x8_rows(x, 60, x, 1, 64, x, x, x, None)
    assert not lib.mmq_x8_rows(x, 64, x, 0, 64, x, x, x, None)
    # moe / ops
    assert not lib.q4x_route(x, 1, 2048, 4, x, x, x, None)
    assert not lib.q4x_route(x, 1, 64, 33, x, x, x, None)
    assert not lib.q4x_route(x, 1, 8, 9, x, x, x, None)
    assert not lib.ops_router(x, x, 2048, 4, 1.0, 1, x, x, None)
    assert not lib.ops_router(x, x, 64, 17, 1.0, 1, x, x, None)
    assert not lib.ops_swiglu_lane(x, x, 8, 7.0, None, 1, x, None)
    assert not lib.ops_gather_sum_add(x, x, x, 2, 2, 8, None, None)
    assert not lib.ops_fp4_round(x, 48, 32, False, None, 0, None)
    assert not lib.ops_fp4_round(x, 64, 32, False, x, 48, None)
    assert not lib.ops_fp4_round(x, 64, 16, False, x, 64, None)  # packed pow2 rows are blocks of 32
    assert not lib.ops_fp8_round(x, 48, None, 0, None)


def test_expert_bounds_is_the_reference_formula(lib):
    b = api.Q4xExpertBounds()
    lib.q4x_expert_bounds(640, 512, b)
    assert list(b.first) == [0, 512, 549, 568] and list(b.count) == [512, 37, 19, 9]
    assert (b.entries, b.slots) == (577, 640 + 15 * 512)
    lib.q4x_expert_bounds(30, 512, b)
    assert list(b.count) == [30, 1, 0, 0] and b.slots == 30 + 15 * 30


def test_lane_scratch_layout(lib):
    layer = api.LaneLayer(18, 18, 2048, 512, 512, 10, 7.0, api.LaneExperts())
    n = lib.lane_scratch_bytes(layer, 64)
    assert n > 0 and n % 256 == 0
    s = api.LaneScratch()
    assert not lib.lane_scratch_bind(layer, 64, 0x10000, n - 1, s)
    assert not lib.lane_scratch_bind(layer, 64, 0x10010, n, s)  # not 256-byte aligned
    assert lib.lane_scratch_bind(layer, 64, 0x10000, n, s)
    assert s.max_tok == 64 and s.tab.max_entries == lib.lane_max_entries(640, 512)
    parts = [s.xq, s.xqd, s.hh, s.hq, s.hqd, s.ye, s.tab.w[0], s.tab.w[1], s.tab.w[2], s.tab.cnt, s.tab.xrow,
             s.tab.tok, s.tab.pair, s.tab.row_of, s.tab.order, s.tab.off, s.tab.counts]
    assert parts == sorted(parts) and all(p % 256 == 0 for p in parts) and parts[-1] + 8 <= 0x10000 + n
    bad = api.LaneLayer(18, 18, 2000, 512, 512, 10, 7.0, api.LaneExperts())
    assert lib.lane_scratch_bytes(bad, 64) == 0
