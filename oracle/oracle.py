"""ctypes bindings for the CPU checkers - TEST INFRASTRUCTURE, NOT PRODUCT CODE.

`Oracle` wraps this repository's scalar C restatement (oracle/osmos_oracle.c). `Reference` wraps the reference's
own CPU lane compiled unmodified into oracle/_ref/libosmos_ref.so, when that file is present (it is built only
where the reference tree is mounted; the file itself travels with the working tree).

Only tests/, the smoke check and bench.py's CPU-baseline / reference legs may import this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "_build", "libosmos_oracle.so")
REF_SO = os.path.join(HERE, "_ref", "libosmos_ref.so")

TYPES = {"Q4_0": 2, "Q8_0": 8, "Q2_K": 10, "Q4_K": 12, "IQ2_XXS": 16, "IQ2_XS": 17, "IQ3_XXS": 18, "IQ1_S": 19,
         "IQ2_S": 22, "IQ1_M": 29, "MXFP4": 39, "NVFP4": 40, "Q5_1": 7, "Q3_K": 11, "Q5_K": 13, "Q6_K": 14,
         "IQ4_NL": 20, "IQ4_XS": 23, "Q2_0": 42, "MXFP8": 43, "F32": 0, "BF16": 30}
BLOCK = {2: (32, 18), 8: (32, 34), 10: (256, 84), 12: (256, 144), 16: (256, 66), 17: (256, 74), 18: (256, 98),
         19: (256, 50), 22: (256, 82), 29: (256, 56), 39: (32, 17), 40: (64, 36),
         7: (32, 24), 11: (256, 110), 13: (256, 176), 14: (256, 210), 20: (32, 18), 23: (256, 136), 42: (64, 18),
         43: (32, 33), 0: (1, 4), 30: (1, 2)}
LANE_TYPES = ("IQ2_XXS", "IQ2_XS", "IQ3_XXS", "IQ1_S", "IQ2_S", "IQ1_M", "Q2_K")


def reference_tree():
    """Where the reference's sources are mounted: $OSMOS_REF, else the `reference_path` the benchmark description at
    the repository's root (BASELINE.json) names; None when neither points at a tree that holds src/cpu."""
    import json
    cand = os.environ.get("OSMOS_REF")
    if not cand:
        try:
            with open(os.path.join(HERE, "..", "BASELINE.json")) as f:
                cand = json.load(f).get("reference_path")
        except (OSError, ValueError):
            cand = None
    return cand if cand and os.path.isdir(os.path.join(cand, "src", "cpu")) else None


def build(ref_tree=None):
    """Compile the restatement, and the reference's CPU lane when its tree is present (ref_tree, else
    reference_tree())."""
    ref_tree = ref_tree or reference_tree()
    grids = os.path.join(HERE, "..", "libosmos_b200", "csrc", "_gen", "osmos_grids.h")
    if not os.path.exists(grids):
        os.makedirs(os.path.dirname(grids), exist_ok=True)
        subprocess.check_call(["python", os.path.join(HERE, "..", "libosmos_b200", "csrc", "gen_grids.py"), grids])
    subprocess.check_call(["make", "-s", "-C", HERE])
    if ref_tree and os.path.isdir(os.path.join(ref_tree, "src", "cpu")):
        subprocess.check_call(["make", "-s", "-C", HERE, "ref", "REF=" + ref_tree])


def _p(a, t=None):
    if a is None:
        return None
    return a.ctypes.data_as(C.c_void_p)


def tensor_bytes(type_id, rows, cols):
    v, b = BLOCK[type_id]
    assert cols % v == 0
    return rows * (cols // v) * b


class Oracle:
    def __init__(self, path=ORACLE_SO):
        if not os.path.exists(path):
            build()
        self.lib = C.CDLL(path)
        L = self.lib
        L.orc_dequant.restype = C.c_int
        L.orc_mv_rows.restype = C.c_int
        L.orc_q8_round.restype = C.c_int
        L.orc_q8_0_round.restype = C.c_int
        L.orc_q8_rows.restype = C.c_int
        L.orc_q8_block_dots.restype = C.c_int
        L.orc_lane_expert.restype = C.c_int
        L.orc_mmq_x8_rows.restype = C.c_int
        L.orc_mmq_rows.restype = C.c_int
        L.orc_fp4_round.restype = C.c_int
        L.orc_x16_attn.restype = C.c_int
        L.orc_fp8_round.restype = C.c_int
        L.orc_lane_exp.restype = C.c_float
        L.orc_lane_exp.argtypes = [C.c_float]
        L.orc_mmq_x8_at.restype = C.c_uint64
        L.orc_mmq_dx_at.restype = C.c_uint64

    def dequant(self, type_id, raw, values):
        raw = np.ascontiguousarray(raw, dtype=np.uint8)
        out = np.empty(values, dtype=np.float32)
        ok = self.lib.orc_dequant(C.c_uint32(type_id), _p(raw), C.c_uint64(values), _p(out))
        return out if ok else None

    def mv_rows(self, type_id, w, rows, cols, x):
        """x: [n_tok, cols] f32 -> y [n_tok, rows]"""
        x = np.ascontiguousarray(x, dtype=np.float32)
        n = x.shape[0]
        y = np.empty((n, rows), dtype=np.float32)
        ok = self.lib.orc_mv_rows(C.c_uint32(type_id), _p(w), C.c_uint32(cols), C.c_uint32(0), C.c_uint32(rows), _p(x),
                                  C.c_uint32(x.shape[1]), C.c_uint32(n), _p(y), C.c_uint32(rows))
        return y if ok else None

    def q8_round(self, x, ggml_q8_0=False):
        x = np.ascontiguousarray(x, dtype=np.float32)
        rows, cols = x.shape
        q = np.empty((rows, cols), dtype=np.int8)
        d = np.empty((rows, cols // 32), dtype=np.float32)
        fn = self.lib.orc_q8_0_round if ggml_q8_0 else self.lib.orc_q8_round
        ok = fn(_p(x), C.c_uint32(rows), C.c_uint32(cols), C.c_uint32(cols), _p(q), _p(d))
        return (q, d) if ok else None

    def q8_rows(self, type_id, w, rows, cols, q, d):
        q = np.ascontiguousarray(q, dtype=np.int8)
        d = np.ascontiguousarray(d, dtype=np.float32)
        n = q.shape[0]
        y = np.empty((n, rows), dtype=np.float32)
        ok = self.lib.orc_q8_rows(C.c_uint32(type_id), _p(w), C.c_uint32(cols), C.c_uint32(0), C.c_uint32(rows),
                                  _p(q), _p(d), C.c_uint32(n), _p(y), C.c_uint32(rows))
        return y if ok else None

    def q8_block_dots(self, type_id, w_row, cols, q_row):
        out = np.empty(2 * (cols // 32), dtype=np.int32)
        q_row = np.ascontiguousarray(q_row, dtype=np.int8)
        ok = self.lib.orc_q8_block_dots(C.c_uint32(type_id), _p(w_row), C.c_uint32(cols), _p(q_row), _p(out))
        return out if ok else None

    def swiglu_lane(self, g, u, lim, scale):
        g = np.ascontiguousarray(g, dtype=np.float32)
        u = np.ascontiguousarray(u, dtype=np.float32)
        scale = np.ascontiguousarray(scale, dtype=np.float32)
        h = np.empty_like(g)
        self.lib.orc_swiglu_lane(_p(g), _p(u), C.c_uint32(g.shape[1]), C.c_float(lim), _p(scale),
                                 C.c_uint32(g.shape[0]), _p(h))
        return h

    def lane_exp(self, x):
        return np.array([self.lib.orc_lane_exp(float(v)) for v in np.asarray(x, dtype=np.float32)], dtype=np.float32)

    def lane_expert(self, type_gu, type_down, gate, up, down, dim, ff, lim, x, scale):
        x = np.ascontiguousarray(x, dtype=np.float32)
        scale = np.ascontiguousarray(scale, dtype=np.float32)
        cnt = x.shape[0]
        y = np.empty((cnt, dim), dtype=np.float32)
        ok = self.lib.orc_lane_expert(C.c_uint32(type_gu), C.c_uint32(type_down), _p(gate), _p(up), _p(down),
                                      C.c_uint32(dim), C.c_uint32(ff), C.c_float(lim), _p(x), _p(scale),
                                      C.c_uint32(cnt), _p(y))
        return y if ok else None

    def gather_sum(self, src, idx, m, add=None):
        src = np.ascontiguousarray(src, dtype=np.float32)
        idx = np.ascontiguousarray(idx, dtype=np.int32)
        n, dim = idx.size // m, src.shape[1]
        y = np.empty((n, dim), dtype=np.float32)
        if add is not None:
            add = np.ascontiguousarray(add, dtype=np.float32)
        self.lib.orc_gather_sum(_p(y), _p(src), _p(idx), C.c_uint32(m), C.c_uint32(n), C.c_uint32(dim), _p(add))
        return y

    def mmq_x8_rows(self, x, idx, cols):
        x = np.ascontiguousarray(x, dtype=np.float32)
        idx = np.ascontiguousarray(idx, dtype=np.int32)
        slots = idx.size
        tiles = (slots + 15) // 16
        x8 = np.zeros(tiles * 16 * cols, dtype=np.int8)
        dx = np.zeros(tiles * 16 * (cols // 32), dtype=np.float32)
        sx = np.zeros_like(dx)
        ok = self.lib.orc_mmq_x8_rows(_p(x), C.c_uint32(x.shape[1]), _p(idx), C.c_uint32(slots), C.c_uint32(cols),
                                      _p(x8), _p(dx), _p(sx))
        return (x8, dx, sx) if ok else None

    def mmq_rows(self, w, rows, cols, x8, dx, sx, soff, cnt, want_ints=False):
        y = np.empty((cnt, rows), dtype=np.float32)
        ints = np.empty((rows, cnt, cols // 32), dtype=np.int32) if want_ints else None
        ok = self.lib.orc_mmq_rows(_p(w), C.c_uint32(0), C.c_uint32(rows), C.c_uint32(cols), _p(x8), _p(dx), _p(sx),
                                   C.c_uint32(soff), C.c_uint32(cnt), _p(y), C.c_uint32(rows), _p(ints))
        if not ok:
            return None
        return (y, ints) if want_ints else y

    def fp4_round(self, x, block=32, e4m3_scale=False, dim=None):
        x = np.array(x, dtype=np.float32, copy=True).reshape(-1)
        packed = None
        if dim:
            packed = np.zeros((x.size // dim) * (dim // 2 + dim // block), dtype=np.uint8)
        ok = self.lib.orc_fp4_round(_p(x), C.c_uint64(x.size), C.c_uint32(block), C.c_int(int(e4m3_scale)),
                                    _p(packed), C.c_uint32(dim or 0))
        return (x, packed) if ok else None

    def x16_rows(self, x, slots, cols, idx=None):
        """(tiled f16 bits, overflow flag) of mm_x16 (idx None) / mm_x16_rows"""
        x = np.ascontiguousarray(x, dtype=np.float32)
        xs = x.shape[1]
        padded = (slots + 15) // 16 * 16
        out = np.zeros(padded * cols, dtype=np.uint16)
        ip = None if idx is None else np.ascontiguousarray(idx, dtype=np.int32)
        over = self.lib.orc_x16_rows(_p(x), C.c_uint32(xs), _p(ip), C.c_uint32(slots), C.c_uint32(cols), _p(out))
        return out, int(over)

    def x16_attn(self, x, n, cols, head_dim, rope_dim, freqs, pos):
        """(tiled f16 bits, overflow flag) of mm_x16_attn"""
        x = np.ascontiguousarray(x, dtype=np.float32)
        freqs = np.ascontiguousarray(freqs, dtype=np.float32)
        pos = np.ascontiguousarray(pos, dtype=np.int32)
        out = np.zeros((n + 15) // 16 * 16 * cols, dtype=np.uint16)
        over = self.lib.orc_x16_attn(_p(x), C.c_uint32(x.shape[1]), C.c_uint32(n), C.c_uint32(cols), C.c_uint32(head_dim),
                                     C.c_uint32(rope_dim), _p(freqs), _p(pos), _p(out))
        assert over >= 0
        return out, int(over)

    def mv_fp4_rows(self, w, rows, cols, x, lanes=32, scale=None):
        """mv_fp4 (lanes 32, scale) / mv_fp4_tok (lanes by the row's length, no scale) of one matrix over x's rows"""
        x = np.ascontiguousarray(x, dtype=np.float32)
        w = np.ascontiguousarray(w, dtype=np.uint8)
        y = np.zeros((x.shape[0], rows), dtype=np.float32)
        self.lib.orc_mv_fp4_rows(_p(w), C.c_uint32(rows), C.c_uint32(cols), _p(x), C.c_uint32(x.shape[1]),
                                 C.c_uint32(x.shape[0]), C.c_uint32(lanes), C.c_float(scale if scale is not None else 1.0),
                                 C.c_int(int(scale is not None)), _p(y), C.c_uint32(rows))
        return y

    def fp4_act(self, x, cols, gs, seed=0, bf16=False):
        """(codes n x cols/2, scale bytes n x cols/16) of mm_fp4_act / mm_fp4_quant; x F32 rows, or (bf16) uint16 rows"""
        x = np.ascontiguousarray(x, dtype=np.uint16 if bf16 else np.float32)
        n, xs = x.shape
        q = np.zeros((n, cols // 2), dtype=np.uint8)
        sc = np.zeros((n, cols // 16), dtype=np.uint8)
        self.lib.orc_fp4_act(_p(x), C.c_int(int(bf16)), C.c_uint32(xs), C.c_uint32(n), C.c_uint32(cols), C.c_float(gs),
                             C.c_uint32(seed), _p(q), _p(sc))
        return q, sc

    def fp4_mm(self, w, rows, cols, q, sc, scale=1.0):
        """(float64 sums, sums of magnitudes), n x rows, of mm_fp4 over the quantized operands"""
        w = np.ascontiguousarray(w, dtype=np.uint8)
        q = np.ascontiguousarray(q, dtype=np.uint8)
        sc = np.ascontiguousarray(sc, dtype=np.uint8)
        n = q.shape[0]
        y = np.zeros((n, rows), dtype=np.float64)
        mag = np.zeros((n, rows), dtype=np.float64)
        self.lib.orc_fp4_mm(_p(w), C.c_uint32(rows), C.c_uint32(cols), _p(q), _p(sc), C.c_uint32(n), C.c_double(scale),
                            _p(y), _p(mag))
        return y, mag

    def fp8_round(self, x, dim=None):
        x = np.array(x, dtype=np.float32, copy=True).reshape(-1)
        packed = None
        if dim:
            packed = np.zeros((x.size // dim) * (dim + dim // 32), dtype=np.uint8)
        ok = self.lib.orc_fp8_round(_p(x), C.c_uint64(x.size), _p(packed), C.c_uint32(dim or 0))
        return (x, packed) if ok else None


class CpuLaneExpert(C.Structure):
    _fields_ = [("gate", C.c_void_p), ("up", C.c_void_p), ("down", C.c_void_p), ("row0", C.c_uint32),
                ("cnt", C.c_uint32)]


class CpuLaneJob(C.Structure):
    _fields_ = [("type_gu", C.c_uint32), ("type_down", C.c_uint32), ("dim", C.c_uint32), ("ff", C.c_uint32),
                ("lim", C.c_float), ("x", C.c_void_p), ("scale", C.c_void_p), ("n_rows", C.c_uint32),
                ("e", C.POINTER(CpuLaneExpert)), ("n_e", C.c_uint32), ("y", C.c_void_p), ("seq", C.c_void_p),
                ("value", C.c_uint32)]


class Reference:
    """The reference's own CPU lane (include/osmos/cpu/{q8,expert,lane}.h), unmodified."""

    def __init__(self, path=REF_SO):
        self.lib = C.CDLL(path)
        L = self.lib
        for f in ("cpu_q8_ready", "cpu_q8_round", "cpu_q8_rows", "cpu_mv_known", "cpu_mv_rows", "cpu_lane_submit",
                  "cpu_lane_wait"):
            getattr(L, f).restype = C.c_bool
        L.cpu_lane_create.restype = C.c_void_p
        L.cpu_lane_create.argtypes = [C.c_int, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32]
        L.cpu_lane_destroy.argtypes = [C.c_void_p]
        L.cpu_lane_submit.argtypes = [C.c_void_p, C.POINTER(CpuLaneJob)]
        L.cpu_lane_wait.argtypes = [C.c_void_p]

    @staticmethod
    def available(path=REF_SO):
        if not os.path.exists(path):
            return False
        try:
            return bool(Reference(path).lib.cpu_q8_ready())
        except OSError:
            return False

    def q8_round(self, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        rows, cols = x.shape
        q = np.empty((rows, cols), dtype=np.int8)
        d = np.empty((rows, cols // 32), dtype=np.float32)
        ok = self.lib.cpu_q8_round(_p(x), C.c_uint32(rows), C.c_uint32(cols), C.c_uint32(cols), _p(q), _p(d))
        return (q, d) if ok else None

    def q8_rows(self, type_id, w, rows, cols, q, d):
        q = np.ascontiguousarray(q, dtype=np.int8)
        d = np.ascontiguousarray(d, dtype=np.float32)
        n = q.shape[0]
        y = np.empty((n, rows), dtype=np.float32)
        ok = self.lib.cpu_q8_rows(C.c_uint32(type_id), _p(w), C.c_uint32(cols), C.c_uint32(0), C.c_uint32(rows),
                                  _p(q), _p(d), C.c_uint32(n), _p(y), C.c_uint32(rows))
        return y if ok else None

    def mv_rows(self, type_id, w, rows, cols, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        n = x.shape[0]
        y = np.empty((n, rows), dtype=np.float32)
        ok = self.lib.cpu_mv_rows(C.c_uint32(type_id), _p(w), C.c_uint32(cols), C.c_uint32(0), C.c_uint32(rows),
                                  _p(x), C.c_uint32(x.shape[1]), C.c_uint32(n), _p(y), C.c_uint32(rows))
        return y if ok else None

    def lane_pool(self, threads, max_rows, dim, ff, pin=True):
        """cpu_lane_create with worker i pinned to the i-th CPU this process may run on (pin False: the scheduler's
        to place); returns (pool handle or None, the CPUs used)"""
        cpus = sorted(os.sched_getaffinity(0))[:threads] if pin and hasattr(os, "sched_getaffinity") else []
        if pin and len(cpus) == threads:
            arr = (C.c_int * threads)(*cpus)
            pool = self.lib.cpu_lane_create(threads, arr, max_rows, dim, ff)
            if pool:
                return pool, cpus
        return self.lib.cpu_lane_create(threads, None, max_rows, dim, ff), []

    def lane_job(self, type_gu, type_down, dim, ff, lim, x, scale, experts):
        """a cpu_lane job built once: returns an object whose .run(pool) submits it and waits (True when it was done)
        and whose .y holds the rows; everything the job points to is kept alive by the object"""
        ref = self

        class Job:
            def __init__(self):
                self.x = np.ascontiguousarray(x, dtype=np.float32)
                self.scale = np.ascontiguousarray(scale, dtype=np.float32)
                self.y = np.zeros((self.x.shape[0], dim), dtype=np.float32)
                self.parts = experts
                self.arr = (CpuLaneExpert * len(experts))()
                for i, (g, u, dn, row0, cnt) in enumerate(experts):
                    self.arr[i] = CpuLaneExpert(g.ctypes.data, u.ctypes.data, dn.ctypes.data, row0, cnt)
                self.seq = np.zeros(1, dtype=np.uint32)
                self.n = 0
                self.job = CpuLaneJob(type_gu, type_down, dim, ff, lim, self.x.ctypes.data, self.scale.ctypes.data,
                                      self.x.shape[0], self.arr, len(experts), self.y.ctypes.data, self.seq.ctypes.data, 0)

            def run(self, pool):
                self.n += 1
                self.job.value = self.n
                ok = ref.lib.cpu_lane_submit(pool, C.byref(self.job)) and ref.lib.cpu_lane_wait(pool)
                return bool(ok) and int(self.seq[0]) == self.n

        return Job()

    def lane_ffn(self, threads, type_gu, type_down, dim, ff, lim, x, scale, experts, pool=None):
        """experts: list of (gate, up, down, row0, cnt) numpy byte arrays; x [n_rows, dim]; returns y [n_rows, dim].
        pool: an existing cpu_lane_create handle to reuse (else one is made and destroyed)."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        scale = np.ascontiguousarray(scale, dtype=np.float32)
        n_rows = x.shape[0]
        y = np.zeros((n_rows, dim), dtype=np.float32)
        arr = (CpuLaneExpert * len(experts))()
        for i, (g, u, dn, row0, cnt) in enumerate(experts):
            arr[i] = CpuLaneExpert(g.ctypes.data, u.ctypes.data, dn.ctypes.data, row0, cnt)
        seq = np.zeros(1, dtype=np.uint32)
        own = pool is None
        if own:
            pool = self.lib.cpu_lane_create(threads, None, max(n_rows, 1), dim, ff)
            if not pool:
                return None
        job = CpuLaneJob(type_gu, type_down, dim, ff, lim, x.ctypes.data, scale.ctypes.data, n_rows, arr,
                         len(experts), y.ctypes.data, seq.ctypes.data, 1)
        ok = self.lib.cpu_lane_submit(pool, C.byref(job)) and self.lib.cpu_lane_wait(pool)
        if own:
            self.lib.cpu_lane_destroy(pool)
        return y if ok and seq[0] == 1 else None
