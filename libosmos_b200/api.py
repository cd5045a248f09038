"""ctypes view of libosmos_b200.so: every entry point of include/osmos_b200/*.h with its C signature.

Pointers are passed as integers (torch `tensor.data_ptr()`, or 0 for NULL); streams as `torch.cuda.Stream.cuda_stream`
or 0 for the default stream. The functions return the C ABI's bool: True = queued, False = refused.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libosmos_b200.so")

P, U32, U64, I32, F32, B = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int32, C.c_float, C.c_bool


class Q4xX16(C.Structure):
    _fields_ = [("x16", P), ("overflow", P), ("cols", U32), ("row0", U32)]


class Q4xExpertTiles(C.Structure):
    _fields_ = [("base", P * 3), ("bytes", U64 * 3), ("tab", P * 3), ("ptr", P * 3), ("cnt", P), ("gidx", P),
                ("hidx", P), ("xg", P), ("yg", P), ("xd", P), ("yd", P), ("where", P), ("off", P)]


class Q4xExpertBounds(C.Structure):
    _fields_ = [("first", U32 * 4), ("count", U32 * 4), ("entries", U32), ("slots", U32)]


class LaneExperts(C.Structure):
    _fields_ = [("base", P * 3), ("bytes", U64 * 3), ("tab", P * 3)]


class LaneTables(C.Structure):
    _fields_ = [("w", P * 3), ("cnt", P), ("xrow", P), ("tok", P), ("pair", P), ("row_of", P), ("order", P),
                ("off", P), ("counts", P), ("max_entries", U32)]


class LaneLayer(C.Structure):
    _fields_ = [("type_gu", U32), ("type_down", U32), ("dim", U32), ("ff", U32), ("n_exp", U32), ("k", U32),
                ("lim", F32), ("experts", LaneExperts)]


class LaneScratch(C.Structure):
    _fields_ = [("max_tok", U32), ("xq", P), ("xqd", P), ("hh", P), ("hq", P), ("hqd", P), ("ye", P),
                ("tab", LaneTables)]


class LaneScratchF32(C.Structure):
    _fields_ = [("max_tok", U32), ("xg", P), ("wg", P), ("ga", P), ("up", P), ("hh", P), ("ye", P), ("tab", LaneTables)]


class SharedExpert(C.Structure):
    _fields_ = [("type_gu", U32), ("type_down", U32), ("dim", U32), ("ff", U32), ("lim", F32), ("gate", P), ("up", P), ("down", P)]


class SharedScratch(C.Structure):
    _fields_ = [("max_tok", U32), ("g", P), ("u", P), ("h", P), ("x16", P), ("overflow", P)]


class Q4xMoeLayer(C.Structure):
    _fields_ = [("type", U32 * 3), ("dim", U32), ("ff", U32), ("n_exp", U32), ("k", U32), ("base", P * 3), ("bytes", U64 * 3),
                ("tab", P * 3)]


class Q4xMoeScratch(C.Structure):
    _fields_ = [("max_tok", U32), ("bounds", Q4xExpertBounds), ("ids", P), ("rows", P), ("w", P), ("ptr", P), ("cnt", P),
                ("gidx", P), ("hidx", P), ("where", P), ("off", P), ("xg", P), ("yg", P), ("xd", P), ("yd", P), ("xe16", P),
                ("ga", P), ("up", P), ("y", P), ("overflow", P)]


class EpSegment(C.Structure):
    _fields_ = [("ids", U64), ("weights", U64), ("q", U64), ("d", U64), ("bytes", U64)]


class EpLayout(C.Structure):
    _fields_ = [("flags_dispatch", U64), ("flags_combine", U64), ("ids", U64 * 2), ("weights", U64 * 2), ("q", U64 * 2),
                ("d", U64 * 2), ("recv", U64 * 2), ("bytes", U64)]


class EpPlan(C.Structure):
    _fields_ = [("rank", U32), ("n_ranks", U32), ("n_tok", U32), ("expert0", U32), ("expert1", U32), ("lay", EpLayout),
                ("peer", P * 16), ("sync", P), ("rows", P), ("layer", LaneLayer), ("scratch", LaneScratch), ("router", U32),
                ("route_bias", P), ("route_scale", F32)]


class GgufValue(C.Union):
    _fields_ = [("u", U64), ("i", C.c_int64), ("f", C.c_double), ("s", C.c_char_p), ("items", P)]


class GgufKv(C.Structure):
    _fields_ = [("key", C.c_char_p), ("type", C.c_int), ("item", C.c_int), ("n", U64), ("v", GgufValue)]


class GgufTensor(C.Structure):
    _fields_ = [("name", C.c_char_p), ("type", U32), ("n_dims", U32), ("dims", U64 * 4), ("file", C.c_int), ("offset", U64),
                ("bytes", U64)]


class Gguf(C.Structure):
    _fields_ = [("n_files", C.c_int), ("paths", C.POINTER(C.c_char_p)), ("sizes", C.POINTER(U64)), ("kv", C.POINTER(GgufKv)),
                ("n_kv", C.c_size_t), ("tensors", C.POINTER(GgufTensor)), ("n_tensors", C.c_size_t)]


class FfnWeights(C.Structure):
    _fields_ = [(n, C.POINTER(GgufTensor)) for n in ("router", "exp_gate", "exp_up", "exp_down", "ffn_norm", "router_bias", "sh_gate",
                                                     "sh_up", "sh_down")] + \
               [("n_embd", U32), ("expert_ff", U32), ("n_experts", U32), ("shared_ff", U32), ("expert_bytes", U64 * 3)]


class QTypeInfo(C.Structure):
    _fields_ = [("id", U32), ("values", U32), ("bytes", U32), ("paths", U32), ("name", C.c_char_p)]


SIGNATURES = {
    # gguf.h
    "gguf_create": (C.POINTER(Gguf), [C.c_char_p, C.c_char_p]),
    "gguf_header": (C.POINTER(Gguf), [C.c_char_p, C.c_char_p]),
    "gguf_destroy": (None, [C.POINTER(Gguf)]),
    "gguf_tensor": (C.POINTER(GgufTensor), [C.POINTER(Gguf), C.c_char_p]),
    "gguf_kv": (C.POINTER(GgufKv), [C.POINTER(Gguf), C.c_char_p]),
    "gguf_bytes": (U64, [U32, U64]),
    "gguf_int": (B, [C.POINTER(GgufKv), C.c_size_t, C.POINTER(C.c_int64)]),
    # weights.h
    "weights_ffn": (B, [C.POINTER(Gguf), C.c_int, C.POINTER(FfnWeights), C.c_char_p]),
    # quant.h / qtype.h
    "qtype_info": (C.POINTER(QTypeInfo), [U32]),
    "qtype_tensor_bytes": (U64, [U32, U64, U64]),
    "quant_known": (B, [U32]),
    "quant_dequant": (B, [U32, P, U64, P, P]),
    "quant_dequant_f16": (B, [U32, P, U64, P, P]),
    # mv.h
    "mv_run": (B, [U32, P, U32, U32, P, U32, P, P]),
    "mv_group": (B, [U32, P, U32, U32, U32, P, U32, U32, P, P]),
    "mv_group_tok": (B, [U32, P, P, P, U32, U32, U32, U32, P, U32, P, U32, P]),
    "mv_strided": (B, [U32, P, U32, U32, P, U32, U32, P, U32, P]),
    "mv_fp4": (B, [P, U32, U32, P, U32, U32, P, U32, C.c_float, P]),
    "mv_fp4_tok": (B, [P, P, P, U32, U32, U32, P, U32, P, U32, P]),
    # mm.h
    "mm_x16": (B, [P, U32, U32, U32, P, P, P]),
    "mm_x16_rows": (B, [P, U32, P, U32, U32, P, P, P]),
    "mm_x16_heads": (B, [P, U32, U32, U32, U32, U32, P, P, P]),
    "mm_x16_attn": (B, [P, U32, U32, U32, U32, U32, P, P, P, P, P]),
    "mm_known": (B, [U32]),
    "mm_fits": (B, [U32, U32, U32]),
    "mm_col_tiles": (U32, [U32, U32]),
    "mm_run": (B, [U32, P, U32, U32, P, U32, P, U32, P]),
    "mm_run_silu": (B, [U32, P, U32, U32, P, U32, P, U32, C.c_float, P, P, P]),
    "mm_run_gated_mean": (B, [U32, P, U32, U32, U32, P, U32, P, P, P, U32, P, P]),
    "mm_run2": (B, [U32, P, U32, P, U32, P, U32, P, U32, U32, P, U32, P]),
    "mm_tokens": (B, [U32, P, U32, P, U32, P, U32, P, U32, U32, P, U32, U32, P, P, C.c_bool, P]),
    "mm_tokens_scaled": (B, [U32, P, U32, P, U32, C.c_float, P, U32, P, U32, C.c_float, U32, P, U32, U32, P, P, C.c_bool, P]),
    "mm_group": (B, [U32, P, P, U32, U32, U32, U32, P, P, U32, P, P, U32, P]),
    "mm_status": (U32, []),
    "mm_fp4_ok": (B, []),
    "mm_fp4_act": (B, [P, U32, U32, U32, C.c_float, P, P, P]),
    "mm_fp4_quant": (B, [P, U32, U32, U32, U32, C.c_float, P, U32, P, P, P]),
    "mm_fp4": (B, [P, U32, U32, P, P, U32, C.c_float, P, U32, P]),
    "mm_fp4_set_tensor": (None, [C.c_int]),
    "mm_fp4_last_route": (C.c_int, []),
    "mm_mxfp4": (B, [P, U32, U32, P, U32, C.c_float, P, U32, P]),
    "mm_fp4_desc": (U32, [U32, U32, U32]),
    # q8.h
    "q8_round": (B, [P, U32, U32, U32, P, P, P]),
    "q8_0_round": (B, [P, U32, U32, U32, P, P, P]),
    "q8_group_tok": (B, [U32, P, P, P, P, U32, U32, U32, U32, P, P, P, U32, P]),
    "q8_gate_up": (B, [U32, P, P, P, P, P, P, U32, U32, U32, U32, P, P, P, F32, P, U32, P]),
    "q8_run": (B, [U32, P, U32, U32, P, P, U32, P, U32, P]),
    "q8_known": (B, [U32]),
    "mv_set_staged": (None, [C.c_int]),
    "mv_status": (U32, []),
    "q8_set_staged": (None, [C.c_int]),
    "q8_status": (U32, []),
    # mmq.h
    "mmq_known": (B, [U32]),
    "mmq_x8_rows": (B, [P, U32, P, U32, U32, P, P, P, P]),
    "mmq_group": (B, [U32, P, P, U32, U32, U32, U32, P, P, P, P, P, P, U32, P]),
    "mmq_set_tensor": (None, [C.c_int]),
    "mmq_status": (U32, []),
    # moe.h
    "q4x_route": (B, [P, U32, U32, U32, P, P, P, P]),
    "q4x_expert_bounds": (None, [U32, U32, C.POINTER(Q4xExpertBounds)]),
    "q4x_expert_tiles": (B, [P, U32, U32, U32, U32, U32, C.POINTER(Q4xExpertTiles), P]),
    "q4x_expert_tiles_static": (B, [P, U32, U32, U32, U32, U32, C.POINTER(Q4xExpertTiles), P]),
    "q4x_swiglu": (B, [P, P, U64, P, C.POINTER(Q4xX16), P]),
    "q4x_swiglu_rows": (B, [P, P, U32, P, U32, P, P, P]),
    "q4x_moe_sum": (B, [P, P, P, U32, U32, U32, P, P, P, P]),
    # ops.h
    "ops_router": (B, [P, P, U32, U32, F32, U32, P, P, P]),
    "ops_router_scored": (B, [P, P, U32, U32, F32, C.c_int, U32, P, P, P]),
    "ops_swiglu": (B, [P, P, U32, F32, P, U32, P, P]),
    "ops_swiglu_lane": (B, [P, P, U32, F32, P, U32, P, P]),
    "ops_gather_rows": (B, [P, P, P, U32, U32, P]),
    "ops_gather_sum": (B, [P, P, P, U32, U32, U32, P]),
    "ops_gather_sum_add": (B, [P, P, P, U32, U32, U32, P, P]),
    "ops_copy_rows": (B, [P, P, P, U32, U32, P]),
    "ops_wait": (B, [P, U32, P]),
    "ops_wait_set_limit_ms": (None, [U32]),
    "ops_wait_limit_ms": (U32, []),
    "ops_wait_status": (U32, []),
    "ops_fp4_round": (B, [P, U64, U32, B, P, U32, P]),
    "ops_fp8_round": (B, [P, U64, P, U32, P]),
    # lane.h
    "lane_max_entries": (U32, [U32, U32]),
    "lane_tables": (B, [P, U32, U32, U32, U32, U32, C.POINTER(LaneExperts), C.POINTER(LaneTables), P]),
    "lane_scratch_bytes": (U64, [C.POINTER(LaneLayer), U32]),
    "lane_scratch_bind": (B, [C.POINTER(LaneLayer), U32, P, U64, C.POINTER(LaneScratch)]),
    "lane_ffn": (B, [C.POINTER(LaneLayer), C.POINTER(LaneScratch), P, P, P, U32, P, P, P]),
    # ffn.h
    "lane_f32_scratch_bytes": (U64, [C.POINTER(LaneLayer), U32]),
    "lane_f32_scratch_bind": (B, [C.POINTER(LaneLayer), U32, P, U64, C.POINTER(LaneScratchF32)]),
    "lane_ffn_f32": (B, [C.POINTER(LaneLayer), C.POINTER(LaneScratchF32), P, P, P, U32, P, P, P]),
    "shared_scratch_bytes": (U64, [C.POINTER(SharedExpert), U32]),
    "shared_scratch_bind": (B, [C.POINTER(SharedExpert), U32, P, U64, C.POINTER(SharedScratch)]),
    "shared_ffn": (B, [C.POINTER(SharedExpert), C.POINTER(SharedScratch), P, U32, P, P]),
    "q4x_moe_scratch_bytes": (U64, [C.POINTER(Q4xMoeLayer), U32]),
    "q4x_moe_scratch_bind": (B, [C.POINTER(Q4xMoeLayer), U32, P, U64, C.POINTER(Q4xMoeScratch)]),
    "q4x_moe": (B, [C.POINTER(Q4xMoeLayer), C.POINTER(Q4xMoeScratch), P, P, P, P, U32, P, P]),
    # ep.h
    "ep_segment": (None, [U32, U32, U32, C.POINTER(EpSegment)]),
    "ep_unpack": (B, [P, U32, U32, U32, U32, P, P, P, P, P]),
    "ep_scatter_rows": (B, [P, P, U32, U32, U32, U32, P, P]),
    "ep_combine": (B, [P, P, U32, U32, U32, U32, P, P, P]),
    "ep_peer_alloc": (B, [C.c_uint64, P, P]),
    "ep_peer_open": (B, [P, P]),
    "ep_peer_close": (B, [P]),
    "ep_peer_free": (B, [P]),
    "ep_push": (B, [P, C.c_uint64, P, P, U32, U32, P, P]),
    "ep_wait": (B, [P, U32, U32, P]),
    "ep_wait_status": (U32, []),
    "ep_scatter_rows_peer": (B, [P, P, U32, U32, U32, U32, P, P, U32, U32, P, P]),
    "ep_layout": (B, [U32, U32, U32, U32, C.POINTER(EpLayout)]),
    "ep_plan_ok": (B, [C.POINTER(EpPlan)]),
    "ep_layer_step": (B, [C.POINTER(EpPlan), P, P, P, P, P]),
    "ep_route_round_push": (B, [C.POINTER(EpPlan), P, P, P]),
    "ep_lane_tables": (B, [C.POINTER(EpPlan), P]),
    "ep_gate_up": (B, [C.POINTER(EpPlan), P]),
    "ep_down_push": (B, [C.POINTER(EpPlan), P]),
    "ep_combine_wait": (B, [C.POINTER(EpPlan), P, P, P]),
    "ep_last_picks": (B, [C.POINTER(EpPlan), P, P]),
    "lane_ffn_rows": (B, [C.POINTER(LaneLayer), C.POINTER(LaneScratch), P, P, P, P, U32, U32, U32, P]),
}


class Lib:
    def __init__(self, path=LIB_PATH):
        if not os.path.exists(path):
            raise RuntimeError(
                "libosmos_b200.so is not built (%s): run `python -m libosmos_b200.build`; there is no fallback" % path)
        self.path = path
        self.dll = C.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(self.dll, name)  # AttributeError = the library does not export what the headers declare
            fn.restype, fn.argtypes = res, args
            setattr(self, name, fn)


_LIB = None


def load():
    global _LIB
    if _LIB is None:
        _LIB = Lib()
    return _LIB
