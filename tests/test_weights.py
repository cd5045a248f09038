"""A layer's feed-forward tensors out of a GGUF (include/osmos_b200/weights.h): files written with gguf-py, taken through the
C ABI - the parts found and their sizes derived, and each of the reference's refusals (src/model/weights.c:205-246) with
the tensor's name and the reason in the same words."""
import ctypes as C

import numpy as np
import pytest

gguf = pytest.importorskip("gguf")

from libosmos_b200 import api, synth  # noqa: E402

GG = gguf.GGMLQuantizationType
D, FF, E, SF = 512, 256, 6, 768  # hidden, expert width, experts, the shared expert's width


def _raw(tid, shape, cols, key):
    """random blocks of type tid for a tensor whose rows are cols values long: uint8 [..., row bytes]"""
    v, b = synth.BLOCK[tid]
    rows = int(np.prod(shape))
    return synth.random_tensor(tid, rows, cols, synth.rng_for(910, key)).reshape(*shape, cols // v * b)


def _layer(layer=3, shared=True, bias=True, norm=True, exp_type=(18, GG.IQ3_XXS), drop=(), replace=None):
    tid, qt = exp_type
    p = "blk.%d." % layer
    t = {
        p + "ffn_gate_exps.weight": (_raw(tid, (E, FF), D, 1), qt),
        p + "ffn_up_exps.weight": (_raw(tid, (E, FF), D, 2), qt),
        p + "ffn_down_exps.weight": (_raw(tid, (E, D), FF, 3), qt),
        p + "ffn_gate_inp.weight": (np.ones((E, D), dtype=np.float32), None),
    }
    if norm:
        t[p + "ffn_norm.weight"] = (np.ones(D, dtype=np.float32), None)
    if bias:
        t[p + "exp_probs_b.bias"] = (np.zeros(E, dtype=np.float32), None)
    if shared:
        t[p + "ffn_gate_shexp.weight"] = (_raw(12, (SF,), D, 4), GG.Q4_K)
        t[p + "ffn_up_shexp.weight"] = (_raw(12, (SF,), D, 5), GG.Q4_K)
        t[p + "ffn_down_shexp.weight"] = (_raw(12, (D,), SF, 6), GG.Q4_K)
    for name in drop:
        del t[p + name]
    for name, val in (replace or {}).items():
        t[p + name] = val
    return t


def _take(lib, tmp_path, tensors, layer=3):
    path = tmp_path / "layer.gguf"
    w = gguf.GGUFWriter(str(path), "test")
    for name, (arr, qt) in tensors.items():
        w.add_tensor(name, arr, raw_dtype=qt)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    err = C.create_string_buffer(256)
    g = lib.gguf_create(str(path).encode(), err)
    assert g, err.value.decode()
    out = api.FfnWeights()
    ok = lib.weights_ffn(g, layer, out, err)
    return g, ok, out, err.value.decode()


def test_whole_layer(lib, tmp_path):
    g, ok, w, err = _take(lib, tmp_path, _layer())
    assert ok, err
    assert (w.n_embd, w.expert_ff, w.n_experts, w.shared_ff) == (D, FF, E, SF)
    per = FF * D // 256 * 98  # IQ3_XXS: 98 bytes a 256 values
    assert list(w.expert_bytes) == [per, per, per]
    assert w.exp_gate.contents.name == b"blk.3.ffn_gate_exps.weight" and list(w.exp_gate.contents.dims[:3]) == [D, FF, E]
    assert w.exp_down.contents.bytes == E * per and list(w.exp_down.contents.dims[:3]) == [FF, D, E]
    assert w.router.contents.type == 0 and w.router_bias.contents.bytes == 4 * E and w.ffn_norm.contents.bytes == 4 * D
    assert w.sh_down.contents.type == 12 and list(w.sh_down.contents.dims[:2]) == [SF, D]
    # an expert's matrix lies a whole number of experts into its tensor, inside its file
    t = w.exp_up.contents
    assert t.offset + t.bytes <= g.contents.sizes[t.file] and t.offset % 32 == 0
    lib.gguf_destroy(g)


def test_optional_parts_absent(lib, tmp_path):
    g, ok, w, err = _take(lib, tmp_path, _layer(shared=False, bias=False, norm=False, exp_type=(39, GG.MXFP4)))
    assert ok, err
    assert not w.sh_gate and not w.sh_up and not w.sh_down and not w.router_bias and not w.ffn_norm and w.shared_ff == 0
    assert w.exp_gate.contents.type == 39 and w.expert_bytes[0] == FF * D // 32 * 17
    lib.gguf_destroy(g)


@pytest.mark.parametrize("case,name,why", [
    (dict(drop=("ffn_up_exps.weight",)), "blk.3.ffn_up_exps.weight", "missing"),
    (dict(drop=("ffn_gate_inp.weight",)), "blk.3.ffn_gate_inp.weight", "missing"),
    (dict(drop=("ffn_down_shexp.weight",)), "blk.3.ffn_down_shexp.weight", "missing"),
    (dict(replace={"ffn_down_exps.weight": ("down_as_gate", None)}), "blk.3.ffn_down_exps.weight", "of another shape"),
    (dict(replace={"exp_probs_b.bias": (np.zeros(E + 1, dtype=np.float32), None)}), "blk.3.exp_probs_b.bias", "of another shape"),
    (dict(replace={"ffn_norm.weight": ("q8_0", None)}), "blk.3.ffn_norm.weight", "of a type this role does not take"),
    (dict(replace={"ffn_up_exps.weight": (np.ones((E, FF, D), dtype=np.float32), None)}), "blk.3.ffn_up_exps.weight",
     "of a type this role does not take"),
])
def test_refusals(lib, tmp_path, case, name, why):
    tensors = _layer(**{k: v for k, v in case.items() if k == "drop"})
    for key, (val, qt) in case.get("replace", {}).items():
        if isinstance(val, str) and val == "down_as_gate":  # the down tensor with the gate's shape
            val, qt = _raw(18, (E, FF), D, 9), GG.IQ3_XXS
        elif isinstance(val, str) and val == "q8_0":  # the norm as a quantized vector
            val, qt = _raw(8, (), D, 7), GG.Q8_0
        tensors["blk.3." + key] = (val, qt)
    g, ok, w, err = _take(lib, tmp_path, tensors)
    assert not ok and err == "%s: %s" % (name, why)
    assert not w.exp_gate and w.n_embd == 0  # nothing half-filled
    lib.gguf_destroy(g)


def test_another_layer_and_bad_arguments(lib, tmp_path):
    g, ok, w, err = _take(lib, tmp_path, _layer(layer=3), layer=4)
    assert not ok and err == "blk.4.ffn_gate_exps.weight: missing"
    out = api.FfnWeights()
    assert not lib.weights_ffn(g, -1, out, None) and not lib.weights_ffn(None, 0, out, None)
    lib.gguf_destroy(g)
