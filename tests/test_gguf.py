"""The GGUF reader (include/osmos_b200/gguf.h) against files written by gguf-py and against damaged files: what the
reference's tests/test_gguf.c checks - a round trip of every value type, split models, truncation at every length,
corrupted counts, duplicate names, the two readings of type 43 - through the C ABI."""
import ctypes as C
import os
import struct

import numpy as np
import pytest

gguf = pytest.importorskip("gguf")

from libosmos_b200 import api, synth  # noqa: E402


def _open(lib, path, header=False):
    err = C.create_string_buffer(256)
    g = (lib.gguf_header if header else lib.gguf_create)(str(path).encode(), err)
    return g, err.value.decode()


def _write_model(path, tensors, kv=(), arrays=()):
    w = gguf.GGUFWriter(str(path), "test")
    for key, kind, val in kv:
        getattr(w, "add_" + kind)(key, val)
    for key, val in arrays:
        w.add_array(key, val)
    for name, arr, qt in tensors:
        w.add_tensor(name, arr, raw_dtype=qt)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()


def _blocks(tid, rows, cols, key):
    v, b = synth.BLOCK[tid]
    return synth.random_tensor(tid, rows, cols, synth.rng_for(900, key)).reshape(rows, cols // v * b)


def test_round_trip(lib, tmp_path):
    GG = gguf.GGMLQuantizationType
    f32 = np.arange(12, dtype=np.float32).reshape(3, 4)
    q8 = _blocks(8, 2, 64, 1)
    iq1m = _blocks(29, 2, 256, 2)
    q6k = _blocks(14, 3, 512, 3)
    path = tmp_path / "m.gguf"
    _write_model(path, [("a.f32", f32, None), ("b.q8_0", q8, GG.Q8_0), ("c.iq1_m", iq1m, GG.IQ1_M), ("d.q6_k", q6k, GG.Q6_K)],
                 kv=[("t.u8", "uint8", 200), ("t.i8", "int8", -5), ("t.u16", "uint16", 60000), ("t.i16", "int16", -300),
                     ("t.u32", "uint32", 4000000000), ("t.i32", "int32", -7), ("t.f32", "float32", 1.5), ("t.bool", "bool", True),
                     ("t.str", "string", "hello"), ("t.u64", "uint64", 2 ** 63 + 5), ("t.i64", "int64", -2 ** 40),
                     ("t.f64", "float64", 2.25)],
                 arrays=[("t.ints", [3, -1, 4]), ("t.strs", ["ab", "", "cde"])])
    g, err = _open(lib, path)
    assert g, err
    G = g.contents
    assert G.n_files == 1 and G.paths[0].decode() == str(path) and G.sizes[0] == os.path.getsize(path)
    kv = lambda k: lib.gguf_kv(g, k.encode()).contents
    assert kv("t.u8").v.u == 200 and kv("t.i8").v.i == -5 and kv("t.u16").v.u == 60000 and kv("t.i16").v.i == -300
    assert kv("t.u32").v.u == 4000000000 and kv("t.i32").v.i == -7 and kv("t.f32").v.f == 1.5 and kv("t.bool").v.u == 1
    assert kv("t.str").v.s == b"hello" and kv("t.u64").v.u == 2 ** 63 + 5 and kv("t.i64").v.i == -2 ** 40 and kv("t.f64").v.f == 2.25
    out = C.c_int64()
    assert lib.gguf_int(lib.gguf_kv(g, b"t.i16"), 0, C.byref(out)) and out.value == -300
    assert not lib.gguf_int(lib.gguf_kv(g, b"t.u64"), 0, C.byref(out))  # past int64
    assert not lib.gguf_int(lib.gguf_kv(g, b"t.f32"), 0, C.byref(out))
    ints = lib.gguf_kv(g, b"t.ints")
    assert ints.contents.type == 9 and ints.contents.n == 3
    assert [lib.gguf_int(ints, i, C.byref(out)) and out.value for i in range(3)] == [3, -1, 4]
    assert not lib.gguf_int(ints, 3, C.byref(out))
    strs = kv("t.strs")
    assert strs.type == 9 and strs.item == 8 and strs.n == 3
    assert [C.cast(strs.v.items, C.POINTER(C.c_char_p))[i] for i in range(3)] == [b"ab", b"", b"cde"]
    assert not lib.gguf_kv(g, b"absent") and not lib.gguf_tensor(g, b"absent")
    data = open(path, "rb").read()
    for name, arr, tid, dims in (("a.f32", f32, 0, [4, 3]), ("b.q8_0", q8, 8, [64, 2]), ("c.iq1_m", iq1m, 29, [256, 2]),
                                 ("d.q6_k", q6k, 14, [512, 3])):
        t = lib.gguf_tensor(g, name.encode()).contents
        assert t.type == tid and t.n_dims == 2 and list(t.dims[:2]) == dims and t.file == 0
        assert t.bytes == arr.nbytes == lib.gguf_bytes(tid, dims[0] * dims[1]) and t.offset % 32 == 0
        assert data[t.offset:t.offset + t.bytes] == arr.tobytes()  # the tensor's bytes lie where the reader says
    lib.gguf_destroy(g)
    lib.gguf_destroy(None)


def test_bytes_by_type(lib):
    assert lib.gguf_bytes(12, 512) == 288 and lib.gguf_bytes(12, 500) == 0 and lib.gguf_bytes(12, 0) == 0
    assert lib.gguf_bytes(0, 7) == 28 and lib.gguf_bytes(30, 7) == 14 and lib.gguf_bytes(26, 3) == 12 and lib.gguf_bytes(27, 3) == 24
    assert lib.gguf_bytes(43, 64) == 66 and lib.gguf_bytes(0x12B, 64) == 64 and lib.gguf_bytes(1, 64) == 0 and lib.gguf_bytes(999, 64) == 0
    assert lib.gguf_bytes(27, 2 ** 62) == 0  # a byte count past 64 bits


# ---- files built by hand: what gguf-py will not write ----------------------------------------------------------------
def _s(b):
    return struct.pack("<Q", len(b)) + b


def _file(tensors, kv=b"", n_kv=0, align=32, version=3, data=None):
    """tensors: (name, type, dims, offset); the data section: `data` bytes (default: enough for every tensor)"""
    head = struct.pack("<IIQQ", 0x46554747, version, len(tensors), n_kv) + kv
    for name, typ, dims, off in tensors:
        head += _s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", typ, off)
    head += b"\0" * (-len(head) % align)
    return head + (data if data is not None else bytes(4096))


def _kv_u16(key, v):
    return _s(key) + struct.pack("<IH", 2, v)


def test_truncated_at_every_length(lib, tmp_path):
    kv = _s(b"k.str") + struct.pack("<I", 8) + _s(b"value") + _s(b"k.arr") + struct.pack("<IIQ", 9, 8, 2) + _s(b"x") + _s(b"yz")
    whole = _file([(b"w", 8, [64, 2], 0)], kv, 2, data=bytes(136))
    path = tmp_path / "t.gguf"
    path.write_bytes(whole)
    g, err = _open(lib, path)
    assert g, err
    lib.gguf_destroy(g)
    for n in range(len(whole)):  # every shorter file is refused, with a reason, and nothing crashes
        path.write_bytes(whole[:n])
        g, err = _open(lib, path)
        assert not g and "t.gguf" in err, n


@pytest.mark.parametrize("what", ["magic", "version", "n_kv", "n_tensors", "key_len", "str_len", "arr_len", "arr_type", "value_type",
                                  "dims", "dim_zero", "dim_overflow", "type", "blocks", "offset", "duplicate", "alignment"])
def test_corrupt(lib, tmp_path, what):
    huge = 2 ** 62
    tensors, kv, n_kv, ver = [(b"w", 8, [64, 2], 0)], _s(b"k") + struct.pack("<I", 8) + _s(b"v"), 1, 3
    raw = None
    if what == "magic":
        raw = b"GGUX" + _file(tensors, kv, n_kv)[4:]
    elif what == "version":
        ver = 7
    elif what == "n_kv":
        n_kv = huge
    elif what == "n_tensors":
        raw = bytearray(_file(tensors, kv, n_kv))
        raw[8:16] = struct.pack("<Q", huge)
    elif what == "key_len":
        kv = struct.pack("<Q", huge) + b"k" + struct.pack("<I", 8) + _s(b"v")
    elif what == "str_len":
        kv = _s(b"k") + struct.pack("<I", 8) + struct.pack("<Q", huge) + b"v"
    elif what == "arr_len":
        kv = _s(b"k") + struct.pack("<IIQ", 9, 4, huge)
    elif what == "arr_type":
        kv = _s(b"k") + struct.pack("<IIQ", 9, 9, 1)
    elif what == "value_type":
        kv = _s(b"k") + struct.pack("<I", 77)
    elif what == "dims":
        tensors = [(b"w", 8, [32, 1, 1, 1, 1], 0)]
    elif what == "dim_zero":
        tensors = [(b"w", 8, [64, 0], 0)]
    elif what == "dim_overflow":
        tensors = [(b"w", 8, [2 ** 40, 2 ** 40], 0)]
    elif what == "type":
        tensors = [(b"w", 1, [64, 2], 0)]  # F16 is not a type this library reads
    elif what == "blocks":
        tensors = [(b"w", 8, [33, 1], 0)]
    elif what == "offset":
        tensors = [(b"w", 8, [64, 2], 1 << 40)]
    elif what == "duplicate":
        tensors = [(b"w", 8, [64, 2], 0), (b"w", 8, [64, 2], 160)]
    elif what == "alignment":
        kv, n_kv = _s(b"general.alignment") + struct.pack("<II", 4, 48), 1
    path = tmp_path / "c.gguf"
    path.write_bytes(bytes(raw) if raw is not None else _file(tensors, kv, n_kv, version=ver))
    g, err = _open(lib, path)
    assert not g and err.startswith(str(path)), (what, err)


def test_tensor_past_the_end(lib, tmp_path):
    path = tmp_path / "e.gguf"
    path.write_bytes(_file([(b"w", 8, [64, 2], 0)], data=bytes(135)))  # 136 bytes wanted
    g, err = _open(lib, path)
    assert not g and "leave the file" in err


def test_custom_alignment(lib, tmp_path):
    kv = _s(b"general.alignment") + struct.pack("<II", 4, 64)
    path = tmp_path / "a.gguf"
    path.write_bytes(_file([(b"w", 0, [5], 0), (b"v", 0, [3], 64)], kv, 1, align=64))
    g, err = _open(lib, path)
    assert g, err
    w, v = lib.gguf_tensor(g, b"w").contents, lib.gguf_tensor(g, b"v").contents
    assert w.offset % 64 == 0 and v.offset == w.offset + 64 and w.bytes == 20 and v.bytes == 12
    lib.gguf_destroy(g)


def test_type_43_both_ways(lib, tmp_path):
    """a type-43 tensor is MXFP8 (33 bytes a 32 values) where that fits its room, and one E4M3 byte a value where only
    that does (id 0x12B)"""
    path = tmp_path / "f8.gguf"
    path.write_bytes(_file([(b"mx", 43, [64, 2], 0), (b"f8", 43, [64, 2], 160), (b"z", 0, [4], 288)], data=bytes(304)))
    g, err = _open(lib, path)
    assert g, err
    mx, f8 = lib.gguf_tensor(g, b"mx").contents, lib.gguf_tensor(g, b"f8").contents
    assert mx.type == 43 and mx.bytes == 132 and f8.type == 0x12B and f8.bytes == 128
    lib.gguf_destroy(g)


def test_split_model(lib, tmp_path):
    def shard(no, count, tensors):
        kv = _kv_u16(b"split.no", no) + _kv_u16(b"split.count", count) + _s(b"general.name") + struct.pack("<I", 8) + _s(b"m%d" % no)
        return _file(tensors, kv, 3)
    p1, p2, p3 = (tmp_path / ("m-%05d-of-00003.gguf" % i) for i in (1, 2, 3))
    p1.write_bytes(shard(0, 3, [(b"a", 0, [8], 0)]))
    p2.write_bytes(shard(1, 3, [(b"b", 8, [64, 2], 0), (b"c", 0, [2], 160)]))
    p3.write_bytes(shard(2, 3, [(b"d", 0, [4], 0)]))
    g, err = _open(lib, p1)
    assert g, err
    G = g.contents
    assert G.n_files == 3 and [G.paths[i].decode() for i in range(3)] == [str(p1), str(p2), str(p3)] and G.n_tensors == 4
    assert [lib.gguf_tensor(g, n).contents.file for n in (b"a", b"b", b"c", b"d")] == [0, 1, 1, 2]
    assert lib.gguf_kv(g, b"general.name").contents.v.s == b"m0"  # the first shard's metadata
    lib.gguf_destroy(g)
    h, err = _open(lib, p1, header=True)  # one file alone: no sibling opened
    assert h and h.contents.n_files == 1 and h.contents.n_tensors == 1
    lib.gguf_destroy(h)
    g, err = _open(lib, p2)
    assert not g and "first" in err  # not the first shard
    p3.unlink()
    g, err = _open(lib, p1)
    assert not g and "00003-of-00003" in err  # a shard is missing
    h, err = _open(lib, p1, header=True)
    assert h
    lib.gguf_destroy(h)
    p3.write_bytes(shard(2, 3, [(b"a", 0, [4], 0)]))  # a name another shard has
    g, err = _open(lib, p1)
    assert not g and "twice" in err
    p3.write_bytes(shard(1, 3, [(b"d", 0, [4], 0)]))  # the wrong shard number
    g, err = _open(lib, p1)
    assert not g and "shard" in err


def test_missing_file(lib, tmp_path):
    g, err = _open(lib, tmp_path / "nope.gguf")
    assert not g and "cannot open" in err


@pytest.mark.gpu
def test_a_tensor_through_quant_dequant(lib, dev, oracle, tmp_path):
    """a written model's tensor, found by the reader, decoded on the GPU where its bytes lie in the file's image"""
    import torch
    GG = gguf.GGMLQuantizationType
    q6k = _blocks(14, 4, 512, 9)
    path = tmp_path / "g.gguf"
    _write_model(path, [("x.q6_k", q6k, GG.Q6_K)])
    g, err = _open(lib, path)
    assert g, err
    t = lib.gguf_tensor(g, b"x.q6_k").contents
    image = torch.from_numpy(np.frombuffer(open(path, "rb").read(), dtype=np.uint8).copy()).to(dev)
    out = torch.empty(4 * 512, dtype=torch.float32, device=dev)
    assert lib.quant_dequant(t.type, image.data_ptr() + t.offset, 4 * 512, out.data_ptr(), None)
    torch.cuda.synchronize()
    want = oracle.dequant(14, q6k.reshape(-1), 4 * 512)
    assert np.array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32))
    lib.gguf_destroy(g)
