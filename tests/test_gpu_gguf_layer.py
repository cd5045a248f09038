"""From a file to the kernels: a layer's experts written to a GGUF by gguf-py, found through gguf_create and weights_ffn,
their bytes read at the offsets the reader gives, run through the fused layer step - with the bits of the CPU lane on
the tensors the file was written from."""
import ctypes as C

import numpy as np
import pytest
import torch

gguf = pytest.importorskip("gguf")

import bench  # noqa: E402
from helpers import same_bits, sync, to_dev  # noqa: E402
from libosmos_b200 import api, ep, synth, workloads  # noqa: E402

pytestmark = pytest.mark.gpu


def test_layer_from_a_gguf_file(lib, dev, tmp_path):
    cfg = dict(name="gguf_layer", type="IQ3_XXS", n_exp=16, k=4, n_tok=8, dim=512, ff=512, sigma=0.005, lim=1.0e30)
    E, D, FF = cfg["n_exp"], cfg["dim"], cfg["ff"]
    host = workloads.moe_layer_host(cfg)
    path = tmp_path / "layer.gguf"
    w = gguf.GGUFWriter(str(path), "test")
    qt = gguf.GGMLQuantizationType.IQ3_XXS
    for name, arr, rows in (("ffn_gate_exps", host[0], FF), ("ffn_up_exps", host[1], FF), ("ffn_down_exps", host[2], D)):
        w.add_tensor("blk.7.%s.weight" % name, arr.reshape(E, rows, -1), raw_dtype=qt)
    w.add_tensor("blk.7.ffn_gate_inp.weight", np.zeros((E, D), dtype=np.float32))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()

    err = C.create_string_buffer(256)
    g = lib.gguf_create(str(path).encode(), err)
    assert g, err.value.decode()
    fw = api.FfnWeights()
    assert lib.weights_ffn(g, 7, fw, err), err.value.decode()
    assert (fw.n_embd, fw.expert_ff, fw.n_experts) == (D, FF, E)
    read = []
    for t, per in zip((fw.exp_gate, fw.exp_up, fw.exp_down), fw.expert_bytes):
        t = t.contents
        assert t.type == synth.TYPE_ID["IQ3_XXS"] and t.bytes == E * per
        read.append(np.fromfile(g.contents.paths[t.file].decode(), dtype=np.uint8, count=t.bytes, offset=t.offset))
    lib.gguf_destroy(g)
    assert all(np.array_equal(a, b) for a, b in zip(read, host))

    layer = ep.EpMoeLane(lib, cfg, dev, 0, 1, host_tensors=tuple(read))
    x, logits = workloads.moe_inputs_host(cfg, 0)
    out = torch.empty((cfg["n_tok"], D), dtype=torch.float32, device=dev)
    layer.step(to_dev(x, dev), to_dev(logits, dev), out, 0, torch.cuda.current_stream().cuda_stream)
    sync()
    ids, wts = layer.last_picks()
    assert same_bits(out.cpu().numpy(), bench.CpuArm(cfg, host).layer(x, ids, wts))
    assert lib.ep_wait_status() == 0 and lib.q8_status() == 0
    layer.close()
