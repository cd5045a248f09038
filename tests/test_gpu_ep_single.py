"""The expert-parallel layer's own kernels on one GPU: a process group of one rank, so every "peer" is this GPU - the
dispatch push, the flags and waits, the unpack, the expert rows, the scatter to the (own) home buffer and the ordered
combine all run, and the output must have the bits of the plain single-GPU layer (tests/test_gpu_ep_peer.py runs
the same layer on two GPUs where there are two)."""
import os

import numpy as np
import pytest
import torch

from libosmos_b200 import ep, runner, workloads

pytestmark = pytest.mark.gpu

SMALL = dict(name="moe_small", type="IQ3_XXS", n_exp=16, k=4, n_tok=24, dim=512, ff=256, sigma=0.005, lim=1.0e30)


@pytest.mark.parametrize("transport", ["peer", "nccl"])
def test_one_rank_group_has_the_single_gpu_bits(lib, dev, transport):
    import torch.distributed as dist
    created = False
    if not dist.is_initialized():
        port = 29700 + os.getpid() % 200
        dist.init_process_group("nccl", init_method="tcp://127.0.0.1:%d" % port, rank=0, world_size=1, device_id=dev)
        created = True
    try:
        cfg = SMALL
        host = workloads.moe_layer_host(cfg)
        plain = runner.MoeLane(lib, cfg, dev, host_tensors=host)
        layer = ep.EpMoeLane(lib, cfg, dev, 0, 1, host_tensors=host, transport=transport)
        stream = torch.cuda.current_stream().cuda_stream
        want = torch.empty((cfg["n_tok"], cfg["dim"]), dtype=torch.float32, device=dev)
        got = torch.empty_like(want)
        for step in range(3):  # both halves of the exchange buffers, and a reuse
            x, logits = workloads.moe_inputs_host(cfg, step)
            xd, ld = torch.from_numpy(x).to(dev), torch.from_numpy(logits).to(dev)
            plain.step(xd, ld, want, cfg["n_tok"], 0, stream)
            layer.step(xd, ld, got, 0, stream)
            torch.cuda.synchronize()
            assert np.array_equal(got.cpu().numpy().view(np.uint32), want.cpu().numpy().view(np.uint32))
        assert lib.ep_wait_status() == 0 and lib.q8_status() == 0
        layer.close()
    finally:
        if created:
            dist.destroy_process_group()
