"""The expert-parallel layer on two GPUs, both transports: each rank checks all its home tokens' output against the CPU
checker's bits inside bench.py before timing (it exits non-zero on a mismatch or a wait that ran out). Needs two GPUs;
skipped on one."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("transport", ["peer", "nccl"])
def test_two_rank_layer_matches_oracle(transport):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, OSMOS_EP_TRANSPORT=transport, NCCL_NVLS_ENABLE="0")
    port = 29600 + (os.getpid() + (0 if transport == "peer" else 1)) % 200
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "bench.py"), "--gpus", "2", "--steps", "6",
           "--warmup", "3"]
    run = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stdout[-2000:] + run.stderr[-2000:]
    line = json.loads([l for l in run.stdout.splitlines() if l.startswith("{")][-1])
    assert line["n_gpus"] == 2 and line["value"] > 0 and line["run"]["transport"].startswith(transport)
