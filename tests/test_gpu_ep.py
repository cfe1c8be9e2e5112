"""Expert-parallel step on 2 GPUs (NCCL) against the single-GPU layer.  Skipped on a one-GPU box; the
orchestration itself is also covered on CPU ranks by tests/test_ep_cpu.py."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_ep_two_gpus_match_single_gpu_layer():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29531", os.path.join(HERE, "ep_worker.py")],
                       capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "EP_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
