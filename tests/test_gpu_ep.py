"""Expert-parallel step against the single-GPU layer: on 2 GPUs (both exchanges; skipped on a one-GPU box), on one
GPU as a world of one rank (the device-initiated kernels with the own region as the only peer), and the bounded
wait for a peer's flag running out.  The orchestration itself is also covered on CPU ranks by tests/test_ep_cpu.py."""
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


def test_ep_peer_exchange_world_of_one():
    """msk_ep_step with one rank: dispatch into the own region, experts with the flag waits and peer-row stores,
    reduce - must reproduce the single-GPU layer on the same requests, over several steps (both buffer parities)."""
    sys.path.insert(0, os.path.dirname(HERE))
    from muse_spark_open_b200 import abi, ep, layer, synth
    dev = torch.device("cuda", 0)
    w = synth.make_layer_weights(3, dev, hidden=1024, hq=8, hkv=1, d=128, n_experts=16, inner=128, bias_std=0.5)
    seqs = [300, 70, 129, 1000, 64, 5, 2047, 512] * 5  # 40 tokens: the gathered-rows path of the experts
    data = synth.make_layer_input(4, dev, seqs, hidden=1024, hq=8, hkv=1, d=128)
    ref_in = dict(data, k_cache=data["k_cache"].clone(), v_cache=data["v_cache"].clone())
    ref_hidden, ref_stream, ref_ids = layer.kernel_fn(ref_in, layer.prepare(w))
    ops = ep.CudaOps(w, 0, 1, 16, exchange="peer")
    for _ in range(3):
        hidden, stream, ids = ep.step(data, ops)
        torch.cuda.synchronize()
        abi.status_for(dev).raise_if_set("ep world 1")
        assert torch.equal(ids, ref_ids)
        torch.testing.assert_close(stream, ref_stream, rtol=1e-4, atol=1e-4)
        torch.testing.assert_close(hidden.float(), ref_hidden.float(), rtol=2e-2, atol=1e-2)
    ops.peer.close()


def test_flag_wait_times_out_and_reports():
    """A wait for a flag that no peer ever sets: the kernel must give up after its budget, record the timeout in the
    status word and return; the context stays usable (nothing traps, nothing hangs)."""
    from muse_spark_open_b200 import abi
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    rc = abi.lib().msk_selftest_flag_timeout(flag.data_ptr(), 2_000_000, status.data_ptr(), None)  # ~1 ms of SM clocks
    assert rc == 0
    torch.cuda.synchronize()
    s = status.tolist()
    assert s[0] == 1 and (s[1] >> 8) == 8, s   # timeout, reported by the expert-parallel kernels
    assert float(torch.ones(4, device="cuda").sum()) == 4.0  # the device still answers
