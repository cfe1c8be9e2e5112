"""StepPipeline: steps fed from pinned host memory through copy streams give, bit for bit, what the same steps give
when their inputs are copied in and their results copied out on the compute stream."""
import pytest
import torch

from oracle import layer as olayer

pytestmark = pytest.mark.gpu


def _dev(d):
    return {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in d.items()}


def test_pipelined_steps_match_serial_steps():
    from muse_spark_open_b200 import abi, layer
    from muse_spark_open_b200.pipeline import StepPipeline
    weights = olayer.make_weights(3, hidden=1024, hq=8, hkv=1, d=128, n_experts=16, inner=128)
    state = layer.prepare(_dev(weights))
    data = _dev(olayer.make_input(5, [70, 300, 5, 1000, 129], 7, q_len=1, hidden=1024, hq=8, hkv=1, d=128, window=0,
                                  rope_theta=0.0))
    keys = ("stream", "seq_lens", "cache_loc", "page_table")
    steps = 7
    gen = torch.Generator().manual_seed(5)
    host_in = []
    for _ in range(steps):
        h = {k: data[k].cpu().pin_memory() for k in keys}
        h["stream"] = torch.randn(data["stream"].shape, generator=gen).pin_memory()
        host_in.append(h)
    # serial: everything on the current stream
    want = []
    for h in host_in:
        for k in keys:
            data[k].copy_(h[k], non_blocking=True)
        hidden, stream, ids = layer.kernel_fn(data, state)
        want.append((hidden.cpu(), stream.cpu(), ids.cpu()))
    torch.cuda.synchronize()
    # pipelined: a separate set of pinned result buffers per step, read after the drain
    pipe = StepPipeline(lambda: layer.kernel_fn(data, state), data, keys, 3)
    host_out = [tuple(torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in want[0]) for _ in range(steps)]
    for h, o in zip(host_in, host_out):
        pipe.submit(h, o)
    pipe.drain()
    torch.cuda.synchronize()
    abi.status_for("cuda").raise_if_set("pipeline")
    for i in range(steps):
        for a, b in zip(host_out[i], want[i]):
            assert torch.equal(a, b), i


def test_pipeline_skips_results_without_a_host_buffer():
    from muse_spark_open_b200 import layer
    from muse_spark_open_b200.pipeline import StepPipeline
    weights = olayer.make_weights(3, hidden=1024, hq=8, hkv=1, d=128, n_experts=16, inner=128)
    state = layer.prepare(_dev(weights))
    data = _dev(olayer.make_input(2, [40, 200], 7, q_len=1, hidden=1024, hq=8, hkv=1, d=128, window=0, rope_theta=0.0))
    keys = ("stream",)
    h = {"stream": data["stream"].cpu().pin_memory()}
    hidden, _, ids = layer.kernel_fn(data, state)
    torch.cuda.synchronize()
    pipe = StepPipeline(lambda: layer.kernel_fn(data, state), data, keys, 3)
    hid_h = torch.empty(hidden.shape, dtype=hidden.dtype).pin_memory()
    ids_h = torch.empty(ids.shape, dtype=ids.dtype).pin_memory()
    for _ in range(3):
        pipe.submit(h, (hid_h, None, ids_h))
    pipe.drain()
    torch.cuda.synchronize()
    assert torch.equal(hid_h, hidden.cpu()) and torch.equal(ids_h, ids.cpu())
