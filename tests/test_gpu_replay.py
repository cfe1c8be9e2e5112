"""Graph-replay stress: an op captured once into a CUDA graph, replayed with FRESH inputs copied into the SAME
buffers and an L2 flush before every replay, must give bit for bit what an eager call gives on those inputs.

This is how the reference hunts stale-data bugs between programmatically chained kernels (its
muse_moe_w4a16/tools/stress.py:12-37 and muse_attention_decode/tools/astress.py:18-39 replay a captured graph
with new inputs and demand bitwise equality): a consumer that starts under its producer and reads the previous
replay's data from L1, or a scratch buffer that keeps state between calls, shows up as a mismatch here and
nowhere else."""
import pytest
import torch

from oracle import attention as oattn
from oracle import layer as olayer
from oracle import moe as omoe

pytestmark = pytest.mark.gpu
REPLAYS = 6


def _dev(d):
    return {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in d.items()}


def _capture(fn):
    from muse_spark_open_b200 import timing
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        fn()  # first call outside the capture: one-time set-up (function attributes, scratch allocation)
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            fn()
    torch.cuda.current_stream().wait_stream(stream)
    torch.cuda.synchronize()
    return g, timing.flush_buffer()


def test_experts_graph_replay_with_fresh_inputs():
    from muse_spark_open_b200 import abi, moe, timing
    weights = omoe.make_weights(5, n_experts=16, hidden=512, inner=256, std=0.05)
    state = moe.prepare(_dev(weights))
    for tokens in (8, 40):  # tokens as columns / rows gathered in expert-list order
        first = _dev(omoe.make_input(tokens, 100, n_experts=16, hidden=512))
        x, ids, wts = first["hidden_states"].clone(), first["topk_ids"].clone(), first["topk_weights"].clone()
        out = torch.empty((tokens, 512), dtype=torch.bfloat16, device="cuda")
        g, flush = _capture(lambda: moe.forward(x, ids, wts, state, 0, 16, out=out))
        for r in range(REPLAYS):
            new = _dev(omoe.make_input(tokens, 101 + r, n_experts=16, hidden=512))
            x.copy_(new["hidden_states"]), ids.copy_(new["topk_ids"]), wts.copy_(new["topk_weights"])
            out.fill_(float("nan"))
            timing.flush_l2(flush)
            g.replay()
            torch.cuda.synchronize()
            got = out.clone()
            want = moe.forward(new["hidden_states"], new["topk_ids"], new["topk_weights"], state, 0, 16)
            torch.cuda.synchronize()
            abi.status_for("cuda").raise_if_set("experts replay")
            assert torch.equal(got, want), (tokens, r)
            ref = omoe.ref_kernel({k: (v.cpu() if isinstance(v, torch.Tensor) else v) for k, v in new.items()}, weights)
            torch.testing.assert_close(got.float().cpu(), ref.float(), rtol=2e-2, atol=1e-2)


def test_attention_graph_replay_with_fresh_inputs():
    from muse_spark_open_b200 import abi, attention, timing
    base = oattn.make_input(6, [700, 64, 1500, 129, 2047, 5], seed=9, q_len=1, hq=16, hkv=2, window=0, rope_theta=0.0)
    dev = oattn.to_device(base, "cuda")
    pristine_k, pristine_v = dev["k_cache"].clone(), dev["v_cache"].clone()
    cfg = dev["config"]
    qkv = dev["qkv"].view(6, -1).clone()
    out = torch.empty((6, 16 * 128), dtype=torch.bfloat16, device="cuda")
    g, flush = _capture(lambda: attention.launch(qkv, out, dev, cfg))
    gen = torch.Generator(device="cuda").manual_seed(3)
    for r in range(REPLAYS):
        fresh = (2 * torch.randn(qkv.shape, generator=gen, device="cuda")).to(torch.bfloat16)
        results = []
        for how in ("graph", "eager"):
            dev["k_cache"].copy_(pristine_k), dev["v_cache"].copy_(pristine_v)  # the step writes its new rows in place
            qkv.copy_(fresh)
            out.fill_(float("nan"))
            timing.flush_l2(flush)
            if how == "graph":
                g.replay()
            else:
                attention.launch(qkv, out, dev, cfg)
            torch.cuda.synchronize()
            results.append((out.clone(), dev["k_cache"].view(torch.uint8).clone()))
        abi.status_for("cuda").raise_if_set("attention replay")
        assert torch.equal(results[0][0], results[1][0]) and torch.equal(results[0][1], results[1][1]), r
        assert not torch.isnan(results[0][0].float()).any()


def test_layer_graph_replay_with_fresh_inputs():
    from muse_spark_open_b200 import abi, layer, timing
    weights = olayer.make_weights(3, hidden=1024, hq=8, hkv=1, d=128, n_experts=16, inner=128)
    state = layer.prepare(_dev(weights))
    data = _dev(olayer.make_input(5, [70, 300, 5, 1000, 129], 7, q_len=1, hidden=1024, hq=8, hkv=1, d=128, window=0,
                                  rope_theta=0.0))
    pristine_k, pristine_v = data["k_cache"].clone(), data["v_cache"].clone()
    outs = {}

    def step():
        outs["r"] = layer.kernel_fn(data, state)

    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        step()
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            step()
    torch.cuda.current_stream().wait_stream(stream)
    torch.cuda.synchronize()
    graph_out = outs["r"]  # the tensors the captured step writes
    flush = timing.flush_buffer()
    gen = torch.Generator(device="cuda").manual_seed(11)
    for r in range(REPLAYS):
        fresh = torch.randn(data["stream"].shape, generator=gen, device="cuda")
        data["k_cache"].copy_(pristine_k), data["v_cache"].copy_(pristine_v)
        data["stream"].copy_(fresh)
        timing.flush_l2(flush)
        g.replay()
        torch.cuda.synchronize()
        got = [t.clone() for t in graph_out]
        data["k_cache"].copy_(pristine_k), data["v_cache"].copy_(pristine_v)
        want = layer.kernel_fn(data, state)
        torch.cuda.synchronize()
        abi.status_for("cuda").raise_if_set("layer replay")
        for a, b in zip(got, want):
            assert torch.equal(a, b), r
