"""NVFP4 routed experts through the C ABI against the oracle and the reference's golden outputs."""
import pytest
import torch

from oracle import moe as omoe
from oracle import nvfp4

pytestmark = pytest.mark.gpu
FP8 = torch.float8_e4m3fn


def _dev(d):
    return {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in d.items()}


def _run(data, weights, **kw):
    from muse_spark_open_b200 import abi, moe
    state = moe.prepare(_dev(weights), weights_start=data["config"].get("weights_start", 0))
    dd = _dev(data)
    out = moe.kernel_fn(dd, state)
    torch.cuda.synchronize()
    abi.status_for("cuda").raise_if_set("moe")
    return out.cpu(), state, dd


def test_dequant_is_bit_exact():
    from muse_spark_open_b200 import moe
    w = omoe.make_weights(2, n_experts=2, hidden=256, inner=128)
    # every code and a spread of scales, zero blocks and subnormal scales included
    g = torch.Generator().manual_seed(1)
    w["w13"] = torch.randint(0, 256, w["w13"].shape, dtype=torch.uint8, generator=g)
    sf = torch.randint(0, 127, w["w13_sf"].shape, dtype=torch.uint8, generator=g)
    sf[0, 0, :4] = torch.tensor([0, 1, 7, 126], dtype=torch.uint8)
    w["w13_sf"] = sf.view(FP8)
    state = moe.prepare(_dev(w))
    got = moe.dequant(state["w13"], 2, 256, 256, gate_up=True).cpu()
    want = nvfp4.dequantize_tile_bf16(w["w13"], w["w13_sf"])
    assert torch.equal(got.view(torch.int16), want.view(torch.int16)) or torch.equal(got.float(), want.float())
    got2 = moe.dequant(state["w2"], 2, 256, 128).cpu()
    assert torch.equal(got2.float(), nvfp4.dequantize_tile_bf16(w["w2"], w["w2_sf"]).float())


@pytest.mark.parametrize("tokens,n_exp,hidden,inner,top_k", [(6, 16, 256, 128, 4), (1, 8, 512, 256, 8), (32, 16, 256, 128, 8),
                                                            (70, 8, 256, 256, 8), (256, 8, 256, 128, 8)])
def test_moe_small_matches_oracle(tokens, n_exp, hidden, inner, top_k):
    weights = omoe.make_weights(tokens, n_experts=n_exp, hidden=hidden, inner=inner, std=0.05)
    data = omoe.make_input(tokens, tokens + 1, n_experts=n_exp, hidden=hidden, top_k=top_k)
    out, _, _ = _run(data, weights)
    ref = omoe.ref_kernel(data, weights)
    torch.testing.assert_close(out.float(), ref.float(), rtol=2e-2, atol=1e-2)


def test_moe_local_range_and_untouched_tokens():
    weights = omoe.make_weights(5, n_experts=16, hidden=256, inner=128, std=0.05)
    data = omoe.make_input(9, 6, n_experts=16, hidden=256, top_k=4, local_start=4, local_count=4)
    out, _, _ = _run(data, weights)
    ref = omoe.ref_kernel(data, weights)
    torch.testing.assert_close(out.float(), ref.float(), rtol=2e-2, atol=1e-2)
    untouched = ~((data["topk_ids"] >= 4) & (data["topk_ids"] < 8)).any(-1)
    assert (out[untouched] == 0).all()


def test_moe_reference_golden(golden):
    blob = golden("moe")
    weights = dict(blob["weights"])
    for k in ("w13_sf", "w2_sf"):
        weights[k] = weights[k].view(FP8)
    for name in ("full_normal", "ep_skewed"):
        item = blob[name]
        out, _, _ = _run(item["data"], weights)
        ref = item["expect_out"]
        err = (out.float() - ref.float()).norm() / ref.float().norm()
        assert err < 1.5e-2, (name, float(err))  # the reference's own bound (reference.py:25)
        torch.testing.assert_close(out.float(), ref.float(), rtol=2e-2, atol=1e-2, msg=name)


def test_moe_routing_from_logits_in_kernel():
    from muse_spark_open_b200 import abi, moe
    weights = omoe.make_weights(11, n_experts=128, hidden=256, inner=128, std=0.05)
    data = omoe.make_input(32, 12, n_experts=128, hidden=256)
    state = moe.prepare(_dev(weights))
    dd = _dev(data)
    ids = torch.full_like(dd["topk_ids"], -1)
    wts = torch.zeros_like(dd["topk_weights"])
    out = moe.forward(dd["hidden_states"], ids, wts, state, 0, 128, logits=dd["router_logits"].contiguous())
    torch.cuda.synchronize()
    abi.status_for("cuda").raise_if_set("moe logits")
    # top-k ids are exact (sets equal; order follows descending probability like torch.topk)
    assert torch.equal(ids.cpu().sort(-1).values, data["topk_ids"].sort(-1).values)
    assert torch.equal(ids.cpu(), data["topk_ids"])
    torch.testing.assert_close(wts.cpu(), data["topk_weights"], rtol=1e-5, atol=1e-7)
    torch.testing.assert_close(out.float().cpu(), omoe.ref_kernel(data, weights).float(), rtol=2e-2, atol=1e-2)


def test_moe_expert_parallel_rank_shape():
    """What one of 8 expert-parallel ranks runs: all 256 tokens of the step, 16 local experts of the benchmark's
    shape (few expert-groups, so gemm 1 runs with 4 K splits and the gathered input rows)."""
    weights = omoe.make_weights(3, n_experts=128, hidden=4096, inner=768)
    data = omoe.make_input(256, 4, local_start=32, local_count=16)
    out, _, _ = _run(data, weights)
    ref = omoe.ref_kernel(data, weights)
    torch.testing.assert_close(out.float(), ref.float(), rtol=2e-2, atol=1e-2)
    untouched = ~((data["topk_ids"] >= 32) & (data["topk_ids"] < 48)).any(-1)
    assert (out[untouched] == 0).all()


def test_moe_benchmark_shape():
    """32 tokens, hidden 4096, 128 experts of gate_up [1536, 4096] / down [4096, 768], softmax top-8."""
    weights = omoe.make_weights(0, n_experts=128, hidden=4096, inner=768)
    data = omoe.make_input(32, 0)
    out, state, dd = _run(data, weights)
    ref = omoe.ref_kernel(data, weights)
    torch.testing.assert_close(out.float(), ref.float(), rtol=2e-2, atol=1e-2)
    from muse_spark_open_b200 import moe
    again = moe.kernel_fn(dd, state).cpu()
    assert torch.equal(out, again)  # bitwise reproducible


def test_moe_more_than_256_tokens():
    """257 tokens (a case of the reference's list, muse_moe_w4a16/bench.py:15): blocks of 256 tokens."""
    weights = omoe.make_weights(7, n_experts=8, hidden=256, inner=128, std=0.05)
    data = omoe.make_input(257, 8, n_experts=8, hidden=256)
    out, _, _ = _run(data, weights)
    torch.testing.assert_close(out.float(), omoe.ref_kernel(data, weights).float(), rtol=2e-2, atol=1e-2)
