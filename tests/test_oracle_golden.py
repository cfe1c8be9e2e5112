"""The oracle must reproduce the reference's own outputs stored under tests/golden/
(made by tests/golden/make_golden.py from the reference's ref_kernel functions on CPU)."""
import torch

from oracle import attention, moe, nvfp4, proj

FP8 = torch.float8_e4m3fn


def _attn_data(item):
    data = {k: v for k, v in item.items() if not k.startswith("expect_")}
    for k in ("k_cache", "v_cache"):
        data[k] = data[k].view(FP8)
    data.setdefault("scheduler_metadata", None)
    return data


def test_attention_matches_reference(golden):
    cases = golden("attention")
    assert len(cases) >= 4
    for name, item in cases.items():
        out, k_new, v_new = attention.ref_kernel(_attn_data(item))
        assert torch.equal(k_new.view(torch.uint8), item["expect_k_new"]), name
        assert torch.equal(v_new.view(torch.uint8), item["expect_v_new"]), name
        torch.testing.assert_close(out, item["expect_out"], rtol=1e-5, atol=1e-6, msg=name)


def test_attention_new_slots_match_cache_loc(golden):
    for name, item in golden("attention").items():
        data = _attn_data(item)
        assert torch.equal(attention.new_slots(data).reshape(-1), item["cache_loc"]), name


def _moe_weights(blob):
    w = dict(blob)
    for k in ("w13_sf", "w2_sf"):
        w[k] = w[k].view(FP8)
    return w


def test_moe_matches_reference(golden):
    blob = golden("moe")
    weights = _moe_weights(blob["weights"])
    for name in ("full_normal", "ep_skewed"):
        item = blob[name]
        out = moe.ref_kernel(item["data"], weights)
        assert out.dtype == torch.bfloat16
        torch.testing.assert_close(out.float(), item["expect_out"].float(), rtol=2e-2, atol=1e-6, msg=name)
        # identical up to BF16 rounding of an FP32 sum taken in another order
        assert (out != item["expect_out"]).float().mean() < 0.01, name


def test_nvfp4_codec_bit_exact(golden):
    c = golden("moe")["codec"]
    packed, sf, gs = nvfp4.quantize(c["x"])
    assert torch.equal(packed, c["packed"])
    assert torch.equal(sf.view(torch.uint8), c["sf"])
    assert torch.equal(gs, c["gs"])
    assert torch.equal(nvfp4.e2m1_values(c["packed"]), c["unpacked"])
    assert torch.equal(nvfp4.dequantize(c["packed"], c["sf"].view(FP8), c["gs"]), c["dequant"])
    # midpoints go to the smaller magnitude, beyond 6 clamps, zero has no sign
    v = nvfp4.e2m1_values(nvfp4.pack_codes(torch.tensor([[0.25, 0.75, 2.5, 5.0, 7.0, -9.0, -0.1, 1.25]])))
    assert v.tolist() == [[0.0, 0.5, 2.0, 4.0, 6.0, -6.0, 0.0, 1.0]]


def test_nvfp4_products_exact_in_bf16():
    e2m1 = torch.tensor(nvfp4.E2M1_VALUES[1:])
    e4m3 = torch.arange(1, 127, dtype=torch.uint8).view(FP8).float()
    prod = e2m1[:, None] * e4m3[None, :]
    assert torch.equal(prod.to(torch.bfloat16).float(), prod)
    assert prod.min() == 2.0 ** -10 and prod.max() == 2688.0


def test_proj_matches_reference(golden):
    for name, item in golden("proj").items():
        fp32 = item["config"]["layer"] == "router"
        n = item["config"]["n"]
        out = proj.ref_kernel(item["x"], item["w"][:n], fp32_out=fp32)
        assert torch.equal(out, item["expect_out"]), name


def test_quant_e4m3_saturates():
    x = torch.tensor([448.0, 460.0, 1000.0, -5000.0])
    assert attention.quant_e4m3(x, 1.0).float().tolist() == [448.0, 448.0, 448.0, -448.0]


def test_native_layer_matches_reference(golden):
    """The layer in the reference's own form (norm-preserving gated residuals, sigmoid + bias routing, pooler /
    sliced unpooler) against the reference's ref_front / ref_back outputs (tests/golden/layer.pt)."""
    from oracle import layer
    blob = golden("layer")
    weights = dict(blob["weights"])
    for k in ("w13_sf", "w2_sf"):
        weights[k] = weights[k].view(FP8)
    for name in ("full_decode", "sliding_verify"):
        item = blob[name]
        data = {k: v for k, v in item.items() if not k.startswith("expect_")}
        for k in ("k_cache", "v_cache"):
            data[k] = data[k].view(FP8)
        fr = layer.native_front(data, weights)
        torch.testing.assert_close(fr["stream1"], item["expect_stream1"], rtol=1e-5, atol=1e-5, msg=name)
        torch.testing.assert_close(fr["scores"], item["expect_scores"], rtol=1e-5, atol=1e-6, msg=name)
        assert (fr["k_new"].view(torch.uint8) != item["expect_k_new"]).float().mean() < 2e-3, name
        hidden, stream, ids, _, _ = layer.native_ref_kernel(data, weights)
        assert torch.equal(ids.long().sort(-1).values, item["expect_ids"].long().sort(-1).values), name
        torch.testing.assert_close(stream, item["expect_stream"], rtol=1e-4, atol=1e-4, msg=name)
        assert (hidden != item["expect_hidden"]).float().mean() < 0.01, name
