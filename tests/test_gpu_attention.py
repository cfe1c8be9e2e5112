"""Gated attention decode / verify through the C ABI against the oracle and the reference's golden outputs."""
import pytest
import torch

from oracle import attention as oattn

pytestmark = pytest.mark.gpu
FP8 = torch.float8_e4m3fn


def _run(data, **kw):
    from muse_spark_open_b200 import abi, attention
    dev = oattn.to_device(data, "cuda")
    dev["k_cache"], dev["v_cache"] = dev["k_cache"].clone(), dev["v_cache"].clone()
    out = attention.kernel_fn(dev, **kw)
    torch.cuda.synchronize()
    abi.status_for("cuda").raise_if_set("attention")
    slots = oattn.new_slots(data)
    hkv, d = data["config"]["num_kv_heads"], data["config"]["head_dim"]
    k_new = dev["k_cache"].view(-1, hkv, d)[slots.cuda()].cpu()
    v_new = dev["v_cache"].view(-1, hkv, d)[slots.cuda()].cpu()
    return out.cpu(), k_new, v_new, dev


def _check_cache(got, want, what):
    """E4M3 bytes equal except where the pre-round FP32 value sat within an ulp of a rounding boundary."""
    g, w = got.view(torch.uint8), want.view(torch.uint8)
    diff = g != w
    assert diff.float().mean() < 5e-3, (what, float(diff.float().mean()))
    if diff.any():
        gf, wf = got.float()[diff], want.float()[diff]
        assert ((gf - wf).abs() <= 0.13 * wf.abs() + 2.0 ** -9).all(), what


def _check(data, out, k_new, v_new, what):
    ref, rk, rv = oattn.ref_kernel(data)
    _check_cache(k_new, rk, what + " keys")
    _check_cache(v_new, rv, what + " values")
    # compare with the oracle attending the kernel's own new entries (as the reference's checker does)
    ref = oattn.ref_kernel(data, new_kv=(k_new, v_new))[0].to(torch.bfloat16)
    torch.testing.assert_close(out.float(), ref.float(), rtol=2e-2, atol=1e-2, msg=lambda m: f"{what}: {m}")


CASES = [
    # batch, seq_lens, q_len, window, chunks
    ("decode_short", 2, [10, 70], 1, 1024, 1),
    ("decode_window_edges", 4, [1023, 1024, 1025, 2047], 1, 1024, 0),
    ("decode_page_edges", 5, [63, 64, 65, 127, 128], 1, 1024, 2),
    ("decode_full_attn", 3, [3000, 129, 1], 1, 0, 4),
    ("decode_empty_cache", 2, [0, 5], 1, 1024, 8),
    ("verify_short", 2, [10, 200], 8, 1024, 1),
    ("verify_window", 3, [1020, 1500, 3001], 8, 1024, 0),
    ("verify_full", 2, [700, 2500], 8, 0, 4),
    ("verify_empty_cache", 1, [0], 8, 1024, 2),
]


@pytest.mark.parametrize("name,batch,seqs,q_len,window,chunks", CASES)
def test_attention_matches_oracle(name, batch, seqs, q_len, window, chunks):
    data = oattn.make_input(batch, seqs, seed=len(name) + batch, q_len=q_len, hq=16, hkv=2, d=128, page=64,
                            window=window, rope_theta=1e6 if window else 0.0)
    out, k_new, v_new, _ = _run(data, chunks=chunks)
    _check(data, out, k_new, v_new, name)


def test_attention_benchmark_shapes():
    """32 / 4 heads, 16 requests with context uniform in [1024, 8192], window 1024, page 64: decode and verify."""
    for q_len in (1, 8):
        data = oattn.make_input(16, (1024, 8192), seed=0, q_len=q_len)
        out, k_new, v_new, _ = _run(data)
        _check(data, out, k_new, v_new, f"benchmark q_len={q_len}")


def test_attention_grid_beyond_one_wave():
    """80 requests x 4 KV heads with very uneven contexts, full attention: more CTAs than the GPU holds at once, so
    every CTA ranks the context lengths and takes the requests longest first, and the one long context makes the
    launch split every request's keys over two CTAs.  This is the branch the 256-request step runs in."""
    g = torch.Generator().manual_seed(17)
    seqs = torch.randint(64, 1501, (80,), generator=g).tolist()
    seqs[37] = 4500   # 36 tiles of 128 keys: the "long contexts" rule picks two chunks
    seqs[5] = seqs[6]  # a tie in the ranking
    data = oattn.make_input(80, seqs, seed=23, q_len=1, window=0, rope_theta=0.0)
    out, k_new, v_new, _ = _run(data)
    _check(data, out, k_new, v_new, "beyond one wave")
    # the same requests through one chunk per request and through four: the order of the slices must not matter
    for chunks in (1, 4):
        out_c = _run(data, chunks=chunks)[0]
        torch.testing.assert_close(out_c.float(), out.float(), rtol=2e-2, atol=1e-2)


def test_attention_outlier_cache_and_small_scale():
    data = oattn.make_input(3, [900, 1500, 64], seed=5, q_len=8, hq=8, hkv=1, cache_dist="outliers", kv_scale=1 / 64)
    out, k_new, v_new, _ = _run(data)
    _check(data, out, k_new, v_new, "outliers")


@pytest.mark.parametrize("page", [16, 32, 128])
def test_attention_page_sizes(page):
    data = oattn.make_input(2, [300, 1100], seed=page, q_len=1, hq=8, hkv=1, page=page)
    out, k_new, v_new, _ = _run(data)
    _check(data, out, k_new, v_new, f"page {page}")


def test_attention_reference_golden(golden):
    """The reference's own outputs (head_dim 128 cases of tests/golden/attention.pt)."""
    n = 0
    for name, item in golden("attention").items():
        if item["config"]["head_dim"] != 128:
            continue
        data = {k: v for k, v in item.items() if not k.startswith("expect_")}
        for k in ("k_cache", "v_cache"):
            data[k] = data[k].view(FP8)
        out, k_new, v_new, _ = _run(data)
        _check_cache(k_new, item["expect_k_new"].view(FP8), name)
        _check_cache(v_new, item["expect_v_new"].view(FP8), name)
        ref = oattn.ref_kernel(data, new_kv=(k_new, v_new))[0]
        torch.testing.assert_close(out.float(), ref.to(torch.bfloat16).float(), rtol=2e-2, atol=1e-2, msg=name)
        # and against the stored reference output itself, with the reference's relative-L2 bound floor
        want = item["expect_out"].reshape(out.shape)
        err = (out.float() - want).norm() / want.norm()
        assert err < 0.03, (name, float(err))
        n += 1
    assert n >= 3


def test_attention_replay_is_bitwise_stable():
    data = oattn.make_input(4, [2000, 1500, 1024, 3000], seed=3, q_len=1)
    a = _run(data)[0]
    b = _run(data)[0]
    assert torch.equal(a, b)


@pytest.mark.parametrize("q_len,stages", [(1, 3), (1, 4), (1, 5), (1, 6), (8, 3), (8, 4)])
def test_attention_ring_depths(q_len, stages):
    """Every ring depth the launch accepts (the library itself picks 3 for decode and 4 for verify): slots and barrier
    parities wrap at different tiles, the result must not change."""
    data = oattn.make_input(3, [1500, 129, 2900], seed=21, q_len=q_len, hq=16, hkv=2, d=128, page=64, window=0,
                            rope_theta=0.0)
    base = _run(data, chunks=1)[0]
    out, k_new, v_new, _ = _run(data, chunks=1, stages=stages)
    assert torch.equal(out, base), (q_len, stages)
    _check(data, out, k_new, v_new, f"stages {stages}")


def test_attention_rejects_ring_depths_that_do_not_fit():
    from muse_spark_open_b200 import abi, attention
    data = oattn.make_input(1, [300], seed=3, q_len=8, hq=16, hkv=2, d=128, page=64, window=0, rope_theta=0.0)
    dev = oattn.to_device(data, "cuda")
    for stages in (2, 5, 7):  # below the minimum; beyond shared memory for the verify form; beyond the maximum
        with pytest.raises(abi.MskError):
            attention.kernel_fn(dev, stages=stages)
