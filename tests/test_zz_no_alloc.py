"""The allocation-free expert entry point (collected last on purpose: a run that stops at the first
failure has then already run every other test).

Some hosts of this library own all device memory themselves or must not stall a decode step on an
allocation, so they can neither pass scratch buffers nor let the library call cudaMalloc.
`msk_moe_forward_static` serves them from a fixed array inside the library.  Here it is called through
the C ABI twice in a row, with different inputs, and each result must equal what the ordinary entry
point (caller-provided scratch) gives for the same inputs."""
import ctypes as C

import pytest
import torch

from oracle import moe as omoe

pytestmark = pytest.mark.gpu


def _dev(d):
    return {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in d.items()}


def test_static_scratch_entry_point_matches_ordinary_one_twice():
    from muse_spark_open_b200 import abi, moe
    weights = omoe.make_weights(21, n_experts=16, hidden=512, inner=256, std=0.05)
    state = moe.prepare(_dev(weights))
    for seed, tokens in ((31, 8), (32, 5)):  # the second call finds the first call's partials in the array
        data = _dev(omoe.make_input(tokens, seed, n_experts=16, hidden=512))
        x, ids, wts = data["hidden_states"], data["topk_ids"], data["topk_weights"]
        want = moe.forward(x, ids, wts, state, 0, 16)
        got = torch.full_like(want, float("nan"))
        moe.forward_no_alloc(x, ids, wts, state, 0, 16, got)
        torch.cuda.synchronize()
        abi.status_for("cuda").raise_if_set("no-alloc experts")
        torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=1e-2)
        ref = omoe.ref_kernel({k: (v.cpu() if isinstance(v, torch.Tensor) else v) for k, v in data.items()}, weights)
        torch.testing.assert_close(got.float().cpu(), ref.float(), rtol=2e-2, atol=1e-2)


def test_static_scratch_entry_point_gathered_rows_and_limit():
    """More than 32 tokens (the gathered input rows then also live in the built-in array), and the size limit: a
    call that needs exactly what `static_scratch_bytes` says is served while it fits in 4 MiB, the first token
    count beyond is refused by both the wrapper and the library."""
    from muse_spark_open_b200 import abi, moe
    weights = omoe.make_weights(22, n_experts=8, hidden=256, inner=128, std=0.05)
    state = moe.prepare(_dev(weights))
    data = _dev(omoe.make_input(40, 33, n_experts=8, hidden=256))
    x, ids, wts = data["hidden_states"], data["topk_ids"], data["topk_weights"]
    want = moe.forward(x, ids, wts, state, 0, 8)
    got = torch.full_like(want, float("nan"))
    moe.forward_no_alloc(x, ids, wts, state, 0, 8, got)
    torch.cuda.synchronize()
    abi.status_for("cuda").raise_if_set("no-alloc experts, 40 tokens")
    torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=1e-2)
    # the largest token count that fits, and the next one
    fits = max(t for t in range(1, 257) if moe.static_scratch_bytes(t, 8, 256, 128, 1, 1) <= moe.STATIC_SCRATCH_BYTES)
    assert fits < 256
    for t, ok in ((fits, True), (fits + 1, False)):
        d = _dev(omoe.make_input(t, 40 + t, n_experts=8, hidden=256))
        out = torch.empty((t, 256), dtype=torch.bfloat16, device="cuda")
        if ok:
            moe.forward_no_alloc(d["hidden_states"], d["topk_ids"], d["topk_weights"], state, 0, 8, out)
            torch.cuda.synchronize()
            ref = moe.forward(d["hidden_states"], d["topk_ids"], d["topk_weights"], state, 0, 8)
            torch.testing.assert_close(out.float(), ref.float(), rtol=2e-2, atol=1e-2)
        else:
            with pytest.raises(abi.MskError):
                moe.forward_no_alloc(d["hidden_states"], d["topk_ids"], d["topk_weights"], state, 0, 8, out)
            p = abi.MoeParams()
            p.T, p.top_k, p.H, p.I, p.s1, p.s2 = t, 8, 256, 128, 1, 1
            assert abi.lib().msk_moe_forward_static(C.byref(p), None, None) == -3


def test_static_scratch_entry_point_rejects_oversize():
    from muse_spark_open_b200 import abi
    p = abi.MoeParams()
    p.T, p.top_k, p.H, p.I, p.s1, p.s2 = 256, 8, 4096, 768, 1, 1  # 11.5 M floats of partials: far over 1 Mi
    rc = abi.lib().msk_moe_forward_static(C.byref(p), None, None)
    assert rc == -3
