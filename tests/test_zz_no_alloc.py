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


def test_static_scratch_entry_point_rejects_oversize():
    from muse_spark_open_b200 import abi
    p = abi.MoeParams()
    p.T, p.top_k, p.H, p.I, p.s1, p.s2 = 256, 8, 4096, 768, 1, 1  # 11.5 M floats of partials: far over 1 Mi
    rc = abi.lib().msk_moe_forward_static(C.byref(p), None, None)
    assert rc == -3
