"""msk_router through the C ABI against an FP64 statement of the two routing rules, over token counts that take the
few-token kernel (K splits and expert tiles, two ticket stages) and the many-token kernel (whole expert range per
block, one ticket), ragged last token groups and expert counts below 128."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu
TOP_K = 8
MULT = 0.1767766952966369


def _run(t, h, e, sigmoid, seed):
    from muse_spark_open_b200 import abi
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(seed)
    x = torch.randn((t, h), generator=g, device=dev)
    w = (0.1 * torch.randn((h,), generator=g, device=dev)).to(torch.bfloat16)
    r = 0.05 * torch.randn((e, h), generator=g, device=dev)
    bias = 0.5 * torch.randn((e,), generator=g, device=dev)
    ssq = torch.zeros((2, t), device=dev)
    ssq[0] = (x * x).sum(-1)
    part = torch.empty((h // 128, t, e), device=dev)
    ticket = torch.zeros((((t + 31) // 32) * ((e + 31) // 32 + 1),), dtype=torch.int32, device=dev)
    logits = torch.empty((t, e), device=dev)
    ids = torch.empty((t, TOP_K), dtype=torch.int32, device=dev)
    wts = torch.empty((t, TOP_K), device=dev)
    p = abi.RouterParams()
    p.x, p.norm_w, p.ssq, p.ssq_parts, p.eps = abi.ptr(x), abi.ptr(w), abi.ptr(ssq), 1, 1e-6
    p.router_w, p.router_bias, p.E, p.T, p.H, p.top_k = abi.ptr(r), abi.ptr(bias), e, t, h, TOP_K
    p.sigmoid_bias, p.multiplier = int(sigmoid), MULT
    p.part, p.ticket, p.logits = abi.ptr(part), abi.ptr(ticket), abi.ptr(logits)
    p.topk_ids, p.topk_weights, p.pdl = abi.ptr(ids), abi.ptr(wts), 0
    st = abi.status_for(dev)
    for _ in range(2):  # the second call finds the tickets as the first left them
        abi.check(abi.lib().msk_router(C.byref(p), st.p, abi.stream_ptr()), "msk_router")
    torch.cuda.synchronize()
    st.raise_if_set("router")
    assert int(ticket.abs().sum()) == 0
    # FP64 statement
    xd = x.double()
    hn = xd * torch.rsqrt((xd * xd).mean(-1, keepdim=True) + 1e-6) * (1.0 + w.double())
    lg = hn @ r.double().T
    if sigmoid:
        scores = torch.sigmoid(lg * MULT)
        pick = scores + bias.double()
        want_logits = lg
    else:
        want_logits = lg + bias.double()
        pick = want_logits
    torch.testing.assert_close(logits.double(), want_logits, rtol=1e-4, atol=1e-4)
    assert torch.allclose(ssq[1], ssq[0])
    top = pick.topk(TOP_K, -1)
    got = ids.long()
    same = got == top.indices
    # a differing id is accepted only where the FP64 values that choose are within 1e-4 of each other
    for tt, kk in (~same).nonzero().tolist():
        assert abs(float(pick[tt, got[tt, kk]] - top.values[tt, kk])) < 1e-4, (tt, kk)
    for tt in range(t):
        assert len(set(got[tt].tolist())) == TOP_K
    chosen = torch.gather(scores if sigmoid else torch.softmax(want_logits, -1), 1, got)
    want_w = chosen / (chosen.sum(-1, keepdim=True) + (1e-15 if sigmoid else 0.0))
    torch.testing.assert_close(wts.double(), want_w, rtol=2e-4, atol=1e-6)


@pytest.mark.parametrize("t", [1, 31, 64, 70, 100, 128, 150, 256])
@pytest.mark.parametrize("sigmoid", [False, True])
def test_router_matches_fp64(t, sigmoid):
    _run(t, 4096, 128, sigmoid, seed=t)


def test_router_fewer_experts_and_narrow_hidden():
    _run(200, 1024, 96, False, seed=3)   # many tokens, 96 experts: the last quarter of every lane's experts is empty
    _run(160, 2048, 128, True, seed=4)
    _run(40, 1024, 16, False, seed=5)    # few tokens, one expert tile
