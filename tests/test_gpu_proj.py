"""Skinny projection through the C ABI against the oracle (FP64 accumulate -> BF16)."""
import pytest
import torch

from oracle import proj as oproj

pytestmark = pytest.mark.gpu


def _check(out, ref, rtol=2e-2, atol=1e-2):
    torch.testing.assert_close(out.float().cpu(), ref.float(), rtol=rtol, atol=atol)


@pytest.mark.parametrize("m,n,k,splits", [(16, 6144, 4096, 0), (1, 256, 128, 1), (3, 384, 512, 2), (32, 4096, 4096, 4),
                                          (17, 200, 192, 3), (33, 1024, 1024, 8), (256, 512, 1024, 2), (200, 384, 512, 0),
                                          (256, 9216, 4096, 0), (96, 4096, 4096, 0)])
def test_proj_matches_oracle(m, n, k, splits):
    from muse_spark_open_b200 import abi, proj
    x, w = oproj.make_input(m, n, k, seed=m + n, probes=True)
    state = proj.prepare({"w": w.cuda()})
    out = proj.kernel_fn({"x": x.cuda(), "config": {"m": m, "n": n, "k": k, "layer": "w"}}, state) if splits == 0 \
        else proj.skinny(x.cuda(), w.cuda(), splits=splits)
    torch.cuda.synchronize()
    abi.status_for("cuda").raise_if_set("proj")
    ref = oproj.ref_kernel(x, w)
    assert out.dtype == torch.bfloat16 and tuple(out.shape) == (m, n)
    _check(out, ref, rtol=1e-2, atol=1e-2)
    rows = oproj.probe_rows(x)
    if len(rows):  # single power-of-two input: the output row is an exact weight column
        assert torch.equal(out.cpu()[rows], ref[rows])


def test_proj_golden(golden):
    from muse_spark_open_b200 import abi, proj
    for name, item in golden("proj").items():
        cfg = item["config"]
        state = proj.prepare({cfg["layer"]: item["w"].cuda()})
        out = proj.kernel_fn({"x": item["x"].cuda(), "config": cfg}, state)
        torch.cuda.synchronize()
        abi.status_for("cuda").raise_if_set(name)
        ref = item["expect_out"]
        assert out.dtype == ref.dtype and out.shape == ref.shape, name
        err = (out.cpu().double() - ref.double()).norm() / ref.double().norm()
        assert err < (1e-4 if cfg["layer"] == "router" else 1e-2), (name, float(err))


@pytest.mark.parametrize("m,splits,token_splits", [(5, 2, 0), (130, 2, 3), (256, 1, 0), (77, 3, 1)])
def test_proj_fused_epilogue(m, splits, token_splits):
    """Row scale from partial sums of squares, FP32 residual, next op's input and per-tile sums of squares, with
    K splits (partials through the workspace), token splits (each CTA its own tokens) and both."""
    from muse_spark_open_b200 import abi, proj
    n, k = 384, 256
    g = torch.Generator().manual_seed(3)
    xs = torch.randn((m, k), generator=g)
    nw = (0.1 * torch.randn((k,), generator=g)).to(torch.bfloat16)
    x_un = (xs * (1 + nw.float())).to(torch.bfloat16)            # un-normalised, weight applied
    ssq = torch.stack([xs[:, :100].pow(2).sum(-1), xs[:, 100:].pow(2).sum(-1)])  # two partial sums
    w = (torch.randn((n, k), generator=g) / 16).to(torch.bfloat16)
    resid = torch.randn((m, n), generator=g)
    nxt = (0.1 * torch.randn((n,), generator=g)).to(torch.bfloat16)
    out = torch.empty((m, n), dtype=torch.float32, device="cuda")
    normed = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    oss = torch.zeros((3, m), dtype=torch.float32, device="cuda")
    proj.skinny(x_un.cuda(), w.cuda(), out=out, splits=splits, token_splits=token_splits, in_ssq=ssq.cuda(), in_dim=k, in_eps=1e-5,
                resid=resid.cuda(), next_norm_w=nxt.cuda(), out_normed=normed, out_ssq=oss)
    torch.cuda.synchronize()
    abi.status_for("cuda").raise_if_set("proj epilogue")
    rs = torch.rsqrt(xs.pow(2).mean(-1, keepdim=True) + 1e-5)
    want = (x_un.float() @ w.float().T) * rs + resid
    _check(out, want, rtol=1e-3, atol=1e-3)
    _check(normed, want * (1 + nxt.float()))
    torch.testing.assert_close(oss.sum(0).cpu(), want.pow(2).sum(-1), rtol=1e-3, atol=1e-3)


def test_proj_more_than_256_tokens():
    """Token counts beyond a decode / verify step (the reference's m = 512 and 1000 cases) run as blocks of 256 rows."""
    from muse_spark_open_b200 import abi, proj
    for m in (512, 1000):
        x, w = oproj.make_input(m, 384, 256, seed=m)
        state = proj.prepare({"w": w.cuda()})
        out = proj.kernel_fn({"x": x.cuda(), "config": {"m": m, "n": 384, "k": 256, "layer": "w"}}, state)
        torch.cuda.synchronize()
        abi.status_for("cuda").raise_if_set("proj blocks")
        assert tuple(out.shape) == (m, 384)
        _check(out, oproj.ref_kernel(x, w), rtol=1e-2, atol=1e-2)
