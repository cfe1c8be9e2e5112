"""Toy products through each tensor-core operand path (descriptor / swizzle / TMEM layout checks)."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(mode, a, b, n):
    from muse_spark_open_b200 import abi
    d = torch.full((128, n), float("nan"), dtype=torch.float32, device="cuda")
    st = abi.status_for("cuda")
    rc = abi.lib().msk_selftest_umma(mode, C.c_void_p(a.data_ptr()), C.c_void_p(b.data_ptr()),
                                     C.c_void_p(d.data_ptr()), n, st.p, abi.stream_ptr())
    abi.check(rc, "msk_selftest_umma")
    torch.cuda.synchronize()
    st.raise_if_set(f"selftest mode {mode}")
    return d.cpu()


@pytest.mark.parametrize("n", [16, 32, 128])
def test_bf16_ss_tma(n):
    g = torch.Generator().manual_seed(n)
    a = torch.randint(-8, 9, (128, 64), generator=g).to(torch.bfloat16)
    b = torch.randint(-8, 9, (n, 64), generator=g).to(torch.bfloat16)
    d = _run(0, a.cuda(), b.cuda(), n)
    assert torch.equal(d, a.float() @ b.float().T)


@pytest.mark.parametrize("n", [16, 128])
def test_bf16_ts_tmem_operand(n):
    g = torch.Generator().manual_seed(100 + n)
    a = torch.randint(-8, 9, (128, 64), generator=g).to(torch.bfloat16)
    b = torch.randint(-8, 9, (n, 64), generator=g).to(torch.bfloat16)
    d = _run(3, a.cuda(), b.cuda(), n)
    assert torch.equal(d, a.float() @ b.float().T)


def _fp8_cache(seed):
    g = torch.Generator().manual_seed(seed)
    cache = torch.randint(-6, 7, (2, 64, 1, 128), generator=g).float().to(torch.float8_e4m3fn)
    keys = torch.cat([cache[1, :, 0], cache[0, :, 0]]).float()  # tile rows 0..63 = page 1, 64..127 = page 0
    return cache, keys


@pytest.mark.parametrize("n", [16, 128])
def test_e4m3_scores_k_major(n):
    cache, keys = _fp8_cache(7)
    g = torch.Generator().manual_seed(8)
    q = torch.randint(-6, 7, (n, 128), generator=g).float().to(torch.float8_e4m3fn)
    d = _run(1, cache.cuda(), q.cuda(), n)
    assert torch.equal(d, keys @ q.float().T)  # [128 keys, n]


@pytest.mark.parametrize("n", [16, 128])
def test_e4m3_values_mn_major(n):
    cache, vals = _fp8_cache(9)
    g = torch.Generator().manual_seed(10)
    p = torch.randint(0, 5, (n, 128), generator=g).float().to(torch.float8_e4m3fn)  # [n, keys]
    d = _run(2, cache.cuda(), p.cuda(), n)
    assert torch.equal(d, vals.T @ p.float().T)  # [128 d, n]
