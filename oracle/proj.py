"""Skinny BF16 projection and FP32 router projection, restated (oracle; test infrastructure only)."""
from __future__ import annotations

import torch


def ref_kernel(x: torch.Tensor, w: torch.Tensor, fp32_out: bool = False) -> torch.Tensor:
    """out = x @ W^T accumulated in FP64, cast to BF16 (FP32 for the router).

    x bf16 [M, K]; W [N, K] bf16 (or fp32 for the router).  muse_bf16_proj/reference.py:72-76.
    """
    out = x.double() @ w.double().T
    return out.to(torch.float32 if fp32_out else torch.bfloat16)


def make_input(m: int, n: int, k: int, seed: int, w_std: float = 0.02, probes: bool = False):
    """The benchmark's config: x ~ N(0,1) bf16 [m,k], W ~ N(0, w_std) bf16 [n,k], CPU generator, seed.

    probes=True replaces about one row in eight of x by a single power-of-two entry, so that the
    output row is an exact weight column (muse_bf16_proj/reference.py:61-68).
    """
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn((m, k), generator=gen)
    w = (w_std * torch.randn((n, k), generator=gen)).to(torch.bfloat16)
    if probes:
        pick = torch.rand((m,), generator=gen) < 1 / 8
        if m >= 8:
            pick[torch.randint(m, (1,), generator=gen)] = True
        cols = torch.randint(k, (m,), generator=gen)
        sign = torch.randint(2, (m,), generator=gen) * 2 - 1
        power = torch.randint(3, 8, (m,), generator=gen)
        spike = torch.zeros_like(x).scatter_(1, cols[:, None], (sign * 2.0 ** power).float()[:, None])
        x = torch.where(pick[:, None], spike, x)
    return x.to(torch.bfloat16), w


def probe_rows(x: torch.Tensor) -> torch.Tensor:
    """Rows of x with exactly one nonzero entry (reference.py:79-81)."""
    return ((x != 0).sum(-1) == 1).nonzero().flatten()


def algorithmic_bytes(m: int, n: int, k: int, w_bytes: int = 2, out_bytes: int = 2) -> int:
    """N*K weights + M*K activations + M*N outputs (reference.py:102-107)."""
    return n * k * w_bytes + m * k * 2 + m * n * out_bytes
