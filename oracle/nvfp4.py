"""NVFP4 codec restated (oracle; test infrastructure only).

Format (reference muse_moe_w4a16/nvfp4.py:1-9): value = e2m1 * block_scale(e4m3) * global_scale(fp32),
16 values per block scale, two 4-bit codes per byte with element 2i in the low nibble.
"""
from __future__ import annotations

import torch

BLOCK = 16
E2M1_MAX = 6.0
E4M3_MAX = 448.0
# 3-bit magnitude code -> value (sign is bit 3).  reference nvfp4.py:24
E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
# decision thresholds between neighbouring magnitudes.  reference nvfp4.py:26
_THRESHOLDS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)


def codes_of(packed: torch.Tensor) -> torch.Tensor:
    """uint8 [..., K/2] -> uint8 [..., K] 4-bit codes, low nibble first (nvfp4.py:40-45)."""
    b = packed.view(torch.uint8)
    return torch.stack((b & 0xF, b >> 4), dim=-1).reshape(*b.shape[:-1], b.shape[-1] * 2)


def e2m1_values(packed: torch.Tensor) -> torch.Tensor:
    """uint8 [..., K/2] -> float32 [..., K] unscaled E2M1 values (nvfp4.py:40-47)."""
    c = codes_of(packed).long()
    table = torch.tensor(E2M1_VALUES + tuple(-v for v in E2M1_VALUES), dtype=torch.float32)
    # code 8 (negative zero) decodes to -0.0 in the table, equal to +0.0 in every comparison
    return table[c]


def pack_codes(values: torch.Tensor) -> torch.Tensor:
    """float [..., K] (already divided by its scale) -> uint8 [..., K/2] (nvfp4.py:50-57).

    Round to the nearest grid magnitude; an exact midpoint goes to the smaller magnitude
    (bucketize with right=False), magnitudes above 6 clamp to 6, and zero never carries a sign.
    """
    v = values.float()
    thr = torch.tensor(_THRESHOLDS, dtype=torch.float32)
    mag = torch.bucketize(v.abs().clamp(max=E2M1_MAX), thr).to(torch.uint8)
    neg = ((v < 0) & (mag > 0)).to(torch.uint8)
    code = (mag | (neg << 3)).reshape(*v.shape[:-1], v.shape[-1] // 2, 2)
    return code[..., 0] | (code[..., 1] << 4)


def quantize(x: torch.Tensor):
    """Quantise the last dim of x: (packed uint8 [..., K/2], sf e4m3 [..., K/16], gs fp32 []).

    gs = amax / (6 * 448) (1 if amax == 0); sf = min(block_amax / 6 / gs, 448) cast to E4M3;
    codes from x / (sf * gs)  (nvfp4.py:60-87, dynamic global scale).
    """
    k = x.shape[-1]
    assert k % BLOCK == 0
    xf = x.float()
    amax = xf.abs().amax()
    gs = torch.where(amax > 0, amax / (E2M1_MAX * E4M3_MAX), torch.ones_like(amax))
    blk = xf.reshape(*xf.shape[:-1], k // BLOCK, BLOCK)
    sf = (blk.abs().amax(-1) / E2M1_MAX / gs).clamp(max=E4M3_MAX).to(torch.float8_e4m3fn)
    scale = (sf.float() * gs).unsqueeze(-1)
    q = torch.where(scale > 0, blk / scale, torch.zeros_like(blk))
    return pack_codes(q.reshape(xf.shape)), sf, gs


def dequantize(packed: torch.Tensor, sf: torch.Tensor, gs) -> torch.Tensor:
    """float32 [..., K] = e2m1 * (sf * gs) per 16-block (nvfp4.py:90-97)."""
    v = e2m1_values(packed)
    k = v.shape[-1]
    gs = torch.as_tensor(gs, dtype=torch.float32)
    scale = (sf.float() * gs).unsqueeze(-1)
    return (v.reshape(*v.shape[:-1], k // BLOCK, BLOCK) * scale).reshape(v.shape)


def dequantize_tile_bf16(packed: torch.Tensor, sf: torch.Tensor) -> torch.Tensor:
    """e2m1 * sf as BF16, without the global scale: the tile a kernel feeds to its BF16 MMAs.

    Every E2M1 x E4M3 product has at most 6 significant bits and lies in [2^-10, 2688], so
    the BF16 result is exact; this is what "bit-exact dequantisation" is tested against.
    """
    v = e2m1_values(packed)
    k = v.shape[-1]
    t = v.reshape(*v.shape[:-1], k // BLOCK, BLOCK) * sf.float().unsqueeze(-1)
    out = t.reshape(v.shape).to(torch.bfloat16)
    assert torch.equal(out.float(), t.reshape(v.shape)), "E2M1 x E4M3 must be exact in BF16"
    return out
