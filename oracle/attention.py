"""Gated attention decode / verify over a paged FP8 cache, restated (oracle; test infrastructure only).

Follows muse_attention_decode/reference.py:294-337 (`ref_kernel`) with every shape read from
`data["config"]` instead of module constants, so it runs at head_dim 64 (the reference's) and
128 (the benchmark's).
"""
from __future__ import annotations

import math

import torch

FP8 = torch.float8_e4m3fn
RMS_EPS = 1e-5
QK_SCALE_FACTOR = 5.4730064863875  # reference.py:21


def rms(x: torch.Tensor, eps: float = RMS_EPS) -> torch.Tensor:
    """Weightless RMSNorm over the last dim in FP32 (reference.py:266-268)."""
    x = x.float()
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def rope(x: torch.Tensor, pos: torch.Tensor, theta: float) -> torch.Tensor:
    """Interleaved (GPT-J) rotary embedding: pair (2i, 2i+1) turns by pos * theta^(-2i/d).

    x [..., heads, d]; pos broadcasts over all but the last two dims (reference.py:271-278).
    """
    d = x.shape[-1]
    inv_freq = 1.0 / (theta ** (torch.arange(0, d, 2).float() / d))
    ang = pos.float()[..., None] * inv_freq
    c, s = ang.cos().unsqueeze(-2), ang.sin().unsqueeze(-2)
    a, b = x[..., 0::2], x[..., 1::2]
    return torch.stack((a * c - b * s, a * s + b * c), dim=-1).flatten(-2)


def quant_e4m3(x: torch.Tensor, scale) -> torch.Tensor:
    """x / scale rounded to E4M3 (reference.py:114-115), saturating at +-448 like cvt.rn.satfinite."""
    return (x.float() / scale).clamp(-448.0, 448.0).to(FP8)


def dequant_e4m3(c: torch.Tensor, scale) -> torch.Tensor:
    return c.float() * scale  # reference.py:118-119


def split_qkv(data):
    """q [B,L,Hq,d], k,v [B,L,Hkv,d], gate [B,L,Hq*d] from the fused row q|k|v|gate (reference.py:256-263)."""
    cfg = data["config"]
    hq, hkv, d = cfg["num_q_heads"], cfg["num_kv_heads"], cfg["head_dim"]
    b, l = cfg["batch"], cfg["q_len"]
    q, k, v, g = data["qkv"].split([hq * d, hkv * d, hkv * d, hq * d], dim=-1)
    return q.reshape(b, l, hq, d), k.reshape(b, l, hkv, d), v.reshape(b, l, hkv, d), g


def cache_rows(data, positions: torch.Tensor) -> torch.Tensor:
    """Flat cache rows of [B, n] positions: page_table[b, p // page] * page + p % page (reference.py:281-285)."""
    size = data["config"]["page_size"]
    page = torch.gather(data["page_table"].long(), 1, positions // size)
    return page * size + positions % size


def new_slots(data) -> torch.Tensor:
    """[B, L] flat rows the step writes (reference.py:288-291)."""
    l = data["config"]["q_len"]
    pos = data["seq_lens"].long()[:, None] + torch.arange(l)
    return cache_rows(data, pos)


def ref_kernel(data, new_kv=None, scale_after_rope: bool = False):
    """(out fp32 [B,L,Hq*d], k_new e4m3 [B,L,Hkv,d], v_new e4m3 [B,L,Hkv,d]).  reference.py:294-337.

    With new_kv the block attends those FP8 entries as its own (reference.py:316-317).
    scale_after_rope: multiply the queries by qk_scale_factor after RoPE instead of before it, the order of the
    layer's reference (muse_decode_layer/reference.py:364-372); the same value up to FP32 rounding.
    """
    cfg = data["config"]
    b_n, l_n = cfg["batch"], cfg["q_len"]
    hq, hkv, d = cfg["num_q_heads"], cfg["num_kv_heads"], cfg["head_dim"]
    grp = hq // hkv
    q_in, k_in, v_in, gate = split_qkv(data)
    pos = data["seq_lens"].long()[:, None] + torch.arange(l_n)
    q = rms(q_in) if scale_after_rope else rms(q_in) * cfg["qk_scale_factor"]
    k = rms(k_in)
    if cfg["rope_theta"]:
        q, k = rope(q, pos, cfg["rope_theta"]), rope(k, pos, cfg["rope_theta"])
    if scale_after_rope:
        q = q * cfg["qk_scale_factor"]
    q = q.to(torch.bfloat16).float()  # queries rounded to BF16 (reference.py:308-310)
    k_new = quant_e4m3(k, data["k_scale"])
    v_new = quant_e4m3(v_in, data["v_scale"])
    if new_kv is not None:
        k_new, v_new = new_kv
    kc = data["k_cache"].view(-1, hkv, d)
    vc = data["v_cache"].view(-1, hkv, d)
    size = cfg["page_size"]
    out = torch.empty((b_n, l_n, hq, d), dtype=torch.float32)
    for b in range(b_n):
        seq = int(data["seq_lens"][b])
        past = torch.arange(seq)
        rows = data["page_table"][b].long()[past // size] * size + past % size
        keys = torch.cat([dequant_e4m3(kc[rows], data["k_scale"]), dequant_e4m3(k_new[b], data["k_scale"])])
        vals = torch.cat([dequant_e4m3(vc[rows], data["v_scale"]), dequant_e4m3(v_new[b], data["v_scale"])])
        for j in range(l_n):
            p = seq + j
            lo = max(0, p - cfg["window"] + 1) if cfg["window"] else 0
            kb, vb = keys[lo:p + 1], vals[lo:p + 1]
            s = torch.einsum("kgd,tkd->kgt", q[b, j].view(hkv, grp, d), kb) * cfg["sm_scale"]
            out[b, j] = torch.einsum("kgt,tkd->kgd", s.softmax(-1), vb).reshape(hq, d)
    out = rms(out) * torch.sigmoid(gate.float()).view(b_n, l_n, hq, d)
    return out.reshape(b_n, l_n, hq * d), k_new, v_new


def make_input(batch: int, seq_lens, seed: int, q_len: int = 1, hq: int = 32, hkv: int = 4, d: int = 128,
               page: int = 64, window: int = 1024, rope_theta: float = 1e6, kv_scale="amax",
               max_len: int | None = None, cache_dist: str = "normal"):
    """Benchmark-shaped attention inputs drawn on a CPU generator.

    Same fields and construction order as the reference's generate_input
    (muse_attention_decode/reference.py:168-253): lengths, scattered pages (randperm), cache
    K,V ~ N(0,1) quantised with one per-tensor scale, q ~ 2N, k_new ~ 2N, v_new ~ N, gate ~ N.
    kv_scale="amax" uses amax/448 of the drawn values (the benchmark's rule); a float is used as given.
    seq_lens: list/tensor of B lengths, or (lo, hi) for a uniform draw.
    """
    gen = torch.Generator().manual_seed(seed)
    if isinstance(seq_lens, tuple):
        lo, hi = seq_lens
        seq = torch.randint(lo, hi + 1, (batch,), generator=gen)
        longest = hi
    else:
        seq = torch.as_tensor(seq_lens, dtype=torch.int64)
        longest = int(seq.max())
    if max_len is not None:
        longest = max_len
    pages_per = (seq + q_len + page - 1) // page
    max_pages = (longest + q_len + page - 1) // page
    total = batch * max_pages
    perm = torch.randperm(total, generator=gen).to(torch.int32)
    table = torch.full((batch, max_pages), -1, dtype=torch.int32)
    off = torch.cumsum(pages_per, 0) - pages_per
    for b in range(batch):
        n, o = int(pages_per[b]), int(off[b])
        table[b, :n] = perm[o:o + n]
    shape = (total, page, hkv, d)
    kf = torch.randn(shape, generator=gen)
    vf = torch.randn(shape, generator=gen)
    if cache_dist == "outliers":  # a few channels 10x, like the reference's dist="outliers"
        idx = torch.randperm(d, generator=gen)[: max(1, d // 64)]
        kf[..., idx] *= 10
        vf[..., idx] *= 10
    if kv_scale == "amax":
        k_scale = float(kf.abs().amax()) / 448.0
        v_scale = float(vf.abs().amax()) / 448.0
    else:
        k_scale = v_scale = float(kv_scale)
    k_cache, v_cache = quant_e4m3(kf, k_scale), quant_e4m3(vf, v_scale)
    q = (2 * torch.randn((batch, q_len, hq * d), generator=gen)).to(torch.bfloat16)
    kn = (2 * torch.randn((batch, q_len, hkv * d), generator=gen)).to(torch.bfloat16)
    vn = torch.randn((batch, q_len, hkv * d), generator=gen).to(torch.bfloat16)
    gate = torch.randn((batch, q_len, hq * d), generator=gen).to(torch.bfloat16)
    qkv = torch.cat([q, kn, vn, gate], dim=-1)
    pos = seq[:, None] + torch.arange(q_len)
    data = {
        "qkv": qkv,
        "positions": pos.reshape(-1),
        "cache_seqlens": (seq + q_len).to(torch.int32),
        "cu_seqlens_q": torch.arange(0, batch * q_len + 1, q_len, dtype=torch.int32),
        "scheduler_metadata": None,
        "k_cache": k_cache,
        "v_cache": v_cache,
        "k_scale": torch.tensor(k_scale, dtype=torch.float32),
        "v_scale": torch.tensor(v_scale, dtype=torch.float32),
        "page_table": table,
        "seq_lens": seq.to(torch.int32),
        "config": {
            "batch": batch, "q_len": q_len, "num_q_heads": hq, "num_kv_heads": hkv, "head_dim": d,
            "page_size": page, "window": window, "rope_theta": rope_theta,
            "qk_scale_factor": QK_SCALE_FACTOR, "sm_scale": d ** -0.5, "kv_scale": k_scale,
        },
    }
    data["cache_loc"] = cache_rows(data, pos).reshape(-1)
    return data


def algorithmic_bytes(data) -> int:
    """Bytes the step must move: visible cached K+V rows, the fused qkv rows read, the output written."""
    cfg = data["config"]
    hq, hkv, d, l = cfg["num_q_heads"], cfg["num_kv_heads"], cfg["head_dim"], cfg["q_len"]
    w = cfg["window"]
    keys = 0
    for s in data["seq_lens"].tolist():
        keys += min(s, (w - 1) if w else s)
    b = cfg["batch"]
    return keys * hkv * d * 2 + b * l * ((2 * hq + 2 * hkv) * d * 2 + hq * d * 2) + b * l * hkv * d * 2


def to_device(data, device):
    return {k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in data.items()}


__all__ = ["ref_kernel", "make_input", "rms", "rope", "quant_e4m3", "dequant_e4m3", "new_slots", "cache_rows",
           "split_qkv", "algorithmic_bytes", "to_device", "math"]
