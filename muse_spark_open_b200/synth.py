"""Seeded synthetic weights and step inputs at the benchmark's shapes, generated on the GPU.

The benchmark's inputs are random by definition (no dataset, no checkpoint): dense weights
N(0, 1/sqrt(K)) BF16, experts N(0, 0.02) quantised to NVFP4 (E2M1 codes, one E4M3 scale per 16 values,
one FP32 scale per expert), KV cache N(0, 1) quantised to E4M3 with one scale amax/448 per tensor,
scattered pages, residual stream N(0, 1).  Field names follow the reference's generators
(muse_decode_layer/reference.py:89-128,244-326; muse_moe_w4a16/nvfp4.py:66-87).
This module only makes inputs; nothing here is on the timed path.
"""
from __future__ import annotations

import math

import torch

FP8 = torch.float8_e4m3fn
QK_SCALE_FACTOR = 5.4730064863875


def quantize_nvfp4(x: torch.Tensor):
    """x [..., K] -> (codes uint8 [..., K/2], block scales e4m3 [..., K/16], tensor scale fp32 [])."""
    xf = x.float()
    k = xf.shape[-1]
    amax = xf.abs().amax()
    gs = torch.where(amax > 0, amax / (6.0 * 448.0), torch.ones_like(amax))
    blk = xf.reshape(*xf.shape[:-1], k // 16, 16)
    sf = (blk.abs().amax(-1) / 6.0 / gs).clamp(max=448.0).to(FP8)
    scale = (sf.float() * gs).unsqueeze(-1)
    q = torch.where(scale > 0, blk / scale, torch.zeros_like(blk)).reshape(xf.shape)
    edges = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], device=x.device)
    mag = torch.bucketize(q.abs().clamp(max=6.0), edges).to(torch.uint8)
    code = mag | (((q < 0) & (mag > 0)).to(torch.uint8) << 3)
    code = code.reshape(*code.shape[:-1], k // 2, 2)
    return code[..., 0] | (code[..., 1] << 4), sf, gs


def make_layer_weights(seed: int, device, hidden: int = 4096, hq: int = 32, hkv: int = 4, d: int = 128,
                       n_experts: int = 128, inner: int = 768, bias_std: float = 0.0,
                       expert_range: tuple[int, int] | None = None) -> dict:
    """All layer weights; with expert_range = (first, count) only those experts are materialised
    (every rank draws the same stream of experts, so shards are consistent across ranks)."""
    gen = torch.Generator(device=device).manual_seed(seed)

    def dense(n, k, dtype=torch.bfloat16):
        return (torch.randn((n, k), generator=gen, device=device) / math.sqrt(k)).to(dtype)

    def vec(n, std=0.1):
        return (std * torch.randn((n,), generator=gen, device=device)).to(torch.bfloat16)

    w = {
        "input_norm": vec(hidden), "qkv_gate": dense((2 * hq + 2 * hkv) * d, hidden), "o": dense(hidden, hq * d),
        "pre_expert_norm": vec(hidden), "router": dense(n_experts, hidden, torch.float32),
        "router_bias": bias_std * torch.randn((n_experts,), generator=gen, device=device),
        "post_expert_norm": vec(hidden),
    }
    first, count = expert_range or (0, n_experts)
    parts = {k: [] for k in ("w13", "w13_sf", "w13_gs", "w2", "w2_sf", "w2_gs")}
    for e in range(n_experts):
        eg = torch.Generator(device=device).manual_seed(seed * 1000003 + e + 1)
        if not first <= e < first + count:
            continue
        a = 0.02 * torch.randn((2 * inner, hidden), generator=eg, device=device)
        b = 0.02 * torch.randn((hidden, inner), generator=eg, device=device)
        for name, t in (("w13", a), ("w2", b)):
            c, s, g = quantize_nvfp4(t)
            parts[name].append(c), parts[name + "_sf"].append(s), parts[name + "_gs"].append(g)
    w.update({k: torch.stack(v) for k, v in parts.items()})
    return w


def make_layer_input(seed: int, device, seq_lens, q_len: int = 1, hidden: int = 4096, hq: int = 32, hkv: int = 4,
                     d: int = 128, page: int = 64, window: int = 0, rope_theta: float = 0.0, max_len: int | None = None):
    """One decode step's inputs for len(seq_lens) requests: stream, paged FP8 cache, metadata, config."""
    gen = torch.Generator(device=device).manual_seed(seed)
    seq = torch.as_tensor(seq_lens, dtype=torch.int64)
    batch = len(seq)
    longest = int(seq.max()) if max_len is None else max_len
    pages_per = (seq + q_len + page - 1) // page
    max_pages = (longest + q_len + page - 1) // page
    total = batch * max_pages
    perm = torch.randperm(total, generator=gen, device=device).to(torch.int32).cpu()
    table = torch.full((batch, max_pages), -1, dtype=torch.int32)
    off = torch.cumsum(pages_per, 0) - pages_per
    for b in range(batch):
        n, o = int(pages_per[b]), int(off[b])
        table[b, :n] = perm[o:o + n]

    def cache(s):
        out = torch.empty((total, page, hkv, d), dtype=FP8, device=device)
        chunk = max(1, (1 << 28) // (page * hkv * d))
        amax = torch.zeros((), device=device)
        for pass_ in range(2):
            g = torch.Generator(device=device).manual_seed(seed * 7919 + s)
            for at in range(0, total, chunk):
                n = min(chunk, total - at)
                x = torch.randn((n, page, hkv, d), generator=g, device=device)
                if pass_ == 0:
                    amax = torch.maximum(amax, x.abs().amax())
                else:
                    out[at:at + n] = (x / scale).clamp(-448, 448).to(FP8)
            scale = amax / 448.0
        return out, scale.float()

    k_cache, k_scale = cache(1)
    v_cache, v_scale = cache(2)
    pos = seq[:, None] + torch.arange(q_len)
    loc = (torch.gather(table.long(), 1, pos // page) * page + pos % page).reshape(-1)
    t = batch * q_len
    return {
        "stream": torch.randn((t, hidden), generator=gen, device=device),
        "positions": pos.reshape(-1).to(device), "cache_loc": loc.to(device),
        "seq_lens": seq.to(torch.int32).to(device), "page_table": table.to(device),
        "k_cache": k_cache, "v_cache": v_cache, "k_scale": k_scale, "v_scale": v_scale,
        "config": {"batch": batch, "q_len": q_len, "tokens": t, "hidden": hidden, "num_q_heads": hq, "num_kv_heads": hkv,
                   "head_dim": d, "page_size": page, "window": window, "rope_theta": rope_theta,
                   "qk_scale_factor": QK_SCALE_FACTOR, "sm_scale": d ** -0.5},
    }


def layer_bytes(weights: dict, data: dict, touched_experts: int) -> int:
    """Algorithmic HBM bytes of one step: dense weights + router + visible K/V + touched experts
    + 12 bytes per token-channel of activations."""
    cfg = data["config"]
    dense = sum(weights[k].numel() * weights[k].element_size() for k in ("qkv_gate", "o", "router"))
    w = cfg["window"]
    keys = sum(min(s, w - 1) if w else s for s in data["seq_lens"].tolist())
    kv = keys * cfg["num_kv_heads"] * cfg["head_dim"] * 2
    per = sum(weights[k][0].numel() * weights[k][0].element_size() for k in ("w13", "w13_sf", "w2", "w2_sf"))
    return dense + kv + touched_experts * per + 12 * cfg["tokens"] * cfg["hidden"]
