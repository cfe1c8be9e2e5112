"""Gated attention decode / verify: the reference's per-op entry point over the C ABI.

`kernel_fn(data) -> bf16 [B, L, Hq*d]` with the `Inputs` / `Config` fields of
muse_attention_decode/submission.py:37-65; the new tokens' K/V are written into
`data["k_cache"]` / `data["v_cache"]` in place at `data["cache_loc"]`, like the reference.
Nothing derived from `data` is cached between calls; only the RoPE frequency table (a function of
theta and head_dim) is kept per device.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import abi

_inv_freq: dict = {}


def inv_freq(theta: float, d: int, device) -> torch.Tensor | None:
    """theta^(-2i/d), computed in FP32 exactly as the reference does (reference.py:274)."""
    if not theta:
        return None
    key = (float(theta), d, torch.device(device).index or 0)
    if key not in _inv_freq:
        _inv_freq[key] = (1.0 / (theta ** (torch.arange(0, d, 2).float() / d))).to(device)
    return _inv_freq[key]


def launch(qkv2d: torch.Tensor, out2d: torch.Tensor, data: dict, cfg: dict, chunks: int = 0, stages: int = 0, issuers: int = 0,
           pdl: bool = False, row_groups: int = 0) -> None:
    """qkv2d bf16 [B*L, >= (2Hq+2Hkv)*d] (row stride free), out2d bf16 [B*L, Hq*d]."""
    p = abi.AttnParams()
    p.qkv, p.ld_qkv, p.out, p.ld_out = abi.ptr(qkv2d), qkv2d.stride(0), abi.ptr(out2d), out2d.stride(0)
    kc, vc = data["k_cache"], data["v_cache"]
    p.k_cache, p.v_cache = abi.ptr(kc), abi.ptr(vc)
    p.k_scale, p.v_scale = abi.ptr(data["k_scale"]), abi.ptr(data["v_scale"])
    p.seq_lens, p.page_table = abi.ptr(data["seq_lens"]), abi.ptr(data["page_table"])
    p.max_pages = data["page_table"].shape[1]
    p.cache_loc = abi.ptr(data["cache_loc"])
    f = inv_freq(cfg["rope_theta"], cfg["head_dim"], qkv2d.device)
    p.inv_freq = abi.ptr(f) if f is not None else None
    p.B, p.L, p.Hq, p.Hkv, p.d = cfg["batch"], cfg["q_len"], cfg["num_q_heads"], cfg["num_kv_heads"], cfg["head_dim"]
    p.page_size, p.num_pages, p.window = cfg["page_size"], kc.shape[0], cfg["window"]
    p.qk_scale_factor, p.sm_scale = cfg["qk_scale_factor"], cfg["sm_scale"]
    p.chunks, p.stages, p.issuers, p.pdl, p.row_groups = chunks, stages, issuers, int(pdl), row_groups
    st = abi.status_for(qkv2d.device)
    abi.check(abi.lib().msk_attn_decode(C.byref(p), st.p, abi.stream_ptr()), "msk_attn_decode")


def kernel_fn(data: dict, chunks: int = 0, stages: int = 0) -> torch.Tensor:
    cfg = data["config"]
    b, l, hq, d = cfg["batch"], cfg["q_len"], cfg["num_q_heads"], cfg["head_dim"]
    qkv = data["qkv"]
    if qkv.dtype != torch.bfloat16 or data["k_cache"].dtype != torch.float8_e4m3fn:
        raise abi.MskError("qkv must be bfloat16 and the cache float8_e4m3fn")
    if data["seq_lens"].dtype != torch.int32 or data["page_table"].dtype != torch.int32 or \
            data["cache_loc"].dtype != torch.int64:
        raise abi.MskError("seq_lens / page_table must be int32 and cache_loc int64")
    out = torch.empty((b, l, hq * d), dtype=torch.bfloat16, device=qkv.device)
    launch(qkv.view(b * l, -1), out.view(b * l, hq * d), data, cfg, chunks, stages)
    return out
