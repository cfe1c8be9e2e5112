"""Skinny BF16 projections: the reference's per-op entry points over the C ABI.

Same call shape as muse_bf16_proj/submission.py: `prepare(weights) -> state` once (untimed),
`kernel_fn(data, state) -> tensor` per step, with `data = {"x": bf16 [m, k], "config": {"m", "n",
"k", "layer"}}` (submission.py:23-40,390-436).  Layer names are whatever keys `weights` has; FP32
weights (the router) are split into BF16 hi + lo halves at prepare time and the two halves are
accumulated in one FP32 pass (the legal fast path the reference's rules name, reference.py:28-29).
The layer hooks `data["out"]` (write into a caller-provided, possibly wider buffer) and `data["ssq"]`
are honoured like submission.py:430-435.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import abi

MAX_M = 256


def prepare(weights: dict) -> dict:
    state = {"w": {}, "fp32": set()}
    for name, w in weights.items():
        if w.dim() != 2:
            continue
        if not w.is_cuda:
            raise abi.MskError("prepare() needs CUDA weights")
        if w.dtype == torch.float32:
            hi = w.to(torch.bfloat16)
            lo = (w - hi.float()).to(torch.bfloat16)
            state["w"][name] = torch.cat([hi, lo], dim=1).contiguous()  # [N, 2K]: x @ hi^T + x @ lo^T in one K loop
            state["fp32"].add(name)
        else:
            state["w"][name] = w.contiguous()
    abi.lib()
    return state


_scratch: dict = {}


def scratch_for(m: int, n: int, k: int, splits: int, device, tag: str = "", token_splits: int = 0) -> torch.Tensor:
    """The split-K workspace of a launch of that shape (tickets + FP32 partial tiles), allocated and zeroed once
    per (shape, tag, device) and reused: launches sharing one must be ordered on the stream (they are,
    unless they overlap by programmatic launch - give those different tags)."""
    key = (m, n, k, splits, token_splits, tag, torch.device(device).index or 0)
    if key not in _scratch:
        nbytes = C.c_size_t()
        abi.check(abi.lib().msk_proj_scratch_bytes(m, n, k, splits, token_splits, C.byref(nbytes)), "msk_proj_scratch_bytes")
        _scratch[key] = torch.zeros(nbytes.value, dtype=torch.uint8, device=device)
    return _scratch[key]


def skinny(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None, fp32_out: bool = False,
           splits: int = 0, token_splits: int = 0, pdl: bool = False, in_ssq=None, in_dim: int = 0, in_eps: float = 0.0, resid=None,
           next_norm_w=None, out_normed=None, out_ssq=None) -> torch.Tensor:
    """One launch of msk_proj_skinny.  x bf16 [M, K] contiguous, w bf16 [N, K] contiguous."""
    m, k = x.shape
    n = w.shape[0]
    if out is None and out_normed is None:
        out = torch.empty((m, n), dtype=torch.float32 if fp32_out else torch.bfloat16, device=x.device)
    p = abi.ProjParams()
    p.x, p.w, p.M, p.N, p.K, p.splits, p.token_splits = abi.ptr(x), abi.ptr(w), m, n, k, splits, token_splits
    if out is not None:
        p.out, p.out_fp32, p.ldo = abi.ptr(out), int(out.dtype == torch.float32), out.stride(0)
    if in_ssq is not None:
        p.in_ssq, p.in_ssq_parts, p.in_inv_dim, p.in_eps = abi.ptr(in_ssq), in_ssq.shape[0], 1.0 / in_dim, in_eps
    if resid is not None:
        p.resid, p.ldr = abi.ptr(resid), resid.stride(0)
    if out_normed is not None:
        p.next_norm_w, p.out_normed, p.ldn = abi.ptr(next_norm_w), abi.ptr(out_normed), out_normed.stride(0)
    if out_ssq is not None:
        p.out_ssq = abi.ptr(out_ssq)
    p.pdl = int(pdl)
    ws = scratch_for(m, n, k, splits, x.device, token_splits=token_splits)
    p.scratch, p.scratch_bytes = abi.ptr(ws), ws.numel()
    st = abi.status_for(x.device)
    abi.check(abi.lib().msk_proj_skinny(C.byref(p), st.p, abi.stream_ptr()), "msk_proj_skinny")
    return out


def kernel_fn(data: dict, state: dict) -> torch.Tensor:
    x, cfg = data["x"], data["config"]
    m, n, layer = cfg["m"], cfg["n"], cfg["layer"]
    if m > MAX_M:
        # the kernel is built for decode / verify steps; larger token counts (the reference's m = 512 and 1000 cases,
        # muse_bf16_proj/bench.py:14-16) run as consecutive blocks of MAX_M rows, each streaming the weights again
        if data.get("ssq") is not None:
            raise abi.MskError(f"the sum-of-squares hook is built for up to {MAX_M} tokens, got {m}")
        fp32 = layer in state["fp32"]
        out = data.get("out")
        if out is None:
            out = torch.empty((m, n), dtype=torch.float32 if fp32 else torch.bfloat16, device=x.device)
        for r0 in range(0, m, MAX_M):
            r1 = min(m, r0 + MAX_M)
            sub = {"x": x[r0:r1], "config": dict(cfg, m=r1 - r0)}
            if fp32:
                out[r0:r1].copy_(kernel_fn(sub, state))
            else:
                sub["out"] = out[r0:r1]
                kernel_fn(sub, state)
        return out
    w = state["w"][layer][:n]
    if layer in state["fp32"]:
        # x against [hi | lo]: the doubled activation row lives in a persistent buffer (two strided copies, no
        # allocation and no concatenation kernel in the timed call)
        key = ("xx", m, x.shape[1], x.device)
        if key not in state:
            state[key] = torch.empty((m, 2 * x.shape[1]), dtype=x.dtype, device=x.device)
        xx = state[key]
        k1 = x.shape[1]
        xx[:, :k1].copy_(x)
        xx[:, k1:].copy_(x)
        return skinny(xx, w, fp32_out=True)
    return skinny(x, w, out=data.get("out"), out_ssq=data.get("ssq"))
