"""NVFP4 routed experts restated (oracle; test infrastructure only).

Follows muse_moe_w4a16/reference.py:88-107 with shapes taken from the weights, plus the
benchmark's routing rule (softmax -> top-k -> renormalise, the renormalisation of reference.py:82).
"""
from __future__ import annotations

import torch

from . import nvfp4

POST_NORM_EPS = 1e-8  # reference.py:24


def route_softmax(logits: torch.Tensor, top_k: int = 8):
    """(ids int32 [T,k], weights fp32 [T,k]): p = softmax(logits); top-k of p; w = p[ids] / sum."""
    p = torch.softmax(logits.float(), dim=-1)
    top = p.topk(top_k, dim=-1)
    return top.indices.to(torch.int32), (top.values / top.values.sum(-1, keepdim=True)).float()


def post_expert_norm(y: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """Scale by (1 + w), then RMSNorm with eps 1e-8 (reference.py:88-90)."""
    y = y.float() * (1.0 + w.float())
    return y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + POST_NORM_EPS)


def expert_forward(x: torch.Tensor, weights, e: int, round_inter=False) -> torch.Tensor:
    """y = (silu(h[:, :I]) * h[:, I:]) @ W2[e]^T with h = x @ W13[e]^T, FP32 (reference.py:101-103).
    round_inter: False, True (= bfloat16) or a 16-bit dtype the activations are rounded to."""
    w13 = nvfp4.dequantize(weights["w13"][e], weights["w13_sf"][e], weights["w13_gs"][e])
    w2 = nvfp4.dequantize(weights["w2"][e], weights["w2_sf"][e], weights["w2_gs"][e])
    inner = w13.shape[0] // 2
    h = x.float() @ w13.T
    inter = torch.nn.functional.silu(h[:, :inner]) * h[:, inner:]
    if round_inter:  # the rounding point kernels add and the rules allow (reference submission.py:478-485)
        inter = inter.to(torch.bfloat16 if round_inter is True else round_inter).float()
    return inter @ w2.T


def ref_kernel(data, weights, fp32_out: bool = False, round_inter=False) -> torch.Tensor:
    """out[t] = sum over local (t, slot) pairs of topk_weight * post_norm(expert(x[t]));  bf16 [T,H].

    Tokens with no local pair stay zero (reference.py:93-107).
    """
    cfg = data["config"]
    x = data["hidden_states"].float()
    out = torch.zeros(x.shape, dtype=torch.float32)
    ids = data["topk_ids"].long()
    lo, hi = cfg["local_start"], cfg["local_start"] + cfg["local_count"]
    for e in torch.unique(ids).tolist():
        if not lo <= e < hi:
            continue
        tok, slot = (ids == e).nonzero(as_tuple=True)
        y = expert_forward(x[tok], weights, e - cfg.get("weights_start", 0), round_inter=round_inter)
        out.index_add_(0, tok, post_expert_norm(y, weights["post_norm_w"]) * data["topk_weights"][tok, slot, None])
    return out if fp32_out else out.to(torch.bfloat16)


def make_weights(seed: int, n_experts: int = 128, hidden: int = 4096, inner: int = 768, std: float = 0.02):
    """The benchmark's experts: gate_up [2I,H] and down [H,I] ~ N(0, std) quantised per expert
    with nvfp4.quantize; post_norm_w ~ 0.1 N bf16.  Field names and layouts as
    muse_moe_w4a16/reference.py:33-50."""
    gen = torch.Generator().manual_seed(seed)
    w13, w13_sf, w13_gs, w2, w2_sf, w2_gs = [], [], [], [], [], []
    for _ in range(n_experts):
        a = std * torch.randn((2 * inner, hidden), generator=gen)
        b = std * torch.randn((hidden, inner), generator=gen)
        p, s, g = nvfp4.quantize(a)
        w13.append(p), w13_sf.append(s), w13_gs.append(g)
        p, s, g = nvfp4.quantize(b)
        w2.append(p), w2_sf.append(s), w2_gs.append(g)
    return {
        "w13": torch.stack(w13), "w13_sf": torch.stack(w13_sf), "w13_gs": torch.stack(w13_gs),
        "w2": torch.stack(w2), "w2_sf": torch.stack(w2_sf), "w2_gs": torch.stack(w2_gs),
        "post_norm_w": (0.1 * torch.randn((hidden,), generator=gen)).to(torch.bfloat16),
    }


def make_input(tokens: int, seed: int, n_experts: int = 128, hidden: int = 4096, top_k: int = 8,
               local_start: int = 0, local_count: int | None = None, bias_std: float = 0.0):
    """x ~ N(0,1) bf16 [T,H]; router logits ~ N(0,1) (+ a per-expert bias ~ N(0, bias_std));
    ids / weights by route_softmax.  Fields as muse_moe_w4a16/reference.py:53-85."""
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn((tokens, hidden), generator=gen).to(torch.bfloat16)
    logits = torch.randn((tokens, n_experts), generator=gen)
    if bias_std:
        logits = logits + bias_std * torch.randn((n_experts,), generator=gen)
    ids, w = route_softmax(logits, top_k)
    return {
        "hidden_states": x, "topk_ids": ids, "topk_weights": w, "router_logits": logits,
        "config": {"bs": tokens, "d_hidden": hidden, "n_experts": n_experts, "top_k": top_k,
                   "local_start": local_start,
                   "local_count": n_experts if local_count is None else local_count, "sharding": "full"},
    }


def touched_experts(data) -> int:
    cfg = data["config"]
    ids = data["topk_ids"].long().flatten()
    local = ids[(ids >= cfg["local_start"]) & (ids < cfg["local_start"] + cfg["local_count"])]
    return int(torch.unique(local).numel())


def algorithmic_bytes(data, weights) -> int:
    """touched experts x (codes + block scales) + x read + out written (reference.py:125-136)."""
    per = sum(weights[k][0].numel() * weights[k][0].element_size() for k in ("w13", "w13_sf", "w2", "w2_sf"))
    t, h = data["hidden_states"].shape
    return touched_experts(data) * per + 2 * t * h * 2
