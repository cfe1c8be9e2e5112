"""One decoder layer's decode step in the benchmark's form, restated (oracle; test infrastructure only).

The op list is the subset of the reference's layer (muse_decode_layer/reference.py:447-477,
TASK.md:15-25) that the benchmark names: input RMSNorm -> fused QKV+gate projection -> paged FP8
gated attention (oracle.attention) -> o_proj -> residual add -> pre-expert RMSNorm -> FP32 router,
softmax top-8 renormalised -> NVFP4 experts with post-expert norm and weighted sum (oracle.moe)
-> residual add.  All norm weights are zero-centred (scale = 1 + w), eps 1e-5
(muse_decode_layer/reference.py:40,452-455); there is no pooler/unpooler because the layer width
equals the MoE width.  Collectives are absent: one rank holds every expert here; the
expert-parallel layer is checked against this same function.

Rounding points: the attention input, the fused projection output, the attention output and the
MoE input are BF16 (as the reference's submission_starter.py:89-216 keeps them); residual stream,
router logits and expert outputs stay FP32.
"""
from __future__ import annotations

import math

import torch

from . import attention as attn
from . import moe

RMS_EPS = 1e-5


def make_weights(seed: int, hidden: int = 4096, hq: int = 32, hkv: int = 4, d: int = 128,
                 n_experts: int = 128, inner: int = 768, bias_std: float = 0.0):
    """Random-init layer weights, CPU generator: dense N(0, 1/sqrt(K)) bf16, norm weights
    0.1 N bf16, router fp32 (same families as muse_decode_layer/reference.py:89-128)."""
    gen = torch.Generator().manual_seed(seed)

    def dense(n, k, dtype=torch.bfloat16):
        return (torch.randn((n, k), generator=gen) / math.sqrt(k)).to(dtype)

    def vec(n, std=0.1):
        return (std * torch.randn((n,), generator=gen)).to(torch.bfloat16)

    qkv_n = 2 * hq * d + 2 * hkv * d
    w = {
        "input_norm": vec(hidden),
        "qkv_gate": dense(qkv_n, hidden),
        "o": dense(hidden, hq * d),
        "pre_expert_norm": vec(hidden),
        # router rows scaled so logits are ~N(0,1) on a unit-RMS input
        "router": dense(n_experts, hidden, torch.float32),
        "router_bias": bias_std * torch.randn((n_experts,), generator=gen),
    }
    ex = moe.make_weights(seed + 1, n_experts=n_experts, hidden=hidden, inner=inner)
    w.update({k: ex[k] for k in ("w13", "w13_sf", "w13_gs", "w2", "w2_sf", "w2_gs")})
    w["post_expert_norm"] = ex["post_norm_w"]
    return w


def make_input(batch: int, seq_lens, seed: int, q_len: int = 1, hidden: int = 4096, hq: int = 32, hkv: int = 4,
               d: int = 128, page: int = 64, window: int = 0, rope_theta: float = 1e6, max_len=None):
    """Residual stream ~ N(0,1) fp32 [T,H] plus the attention step's cache and metadata
    (oracle.attention.make_input; its `qkv` field is dropped: the layer computes it)."""
    data = attn.make_input(batch, seq_lens, seed, q_len=q_len, hq=hq, hkv=hkv, d=d, page=page,
                           window=window, rope_theta=rope_theta, max_len=max_len)
    del data["qkv"]
    gen = torch.Generator().manual_seed(seed + 77)
    t = batch * q_len
    data["stream"] = torch.randn((t, hidden), generator=gen)
    data["config"]["tokens"] = t
    data["config"]["hidden"] = hidden
    return data


def front(data, weights):
    """Everything up to the router logits.  Returns a dict of intermediates."""
    cfg = data["config"]
    stream = data["stream"].float()
    x = (attn.rms(stream, RMS_EPS) * (1.0 + weights["input_norm"].float())).to(torch.bfloat16)
    qkv = (x.float() @ weights["qkv_gate"].float().T).to(torch.bfloat16)
    a_in = dict(data)
    a_in["qkv"] = qkv.view(cfg["batch"], cfg["q_len"], -1)
    o, k_new, v_new = attn.ref_kernel(a_in)
    o = o.reshape(cfg["tokens"], -1).to(torch.bfloat16)
    stream1 = stream + o.float() @ weights["o"].float().T
    h = attn.rms(stream1, RMS_EPS) * (1.0 + weights["pre_expert_norm"].float())
    logits = (h.double() @ weights["router"].double().T).float() + weights["router_bias"].float()
    return {"x": x, "qkv": qkv, "o": o, "stream1": stream1, "h": h, "logits": logits,
            "k_new": k_new, "v_new": v_new}


def back(fr, weights, ids: torch.Tensor, local_start: int = 0, local_count: int | None = None):
    """Experts and the second residual with the given expert choice ids [T,8]."""
    p = torch.softmax(fr["logits"].float(), dim=-1).gather(1, ids.long())
    tw = p / p.sum(-1, keepdim=True)
    n_exp = weights["router"].shape[0]
    md = {"hidden_states": fr["h"].to(torch.bfloat16), "topk_ids": ids.to(torch.int32), "topk_weights": tw,
          "config": {"local_start": local_start, "local_count": n_exp if local_count is None else local_count}}
    mw = dict(weights)
    mw["post_norm_w"] = weights["post_expert_norm"]
    y = moe.ref_kernel(md, mw, fp32_out=True)
    return fr["stream1"] + y, y


def ref_kernel(data, weights, topk_ids=None):
    """(hidden bf16 [T,H], stream fp32 [T,H], topk_ids int32 [T,8], k_new, v_new)."""
    fr = front(data, weights)
    ids = moe.route_softmax(fr["logits"])[0] if topk_ids is None else topk_ids
    stream2, _ = back(fr, weights, ids)
    return stream2.to(torch.bfloat16), stream2, ids, fr["k_new"], fr["v_new"]


# ---------------------------------------------------------------------------------------------------------------
# The reference's own form of the layer (muse_decode_layer/reference.py:339-477): the attention input arrives
# normalised, both residual boundaries are norm-preserving gated mixes, the router scores are sigmoids chosen by
# score + bias, and the experts sit between a pooler and an unpooler projection.  Shapes come from the weights and
# the config instead of module constants.
RESIDUAL_TEMPERATURE = 0.3   # reference.py:52
RESIDUAL_GATE_EPS = 1e-3     # reference.py:53
ROUTER_MULTIPLIER = 0.1767766952966369  # reference.py:49
ROUTE_EPS = 1e-15            # reference.py:51
SLICED_MAX_TOKENS = 8        # reference.py:56
BRANCH_EPS = 1e-8            # the boundary's RMSNorm of the branch (POST_NORM_EPS, reference.py:40)


def residual_coefficients(gate: torch.Tensor):
    """(alpha, beta) of new = alpha * stream + beta * branch (reference.py:339-344)."""
    w = gate.float() / RESIDUAL_TEMPERATURE
    beta = torch.sigmoid(w)
    alpha = torch.sqrt(torch.clamp(torch.sigmoid(-w) * (1.0 + beta), min=RESIDUAL_GATE_EPS))
    return alpha, beta


def route_sigmoid(h: torch.Tensor, weights):
    """(unbiased sigmoid scores, biased scores that choose the experts), FP32 [T, E]; logits in FP64
    (reference.py:419-424)."""
    logits = h.double() @ weights["router"].double().T
    scores = torch.sigmoid(logits * ROUTER_MULTIPLIER).float()
    return scores, scores + weights["router_bias"].float()


def native_front(data, weights):
    """Everything up to the router in the reference's form (reference.py:447-457)."""
    cfg = data["config"]
    a_in = dict(data)
    qkv = data["attn_input"].float() @ weights["qkv_gate"].float().T   # stays FP32 (reference.py:360)
    a_in["qkv"] = qkv.view(cfg["batch"], cfg["q_len"], -1)
    o, k_new, v_new = attn.ref_kernel(a_in, scale_after_rope=True)
    a = o.reshape(cfg["tokens"], -1) @ weights["o"].float().T
    alpha1, beta1 = residual_coefficients(weights["attn_residual_gate"])
    stream1 = alpha1 * data["stream"].float() + beta1 * attn.rms(a, BRANCH_EPS)
    h = attn.rms(stream1, RMS_EPS) * (1.0 + weights["pre_ffn_norm"].float())
    scores, biased = route_sigmoid(h, weights)
    return {"stream1": stream1, "h": h, "scores": scores, "biased": biased, "k_new": k_new, "v_new": v_new,
            "local_start": int(data["local_start"])}


def native_back(fr, weights, ids: torch.Tensor):
    """Pooler, local experts, (sliced) unpooler and the second boundary (reference.py:460-477)."""
    n_exp = weights["router"].shape[0]
    picked = fr["scores"].gather(1, ids.long())
    tw = picked / (picked.sum(-1, keepdim=True) + ROUTE_EPS)
    p = attn.rms(fr["h"] @ weights["pooler"].float().T, RMS_EPS) * (1.0 + weights["pre_expert_norm"].float())
    local = (ids.long() - fr["local_start"]) % n_exp
    md = {"hidden_states": p, "topk_ids": local.to(torch.int32), "topk_weights": tw,
          "config": {"local_start": 0, "local_count": weights["w13"].shape[0]}}
    mw = dict(weights, post_norm_w=weights["post_expert_norm"])
    y = moe.ref_kernel(md, mw, fp32_out=True)
    hidden_dim = fr["stream1"].shape[1]
    if y.shape[0] <= SLICED_MAX_TOKENS:   # few tokens: this GPU computes only its eighth of the unpooler's columns
        f = torch.zeros_like(fr["stream1"])
        sl = hidden_dim // 8
        f[:, :sl] = y @ weights["unpooler"][:sl].float().T
    else:
        f = y @ weights["unpooler"].float().T
    f = f * (1.0 + weights["post_ffn_norm"].float())
    alpha2, beta2 = residual_coefficients(weights["ffn_residual_gate"])
    stream2 = alpha2 * fr["stream1"] + beta2 * attn.rms(f, BRANCH_EPS)
    hidden = attn.rms(stream2, RMS_EPS) * (1.0 + weights["next_pre_attn_norm"].float())
    return hidden.to(torch.bfloat16), stream2


def native_ref_kernel(data, weights, topk_ids=None, top_k: int = 8):
    """(hidden bf16, stream fp32, ids int32, k_new, v_new) in the reference's form (reference.py:559-566)."""
    fr = native_front(data, weights)
    ids = fr["biased"].topk(top_k, dim=-1).indices.to(torch.int32) if topk_ids is None else topk_ids
    hidden, stream = native_back(fr, weights, ids)
    return hidden, stream, ids, fr["k_new"], fr["v_new"]


def algorithmic_bytes(data, weights, ids: torch.Tensor) -> int:
    """Dense weights + router + visible KV + touched experts + 12 B per token-channel of activations."""
    cfg = data["config"]
    dense = sum(weights[k].numel() * weights[k].element_size() for k in ("qkv_gate", "o", "router"))
    kv = attn.algorithmic_bytes({**data, "config": cfg}) - cfg["tokens"] * (
        (2 * cfg["num_q_heads"] + 2 * cfg["num_kv_heads"]) * cfg["head_dim"] * 2
        + cfg["num_q_heads"] * cfg["head_dim"] * 2 + cfg["num_kv_heads"] * cfg["head_dim"] * 2)
    per = sum(weights[k][0].numel() * weights[k][0].element_size() for k in ("w13", "w13_sf", "w2", "w2_sf"))
    touched = int(torch.unique(ids.long()).numel())
    return dense + kv + touched * per + 12 * cfg["tokens"] * cfg["hidden"]
