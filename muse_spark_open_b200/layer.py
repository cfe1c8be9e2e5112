"""The whole decoder layer's decode step: `prepare(weights) -> state`, `kernel_fn(data, state)`.

Same call shape as muse_decode_layer/submission.py:3978-4038: `data` carries the FP32 residual
`stream` [T, H], the attention step's cache and metadata (muse_attention_decode `Inputs` fields) and
`config`; the result is `(hidden bf16 [T, H], stream fp32 [T, H], topk_ids int32 [T, 8])`, and the
new K/V rows are written into `data["k_cache"]` / `data["v_cache"]` in place.  The op list is the
benchmark's: input RMSNorm, QKV+gate projection, gated attention, o_proj, residual, pre-expert
RMSNorm, FP32 router (softmax top-8 renormalised), NVFP4 experts, residual.
All scratch lives in `state`, sized per token count on first use (outside timing), so the timed
call allocates only its three outputs.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import abi, attention, moe, proj

RMS_EPS = 1e-5
TOP_K = 8


def launches_per_step(tokens: int) -> int:
    """Kernels one layer step launches: input norm, QKV projection, attention, o projection, router, the two expert
    GEMMs (the first applies the activation) and the combine; above 32 tokens also the pass that gathers the
    expert inputs into expert-list order."""
    return 8 + (tokens > 32)


def prepare(weights: dict, local_start: int = 0, local_count: int | None = None) -> dict:
    """weights: input_norm, qkv_gate, o, pre_expert_norm, router (fp32), router_bias (optional),
    w13, w13_sf, w13_gs, w2, w2_sf, w2_gs, post_expert_norm (the experts given may be only this
    rank's: then pass local_start / local_count)."""
    if not weights["qkv_gate"].is_cuda:
        raise abi.MskError("prepare() needs CUDA weights")
    n_exp = weights["router"].shape[0]
    st = {
        "input_norm": weights["input_norm"].contiguous(), "qkv_gate": weights["qkv_gate"].contiguous(),
        "o": weights["o"].contiguous(), "pre_expert_norm": weights["pre_expert_norm"].contiguous(),
        "router": weights["router"].float().contiguous(),
        "router_bias": weights["router_bias"].float().contiguous() if weights.get("router_bias") is not None else None,
        "E": n_exp, "local_start": local_start,
        "local_count": weights["w13"].shape[0] if local_count is None else local_count,
        "moe": moe.prepare(weights, weights_start=local_start), "bufs": {},
    }
    return st


def buffers(state: dict, t: int, device) -> dict:
    if t not in state["bufs"]:
        h = state["qkv_gate"].shape[1]
        nqkv, no = state["qkv_gate"].shape[0], state["o"].shape[1]
        e = state["E"]
        f32, bf = torch.float32, torch.bfloat16
        mk = lambda shape, dt: torch.empty(shape, dtype=dt, device=device)
        state["bufs"][t] = {
            "xn0": mk((t, h), bf), "ssq0": mk((t,), f32), "qkv": mk((t, nqkv), bf), "attn": mk((t, no), bf),
            "stream1": mk((t, h), f32), "xn1": mk((t, h), torch.float16), "ssq1": mk((h // 128 + 1, t), f32),
            "router_part": mk((h // 128, t, e), f32),
            "router_ticket": torch.zeros((((t + 31) // 32) * ((e + 31) // 32 + 1),), dtype=torch.int32, device=device),
            "logits": mk((t, e), f32), "topk_ids": mk((t, TOP_K), torch.int32), "topk_weights": mk((t, TOP_K), f32),
        }
    return state["bufs"][t]


def fill_front(f: abi.LayerFront, data: dict, state: dict, buf: dict, tune: dict) -> None:
    cfg = data["config"]
    f.B, f.L, f.H = cfg["batch"], cfg["q_len"], state["qkv_gate"].shape[1]
    f.Hq, f.Hkv, f.d = cfg["num_q_heads"], cfg["num_kv_heads"], cfg["head_dim"]
    f.page_size, f.num_pages, f.max_pages = cfg["page_size"], data["k_cache"].shape[0], data["page_table"].shape[1]
    f.window, f.qk_scale_factor, f.sm_scale, f.norm_eps = cfg["window"], cfg["qk_scale_factor"], cfg["sm_scale"], RMS_EPS
    f.stream = abi.ptr(data["stream"])
    f.k_cache, f.v_cache = abi.ptr(data["k_cache"]), abi.ptr(data["v_cache"])
    f.k_scale, f.v_scale = abi.ptr(data["k_scale"]), abi.ptr(data["v_scale"])
    f.seq_lens, f.page_table, f.cache_loc = abi.ptr(data["seq_lens"]), abi.ptr(data["page_table"]), abi.ptr(data["cache_loc"])
    fr = attention.inv_freq(cfg["rope_theta"], cfg["head_dim"], data["stream"].device)
    f.inv_freq = abi.ptr(fr) if fr is not None else None
    f.input_norm_w, f.w_qkv, f.w_o = abi.ptr(state["input_norm"]), abi.ptr(state["qkv_gate"]), abi.ptr(state["o"])
    f.pre_expert_norm_w, f.router_w = abi.ptr(state["pre_expert_norm"]), abi.ptr(state["router"])
    f.router_bias = abi.ptr(state["router_bias"]) if state["router_bias"] is not None else None
    f.E = state["E"]
    for name in ("xn0", "ssq0", "qkv", "attn", "stream1", "xn1", "ssq1", "router_part", "router_ticket", "logits",
                 "topk_ids", "topk_weights"):
        setattr(f, name, abi.ptr(buf[name]))
    # split-K workspaces of the two projections (one each: their launches are chained programmatically), kept per
    # (shape, splits) and allocated on first use
    t, h = buf["xn0"].shape
    dev = buf["xn0"].device
    qs = proj.scratch_for(t, buf["qkv"].shape[1], h, tune.get("qkv_splits", 0), dev, tag=("qkv", id(state)))
    os_ = proj.scratch_for(t, h, buf["attn"].shape[1], tune.get("o_splits", 0), dev, tag=("o", id(state)))
    f.qkv_scratch, f.o_scratch = abi.ptr(qs), abi.ptr(os_)
    f.qkv_scratch_bytes, f.o_scratch_bytes = qs.numel(), os_.numel()
    f.top_k = TOP_K
    f.attn_chunks, f.attn_stages = tune.get("attn_chunks", 0), tune.get("attn_stages", 0)
    f.attn_issuers, f.attn_row_groups = tune.get("attn_issuers", 0), tune.get("attn_row_groups", 0)
    f.qkv_splits, f.o_splits, f.pdl = tune.get("qkv_splits", 0), tune.get("o_splits", 0), 0


def front(data: dict, state: dict, **tune) -> dict:
    """Everything up to the router's expert choice (the part an expert-parallel rank runs before the exchange)."""
    cfg = data["config"]
    t = cfg["batch"] * cfg["q_len"]
    buf = buffers(state, t, data["stream"].device)
    # the argument block depends only on addresses, shapes and a few config scalars: it is rebuilt when one of
    # them changes, not on every step (filling it costs as much host time as a small kernel takes on the GPU)
    key = (tuple(data[k].data_ptr() for k in ("stream", "k_cache", "v_cache", "k_scale", "v_scale", "seq_lens", "page_table",
                                              "cache_loc")),
           data["k_cache"].shape[0], data["page_table"].shape[1], tuple(sorted(cfg.items())), tuple(sorted(tune.items())))
    cached = state.get("front_args")
    if cached is None or cached[0] != key:
        f = abi.LayerFront()
        fill_front(f, data, state, buf, tune)
        state["front_args"] = cached = (key, f)
    f = cached[1]
    st = abi.status_for(data["stream"].device)
    abi.check(abi.lib().msk_layer_front(C.byref(f), st.p, abi.stream_ptr()), "msk_layer_front")
    return buf


MAX_TOKENS = 256


def kernel_fn(data: dict, state: dict, **tune):
    stream = data["stream"]
    if stream.dtype != torch.float32 or not stream.is_cuda:
        raise abi.MskError("stream must be a float32 CUDA tensor")
    t, h = stream.shape
    if t > MAX_TOKENS:
        # the chain is built for decode / verify steps of up to MAX_TOKENS tokens; larger batches run as consecutive
        # groups of requests over the same cache (each group streams the weights again)
        cfg = data["config"]
        l = cfg["q_len"]
        per = max(1, MAX_TOKENS // l)
        outs = []
        for b0 in range(0, cfg["batch"], per):
            b1 = min(cfg["batch"], b0 + per)
            sub = dict(data, config=dict(cfg, batch=b1 - b0, tokens=(b1 - b0) * l))
            for k in ("seq_lens", "page_table"):
                sub[k] = data[k][b0:b1]
            for k in ("stream", "cache_loc", "positions"):
                if k in data:
                    sub[k] = data[k][b0 * l:b1 * l]
            outs.append(kernel_fn(sub, state, **tune))
        return tuple(torch.cat([o[i] for o in outs]) for i in range(3))
    buf = buffers(state, t, stream.device)
    ms = state["moe"]
    s1, s2 = tune.get("moe_splits") or moe.splits_for(t, ms["H"], ms["I"], state["local_count"], TOP_K)
    h1, y, inter, xs, pub = moe.scratch(ms, t, TOP_K, s1, s2, stream.device)
    hidden = torch.empty((t, h), dtype=torch.bfloat16, device=stream.device)
    out = torch.empty((t, h), dtype=torch.float32, device=stream.device)
    ids = torch.empty((t, TOP_K), dtype=torch.int32, device=stream.device)
    p = abi.LayerParams()
    fill_front(p.front, data, state, buf, tune)
    p.front.topk_ids = abi.ptr(ids)
    m = p.moe
    m.local_start, m.local_count = state["local_start"], state["local_count"]
    m.w13_packed, m.w2_packed = abi.ptr(ms["w13"]), abi.ptr(ms["w2"])
    m.w13_gs, m.w2_gs = abi.ptr(ms["w13_gs"]), abi.ptr(ms["w2_gs"])
    m.post_norm_w, m.post_eps, m.I = abi.ptr(ms["post_w"]), moe.POST_NORM_EPS, ms["I"]
    m.h1_part, m.y_part, m.s1, m.s2 = abi.ptr(h1), abi.ptr(y), s1, s2
    m.inter_sorted, m.x_sorted, m.route_pub = abi.ptr(inter), abi.ptr(xs), abi.ptr(pub)
    m.out, m.out_fp32, m.ldo = abi.ptr(out), 1, h
    m.out_copy, m.ldc = abi.ptr(hidden), h
    st = abi.status_for(stream.device)
    abi.check(abi.lib().msk_layer_decode(C.byref(p), st.p, abi.stream_ptr()), "msk_layer_decode")
    return hidden, out, ids


# ---------------------------------------------------------------------------------------------------------------
# The reference's own layer form (muse_decode_layer/reference.py:447-477), for head_dim 128: the attention input
# arrives normalised (bf16), both residual boundaries are norm-preserving gated mixes, the router scores are sigmoids
# chosen by score + bias, and the experts sit between a pooler and an unpooler projection (for up to 8 tokens only the
# first eighth of the unpooler's columns is computed, the rest of the branch is zero).  A chain of the same kernels
# plus msk_residual_boundary / msk_router / msk_rmsnorm; nothing is fused across the boundaries (13 launches).
ROUTER_MULTIPLIER = 0.1767766952966369
BRANCH_EPS = 1e-8
SLICED_MAX_TOKENS = 8


def native_prepare(weights: dict) -> dict:
    """weights: the reference's names (muse_decode_layer/reference.py:89-128): qkv_gate, o, attn_residual_gate,
    pre_ffn_norm, router, router_bias, pooler, pre_expert_norm, w13 / w13_sf / w13_gs / w2 / w2_sf / w2_gs (this GPU's
    experts), post_expert_norm, unpooler, post_ffn_norm, ffn_residual_gate, next_pre_attn_norm."""
    if not weights["qkv_gate"].is_cuda:
        raise abi.MskError("native_prepare() needs CUDA weights")
    st = {k: weights[k].contiguous() for k in ("qkv_gate", "o", "attn_residual_gate", "pre_ffn_norm", "pooler", "pre_expert_norm",
                                               "unpooler", "post_ffn_norm", "ffn_residual_gate", "next_pre_attn_norm")}
    st["router"] = weights["router"].float().contiguous()
    st["router_bias"] = weights["router_bias"].float().contiguous()
    st["moe"] = moe.prepare(weights)
    st["local_count"] = weights["w13"].shape[0]
    st["bufs"] = {}
    return st


def native_kernel_fn(data: dict, state: dict):
    """(hidden bf16 [T, H], stream fp32 [T, H], topk_ids int32 [T, 8]); new K/V rows written in place.  `data` as the
    reference's generate_input gives it (stream, attn_input, the attention step's cache and metadata, local_start)."""
    cfg = data["config"]
    stream, x = data["stream"], data["attn_input"]
    t, h = stream.shape
    dev = stream.device
    if t > MAX_TOKENS or h % 1024 or cfg["head_dim"] != 128:
        raise abi.MskError("native layer form: up to 256 tokens, hidden a multiple of 1024, head_dim 128")
    lib, sp = abi.lib(), abi.stream_ptr
    d_exp, e = state["pooler"].shape[0], state["router"].shape[0]
    nqkv, no = state["qkv_gate"].shape[0], state["o"].shape[1]
    key = (t, dev.index)
    if key not in state["bufs"]:
        f32, bf = torch.float32, torch.bfloat16
        mk = lambda shape, dt: torch.empty(shape, dtype=dt, device=dev)  # noqa: E731
        state["bufs"][key] = {
            "qkv": mk((t, nqkv), bf), "attn": mk((t, no), bf), "a": mk((t, h), f32), "s1": mk((t, h), f32), "hn": mk((t, h), bf),
            "ssq": mk((2, t), f32), "part": mk((h // 128, t, e), f32),
            "ticket": torch.zeros((((t + 31) // 32) * ((e + 31) // 32 + 1),), dtype=torch.int32, device=dev),
            "logits": mk((t, e), f32), "wts": mk((t, TOP_K), f32), "pool": mk((t, d_exp), f32), "p": mk((t, d_exp), bf),
            "pssq": mk((t,), f32), "y": mk((t, d_exp), bf), "f": mk((t, h), f32),
        }
    b = state["bufs"][key]
    st = abi.status_for(dev)
    # attention on the given (already normalised) input
    proj.skinny(x, state["qkv_gate"], out=b["qkv"])
    attention.launch(b["qkv"], b["attn"], data, cfg, pdl=True)
    proj.skinny(b["attn"], state["o"], out=b["a"], pdl=True)
    # boundary 1: stream1, the FFN input h = rmsnorm(stream1) * (1 + w) and its sum of squares
    bp = abi.BoundaryParams()
    bp.stream, bp.branch, bp.branch_bf16, bp.ldb = abi.ptr(stream), abi.ptr(b["a"]), 0, h
    bp.gate, bp.next_norm_w = abi.ptr(state["attn_residual_gate"]), abi.ptr(state["pre_ffn_norm"])
    bp.stream_out, bp.normed_out, bp.ssq_out = abi.ptr(b["s1"]), abi.ptr(b["hn"]), abi.ptr(b["ssq"][0])
    bp.T, bp.H, bp.branch_eps, bp.eps, bp.temperature, bp.gate_eps, bp.pdl = t, h, BRANCH_EPS, RMS_EPS, 0.3, 1e-3, 1
    abi.check(lib.msk_residual_boundary(C.byref(bp), sp()), "msk_residual_boundary")
    # router on FP32 rmsnorm(stream1) * (1 + w): sigmoid scores, chosen by score + bias
    ids = torch.empty((t, TOP_K), dtype=torch.int32, device=dev)
    rp = abi.RouterParams()
    rp.x, rp.norm_w, rp.ssq, rp.ssq_parts, rp.eps = abi.ptr(b["s1"]), abi.ptr(state["pre_ffn_norm"]), abi.ptr(b["ssq"]), 1, RMS_EPS
    rp.router_w, rp.router_bias, rp.E, rp.T, rp.H, rp.top_k = abi.ptr(state["router"]), abi.ptr(state["router_bias"]), e, t, h, TOP_K
    rp.sigmoid_bias, rp.multiplier = 1, ROUTER_MULTIPLIER
    rp.part, rp.ticket, rp.logits = abi.ptr(b["part"]), abi.ptr(b["ticket"]), abi.ptr(b["logits"])
    rp.topk_ids, rp.topk_weights, rp.pdl = abi.ptr(ids), abi.ptr(b["wts"]), 1
    abi.check(lib.msk_router(C.byref(rp), st.p, sp()), "msk_router")
    # pooler, pre-expert norm, local experts
    proj.skinny(b["hn"], state["pooler"], out=b["pool"], pdl=True)
    abi.check(lib.msk_rmsnorm(abi.ptr(b["pool"]), abi.ptr(state["pre_expert_norm"]), abi.ptr(b["p"]), abi.ptr(b["pssq"]), t, d_exp,
                              RMS_EPS, 1, sp()), "msk_rmsnorm")
    local_start = int(data["local_start"])             # the prepared experts are, by definition, the ones that start here
    state["moe"]["weights_start"] = local_start
    moe.forward(b["p"], ids, b["wts"], state["moe"], local_start, state["local_count"], out=b["y"], pdl=True)
    # unpooler (sliced for few tokens), boundary 2
    if t <= SLICED_MAX_TOKENS:
        b["f"].zero_()
        sl = h // 8
        proj.skinny(b["y"], state["unpooler"][:sl], out=b["f"][:, :sl])
    else:
        proj.skinny(b["y"], state["unpooler"], out=b["f"], pdl=True)
    out = torch.empty((t, h), dtype=torch.float32, device=dev)
    hidden = torch.empty((t, h), dtype=torch.bfloat16, device=dev)
    bp2 = abi.BoundaryParams()
    bp2.stream, bp2.branch, bp2.branch_bf16, bp2.ldb = abi.ptr(b["s1"]), abi.ptr(b["f"]), 0, h
    bp2.branch_w, bp2.gate, bp2.next_norm_w = abi.ptr(state["post_ffn_norm"]), abi.ptr(state["ffn_residual_gate"]), abi.ptr(state["next_pre_attn_norm"])
    bp2.stream_out, bp2.normed_out = abi.ptr(out), abi.ptr(hidden)
    bp2.T, bp2.H, bp2.branch_eps, bp2.eps, bp2.temperature, bp2.gate_eps, bp2.pdl = t, h, BRANCH_EPS, RMS_EPS, 0.3, 1e-3, 1
    abi.check(lib.msk_residual_boundary(C.byref(bp2), sp()), "msk_residual_boundary")
    return hidden, out, ids
