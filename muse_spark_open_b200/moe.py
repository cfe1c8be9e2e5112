"""NVFP4 routed experts: the reference's per-op entry points over the C ABI.

`prepare(weights) -> state` repacks the experts once (lossless: same E2M1 codes and E4M3 scales,
re-ordered into 9216-byte blocks, gate and up rows of W13 interleaved); `kernel_fn(data, state) -> bf16 [T, H]`
with the `Weights` / `Config` / `Inputs` fields of muse_moe_w4a16/submission.py:32-57 (ids and
weights are inputs, experts outside [local_start, local_start + local_count) are skipped).
Layer hooks like the reference's (submission.py:888-896): `data["pre_norm"] = (ssq [parts, T], dim,
eps)` folds the pre-expert RMSNorm row scale into the first GEMM; `data["router_logits"]` moves
softmax / top-8 / renormalisation into the GEMM CTAs (ids and weights are then outputs).
"""
from __future__ import annotations

import ctypes as C

import torch

from . import abi

POST_NORM_EPS = 1e-8
MAX_TOKENS = 256


def splits_for(tokens: int, h: int, inner: int, local_count: int = 128, top_k: int = 8, sms: int = 148) -> tuple[int, int]:
    """K splits of the two GEMMs.  gemm 1 runs unsplit: its epilogue then applies silu(gate) * up itself and
    the activation kernel and the FP32 partials between the GEMMs disappear (a unit is 32 blocks of 9 KB, long
    enough to stream at full rate).  gemm 2's units are 6 blocks: with few expert-groups (few tokens, or few
    local experts under expert parallelism) two splits give every SM a few of them."""
    s2 = 2 if tokens <= 4 else 1
    groups = max(1, min(local_count, tokens * top_k))  # expert-groups (<= 32 pairs each) touched, roughly
    chunks = inner // 128
    while s2 < 2 and groups * (h // 128) * s2 < 3 * sms and chunks % (2 * s2) == 0 and chunks // (2 * s2) >= 2:
        s2 *= 2
    while chunks % s2:
        s2 //= 2
    return 1, max(s2, 1)


def prepare(weights: dict, weights_start: int = 0) -> dict:
    w13, w2 = weights["w13"], weights["w2"]
    if not w13.is_cuda:
        raise abi.MskError("prepare() needs CUDA weights")
    e, r13, hk = w13.shape
    h, inner = hk * 2, r13 // 2
    lib = abi.lib()
    n13, n2 = C.c_size_t(), C.c_size_t()
    abi.check(lib.msk_moe_packed_bytes(e, h, inner, C.byref(n13), C.byref(n2)), "msk_moe_packed_bytes")
    p13 = torch.empty(n13.value, dtype=torch.uint8, device=w13.device)
    p2 = torch.empty(n2.value, dtype=torch.uint8, device=w13.device)
    mw = abi.MoeWeights()
    mw.w13, mw.w13_sf = abi.ptr(w13.contiguous()), abi.ptr(weights["w13_sf"].contiguous())
    mw.w2, mw.w2_sf = abi.ptr(w2.contiguous()), abi.ptr(weights["w2_sf"].contiguous())
    mw.E, mw.H, mw.I = e, h, inner
    abi.check(lib.msk_moe_pack(C.byref(mw), abi.ptr(p13), abi.ptr(p2), abi.stream_ptr()), "msk_moe_pack")
    torch.cuda.synchronize()
    post = weights.get("post_norm_w", weights.get("post_expert_norm"))
    return {"w13": p13, "w2": p2, "w13_gs": weights["w13_gs"].float().contiguous(),
            "w2_gs": weights["w2_gs"].float().contiguous(), "post_w": post.contiguous(),
            "E": e, "H": h, "I": inner, "weights_start": weights_start, "scratch": {}}


def scratch(state: dict, tokens: int, top_k: int, s1: int, s2: int, device):
    """The scratch buffers (FP32 partials, FP16 activations and staged inputs, routing list), kept per
    (tokens, splits) in `state` (allocated once, outside timing)."""
    key = (tokens, top_k, s1, s2)
    if key not in state["scratch"]:
        pairs = tokens * top_k
        h1 = torch.empty((s1, pairs, 2 * state["I"]), dtype=torch.float32, device=device) if s1 > 1 else None
        y = torch.empty((s2, pairs, state["H"]), dtype=torch.float32, device=device)
        inter = torch.empty((pairs, state["I"]), dtype=torch.float16, device=device)
        xs = torch.empty((pairs if tokens > 32 else tokens, state["H"]), dtype=torch.float16, device=device)
        pub = torch.zeros((2 + pairs,), dtype=torch.int32, device=device) if s1 > 1 else None
        state["scratch"][key] = (h1, y, inter, xs, pub)
    return state["scratch"][key]


def forward(x, ids, wts, state, local_start, local_count, out=None, logits=None, pre_norm=None, resid=None,
            splits=None, pdl=False):
    t, h = x.shape
    top_k = ids.shape[1]
    if out is None:
        out = torch.empty((t, h), dtype=torch.bfloat16, device=x.device)
    if t > MAX_TOKENS:
        # the kernels are built for decode / verify steps; more tokens (the reference's 257-token case,
        # muse_moe_w4a16/bench.py:15) run as consecutive blocks of MAX_TOKENS, each streaming its experts again
        for r0 in range(0, t, MAX_TOKENS):
            r1 = min(t, r0 + MAX_TOKENS)
            pn = None
            if pre_norm is not None:
                ssq = pre_norm[0]
                pn = ((ssq[:, r0:r1].contiguous() if ssq.dim() == 2 else ssq[r0:r1]), pre_norm[1], pre_norm[2])
            forward(x[r0:r1], ids[r0:r1], wts[r0:r1], state, local_start, local_count, out=out[r0:r1],
                    logits=None if logits is None else logits[r0:r1], pre_norm=pn,
                    resid=None if resid is None else resid[r0:r1], splits=splits, pdl=pdl)
        return out
    # the argument block depends only on addresses, strides and scalars: rebuilt when one changes, not per call
    if x.dtype not in (torch.bfloat16, torch.float16):
        raise abi.MskError("the expert input must be bfloat16 or float16")
    key = (x.data_ptr(), x.stride(0), x.dtype, ids.data_ptr(), wts.data_ptr(), ids.stride(0), out.data_ptr(), out.stride(0), out.dtype,
           t, top_k, local_start, local_count, splits, pdl,
           None if logits is None else (logits.data_ptr(), logits.stride(0)),
           None if pre_norm is None else (pre_norm[0].data_ptr(), tuple(pre_norm[0].shape), pre_norm[0].stride(0), pre_norm[1], pre_norm[2]),
           None if resid is None else (resid.data_ptr(), resid.stride(0)))
    cached = state.get("forward_args")
    if cached is not None and cached[0] == key:
        st = abi.status_for(x.device)
        abi.check(abi.lib().msk_moe_forward(C.byref(cached[1]), st.p, abi.stream_ptr()), "msk_moe_forward")
        return out
    s1, s2 = splits or splits_for(t, state["H"], state["I"], local_count, top_k)
    h1, y, inter, xs, pub = scratch(state, t, top_k, s1, s2, x.device)
    p = abi.MoeParams()
    p.x, p.ldx, p.x_fp16 = abi.ptr(x), x.stride(0), int(x.dtype == torch.float16)
    if pre_norm is not None:
        ssq, dim, eps = pre_norm  # [parts, T] contiguous, or one value per token with any stride
        p.x_ssq, p.x_inv_dim, p.x_eps = abi.ptr(ssq), 1.0 / dim, eps
        p.x_ssq_parts, p.x_ssq_tstride = (ssq.shape[0], 1) if ssq.dim() == 2 else (1, ssq.stride(0))
    if ids.stride(0) != wts.stride(0) or ids.stride(1) != 1 or wts.stride(1) != 1:
        raise abi.MskError("topk_ids and topk_weights need the same row stride and unit column stride")
    p.topk_ids, p.topk_weights, p.ld_topk = abi.ptr(ids), abi.ptr(wts), ids.stride(0)
    if logits is not None:
        p.logits, p.n_logits, p.ld_logits = abi.ptr(logits), logits.shape[1], logits.stride(0)
    p.T, p.top_k = t, top_k
    first = local_start - state["weights_start"]
    if first < 0 or first + local_count > state["E"]:
        raise abi.MskError("local expert range outside the prepared weights")
    blob13 = (2 * state["I"] // 128) * (state["H"] // 128) * 9216
    blob2 = (state["H"] // 128) * (state["I"] // 128) * 9216
    p.local_start, p.local_count = local_start, local_count
    p.w13_packed, p.w2_packed = state["w13"].data_ptr() + first * blob13, state["w2"].data_ptr() + first * blob2
    p.w13_gs, p.w2_gs = state["w13_gs"].data_ptr() + 4 * first, state["w2_gs"].data_ptr() + 4 * first
    p.post_norm_w, p.post_eps, p.H, p.I = abi.ptr(state["post_w"]), POST_NORM_EPS, state["H"], state["I"]
    p.h1_part, p.y_part, p.s1, p.s2 = abi.ptr(h1), abi.ptr(y), s1, s2
    p.inter_sorted, p.x_sorted, p.route_pub = abi.ptr(inter), abi.ptr(xs), abi.ptr(pub)
    if resid is not None:
        p.resid, p.ldr = abi.ptr(resid), resid.stride(0)
    p.out, p.out_fp32, p.ldo, p.pdl = abi.ptr(out), int(out.dtype == torch.float32), out.stride(0), int(pdl)
    state["forward_args"] = (key, p)
    st = abi.status_for(x.device)
    abi.check(abi.lib().msk_moe_forward(C.byref(p), st.p, abi.stream_ptr()), "msk_moe_forward")
    return out


def kernel_fn(data: dict, state: dict) -> torch.Tensor:
    cfg = data["config"]
    x = data["hidden_states"]
    logits = data.get("router_logits_dev")
    return forward(x, data["topk_ids"], data["topk_weights"], state, cfg["local_start"], cfg["local_count"],
                   logits=logits, pre_norm=data.get("pre_norm"))


def dequant(packed: torch.Tensor, e: int, rows: int, k: int, gate_up: bool = False) -> torch.Tensor:
    """Test hook: BF16 [e, rows, k] = e2m1 * block scale, as the kernels' decoder produces it (rows in the
    original order; gate_up=True for a packed W13)."""
    out = torch.empty((e, rows, k), dtype=torch.bfloat16, device=packed.device)
    abi.check(abi.lib().msk_moe_dequant(abi.ptr(packed), abi.ptr(out), e, rows, k, int(gate_up), abi.stream_ptr()), "msk_moe_dequant")
    return out


STATIC_SCRATCH_BYTES = 4 << 20


def static_scratch_bytes(tokens: int, top_k: int, h: int, inner: int, s1: int, s2: int) -> int:
    """What a call of `msk_moe_forward_static` takes out of the library's built-in array: the five sizes
    `msk_moe_scratch_bytes` reports, each rounded up to 256 bytes."""
    parts = [C.c_size_t() for _ in range(5)]
    abi.check(abi.lib().msk_moe_scratch_bytes(tokens, top_k, h, inner, s1, s2, *[C.byref(v) for v in parts]), "msk_moe_scratch_bytes")
    return sum((v.value + 255) // 256 * 256 for v in parts)


def forward_no_alloc(x, ids, wts, state, local_start, local_count, out, splits=None):
    """The routed experts through `msk_moe_forward_static`: for hosts that cannot give the library scratch
    memory and cannot let it allocate (their pool owns the device, or the step must not stall on an
    allocation).  All scratch sits in a 4 MiB array inside the library, so the call is accepted while
    `static_scratch_bytes(...)` <= STATIC_SCRATCH_BYTES; `out` is the caller's.  Calls share that array: keep
    them in stream order.  Make the first call on a device outside any stream capture."""
    t, h = x.shape
    top_k = ids.shape[1]
    s1, s2 = splits or splits_for(t, state["H"], state["I"], local_count, top_k)
    need = static_scratch_bytes(t, top_k, state["H"], state["I"], s1, s2)
    if need > STATIC_SCRATCH_BYTES:
        raise abi.MskError(f"this step needs {need} bytes of scratch, more than the library's built-in {STATIC_SCRATCH_BYTES}: use forward()")
    p = abi.MoeParams()
    p.x, p.ldx, p.x_fp16 = abi.ptr(x), x.stride(0), int(x.dtype == torch.float16)
    p.topk_ids, p.topk_weights, p.T, p.top_k = abi.ptr(ids), abi.ptr(wts), t, top_k
    first = local_start - state["weights_start"]
    blob13 = (2 * state["I"] // 128) * (state["H"] // 128) * 9216
    blob2 = (state["H"] // 128) * (state["I"] // 128) * 9216
    p.local_start, p.local_count = local_start, local_count
    p.w13_packed, p.w2_packed = state["w13"].data_ptr() + first * blob13, state["w2"].data_ptr() + first * blob2
    p.w13_gs, p.w2_gs = state["w13_gs"].data_ptr() + 4 * first, state["w2_gs"].data_ptr() + 4 * first
    p.post_norm_w, p.post_eps, p.H, p.I = abi.ptr(state["post_w"]), POST_NORM_EPS, state["H"], state["I"]
    p.s1, p.s2 = s1, s2
    p.out, p.out_fp32, p.ldo = abi.ptr(out), int(out.dtype == torch.float32), out.stride(0)
    st = abi.status_for(x.device)
    abi.check(abi.lib().msk_moe_forward_static(C.byref(p), st.p, abi.stream_ptr()), "msk_moe_forward_static")
    return out
