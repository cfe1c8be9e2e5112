"""ctypes binding of libmsk_b200.so (the C ABI declared in include/msk.h).

The library is the product; this module only loads it, mirrors its parameter structs and turns
return codes / the device status word into Python exceptions, the way the reference turns a
failed TORCH_CHECK into one (muse_attention_decode/submission.py:1899).  There is no fallback:
if the library is missing or a GPU is absent, calls raise.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "libmsk_b200.so")

_lib = None

STATUS_CODES = {1: "a bounded device wait expired", 2: "an index was out of range", 3: "a work list overflowed"}
RETURN_CODES = {-1: "invalid argument", -2: "CUDA error", -3: "unsupported shape"}
KERNEL_NAMES = {1: "selftest", 2: "proj_skinny", 3: "attn_decode", 4: "moe_gemm1", 5: "moe_gemm2", 6: "moe_combine",
                7: "layer_glue", 8: "ep_pack"}


class MskError(RuntimeError):
    pass


class ProjParams(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("w", C.c_void_p), ("M", C.c_int), ("N", C.c_int), ("K", C.c_int), ("splits", C.c_int),
        ("token_splits", C.c_int), ("out", C.c_void_p), ("out_fp32", C.c_int), ("ldo", C.c_int),
        ("in_ssq", C.c_void_p), ("in_ssq_parts", C.c_int), ("in_inv_dim", C.c_float), ("in_eps", C.c_float),
        ("resid", C.c_void_p), ("ldr", C.c_int),
        ("next_norm_w", C.c_void_p), ("out_normed", C.c_void_p), ("ldn", C.c_int),
        ("out_ssq", C.c_void_p), ("pdl", C.c_int), ("normed_fp16", C.c_int),
        ("scratch", C.c_void_p), ("scratch_bytes", C.c_size_t),
    ]


def lib() -> C.CDLL:
    """The loaded library.  Raises if it has not been built (python -m muse_spark_open_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise MskError(f"{LIB_PATH} is missing: build it with `python -m muse_spark_open_b200.build`")
        _lib = C.CDLL(LIB_PATH)
        _lib.msk_version.restype = C.c_int
        for name in EXPORTS:
            getattr(_lib, name).restype = C.c_int
        vp, ci = C.c_void_p, C.c_int
        # explicit argument types: a bare Python int would be passed as a 32-bit C int and truncate pointers
        _lib.msk_device_info.argtypes = [vp, vp]
        _lib.msk_selftest_umma.argtypes = [ci, vp, vp, vp, ci, vp, vp]
        _lib.msk_proj_skinny.argtypes = [vp, vp, vp]
        _lib.msk_proj_scratch_bytes.argtypes = [ci, ci, ci, ci, ci, vp]
        _lib.msk_attn_decode.argtypes = [vp, vp, vp]
        _lib.msk_moe_packed_bytes.argtypes = [ci, ci, ci, vp, vp]
        _lib.msk_moe_pack.argtypes = [vp, vp, vp, vp]
        _lib.msk_moe_dequant.argtypes = [vp, vp, ci, ci, ci, ci, vp]
        _lib.msk_moe_scratch_bytes.argtypes = [ci, ci, ci, ci, ci, ci, vp, vp, vp, vp, vp]
        _lib.msk_moe_forward.argtypes = [vp, vp, vp]
        _lib.msk_moe_forward_static.argtypes = [vp, vp, vp]
        _lib.msk_layer_front.argtypes = [vp, vp, vp]
        _lib.msk_layer_decode.argtypes = [vp, vp, vp]
        _lib.msk_router.argtypes = [vp, vp, vp]
        _lib.msk_residual_boundary.argtypes = [vp, vp]
        _lib.msk_rmsnorm.argtypes = [vp, vp, vp, vp, ci, ci, C.c_float, ci, vp]
        _lib.msk_ep_row_bytes.argtypes = [ci, ci]
        _lib.msk_ep_region_bytes.argtypes = [ci, ci, ci, ci, vp]
        _lib.msk_ep_region_alloc.argtypes = [C.c_size_t, vp, vp]
        _lib.msk_ep_region_open.argtypes = [vp, vp]
        _lib.msk_ep_region_close.argtypes = [vp]
        _lib.msk_ep_region_free.argtypes = [vp]
        _lib.msk_ep_step.argtypes = [vp, vp, vp]
        _lib.msk_selftest_flag_timeout.argtypes = [vp, C.c_longlong, vp, vp]
        _lib.msk_ep_pack.argtypes = [vp, vp, vp, vp, ci, vp, ci, ci, ci, vp]
        _lib.msk_ep_reduce.argtypes = [vp, vp, ci, vp, vp, ci, ci, vp]
    return _lib


# every symbol include/msk.h declares
EXPORTS = ["msk_version", "msk_device_info", "msk_selftest_umma", "msk_proj_skinny", "msk_proj_scratch_bytes", "msk_attn_decode",
           "msk_moe_packed_bytes", "msk_moe_pack", "msk_moe_dequant", "msk_moe_scratch_bytes", "msk_moe_forward", "msk_moe_forward_static", "msk_layer_front", "msk_layer_decode", "msk_router", "msk_residual_boundary", "msk_rmsnorm",
           "msk_ep_row_bytes", "msk_ep_pack", "msk_ep_reduce", "msk_ep_region_bytes", "msk_ep_region_alloc", "msk_ep_region_open",
           "msk_ep_region_close", "msk_ep_region_free", "msk_ep_step", "msk_selftest_flag_timeout"]


def ptr(t: torch.Tensor | None) -> int | None:
    if t is None:
        return None
    if not t.is_cuda:
        raise MskError("the CUDA path needs CUDA tensors; there is no CPU fallback")
    return t.data_ptr()


def stream_ptr() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise MskError(f"{what}: {RETURN_CODES.get(rc, rc)}")


class Status:
    """The device int32[4] status word kernels report into."""

    def __init__(self, device):
        self.t = torch.zeros(4, dtype=torch.int32, device=device)

    @property
    def p(self) -> C.c_void_p:
        return C.c_void_p(self.t.data_ptr())

    def raise_if_set(self, what: str = "") -> None:
        """Host read (synchronises): call outside timed regions."""
        s = self.t.tolist()
        if s[0] != 0:
            self.t.zero_()
            kern = KERNEL_NAMES.get(s[1] >> 8, s[1] >> 8)
            raise MskError(f"{what} device status: {STATUS_CODES.get(s[0], s[0])} in {kern} site {s[1] & 255} "
                           f"detail {s[2]} {s[3]}")


_status: dict = {}


def status_for(device) -> Status:
    key = torch.device(device).index or 0
    if key not in _status:
        _status[key] = Status(device)
    return _status[key]


class AttnParams(C.Structure):
    _fields_ = [
        ("qkv", C.c_void_p), ("ld_qkv", C.c_int), ("out", C.c_void_p), ("ld_out", C.c_int),
        ("k_cache", C.c_void_p), ("v_cache", C.c_void_p), ("k_scale", C.c_void_p), ("v_scale", C.c_void_p),
        ("seq_lens", C.c_void_p), ("page_table", C.c_void_p), ("max_pages", C.c_int),
        ("cache_loc", C.c_void_p), ("inv_freq", C.c_void_p),
        ("B", C.c_int), ("L", C.c_int), ("Hq", C.c_int), ("Hkv", C.c_int), ("d", C.c_int), ("page_size", C.c_int),
        ("num_pages", C.c_int), ("window", C.c_int),
        ("qk_scale_factor", C.c_float), ("sm_scale", C.c_float),
        ("chunks", C.c_int), ("stages", C.c_int), ("issuers", C.c_int), ("pdl", C.c_int), ("row_groups", C.c_int),
    ]


class MoeWeights(C.Structure):
    _fields_ = [("w13", C.c_void_p), ("w13_sf", C.c_void_p), ("w2", C.c_void_p), ("w2_sf", C.c_void_p),
                ("E", C.c_int), ("H", C.c_int), ("I", C.c_int)]


class MoeParams(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("ldx", C.c_int),
        ("x_ssq", C.c_void_p), ("x_ssq_parts", C.c_int), ("x_inv_dim", C.c_float), ("x_eps", C.c_float),
        ("topk_ids", C.c_void_p), ("topk_weights", C.c_void_p), ("ld_topk", C.c_int), ("logits", C.c_void_p),
        ("n_logits", C.c_int),
        ("ld_logits", C.c_int), ("x_ssq_tstride", C.c_int),
        ("T", C.c_int), ("top_k", C.c_int), ("local_start", C.c_int), ("local_count", C.c_int),
        ("w13_packed", C.c_void_p), ("w2_packed", C.c_void_p), ("w13_gs", C.c_void_p), ("w2_gs", C.c_void_p),
        ("post_norm_w", C.c_void_p), ("post_eps", C.c_float), ("H", C.c_int), ("I", C.c_int),
        ("h1_part", C.c_void_p), ("y_part", C.c_void_p), ("inter_sorted", C.c_void_p), ("x_sorted", C.c_void_p),
        ("route_pub", C.c_void_p), ("s1", C.c_int), ("s2", C.c_int),
        ("resid", C.c_void_p), ("ldr", C.c_int), ("out", C.c_void_p), ("out_fp32", C.c_int), ("ldo", C.c_int),
        ("out_copy", C.c_void_p), ("ldc", C.c_int), ("pdl", C.c_int), ("x_fp16", C.c_int),
        ("ep", C.c_void_p),
    ]


class LayerFront(C.Structure):
    _fields_ = [
        ("B", C.c_int), ("L", C.c_int), ("H", C.c_int), ("Hq", C.c_int), ("Hkv", C.c_int), ("d", C.c_int),
        ("page_size", C.c_int), ("num_pages", C.c_int), ("max_pages", C.c_int), ("window", C.c_int),
        ("qk_scale_factor", C.c_float), ("sm_scale", C.c_float), ("norm_eps", C.c_float),
        ("stream", C.c_void_p),
        ("k_cache", C.c_void_p), ("v_cache", C.c_void_p), ("k_scale", C.c_void_p), ("v_scale", C.c_void_p),
        ("seq_lens", C.c_void_p), ("page_table", C.c_void_p), ("cache_loc", C.c_void_p), ("inv_freq", C.c_void_p),
        ("input_norm_w", C.c_void_p), ("w_qkv", C.c_void_p), ("w_o", C.c_void_p), ("pre_expert_norm_w", C.c_void_p),
        ("router_w", C.c_void_p), ("router_bias", C.c_void_p), ("E", C.c_int),
        ("xn0", C.c_void_p), ("ssq0", C.c_void_p), ("qkv", C.c_void_p), ("attn", C.c_void_p), ("stream1", C.c_void_p),
        ("xn1", C.c_void_p), ("ssq1", C.c_void_p), ("router_part", C.c_void_p), ("router_ticket", C.c_void_p),
        ("qkv_scratch", C.c_void_p), ("o_scratch", C.c_void_p), ("qkv_scratch_bytes", C.c_size_t), ("o_scratch_bytes", C.c_size_t),
        ("logits", C.c_void_p), ("top_k", C.c_int), ("topk_ids", C.c_void_p), ("topk_weights", C.c_void_p),
        ("attn_chunks", C.c_int), ("attn_stages", C.c_int), ("attn_issuers", C.c_int), ("qkv_splits", C.c_int),
        ("o_splits", C.c_int), ("attn_row_groups", C.c_int),
        ("pdl", C.c_int),
    ]


class LayerParams(C.Structure):
    _fields_ = [("front", LayerFront), ("moe", MoeParams)]


class RouterParams(C.Structure):
    _fields_ = [("x", C.c_void_p), ("norm_w", C.c_void_p), ("ssq", C.c_void_p), ("ssq_parts", C.c_int), ("eps", C.c_float),
                ("router_w", C.c_void_p), ("router_bias", C.c_void_p), ("E", C.c_int), ("T", C.c_int), ("H", C.c_int),
                ("top_k", C.c_int), ("sigmoid_bias", C.c_int), ("multiplier", C.c_float), ("part", C.c_void_p),
                ("ticket", C.c_void_p), ("logits", C.c_void_p), ("topk_ids", C.c_void_p), ("topk_weights", C.c_void_p),
                ("pdl", C.c_int)]


class BoundaryParams(C.Structure):
    _fields_ = [("stream", C.c_void_p), ("branch", C.c_void_p), ("branch_bf16", C.c_int), ("ldb", C.c_int),
                ("branch_w", C.c_void_p), ("gate", C.c_void_p), ("next_norm_w", C.c_void_p), ("stream_out", C.c_void_p),
                ("normed_out", C.c_void_p), ("ssq_out", C.c_void_p), ("T", C.c_int), ("H", C.c_int),
                ("branch_eps", C.c_float), ("eps", C.c_float), ("temperature", C.c_float), ("gate_eps", C.c_float),
                ("pdl", C.c_int)]


class EpComm(C.Structure):
    _fields_ = [("rank", C.c_int), ("world", C.c_int), ("T_local", C.c_int), ("n_experts", C.c_int), ("step", C.c_int),
                ("self", C.c_void_p), ("peers", C.c_void_p), ("counters", C.c_void_p), ("wait_cycles", C.c_longlong)]


class EpStep(C.Structure):
    _fields_ = [("front", LayerFront), ("moe", MoeParams), ("comm", EpComm), ("out", C.c_void_p), ("hidden", C.c_void_p)]
