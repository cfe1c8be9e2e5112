"""Generate the golden fixtures in this folder by running the reference's own Python on CPU.

Usage (only where the reference checkout is present; the fixtures are committed):
    python tests/golden/make_golden.py /path/to/reference

Each problem folder of the reference has its own `reference.py` / `checks.py` / `nvfp4.py`; they are
imported under unique names with that folder first on sys.path.  The reference hard-codes its
shapes as module constants, which its functions read at call time, so the constants are
re-assigned before calling to get small cases and the benchmark's head_dim 128; the code that
runs is still the reference's.  FP8 tensors are stored as their uint8 bytes.
"""
from __future__ import annotations

import importlib.util
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load(ref_root: str, folder: str):
    path = os.path.join(ref_root, folder)
    for name in ("checks", "nvfp4", "reference"):
        sys.modules.pop(name, None)
    sys.path.insert(0, path)
    try:
        spec = importlib.util.spec_from_file_location(f"ref_{folder}", os.path.join(path, "reference.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        nv = sys.modules.get("nvfp4")
    finally:
        sys.path.remove(path)
    return mod, nv


def as_bytes(t):
    return t.view(torch.uint8) if t.dtype == torch.float8_e4m3fn else t


def pack(d):
    return {k: (as_bytes(v) if isinstance(v, torch.Tensor) else v) for k, v in d.items() if v is not None}


def attention_cases(ref):
    cases = []
    # (name, head_dim, heads, window, theta, generate_input kwargs)
    specs = [
        ("native_d64_sliding_decode", 64, (16, 2), 96, 500_000.0,
         dict(batch=2, ctx=150, heads="x", layer="sliding", seed=11, q_len=1, page=16)),
        ("d128_sliding_verify_edges", 128, (16, 2), 64, 1e6,
         dict(batch=2, ctx=100, heads="x", layer="sliding", seed=12, q_len=8, page=16, dist="edges",
              kv_scale=1 / 64)),
        ("d128_full_decode_mixed", 128, (16, 2), 64, 1e6,
         dict(batch=3, ctx=60, heads="x", layer="full", seed=13, q_len=1, page=16, spread="mixed")),
        ("d128_short_ctx_verify", 128, (8, 1), 64, 1e6,
         dict(batch=2, ctx=10, heads="x", layer="sliding", seed=14, q_len=8, page=16)),
    ]
    for name, d, heads, window, theta, kw in specs:
        ref.HEAD_DIM = d
        ref.SM_SCALE = d ** -0.5
        ref.HEADS["x"] = heads
        ref.SLIDING_WINDOW = window
        ref.ROPE_THETA = theta
        data = ref.generate_input(device="cpu", **kw)
        out, k_new, v_new = ref.ref_kernel(data)
        item = pack(data)
        item["expect_out"] = out
        item["expect_k_new"] = as_bytes(k_new)
        item["expect_v_new"] = as_bytes(v_new)
        cases.append((name, item))
    return cases


def moe_cases(ref, nv):
    ref.D_HIDDEN, ref.D_EXPERT, ref.N_EXPERTS, ref.ROUTED_PER_TOKEN = 256, 128, 16, 4
    ref.LOCAL = {"ep8": (0, 4), "full": (0, 16)}
    weights = ref.generate_weights(21, device="cpu")
    cases = []
    for name, kw in (("full_normal", dict(bs=6, sharding="full", seed=22)),
                     ("ep_skewed", dict(bs=9, sharding="ep8", seed=23, dist="skewed"))):
        data = ref.generate_input(device="cpu", **kw)
        out = ref.ref_kernel(data, weights)
        cases.append((name, {"data": pack(data), "expect_out": out}))
    cases.append(("weights", pack(weights)))
    # codec: quantise values that include exact rounding midpoints, then dequantise
    gen = torch.Generator().manual_seed(24)
    x = torch.randn((8, 64), generator=gen)
    x[0, :16] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -2.5, -5.0, 7.0, -9.0, 0.0, 6.0])
    packed, sf, gs = nv.quantize(x)
    codec = {"x": x, "packed": packed, "sf": as_bytes(sf), "gs": gs, "dequant": nv.dequantize(packed, sf, gs),
             "unpacked": nv.unpack_e2m1(packed)}
    cases.append(("codec", codec))
    return cases


def proj_cases(ref):
    ref.LAYERS = {"qkv_gate": (96, 256), "o": (128, 64), "router": (16, 256)}
    ref.FP32_LAYERS = {"router"}
    weights = ref.generate_weights(31, device="cpu")
    cases = []
    for layer, m, seed, dist in (("qkv_gate", 8, 32, "normal"), ("o", 16, 33, "outliers"), ("router", 5, 34, "normal")):
        data = ref.generate_input(m=m, layer=layer, seed=seed, dist=dist, device="cpu")
        cases.append((f"{layer}_m{m}", {"x": data["x"], "w": weights[layer], "config": data["config"],
                                       "expect_out": ref.ref_kernel(data, weights)}))
    return cases


def layer_cases(ref):
    """The reference's own layer functions (ref_front / ref_back behind ref_kernel) at small shapes, head_dim 128."""
    ref.HIDDEN, ref.HEAD_DIM, ref.HQ, ref.HKV = 1024, 128, 8, 1
    ref.Q_SIZE, ref.KV_SIZE = ref.HQ * ref.HEAD_DIM, ref.HKV * ref.HEAD_DIM
    ref.QKV_SIZE = 2 * ref.Q_SIZE + 2 * ref.KV_SIZE
    ref.SM_SCALE = ref.HEAD_DIM ** -0.5
    ref.SLIDING_WINDOW, ref.ROPE_THETA = 48, 1e6
    ref.D_EXPERT, ref.N_EXPERTS, ref.LOCAL_EXPERTS = 256, 16, 8
    ref.UNPOOL_SLICE = ref.HIDDEN // 8
    ref._stream_basis.cache_clear()
    weights = ref.generate_weights(41, device="cpu")
    cases = [("weights", pack(weights))]
    for name, kw in (("full_decode", dict(batch=3, ctx=70, layer="full", seed=42, q_len=1, page=16, local_start=8)),
                     ("sliding_verify", dict(batch=2, ctx=90, layer="sliding", seed=43, q_len=8, page=16, spread="agentic"))):
        data = ref.generate_input(device="cpu", **kw)
        front = ref.ref_front(data, weights)
        hidden, stream, ids, k_new, v_new = ref.ref_kernel(data, weights)
        item = pack(data)
        item.update(expect_hidden=hidden, expect_stream=stream, expect_ids=ids, expect_stream1=front["stream1"],
                    expect_scores=front["scores"], expect_k_new=as_bytes(k_new), expect_v_new=as_bytes(v_new))
        cases.append((name, item))
    return cases


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <checkout of Kushagrabainsla/muse-spark-open>")
    ref_root = sys.argv[1]
    out = {}
    att, _ = load(ref_root, "muse_attention_decode")
    out["attention"] = dict(attention_cases(att))
    m, nv = load(ref_root, "muse_moe_w4a16")
    out["moe"] = dict(moe_cases(m, nv))
    p, _ = load(ref_root, "muse_bf16_proj")
    out["proj"] = dict(proj_cases(p))
    lay, _ = load(ref_root, "muse_decode_layer")
    out["layer"] = dict(layer_cases(lay))
    for name, blob in out.items():
        path = os.path.join(HERE, f"{name}.pt")
        torch.save(blob, path)
        print(name, list(blob), os.path.getsize(path) // 1024, "KB")


if __name__ == "__main__":
    main()
