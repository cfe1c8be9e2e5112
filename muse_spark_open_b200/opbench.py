"""Per-op micro-benchmarks at the benchmark's shapes (the counterpart of the reference's per-problem
bench.py files, e.g. muse_moe_w4a16/bench.py): cold-L2 device time, achieved GB/s over algorithmic bytes.

    python -m muse_spark_open_b200.opbench proj  [--m 16 --n 6144 --k 4096 --splits 0]
    python -m muse_spark_open_b200.opbench attn  [--batch 16 --ctx 1024:8192 --window 1024 --q-len 1]
    python -m muse_spark_open_b200.opbench moe   [--tokens 32]
    python -m muse_spark_open_b200.opbench layer [--batch 32 --ctx 8192 --q-len 1]

`--eager N` replaces the graph timing by N plain launches (what a profiler capture of a single launch wants).
One JSON line per run.
"""
from __future__ import annotations

import argparse
import json

import torch

from . import abi, attention, layer, moe, proj, synth, timing

DEV = "cuda"


def _time(fn, args):
    if args.eager:
        for _ in range(args.eager):
            fn()
        torch.cuda.synchronize()
        return None
    return timing.graph_time_us(fn, reps=args.reps)


def _emit(name, us, byt, **extra):
    out = {"op": name, "algorithmic_mb": round(byt / 1e6, 2), **extra}
    if us is not None:
        out.update(us=round(us, 2), gbs=round(byt / us / 1e3, 1), frac_of_8tbs=round(byt / us / 1e3 / 8000, 3))
    print(json.dumps(out), flush=True)


def run_proj(a):
    g = torch.Generator(device=DEV).manual_seed(0)
    x = torch.randn((a.m, a.k), generator=g, device=DEV).to(torch.bfloat16)
    w = (0.02 * torch.randn((a.n, a.k), generator=g, device=DEV)).to(torch.bfloat16)
    out = torch.empty((a.m, a.n), dtype=torch.bfloat16, device=DEV)
    us = _time(lambda: proj.skinny(x, w, out=out, splits=a.splits), a)
    _emit("proj_skinny", us, a.n * a.k * 2 + a.m * a.k * 2 + a.m * a.n * 2, m=a.m, n=a.n, k=a.k, splits=a.splits)


def _seqs(a, batch):
    if ":" in a.ctx:
        lo, hi = (int(v) for v in a.ctx.split(":"))
        g = torch.Generator().manual_seed(1)
        return torch.randint(lo, hi + 1, (batch,), generator=g).tolist()
    return [int(a.ctx)] * batch


def run_attn(a):
    seqs = _seqs(a, a.batch)
    data = synth.make_layer_input(0, DEV, seqs, q_len=a.q_len, window=a.window, rope_theta=1e6 if a.window else 0.0)
    cfg = data["config"]
    t = a.batch * a.q_len
    g = torch.Generator(device=DEV).manual_seed(2)
    qkv = torch.randn((t, 9216), generator=g, device=DEV).to(torch.bfloat16)
    out = torch.empty((t, 4096), dtype=torch.bfloat16, device=DEV)
    us = _time(lambda: attention.launch(qkv, out, data, cfg, chunks=a.chunks, stages=a.stages, issuers=a.issuers,
                                         row_groups=a.row_groups), a)
    keys = sum(min(s, a.window - 1) if a.window else s for s in seqs)
    _emit("attn_decode", us, keys * 4 * 128 * 2 + t * (9216 + 4096) * 2, batch=a.batch, q_len=a.q_len, window=a.window,
          ctx=a.ctx, chunks=a.chunks, stages=a.stages, issuers=a.issuers)


def run_moe(a):
    w = synth.make_layer_weights(0, DEV)
    state = moe.prepare(w)
    g = torch.Generator(device=DEV).manual_seed(3)
    x = torch.randn((a.tokens, 4096), generator=g, device=DEV).to(torch.bfloat16)
    logits = torch.randn((a.tokens, 128), generator=g, device=DEV)
    # the expert choice as the router kernel leaves it (the experts take ids and weights as inputs, like the
    # reference's op); --logits moves softmax / top-8 into the GEMM CTAs instead
    pk, ids = torch.softmax(logits, -1).topk(8, -1)
    ids, wts = ids.to(torch.int32).contiguous(), (pk / pk.sum(-1, keepdim=True)).contiguous()
    out = torch.empty((a.tokens, 4096), dtype=torch.bfloat16, device=DEV)
    sp = (a.s1, a.s2) if a.s1 else None
    fn = lambda: moe.forward(x, ids, wts, state, 0, 128, out=out, logits=logits if a.logits else None, splits=sp)  # noqa: E731
    fn()
    torch.cuda.synchronize()
    touched = int(torch.unique(ids).numel())
    per = sum(w[k][0].numel() * w[k][0].element_size() for k in ("w13", "w13_sf", "w2", "w2_sf"))
    us = _time(fn, a)
    _emit("moe_forward (gather + gemm1 + act + gemm2 + combine)", us, touched * per + 2 * a.tokens * 4096 * 2, tokens=a.tokens, touched=touched,
          splits=sp)


def run_layer(a):
    w = synth.make_layer_weights(0, DEV)
    state = layer.prepare(w)
    data = synth.make_layer_input(0, DEV, _seqs(a, a.batch), q_len=a.q_len, window=a.window,
                                  rope_theta=1e6 if a.window else 0.0)
    _, _, ids = layer.kernel_fn(data, state)
    torch.cuda.synchronize()
    us = _time(lambda: layer.kernel_fn(data, state), a)
    _emit("layer_decode", us, synth.layer_bytes(w, data, int(torch.unique(ids).numel())), batch=a.batch, q_len=a.q_len, ctx=a.ctx)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("op", choices=["proj", "attn", "moe", "layer"])
    ap.add_argument("--m", type=int, default=16)
    ap.add_argument("--n", type=int, default=6144)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--ctx", default="1024:8192")
    ap.add_argument("--window", type=int, default=1024)
    ap.add_argument("--q-len", type=int, default=1)
    ap.add_argument("--chunks", type=int, default=0)
    ap.add_argument("--stages", type=int, default=0)
    ap.add_argument("--issuers", type=int, default=0)
    ap.add_argument("--row-groups", type=int, default=0)
    ap.add_argument("--tokens", type=int, default=32)
    ap.add_argument("--logits", action="store_true")
    ap.add_argument("--s1", type=int, default=0)
    ap.add_argument("--s2", type=int, default=0)
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--eager", type=int, default=0)
    a = ap.parse_args()
    {"proj": run_proj, "attn": run_attn, "moe": run_moe, "layer": run_layer}[a.op](a)
    abi.status_for(DEV).raise_if_set(a.op)


if __name__ == "__main__":
    main()
