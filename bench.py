"""Benchmark of the decoder layer's decode step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload (the same at every N, so that the per-N values compare): the benchmark's expert-parallel
config: 256 concurrent requests, context uniform in [2048, 16384], full attention, hidden 4096, 32/4
heads of 128, page 64, 128 NVFP4 experts (top-8, router logits + per-expert bias N(0, 0.5)).  At N GPUs
requests and experts are split evenly (strong scaling); at N = 1 one GPU holds everything.  A step is
one decode step of the layer for all 256 requests; value = tokens / s over all ranks.
One JSON line on stdout (rank 0).  Extra keys at N = 1: `layer_us_per_step` (the single-GPU layer at
batch 1 / 16 / 32, context 8192, cold L2), `kernels`, `roofline`, `cpu_baseline`.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

REQUESTS, CTX_LO, CTX_HI = 256, 2048, 16384
HIDDEN, HQ, HKV, HEAD, PAGE, NEXP, INNER = 4096, 32, 4, 128, 64, 128, 768
BIAS_STD = 0.5
SEED = 0
METRIC, UNIT = "decoder_layer_decode_tokens_per_s", "tokens/s"


def workload_name(n):
    return (f"expert-parallel decoder layer decode step: {REQUESTS} requests, ctx U[{CTX_LO},{CTX_HI}], full attention, "
            f"hidden {HIDDEN}, {HQ}/{HKV} heads x {HEAD}, page {PAGE}, {NEXP} NVFP4 experts top-8 "
            f"(gate_up [1536,4096], down [4096,768]), requests and experts split over {n} GPU(s)")


def seq_lens_all():
    g = torch.Generator().manual_seed(SEED + 11)
    return torch.randint(CTX_LO, CTX_HI + 1, (REQUESTS,), generator=g)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return float(p["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 200 ms while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.p = subprocess.Popen(["nvidia-smi", "-i", str(index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                       "-lms", "200"], stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None

    def stop(self):
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.p.terminate()
        self.p.wait()
        self.f.flush()
        rows = [r.split(",") for r in open(self.f.name).read().strip().splitlines() if r.strip()]
        os.unlink(self.f.name)
        sm = [float(r[0]) for r in rows if r[0].strip().replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in rows for i in range(4) if len(r) >= 6 and "Active" in r[2 + i] and "Not" not in r[2 + i]})
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": float(rows[0][1]) if rows else None, "reasons": reasons, "samples": len(rows)}


def event_time_ms(fn, steps, stream=None):
    """Device time of `steps` calls of fn() between two CUDA events on the launching stream."""
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for _ in range(steps):
        fn()
    b.record()
    b.synchronize()
    return a.elapsed_time(b)


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))


def cpu_sample(weights_cpu, n_req, threads):
    """The oracle's layer (plain PyTorch restatement of the reference math) on host cores, for the first
    n_req requests of the workload.  Returns seconds for one step of those requests."""
    from oracle import layer as olayer
    torch.set_num_threads(threads)
    seqs = seq_lens_all()[:n_req].tolist()
    data = olayer.make_input(n_req, seqs, SEED + 1, hidden=HIDDEN, hq=HQ, hkv=HKV, d=HEAD, page=PAGE, window=0,
                             rope_theta=0.0)
    reps = 8  # one step of n_req requests is under a second on a many-core host: repeat it
    t0 = time.perf_counter()
    for _ in range(reps):
        olayer.ref_kernel(data, weights_cpu)
    return (time.perf_counter() - t0) / reps


def run_reference(args):
    """Reference arm: the reference's PyTorch math (oracle port) on the host cores, bounded sample per step."""
    rank, world, _ = dist_env()
    if rank != 0:
        return
    from oracle import layer as olayer
    threads = os.cpu_count() or 1
    n_req = 64
    weights = olayer.make_weights(SEED, hidden=HIDDEN, hq=HQ, hkv=HKV, d=HEAD, n_experts=NEXP, inner=INNER, bias_std=BIAS_STD)
    times = [cpu_sample(weights, n_req, threads) for _ in range(args.warmup + args.steps)][args.warmup:]
    sec = sum(times) / len(times)
    val = n_req / sec
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic", "config": {"workload": workload_name(args.gpus)},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"8 layer steps for the first {n_req} of the {REQUESTS} requests per timed step"},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def single_gpu_extras(weights, dev):
    """Single-GPU layer at batch 1 / 16 / 32 (context 8192, full attention) from a cold L2, and the
    four main kernels of the 256-request step timed on their own."""
    from muse_spark_open_b200 import layer, synth, timing
    state = layer.prepare(weights)
    out = {}
    for b in (1, 16, 32):
        data = synth.make_layer_input(SEED + 100 + b, dev, [8192] * b)
        _, _, ids = layer.kernel_fn(data, state)
        torch.cuda.synchronize()
        us = timing.graph_time_us(lambda: layer.kernel_fn(data, state), reps=5)
        byt = synth.layer_bytes(weights, data, int(torch.unique(ids).numel()))
        out[f"batch{b}"] = {"us_per_step": round(us, 1), "algorithmic_mb": round(byt / 1e6, 1), "hbm_gbs": round(byt / us / 1e3, 1),
                            "frac_of_8tbs": round(byt / us / 1e3 / 8000, 3)}
        del data
    return out, state


# dram__bytes_read.sum + dram__bytes_write.sum over algorithmic bytes, from the captures summarised under profiles/
# (attention 32 requests x 8192; experts 32 tokens; projection 16 x 6144 x 4096)
NCU_TRAFFIC_RATIO = {"attn_decode": 1.014, "moe": 1.019, "proj_skinny": 0.997}


def run_ours(args):
    from muse_spark_open_b200 import abi, ep, layer, synth, timing
    rank, world, local_rank = dist_env()
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device (there is no CPU fallback); use --impl reference for the CPU arm")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    e_first, e_count = ep.shard(NEXP, world, rank)
    r_first, r_count = ep.shard(REQUESTS, world, rank)
    weights = synth.make_layer_weights(SEED, dev, hidden=HIDDEN, hq=HQ, hkv=HKV, d=HEAD, n_experts=NEXP, inner=INNER,
                                       bias_std=BIAS_STD, expert_range=(e_first, e_count))
    seqs = seq_lens_all()[r_first:r_first + r_count].tolist()
    data = synth.make_layer_input(SEED + 1 + rank, dev, seqs, max_len=CTX_HI)
    if world == 1:
        state = layer.prepare(weights)
        step = lambda: layer.kernel_fn(data, state)  # noqa: E731
        # prep_norm, qkv projection, attention, o projection, router, [gather when > 32 tokens], gemm 1, activation,
        # gemm 2, combine
        launches = 9 + (r_count > 32)
    else:
        ops = ep.CudaOps(weights, rank, world, NEXP)
        step = lambda: ep.step(data, ops)  # noqa: E731
        # the five kernels up to the router, the row pack, the experts over all ranks' tokens (4 or 5), the reduce;
        # NCCL's own kernels (all-gather, all-to-all) are not counted
        launches = 5 + 1 + 4 + (REQUESTS > 32) + 1
    for _ in range(max(args.warmup, 3)):
        out = step()
    torch.cuda.synchronize()
    abi.status_for(dev).raise_if_set("bench warm-up")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    # ---- device-resident timing
    barrier()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    ms = event_time_ms(step, args.steps)
    barrier()
    ms = max_over_ranks(ms)
    # ---- end to end: this step's inputs come from pinned host memory, its results go back
    host = {k: data[k].cpu().pin_memory() for k in ("stream", "seq_lens", "cache_loc", "page_table")}
    hid_h = torch.empty((r_count, HIDDEN), dtype=torch.bfloat16).pin_memory()
    ids_h = torch.empty((r_count, 8), dtype=torch.int32).pin_memory()

    def e2e_step():
        for k, v in host.items():
            data[k].copy_(v, non_blocking=True)
        hidden, _, ids = step()
        hid_h.copy_(hidden, non_blocking=True)
        ids_h.copy_(ids, non_blocking=True)

    e2e_step()
    barrier()
    ms_e2e = event_time_ms(e2e_step, args.steps)
    barrier()
    ms_e2e = max_over_ranks(ms_e2e)
    clocks = sampler.stop() if sampler else None
    abi.status_for(dev).raise_if_set("bench")
    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    peak, peak_src = peaks()
    h2d = sum(v.numel() * v.element_size() for v in host.values())
    d2h = hid_h.numel() * 2 + ids_h.numel() * 4
    line = {
        "metric": METRIC, "value": REQUESTS * args.steps / (ms / 1e3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": workload_name(world), "l2": "inputs larger than L2 (KV cache 2.4 GB, experts 0.68 GB per step)",
                   "parallelism": f"dp{world} attention x ep{world} experts"},
        "e2e": {"value": REQUESTS * args.steps / (ms_e2e / 1e3), "unit": UNIT, "h2d_bytes_per_step": h2d * world,
                "d2h_bytes_per_step": d2h * world},
        "gpu_launches": launches * args.steps, "clocks": clocks,
    }
    if world == 1 and not args.skip_extras:
        hidden, stream_out, ids = out
        touched = int(torch.unique(ids).numel())
        buf = state["bufs"][r_count]
        ms_state = state["moe"]
        cfg = data["config"]
        from muse_spark_open_b200 import attention, moe, proj
        mo = torch.empty((r_count, HIDDEN), dtype=torch.float32, device=dev)
        kv_bytes = sum(seqs) * HKV * HEAD * 2
        per_exp = sum(weights[k][0].numel() * weights[k][0].element_size() for k in ("w13", "w13_sf", "w2", "w2_sf"))
        kern = {
            "attn_decode": (lambda: attention.launch(buf["qkv"], buf["attn"], data, cfg), kv_bytes + r_count * 9216 * 2 + r_count * 4096 * 2),
            "moe (gather + gemm1 + act + gemm2 + combine)": (lambda: moe.forward(buf["xn1"], ids, buf["topk_weights"], ms_state, 0, NEXP, out=mo,
                                                                                 pre_norm=(buf["ssq1"][-1], HIDDEN, 1e-5)),
                                                             touched * per_exp + 2 * r_count * HIDDEN * 2),
            "proj_skinny qkv": (lambda: proj.skinny(buf["xn0"], state["qkv_gate"], out=buf["qkv"]), 9216 * 4096 * 2 + r_count * (4096 + 9216) * 2),
            "proj_skinny o": (lambda: proj.skinny(buf["attn"], state["o"], out=buf["stream1"], resid=data["stream"]), 4096 * 4096 * 2 + r_count * 4096 * 10),
        }
        kernels = {}
        for name, (fn, byt) in kern.items():
            us = timing.graph_time_us(fn, reps=3, replays=5, rounds=2)
            kernels[name] = {"us": round(us, 1), "algorithmic_mb": round(byt / 1e6, 1), "gbs": round(byt / us / 1e3, 1)}
        top = max(kernels, key=lambda k: kernels[k]["us"])
        line["kernels"] = kernels
        # DRAM traffic of one launch: the kernel's dram__bytes (read + write) from the ncu capture of a smaller case
        # (profiles/), which grows in proportion to the algorithmic bytes, scaled to this launch
        ratio = next((r for key, r in NCU_TRAFFIC_RATIO.items() if top.startswith(key)), None)
        line["roofline"] = {"bound": "hbm", "kernel": top, "achieved": kernels[top]["gbs"], "peak": peak, "unit": "GB/s",
                            "frac": round(kernels[top]["gbs"] / peak, 4), "peak_source": peak_src,
                            "traffic": round(kern[top][1] * ratio) if ratio else None,
                            "traffic_source": "ncu dram bytes / algorithmic bytes on the profiled case, times this launch's algorithmic bytes"}
        step_bytes = synth.layer_bytes(weights, data, touched)
        line["step_algorithmic_mb"] = round(step_bytes / 1e6, 1)
        line["step_hbm_gbs"] = round(step_bytes / (ms / args.steps) / 1e6, 1)
        del data, state
        torch.cuda.empty_cache()
        line["layer_us_per_step"], _ = single_gpu_extras(weights, dev)
        # CPU baseline: the oracle on the host cores, a bounded sample of the same workload
        w_cpu = {k: (v.cpu() if isinstance(v, torch.Tensor) else v) for k, v in weights.items()}
        threads = os.cpu_count() or 1
        n_req = 64
        sec = cpu_sample(w_cpu, n_req, threads)
        line["cpu_baseline"] = {"value": n_req / sec, "unit": UNIT, "cores": threads, "kind": "port",
                                "sample": f"8 layer steps for the first {n_req} of the {REQUESTS} requests ({8 * sec:.1f} s of CPU time)"}
    print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-extras", action="store_true",
                    help="only the timed step (no per-kernel, per-batch or CPU legs): what a profiler launch list wants")
    args = ap.parse_args()
    if args.impl == "reference":
        if args.steps > 5:
            args.steps = 5  # each step is seconds of CPU work
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
