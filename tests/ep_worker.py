"""Worker of tests/test_gpu_ep.py, run under torch.distributed.run: the expert-parallel step on this rank's
requests and experts must match the single-GPU layer run on the whole batch (same GPU, same seeds)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from muse_spark_open_b200 import abi, ep, layer, synth  # noqa: E402

HID, HQ, HKV, D, NEXP, INNER = 1024, 8, 1, 128, 16, 128


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
    full_w = synth.make_layer_weights(3, dev, hidden=HID, hq=HQ, hkv=HKV, d=D, n_experts=NEXP, inner=INNER, bias_std=0.5)
    seqs = [300, 70, 129, 1000, 64, 5, 2047, 512]
    full = synth.make_layer_input(4, dev, seqs, hidden=HID, hq=HQ, hkv=HKV, d=D)
    ref_state = layer.prepare(full_w)
    ref_in = dict(full, k_cache=full["k_cache"].clone(), v_cache=full["v_cache"].clone())
    ref_hidden, ref_stream, ref_ids = layer.kernel_fn(ref_in, ref_state)
    e0, ec = ep.shard(NEXP, world, rank)
    r0, rc = ep.shard(len(seqs), world, rank)
    mine_w = dict(full_w)
    for k in ("w13", "w13_sf", "w13_gs", "w2", "w2_sf", "w2_gs"):
        mine_w[k] = full_w[k][e0:e0 + ec].contiguous()
    mine = dict(full)
    for k in ("seq_lens", "page_table", "stream", "cache_loc", "positions"):
        mine[k] = full[k][r0:r0 + rc].contiguous()
    mine["config"] = dict(full["config"], batch=rc, tokens=rc)
    ok = True
    for exchange in ("peer", "nccl"):  # device-initiated stores into peers' memory, then the collective-library form
        ops = ep.CudaOps(mine_w, rank, world, NEXP, exchange=exchange)
        for _ in range(3):  # both buffer parities, and a buffer's reuse
            hidden, stream, ids = ep.step(mine, ops)
        torch.cuda.synchronize()
        abi.status_for(dev).raise_if_set("ep " + exchange)
        ok = ok and torch.equal(ids, ref_ids[r0:r0 + rc])
        ok = ok and torch.allclose(stream, ref_stream[r0:r0 + rc], rtol=1e-4, atol=1e-4)
        ok = ok and torch.allclose(hidden.float(), ref_hidden[r0:r0 + rc].float(), rtol=2e-2, atol=1e-2)
        if ops.peer is not None:
            dist.barrier()
            ops.peer.close()
    flag = torch.tensor([int(ok)], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("EP_OK" if int(flag) == 1 else "EP_MISMATCH", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if int(flag) == 1 else 1)


if __name__ == "__main__":
    main()
