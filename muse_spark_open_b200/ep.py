"""Expert-parallel decode layer on G GPUs of one box: one process per GPU, torch.distributed (NCCL).

Partition (the benchmark's multi-GPU config): requests are data-parallel, rank g owns requests
[g*R/G, (g+1)*R/G) with their KV pages; the experts are expert-parallel, rank g holds experts
[g*E/G, (g+1)*E/G); dense weights and the router are replicated.  The reference has no collective (its
all-reduces are identities, muse_decode_layer/reference.py:8-10,467); here the exchange is real:

  front      (local tokens)   norms, QKV, attention, o_proj, residual, router (logits, softmax, top-8)
  dispatch   every local token's row (x fp16 | expert ids | weights | sum of squares) goes to every rank, fixed
             capacity T_local rows per peer: sizes are static, nothing depends on the routing, so the
             step never syncs with the host and every rank posts the same collectives in the same order.
             With dense fixed-capacity rows an all-to-all and an all-gather move the same bytes; NCCL's
             all-gather is used.
  experts    each rank runs the grouped GEMMs over all T tokens; the GEMM CTAs build their routing tables
             from the gathered expert ids and only pairs of local experts are touched; a token with no
             local expert yields a zero row.
  combine    all-to-all (NCCL): rank g sends rank h the FP32 partial rows of h's tokens.
  reduce     home rank adds the G partials to the residual in rank order (bitwise reproducible).

`step()` takes its compute stages as an `ops` object, so the same orchestration runs on CPU ranks
(gloo) in the tests with plain-PyTorch stages, and on GPUs with the CUDA kernels (`CudaOps`).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

TOP_K = 8


def shard(n: int, world: int, rank: int) -> tuple[int, int]:
    """(first, count) of an even split of n items; n must divide by world."""
    if n % world:
        raise ValueError(f"{n} items do not split evenly over {world} ranks")
    return rank * (n // world), n // world


def row_bytes(hidden: int, top_k: int = TOP_K) -> int:
    """Bytes of one dispatched token row: x fp16 [H] | ids int32 [k] | weights fp32 [k] | pad to 16 |
    sum of squares fp32 + padding."""
    return 2 * hidden + ((8 * top_k + 15) & ~15) + 16


def row_views(rows: torch.Tensor, hidden: int, top_k: int = TOP_K):
    """Strided views (x fp16 [T, H], ids int32 [T, k], weights fp32 [T, k], ssq fp32 [T]) into a uint8
    [T, row_bytes] buffer."""
    t = rows.shape[0]
    rb = rows.shape[1]
    x = rows.view(torch.float16).view(t, rb // 2)[:, :hidden]
    f = rows.view(torch.float32).view(t, rb // 4)
    i = rows.view(torch.int32).view(t, rb // 4)
    return x, i[:, hidden // 2: hidden // 2 + top_k], f[:, hidden // 2 + top_k: hidden // 2 + 2 * top_k], f[:, rb // 4 - 4]


def step(data: dict, ops, group=None):
    """One expert-parallel decode step for this rank's requests.  Returns (hidden bf16 [T_local, H],
    stream fp32 [T_local, H], topk_ids int32 [T_local, 8])."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    rows, stream1 = ops.front(data)                      # uint8 [T_local, row_bytes], fp32 [T_local, H]
    t_local = rows.shape[0]
    if world > 1:
        gathered = ops.buffer("gathered", (world * t_local, rows.shape[1]), torch.uint8)
        dist.all_gather_into_tensor(gathered, rows, group=group)
    else:
        gathered = rows
    partial, ids = ops.experts(gathered)                 # fp32 [world*T_local, H], int32 [world*T_local, 8]
    if world > 1:
        recv = ops.buffer("recv", tuple(partial.shape), torch.float32)
        dist.all_to_all_single(recv, partial, group=group)
    else:
        recv = partial
    hidden, stream = ops.reduce(stream1, recv.view(world, t_local, -1))
    return hidden, stream, ids[rank * t_local:(rank + 1) * t_local]


class CudaOps:
    """The CUDA stages of `step` for one rank (kernels through the C ABI; raises without a GPU)."""

    def __init__(self, weights: dict, rank: int, world: int, n_experts: int, **tune):
        from . import layer
        first, count = shard(n_experts, world, rank)
        if weights["w13"].shape[0] != count:
            raise ValueError("weights must hold exactly this rank's experts")
        self.state = layer.prepare(weights, local_start=first, local_count=count)
        self.rank, self.world, self.n_experts, self.tune = rank, world, n_experts, tune
        self.bufs: dict = {}

    exchange = "nccl all-gather (dispatch) + all-to-all (combine)"

    def launches_per_step(self, tokens_local: int) -> int:
        """This repo's kernels per step and rank (NCCL's own are not counted): the five up to the router, the row
        pack, the experts over all ranks' tokens (gather, two GEMMs, combine) and the reduce."""
        return 5 + 1 + 4 + 1

    def buffer(self, name, shape, dtype):
        key = (name, shape, dtype)
        if key not in self.bufs:
            self.bufs[key] = torch.empty(shape, dtype=dtype, device="cuda")
        return self.bufs[key]

    def front(self, data):
        import ctypes as C

        from . import abi, layer
        buf = layer.front(data, self.state, **self.tune)
        t, h = data["stream"].shape
        rows = self.buffer("rows", (t, row_bytes(h)), torch.uint8)
        abi.check(abi.lib().msk_ep_pack(abi.ptr(buf["xn1"]), abi.ptr(buf["topk_ids"]), abi.ptr(buf["topk_weights"]),
                                        abi.ptr(buf["ssq1"][-1]), 1, abi.ptr(rows), t, h, TOP_K, abi.stream_ptr()),
                  "msk_ep_pack")
        del C
        return rows, buf["stream1"]

    def experts(self, gathered):
        from . import layer, moe
        t = gathered.shape[0]
        ms = self.state["moe"]
        h = ms["H"]
        key = ("views", gathered.data_ptr(), t)
        if key not in self.bufs:  # the gathered buffer is persistent: its strided views are built once
            self.bufs[key] = row_views(gathered, h)
        x, ids, wts, ssq = self.bufs[key]
        out = self.buffer("partial", (t, h), torch.float32)
        moe.forward(x, ids, wts, ms, self.state["local_start"], self.state["local_count"], out=out,
                    pre_norm=(ssq, h, layer.RMS_EPS), splits=self.tune.get("moe_splits"), pdl=True)
        return out, ids

    def reduce(self, stream1, recv):
        from . import abi
        t, h = stream1.shape
        out = torch.empty((t, h), dtype=torch.float32, device=stream1.device)
        hidden = torch.empty((t, h), dtype=torch.bfloat16, device=stream1.device)
        abi.check(abi.lib().msk_ep_reduce(abi.ptr(stream1), abi.ptr(recv), recv.shape[0], abi.ptr(out), abi.ptr(hidden),
                                          t, h, abi.stream_ptr()), "msk_ep_reduce")
        return hidden, out
