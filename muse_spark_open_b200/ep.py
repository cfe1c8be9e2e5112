"""Expert-parallel decode layer on G GPUs of one box: one process per GPU, torch.distributed (NCCL).

Partition (the benchmark's multi-GPU config): requests are data-parallel, rank g owns requests
[g*R/G, (g+1)*R/G) with their KV pages; the experts are expert-parallel, rank g holds experts
[g*E/G, (g+1)*E/G); dense weights and the router are replicated.  The reference has no collective (its
all-reduces are identities, muse_decode_layer/reference.py:8-10,467); here the exchange is real:

  front      (local tokens)   norms, QKV, attention, o_proj, residual, router (logits, softmax, top-8)
  dispatch   every local token's row (x fp16 | expert ids | weights | sum of squares) goes to every rank, fixed
             capacity T_local rows per peer: sizes are static, nothing depends on the routing, so the
             step never syncs with the host.
  experts    each rank runs the grouped GEMMs over all T tokens; the GEMM CTAs build their routing tables
             from the gathered expert ids and only pairs of local experts are touched.
  combine    rank g gives rank h the FP32 partial rows of h's tokens.
  reduce     home rank adds the partials to the residual in rank order (bitwise reproducible).

Two exchanges.  "peer" (the default on GPUs): device-initiated, one C call per step (`msk_ep_step`): the
dispatch kernel stores the rows straight into every peer's memory over NVLink (regions mapped with CUDA IPC),
the experts' combine kernel stores each partial row into its token's home GPU, flags carrying the step number
tell the consumers (bounded waits), and only the ranks that hold one of a token's experts send it a row.
"nccl": the same kernels around an all-gather of the rows and an all-to-all of the partials, enqueued from
Python; kept as the collective-library form (and as the stand-in when peer mapping is unavailable).

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
    if hasattr(ops, "_peer_setup"):
        ops._peer_setup(data["stream"].shape[0], data["stream"].shape[1], data["stream"].device)
    if getattr(ops, "peer", None) is not None:
        return ops.fused_step(data)
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


def owner_ranks(ids: torch.Tensor, n_experts: int, world: int) -> torch.Tensor:
    """bool [T, world]: the ranks that hold at least one of a token's experts (the ranks that send it a partial row
    in the peer exchange, and the only ones whose rows the home rank adds)."""
    per = n_experts // world
    out = torch.zeros((ids.shape[0], world), dtype=torch.bool, device=ids.device)
    out.scatter_(1, (ids.long() // per).clamp(0, world - 1), True)
    return out


def region_slots(world: int, rank: int, t_local: int) -> dict:
    """Where rank `rank` writes in a peer's region, in rows: its dispatch rows are rows [rank * T_local, (rank + 1) *
    T_local) of the step's row buffer, its partial rows for the peer's token t are row rank * T_local + t of the
    step's partial buffer (the index math of csrc/ep_exchange.cu, restated for the tests)."""
    return {"dispatch_first_row": rank * t_local, "partial_first_row": rank * t_local, "rows": world * t_local}


class PeerRegions:
    """One region of device memory per rank, mapped by every peer (CUDA IPC), for the device-initiated exchange."""

    def __init__(self, world: int, rank: int, t_local: int, hidden: int, device, group=None):
        import ctypes as C

        from . import abi
        lib = abi.lib()
        self.world, self.rank, self.lib = world, rank, lib
        nbytes = C.c_size_t()
        abi.check(lib.msk_ep_region_bytes(world, t_local, hidden, TOP_K, C.byref(nbytes)), "msk_ep_region_bytes")
        self.nbytes = nbytes.value
        ptr, handle = C.c_void_p(), (C.c_ubyte * 64)()
        abi.check(lib.msk_ep_region_alloc(self.nbytes, C.byref(ptr), handle), "msk_ep_region_alloc")
        self.self_ptr = ptr.value
        self.opened: list = []
        ptrs = [0] * world
        ptrs[rank] = self.self_ptr
        if world > 1:
            mine = torch.tensor(list(handle), dtype=torch.uint8, device=device)
            every = torch.empty((world, 64), dtype=torch.uint8, device=device)
            dist.all_gather_into_tensor(every, mine, group=group)
            every = every.cpu()
            for r in range(world):
                if r == rank:
                    continue
                h = (C.c_ubyte * 64)(*every[r].tolist())
                p = C.c_void_p()
                abi.check(lib.msk_ep_region_open(h, C.byref(p)), f"msk_ep_region_open (rank {r}'s region)")
                self.opened.append(p.value)
                ptrs[r] = p.value
        self.peers = torch.tensor(ptrs, dtype=torch.int64, device=device)
        self.counters = torch.zeros(2, dtype=torch.int32, device=device)
        self.step = 0
        if world > 1:
            dist.barrier(group=group)

    def close(self):
        for p in self.opened:
            self.lib.msk_ep_region_close(p)
        self.opened = []
        if self.self_ptr:
            self.lib.msk_ep_region_free(self.self_ptr)
            self.self_ptr = 0


class CudaOps:
    """The CUDA stages of `step` for one rank (kernels through the C ABI; raises without a GPU).
    exchange: "peer" (device-initiated, one C call per step), "nccl", or "auto" = peer when the regions can be
    mapped, else nccl."""

    def __init__(self, weights: dict, rank: int, world: int, n_experts: int, exchange: str = "auto", group=None, **tune):
        from . import layer
        first, count = shard(n_experts, world, rank)
        if weights["w13"].shape[0] != count:
            raise ValueError("weights must hold exactly this rank's experts")
        self.state = layer.prepare(weights, local_start=first, local_count=count)
        self.rank, self.world, self.n_experts, self.tune, self.group = rank, world, n_experts, tune, group
        self.bufs: dict = {}
        self.want, self.peer, self.peer_error = exchange, None, None
        self.exchange = "nccl all-gather (dispatch) + all-to-all (combine)"

    def _peer_setup(self, t_local: int, hidden: int, device):
        """Map the regions on first use (the token count is known then).  Every rank must take the same branch:
        the outcome is agreed on with an all-reduce."""
        if self.want == "nccl" or self.peer is not None or self.peer_error is not None:
            return
        try:
            peer = PeerRegions(self.world, self.rank, t_local, hidden, device, self.group)
            ok = 1
        except Exception as exc:  # noqa: BLE001 - any failure of the mapping means "use the collective form"
            peer, ok, self.peer_error = None, 0, repr(exc)
        if self.world > 1:
            flag = torch.tensor([ok], device=device)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
            ok = int(flag)
        if ok:
            self.peer = peer
            self.exchange = "peer stores over NVLink with flags (device-initiated, one launch chain per step)"
        else:
            if peer is not None:
                peer.close()
            if self.want == "peer":
                raise RuntimeError(f"peer exchange unavailable: {self.peer_error}")
            self.peer_error = self.peer_error or "a peer could not map the regions"

    def launches_per_step(self, tokens_local: int) -> int:
        """This repo's kernels per step and rank: the five up to the router, the dispatch (row pack), the experts
        over all ranks' tokens (gather, two GEMMs, combine) and the reduce.  NCCL's own kernels (nccl exchange)
        are not counted."""
        return 5 + 1 + 4 + 1

    def fused_step(self, data):
        """One expert-parallel step through `msk_ep_step` (peer exchange).  The three results live in buffers of
        this object and are overwritten by the next step."""
        import ctypes as C

        from . import abi, layer, moe
        stream = data["stream"]
        t, h = stream.shape
        st = self.state
        buf = layer.buffers(st, t, stream.device)
        key = ("ep_step", tuple(data[k].data_ptr() for k in ("stream", "k_cache", "v_cache", "k_scale", "v_scale", "seq_lens",
                                                               "page_table", "cache_loc")), data["k_cache"].shape[0])
        cached = self.bufs.get("ep_step")
        if cached is None or cached[0] != key:
            ms = st["moe"]
            tt = self.world * t
            s1, s2 = self.tune.get("moe_splits") or moe.splits_for(tt, ms["H"], ms["I"], st["local_count"], TOP_K)
            h1, y, inter, xs, pub = moe.scratch(ms, tt, TOP_K, s1, s2, stream.device)
            p = abi.EpStep()
            layer.fill_front(p.front, data, st, buf, self.tune)
            m = p.moe
            m.w13_packed, m.w2_packed = abi.ptr(ms["w13"]), abi.ptr(ms["w2"])
            m.w13_gs, m.w2_gs = abi.ptr(ms["w13_gs"]), abi.ptr(ms["w2_gs"])
            m.post_norm_w, m.post_eps, m.I = abi.ptr(ms["post_w"]), moe.POST_NORM_EPS, ms["I"]
            m.h1_part, m.y_part, m.s1, m.s2 = abi.ptr(h1), abi.ptr(y), s1, s2
            m.inter_sorted, m.x_sorted, m.route_pub = abi.ptr(inter), abi.ptr(xs), abi.ptr(pub)
            c = p.comm
            c.rank, c.world, c.T_local, c.n_experts = self.rank, self.world, t, self.n_experts
            c.self, c.peers, c.counters = self.peer.self_ptr, abi.ptr(self.peer.peers), abi.ptr(self.peer.counters)
            c.wait_cycles = int(self.tune.get("wait_cycles", 0))
            out = torch.empty((t, h), dtype=torch.float32, device=stream.device)
            hidden = torch.empty((t, h), dtype=torch.bfloat16, device=stream.device)
            p.out, p.hidden = abi.ptr(out), abi.ptr(hidden)
            cached = (key, p, out, hidden, (h1, y, inter, xs, pub))
            self.bufs["ep_step"] = cached
        _, p, out, hidden, _ = cached
        self.peer.step += 1
        p.comm.step = self.peer.step
        abi.check(abi.lib().msk_ep_step(C.byref(p), abi.status_for(stream.device).p, abi.stream_ptr()), "msk_ep_step")
        return hidden, out, buf["topk_ids"]

    def buffer(self, name, shape, dtype):
        key = (name, shape, dtype)
        if key not in self.bufs:
            self.bufs[key] = torch.empty(shape, dtype=dtype, device="cuda")
        return self.bufs[key]

    def front(self, data):
        import ctypes as C

        from . import abi, layer
        buf = layer.front(data, self.state, **{k: v for k, v in self.tune.items() if k not in ("moe_splits", "wait_cycles")})
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
