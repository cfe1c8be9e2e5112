"""Expert-parallel orchestration on CPU ranks (gloo, world size 2): the same `ep.step` the GPUs run,
with plain-PyTorch stages built from the oracle, must reproduce the unsharded oracle layer."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HID, HQ, HKV, D, NEXP, INNER = 256, 8, 1, 32, 8, 64


class OracleOps:
    """CPU stand-ins for the three compute stages, in the layout `ep.step` moves between ranks."""

    def __init__(self, weights, rank, world):
        from muse_spark_open_b200 import ep
        self.w, self.rank, self.world, self.ep = weights, rank, world, ep
        self.first, self.count = ep.shard(NEXP, world, rank)

    def buffer(self, name, shape, dtype):
        return torch.empty(shape, dtype=dtype)

    def front(self, data):
        from oracle import layer as olayer
        fr = olayer.front(data, self.w)
        s1 = fr["stream1"]
        t = s1.shape[0]
        from oracle import moe as omoe
        rows = torch.zeros((t, self.ep.row_bytes(HID)), dtype=torch.uint8)
        x, ids, wts, ssq = self.ep.row_views(rows, HID)
        # the row carries the already normalised expert input and a sum of squares that makes the
        # receiver's row scale exactly 1, so this stand-in rounds to BF16 where the oracle does
        x.copy_(fr["h"].to(torch.bfloat16))
        top_ids, top_w = omoe.route_softmax(fr["logits"])
        ids.copy_(top_ids)
        wts.copy_(top_w)
        ssq.fill_(HID * (1.0 - 1e-5))
        return rows, s1

    def experts(self, gathered):
        from oracle import moe as omoe
        x, ids, wts, ssq = self.ep.row_views(gathered, HID)
        ids, wts = ids.contiguous(), wts.contiguous()
        h = (x.float() * torch.rsqrt(ssq.double() / HID + 1e-5).float()[:, None]).to(torch.bfloat16)
        md = {"hidden_states": h, "topk_ids": ids, "topk_weights": wts,
              "config": {"local_start": self.first, "local_count": self.count}}
        mw = dict(self.w)
        mw["post_norm_w"] = self.w["post_expert_norm"]
        return omoe.ref_kernel(md, mw, fp32_out=True).contiguous(), ids

    def reduce(self, stream1, recv):
        out = stream1.clone()
        for r in range(recv.shape[0]):
            out += recv[r]
        return out.to(torch.bfloat16), out


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from muse_spark_open_b200 import ep
    from oracle import layer as olayer
    torch.set_num_threads(2)
    weights = olayer.make_weights(5, hidden=HID, hq=HQ, hkv=HKV, d=D, n_experts=NEXP, inner=INNER, bias_std=0.5)
    seqs = [40, 17, 70, 9]
    full = olayer.make_input(len(seqs), seqs, 9, hidden=HID, hq=HQ, hkv=HKV, d=D, page=16, window=0, rope_theta=0.0)
    first, count = ep.shard(len(seqs), world, rank)
    sl = slice(first, first + count)
    mine = dict(full)
    for k in ("seq_lens", "page_table", "stream", "cache_loc", "positions", "cache_seqlens"):
        mine[k] = full[k][sl]
    mine["config"] = dict(full["config"], batch=count, tokens=count)
    hidden, stream, ids = ep.step(mine, OracleOps(weights, rank, world))
    ref_hidden, ref_stream, ref_ids, _, _ = olayer.ref_kernel(full, weights)
    ok = (torch.allclose(stream, ref_stream[sl], rtol=1e-4, atol=1e-4) and torch.equal(ids, ref_ids[sl])
          and hidden.shape == (count, HID))
    ret[rank] = bool(ok)
    dist.barrier()
    dist.destroy_process_group()


def test_ep_step_two_cpu_ranks_matches_unsharded_oracle():
    world = 2
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_worker, args=(world, 29517, ret), nprocs=world, join=True)
        assert dict(ret) == {0: True, 1: True}


def test_shard_and_row_layout():
    from muse_spark_open_b200 import ep
    assert ep.shard(128, 8, 3) == (48, 16)
    assert ep.row_bytes(4096) == 8192 + 64 + 16 and ep.row_bytes(4096, 3) == 8192 + 32 + 16
    rows = torch.zeros((3, ep.row_bytes(64)), dtype=torch.uint8)
    x, ids, wts, ssq = ep.row_views(rows, 64)
    x.fill_(1.0), ids.fill_(7), wts.fill_(2.0), ssq.fill_(3.0)
    assert x.shape == (3, 64) and ids.shape == (3, 8) and wts.shape == (3, 8) and ssq.shape == (3,)
    raw = rows.view(torch.float32).view(3, -1)
    assert (rows.view(torch.int32).view(3, -1)[:, 32:40] == 7).all() and (raw[:, 40:48] == 2.0).all()
    assert (raw[:, 48] == 3.0).all() and (raw[:, 49:] == 0).all()


def test_peer_exchange_index_math():
    """Who sends a token a partial row, and where a rank writes inside a peer's region (the index math of the
    device-initiated exchange, restated in ep.py for the tests)."""
    from muse_spark_open_b200 import ep
    ids = torch.tensor([[0, 1, 2, 3, 4, 5, 6, 7], [0, 16, 32, 48, 64, 80, 96, 112], [127, 126, 125, 124, 123, 122, 121, 120]])
    own = ep.owner_ranks(ids, 128, 8)
    assert own[0].tolist() == [True] + [False] * 7 and own[1].all() and own[2].tolist() == [False] * 7 + [True]
    own2 = ep.owner_ranks(ids, 128, 2)
    assert own2.tolist() == [[True, False], [True, True], [False, True]]
    seen = set()
    for r in range(4):
        sl = ep.region_slots(4, r, 8)
        rows = range(sl["dispatch_first_row"], sl["dispatch_first_row"] + 8)
        assert not seen & set(rows) and max(rows) < sl["rows"]
        seen |= set(rows)
    assert seen == set(range(32))  # the ranks' rows tile a region's row buffer exactly
