"""Device timing of one op from a cold L2, after the reference's method (muse_bf16_proj/timing.py:11-67):
capture a CUDA graph of REPS x (flush L2; op) and one of REPS x (flush L2), replay both several
times with CUDA events on the launching stream, report (median_op - median_flush) / REPS.
The flush READS a buffer twice the size of the device's L2 (a write would leave dirty lines whose
write-back is then charged to the op that evicts them)."""
from __future__ import annotations

import statistics

import torch

_flush = {}


def flush_buffer(device=None) -> torch.Tensor:
    dev = torch.device("cuda" if device is None else device)
    key = dev.index or 0
    if key not in _flush:
        l2 = torch.cuda.get_device_properties(dev).L2_cache_size
        _flush[key] = torch.zeros(max(2 * l2, 128 << 20) // 4, dtype=torch.int32, device=dev)
    return _flush[key]


def flush_l2(buf: torch.Tensor) -> None:
    """Evict L2 by streaming `buf` through it (read-only; the 4-byte result is discarded)."""
    torch.sum(buf, dtype=torch.int32)


def graph_time_us(fn, reps: int = 10, replays: int = 7, rounds: int = 3, cold: bool = True) -> float:
    """Median device time of fn() in microseconds (cold L2 when cold=True)."""
    buf = flush_buffer()
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for _ in range(3):
            fn()
        stream.synchronize()
        g_op, g_fl = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_op, stream=stream):
            for _ in range(reps):
                if cold:
                    flush_l2(buf)
                fn()
        with torch.cuda.graph(g_fl, stream=stream):
            for _ in range(reps):
                if cold:
                    flush_l2(buf)

        def once(g):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            g.replay()
            b.record(stream)
            b.synchronize()
            return a.elapsed_time(b) * 1e3
        ops, fls = [], []
        for _ in range(rounds):
            for _ in range(replays):
                ops.append(once(g_op))
                fls.append(once(g_fl))
    torch.cuda.current_stream().wait_stream(stream)
    return (statistics.median(ops) - statistics.median(fls)) / reps
