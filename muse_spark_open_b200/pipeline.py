"""Decode steps whose inputs and results live in pinned host memory, with the copies under the kernels.

A step needs its per-step inputs (residual stream, sequence lengths, cache rows, page table) on the device and gives
its results (hidden states, expert ids) back to the host.  Run on one stream, the copies and the kernels queue up
behind one another: at 256 requests the 4.5 MB in and 2.1 MB out cost a fifth of the step.  `StepPipeline` puts
them on two copy streams with two staging sets each:

    copy-in stream    H2D(i+1) ........
    compute stream    [stage -> data] step(i) [results -> stage]   [stage -> data] step(i+1) ...
    copy-out stream                                       D2H(i) ........

The device-to-device moves between the staging sets and the tensors the kernels use are a few microseconds; the
step function and its argument blocks (which are keyed on tensor addresses) stay as they are.  Every wait is a
stream-to-event dependency; the host never blocks inside `submit`.
"""
from __future__ import annotations

import torch


class StepPipeline:
    """step_fn() -> tuple of device tensors, reading `data[k]` for k in `in_keys`.

    submit(host_in, host_out): host_in maps each key to a pinned host tensor shaped like data[k]; host_out is a
    tuple of pinned host tensors (or None to skip a result) shaped like step_fn's results.  The copy of a result is
    complete after `drain()`, or once a later `submit` reuses its staging set (two submits on)."""

    DEPTH = 2

    def __init__(self, step_fn, data: dict, in_keys, n_results: int):
        dev = data[in_keys[0]].device
        if dev.type != "cuda":
            raise RuntimeError("StepPipeline needs CUDA tensors (there is no CPU path)")
        self.step_fn, self.data, self.in_keys, self.n_results = step_fn, data, tuple(in_keys), n_results
        self.dev = dev
        self.s_in, self.s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        self.stage_in = [{k: torch.empty_like(data[k]) for k in self.in_keys} for _ in range(self.DEPTH)]
        self.stage_out = [None] * self.DEPTH  # allocated from the first results
        ev = lambda: torch.cuda.Event()  # noqa: E731
        self.ev_h2d = [ev() for _ in range(self.DEPTH)]       # staging set filled from the host
        self.ev_in_free = [ev() for _ in range(self.DEPTH)]   # staging set moved into `data`
        self.ev_done = [ev() for _ in range(self.DEPTH)]      # results moved into their staging set
        self.ev_out_free = [ev() for _ in range(self.DEPTH)]  # staging set copied to the host
        self.count = 0

    def submit(self, host_in: dict, host_out):
        i, slot = self.count, self.count % self.DEPTH
        self.count += 1
        cur = torch.cuda.current_stream(self.dev)
        # host -> staging, on the copy-in stream, as soon as the set's previous contents have been moved on
        if i >= self.DEPTH:
            self.s_in.wait_event(self.ev_in_free[slot])
        else:
            self.s_in.wait_stream(cur)  # whatever produced the host buffers' device twins is ordered before
        with torch.cuda.stream(self.s_in):
            for k in self.in_keys:
                self.stage_in[slot][k].copy_(host_in[k], non_blocking=True)
            self.ev_h2d[slot].record(self.s_in)
        # staging -> the tensors the kernels read; the step; results -> staging
        cur.wait_event(self.ev_h2d[slot])
        for k in self.in_keys:
            self.data[k].copy_(self.stage_in[slot][k], non_blocking=True)
        self.ev_in_free[slot].record(cur)
        res = self.step_fn()
        if self.stage_out[slot] is None:
            self.stage_out[slot] = [torch.empty_like(r) for r in res[:self.n_results]]
        if i >= self.DEPTH:
            cur.wait_event(self.ev_out_free[slot])
        for dst, r in zip(self.stage_out[slot], res):
            dst.copy_(r, non_blocking=True)
        self.ev_done[slot].record(cur)
        # staging -> host, on the copy-out stream
        self.s_out.wait_event(self.ev_done[slot])
        with torch.cuda.stream(self.s_out):
            for dst, src in zip(host_out, self.stage_out[slot]):
                if dst is not None:
                    dst.copy_(src, non_blocking=True)
            self.ev_out_free[slot].record(self.s_out)

    def drain(self):
        """Order the current stream after every copy issued so far (a following event or synchronize then covers
        them)."""
        cur = torch.cuda.current_stream(self.dev)
        cur.wait_stream(self.s_in)
        cur.wait_stream(self.s_out)
