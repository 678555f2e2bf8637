"""Host <-> device streaming around a device-side callable.

`HostPipeline` overlaps the three legs of a host-resident workload -- pinned host
inputs -> device, the quantized layers, result -> pinned host memory -- on three
CUDA streams with double-buffered device staging, so that a sequence of calls
runs at the pace of its slowest leg instead of the sum of all three.  Each call
still performs its own copies; nothing is cached between calls.
"""

from __future__ import annotations

import torch


class HostPipeline:
    def __init__(self, fn, example_inputs, example_output, device=None, depth: int = 2):
        """`fn(*device_inputs) -> device tensor`; the examples fix shapes / dtypes of the
        staging buffers (`depth` sets of them)."""
        self.fn = fn
        self.device = torch.device(device) if device is not None else torch.device(
            "cuda", torch.cuda.current_device())
        self.depth = depth
        self.s_in = torch.cuda.Stream(self.device)
        self.s_run = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)
        self.bufs_in = [[torch.empty(t.shape, dtype=t.dtype, device=self.device) for t in example_inputs]
                        for _ in range(depth)]
        self.bufs_out = [torch.empty(example_output.shape, dtype=example_output.dtype, device=self.device)
                         for _ in range(depth)]
        self.ev_in = [torch.cuda.Event() for _ in range(depth)]      # inputs landed
        self.ev_run = [torch.cuda.Event() for _ in range(depth)]     # compute done (inputs free)
        self.ev_out = [torch.cuda.Event() for _ in range(depth)]     # result copied out
        self.count = 0

    def submit(self, host_inputs, host_output) -> None:
        """Enqueue one call: copy `host_inputs` (pinned) in, run, copy the result into
        `host_output` (pinned).  Returns without waiting."""
        slot = self.count % self.depth
        first_use = self.count < self.depth
        with torch.cuda.stream(self.s_in):
            if not first_use:
                self.s_in.wait_event(self.ev_run[slot])  # the previous user of this slot has read it
            for dst, src in zip(self.bufs_in[slot], host_inputs):
                dst.copy_(src, non_blocking=True)
            self.ev_in[slot].record(self.s_in)
        with torch.cuda.stream(self.s_run):
            self.s_run.wait_event(self.ev_in[slot])
            if not first_use:
                self.s_run.wait_event(self.ev_out[slot])  # the slot's result buffer has been drained
            y = self.fn(*self.bufs_in[slot])
            self.bufs_out[slot].copy_(y)
            self.ev_run[slot].record(self.s_run)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.ev_run[slot])
            host_output.copy_(self.bufs_out[slot], non_blocking=True)
            self.ev_out[slot].record(self.s_out)
        self.count += 1

    def drain(self) -> None:
        """Wait until every submitted call has delivered its result."""
        self.s_out.synchronize()
        self.s_run.synchronize()
        self.s_in.synchronize()
