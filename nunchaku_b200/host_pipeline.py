"""Host-resident batches through a device module: copy in, compute and copy out on three CUDA streams.

A caller whose activations live in pinned host memory pays for two PCIe transfers per batch.  Issued on
one stream they run one after the other (copy in, kernels, copy out); here each has its own stream and the
device tensors are double-buffered, so batch i+1 is copied in and batch i-1 copied out while batch i is
computed, and the steady-state cost per batch is the longest of the three instead of their sum.
"""
from __future__ import annotations

import torch


class HostPipeline:
    def __init__(self, module, in_shape, out_shape, dtype=torch.bfloat16, device=None, depth: int = 2):
        self.module = module
        self.device = torch.device(device if device is not None else torch.cuda.current_device())
        self.depth = depth
        self.x = [torch.empty(in_shape, dtype=dtype, device=self.device) for _ in range(depth)]
        self.y = [torch.empty(out_shape, dtype=dtype, device=self.device) for _ in range(depth)]
        self.s_in = torch.cuda.Stream(self.device)
        self.s_run = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)
        self.loaded = [torch.cuda.Event() for _ in range(depth)]     # x[i] holds a fresh batch
        self.computed = [torch.cuda.Event() for _ in range(depth)]   # y[i] holds its result, x[i] is free again
        self.drained = [torch.cuda.Event() for _ in range(depth)]    # y[i] has been copied out
        self.n = 0

    def submit(self, x_host: torch.Tensor, out_host: torch.Tensor) -> None:
        """Queue one batch: x_host (pinned) -> device -> module -> out_host (pinned).  Returns at once."""
        i = self.n % self.depth
        first = self.n < self.depth
        with torch.cuda.stream(self.s_in):
            if not first:
                self.s_in.wait_event(self.computed[i])      # the previous user of x[i] has been consumed
            self.x[i].copy_(x_host, non_blocking=True)
            self.loaded[i].record(self.s_in)
        with torch.cuda.stream(self.s_run):
            self.s_run.wait_event(self.loaded[i])
            if not first:
                self.s_run.wait_event(self.drained[i])      # the previous result in y[i] has left
            self.module(self.x[i], self.y[i])
            self.computed[i].record(self.s_run)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.computed[i])
            out_host.copy_(self.y[i], non_blocking=True)
            self.drained[i].record(self.s_out)
        self.n += 1

    def join(self, stream: torch.cuda.Stream | None = None) -> None:
        """Make `stream` (default: the current one) wait for everything submitted so far."""
        stream = stream or torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_run, self.s_out):
            e = torch.cuda.Event()
            e.record(s)
            stream.wait_event(e)

    def fork(self, stream: torch.cuda.Stream | None = None) -> None:
        """Make the three streams wait for what `stream` (default: the current one) has queued so far."""
        stream = stream or torch.cuda.current_stream(self.device)
        e = torch.cuda.Event()
        e.record(stream)
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_event(e)
