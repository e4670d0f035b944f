"""Host-resident batches through a module with the copies overlapped.

The reference has no counterpart: it is called with device tensors (or runs on the CPU).  A caller
whose activations live in host memory pays two PCIe transfers per call that are each several times
longer than the layer itself; the three steps of consecutive calls — host→device copy, forward,
device→host copy — are independent of each other, so they run on three streams over a small ring
of device buffers and the steady-state cost of a call is the longest of the three.

    pipe = HostPipeline(module, x_host.shape, x_host.dtype, device)
    for x_host, y_host in batches:        # pinned host tensors
        pipe.submit(x_host, y_host)       # returns at once
    pipe.drain()                          # all y_host written
"""

from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch


class HostPipeline:
    def __init__(self, fn: Callable[[torch.Tensor], torch.Tensor], shape: Sequence[int], dtype: torch.dtype,
                 device: torch.device, depth: int = 2):
        if depth < 1:
            raise ValueError("depth must be at least 1")
        self.fn, self.device, self.depth = fn, torch.device(device), depth
        if self.device.type != "cuda":
            raise ValueError("HostPipeline needs a CUDA device")
        self.copy_in = torch.cuda.Stream(self.device)
        self.compute = torch.cuda.Stream(self.device)
        self.copy_out = torch.cuda.Stream(self.device)
        self.x_dev = [torch.empty(tuple(shape), dtype=dtype, device=self.device) for _ in range(depth)]
        self.y_dev: List[Optional[torch.Tensor]] = [None] * depth
        mk = lambda: [torch.cuda.Event() for _ in range(depth)]  # noqa: E731
        self.in_done, self.fwd_done, self.out_done = mk(), mk(), mk()
        self.n = 0
        self.follow()

    def submit(self, x_host: torch.Tensor, y_host: torch.Tensor) -> None:
        """Enqueue one batch; ``x_host`` must stay unchanged and ``y_host`` unread until :meth:`drain`
        (or until ``depth`` further batches have been submitted)."""
        if not (x_host.is_pinned() and y_host.is_pinned()):
            raise ValueError("HostPipeline needs pinned host tensors (the copies would synchronise otherwise)")
        s = self.n % self.depth
        reused = self.n >= self.depth
        with torch.cuda.stream(self.copy_in):
            if reused:
                self.copy_in.wait_event(self.fwd_done[s])  # the forward that read this buffer
            self.x_dev[s].copy_(x_host, non_blocking=True)
            self.in_done[s].record(self.copy_in)
        with torch.cuda.stream(self.compute):
            self.compute.wait_event(self.in_done[s])
            if reused:
                self.compute.wait_event(self.out_done[s])  # the copy that read this slot's previous output
            y = self.fn(self.x_dev[s])
            self.fwd_done[s].record(self.compute)
        y.record_stream(self.copy_out)
        self.y_dev[s] = y
        with torch.cuda.stream(self.copy_out):
            self.copy_out.wait_event(self.fwd_done[s])
            y_host.copy_(y, non_blocking=True)
            self.out_done[s].record(self.copy_out)
        self.n += 1

    def follow(self, stream: Optional[torch.cuda.Stream] = None) -> None:
        """Make everything submitted from now on wait for the work already on ``stream`` (default: current)."""
        stream = stream or torch.cuda.current_stream(self.device)
        for s in (self.copy_in, self.compute, self.copy_out):
            s.wait_stream(stream)

    def join(self, stream: Optional[torch.cuda.Stream] = None) -> None:
        """Make ``stream`` (default: the current one) wait for everything submitted so far."""
        stream = stream or torch.cuda.current_stream(self.device)
        for s in (self.copy_in, self.compute, self.copy_out):
            stream.wait_stream(s)

    def drain(self) -> None:
        self.copy_out.synchronize()
        self.compute.synchronize()
        self.copy_in.synchronize()
