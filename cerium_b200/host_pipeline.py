"""Host-buffer pipeline around a device operation.

A caller whose ciphertexts live in host memory (the reference's runtime uploads program inputs
and downloads results around every run: cerium/runtime/execution/program.cpp) pays one PCIe
transfer in and one out per operation.  `HostPipeline` overlaps the three legs -- upload of
operation i+1, evaluation of operation i, download of operation i-1 -- on three CUDA streams
over a ring of device buffers, so a stream of operations runs at the pace of the slowest leg
instead of the sum.  torch is used for the buffers, streams and events only.
"""
from __future__ import annotations

from typing import Callable, List, Sequence


class HostPipeline:
    """op(dev_ins, dev_outs, stream_handle) is enqueued on the pipeline's compute stream; dev_ins /
    dev_outs are lists of device tensors shaped like in_shapes / out_shapes (dtype int64)."""

    def __init__(self, torch, in_shapes: Sequence[Sequence[int]], out_shapes: Sequence[Sequence[int]],
                 op: Callable, depth: int = 3, dtype=None):
        self.torch = torch
        self.op = op
        self.depth = depth
        dtype = dtype or torch.int64
        dev = torch.device("cuda", torch.cuda.current_device())
        self.dev_in = [[torch.empty(tuple(s), dtype=dtype, device=dev) for s in in_shapes] for _ in range(depth)]
        self.dev_out = [[torch.empty(tuple(s), dtype=dtype, device=dev) for s in out_shapes] for _ in range(depth)]
        self.host_out = [[torch.empty(tuple(s), dtype=dtype).pin_memory() for s in out_shapes] for _ in range(depth)]
        self.s_in, self.s_op, self.s_out = (torch.cuda.Stream(device=dev) for _ in range(3))
        ev = lambda: [torch.cuda.Event() for _ in range(depth)]  # noqa: E731
        self.ev_in, self.ev_op, self.ev_out = ev(), ev(), ev()
        self.count = 0
        self.in_bytes = sum(t.numel() * t.element_size() for t in self.dev_in[0])
        self.out_bytes = sum(t.numel() * t.element_size() for t in self.dev_out[0])

    def submit(self, host_ins: List) -> int:
        """Queues one operation on pinned host inputs; returns the slot whose host_out will hold the
        result once `wait(slot)` (or `drain()`) has returned."""
        torch = self.torch
        slot = self.count % self.depth
        first_use = self.count < self.depth
        self.count += 1
        self.last_host_ins = host_ins
        with torch.cuda.stream(self.s_in):
            if not first_use:
                self.s_in.wait_event(self.ev_op[slot])   # the slot's previous inputs have been consumed
            for d, h in zip(self.dev_in[slot], host_ins):
                d.copy_(h, non_blocking=True)
            self.ev_in[slot].record(self.s_in)
        with torch.cuda.stream(self.s_op):
            self.s_op.wait_event(self.ev_in[slot])
            if not first_use:
                self.s_op.wait_event(self.ev_out[slot])  # the slot's previous result has left the device
            self.op(self.dev_in[slot], self.dev_out[slot], self.s_op.cuda_stream)
            self.ev_op[slot].record(self.s_op)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.ev_op[slot])
            for h, d in zip(self.host_out[slot], self.dev_out[slot]):
                h.copy_(d, non_blocking=True)
            self.ev_out[slot].record(self.s_out)
        return slot

    def wait(self, slot: int) -> List:
        self.ev_out[slot].synchronize()
        return self.host_out[slot]

    def drain(self) -> None:
        for s in (self.s_in, self.s_op, self.s_out):
            s.synchronize()
