"""A caller-provided transport for the library's limb collectives over HOST memory: the collectives of a
torch.distributed (gloo) process group applied to raw addresses.  TEST INFRASTRUCTURE: it lets the
multi-rank host logic of the library run on CPU ranks through the emulation build, where "device"
pointers are host pointers."""
import ctypes

import numpy as np
import torch
import torch.distributed as dist


def _view(addr: int, count: int, dtype):
    n = count * np.dtype(dtype).itemsize
    buf = (ctypes.c_char * n).from_address(addr)
    return torch.from_numpy(np.frombuffer(buf, dtype=dtype))


class GlooHostTransport:
    def __init__(self, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.calls = {"allgather": 0, "reducescatter": 0, "allreduce": 0, "broadcast": 0}

    def allgather(self, recv, send, bytes_per_rank, stream):
        self.calls["allgather"] += 1
        s = _view(send, bytes_per_rank, np.uint8).clone()          # send may be a block of recv
        dist.all_gather_into_tensor(_view(recv, bytes_per_rank * self.world, np.uint8), s, group=self.group)

    def reducescatter(self, recv, send, words, word_bits, stream):
        self.calls["reducescatter"] += 1
        dt = np.int64 if word_bits == 64 else np.int32             # wrapping sums: the bit patterns agree
        s = _view(send, words * self.world, dt).clone()
        dist.all_reduce(s, op=dist.ReduceOp.SUM, group=self.group)
        _view(recv, words, dt).copy_(s[self.rank * words:(self.rank + 1) * words])

    def allreduce(self, recv, send, words, word_bits, stream):
        self.calls["allreduce"] += 1
        dt = np.int64 if word_bits == 64 else np.int32
        s = _view(send, words, dt).clone()
        dist.all_reduce(s, op=dist.ReduceOp.SUM, group=self.group)
        _view(recv, words, dt).copy_(s)

    def broadcast(self, buf, nbytes, root, stream):
        self.calls["broadcast"] += 1
        dist.broadcast(_view(buf, nbytes, np.uint8), src=root, group=self.group)
