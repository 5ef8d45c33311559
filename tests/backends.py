"""Where the test buffers live: CUDA tensors for the real library, numpy arrays for the
g++-compiled emulation build (tests/emu).  Both expose the same four calls so a parity case
is written once and runs through the same C ABI on either."""
from __future__ import annotations

import os
import sys

import numpy as np

from cerium_b200 import _capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class EmuBackend:
    """Kernel sources compiled for the host (index arithmetic / orchestration checks)."""

    name = "emu"

    def __init__(self):
        sys.path.insert(0, os.path.join(ROOT, "tests", "emu"))
        import build_emu
        self.lib = _capi.Library(build_emu.build())
        self._keep = []

    def to_dev(self, a: np.ndarray):
        b = np.ascontiguousarray(a).copy()
        assert b.ctypes.data % 16 == 0
        return b

    def empty(self, shape, dtype):
        b = np.zeros(shape, dtype=dtype)
        assert b.ctypes.data % 16 == 0
        return b

    def ptr(self, buf) -> int:
        return buf.ctypes.data

    def to_host(self, buf) -> np.ndarray:
        return buf.copy()

    def sync(self):
        pass


class CudaBackend:
    """The shipped CUDA library on cuda:0."""

    name = "cuda"

    def __init__(self):
        import torch
        self.torch = torch
        if not torch.cuda.is_available():
            raise RuntimeError("CUDA backend requested without a GPU")
        self.lib = _capi.load()
        self.dev = torch.device("cuda:0")

    def _tdtype(self, dtype):
        return {np.dtype(np.uint64): self.torch.int64, np.dtype(np.uint32): self.torch.int32}[np.dtype(dtype)]

    def to_dev(self, a: np.ndarray):
        a = np.ascontiguousarray(a)
        signed = a.view(np.int64 if a.dtype == np.uint64 else np.int32)
        return self.torch.from_numpy(signed.copy()).to(self.dev)

    def empty(self, shape, dtype):
        return self.torch.zeros(shape, dtype=self._tdtype(dtype), device=self.dev)

    def ptr(self, buf) -> int:
        return buf.data_ptr()

    def to_host(self, buf) -> np.ndarray:
        self.torch.cuda.synchronize()
        a = buf.cpu().numpy()
        return a.view(np.uint64 if a.dtype == np.int64 else np.uint32).copy()

    def sync(self):
        self.torch.cuda.synchronize()
