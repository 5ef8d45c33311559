"""ctypes binding of oracle/_ref/libref_cuda.so: the reference's own CUDA device headers behind
thin wrappers (oracle/ref_cuda_harness.cu).  Test infrastructure: the 32-bit GPU oracle."""
from __future__ import annotations

import ctypes as C
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "oracle", "_ref", "libref_cuda.so")
_u32p = C.POINTER(C.c_uint32)


def available() -> bool:
    return os.path.exists(LIB)


class RefCuda:
    def __init__(self, primes):
        self.dll = C.CDLL(LIB)
        self.dll.refcuda_create.argtypes = [C.POINTER(C.c_void_p), _u32p, C.c_int]
        self.dll.refcuda_destroy.argtypes = [C.c_void_p]
        self.dll.refcuda_ntt.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, _u32p, C.c_int, C.c_int, C.c_int,
                                         C.POINTER(C.c_float)]
        self.dll.refcuda_sud.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, _u32p, C.c_int, _u32p,
                                         C.c_int, C.POINTER(C.c_float)]
        self.dll.refcuda_bconv.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, _u32p, C.c_int, _u32p, C.c_int,
                                           C.c_int, C.c_int, C.POINTER(C.c_float)]
        self.primes = [int(p) for p in primes]
        h = C.c_void_p()
        arr = (C.c_uint32 * len(primes))(*self.primes)
        rc = self.dll.refcuda_create(C.byref(h), arr, len(primes))
        assert rc == 0, "refcuda_create failed"
        self.h = h

    def __del__(self):
        if getattr(self, "h", None):
            self.dll.refcuda_destroy(self.h)
            self.h = None

    @staticmethod
    def _u32(v):
        return (C.c_uint32 * len(v))(*[int(x) for x in v])

    def ntt(self, out_ptr, in_ptr, bases, inverse=False, iters=1):
        ms = C.c_float(0)
        rc = self.dll.refcuda_ntt(self.h, out_ptr, in_ptr, self._u32(bases), len(bases), int(inverse), iters, C.byref(ms))
        assert rc == 0, "refcuda_ntt failed"
        return ms.value

    def sud(self, out_ptr, in1_ptr, in2_ptr, bases, factors, iters=1):
        ms = C.c_float(0)
        rc = self.dll.refcuda_sud(self.h, out_ptr, in1_ptr, in2_ptr, self._u32(bases), len(bases), self._u32(factors),
                                  iters, C.byref(ms))
        assert rc == 0, "refcuda_sud failed"
        return ms.value

    def bconv(self, out_ptr, in_ptr, in_idx, out_idx, n_conv=1, iters=1):
        ms = C.c_float(0)
        rc = self.dll.refcuda_bconv(self.h, out_ptr, in_ptr, self._u32(in_idx), len(in_idx), self._u32(out_idx),
                                    len(out_idx), n_conv, iters, C.byref(ms))
        assert rc == 0, "refcuda_bconv failed (rc=%d; 3 = shape not instantiated)" % rc
        return ms.value
