"""ctypes binding of ``include/cerium_b200.h``.

``Library(path)`` declares every entry point of the C ABI; ``load()`` opens the in-tree CUDA
build and raises if it is missing: there is no CPU implementation to fall back to.
Arguments that the C ABI takes as device pointers are plain integers here (``tensor.data_ptr()``).
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional, Sequence

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libcerium_b200.so")

OK, ERR_INVALID, ERR_CUDA, ERR_UNSUPPORTED = 0, 1, 2, 3
BCONV_LAZY, BCONV_EXACT = 0, 1
ROUND_FLOOR, ROUND_HALF = 0, 1
EW_ADD, EW_SUB, EW_NEG, EW_MUL, EW_MAD, EW_PMU, EW_MUL_SCALAR, EW_REDUCE = range(8)
COMM_ID_BYTES = 128

_vp = C.c_void_p
_u32p = C.POINTER(C.c_uint32)
_u64p = C.POINTER(C.c_uint64)
_sz = C.c_size_t

# name -> (restype, argtypes); the list is also what the symbol-export test checks
SIGNATURES = {
    "cerium_version": (C.c_int, []),
    "cerium_last_error": (C.c_char_p, []),
    "cerium_context_create": (C.c_int, [C.POINTER(_vp), C.c_int, C.c_int, C.c_int, _u64p, C.c_int]),
    "cerium_context_destroy": (C.c_int, [_vp]),
    "cerium_context_check": (C.c_int, [_vp]),
    "cerium_context_word_bits": (C.c_int, [_vp]),
    "cerium_context_num_moduli": (C.c_int, [_vp]),
    "cerium_context_modulus": (C.c_uint64, [_vp, C.c_int]),
    "cerium_context_root": (C.c_uint64, [_vp, C.c_int]),
    "cerium_ntt_forward": (C.c_int, [_vp, _vp, _sz, _vp, _sz, _u32p, C.c_int, _vp]),
    "cerium_ntt_inverse": (C.c_int, [_vp, _vp, _sz, _vp, _sz, _u32p, C.c_int, _vp]),
    "cerium_ntt_forward_ptrs": (C.c_int, [_vp, _vp, _vp, _vp, _sz, _vp]),
    "cerium_ntt_inverse_ptrs": (C.c_int, [_vp, _vp, _vp, _vp, _sz, _vp]),
    "cerium_function_map_bind": (C.c_int, [_vp, C.c_int]),
    "cerium_function_map_get": (_vp, [C.c_char_p, C.c_char_p, C.c_int]),
    "cerium_function_map_error": (C.c_char_p, []),
    "cerium_function_map_size": (C.c_int, [C.c_char_p, C.c_int]),
    "cerium_function_map_lookup": (_vp, [C.c_char_p, C.c_int, C.c_uint32]),
    "cerium_function_map_launcher": (_vp, [C.c_char_p, C.c_int]),
    "cerium_sud_ptrs": (C.c_int, [_vp, _vp, _vp, _vp, _sz, _vp, _vp]),
    "cerium_bconv_ptrs": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _vp]),
    "cerium_sud": (C.c_int, [_vp, _vp, _sz, _vp, _sz, _vp, _sz, _vp, _sz, _u32p, C.c_int, _u32p, C.c_int, _vp]),
    "cerium_ewise": (C.c_int, [_vp, C.c_int, _vp, _sz, _vp, _sz, _vp, _sz, _vp, _sz, _u64p, _u32p, C.c_int, _vp]),
    "cerium_tensor": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _u32p, C.c_int, _vp]),
    "cerium_galois_elt_from_step": (C.c_uint32, [C.c_int, C.c_int]),
    "cerium_automorph": (C.c_int, [_vp, _vp, _sz, _vp, _sz, C.c_uint32, C.c_int, _vp]),
    "cerium_mul_plain_periodic": (C.c_int, [_vp, _vp, _sz, _vp, _sz, _vp, _sz, C.c_int, _vp, _sz, C.POINTER(C.c_uint32),
                                            C.c_int, _vp]),
    "cerium_resolve2": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _sz, C.c_uint32, C.c_uint32, C.c_int, _vp]),
    "cerium_mod2": (C.c_int, [_vp, _vp, _sz, _vp, _vp, _u32p, C.c_int, _vp]),
    "cerium_bconv_create": (C.c_int, [_vp, C.POINTER(_vp), C.c_int, _u32p, C.c_int, _u32p, C.c_int]),
    "cerium_bconv_destroy": (C.c_int, [_vp]),
    "cerium_bconv_apply": (C.c_int, [_vp, _vp, _sz, _vp, _sz, _vp]),
    "cerium_bconv_apply_batch": (C.c_int, [C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp), C.c_int, _sz, _sz, _vp]),
    "cerium_keyswitch_create": (C.c_int, [_vp, C.POINTER(_vp), C.c_int, C.c_int, _u32p, C.c_int, _u32p, C.c_int, C.c_int]),
    "cerium_keyswitch_create_sharded": (C.c_int, [_vp, C.POINTER(_vp), C.c_int, C.c_int, _u32p, C.c_int, _u32p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    "cerium_keyswitch_local_limbs": (C.c_int, [_vp]),
    "cerium_keyswitch_local_ext_limbs": (C.c_int, [_vp]),
    "cerium_keyswitch_sharded_apply": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "cerium_hrot_sharded": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, C.c_uint32, _vp]),
    "cerium_rescale_sharded": (C.c_int, [_vp, _vp, C.c_int, _vp, _vp, _u32p, C.c_int, C.c_int, _vp, _vp]),
    "cerium_comm_unique_id": (C.c_int, [_vp, _sz]),
    "cerium_comm_init": (C.c_int, [C.POINTER(_vp), _vp, _sz, C.c_int, C.c_int, C.c_int]),
    "cerium_comm_init_callbacks": (C.c_int, [C.POINTER(_vp), C.c_int, C.c_int, C.c_int, _vp]),
    "cerium_comm_split": (C.c_int, [_vp, C.c_int, C.POINTER(_vp)]),
    "cerium_comm_destroy": (C.c_int, [_vp]),
    "cerium_comm_rank": (C.c_int, [_vp]),
    "cerium_comm_world": (C.c_int, [_vp]),
    "cerium_allgather_limbs": (C.c_int, [_vp, _vp, _vp, _vp, _sz, _vp]),
    "cerium_reducescatter_limbs": (C.c_int, [_vp, _vp, _vp, _vp, _u32p, C.c_int, _vp]),
    "cerium_allreduce_limbs": (C.c_int, [_vp, _vp, _vp, _vp, _u32p, C.c_int, _vp]),
    "cerium_broadcast_limbs": (C.c_int, [_vp, _vp, _vp, _sz, C.c_int, _vp]),
    "cerium_keyswitch_gather_limbs": (C.c_int, [_vp]),
    "cerium_keyswitch_sharded_begin": (C.c_int, [_vp, _vp, _vp, _vp]),
    "cerium_keyswitch_sharded_finish": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "cerium_keyswitch_destroy": (C.c_int, [_vp]),
    "cerium_keyswitch_workspace_bytes": (_sz, [_vp]),
    "cerium_keyswitch_apply": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "cerium_keyswitch_apply_rescale": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, C.c_int, _vp]),
    "cerium_plaintext_mac": (C.c_int, [_vp, C.c_int, C.c_int, C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp),
                                       C.POINTER(_vp), _u32p, C.c_int, _vp]),
    "cerium_bsgs_work_limbs": (_sz, [_vp, C.c_int, C.c_int]),
    "cerium_bsgs_apply": (C.c_int, [_vp, _vp, _vp, _vp, _vp, C.c_int, C.c_int, C.POINTER(_vp), C.POINTER(_vp), _u32p,
                                    C.POINTER(_vp), _u32p, C.c_int, _vp, _vp]),
    "cerium_hrot": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, C.c_uint32, _vp]),
    "cerium_hoisted_begin": (C.c_int, [_vp, _vp, _vp]),
    "cerium_hoisted_rotate": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, C.c_uint32, _vp]),
    "cerium_hmult": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, C.c_int, _vp]),
    "cerium_rescale": (C.c_int, [_vp, C.c_int, _vp, _vp, _u32p, C.c_int, C.c_int, _vp, _vp]),
    "cerium_keyswitch_create_lifted": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.c_int, C.c_int,
                                                 C.POINTER(C.c_uint32), C.c_int, C.POINTER(C.c_uint32), C.c_int]),
    "cerium_mod_raise": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32,
                                   C.c_void_p, C.c_void_p]),
    "cerium_rescale_local": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.POINTER(C.c_uint32), C.c_int,
                                       C.c_uint32, C.c_void_p, C.c_int, C.c_void_p]),
    "cerium_double_rescale": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(C.c_uint32), C.c_int, C.c_int,
                                        C.c_void_p, C.c_void_p]),
    "cerium_rescale_static": (C.c_int, [_vp, C.c_int, _vp, _vp, _u32p, C.c_int, C.c_int, _vp]),
    "cerium_program_load": (C.c_int, [_vp, C.POINTER(_vp), C.c_char_p, C.c_char_p, C.POINTER(C.c_char_p), _u64p, C.c_int, _vp]),
    "cerium_program_destroy": (C.c_int, [_vp]),
    "cerium_program_num_steps": (C.c_int, [_vp]),
    "cerium_program_memory": (C.c_int, [_vp, C.c_char_p, C.POINTER(_vp)]),
    "cerium_program_run": (C.c_int, [_vp, _vp]),
    "cerium_program_capture": (C.c_int, [_vp]),
    "cerium_program_write": (C.c_int, [_vp, C.c_char_p, C.POINTER(C.c_uint32), C.c_int, _vp, _vp]),
    "cerium_program_read": (C.c_int, [_vp, C.c_char_p, C.POINTER(C.c_uint32), C.c_int, _vp, _vp]),
    "cerium_program_inspect": (C.c_int, [C.c_char_p, C.c_char_p, _sz, C.POINTER(C.c_int)]),
}


class CeriumError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__("cerium_b200 error %d: %s" % (code, message))
        self.code = code
        self.message = message


def _u32(values: Sequence[int]):
    arr = (C.c_uint32 * len(values))(*[int(v) for v in values])
    return arr


def _u64(values: Sequence[int]):
    arr = (C.c_uint64 * len(values))(*[int(v) for v in values])
    return arr


class Library:
    """One loaded copy of the C ABI."""

    def __init__(self, path: str):
        if not os.path.exists(path):
            raise FileNotFoundError(
                "%s not found: build it with `python -m cerium_b200.build` (there is no CPU fallback)" % path)
        self.path = path
        self.dll = C.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(self.dll, name)
            fn.restype = res
            fn.argtypes = args

    def check(self, rc: int) -> None:
        if rc != OK:
            raise CeriumError(rc, self.dll.cerium_last_error().decode())

    def galois_elt_from_step(self, step: int, logn: int = 16) -> int:
        return int(self.dll.cerium_galois_elt_from_step(step, logn))


class Context:
    """Device tables for a prime list (handle of ``cerium_context``)."""

    def __init__(self, lib: Library, moduli: Sequence[int], word_bits: int, device: int = 0, logn: int = 16):
        self.lib = lib
        self.moduli = [int(m) for m in moduli]
        self.word_bits = int(word_bits)
        self.logn = logn
        self.n = 1 << logn
        self.device = device
        h = _vp()
        lib.check(lib.dll.cerium_context_create(C.byref(h), device, logn, word_bits, _u64(self.moduli), len(self.moduli)))
        self.h = h

    def close(self):
        if getattr(self, "h", None):
            self.lib.dll.cerium_context_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def word_bytes(self) -> int:
        return self.word_bits // 8

    def root(self, k: int) -> int:
        return int(self.lib.dll.cerium_context_root(self.h, k))

    def check(self):
        """Waits for the device and raises if a kernel skipped a malformed work item since the last check."""
        self.lib.check(self.lib.dll.cerium_context_check(self.h))

    # -- transforms ------------------------------------------------------------------
    def ntt_forward(self, out: int, inp: int, prime_idx: Sequence[int], out_stride: Optional[int] = None,
                    in_stride: Optional[int] = None, stream: int = 0):
        n = self.n
        self.lib.check(self.lib.dll.cerium_ntt_forward(self.h, out, out_stride or n, inp, in_stride or n,
                                                       _u32(prime_idx), len(prime_idx), stream))

    def ntt_inverse(self, out: int, inp: int, prime_idx: Sequence[int], out_stride: Optional[int] = None,
                    in_stride: Optional[int] = None, stream: int = 0):
        n = self.n
        self.lib.check(self.lib.dll.cerium_ntt_inverse(self.h, out, out_stride or n, inp, in_stride or n,
                                                       _u32(prime_idx), len(prime_idx), stream))

    def ntt_forward_ptrs(self, outs: int, ins: int, bases: int, num_bases: int, stream: int = 0):
        self.lib.check(self.lib.dll.cerium_ntt_forward_ptrs(self.h, outs, ins, bases, num_bases, stream))

    def ntt_inverse_ptrs(self, outs: int, ins: int, bases: int, num_bases: int, stream: int = 0):
        self.lib.check(self.lib.dll.cerium_ntt_inverse_ptrs(self.h, outs, ins, bases, num_bases, stream))

    def sud_ptrs(self, outs: int, ins: int, bases: int, num_bases: int, factors: int, stream: int = 0):
        """SuD on device pointer tables (two inputs per entry), the reference launcher's layout."""
        self.lib.check(self.lib.dll.cerium_sud_ptrs(self.h, outs, ins, bases, num_bases, factors, stream))

    def bconv_ptrs(self, outs: int, n_out: int, ins: int, n_in: int, factors: int, out_moduli: int,
                   max_in: int, max_out: int, num_conversions: int, stream: int = 0):
        """Base conversion driven by device tables only, the reference launcher's layout."""
        self.lib.check(self.lib.dll.cerium_bconv_ptrs(self.h, outs, n_out, ins, n_in, factors, out_moduli,
                                                      max_in, max_out, num_conversions, stream))

    def sud(self, out: int, minuend: int, in_coeff: int, prime_idx: Sequence[int], divide_primes: Sequence[int],
            addend: int = 0, stream: int = 0):
        n = self.n
        self.lib.check(self.lib.dll.cerium_sud(self.h, out, n, minuend, n, in_coeff, n, addend or None, n,
                                               _u32(prime_idx), len(prime_idx), _u32(divide_primes),
                                               len(divide_primes), stream))

    # -- element-wise ----------------------------------------------------------------
    def ewise(self, op: int, out: int, a: int, prime_idx: Sequence[int], b: int = 0, c: int = 0,
              scalars: Optional[Sequence[int]] = None, stream: int = 0):
        n = self.n
        sc = _u64(scalars) if scalars is not None else None
        self.lib.check(self.lib.dll.cerium_ewise(self.h, op, out, n, a, n, b or None, n, c or None, n, sc,
                                                 _u32(prime_idx), len(prime_idx), stream))

    def tensor(self, d0: int, d1: int, d2: int, a0: int, a1: int, b0: int, b1: int, prime_idx: Sequence[int],
               stream: int = 0):
        self.lib.check(self.lib.dll.cerium_tensor(self.h, d0, d1, d2, a0, a1, b0, b1, self.n, _u32(prime_idx),
                                                  len(prime_idx), stream))

    def mul_plain_periodic(self, out: int, a: int, pt: int, log2_repeat: int, prime_idx: Sequence[int], addend: int = 0,
                           pt_stride: Optional[int] = None, stream: int = 0):
        """out = a * pt[i >> log2_repeat] (+ addend): the plaintext is stored once per period."""
        n = self.n
        self.lib.check(self.lib.dll.cerium_mul_plain_periodic(self.h, out, n, a, n, pt, pt_stride or (n >> log2_repeat),
                                                              log2_repeat, addend or None, n, _u32(prime_idx),
                                                              len(prime_idx), stream))

    def automorph(self, out: int, inp: int, galois_elt: int, count: int, stream: int = 0):
        n = self.n
        self.lib.check(self.lib.dll.cerium_automorph(self.h, out, n, inp, n, galois_elt, count, stream))

    def resolve2(self, lo: int, hi: int, x0: int, x1: int, prime0: int, prime1: int, count: int = 1, stream: int = 0):
        self.lib.check(self.lib.dll.cerium_resolve2(self.h, lo, hi, x0, x1, self.n, prime0, prime1, count, stream))

    def mod2(self, out: int, lo: int, hi: int, prime_idx: Sequence[int], stream: int = 0):
        self.lib.check(self.lib.dll.cerium_mod2(self.h, out, self.n, lo, hi, _u32(prime_idx), len(prime_idx), stream))

    def rescale(self, out: int, inp: int, q_idx: Sequence[int], n_polys: int, scratch: int,
                round_mode: int = ROUND_FLOOR, stream: int = 0):
        self.lib.check(self.lib.dll.cerium_rescale(self.h, round_mode, out, inp, _u32(q_idx), len(q_idx), n_polys,
                                                   scratch, stream))


    def rescale_local(self, out: int, inp: int, local_idx: Sequence[int], last_prime: int, last_coef: int,
                      n_polys: int, round_mode: int = ROUND_FLOOR, stream: int = 0):
        """Rescale of one rank's remaining limbs against the broadcast coefficient-form last limb."""
        self.lib.check(self.lib.dll.cerium_rescale_local(self.h, round_mode, out, inp, _u32(local_idx), len(local_idx),
                                                         last_prime, last_coef, n_polys, stream))

    def plaintext_mac(self, out0: Sequence[int], out1: Sequence[int], src0: Sequence[int], src1: Sequence[int],
                      plaintexts: Sequence[int], prime_idx: Sequence[int], stream: int = 0):
        """out_i = sum_j pt[i][j] (.) src_j for both polynomials; plaintexts: len(out0) * len(src0) device
        addresses, entry i * n_src + j, 0 = no such term."""
        vp = lambda seq: (_vp * len(seq))(*[_vp(int(p)) if p else _vp() for p in seq])  # noqa: E731
        self.lib.check(self.lib.dll.cerium_plaintext_mac(self.h, len(out0), len(src0), vp(out0), vp(out1), vp(src0),
                                                         vp(src1), vp(plaintexts), _u32(prime_idx), len(prime_idx), stream))

    def rescale_sharded(self, comm: "Comm", out: int, inp: int, q_idx: Sequence[int], n_polys: int, last_coef: int,
                        round_mode: int = ROUND_FLOOR, stream: int = 0):
        """Rescale of this rank's limbs of a limb-sharded ciphertext (owner's inverse transform of the
        last limb, broadcast, division of the remaining local limbs)."""
        self.lib.check(self.lib.dll.cerium_rescale_sharded(self.h, comm.h, round_mode, out or None, inp or None,
                                                           _u32(q_idx), len(q_idx), n_polys, last_coef, stream))

    def double_rescale(self, out: int, inp: int, q_idx: Sequence[int], n_polys: int, scratch: int, stream: int = 0):
        """Drops the last two limbs at once; scratch holds 4 * n_polys limbs."""
        self.lib.check(self.lib.dll.cerium_double_rescale(self.h, out, inp, _u32(q_idx), len(q_idx), n_polys,
                                                          scratch, stream))

    def rescale_static(self, out: int, inp: int, q_idx: Sequence[int], n_polys: int,
                       round_mode: int = ROUND_FLOOR, stream: int = 0):
        """Rescale with the library's built-in scratch (no device allocation anywhere; n_polys <= 2)."""
        self.lib.check(self.lib.dll.cerium_rescale_static(self.h, round_mode, out, inp, _u32(q_idx), len(q_idx),
                                                          n_polys, stream))


ALLGATHER_FN = C.CFUNCTYPE(C.c_int, _vp, _vp, _vp, _sz, _vp)
REDUCESCATTER_FN = C.CFUNCTYPE(C.c_int, _vp, _vp, _vp, _sz, C.c_int, _vp)
ALLREDUCE_FN = C.CFUNCTYPE(C.c_int, _vp, _vp, _vp, _sz, C.c_int, _vp)
BROADCAST_FN = C.CFUNCTYPE(C.c_int, _vp, _vp, _sz, C.c_int, _vp)


class CommCallbacks(C.Structure):
    """``cerium_comm_callbacks``: the caller's own collectives."""
    _fields_ = [("user", _vp), ("allgather", ALLGATHER_FN), ("reducescatter", REDUCESCATTER_FN),
                ("allreduce", ALLREDUCE_FN), ("broadcast", BROADCAST_FN)]


class Comm:
    """Communicator of the limb collectives (handle of ``cerium_comm``).

    ``Comm(lib, rank, world, device, nccl_id=...)`` joins an NCCL communicator (``Comm.unique_id(lib)``
    on rank 0, handed to every rank by the caller); ``Comm(lib, rank, world, device, transport=obj)``
    uses the caller's collectives: ``obj`` has methods ``allgather(recv, send, bytes_per_rank,
    stream)``, ``reducescatter(recv, send, words_per_rank, word_bits, stream)``, ``allreduce(recv,
    send, words, word_bits, stream)``, ``broadcast(buf, bytes, root, stream)`` over raw addresses
    (missing methods leave that collective unsupported)."""

    def __init__(self, lib: Library, rank: int, world: int, device: int = 0, nccl_id: Optional[bytes] = None,
                 transport=None):
        self.lib, self.rank, self.world = lib, rank, world
        h = _vp()
        if transport is not None:
            def wrap(fn_type, method):
                m = getattr(transport, method, None)
                if m is None:
                    return fn_type()

                def call(user, *args):
                    try:
                        m(*[0 if a is None else a for a in args])
                        return 0
                    except Exception:       # an exception cannot cross the C boundary
                        import traceback
                        traceback.print_exc()
                        return 1
                return fn_type(call)
            self._cb = CommCallbacks(None, wrap(ALLGATHER_FN, "allgather"), wrap(REDUCESCATTER_FN, "reducescatter"),
                                     wrap(ALLREDUCE_FN, "allreduce"), wrap(BROADCAST_FN, "broadcast"))
            lib.check(lib.dll.cerium_comm_init_callbacks(C.byref(h), rank, world, device, C.byref(self._cb)))
        else:
            if nccl_id is None or len(nccl_id) < COMM_ID_BYTES:
                raise ValueError("an NCCL communicator needs the %d-byte id made by Comm.unique_id" % COMM_ID_BYTES)
            buf = C.create_string_buffer(bytes(nccl_id), COMM_ID_BYTES)
            lib.check(lib.dll.cerium_comm_init(C.byref(h), buf, COMM_ID_BYTES, rank, world, device))
        self.h = h

    @staticmethod
    def unique_id(lib: Library) -> bytes:
        buf = C.create_string_buffer(COMM_ID_BYTES)
        lib.check(lib.dll.cerium_comm_unique_id(buf, COMM_ID_BYTES))
        return buf.raw

    def split(self, size: int) -> int:
        """Handle of the communicator of the `size` consecutive ranks that hold this rank (owned by this one);
        collective over all ranks.  Raises where the transport has no sub-groups."""
        h = _vp()
        self.lib.check(self.lib.dll.cerium_comm_split(self.h, size, C.byref(h)))
        return int(h.value)

    def allgather_limbs(self, ctx: "Context", gathered: int, send: int, limbs_per_rank: int, stream: int = 0):
        self.lib.check(self.lib.dll.cerium_allgather_limbs(self.h, ctx.h, gathered, send, limbs_per_rank, stream))

    def reducescatter_limbs(self, ctx: "Context", out: int, inp: int, prime_idx: Sequence[int], stream: int = 0):
        self.lib.check(self.lib.dll.cerium_reducescatter_limbs(self.h, ctx.h, out, inp, _u32(prime_idx),
                                                               len(prime_idx), stream))

    def allreduce_limbs(self, ctx: "Context", out: int, inp: int, prime_idx: Sequence[int], stream: int = 0):
        self.lib.check(self.lib.dll.cerium_allreduce_limbs(self.h, ctx.h, out, inp, _u32(prime_idx), len(prime_idx),
                                                           stream))

    def broadcast_limbs(self, ctx: "Context", buf: int, limbs: int, root: int, stream: int = 0):
        self.lib.check(self.lib.dll.cerium_broadcast_limbs(self.h, ctx.h, buf, limbs, root, stream))

    def close(self):
        if getattr(self, "h", None):
            self.lib.dll.cerium_comm_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def inspect_program(lib: Library, functions_path: str):
    """Parses a compiled function's kernel stream (no device): list of dicts, one per record."""
    n = C.c_int()
    buf = C.create_string_buffer(1 << 22)
    lib.check(lib.dll.cerium_program_inspect(functions_path.encode(), buf, len(buf), C.byref(n)))
    keys = ("id", "type", "outputs", "inputs", "bases", "rots", "units", "sud", "pmu", "rsv", "scalars", "comm_size",
            "comm_num_limbs", "comm_srcs", "comm_dests", "call_args", "callee")
    out = []
    for line in buf.value.decode().splitlines():
        f = line.split()
        out.append({k: (v if k in ("type", "callee") else int(v)) for k, v in zip(keys, f)})
    assert len(out) == n.value
    return out


class Program:
    """One partition of a compiled Cerium function, loaded for replay (handle of ``cerium_program``)."""

    def __init__(self, ctx: Context, functions_path: str, plugin_path: str, scalars: Optional[dict] = None,
                 comm: Optional["Comm"] = None):
        self.ctx, self.comm = ctx, comm
        scalars = scalars or {}
        names = (C.c_char_p * max(1, len(scalars)))(*[k.encode() for k in scalars])
        vals = _u64(list(scalars.values()) or [0])
        h = _vp()
        ctx.lib.check(ctx.lib.dll.cerium_program_load(ctx.h, C.byref(h), functions_path.encode(), plugin_path.encode(),
                                                      names, vals, len(scalars), comm.h if comm is not None else None))
        self.h = h

    @property
    def num_steps(self) -> int:
        return int(self.ctx.lib.dll.cerium_program_num_steps(self.h))

    def memory(self, term: str) -> int:
        """Device address of a named memory term such as "i1(0)" (one limb)."""
        p = _vp()
        self.ctx.lib.check(self.ctx.lib.dll.cerium_program_memory(self.h, term.encode(), C.byref(p)))
        return int(p.value)

    def write(self, name: str, limb_ids: Sequence[int], host, stream: int = 0):
        """Copies host limbs ([len(limb_ids)][N] uint32, C-contiguous numpy) into the terms "name(limb)"."""
        assert host.dtype.itemsize == 4 and host.flags.c_contiguous and host.size == len(limb_ids) * self.ctx.n
        self.ctx.lib.check(self.ctx.lib.dll.cerium_program_write(self.h, name.encode(), _u32(limb_ids), len(limb_ids),
                                                                 host.ctypes.data, stream))

    def read(self, name: str, limb_ids: Sequence[int], host, stream: int = 0):
        assert host.dtype.itemsize == 4 and host.flags.c_contiguous and host.size == len(limb_ids) * self.ctx.n
        self.ctx.lib.check(self.ctx.lib.dll.cerium_program_read(self.h, name.encode(), _u32(limb_ids), len(limb_ids),
                                                                host.ctypes.data, stream))

    def run(self, stream: int = 0):
        self.ctx.lib.check(self.ctx.lib.dll.cerium_program_run(self.h, stream))

    def capture(self):
        """Records one run into a CUDA graph; later runs replay it."""
        self.ctx.lib.check(self.ctx.lib.dll.cerium_program_capture(self.h))

    def close(self):
        if getattr(self, "h", None) and self.ctx.h:
            self.ctx.lib.dll.cerium_program_destroy(self.h)
        self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class BaseConverter:
    """Fast base conversion between two prime sets (handle of ``cerium_bconv``)."""

    def __init__(self, ctx: Context, in_primes: Sequence[int], out_primes: Sequence[int], mode: int = BCONV_LAZY):
        self.ctx = ctx
        self.n_in, self.n_out = len(in_primes), len(out_primes)
        h = _vp()
        ctx.lib.check(ctx.lib.dll.cerium_bconv_create(ctx.h, C.byref(h), mode, _u32(in_primes), len(in_primes),
                                                      _u32(out_primes), len(out_primes)))
        self.h = h

    def apply(self, out: int, inp: int, out_stride: Optional[int] = None, in_stride: Optional[int] = None,
              stream: int = 0):
        n = self.ctx.n
        self.ctx.lib.check(self.ctx.lib.dll.cerium_bconv_apply(self.h, out, out_stride or n, inp, in_stride or n, stream))

    @staticmethod
    def apply_batch(converters, outs: Sequence[int], ins: Sequence[int], stream: int = 0):
        """Several conversions (converters of one context) in one launch."""
        ctx = converters[0].ctx
        n = ctx.n
        k = len(converters)
        hs = (_vp * k)(*[c.h for c in converters])
        o = (_vp * k)(*[_vp(int(p)) for p in outs])
        i = (_vp * k)(*[_vp(int(p)) for p in ins])
        ctx.lib.check(ctx.lib.dll.cerium_bconv_apply_batch(hs, o, i, k, n, n, stream))

    def close(self):
        if getattr(self, "h", None) and self.ctx.h:
            self.ctx.lib.dll.cerium_bconv_destroy(self.h)
        self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class KeySwitch:
    """Hybrid key-switching plan (handle of ``cerium_keyswitch``)."""

    def __init__(self, ctx: Context, q_idx: Sequence[int], p_idx: Sequence[int], dnum: int,
                 bconv_mode: int = BCONV_LAZY, round_mode: int = ROUND_FLOOR, rank: int = 0, world: int = 1,
                 lifted: bool = False, ext_split: bool = False):
        self.ctx = ctx
        self.q_idx, self.p_idx, self.dnum = list(q_idx), list(p_idx), dnum
        self.rank, self.world, self.ext_split = rank, world, bool(ext_split) and world > 1
        h = _vp()
        if lifted:
            # ModRaise plan: q_idx = target primes + the prime the final rescale drops; one lifted digit
            ctx.lib.check(ctx.lib.dll.cerium_keyswitch_create_lifted(ctx.h, C.byref(h), bconv_mode, round_mode,
                                                                     _u32(q_idx), len(q_idx), _u32(p_idx), len(p_idx)))
        else:
            ctx.lib.check(ctx.lib.dll.cerium_keyswitch_create_sharded(ctx.h, C.byref(h), bconv_mode, round_mode,
                                                                      _u32(q_idx), len(q_idx), _u32(p_idx), len(p_idx),
                                                                      dnum, rank, world, 1 if ext_split else 0))
        self.h = h

    def mod_raise(self, out0: int, out1: int, c0: int, c1: int, base0: int, base1: int, evk: int, stream: int = 0):
        self.ctx.lib.check(self.ctx.lib.dll.cerium_mod_raise(self.h, out0, out1, c0, c1, base0, base1, evk, stream))

    @property
    def local_limbs(self) -> int:
        return int(self.ctx.lib.dll.cerium_keyswitch_local_limbs(self.h))

    @property
    def gather_limbs(self) -> int:
        return int(self.ctx.lib.dll.cerium_keyswitch_gather_limbs(self.h))

    @property
    def local_ext_limbs(self) -> int:
        return int(self.ctx.lib.dll.cerium_keyswitch_local_ext_limbs(self.h))

    def sharded_apply(self, comm: "Comm", out0: int, out1: int, cpoly_local: int, evk_local: int, add0: int = 0,
                      add1: int = 0, stream: int = 0):
        self.ctx.lib.check(self.ctx.lib.dll.cerium_keyswitch_sharded_apply(
            self.h, comm.h, out0 or None, out1 or None, cpoly_local or None, evk_local, add0 or None, add1 or None,
            stream))

    def hrot_sharded(self, comm: "Comm", out0: int, out1: int, c0_local: int, c1_local: int, evk_local: int,
                     galois_elt: int, stream: int = 0):
        self.ctx.lib.check(self.ctx.lib.dll.cerium_hrot_sharded(
            self.h, comm.h, out0 or None, out1 or None, c0_local or None, c1_local or None, evk_local, galois_elt,
            stream))

    def sharded_begin(self, send: int, cpoly_local: int, stream: int = 0):
        self.ctx.lib.check(self.ctx.lib.dll.cerium_keyswitch_sharded_begin(self.h, send, cpoly_local or None, stream))

    def sharded_finish(self, out0: int, out1: int, gathered: int, cpoly_local: int, evk_local: int, add0: int = 0,
                       add1: int = 0, stream: int = 0):
        self.ctx.lib.check(self.ctx.lib.dll.cerium_keyswitch_sharded_finish(
            self.h, out0 or None, out1 or None, gathered, cpoly_local or None, evk_local, add0 or None,
            add1 or None, stream))

    @property
    def workspace_bytes(self) -> int:
        return int(self.ctx.lib.dll.cerium_keyswitch_workspace_bytes(self.h))

    def apply(self, out0: int, out1: int, cpoly: int, evk: int, add0: int = 0, add1: int = 0, stream: int = 0):
        self.ctx.lib.check(self.ctx.lib.dll.cerium_keyswitch_apply(self.h, out0, out1, cpoly, evk, add0 or None,
                                                                   add1 or None, stream))

    def apply_rescale(self, out0: int, out1: int, cpoly: int, evk: int, rescale_levels: int, add0: int = 0,
                      add1: int = 0, stream: int = 0):
        """Key switch with the PMU pre-additions and the rescale folded into the ModDown (one division)."""
        self.ctx.lib.check(self.ctx.lib.dll.cerium_keyswitch_apply_rescale(self.h, out0, out1, cpoly, evk, add0 or None,
                                                                           add1 or None, rescale_levels, stream))

    def bsgs_work_limbs(self, g: int, n_giant: int) -> int:
        return int(self.ctx.lib.dll.cerium_bsgs_work_limbs(self.h, g, n_giant))

    def bsgs_apply(self, out0: int, out1: int, c0: int, c1: int, g: int, n_giant: int, plaintexts: Sequence[int],
                   baby_keys_pre: Sequence[int], baby_elts: Sequence[int], giant_keys: Sequence[int],
                   giant_elts: Sequence[int], rescale_levels: int, work: int, stream: int = 0):
        """plaintexts: n_giant * g device addresses (0 = absent diagonal), entry i * g + j; baby_* have g
        entries (entry 0 unused), giant_* have n_giant entries (element 1 = no rotation, key 0)."""
        vp = lambda seq: (_vp * len(seq))(*[_vp(int(p)) if p else _vp() for p in seq])  # noqa: E731
        self.ctx.lib.check(self.ctx.lib.dll.cerium_bsgs_apply(
            self.h, out0, out1, c0, c1, g, n_giant, vp(plaintexts), vp(baby_keys_pre), _u32(baby_elts), vp(giant_keys),
            _u32(giant_elts), rescale_levels, work, stream))

    def hrot(self, out0: int, out1: int, c0: int, c1: int, evk: int, galois_elt: int, stream: int = 0):
        self.ctx.lib.check(self.ctx.lib.dll.cerium_hrot(self.h, out0, out1, c0, c1, evk, galois_elt, stream))

    def hoisted_begin(self, c1: int, stream: int = 0):
        self.ctx.lib.check(self.ctx.lib.dll.cerium_hoisted_begin(self.h, c1, stream))

    def hoisted_rotate(self, out0: int, out1: int, c0: int, c1: int, evk_pre: int, galois_elt: int, stream: int = 0):
        self.ctx.lib.check(self.ctx.lib.dll.cerium_hoisted_rotate(self.h, out0, out1, c0, c1, evk_pre, galois_elt, stream))

    def hmult(self, out0: int, out1: int, a0: int, a1: int, b0: int, b1: int, evk: int, do_rescale,
              stream: int = 0):
        """do_rescale: False / 0 none, True / 1 ModDown then rescale, 2 the rescale folded into the ModDown."""
        self.ctx.lib.check(self.ctx.lib.dll.cerium_hmult(self.h, out0, out1, a0, a1, b0, b1, evk,
                                                         int(do_rescale), stream))

    def close(self):
        if getattr(self, "h", None) and self.ctx.h:
            self.ctx.lib.dll.cerium_keyswitch_destroy(self.h)
        self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


_default: Optional[Library] = None


def load() -> Library:
    """The shipped CUDA build.  Raises if the shared object is missing."""
    global _default
    if _default is None:
        _default = Library(LIB_PATH)
    return _default
