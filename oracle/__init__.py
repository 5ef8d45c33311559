"""ctypes binding of the CPU oracle (``cerium_oracle.c``).  TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark
may import this package; the shipped library never does.  All arrays are numpy
``uint64`` holding canonical residues in ``[0, q)``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")

BCONV_LAZY = 0   # Cerium semantics (factors fold the CRT inverse, no inner reduction)
BCONV_EXACT = 1  # textbook semantics (inner product reduced by q_i first)
ROUND_FLOOR = 0
ROUND_HALF = 1


def build(force: bool = False) -> str:
    """Compile ``liboracle.so`` with gcc if it is missing or older than its source."""
    src = os.path.join(_HERE, "cerium_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(
            ["gcc", "-O3", "-std=gnu11", "-fPIC", "-fopenmp", "-fvisibility=hidden", "-shared",
             "-o", _LIB_PATH, src])
    return _LIB_PATH


_lib = None
_u64p = C.POINTER(C.c_uint64)
_u32p = C.POINTER(C.c_uint32)


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        L.orc_mulmod.restype = C.c_uint64
        L.orc_mulmod.argtypes = [C.c_uint64] * 3
        L.orc_powmod.restype = C.c_uint64
        L.orc_powmod.argtypes = [C.c_uint64] * 3
        L.orc_invmod.restype = C.c_uint64
        L.orc_invmod.argtypes = [C.c_uint64] * 2
        L.orc_is_prime.restype = C.c_int
        L.orc_is_prime.argtypes = [C.c_uint64]
        L.orc_min_primitive_root.restype = C.c_uint64
        L.orc_min_primitive_root.argtypes = [C.c_uint64, C.c_int]
        L.orc_ctx_create.restype = C.c_void_p
        L.orc_ctx_create.argtypes = [C.c_int, _u64p, C.c_int]
        L.orc_ctx_destroy.argtypes = [C.c_void_p]
        L.orc_ctx_modulus.restype = C.c_uint64
        L.orc_ctx_modulus.argtypes = [C.c_void_p, C.c_int]
        L.orc_ctx_root.restype = C.c_uint64
        L.orc_ctx_root.argtypes = [C.c_void_p, C.c_int]
        L.orc_ctx_twiddle.restype = C.c_uint64
        L.orc_ctx_twiddle.argtypes = [C.c_void_p, C.c_int, C.c_size_t]
        L.orc_ntt_forward.argtypes = [C.c_void_p, C.c_int, _u64p]
        L.orc_ntt_inverse.argtypes = [C.c_void_p, C.c_int, _u64p]
        L.orc_ntt_forward_batch.argtypes = [C.c_void_p, _u64p, _u32p, C.c_int]
        L.orc_ntt_inverse_batch.argtypes = [C.c_void_p, _u64p, _u32p, C.c_int]
        L.orc_negacyclic_mul_schoolbook.argtypes = [C.c_uint64, C.c_size_t, _u64p, _u64p, _u64p]
        L.orc_galois_elt_from_step.restype = C.c_uint32
        L.orc_galois_elt_from_step.argtypes = [C.c_int, C.c_int]
        L.orc_galois_table_ntt.argtypes = [C.c_uint32, C.c_int, _u32p]
        L.orc_apply_galois_ntt.argtypes = [C.c_uint32, C.c_int, _u64p, _u64p]
        L.orc_apply_galois_coeff.argtypes = [C.c_uint32, C.c_int, C.c_uint64, _u64p, _u64p]
        L.orc_resolve2.argtypes = [C.c_uint64, C.c_uint64, C.c_size_t, _u64p, _u64p, _u64p, _u64p]
        L.orc_mod2.argtypes = [C.c_uint64, C.c_size_t, _u64p, _u64p, _u64p]
        L.orc_bconv.argtypes = [C.c_int, C.c_size_t, C.c_int, _u64p, _u64p, C.c_int, _u64p, _u64p]
        L.orc_sud.argtypes = [C.c_void_p, C.c_int, _u64p, _u64p, C.c_uint64, _u64p]
        L.orc_moddown.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, _u32p, C.c_int, _u32p,
                                  _u64p, _u64p, _u64p]
        L.orc_keyswitch.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, _u32p, C.c_int, _u32p,
                                    C.c_int, _u64p, _u64p, _u64p, _u64p]
        L.orc_keyswitch_acc.argtypes = [C.c_void_p, C.c_int, C.c_int, _u32p, C.c_int, _u32p, C.c_int, _u64p, _u64p,
                                        _u64p, _u64p]
        L.orc_moddown_rescale.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, _u32p, C.c_int, _u32p, C.c_int,
                                          _u64p, _u64p]
        L.orc_keyswitch_rescale.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, _u32p, C.c_int, _u32p, C.c_int,
                                            C.c_int, _u64p, _u64p, _u64p, _u64p, _u64p, _u64p]
        L.orc_hmult_relin_fused.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, _u32p, C.c_int, _u32p, C.c_int,
                                            _u64p, _u64p, _u64p, _u64p, _u64p, _u64p, _u64p]
        L.orc_bsgs.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, _u32p, C.c_int, _u32p, C.c_int, C.c_int, C.c_int,
                               C.c_int, _u64p, _u64p, C.POINTER(C.c_uint8), _u32p, _u64p, _u64p, _u64p]
        L.orc_rescale.argtypes = [C.c_void_p, C.c_int, C.c_int, _u32p, _u64p, _u64p]
        L.orc_double_rescale.argtypes = [C.c_void_p, C.c_int, _u32p, _u64p, _u64p]
        L.orc_mod_raise.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, _u32p, C.c_int, _u32p, C.c_uint32,
                                    C.c_uint32, _u64p, _u64p, _u64p, _u64p, _u64p]
        L.orc_hrot.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, _u32p, C.c_int, _u32p,
                               C.c_int, C.c_uint32, _u64p, _u64p, _u64p, _u64p, _u64p]
        L.orc_hmult_relin.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, _u32p,
                                      C.c_int, _u32p, C.c_int, _u64p, _u64p, _u64p, _u64p, _u64p,
                                      _u64p, _u64p]
        L.orc_num_threads.restype = C.c_int
        L.orc_set_num_threads.argtypes = [C.c_int]
        for name in ("orc_ew_add", "orc_ew_sub", "orc_ew_mul"):
            getattr(L, name).argtypes = [C.c_uint64, C.c_size_t, _u64p, _u64p, _u64p]
        L.orc_ew_neg.argtypes = [C.c_uint64, C.c_size_t, _u64p, _u64p]
        L.orc_ew_mad.argtypes = [C.c_uint64, C.c_size_t, _u64p, _u64p, _u64p, _u64p]
        L.orc_ew_pmu.argtypes = [C.c_uint64, C.c_size_t, _u64p, _u64p, C.c_uint64, _u64p]
        _lib = L
    return _lib


def _p64(a: np.ndarray):
    assert a.dtype == np.uint64 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_u64p)


def _p32(a: np.ndarray):
    assert a.dtype == np.uint32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_u32p)


def _idx(v) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(v, dtype=np.uint32))


def _c64(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=np.uint64))


class OracleContext:
    """NTT tables for a list of primes at ring degree ``2**logn``."""

    def __init__(self, logn: int, moduli):
        self.logn = int(logn)
        self.n = 1 << self.logn
        self.moduli = [int(m) for m in moduli]
        arr = np.asarray(self.moduli, dtype=np.uint64)
        self._h = lib().orc_ctx_create(self.logn, _p64(arr), len(self.moduli))
        if not self._h:
            raise ValueError("oracle: a modulus is not an NTT-friendly prime below 2^62")

    def __del__(self):
        if getattr(self, "_h", None):
            lib().orc_ctx_destroy(self._h)
            self._h = None

    def root(self, k: int) -> int:
        return int(lib().orc_ctx_root(self._h, k))

    def twiddle(self, k: int, i: int) -> int:
        return int(lib().orc_ctx_twiddle(self._h, k, i))

    # ---- NTT over a stack of limbs: x is [count, n], limb i uses prime prime_idx[i]
    def ntt_forward(self, x, prime_idx) -> np.ndarray:
        y = _c64(x).copy().reshape(-1, self.n)
        pi = _idx(prime_idx)
        assert len(pi) == y.shape[0]
        lib().orc_ntt_forward_batch(self._h, _p64(y), _p32(pi), len(pi))
        return y

    def ntt_inverse(self, x, prime_idx) -> np.ndarray:
        y = _c64(x).copy().reshape(-1, self.n)
        pi = _idx(prime_idx)
        assert len(pi) == y.shape[0]
        lib().orc_ntt_inverse_batch(self._h, _p64(y), _p32(pi), len(pi))
        return y

    def sud(self, k: int, in1, in2_coeff, factor: int) -> np.ndarray:
        a, b = _c64(in1), _c64(in2_coeff)
        out = np.empty(self.n, dtype=np.uint64)
        lib().orc_sud(self._h, k, _p64(a), _p64(b), int(factor), _p64(out))
        return out

    def moddown(self, bconv_mode, round_mode, q_idx, p_idx, tq, tp) -> np.ndarray:
        qi, pi = _idx(q_idx), _idx(p_idx)
        tq, tp = _c64(tq), _c64(tp)
        out = np.empty((len(qi), self.n), dtype=np.uint64)
        lib().orc_moddown(self._h, bconv_mode, round_mode, len(qi), _p32(qi), len(pi), _p32(pi),
                          _p64(tq), _p64(tp), _p64(out))
        return out

    def keyswitch(self, bconv_mode, round_mode, q_idx, p_idx, dnum, cpoly, evk):
        qi, pi = _idx(q_idx), _idx(p_idx)
        cpoly, evk = _c64(cpoly), _c64(evk)
        L, K = len(qi), len(pi)
        assert cpoly.size == L * self.n and evk.size == dnum * 2 * (L + K) * self.n
        o0 = np.empty((L, self.n), dtype=np.uint64)
        o1 = np.empty((L, self.n), dtype=np.uint64)
        lib().orc_keyswitch(self._h, bconv_mode, round_mode, L, _p32(qi), K, _p32(pi), dnum,
                            _p64(cpoly), _p64(evk), _p64(o0), _p64(o1))
        return o0, o1

    def moddown_rescale(self, bconv_mode, round_mode, q_idx, p_idx, r, t) -> np.ndarray:
        """ModDown of t ([L+K][N], extended basis) with r rescale levels in the same division: [L-r][N]."""
        qi, pi = _idx(q_idx), _idx(p_idx)
        t = _c64(t)
        out = np.empty((len(qi) - r, self.n), dtype=np.uint64)
        lib().orc_moddown_rescale(self._h, bconv_mode, round_mode, len(qi), _p32(qi), len(pi), _p32(pi), int(r),
                                  _p64(t), _p64(out))
        return out

    def keyswitch_rescale(self, bconv_mode, round_mode, q_idx, p_idx, dnum, r, cpoly, evk, add0=None, add1=None):
        """Key switch with the PMU pre-additions and r rescale levels inside the ModDown: two [L-r][N]."""
        qi, pi = _idx(q_idx), _idx(p_idx)
        cpoly, evk = _c64(cpoly), _c64(evk)
        a0 = _c64(add0) if add0 is not None else None
        a1 = _c64(add1) if add1 is not None else None
        o0 = np.empty((len(qi) - r, self.n), dtype=np.uint64)
        o1 = np.empty((len(qi) - r, self.n), dtype=np.uint64)
        lib().orc_keyswitch_rescale(self._h, bconv_mode, round_mode, len(qi), _p32(qi), len(pi), _p32(pi), dnum,
                                    int(r), _p64(cpoly), _p64(evk), _p64(a0) if a0 is not None else None,
                                    _p64(a1) if a1 is not None else None, _p64(o0), _p64(o1))
        return o0, o1

    def hmult_relin_fused(self, bconv_mode, round_mode, q_idx, p_idx, dnum, a0, a1, b0, b1, evk):
        """HMult + relinearize + rescale with one division (the rescale folded into the ModDown)."""
        qi, pi = _idx(q_idx), _idx(p_idx)
        a0, a1, b0, b1, evk = map(_c64, (a0, a1, b0, b1, evk))
        o0 = np.empty((len(qi) - 1, self.n), dtype=np.uint64)
        o1 = np.empty((len(qi) - 1, self.n), dtype=np.uint64)
        lib().orc_hmult_relin_fused(self._h, bconv_mode, round_mode, len(qi), _p32(qi), len(pi), _p32(pi), dnum,
                                    _p64(a0), _p64(a1), _p64(b0), _p64(b1), _p64(evk), _p64(o0), _p64(o1))
        return o0, o1

    def bsgs(self, bconv_mode, round_mode, q_idx, p_idx, dnum, r, baby, pts, present, elts, keys):
        """Baby-step / giant-step multiply-accumulate with the giant-step key switches accumulated in the
        extended basis and one ModDown (r rescale levels).  baby [g][2][L][N], pts [n_giant][g][L][N],
        present [n_giant][g], elts [n_giant] (1 = no rotation), keys [n_giant][dnum][2][L+K][N]."""
        qi, pi = _idx(q_idx), _idx(p_idx)
        baby, pts, keys = _c64(baby), _c64(pts), _c64(keys)
        g, n_giant = baby.shape[0], pts.shape[0]
        pres = np.ascontiguousarray(np.asarray(present, dtype=np.uint8).reshape(n_giant * g))
        el = _idx(elts)
        o0 = np.empty((len(qi) - r, self.n), dtype=np.uint64)
        o1 = np.empty((len(qi) - r, self.n), dtype=np.uint64)
        lib().orc_bsgs(self._h, bconv_mode, round_mode, len(qi), _p32(qi), len(pi), _p32(pi), dnum, g, n_giant, int(r),
                       _p64(baby), _p64(pts), pres.ctypes.data_as(C.POINTER(C.c_uint8)), _p32(el), _p64(keys),
                       _p64(o0), _p64(o1))
        return o0, o1

    def rescale(self, round_mode, q_idx, cpoly) -> np.ndarray:
        qi = _idx(q_idx)
        cpoly = _c64(cpoly)
        out = np.empty((len(qi) - 1, self.n), dtype=np.uint64)
        lib().orc_rescale(self._h, round_mode, len(qi), _p32(qi), _p64(cpoly), _p64(out))
        return out

    def mod_raise(self, bconv_mode, round_mode, q_idx, p_idx, base0, base1, c0, c1, evk):
        """Bootstrap ModRaise: (c0, c1) with limbs (base0, base1) -> two polynomials of len(q_idx) - 1 limbs."""
        qi, pi = _idx(q_idx), _idx(p_idx)
        c0, c1, evk = _c64(c0), _c64(c1), _c64(evk)
        o0 = np.empty((len(qi) - 1, self.n), dtype=np.uint64)
        o1 = np.empty((len(qi) - 1, self.n), dtype=np.uint64)
        lib().orc_mod_raise(self._h, bconv_mode, round_mode, len(qi), _p32(qi), len(pi), _p32(pi), int(base0),
                            int(base1), _p64(c0), _p64(c1), _p64(evk), _p64(o0), _p64(o1))
        return o0, o1

    def double_rescale(self, q_idx, cpoly) -> np.ndarray:
        """Drops the last two limbs at once (floor division by their product)."""
        qi = _idx(q_idx)
        cpoly = _c64(cpoly)
        out = np.empty((len(qi) - 2, self.n), dtype=np.uint64)
        lib().orc_double_rescale(self._h, len(qi), _p32(qi), _p64(cpoly), _p64(out))
        return out

    def hrot(self, bconv_mode, round_mode, q_idx, p_idx, dnum, elt, c0, c1, evk):
        qi, pi = _idx(q_idx), _idx(p_idx)
        c0, c1, evk = _c64(c0), _c64(c1), _c64(evk)
        L, K = len(qi), len(pi)
        o0 = np.empty((L, self.n), dtype=np.uint64)
        o1 = np.empty((L, self.n), dtype=np.uint64)
        lib().orc_hrot(self._h, bconv_mode, round_mode, L, _p32(qi), K, _p32(pi), dnum, int(elt),
                       _p64(c0), _p64(c1), _p64(evk), _p64(o0), _p64(o1))
        return o0, o1

    def hmult_relin(self, bconv_mode, round_mode, do_rescale, q_idx, p_idx, dnum, a0, a1, b0, b1, evk):
        qi, pi = _idx(q_idx), _idx(p_idx)
        a0, a1, b0, b1, evk = map(_c64, (a0, a1, b0, b1, evk))
        L, K = len(qi), len(pi)
        lo = L - 1 if do_rescale else L
        o0 = np.empty((lo, self.n), dtype=np.uint64)
        o1 = np.empty((lo, self.n), dtype=np.uint64)
        lib().orc_hmult_relin(self._h, bconv_mode, round_mode, int(bool(do_rescale)), L, _p32(qi), K,
                              _p32(pi), dnum, _p64(a0), _p64(a1), _p64(b0), _p64(b1), _p64(evk),
                              _p64(o0), _p64(o1))
        return o0, o1


def bconv(mode, in_mod, x, out_mod) -> np.ndarray:
    """x: [I, n] residues mod in_mod -> [O, n] residues mod out_mod."""
    x = _c64(x)
    im, om = _c64(in_mod), _c64(out_mod)
    n = x.shape[-1]
    out = np.empty((len(om), n), dtype=np.uint64)
    lib().orc_bconv(mode, n, len(im), _p64(im), _p64(x), len(om), _p64(om), _p64(out))
    return out


def resolve2(m0: int, m1: int, x0, x1):
    """Exact CRT of two limbs -> (lo, hi) 64-bit words of the integer in [0, m0*m1)."""
    x0, x1 = _c64(x0), _c64(x1)
    lo, hi = np.empty_like(x0), np.empty_like(x0)
    lib().orc_resolve2(m0, m1, x0.size, _p64(x0), _p64(x1), _p64(lo), _p64(hi))
    return lo, hi


def mod2(q: int, lo, hi) -> np.ndarray:
    lo, hi = _c64(lo), _c64(hi)
    out = np.empty_like(lo)
    lib().orc_mod2(q, lo.size, _p64(lo), _p64(hi), _p64(out))
    return out


def galois_elt_from_step(step: int, logn: int) -> int:
    return int(lib().orc_galois_elt_from_step(step, logn))


def galois_table_ntt(elt: int, logn: int) -> np.ndarray:
    t = np.empty(1 << logn, dtype=np.uint32)
    lib().orc_galois_table_ntt(elt, logn, _p32(t))
    return t


def apply_galois_ntt(elt: int, logn: int, x) -> np.ndarray:
    x = _c64(x)
    out = np.empty_like(x)
    lib().orc_apply_galois_ntt(elt, logn, _p64(x), _p64(out))
    return out


def apply_galois_coeff(elt: int, logn: int, q: int, x) -> np.ndarray:
    x = _c64(x)
    out = np.empty_like(x)
    lib().orc_apply_galois_coeff(elt, logn, q, _p64(x), _p64(out))
    return out


def negacyclic_mul_schoolbook(q: int, a, b) -> np.ndarray:
    a, b = _c64(a), _c64(b)
    out = np.empty_like(a)
    lib().orc_negacyclic_mul_schoolbook(q, a.size, _p64(a), _p64(b), _p64(out))
    return out


def ew(op: str, q: int, *arrays, scalar: int | None = None) -> np.ndarray:
    """Element-wise add/sub/neg/mul/mad/pmu on one limb."""
    arrs = [_c64(a) for a in arrays]
    out = np.empty_like(arrs[0])
    n = arrs[0].size
    f = getattr(lib(), "orc_ew_" + op)
    if op == "pmu":
        f(q, n, _p64(arrs[0]), _p64(arrs[1]), int(scalar), _p64(out))
    else:
        f(q, n, *[_p64(a) for a in arrs], _p64(out))
    return out


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_num_threads(n: int) -> None:
    """Number of OpenMP threads of the following calls (launchers such as torchrun export
    OMP_NUM_THREADS=1 to their children)."""
    lib().orc_set_num_threads(int(n))
