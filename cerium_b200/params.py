"""Parameter sets: NTT-friendly prime search and the benchmark configurations.

The reference fixes 64 primes of 28 bits in ``examples/primes.py:16`` and takes
the key-switching extension primes from the top of that list
(``cerium/runtime/io/ckks-encryptor.cpp:550-555``).  The 64-bit configurations
use primes found by a deterministic downward search, so every run (and the CPU
oracle) sees the same moduli without shipping a table.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List

_MR_BASES = (2, 3, 5, 7, 11, 13, 17, 19, 23, 29, 31, 37)


def is_prime(n: int) -> bool:
    """Deterministic Miller-Rabin for n < 2^64."""
    if n < 2:
        return False
    for p in _MR_BASES:
        if n % p == 0:
            return n == p
    d, s = n - 1, 0
    while d % 2 == 0:
        d //= 2
        s += 1
    for a in _MR_BASES:
        x = pow(a, d, n)
        if x in (1, n - 1):
            continue
        for _ in range(s - 1):
            x = x * x % n
            if x == n - 1:
                break
        else:
            return False
    return True


def ntt_primes_below(bits: int, count: int, logn: int, exclude=()) -> List[int]:
    """First ``count`` primes q = 1 (mod 2^(logn+1)) met searching downward from 2^bits."""
    step = 1 << (logn + 1)
    q = (1 << bits) + 1 - step
    out: List[int] = []
    seen = set(exclude)
    while len(out) < count:
        if q < (1 << (bits - 1)):
            raise ValueError("ran out of %d-bit NTT primes" % bits)
        if q not in seen and is_prime(q):
            out.append(q)
        q -= step
    return out


def ntt_primes_above(lo: int, count: int, logn: int) -> List[int]:
    """First ``count`` primes q = 1 (mod 2^(logn+1)) with q > lo (ascending)."""
    step = 1 << (logn + 1)
    q = (lo // step) * step + 1
    if q <= lo:
        q += step
    out: List[int] = []
    while len(out) < count:
        if is_prime(q):
            out.append(q)
        q += step
    return out


def reference_primes_28bit(count: int = 64, logn: int = 16) -> List[int]:
    """The 28-bit prime chain of the reference's examples: the ``count`` NTT-friendly
    primes (q = 1 mod 2^17) above 204 865 536 in ascending order.  For
    count=64, logn=16 the first is 204865537 and the last 268042241, the end points
    of ``examples/primes.py:16``."""
    return ntt_primes_above(204865536, count, logn)


@dataclass
class CkksParams:
    """One RNS-CKKS parameter set.

    ``moduli`` lists every prime of the context; a ciphertext at level ``L`` uses
    primes ``0..L-1`` and the ``K`` extension primes are the last ``K`` entries
    (taken from the top like the reference does).  ``dnum`` digits are formed by
    stride: limb ``i`` belongs to digit ``i % dnum``
    (``cerium/compiler/backend/compiler_keyswitch.cc:68-99``).
    """

    logn: int
    word_bits: int
    moduli: List[int]
    L: int
    K: int
    dnum: int
    name: str = ""
    q_idx: List[int] = field(default_factory=list)
    p_idx: List[int] = field(default_factory=list)

    def __post_init__(self):
        if not self.q_idx:
            self.q_idx = list(range(self.L))
        if not self.p_idx:
            self.p_idx = [len(self.moduli) - 1 - k for k in range(self.K)]
        alpha = -(-self.L // self.dnum)
        if alpha > self.K:
            raise ValueError("digit size %d exceeds the %d extension primes" % (alpha, self.K))

    @property
    def n(self) -> int:
        return 1 << self.logn

    @property
    def alpha(self) -> int:
        return -(-self.L // self.dnum)


def config_hrot(logn: int = 16, L: int = 35, K: int = 5, dnum: int = 7) -> CkksParams:
    """HRot benchmark set: L primes of 50 bits + K extension primes of 60 bits."""
    q = ntt_primes_below(50, L, logn)
    p = ntt_primes_below(60, K, logn)
    return CkksParams(logn, 64, q + p[::-1], L, K, dnum, name="hrot_L%d_K%d_dnum%d" % (L, K, dnum))


def config_hmult(logn: int = 16, L: int = 24) -> CkksParams:
    """HMult+relinearize+rescale set: first prime 60 bits, the rest 50 bits, one
    60-bit extension prime, one digit per limb (dnum = L)."""
    p60 = ntt_primes_below(60, 2, logn)
    q = [p60[1]] + ntt_primes_below(50, L - 1, logn)
    return CkksParams(logn, 64, q + [p60[0]], L, 1, L, name="hmult_L%d_dnum%d" % (L, L))


def config_ntt(logn: int = 16, limbs: int = 48) -> List[int]:
    """Standalone NTT benchmark moduli: ``limbs`` primes of 50 bits."""
    return ntt_primes_below(50, limbs, logn)


def config_ref28(logn: int = 16, L: int = 35, K: int = 5, dnum: int = 7, total: int = 64) -> CkksParams:
    """32-bit twin on the reference's 28-bit prime chain."""
    return CkksParams(logn, 32, reference_primes_28bit(total, logn), L, K, dnum,
                      name="ref28_L%d_K%d_dnum%d" % (L, K, dnum))
