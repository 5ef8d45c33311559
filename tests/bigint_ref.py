"""Big-integer (Python int) definitions used to pin the CPU oracle.

Everything here is written directly from the mathematical definition
(evaluation at odd powers of psi, CRT reconstruction, integer division) and
shares no code with the oracle or the CUDA kernels.
"""
from __future__ import annotations

import numpy as np


def brev(x: int, bits: int) -> int:
    r = 0
    for _ in range(bits):
        r = (r << 1) | (x & 1)
        x >>= 1
    return r


def ntt_by_definition(x, q: int, psi: int, logn: int):
    """out[i] = sum_j x[j] * psi^((2*brev(i)+1) * j) mod q  (bit-reversed output order)."""
    n = 1 << logn
    out = []
    for i in range(n):
        e = 2 * brev(i, logn) + 1
        w = pow(psi, e, q)
        acc, p = 0, 1
        for j in range(n):
            acc = (acc + int(x[j]) * p) % q
            p = p * w % q
        out.append(acc)
    return np.array(out, dtype=np.uint64)


def crt_reconstruct(residues, moduli) -> int:
    """Integer in [0, prod moduli) with the given residues."""
    Q = 1
    for m in moduli:
        Q *= m
    x = 0
    for r, m in zip(residues, moduli):
        Qi = Q // m
        x += int(r) * Qi * pow(Qi, -1, m)
    return x % Q


def bconv_lazy(residues, in_mod, out_mod):
    """Cerium's lazy conversion: sum_i x_i * [Qhat_i^-1]_{q_i} * Qhat_i  (no reduction by q_i)."""
    Q = 1
    for m in in_mod:
        Q *= m
    s = 0
    for r, m in zip(residues, in_mod):
        Qi = Q // m
        s += int(r) * pow(Qi, -1, m) * Qi
    return [s % p for p in out_mod]


def bconv_exact(residues, in_mod, out_mod):
    """Textbook fast base conversion: sum_i [x_i * Qhat_i^-1]_{q_i} * Qhat_i."""
    Q = 1
    for m in in_mod:
        Q *= m
    s = 0
    for r, m in zip(residues, in_mod):
        Qi = Q // m
        s += (int(r) * pow(Qi, -1, m) % m) * Qi
    return [s % p for p in out_mod]
