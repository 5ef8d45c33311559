"""The bootstrap operator list of cerium_b200/bootstrap.py evaluated on the CPU oracle: same interface as
GpuEvaluator, numpy arrays instead of device tensors, every step the oracle's restatement of the
reference lowering.  TEST INFRASTRUCTURE (it imports the oracle)."""
from __future__ import annotations

from typing import List, Sequence

import numpy as np

import oracle
from cerium_b200.bootstrap import Ct

LOGN = 16
N = 1 << LOGN


class OracleEvaluator:
    def __init__(self, material, bconv_mode, round_mode):
        self.m = material
        self.bm, self.rm = bconv_mode, round_mode
        self.orc = oracle.OracleContext(LOGN, material.moduli)

    def at_level(self, a: Ct, level: int) -> Ct:
        return Ct(a.c0[:level], a.c1[:level], level)

    def mod_raise(self, ct2) -> Ct:
        m = self.m
        o0, o1 = self.orc.mod_raise(self.bm, self.rm, m.q_idx[:m.top + 1], m.p_idx, m.q_idx[0], m.q_idx[1], ct2[0], ct2[1],
                                    m.lift_key)
        return Ct(o0, o1, m.top)

    def _ew2(self, op, a, b, L):
        idx = self.m.q_idx[:L]
        f = lambda x, y: np.stack([oracle.ew(op, self.m.moduli[p], x[i], y[i]) for i, p in enumerate(idx)])  # noqa: E731
        return Ct(f(a.c0, b.c0), f(a.c1, b.c1), L)

    def add(self, a, b):
        return self._ew2("add", a, b, min(a.level, b.level))

    def sub(self, a, b):
        return self._ew2("sub", a, b, min(a.level, b.level))

    def _scale(self, a, scalars):
        L = a.level
        idx = self.m.q_idx[:L]
        f = lambda x: np.stack([oracle.ew("mul", self.m.moduli[p], x[i], np.full(N, int(scalars[i]) % self.m.moduli[p], dtype=np.uint64))  # noqa: E731
                                for i, p in enumerate(idx)])
        return Ct(f(a.c0), f(a.c1), L)

    def mul_small(self, a, k: int):
        return self._scale(a, [k] * a.level)

    def mul_scalar(self, a, scalars: Sequence[int], same_level: bool = False):
        prod = self._scale(a, scalars)
        return prod if same_level else self.rescale(prod)

    def add_const(self, a, c: int):
        L = a.level
        idx = self.m.q_idx[:L]
        c0 = np.stack([oracle.ew("add", self.m.moduli[p], a.c0[i], np.full(N, c % self.m.moduli[p], dtype=np.uint64))
                       for i, p in enumerate(idx)])
        return Ct(c0, a.c1[:L], L)

    def pt_mac(self, sources, names, level):
        idx = self.m.q_idx[:level]
        outs = []
        for row in names:
            acc = [np.zeros((level, N), dtype=np.uint64), np.zeros((level, N), dtype=np.uint64)]
            for src, name in zip(sources, row):
                pt = self.m.plaintext(name, level)
                for k, poly in enumerate((src.c0, src.c1)):
                    acc[k] = np.stack([oracle.ew("mad", self.m.moduli[p], poly[i], pt[i], acc[k][i]) for i, p in enumerate(idx)])
            outs.append(Ct(acc[0], acc[1], level))
        return outs

    def rescale(self, a: Ct) -> Ct:
        L = a.level
        idx = self.m.q_idx[:L]
        return Ct(self.orc.rescale(self.rm, idx, a.c0[:L]), self.orc.rescale(self.rm, idx, a.c1[:L]), L - 1)

    def scalars(self, what, level) -> List[int]:
        return self.m.scalars(what, level)

    def conjugate(self, ct: Ct) -> Ct:
        m, L = self.m, ct.level
        o0, o1 = self.orc.hrot(self.bm, self.rm, m.q_idx[:L], m.p_idx, m.dnum_at(L), 2 * N - 1, ct.c0[:L], ct.c1[:L], m.conj_key(L))
        return Ct(o0, o1, L)

    def hmult(self, a: Ct, b: Ct) -> Ct:
        m = self.m
        L = min(a.level, b.level)
        o0, o1 = self.orc.hmult_relin_fused(self.bm, self.rm, m.q_idx[:L], m.p_idx, m.dnum_at(L), a.c0[:L], a.c1[:L], b.c0[:L],
                                            b.c1[:L], m.relin_key(L))
        return Ct(o0, o1, L - 1)

    def bsgs(self, ct: Ct, stage) -> Ct:
        m, L = self.m, ct.level
        st = m.stage(stage, L)
        q_idx, dnum = m.q_idx[:L], m.dnum_at(L)
        c0, c1 = ct.c0[:L], ct.c1[:L]
        baby = [np.stack([c0, c1])]
        for j in range(1, st.g):
            k0, k1 = self.orc.keyswitch(self.bm, self.rm, q_idx, m.p_idx, dnum, c1, st.baby_keys[j])
            k0 = np.stack([oracle.ew("add", m.moduli[p], k0[i], c0[i]) for i, p in enumerate(q_idx)])
            e = st.baby_elts[j]
            baby.append(np.stack([np.stack([oracle.apply_galois_ntt(e, LOGN, k[i]) for i in range(L)]) for k in (k0, k1)]))
        present = np.array([0 if p is None else 1 for p in st.pts], dtype=np.uint8).reshape(st.n_giant, st.g)
        zero = np.zeros((L, N), dtype=np.uint64)
        pts = np.stack([zero if p is None else p for p in st.pts]).reshape(st.n_giant, st.g, L, N)
        keys = np.stack(st.giant_keys)
        o0, o1 = self.orc.bsgs(self.bm, self.rm, q_idx, m.p_idx, dnum, 1, np.stack(baby), pts, present, st.giant_elts, keys)
        return Ct(o0, o1, L - 1)
