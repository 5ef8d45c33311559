"""CKKS bootstrapping as an operator list over the library's C ABI.

The reference's bootstrap is a DSL program (``benchmarks/bootstrap_32K/bootstrap.py:299-358``):
ModRaise, CoeffToSlot as a chain of BSGS multiply-accumulates with the rescale folded into each
(``:319-337``), EvalMod as a Chebyshev polynomial of the scaled sine followed by double-angle
iterations (``:31-117, 140-144``), SlotToCoeff as a second chain of BSGS stages (``:343-356``).  This
module is that program's STRUCTURE for the parameterisation the benchmark names - three BSGS levels
each way, a degree-63 Chebyshev polynomial evaluated baby-step / giant-step over T_1..T_8, T_16, T_32,
two double-angle steps - written once against a small evaluator interface, so that the same list
runs on the GPU (``GpuEvaluator``, every step one call of the C ABI: ``cerium_mod_raise``,
``cerium_bsgs_apply``, ``cerium_hrot``, ``cerium_hmult`` with the rescale folded into the ModDown,
``cerium_ewise``) and on the CPU checker in the tests.

What it is not: a numerically meaningful bootstrap.  The diagonals of the linear transforms and the
polynomial's coefficients are SEEDED RANDOM residues of the right shapes (there is no encoder in
the library, and the benchmark's inputs are synthetic), so decrypted slots mean nothing and no
precision figure comes out of it; the integer results are compared with the checker bit for bit,
and the latency is that of the real operator sequence: the same kernels on the same limb counts,
the same number of key switches, plaintext products and rescales, level by level.
"""
from __future__ import annotations

import zlib
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

BABY = 8          # baby steps of a linear-transform stage and of the polynomial
GIANT = 8         # giant steps of a linear-transform stage
STAGES = 3        # BSGS levels of CoeffToSlot and of SlotToCoeff
DOUBLE_ANGLE = 2  # double-angle iterations after the polynomial


@dataclass
class Ct:
    """A ciphertext at `level` limbs: (c0, c1) buffers of at least `level` limbs each."""
    c0: object
    c1: object
    level: int


@dataclass
class BootstrapShape:
    top: int                 # limbs right after ModRaise (the lifted plan has top + 1 Q primes)
    stages: int = STAGES
    baby: int = BABY
    giant: int = GIANT
    double_angle: int = DOUBLE_ANGLE

    @property
    def levels_used(self) -> int:
        # C2S stages; polynomial: 3 levels to T_8, one for the scalar products, 3 giant-step products;
        # double angles; S2C stages
        return self.stages + 3 + 1 + 3 + self.double_angle + self.stages

    def check(self):
        if self.top - self.levels_used < 1:
            raise ValueError("bootstrap needs %d levels below the raised ciphertext, only %d there"
                             % (self.levels_used, self.top - 1))


class OpCounter:
    """Counts what a run issues (for the benchmark's launch / byte accounting)."""

    def __init__(self):
        self.n: Dict[str, int] = {}

    def add(self, what: str, k: int = 1):
        self.n[what] = self.n.get(what, 0) + k


def bootstrap(ev, shape: BootstrapShape, ct_in, rng_seed: int = 0xB0075) -> Ct:
    """Runs the operator list on evaluator `ev`; `ct_in` is whatever ev.mod_raise takes (a two-limb
    ciphertext).  Every random choice (which diagonals are absent, scalar coefficients) comes from
    `rng_seed`, so two evaluators given the same seed and the same material compute the same thing."""
    shape.check()
    rng = np.random.default_rng(rng_seed)
    ct = ev.mod_raise(ct_in)                                   # level = shape.top
    # --- CoeffToSlot: `stages` BSGS multiply-accumulates, each dividing one level away
    for s in range(shape.stages):
        ct = ev.bsgs(ct, ("c2s", s))
    # real and imaginary parts: ct +- conj(ct) (the factor 1/2 and i sit in the next plaintexts)
    cj = ev.conjugate(ct)
    parts = [ev.add(ct, cj), ev.sub(ct, cj)]
    outs = []
    for part in parts:
        outs.append(_eval_mod(ev, shape, part, rng))
    # recombine: real + i * imag (the multiplication by i is a plaintext scalar per limb)
    ct = ev.add(outs[0], ev.mul_scalar(outs[1], ev.scalars("i", outs[1].level), same_level=True))
    # --- SlotToCoeff
    for s in range(shape.stages):
        ct = ev.bsgs(ct, ("s2c", s))
    return ct


def _eval_mod(ev, shape: BootstrapShape, x: Ct, rng) -> Ct:
    """Chebyshev polynomial of degree 63 by baby steps T_1..T_8 and giant steps T_8, T_16, T_32
    (Paterson-Stockmeyer over the Chebyshev basis), then `double_angle` squarings."""
    def cheb_double(t):        # T_2k = 2 T_k^2 - 1
        return ev.add_const(ev.mul_small(ev.hmult(t, t), 2), -1)

    def cheb_prod(a, b, c):    # T_{i+j} = 2 T_i T_j - T_{|i-j|}
        return ev.sub(ev.mul_small(ev.hmult(a, b), 2), c)

    T = {1: x}
    T[2] = cheb_double(T[1])
    T[3] = cheb_prod(T[2], T[1], T[1])
    T[4] = cheb_double(T[2])
    T[5] = cheb_prod(T[3], T[2], T[1])
    T[6] = cheb_double(T[3])
    T[7] = cheb_prod(T[4], T[3], T[1])
    T[8] = cheb_double(T[4])
    T[16] = cheb_double(T[8])
    T[32] = cheb_double(T[16])
    # baby polynomials q_j = sum_i c[j][i] T_i + c[j][0], j = 0..7, at the level of T_7: one
    # multiply-accumulate pass over the seven T_i for all eight polynomials (the coefficients enter as
    # plaintexts, the general case of the constants a sine approximation has), one rescale each
    lvl = min(T[i].level for i in range(1, 8))
    sums = ev.pt_mac([ev.at_level(T[i], lvl) for i in range(1, 8)], [[("coef", j, i) for i in range(1, 8)] for j in range(8)], lvl)
    q = [ev.add_const(ev.rescale(t), int(rng.integers(1, 1000))) for t in sums]
    # combine over the giant steps: pairs with T_8, then T_16, then T_32
    for giant in (8, 16, 32):
        nxt = []
        for k in range(0, len(q), 2):
            nxt.append(ev.add(ev.hmult(q[k + 1], T[giant]), q[k]))
        q = nxt
    r = q[0]
    for _ in range(shape.double_angle):
        r = cheb_double(r)
    return r


# ---------------------------------------------------------------------------------------
# the GPU evaluator: every method is one (or a few) calls of the C ABI
# ---------------------------------------------------------------------------------------

class GpuEvaluator:
    """Holds the per-level key-switching plans, keys and plaintexts (device tensors) and runs the
    operators through the library.  `material` is a BootstrapMaterial (below) already on the device."""

    def __init__(self, torch, capi, ctx, material, bconv_mode, round_mode):
        self.torch, self.capi, self.ctx, self.m = torch, capi, ctx, material
        self.bm, self.rm = bconv_mode, round_mode
        self.n = ctx.n
        self.plans: Dict[int, object] = {}
        self.work: Dict[Tuple[int, int, int], object] = {}
        self.count = OpCounter()
        self.stream = 0
        self.ones = None
        self.lift = capi.KeySwitch(ctx, material.q_idx[:material.top + 1], material.p_idx, 1, bconv_mode, round_mode, lifted=True)

    def plan(self, level: int):
        ks = self.plans.get(level)
        if ks is None:
            m = self.m
            ks = self.capi.KeySwitch(self.ctx, m.q_idx[:level], m.p_idx, m.dnum_at(level), self.bm, self.rm)
            self.plans[level] = ks
        return ks

    def _new(self, level: int) -> Ct:
        t = self.torch
        return Ct(t.empty((level, self.n), dtype=t.int64, device="cuda"), t.empty((level, self.n), dtype=t.int64, device="cuda"), level)

    def at_level(self, a: Ct, level: int) -> Ct:
        return Ct(a.c0, a.c1, level)          # dropping limbs is free: the first `level` limbs are the ciphertext

    def mod_raise(self, ct2) -> Ct:
        m = self.m
        out = self._new(m.top)
        self.lift.mod_raise(out.c0.data_ptr(), out.c1.data_ptr(), ct2[0].data_ptr(), ct2[1].data_ptr(), m.q_idx[0], m.q_idx[1],
                            m.lift_key.data_ptr(), self.stream)
        self.count.add("mod_raise")
        return out

    def bsgs(self, ct: Ct, stage) -> Ct:
        m = self.m
        L = ct.level
        ks = self.plan(L)
        st = m.stage(stage, L)
        key = (L, st.g, st.n_giant)
        work = self.work.get(key)
        if work is None:
            work = self.torch.empty((ks.bsgs_work_limbs(st.g, st.n_giant), self.n), dtype=self.torch.int64, device="cuda")
            self.work[key] = work
        out = self._new(L - 1)
        ks.bsgs_apply(out.c0.data_ptr(), out.c1.data_ptr(), ct.c0.data_ptr(), ct.c1.data_ptr(), st.g, st.n_giant,
                      [p.data_ptr() if p is not None else 0 for p in st.pts],
                      [k.data_ptr() if k is not None else 0 for k in st.baby_keys], st.baby_elts,
                      [k.data_ptr() if k is not None else 0 for k in st.giant_keys], st.giant_elts, 1, work.data_ptr(), self.stream)
        self.count.add("bsgs")
        self.count.add("keyswitch", (st.g - 1) + sum(1 for e in st.giant_elts if e != 1))
        return out

    def conjugate(self, ct: Ct) -> Ct:
        L = ct.level
        out = self._new(L)
        self.plan(L).hrot(out.c0.data_ptr(), out.c1.data_ptr(), ct.c0.data_ptr(), ct.c1.data_ptr(), self.m.conj_key(L).data_ptr(),
                          2 * self.n - 1, self.stream)
        self.count.add("keyswitch")
        return out

    def hmult(self, a: Ct, b: Ct) -> Ct:
        L = min(a.level, b.level)
        out = self._new(L - 1)
        self.plan(L).hmult(out.c0.data_ptr(), out.c1.data_ptr(), a.c0.data_ptr(), a.c1.data_ptr(), b.c0.data_ptr(), b.c1.data_ptr(),
                           self.m.relin_key(L).data_ptr(), 2, self.stream)
        self.count.add("hmult")
        self.count.add("keyswitch")
        return out

    def _ew(self, op, a: Ct, b: Optional[Ct], scalars=None, level=None) -> Ct:
        L = level or (min(a.level, b.level) if b is not None else a.level)
        out = self._new(L)
        idx = self.m.q_idx[:L]
        for k in ("c0", "c1"):
            self.ctx.ewise(op, getattr(out, k).data_ptr(), getattr(a, k).data_ptr(), idx,
                           b=getattr(b, k).data_ptr() if b is not None else 0, scalars=scalars, stream=self.stream)
        self.count.add("ewise", 2)
        return out

    def add(self, a, b):
        return self._ew(self.capi.EW_ADD, a, b)

    def sub(self, a, b):
        return self._ew(self.capi.EW_SUB, a, b)

    def mul_small(self, a, k: int):
        return self._ew(self.capi.EW_MUL_SCALAR, a, None, scalars=[k] * a.level)

    def mul_scalar(self, a, scalars: Sequence[int], same_level: bool = False):
        """Plaintext scalar per limb; consumes a level like every plaintext product unless same_level."""
        prod = self._ew(self.capi.EW_MUL_SCALAR, a, None, scalars=list(scalars))
        return prod if same_level else self.rescale(prod)

    def add_const(self, a, c: int):
        """Adds the constant polynomial c (its NTT form is c in every position) to c0."""
        L = a.level
        if self.ones is None or self.ones.shape[0] < L:
            self.ones = self.torch.ones((self.m.top, self.n), dtype=self.torch.int64, device="cuda")
        out = Ct(self.torch.empty_like(a.c0[:L]), a.c1, L)
        mods = self.m.moduli
        self.ctx.ewise(self.capi.EW_PMU, out.c0.data_ptr(), a.c0.data_ptr(), self.m.q_idx[:L], b=self.ones.data_ptr(),
                       scalars=[c % mods[p] for p in self.m.q_idx[:L]], stream=self.stream)
        self.count.add("ewise")
        return out

    def pt_mac(self, sources: List[Ct], names, level: int) -> List[Ct]:
        outs = [self._new(level) for _ in names]
        pts = [self.m.plaintext(n, level).data_ptr() for row in names for n in row]
        self.ctx.plaintext_mac([o.c0.data_ptr() for o in outs], [o.c1.data_ptr() for o in outs],
                               [s.c0.data_ptr() for s in sources], [s.c1.data_ptr() for s in sources], pts,
                               self.m.q_idx[:level], self.stream)
        self.count.add("pt_mac")
        return outs

    def rescale(self, a: Ct) -> Ct:
        L = a.level
        t = self.torch
        both = t.stack([a.c0[:L], a.c1[:L]])
        out = t.empty((2, L - 1, self.n), dtype=t.int64, device="cuda")
        scratch = t.empty((2, self.n), dtype=t.int64, device="cuda")
        self.ctx.rescale(out.data_ptr(), both.data_ptr(), self.m.q_idx[:L], 2, scratch.data_ptr(), self.rm, self.stream)
        self.count.add("rescale")
        return Ct(out[0], out[1], L - 1)

    def scalars(self, what, level: int) -> List[int]:
        return self.m.scalars(what, level)


# ---------------------------------------------------------------------------------------
# seeded material (shapes only: random residues stand in for keys, diagonals and coefficients)
# ---------------------------------------------------------------------------------------

@dataclass
class Stage:
    g: int
    n_giant: int
    pts: List[object]
    baby_keys: List[object]
    baby_elts: List[int]
    giant_keys: List[object]
    giant_elts: List[int]


class BootstrapMaterial:
    """Keys, diagonals and scalars of one bootstrap, made lazily per level by `make(kind, shape)` -
    a callable that returns a buffer of seeded uniform residues for the given prime indices (device
    tensors in the benchmark, numpy arrays in the tests' checker).  Real keys and encoded diagonals
    have exactly these shapes; their values do not change what the kernels do."""

    def __init__(self, moduli: Sequence[int], q_idx: Sequence[int], p_idx: Sequence[int], dnum: int, shape: BootstrapShape,
                 make, galois_elt_from_step, seed: int = 0xB007):
        self.moduli, self.q_idx, self.p_idx, self.dnum = list(moduli), list(q_idx), list(p_idx), dnum
        self.shape, self.make, self.elt = shape, make, galois_elt_from_step
        self.top = shape.top
        self.seed = seed
        self._stages: Dict[Tuple, Stage] = {}
        self._keys: Dict[Tuple, object] = {}
        self._sc: Dict[Tuple, List[int]] = {}
        all_top = self.q_idx[:self.top + 1] + self.p_idx
        self.lift_key = make(("lift",), (1, 2), all_top)

    def dnum_at(self, level: int) -> int:
        # the digit size alpha = ceil(top / dnum) is fixed by the number of extension primes; fewer limbs, fewer digits
        alpha = -(-len(self.q_idx) // self.dnum)
        return max(1, min(level, -(-level // alpha)))

    def _key(self, tag, level):
        k = self._keys.get((tag, level))
        if k is None:
            k = self.make(("key", tag, level), (self.dnum_at(level), 2), self.q_idx[:level] + self.p_idx)
            self._keys[(tag, level)] = k
        return k

    def plaintext(self, name, level):
        k = self._keys.get(("pt", name, level))
        if k is None:
            k = self.make(("pt", name, level), (), self.q_idx[:level])
            self._keys[("pt", name, level)] = k
        return k

    def relin_key(self, level):
        return self._key("relin", level)

    def conj_key(self, level):
        return self._key("conj", level)

    def stage(self, stage, level) -> Stage:
        st = self._stages.get((stage, level))
        if st is None:
            g, ng = self.shape.baby, self.shape.giant
            kind, s = stage
            # stage s of a radix-r decomposition of the slot transform (r = g * ng / 2, 32 for 8 x 8) has the
            # 2r - 1 diagonals k * r^s, -r < k < r: k + r - 1 = g * i + j, so baby step j rotates by j * r^s
            # and giant step i by (g * i - (r - 1)) * r^s - never by zero
            r = max(1, g * ng // 2)
            stride = r ** s
            pts = []
            for i in range(ng):
                for j in range(g):
                    absent = (i == ng - 1 and j == g - 1 and g * ng > 1)     # 2r - 1 diagonals of g * ng places
                    pts.append(None if absent else self.make(("pt", stage, i, j, level), (), self.q_idx[:level]))
            baby_elts = [1] + [self.elt(j * stride) for j in range(1, g)]
            giant_elts = [self.elt((g * i - (r - 1)) * stride) for i in range(ng)]
            if any(e in (0, 1) for e in baby_elts[1:] + giant_elts):
                raise ValueError("rotation steps of stage %r fall outside the slot count" % (stage,))
            st = Stage(g, ng, pts,
                       [None] + [self._key(("baby", stage, j), level) for j in range(1, g)], baby_elts,
                       [self._key(("giant", stage, i), level) for i in range(ng)], giant_elts)
            self._stages[(stage, level)] = st
        return st

    def scalars(self, what, level) -> List[int]:
        v = self._sc.get((what, level))
        if v is None:
            rng = np.random.default_rng([self.seed, zlib.crc32(repr(what).encode())])
            base = int(rng.integers(1, 1 << 40))
            v = [base % self.moduli[p] for p in self.q_idx[:level]]
            self._sc[(what, level)] = v
        return v
