"""Baby-step / giant-step multiply-accumulate: out = sum_k pt_k (.) rot_k(ct) over rotation steps
k = g * j + i, 0 <= i < g (baby), 0 <= j < n_giant.

Restates BsgsMultiplyAccumulate of the reference (``cerium/python/compiler/dsl/__init__.py``,
lowered in ``cerium/compiler/backend/compiler.cc:2457-2822``): the g - 1 baby rotations of the
input share one ModUp (``cerium_hoisted_begin`` / ``cerium_hoisted_rotate``), every giant step
rotates the inner sum once:

    out = sum_j rot_{g j}( sum_i pt[j][i] (.) rot_i(ct) ),   pt[j][i] = rot_{-g j}(diagonal_{g j + i}).

This is the linear-transform building block of bootstrapping (CoeffToSlot / SlotToCoeff) and of
matrix-vector products.  Host orchestration only: all arithmetic runs in the library's kernels.
Buffers are whatever the caller's `alloc` returns (torch CUDA tensors with the CUDA build); `ptr`
maps a buffer to its device address.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

from . import _capi


class BsgsMultiplyAccumulate:
    def __init__(self, ctx: _capi.Context, ks: _capi.KeySwitch, g: int, n_giant: int,
                 alloc: Callable[[Sequence[int]], object], ptr: Callable[[object], int]):
        if g < 1 or n_giant < 1:
            raise ValueError("need at least one baby and one giant step")
        self.ctx, self.ks, self.g, self.n_giant = ctx, ks, g, n_giant
        self.ptr = ptr
        L, n = len(ks.q_idx), ctx.n
        self.L = L
        # rotated copies of the input (baby steps 1 .. g-1), one inner sum, one rotated inner sum
        self.baby = [alloc((2, L, n)) for _ in range(g - 1)]
        self.inner = alloc((2, L, n))
        self.rotated = alloc((2, L, n))
        self.limb_bytes = n * ctx.word_bytes

    def _poly(self, buf, k: int) -> int:
        return self.ptr(buf) + k * self.L * self.limb_bytes

    def run(self, out, ct, plaintexts: List[List[Optional[object]]], baby_keys_pre: Sequence[object],
            giant_keys: Sequence[object], baby_elts: Sequence[int], giant_elts: Sequence[int], stream: int = 0):
        """out, ct: [2][L][N] buffers (c0, c1).  plaintexts[j][i]: [L][N] NTT-form plaintext or None
        (an absent diagonal).  baby_keys_pre[i - 1], baby_elts[i - 1]: pre-permuted key and Galois
        element of rotation step i; giant_keys[j - 1], giant_elts[j - 1]: ordinary key and element
        of step g * j."""
        ctx, ks, p = self.ctx, self.ks, self.ptr
        q_idx = list(ks.q_idx)
        if self.g > 1:
            ks.hoisted_begin(self._poly(ct, 1), stream)
            for i in range(1, self.g):
                b = self.baby[i - 1]
                ks.hoisted_rotate(self._poly(b, 0), self._poly(b, 1), self._poly(ct, 0), self._poly(ct, 1),
                                  p(baby_keys_pre[i - 1]), baby_elts[i - 1], stream)
        sources = [ct] + self.baby
        first_giant = True
        for j in range(self.n_giant):
            dst = out if j == 0 else self.inner
            started = False
            for i in range(self.g):
                pt = plaintexts[j][i]
                if pt is None:
                    continue
                for k in range(2):
                    if not started:
                        ctx.ewise(_capi.EW_MUL, self._poly(dst, k), self._poly(sources[i], k), q_idx, b=p(pt),
                                  stream=stream)
                    else:
                        ctx.ewise(_capi.EW_MAD, self._poly(dst, k), self._poly(sources[i], k), q_idx, b=p(pt),
                                  c=self._poly(dst, k), stream=stream)
                started = True
            if not started:
                if j == 0:
                    raise ValueError("giant step 0 needs at least one diagonal")
                continue
            if j == 0:
                first_giant = False
                continue
            r = self.rotated
            ks.hrot(self._poly(r, 0), self._poly(r, 1), self._poly(dst, 0), self._poly(dst, 1), p(giant_keys[j - 1]),
                    giant_elts[j - 1], stream)
            for k in range(2):
                ctx.ewise(_capi.EW_ADD, self._poly(out, k), self._poly(out, k), q_idx, b=self._poly(r, k), stream=stream)
        if first_giant:
            raise ValueError("giant step 0 needs at least one diagonal")
