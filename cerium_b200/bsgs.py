"""Baby-step / giant-step multiply-accumulate: out = sum_k pt_k (.) rot_k(ct) over rotation steps
k = g * j + i, 0 <= i < g (baby), 0 <= j < n_giant.

The Python face of ``cerium_bsgs_apply``, which restates BsgsMultiplyAccumulate of the reference
(``cerium/python/compiler/dsl/__init__.py``, lowered in ``cerium/compiler/backend/compiler.cc:2457-2822``):
the g - 1 baby rotations of the input share one ModUp, every giant step rotates its inner sum,
the giant steps' key-switch products are accumulated in the extended basis and ONE ModDown (with
optional rescale levels in the same division) ends the operation:

    out = sum_j rot_{g j}( sum_i pt[j][i] (.) rot_i(ct) ),   pt[j][i] = rot_{-g j}(diagonal_{g j + i}).

This is the linear-transform building block of bootstrapping (CoeffToSlot / SlotToCoeff) and of
matrix-vector products.  This class only owns the scratch buffer and forwards addresses; buffers are
whatever the caller's `alloc` returns (torch CUDA tensors with the CUDA build), `ptr` maps a buffer
to its device address.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

from . import _capi


class BsgsMultiplyAccumulate:
    def __init__(self, ctx: _capi.Context, ks: _capi.KeySwitch, g: int, n_giant: int,
                 alloc: Callable[[Sequence[int]], object], ptr: Callable[[object], int], rescale_levels: int = 0):
        if g < 1 or n_giant < 1:
            raise ValueError("need at least one baby and one giant step")
        self.ctx, self.ks, self.g, self.n_giant, self.r = ctx, ks, g, n_giant, rescale_levels
        self.ptr = ptr
        self.L = len(ks.q_idx)
        self.work = alloc((ks.bsgs_work_limbs(g, n_giant), ctx.n))
        self.limb_bytes = ctx.n * ctx.word_bytes

    def run(self, out, ct, plaintexts: List[List[Optional[object]]], baby_keys_pre: Sequence[object],
            giant_keys: Sequence[object], baby_elts: Sequence[int], giant_elts: Sequence[int], stream: int = 0):
        """ct: [2][L][N] (c0, c1); out: [2][L - rescale_levels][N].  plaintexts[j][i]: [L][N] NTT-form
        plaintext or None (an absent diagonal).  baby_keys_pre[i - 1], baby_elts[i - 1]: pre-permuted key
        and Galois element of rotation step i; giant_keys[j - 1], giant_elts[j - 1]: ordinary key and
        element of step g * j (giant step 0 is not rotated)."""
        p = self.ptr
        poly = self.L * self.limb_bytes
        out_poly = (self.L - self.r) * self.limb_bytes
        flat = [p(t) if t is not None else 0 for row in plaintexts for t in row]
        self.ks.bsgs_apply(p(out), p(out) + out_poly, p(ct), p(ct) + poly, self.g, self.n_giant, flat,
                           [0] + [p(k) for k in baby_keys_pre], [1] + list(baby_elts),
                           [0] + [p(k) for k in giant_keys], [1] + list(giant_elts), self.r, p(self.work), stream)
