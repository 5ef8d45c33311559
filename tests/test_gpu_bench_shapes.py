"""Parity at the shapes bench.py times: the CUDA build through the C ABI against the CPU oracle,
bit-exact, at HRot L=35 / K=5 / dnum=7 and HMult L=24 / K=1 / dnum=24 (64-bit words, exact base
conversion, rounding division).  These shapes take code paths the small cases never reach: 245
raised limbs, seven 5 -> 35 conversions with the output split chosen from the wave count, 576
raised limbs split over two transform launches with the one-limb-digit loader, two-polynomial
SuD launches of 70 limbs.  The sequence compared is the reference's key-switch lowering
(cerium/compiler/backend/compiler_keyswitch.cc:253-432); comparison style as
examples/common.py:134-142, but on every integer limb instead of decrypted slots."""
import numpy as np
import pytest

import oracle
from cerium_b200 import _capi, params
from tests import parity_cases as pc

pytestmark = pytest.mark.gpu

BM, RM = _capi.BCONV_EXACT, _capi.ROUND_HALF


@pytest.fixture(scope="module")
def be():
    from tests.backends import CudaBackend
    return CudaBackend()


@pytest.fixture(scope="module")
def hrot_case(be):
    prm = params.config_hrot(pc.LOGN, 35, 5, 7)
    h = pc.Harness(be, 64, prm.moduli)
    rng = np.random.default_rng(0xCE210003)
    c0, c1, evk = pc.make_keyswitch_inputs(rng, prm)
    ks = _capi.KeySwitch(h.ctx, prm.q_idx, prm.p_idx, prm.dnum, BM, RM)
    return prm, h, ks, c0, c1, evk, h.up(c0), h.up(c1), h.up(evk)


def test_hrot_bench_shape(be, hrot_case):
    prm, h, ks, c0, c1, evk, d0, d1, dk = hrot_case
    step = int(np.random.default_rng(0xCE210003).integers(1, 1 << 15))     # the benchmark's seeded step
    elt = be.lib.galois_elt_from_step(step, pc.LOGN)
    assert elt == pow(5, step, 2 * pc.N)
    o0, o1 = h.new(prm.L, pc.N), h.new(prm.L, pc.N)
    ks.hrot(h.p(o0), h.p(o1), h.p(d0), h.p(d1), h.p(dk), elt)
    w0, w1 = h.orc.hrot(BM, RM, prm.q_idx, prm.p_idx, prm.dnum, elt, c0, c1, evk)
    assert np.array_equal(h.down(o0), w0), "HRot c0 differs at L=35, K=5, dnum=7"
    assert np.array_equal(h.down(o1), w1), "HRot c1 differs at L=35, K=5, dnum=7"
    # in place: the rotation goes through the workspace instead of the folded reads
    i0, i1 = h.up(c0), h.up(c1)
    ks.hrot(h.p(i0), h.p(i1), h.p(i0), h.p(i1), h.p(dk), elt)
    assert np.array_equal(h.down(i0), w0) and np.array_equal(h.down(i1), w1)


def test_keyswitch_and_hoisted_bench_shape(be, hrot_case):
    prm, h, ks, c0, c1, evk, d0, d1, dk = hrot_case
    L = prm.L
    o0, o1 = h.new(L, pc.N), h.new(L, pc.N)
    ks.apply(h.p(o0), h.p(o1), h.p(d1), h.p(dk))
    k0, k1 = h.orc.keyswitch(BM, RM, prm.q_idx, prm.p_idx, prm.dnum, c1, evk)
    assert np.array_equal(h.down(o0), k0) and np.array_equal(h.down(o1), k1), "key switch differs at L=35"
    # hoisted rotation: phi(KeySwitch(c1) + (c0, 0)) with the automorphism as the store pattern
    ks.hoisted_begin(h.p(d1))
    s0 = np.stack([oracle.ew("add", prm.moduli[p], k0[i], c0[i]) for i, p in enumerate(prm.q_idx)])
    for step in (3, -1000):
        elt = be.lib.galois_elt_from_step(step, pc.LOGN)
        ks.hoisted_rotate(h.p(o0), h.p(o1), h.p(d0), h.p(d1), h.p(dk), elt)
        w0 = np.stack([oracle.apply_galois_ntt(elt, pc.LOGN, s0[i]) for i in range(L)])
        w1 = np.stack([oracle.apply_galois_ntt(elt, pc.LOGN, k1[i]) for i in range(L)])
        assert np.array_equal(h.down(o0), w0) and np.array_equal(h.down(o1), w1), "hoisted rotation differs at L=35"


def test_hmult_bench_shape(be):
    prm = params.config_hmult(pc.LOGN, 24)
    h = pc.Harness(be, 64, prm.moduli)
    rng = np.random.default_rng(0xCE210001)
    a0, a1, evk = pc.make_keyswitch_inputs(rng, prm)
    b0, b1 = pc.rand_limbs(rng, prm.moduli, prm.q_idx), pc.rand_limbs(rng, prm.moduli, prm.q_idx)
    ks = _capi.KeySwitch(h.ctx, prm.q_idx, prm.p_idx, prm.dnum, BM, RM)
    dk = h.up(evk)
    da0, da1, db0, db1 = h.up(a0), h.up(a1), h.up(b0), h.up(b1)
    r0, r1 = h.new(prm.L - 1, pc.N), h.new(prm.L - 1, pc.N)
    ks.hmult(h.p(r0), h.p(r1), h.p(da0), h.p(da1), h.p(db0), h.p(db1), h.p(dk), True)
    w0, w1 = h.orc.hmult_relin(BM, RM, True, prm.q_idx, prm.p_idx, prm.dnum, a0, a1, b0, b1, evk)
    assert np.array_equal(h.down(r0), w0), "HMult+relin+rescale c0 differs at L=24, dnum=24"
    assert np.array_equal(h.down(r1), w1), "HMult+relin+rescale c1 differs at L=24, dnum=24"
    # the rescale folded into the relinearisation's ModDown: one division by P * q_last
    ks.hmult(h.p(r0), h.p(r1), h.p(da0), h.p(da1), h.p(db0), h.p(db1), h.p(dk), 2)
    w0, w1 = h.orc.hmult_relin_fused(BM, RM, prm.q_idx, prm.p_idx, prm.dnum, a0, a1, b0, b1, evk)
    assert np.array_equal(h.down(r0), w0) and np.array_equal(h.down(r1), w1), "HMult with the fused rescale differs at L=24"
    o0, o1 = h.new(prm.L, pc.N), h.new(prm.L, pc.N)
    ks.hmult(h.p(o0), h.p(o1), h.p(da0), h.p(da1), h.p(db0), h.p(db1), h.p(dk), False)
    w0, w1 = h.orc.hmult_relin(BM, RM, False, prm.q_idx, prm.p_idx, prm.dnum, a0, a1, b0, b1, evk)
    assert np.array_equal(h.down(o0), w0) and np.array_equal(h.down(o1), w1), "HMult+relin differs at L=24"
    ks.close()


def test_bsgs_bench_shape(be):
    """A 3 x 3 multiply-accumulate (one absent diagonal) and a 2 x 5 one with two rescale levels at the
    HRot parameter set."""
    prm = params.config_hrot(pc.LOGN, 35, 5, 7)
    pc.case_bsgs(be, 64, 35, 5, 7, BM, RM, g=3, n_giant=3, r=0, prm=prm)
    pc.case_bsgs(be, 64, 35, 5, 7, BM, RM, g=2, n_giant=5, r=2, missing=(), prm=prm)
