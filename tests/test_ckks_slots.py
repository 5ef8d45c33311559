"""Slot-level checks in the style of the reference's example runners (encrypt, evaluate, decrypt,
compare with numpy; examples/common.py:134-142, tolerance rtol=1e-5 / atol=1e-4): rotation and
multiplication must be right as CKKS operations, which pins the key layout, the digit gadget
and the ModDown direction independently of the oracle-vs-kernel comparison."""
import numpy as np
import pytest

import oracle
from cerium_b200 import _capi, params
from tests.ckks_ref import CkksRef

LOGN = 16
N = 1 << LOGN


def small_set(L, K, dnum):
    q = params.ntt_primes_below(60, 1, LOGN) + params.ntt_primes_below(50, L - 1, LOGN)
    p = params.ntt_primes_below(60, K + 1, LOGN)[1:]
    return params.CkksParams(LOGN, 64, q + p[::-1], L, K, dnum)


def test_oracle_rotation_decrypts_to_rolled_slots():
    prm = small_set(3, 2, 2)
    ck = CkksRef(prm, seed=10)
    rng = np.random.default_rng(3)
    z = rng.uniform(-1, 1, N // 2)
    scale = 2.0 ** 40
    c0, c1 = ck.encrypt(z, scale)
    assert np.allclose(ck.decrypt(c0, c1, scale).real, z, rtol=1e-5, atol=1e-4)
    step = 5
    elt = oracle.galois_elt_from_step(step, LOGN)
    evk = ck.rotation_key(elt)
    o0, o1 = ck.octx.hrot(oracle.BCONV_EXACT, oracle.ROUND_HALF, prm.q_idx, prm.p_idx, prm.dnum, elt, c0, c1, evk)
    assert np.allclose(ck.decrypt(o0, o1, scale).real, np.roll(z, -step), rtol=1e-5, atol=1e-4)
    o0, o1 = ck.octx.hrot(oracle.BCONV_EXACT, oracle.ROUND_FLOOR, prm.q_idx, prm.p_idx, prm.dnum, elt, c0, c1, evk)
    assert np.allclose(ck.decrypt(o0, o1, scale).real, np.roll(z, -step), rtol=1e-5, atol=1e-4)


def test_oracle_lazy_conversion_on_the_reference_prime_chain():
    """The reference's lazy base conversion leaves every digit overshooting by up to alpha * q_max
    multiples of its modulus and ModDown off by up to K * q_max, because inputs are not reduced by
    q_i first (cerium/compiler/backend/kernels/fhe_bconv.cuh:123-150).  With 28-bit primes and the
    reference's 2^56 scale (two primes per level, examples/relinearization/program.py:26-38) that
    ModDown offset (a positive bias of about K * 2^27 in every coefficient, i.e. up to ~2^45 in the slot
    next to zeta = 1) disappears under the scale the reference's rotation example uses, 2^84 (three
    primes, examples/rotation/runner.py:22-25), and the result passes the tolerance of
    examples/common.py:141; at 2^56 it would not, and with 50/60-bit primes the bias is 2^60 * K,
    which is why the 64-bit configurations use the exact conversion."""
    prm = params.config_ref28(LOGN, 6, 4, 2, total=10)  # K = alpha + 1: P exceeds the digit modulus by one prime
    ck = CkksRef(prm, seed=13)
    rng = np.random.default_rng(6)
    z = rng.uniform(-1, 1, N // 2)
    scale = 2.0 ** 84
    c0, c1 = ck.encrypt(z, scale)
    assert np.allclose(ck.decrypt(c0, c1, scale, use=4).real, z, rtol=1e-5, atol=1e-4)
    step = 3
    elt = oracle.galois_elt_from_step(step, LOGN)
    evk = ck.rotation_key(elt)
    o0, o1 = ck.octx.hrot(oracle.BCONV_LAZY, oracle.ROUND_FLOOR, prm.q_idx, prm.p_idx, prm.dnum, elt, c0, c1, evk)
    assert np.allclose(ck.decrypt(o0, o1, scale, use=4).real, np.roll(z, -step), rtol=1e-5, atol=1e-4)


def prepermuted_key(evk, elt):
    """phi^-1 applied to every limb of a key: the reference's RotationInv key for hoisting."""
    inv = pow(int(elt), -1, 2 * N)
    flat = evk.reshape(-1, N)
    return np.stack([oracle.apply_galois_ntt(inv, LOGN, row) for row in flat]).reshape(evk.shape)


def test_oracle_hoisted_rotation_identity():
    """phi( KeySwitch(c1; phi^-1(key)) + (c0, 0) ) decrypts to the rotated slots."""
    prm = small_set(3, 2, 2)
    ck = CkksRef(prm, seed=14)
    rng = np.random.default_rng(7)
    z = rng.uniform(-1, 1, N // 2)
    scale = 2.0 ** 40
    c0, c1 = ck.encrypt(z, scale)
    step = 9
    elt = oracle.galois_elt_from_step(step, LOGN)
    pre = prepermuted_key(ck.rotation_key(elt), elt)
    k0, k1 = ck.octx.keyswitch(oracle.BCONV_EXACT, oracle.ROUND_HALF, prm.q_idx, prm.p_idx, prm.dnum, c1, pre)
    k0 = np.stack([oracle.ew("add", prm.moduli[p], k0[i], c0[i]) for i, p in enumerate(prm.q_idx)])
    o0 = np.stack([oracle.apply_galois_ntt(elt, LOGN, k0[i]) for i in range(prm.L)])
    o1 = np.stack([oracle.apply_galois_ntt(elt, LOGN, k1[i]) for i in range(prm.L)])
    assert np.allclose(ck.decrypt(o0, o1, scale).real, np.roll(z, -step), rtol=1e-5, atol=1e-4)


def test_oracle_hmult_relin_rescale_decrypts_to_product():
    prm = small_set(3, 1, 3)
    ck = CkksRef(prm, seed=11)
    rng = np.random.default_rng(4)
    x, y = rng.uniform(-1, 1, N // 2), rng.uniform(-1, 1, N // 2)
    scale = 2.0 ** 40
    a0, a1 = ck.encrypt(x, scale)
    b0, b1 = ck.encrypt(y, scale)
    evk = ck.relin_key()
    o0, o1 = ck.octx.hmult_relin(oracle.BCONV_EXACT, oracle.ROUND_HALF, True, prm.q_idx, prm.p_idx, prm.dnum,
                                 a0, a1, b0, b1, evk)
    q_last = prm.moduli[prm.q_idx[-1]]
    got = ck.decrypt(o0, o1, scale * scale / q_last).real
    assert np.allclose(got, x * y, rtol=1e-5, atol=1e-4)


def test_oracle_hmult_precision_at_the_benchmark_configuration():
    """The HMult benchmark's own parameters: N = 2^16, 24 limbs (one 60-bit, 23 of 50 bits), one 60-bit special
    prime, one digit per limb, slots uniform in [-1, 1] at scale 2^50, ternary secret of Hamming weight 192,
    errors of standard deviation 3.2.  HMult + relinearise + rescale as two divisions and as the single division
    by P * q_last; the precision of the decrypted product is printed in bits (GPU and oracle agree on every
    limb at this shape: tests/test_gpu_bench_shapes.py)."""
    prm = params.config_hmult(LOGN, 24)
    ck = CkksRef(prm, seed=21, hamming_weight=192, sigma=3.2)
    rng = np.random.default_rng(22)
    x, y = rng.uniform(-1, 1, N // 2), rng.uniform(-1, 1, N // 2)
    scale = 2.0 ** 50
    a0, a1 = ck.encrypt(x, scale)
    b0, b1 = ck.encrypt(y, scale)
    evk = ck.relin_key()
    q_last = prm.moduli[prm.q_idx[-1]]
    o0, o1 = ck.octx.hmult_relin(oracle.BCONV_EXACT, oracle.ROUND_HALF, True, prm.q_idx, prm.p_idx, prm.dnum,
                                 a0, a1, b0, b1, evk)
    two = ck.decrypt(o0, o1, scale * scale / q_last).real
    f0, f1 = ck.octx.hmult_relin_fused(oracle.BCONV_EXACT, oracle.ROUND_HALF, prm.q_idx, prm.p_idx, prm.dnum,
                                       a0, a1, b0, b1, evk)
    one = ck.decrypt(f0, f1, scale * scale / q_last).real
    bits_two = -np.log2(np.max(np.abs(two - x * y)))
    bits_one = -np.log2(np.max(np.abs(one - x * y)))
    print("HMult at L=24, dnum=24, scale 2^50: %.1f bits with two divisions, %.1f bits with one" % (bits_two, bits_one))
    assert bits_two > 20 and bits_one > 20
    assert np.max(np.abs(one - two)) < 2.0 ** -30                    # the two roundings differ in the last bits only


def test_oracle_hrot_precision_at_the_benchmark_configuration():
    """The HRot benchmark's own parameters (N = 2^16, L = 35 of 50 bits, K = 5 of 60 bits, dnum = 7) with a real key
    and message: rotation by the benchmark's seeded step, precision of the decrypted slots in bits."""
    prm = params.config_hrot(LOGN, 35, 5, 7)
    ck = CkksRef(prm, seed=23, hamming_weight=192, sigma=3.2)
    rng = np.random.default_rng(24)
    z = rng.uniform(-1, 1, N // 2)
    scale = 2.0 ** 50
    c0, c1 = ck.encrypt(z, scale)
    step = int(np.random.default_rng(0xCE210003).integers(1, 1 << 15))
    elt = oracle.galois_elt_from_step(step, LOGN)
    evk = ck.rotation_key(elt)
    o0, o1 = ck.octx.hrot(oracle.BCONV_EXACT, oracle.ROUND_HALF, prm.q_idx, prm.p_idx, prm.dnum, elt, c0, c1, evk)
    got = ck.decrypt(o0, o1, scale).real
    bits = -np.log2(np.max(np.abs(got - np.roll(z, -step))))
    print("HRot at L=35, K=5, dnum=7, scale 2^50: %.1f bits" % bits)
    assert bits > 25


@pytest.mark.gpu
def test_gpu_rotation_and_product_decrypt_correctly():
    import torch
    from tests.backends import CudaBackend
    be = CudaBackend()
    prm = small_set(6, 2, 3)
    ck = CkksRef(prm, seed=12)
    rng = np.random.default_rng(5)
    x, y = rng.uniform(-1, 1, N // 2), rng.uniform(-1, 1, N // 2)
    scale = 2.0 ** 40
    a0, a1 = ck.encrypt(x, scale)
    b0, b1 = ck.encrypt(y, scale)
    ctx = _capi.Context(be.lib, prm.moduli, 64)
    ks = _capi.KeySwitch(ctx, prm.q_idx, prm.p_idx, prm.dnum, _capi.BCONV_EXACT, _capi.ROUND_HALF)
    up = be.to_dev
    step = -7
    elt = be.lib.galois_elt_from_step(step, LOGN)
    d = [up(v) for v in (a0, a1, b0, b1)]
    o0, o1 = be.empty((prm.L, N), np.uint64), be.empty((prm.L, N), np.uint64)
    evk = up(ck.rotation_key(elt))
    ks.hrot(be.ptr(o0), be.ptr(o1), be.ptr(d[0]), be.ptr(d[1]), be.ptr(evk), elt)
    got = ck.decrypt(be.to_host(o0), be.to_host(o1), scale).real
    assert np.allclose(got, np.roll(x, -step), rtol=1e-5, atol=1e-4)
    # hoisted: one ModUp of c1, two rotations with pre-permuted keys
    ks.hoisted_begin(be.ptr(d[1]))
    for st in (1, 64):
        e2 = be.lib.galois_elt_from_step(st, LOGN)
        pre = up(prepermuted_key(ck.rotation_key(e2), e2))
        ks.hoisted_rotate(be.ptr(o0), be.ptr(o1), be.ptr(d[0]), be.ptr(d[1]), be.ptr(pre), e2)
        got = ck.decrypt(be.to_host(o0), be.to_host(o1), scale).real
        assert np.allclose(got, np.roll(x, -st), rtol=1e-5, atol=1e-4)
    rk = up(ck.relin_key())
    r0, r1 = be.empty((prm.L - 1, N), np.uint64), be.empty((prm.L - 1, N), np.uint64)
    ks.hmult(be.ptr(r0), be.ptr(r1), be.ptr(d[0]), be.ptr(d[1]), be.ptr(d[2]), be.ptr(d[3]), be.ptr(rk), True)
    q_last = prm.moduli[prm.q_idx[-1]]
    got = ck.decrypt(be.to_host(r0), be.to_host(r1), scale * scale / q_last).real
    err = np.max(np.abs(got - x * y))
    assert np.allclose(got, x * y, rtol=1e-5, atol=1e-4), err


def test_oracle_conjugation_decrypts_to_conjugated_slots():
    """Step 0 is the conjugation (Galois element 2N - 1, cerium/runtime/math/galois.cpp:79-113):
    the same rotate + key-switch path with the key for that element."""
    prm = small_set(3, 2, 2)
    ck = CkksRef(prm, seed=12)
    rng = np.random.default_rng(5)
    z = rng.uniform(-1, 1, N // 2) + 1j * rng.uniform(-1, 1, N // 2)
    scale = 2.0 ** 40
    c0, c1 = ck.encrypt(z, scale)
    elt = oracle.galois_elt_from_step(0, LOGN)
    assert elt == 2 * N - 1
    evk = ck.rotation_key(elt)
    o0, o1 = ck.octx.hrot(oracle.BCONV_EXACT, oracle.ROUND_HALF, prm.q_idx, prm.p_idx, prm.dnum, elt, c0, c1, evk)
    assert np.allclose(ck.decrypt(o0, o1, scale), np.conj(z), rtol=1e-5, atol=1e-4)


def _bsgs_case(be):
    """Four generalised diagonals (steps 0..3) as baby steps {0, 1} x giant steps {0, 2}: the hoisted
    baby rotation, the plaintext products, the giant rotation and the accumulation decrypt to
    sum_k diag_k * roll(z, -k)."""
    from cerium_b200 import _capi
    from cerium_b200.bsgs import BsgsMultiplyAccumulate
    prm = small_set(3, 2, 2)
    ck = CkksRef(prm, seed=14)
    rng = np.random.default_rng(9)
    n_slots = N // 2
    z = rng.uniform(-1, 1, n_slots)
    diags = [rng.uniform(-1, 1, n_slots) for _ in range(4)]
    scale = 2.0 ** 40
    c0, c1 = ck.encrypt(z, scale)
    g = 2
    idx = list(prm.q_idx)

    def plaintext(v):
        m = ck.encode(v, scale)
        return np.stack([ck.octx.ntt_forward(ck._signed_to_limb(m, p), [p])[0] for p in idx])

    pts = [[plaintext(np.roll(diags[g * j + i], g * j)) for i in range(g)] for j in range(2)]
    e1 = oracle.galois_elt_from_step(1, LOGN)
    e2 = oracle.galois_elt_from_step(2, LOGN)
    ctx = _capi.Context(be.lib, prm.moduli, 64)
    ks = _capi.KeySwitch(ctx, prm.q_idx, prm.p_idx, prm.dnum, _capi.BCONV_EXACT, _capi.ROUND_HALF)
    keep = []

    def up(a):
        b = be.to_dev(np.ascontiguousarray(a).astype(np.uint64))
        keep.append(b)
        return b

    op = BsgsMultiplyAccumulate(ctx, ks, g, 2, lambda shape: be.empty(tuple(shape), np.uint64), be.ptr)
    ct = up(np.stack([c0, c1]))
    out = be.empty((2, prm.L, N), np.uint64)
    op.run(out, ct, [[up(p) for p in row] for row in pts], [up(prepermuted_key(ck.rotation_key(e1), e1))],
           [up(ck.rotation_key(e2))], [e1], [e2])
    res = be.to_host(out)
    want = sum(diags[k] * np.roll(z, -k) for k in range(4))
    got = ck.decrypt(res[0], res[1], scale * scale).real
    assert np.allclose(got, want, rtol=1e-5, atol=1e-4)


def test_bsgs_multiply_accumulate_is_a_matrix_vector_product():
    from tests.backends import EmuBackend
    _bsgs_case(EmuBackend())


@pytest.mark.gpu
def test_gpu_bsgs_multiply_accumulate():
    from tests.backends import CudaBackend
    _bsgs_case(CudaBackend())
