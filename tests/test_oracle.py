"""Pins the CPU oracle against big-integer definitions (no GPU needed)."""
import numpy as np
import pytest

import oracle
from cerium_b200 import params
from tests import bigint_ref as B


def _rand_limbs(rng, moduli, n):
    return np.stack([rng.integers(0, q, size=n, dtype=np.uint64) for q in moduli])


@pytest.mark.parametrize("bits,logn", [(28, 4), (50, 5), (60, 6)])
def test_ntt_matches_definition(bits, logn):
    q = params.ntt_primes_below(bits, 1, logn)[0]
    ctx = oracle.OracleContext(logn, [q])
    psi = ctx.root(0)
    assert pow(psi, 1 << logn, q) == q - 1
    # minimal among all primitive 2N-th roots
    assert psi == min(pow(psi, 2 * k + 1, q) for k in range(1 << logn))
    rng = np.random.default_rng(1)
    x = rng.integers(0, q, size=1 << logn, dtype=np.uint64)
    got = ctx.ntt_forward(x, [0])[0]
    assert np.array_equal(got, B.ntt_by_definition(x, q, psi, logn))
    assert np.array_equal(ctx.ntt_inverse(got, [0])[0], x)
    # table order of cerium/runtime/math/ntt.cpp:118-125
    for i in range(1, 1 << logn):
        assert ctx.twiddle(0, B.brev(i, logn)) == pow(psi, i, q)


def test_ntt_roundtrip_and_convolution_full_size():
    logn = 16
    mods = params.ntt_primes_below(50, 2, logn) + params.reference_primes_28bit(1) + params.ntt_primes_below(60, 1, logn)
    ctx = oracle.OracleContext(logn, mods)
    rng = np.random.default_rng(2)
    x = _rand_limbs(rng, mods, 1 << logn)
    idx = list(range(len(mods)))
    f = ctx.ntt_forward(x, idx)
    assert np.array_equal(ctx.ntt_inverse(f, idx), x)
    for k, q in enumerate(mods):
        assert f[k].max() < q


def test_negacyclic_convolution_small():
    logn = 6
    q = params.ntt_primes_below(50, 1, logn)[0]
    ctx = oracle.OracleContext(logn, [q])
    rng = np.random.default_rng(3)
    a = rng.integers(0, q, size=64, dtype=np.uint64)
    b = rng.integers(0, q, size=64, dtype=np.uint64)
    fa, fb = ctx.ntt_forward(a, [0])[0], ctx.ntt_forward(b, [0])[0]
    prod = oracle.ew("mul", q, fa, fb)
    assert np.array_equal(ctx.ntt_inverse(prod, [0])[0], oracle.negacyclic_mul_schoolbook(q, a, b))


def test_galois_step_elements():
    logn = 16
    n = 1 << logn
    assert oracle.galois_elt_from_step(0, logn) == 2 * n - 1
    assert oracle.galois_elt_from_step(1, logn) == 5
    assert oracle.galois_elt_from_step(3, logn) == 125
    assert oracle.galois_elt_from_step(-1, logn) == pow(5, n // 2 - 1, 2 * n)


@pytest.mark.parametrize("step", [0, 1, 5, -3])
def test_galois_ntt_matches_coefficient_definition(step):
    logn = 6
    q = params.ntt_primes_below(28, 1, logn)[0]
    ctx = oracle.OracleContext(logn, [q])
    elt = oracle.galois_elt_from_step(step, logn)
    rng = np.random.default_rng(4)
    x = rng.integers(0, q, size=1 << logn, dtype=np.uint64)
    via_coeff = ctx.ntt_forward(oracle.apply_galois_coeff(elt, logn, q, x), [0])[0]
    via_ntt = oracle.apply_galois_ntt(elt, logn, ctx.ntt_forward(x, [0])[0])
    assert np.array_equal(via_coeff, via_ntt)
    t = oracle.galois_table_ntt(elt, logn)
    assert sorted(t.tolist()) == list(range(1 << logn))


@pytest.mark.parametrize("bits", [28, 50])
def test_bconv_both_modes_vs_bigint(bits):
    logn = 4
    mods = params.ntt_primes_below(bits, 9, logn)
    in_mod, out_mod = mods[:4], mods[4:]
    rng = np.random.default_rng(5)
    x = _rand_limbs(rng, in_mod, 16)
    lazy = oracle.bconv(oracle.BCONV_LAZY, in_mod, x, out_mod)
    exact = oracle.bconv(oracle.BCONV_EXACT, in_mod, x, out_mod)
    Q = int(np.prod([int(m) for m in in_mod], dtype=object))
    for c in range(16):
        col = [int(v) for v in x[:, c]]
        assert [int(v) for v in lazy[:, c]] == B.bconv_lazy(col, in_mod, out_mod)
        assert [int(v) for v in exact[:, c]] == B.bconv_exact(col, in_mod, out_mod)
        # exact mode overshoots the true value by less than I multiples of Q
        X = B.crt_reconstruct(col, in_mod)
        s = sum((int(r) * pow(Q // m, -1, m) % m) * (Q // m) for r, m in zip(col, in_mod))
        assert (s - X) % Q == 0 and 0 <= (s - X) // Q < len(in_mod)


def test_single_limb_bconv_is_plain_reduction():
    mods = params.ntt_primes_below(50, 3, 4)
    rng = np.random.default_rng(6)
    x = _rand_limbs(rng, mods[:1], 16)
    for mode in (oracle.BCONV_LAZY, oracle.BCONV_EXACT):
        out = oracle.bconv(mode, mods[:1], x, mods[1:])
        for j, p in enumerate(mods[1:]):
            assert np.array_equal(out[j], x[0] % np.uint64(p))


@pytest.mark.parametrize("round_mode", [oracle.ROUND_FLOOR, oracle.ROUND_HALF])
def test_moddown_vs_bigint_division(round_mode):
    logn = 4
    n = 1 << logn
    q = params.ntt_primes_below(50, 3, logn)
    p = params.ntt_primes_below(60, 2, logn)
    ctx = oracle.OracleContext(logn, q + p)
    rng = np.random.default_rng(7)
    Q = q[0] * q[1] * q[2]
    P = p[0] * p[1]
    # integer polynomial T in [0, QP), reduced to every prime and transformed
    T = [int(rng.integers(0, 2**62)) * int(rng.integers(0, 2**62)) * int(rng.integers(0, 2**62)) % (Q * P)
         for _ in range(n)]
    coeffs = np.array([[t % m for t in T] for m in q + p], dtype=np.uint64)
    ntt = ctx.ntt_forward(coeffs, list(range(5)))
    out = ctx.moddown(oracle.BCONV_EXACT, round_mode, [0, 1, 2], [3, 4], ntt[:3], ntt[3:])
    got = ctx.ntt_inverse(out, [0, 1, 2])
    for c in range(n):
        t = T[c]
        want = (t + P // 2) // P if round_mode == oracle.ROUND_HALF else t // P
        # fast base conversion may overshoot [t]_P by u*P with 0 <= u < K: result is off by -u
        cands = [[(want - u) % m for m in q] for u in range(3)]
        assert [int(v) for v in got[:, c]] in cands


@pytest.mark.parametrize("round_mode", [oracle.ROUND_FLOOR, oracle.ROUND_HALF])
@pytest.mark.parametrize("r", [1, 2])
def test_moddown_with_fused_rescale_vs_bigint_division(round_mode, r):
    """ModDown with r rescale levels is ONE division by P * q_{L-r} ... q_{L-1}: the dropped Q limbs join
    the extension limbs (cerium/compiler/backend/compiler_keyswitch.cc:26-39, 402-412)."""
    logn = 4
    n = 1 << logn
    q = params.ntt_primes_below(50, 4, logn)
    p = params.ntt_primes_below(60, 2, logn)
    ctx = oracle.OracleContext(logn, q + p)
    rng = np.random.default_rng(70 + r)
    QP = 1
    for m in q + p:
        QP *= m
    D = p[0] * p[1]
    for m in q[4 - r:]:
        D *= m
    T = [int.from_bytes(rng.bytes(40), "little") % QP for _ in range(n)]
    coeffs = np.array([[t % m for t in T] for m in q + p], dtype=np.uint64)
    ntt = ctx.ntt_forward(coeffs, list(range(6)))
    keep = list(range(4 - r))
    out = ctx.moddown_rescale(oracle.BCONV_EXACT, round_mode, [0, 1, 2, 3], [4, 5], r, ntt)
    got = ctx.ntt_inverse(out, keep)
    for c in range(n):
        want = (T[c] + D // 2) // D if round_mode == oracle.ROUND_HALF else T[c] // D
        cands = [[(want - u) % q[i] for i in keep] for u in range(2 + r + 1)]
        assert [int(v) for v in got[:, c]] in cands
    # r = 0 is the plain ModDown
    assert np.array_equal(ctx.moddown_rescale(oracle.BCONV_EXACT, round_mode, [0, 1, 2, 3], [4, 5], 0, ntt),
                          ctx.moddown(oracle.BCONV_EXACT, round_mode, [0, 1, 2, 3], [4, 5], ntt[:4], ntt[4:]))


def test_keyswitch_rescale_and_bsgs_compose_from_pinned_parts():
    """The fused entries are compositions of pinned parts: with r = 0 the key switch with PMU additions
    equals key switch + additions; the BSGS accumulation equals, before its single ModDown, the sum
    of the giant steps' extended-basis key switches (linearity), so with r = 0 and exact division it
    differs from the sum of separately divided rotations by at most the rounding of each division."""
    logn = 4
    n = 1 << logn
    L, K, dnum = 4, 2, 2
    q = params.ntt_primes_below(50, L, logn)
    p = params.ntt_primes_below(60, K, logn)
    mods = q + p
    ctx = oracle.OracleContext(logn, mods)
    rng = np.random.default_rng(81)
    q_idx, p_idx = list(range(L)), list(range(L, L + K))
    rl = lambda idx: np.stack([rng.integers(0, mods[i], size=n, dtype=np.uint64) for i in idx])  # noqa: E731
    c, a0, a1 = rl(q_idx), rl(q_idx), rl(q_idx)
    evk = np.stack([np.stack([rl(q_idx + p_idx) for _ in range(2)]) for _ in range(dnum)])
    k0, k1 = ctx.keyswitch(1, 1, q_idx, p_idx, dnum, c, evk)
    f0, f1 = ctx.keyswitch_rescale(1, 1, q_idx, p_idx, dnum, 0, c, evk, a0, a1)
    for i in range(L):
        assert np.array_equal(f0[i], oracle.ew("add", mods[i], k0[i], a0[i]))
        assert np.array_equal(f1[i], oracle.ew("add", mods[i], k1[i], a1[i]))
    # one giant step without rotation and one with: compare with the explicit composition
    g, n_giant = 2, 2
    baby = np.stack([np.stack([rl(q_idx), rl(q_idx)]) for _ in range(g)])
    pts = np.stack([np.stack([rl(q_idx) for _ in range(g)]) for _ in range(n_giant)])
    elt = oracle.galois_elt_from_step(2, logn)
    keys = np.stack([evk, np.stack([np.stack([rl(q_idx + p_idx) for _ in range(2)]) for _ in range(dnum)])])
    o0, o1 = ctx.bsgs(1, 0, q_idx, p_idx, dnum, 0, baby, pts, np.ones((n_giant, g)), [1, elt], keys)

    def inner(i, poly):
        s = np.zeros((L, n), dtype=np.uint64)
        for j in range(g):
            s = np.stack([oracle.ew("mad", mods[l], baby[j, poly, l], pts[i, j, l], s[l]) for l in range(L)])
        return s
    s00, s01, s10, s11 = inner(0, 0), inner(0, 1), inner(1, 0), inner(1, 1)
    r10 = np.stack([oracle.apply_galois_ntt(elt, logn, s10[l]) for l in range(L)])
    r11 = np.stack([oracle.apply_galois_ntt(elt, logn, s11[l]) for l in range(L)])
    add0 = np.stack([oracle.ew("add", mods[l], s00[l], r10[l]) for l in range(L)])
    w0, w1 = ctx.keyswitch_rescale(1, 0, q_idx, p_idx, dnum, 0, r11, keys[1], add0, s01)
    assert np.array_equal(o0, w0) and np.array_equal(o1, w1)


def test_rescale_vs_bigint_division():
    logn = 4
    n = 1 << logn
    q = params.ntt_primes_below(50, 3, logn)
    ctx = oracle.OracleContext(logn, q)
    rng = np.random.default_rng(8)
    Q = q[0] * q[1] * q[2]
    T = [int(rng.integers(0, 2**62)) * int(rng.integers(0, 2**62)) * int(rng.integers(0, 2**50)) % Q
         for _ in range(n)]
    coeffs = np.array([[t % m for t in T] for m in q], dtype=np.uint64)
    ntt = ctx.ntt_forward(coeffs, [0, 1, 2])
    for mode in (oracle.ROUND_FLOOR, oracle.ROUND_HALF):
        got = ctx.ntt_inverse(ctx.rescale(mode, [0, 1, 2], ntt), [0, 1])
        for c in range(n):
            want = (T[c] + q[2] // 2) // q[2] if mode == oracle.ROUND_HALF else T[c] // q[2]
            assert [int(v) for v in got[:, c]] == [want % q[0], want % q[1]]


def test_double_rescale_vs_bigint_division():
    logn = 4
    n = 1 << logn
    q = params.ntt_primes_below(50, 4, logn)
    ctx = oracle.OracleContext(logn, q)
    rng = np.random.default_rng(9)
    Q = q[0] * q[1] * q[2] * q[3]
    T = [int(rng.integers(0, 2**62)) * int(rng.integers(0, 2**62)) * int(rng.integers(0, 2**62))
         * int(rng.integers(0, 2**14)) % Q for _ in range(n)]
    T[0], T[1] = Q - 1, q[2] * q[3] - 1       # extremes: largest value, largest dropped part
    coeffs = np.array([[t % m for t in T] for m in q], dtype=np.uint64)
    ntt = ctx.ntt_forward(coeffs, [0, 1, 2, 3])
    got = ctx.ntt_inverse(ctx.double_rescale([0, 1, 2, 3], ntt), [0, 1])
    for c in range(n):
        want = T[c] // (q[2] * q[3])
        assert [int(v) for v in got[:, c]] == [want % q[0], want % q[1]]


def test_mod_raise_with_a_noiseless_key_is_exact():
    """ModRaise pinned on integers: with the key (P * q_drop * s', 0) and no noise every step is an
    exact division, so out0 = NTT(v0 + v1 (*) s') and out1 = 0, where v0, v1 are the integers the two
    base limbs compose to and (*) is the negacyclic product over the integers."""
    logn = 4
    n = 1 << logn
    q = params.ntt_primes_below(50, 4, logn)          # base = q[0], q[1]; targets q[0..2]; q[3] is dropped
    p = params.ntt_primes_below(60, 2, logn)
    mods = q + p
    ctx = oracle.OracleContext(logn, mods)
    q_idx, p_idx = [0, 1, 2, 3], [4, 5]
    rng = np.random.default_rng(11)
    B01 = q[0] * q[1]
    V0 = [int(rng.integers(0, 2**62)) * int(rng.integers(0, 2**40)) % B01 for _ in range(n)]
    V1 = [int(rng.integers(0, 2**62)) * int(rng.integers(0, 2**40)) % B01 for _ in range(n)]
    V1[0] = B01 - 1
    s = [int(v) for v in rng.integers(-1, 2, size=n)]
    # negacyclic product over the integers
    Z = [0] * n
    for i in range(n):
        for j in range(n):
            k = i + j
            Z[k % n] += V1[i] * s[j] * (1 if k < n else -1)

    def limbs(poly, idx):
        return ctx.ntt_forward(np.array([[c % mods[i] for c in poly] for i in idx], dtype=np.uint64), idx)

    c0, c1 = limbs(V0, [0, 1]), limbs(V1, [0, 1])
    P = p[0] * p[1]
    key = [P * q[3] * c for c in s]
    evk = np.stack([limbs(key, q_idx + p_idx), np.zeros((6, n), dtype=np.uint64)])
    o0, o1 = ctx.mod_raise(oracle.BCONV_EXACT, oracle.ROUND_FLOOR, q_idx, p_idx, 0, 1, c0, c1, evk)
    want = limbs([a + b for a, b in zip(V0, Z)], [0, 1, 2])
    assert np.array_equal(o0, want)
    assert not o1.any()
