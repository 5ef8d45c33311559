"""Parity cases: the C ABI against the CPU oracle on the same seeded inputs.

Every case takes a backend (tests/backends.py) so that it runs both on the emulation build
(no GPU; checks index arithmetic and host orchestration) and on the CUDA build (the parity
tests proper).  Comparison is bit-exact: all residues are canonical on both sides.
"""
from __future__ import annotations

import numpy as np

import oracle
from cerium_b200 import _capi, params

LOGN = 16
N = 1 << LOGN


def wdtype(word_bits):
    return np.uint64 if word_bits == 64 else np.uint32


_U32_BITS = 28   # case_u32_widest_primes switches the 32-bit cases to primes just below 2^30


def moduli_for(word_bits, count, sixty=0):
    """`count` primes for the word size; for 64-bit the first `sixty` are 60-bit, the rest 50-bit."""
    if word_bits == 32:
        if _U32_BITS != 28:
            return params.ntt_primes_below(_U32_BITS, count, LOGN)
        return params.reference_primes_28bit(count, LOGN)
    return params.ntt_primes_below(60, sixty, LOGN) + params.ntt_primes_below(50, count - sixty, LOGN)


def rand_limbs(rng, moduli, prime_idx, extra=()):
    """[len(prime_idx)] + extra + [N] uniform residues below each limb's modulus (uint64)."""
    rows = [rng.integers(0, moduli[p], size=tuple(extra) + (N,), dtype=np.uint64) for p in prime_idx]
    return np.stack(rows)


def edge_limbs(moduli, prime_idx):
    """Extreme residues: 0, 1, q-1 patterns."""
    rows = []
    for k, p in enumerate(prime_idx):
        q = moduli[p]
        r = np.zeros(N, dtype=np.uint64)
        if k % 3 == 0:
            r[:] = q - 1
        elif k % 3 == 1:
            r[::2] = q - 1
            r[1::2] = 1
        rows.append(r)
    return np.stack(rows)


class Harness:
    def __init__(self, backend, word_bits, moduli):
        self.be = backend
        self.word_bits = word_bits
        self.moduli = list(moduli)
        self.dt = wdtype(word_bits)
        self.ctx = _capi.Context(backend.lib, moduli, word_bits)
        self.orc = oracle.OracleContext(LOGN, moduli)

    def up(self, a):
        return self.be.to_dev(np.ascontiguousarray(a).astype(self.dt))

    def down(self, buf):
        return self.be.to_host(buf).astype(np.uint64)

    def new(self, *shape):
        return self.be.empty(shape, self.dt)

    def p(self, buf):
        return self.be.ptr(buf)


# ---------------------------------------------------------------------------------------

def case_ntt(be, word_bits, n_limbs=3, sixty=1):
    mods = moduli_for(word_bits, n_limbs, sixty)
    h = Harness(be, word_bits, mods)
    rng = np.random.default_rng(100 + word_bits)
    idx = list(range(n_limbs)) + [0]
    x = rand_limbs(rng, mods, idx)
    x[-1] = edge_limbs(mods, [0])[0]
    want = h.orc.ntt_forward(x, idx)
    d_in = h.up(x)
    d_out = h.new(len(idx), N)
    h.ctx.ntt_forward(h.p(d_out), h.p(d_in), idx)
    got = h.down(d_out)
    assert np.array_equal(got, want), "forward NTT differs from the oracle"
    assert np.array_equal(h.down(d_in), x), "out-of-place forward NTT modified its input"
    # inverse, out of place then in place
    d_back = h.new(len(idx), N)
    h.ctx.ntt_inverse(h.p(d_back), h.p(d_out), idx)
    assert np.array_equal(h.down(d_back), x), "inverse NTT does not undo the forward NTT"
    h.ctx.ntt_forward(h.p(d_in), h.p(d_in), idx)
    assert np.array_equal(h.down(d_in), want), "in-place forward NTT differs"
    h.ctx.ntt_inverse(h.p(d_in), h.p(d_in), idx)
    assert np.array_equal(h.down(d_in), x), "in-place inverse NTT differs"
    # inverse against the oracle on arbitrary NTT-domain data
    y = rand_limbs(rng, mods, idx)
    d_y = h.up(y)
    h.ctx.ntt_inverse(h.p(d_y), h.p(d_y), idx)
    assert np.array_equal(h.down(d_y), h.orc.ntt_inverse(y, idx)), "inverse NTT differs from the oracle"
    # empty batch is a no-op
    h.ctx.ntt_forward(h.p(d_y), h.p(d_y), [])


def case_ntt_fp_extremes(be):
    """Primes just below 2^50 (the least headroom of the double-precision butterflies) on inputs
    made of extreme residues; forward and inverse against the oracle, and the round trip."""
    mods = params.ntt_primes_below(50, 3, LOGN)
    assert all((1 << 49) < q < (1 << 50) for q in mods)
    h = Harness(be, 64, mods)
    rng = np.random.default_rng(77)
    rows, idx = [], []
    for p, q in enumerate(mods):
        a = np.full(N, q - 1, dtype=np.uint64)
        b = np.full(N, (q - 1) // 2, dtype=np.uint64)
        c = np.where(np.arange(N) % 2 == 0, q - 1, 0).astype(np.uint64)
        d = np.where(rng.integers(0, 2, size=N) == 0, q - 1, 1).astype(np.uint64)
        e = np.zeros(N, dtype=np.uint64)
        e[0] = q - 1
        for r in (a, b, c, d, e):
            rows.append(r)
            idx.append(p)
    x = np.stack(rows)
    dx = h.up(x)
    out = h.new(len(idx), N)
    h.ctx.ntt_forward(h.p(out), h.p(dx), idx)
    f = h.down(out)
    assert np.array_equal(f, h.orc.ntt_forward(x, idx)), "forward NTT of extreme inputs differs"
    h.ctx.ntt_inverse(h.p(out), h.p(out), idx)
    assert np.array_equal(h.down(out), x), "round trip of extreme inputs differs"
    h.ctx.ntt_inverse(h.p(out), h.p(dx), idx)
    assert np.array_equal(h.down(out), h.orc.ntt_inverse(x, idx)), "inverse NTT of extreme inputs differs"


def case_ntt_ptrs(be, word_bits):
    """Pointer-table entry points (the reference launchers' layout), ragged limb placement."""
    mods = moduli_for(word_bits, 2, 0)
    h = Harness(be, word_bits, mods)
    rng = np.random.default_rng(7)
    idx = [1, 0, 1]
    x = rand_limbs(rng, mods, idx)
    pool = h.new(8, N)          # limbs scattered inside a larger pool
    host_pool = np.zeros((8, N), dtype=np.uint64)
    in_slots, out_slots = [6, 0, 3], [1, 7, 4]
    for s, row in zip(in_slots, x):
        host_pool[s] = row
    pool = h.up(host_pool)
    base = h.p(pool)
    limb_bytes = N * h.ctx.word_bytes
    ins = be.to_dev(np.array([base + s * limb_bytes for s in in_slots], dtype=np.uint64))
    outs = be.to_dev(np.array([base + s * limb_bytes for s in out_slots], dtype=np.uint64))
    bases = be.to_dev(np.array(idx, dtype=np.uint32))
    h.ctx.ntt_forward_ptrs(be.ptr(outs), be.ptr(ins), be.ptr(bases), 3)
    got = h.down(pool)
    want = h.orc.ntt_forward(x, idx)
    for s, row in zip(out_slots, want):
        assert np.array_equal(got[s], row)
    # inverse back into the input slots
    h.ctx.ntt_inverse_ptrs(be.ptr(ins), be.ptr(outs), be.ptr(bases), 3)
    got = h.down(pool)
    for s, row in zip(in_slots, x):
        assert np.array_equal(got[s], row)


def case_sud_ptrs(be, word_bits):
    """SuD with the reference launcher's tables: two device pointers per entry, factors per prime."""
    mods = moduli_for(word_bits, 4, 1)
    h = Harness(be, word_bits, mods)
    rng = np.random.default_rng(71)
    idx = [2, 0, 1, 2]
    minuend, coeff = rand_limbs(rng, mods, idx), rand_limbs(rng, mods, idx)
    fac = [int(rng.integers(1, m)) for m in mods]          # one residue per prime of the context
    want = np.stack([h.orc.sud(p, minuend[i], coeff[i], fac[p]) for i, p in enumerate(idx)])
    dm, dc, out = h.up(minuend), h.up(coeff), h.new(len(idx), N)
    lb = N * h.ctx.word_bytes
    ins = np.empty(2 * len(idx), dtype=np.uint64)
    ins[0::2] = [h.p(dm) + i * lb for i in range(len(idx))]
    ins[1::2] = [h.p(dc) + i * lb for i in range(len(idx))]
    d_ins = be.to_dev(ins)
    d_outs = be.to_dev(np.array([h.p(out) + i * lb for i in range(len(idx))], dtype=np.uint64))
    d_bases = be.to_dev(np.array(idx, dtype=np.uint32))
    wdt = np.uint32 if word_bits == 32 else np.uint64
    d_fac = be.to_dev(np.array(fac, dtype=wdt))
    h.ctx.sud_ptrs(be.ptr(d_outs), be.ptr(d_ins), be.ptr(d_bases), len(idx), be.ptr(d_fac))
    assert np.array_equal(h.down(out), want)
    # in place on the coefficient-form input, as the reference's stage 0 / stage 1 pair allows
    d_outs2 = be.to_dev(ins[1::2].copy())
    h.ctx.sud_ptrs(be.ptr(d_outs2), be.ptr(d_ins), be.ptr(d_bases), len(idx), be.ptr(d_fac))
    assert np.array_equal(h.down(dc), want)


def case_bconv_ptrs(be, word_bits):
    """Base conversion from device tables only (shapes, factor matrices and output primes), two
    conversions of different shape in one launch, one of them with more than eight inputs."""
    n_mod = 36
    mods = moduli_for(word_bits, n_mod, 0)
    h = Harness(be, word_bits, mods)
    rng = np.random.default_rng(72)
    wdt = np.uint32 if word_bits == 32 else np.uint64
    # the last two take the 32-bit path for 9 to 32 inputs (13 inputs: padded rows; 17: two partial sums)
    shapes = [([0, 1, 2], [3, 4, 5, 6, 7]), (list(range(9)), [9, 10, 11, 12, 13]),
              (list(range(13)), list(range(13, 20))), (list(range(17)), list(range(17, 36)))]
    keep, outs, ins, facs, omods, wants, d_out = [], [], [], [], [], [], []
    for in_idx, out_idx in shapes:
        x = rand_limbs(rng, mods, in_idx)
        # F[j][i] = [Qhat_i^-1]_{q_i} * (Qhat_i mod p_j) mod p_j  (cerium/runtime/execution/evaluator.cpp:1539-1578)
        qs, ps = [mods[i] for i in in_idx], [mods[j] for j in out_idx]
        Q = 1
        for q in qs:
            Q *= q
        fac = [[pow(Q // q % q, -1, q) % pj * (Q // q % pj) % pj for q in qs] for pj in ps]
        wants.append(oracle.bconv(oracle.BCONV_LAZY, qs, x, ps))
        dx, do = h.up(x), h.new(len(out_idx), N)
        dfac = be.to_dev(np.asarray(fac, dtype=wdt).reshape(-1))
        dmod = be.to_dev(np.array([mods[j] for j in out_idx], dtype=wdt))
        keep += [dx, dfac, dmod]
        d_out.append(do)
        outs.append(h.p(do)); ins.append(h.p(dx)); facs.append(be.ptr(dfac)); omods.append(be.ptr(dmod))
    t = lambda v: be.to_dev(np.array(v, dtype=np.uint64))
    d_outs, d_ins, d_facs, d_omods = t(outs), t(ins), t(facs), t(omods)
    d_nin, d_nout = t([len(a) for a, _ in shapes]), t([len(b) for _, b in shapes])
    h.ctx.bconv_ptrs(be.ptr(d_outs), be.ptr(d_nout), be.ptr(d_ins), be.ptr(d_nin), be.ptr(d_facs), be.ptr(d_omods),
                     17, 19, len(shapes))
    for do, want in zip(d_out, wants):
        assert np.array_equal(h.down(do), want)
    # a table entry above the launch's shape bounds (9 inputs against max_in = 8) is skipped on the
    # device, not staged past the shared memory: its outputs stay untouched, the other conversion
    # runs, and the context reports it once
    import pytest
    h.ctx.check()
    for do in d_out:
        do[...] = 0 if isinstance(do, np.ndarray) else do.zero_()
    h.ctx.bconv_ptrs(be.ptr(d_outs), be.ptr(d_nout), be.ptr(d_ins), be.ptr(d_nin), be.ptr(d_facs), be.ptr(d_omods),
                     8, 5, len(shapes))
    with pytest.raises(_capi.CeriumError) as e:
        h.ctx.check()
    assert e.value.code == _capi.ERR_INVALID and "shape bounds" in e.value.message
    h.ctx.check()                                            # reading the status cleared it
    assert np.array_equal(h.down(d_out[0]), wants[0])
    for k in (1, 2, 3):
        assert not h.down(d_out[k]).any(), "an over-bound conversion wrote its outputs"


def case_ewise(be, word_bits):
    mods = moduli_for(word_bits, 3, 1)
    h = Harness(be, word_bits, mods)
    rng = np.random.default_rng(8)
    idx = [2, 0, 1, 0]
    a, b, c = (rand_limbs(rng, mods, idx) for _ in range(3))
    a[3] = edge_limbs(mods, [0])[0]
    b[3] = edge_limbs(mods, [0])[0]
    da, db, dc = h.up(a), h.up(b), h.up(c)
    out = h.new(len(idx), N)
    scal = [int(rng.integers(0, mods[p])) for p in idx]

    def expect(op, **kw):
        return np.stack([oracle.ew(op, mods[p], *[arr[i] for arr in kw["arrs"]], scalar=kw.get("scalars", [None] * 9)[i])
                         for i, p in enumerate(idx)])

    h.ctx.ewise(_capi.EW_ADD, h.p(out), h.p(da), idx, b=h.p(db))
    assert np.array_equal(h.down(out), expect("add", arrs=(a, b)))
    h.ctx.ewise(_capi.EW_SUB, h.p(out), h.p(da), idx, b=h.p(db))
    assert np.array_equal(h.down(out), expect("sub", arrs=(a, b)))
    h.ctx.ewise(_capi.EW_NEG, h.p(out), h.p(da), idx)
    assert np.array_equal(h.down(out), expect("neg", arrs=(a,)))
    h.ctx.ewise(_capi.EW_MUL, h.p(out), h.p(da), idx, b=h.p(db))
    assert np.array_equal(h.down(out), expect("mul", arrs=(a, b)))
    h.ctx.ewise(_capi.EW_MAD, h.p(out), h.p(da), idx, b=h.p(db), c=h.p(dc))
    assert np.array_equal(h.down(out), expect("mad", arrs=(a, b, c)))
    h.ctx.ewise(_capi.EW_PMU, h.p(out), h.p(da), idx, b=h.p(db), scalars=scal)
    assert np.array_equal(h.down(out), expect("pmu", arrs=(a, b), scalars=scal))
    h.ctx.ewise(_capi.EW_MUL_SCALAR, h.p(out), h.p(da), idx, scalars=scal)
    want = np.stack([oracle.ew("mul", mods[p], a[i], np.full(N, scal[i], dtype=np.uint64)) for i, p in enumerate(idx)])
    assert np.array_equal(h.down(out), want)
    # periodic plaintext: stored once per period, read as pt[i >> shift] (cuda_kernel.cc:919-934)
    for shift in (0, 1, 6):
        period = N >> shift
        pt = np.stack([rng.integers(0, mods[p], size=period, dtype=np.uint64) for p in idx])
        dpt = h.up(pt)
        full = np.repeat(pt, 1 << shift, axis=1)
        h.ctx.mul_plain_periodic(h.p(out), h.p(da), h.p(dpt), shift, idx)
        assert np.array_equal(h.down(out), expect("mul", arrs=(a, full))), "periodic plaintext product, shift %d" % shift
        h.ctx.mul_plain_periodic(h.p(out), h.p(da), h.p(dpt), shift, idx, addend=h.p(dc))
        assert np.array_equal(h.down(out), expect("mad", arrs=(a, full, c))), "periodic plaintext multiply-add, shift %d" % shift
    # tensor product
    a1, b1 = rand_limbs(rng, mods, idx), rand_limbs(rng, mods, idx)
    d0, d1, d2 = h.new(len(idx), N), h.new(len(idx), N), h.new(len(idx), N)
    da1, db1 = h.up(a1), h.up(b1)
    h.ctx.tensor(h.p(d0), h.p(d1), h.p(d2), h.p(da), h.p(da1), h.p(db), h.p(db1), idx)
    assert np.array_equal(h.down(d0), expect("mul", arrs=(a, b)))
    assert np.array_equal(h.down(d2), expect("mul", arrs=(a1, b1)))
    w = np.stack([oracle.ew("mad", mods[p], a[i], b1[i], oracle.ew("mul", mods[p], a1[i], b[i])) for i, p in enumerate(idx)])
    assert np.array_equal(h.down(d1), w)


def case_automorph(be, word_bits):
    mods = moduli_for(word_bits, 2, 0)
    h = Harness(be, word_bits, mods)
    rng = np.random.default_rng(9)
    idx = [0, 1]
    x = rand_limbs(rng, mods, idx)
    dx = h.up(x)
    out = h.new(2, N)
    for step in (0, 1, 7, -3, 12345, -(N // 2 - 1)):
        elt = be.lib.galois_elt_from_step(step, LOGN)
        assert elt == oracle.galois_elt_from_step(step, LOGN)
        h.ctx.automorph(h.p(out), h.p(dx), elt, 2)
        want = np.stack([oracle.apply_galois_ntt(elt, LOGN, x[i]) for i in range(2)])
        assert np.array_equal(h.down(out), want), "automorphism differs for step %d" % step
    assert be.lib.galois_elt_from_step(N // 2, LOGN) == 0  # step count too large


def case_bconv(be, word_bits, n_in, n_out, mode):
    mods = moduli_for(word_bits, n_in + n_out, min(2, n_in))
    h = Harness(be, word_bits, mods)
    rng = np.random.default_rng(10 + n_in)
    in_idx = list(range(n_in))
    out_idx = list(range(n_in, n_in + n_out))
    x = rand_limbs(rng, mods, in_idx)
    x[0, :8] = mods[0] - 1
    for i in in_idx:
        x[i, 8:16] = mods[i] - 1                          # every residue at its maximum: the largest sums
    dx = h.up(x)
    out = h.new(n_out, N)
    bc = _capi.BaseConverter(h.ctx, in_idx, out_idx, mode)
    bc.apply(h.p(out), h.p(dx))
    want = oracle.bconv(mode, [mods[i] for i in in_idx], x, [mods[j] for j in out_idx])
    assert np.array_equal(h.down(out), want), "base conversion differs (mode %d, %d -> %d)" % (mode, n_in, n_out)
    # two conversions in one launch (second on shifted data)
    x2 = np.roll(x, 3, axis=1)
    dx2 = h.up(x2)
    out2 = h.new(n_out, N)
    out1 = h.new(n_out, N)
    _capi.BaseConverter.apply_batch([bc, bc], [h.p(out1), h.p(out2)], [h.p(dx), h.p(dx2)])
    assert np.array_equal(h.down(out1), want)
    assert np.array_equal(h.down(out2), np.roll(want, 3, axis=1))
    bc.close()


def case_sud(be, word_bits):
    mods = moduli_for(word_bits, 5, 1)
    h = Harness(be, word_bits, mods)
    rng = np.random.default_rng(11)
    idx = [0, 1, 2]
    div = [3, 4]
    minuend = rand_limbs(rng, mods, idx)
    coeff = rand_limbs(rng, mods, idx)
    addend = rand_limbs(rng, mods, idx)
    want = []
    for i, p in enumerate(idx):
        q = mods[p]
        f = pow(mods[3] * mods[4] % q, -1, q)
        want.append(h.orc.sud(p, minuend[i], coeff[i], f))
    want = np.stack(want)
    dm, dc, da = h.up(minuend), h.up(coeff), h.up(addend)
    out = h.new(3, N)
    h.ctx.sud(h.p(out), h.p(dm), h.p(dc), idx, div)
    assert np.array_equal(h.down(out), want)
    dc = h.up(coeff)
    h.ctx.sud(h.p(dm), h.p(dm), h.p(dc), idx, div, addend=h.p(da))  # in place on the minuend, with addend
    want2 = np.stack([oracle.ew("add", mods[p], want[i], addend[i]) for i, p in enumerate(idx)])
    assert np.array_equal(h.down(dm), want2)


def case_u32_widest_primes(be):
    """32-bit words with primes just below 2^30, the widest the library accepts: sums such as
    minuend + 4q pass 2^32 there, which the 28-bit reference chain never shows."""
    global _U32_BITS
    _U32_BITS = 30
    try:
        assert min(moduli_for(32, 6)) > 0.99 * 2**30
        case_sud(be, 32)
        case_bconv(be, 32, 15, 3, _capi.BCONV_LAZY)          # fifteen products just below 2^60 in one 64-bit sum:
        case_bconv(be, 32, 15, 2, _capi.BCONV_EXACT)         # the most inputs the library takes at this width
        case_rescale(be, 32, 0)
        case_rescale(be, 32, 1, L=3, n_polys=1)
        case_double_rescale(be, 32)
    finally:
        _U32_BITS = 28


def case_rescale(be, word_bits, round_mode, L=4, n_polys=2):
    mods = moduli_for(word_bits, L, 1)
    if word_bits == 64:
        mods = mods[1:] + mods[:1]   # 60-bit prime last: the dropped limb is wider than the rest
    h = Harness(be, word_bits, mods)
    rng = np.random.default_rng(12)
    q_idx = list(range(L))
    x = np.stack([rand_limbs(rng, mods, q_idx) for _ in range(n_polys)])
    dx = h.up(x)
    out = h.new(n_polys, L - 1, N)
    scratch = h.new(n_polys, N)
    h.ctx.rescale(h.p(out), h.p(dx), q_idx, n_polys, h.p(scratch), round_mode)
    want = np.stack([h.orc.rescale(round_mode, q_idx, x[p]) for p in range(n_polys)])
    assert np.array_equal(h.down(out), want)


def case_mod_raise(be, word_bits, bconv_mode, round_mode, Lt=4, K=2):
    """Bootstrap ModRaise: two base limbs -> Lt target limbs through an exact lift, a one-digit key
    switch over Lt + 1 + K limbs, ModDown and a rescale."""
    if word_bits == 32:
        mods = moduli_for(32, Lt + 1 + K)
        q_idx, p_idx = list(range(Lt + 1)), list(range(Lt + 1, Lt + 1 + K))
    else:
        mods = moduli_for(64, Lt + 1 + K, K)          # the K 60-bit primes first
        q_idx, p_idx = list(range(K, K + Lt + 1)), list(range(K))
    h = Harness(be, word_bits, mods)
    rng = np.random.default_rng(33)
    base = [q_idx[0], q_idx[1]]                        # the level-2 ciphertext lives on the first two primes
    c0, c1 = rand_limbs(rng, mods, base), rand_limbs(rng, mods, base)
    evk = np.stack([rand_limbs(rng, mods, q_idx + p_idx) for _ in range(2)])
    ks = _capi.KeySwitch(h.ctx, q_idx, p_idx, 1, bconv_mode, round_mode, lifted=True)
    o0, o1 = h.new(Lt, N), h.new(Lt, N)
    d0, d1, dk = h.up(c0), h.up(c1), h.up(evk)
    ks.mod_raise(h.p(o0), h.p(o1), h.p(d0), h.p(d1), base[0], base[1], h.p(dk))
    w0, w1 = h.orc.mod_raise(bconv_mode, round_mode, q_idx, p_idx, base[0], base[1], c0, c1, evk)
    assert np.array_equal(h.down(o0), w0), "ModRaise c0 differs"
    assert np.array_equal(h.down(o1), w1), "ModRaise c1 differs"
    # a lifted plan serves nothing else
    try:
        ks.apply(h.p(o0), h.p(o1), h.p(o0), h.p(dk))
    except _capi.CeriumError:
        pass
    else:
        raise AssertionError("a lifted plan accepted an ordinary key switch")


def case_double_rescale(be, word_bits, L=5, n_polys=3):
    """Two limbs dropped at once (INTT x2, Resolve, Mod, SuD); one pair of polynomials and a single."""
    mods = moduli_for(word_bits, L, 1)
    if word_bits == 64:
        mods = mods[1:] + mods[:1]   # the 60-bit prime is one of the two dropped ones
    h = Harness(be, word_bits, mods)
    rng = np.random.default_rng(21)
    q_idx = list(range(L))
    x = np.stack([rand_limbs(rng, mods, q_idx) for _ in range(n_polys)])
    dx = h.up(x)
    out = h.new(n_polys, L - 2, N)
    scratch = h.new(4 * n_polys, N)
    h.ctx.double_rescale(h.p(out), h.p(dx), q_idx, n_polys, h.p(scratch))
    want = np.stack([h.orc.double_rescale(q_idx, x[p]) for p in range(n_polys)])
    assert np.array_equal(h.down(out), want)


def case_resolve_mod(be, word_bits):
    """Two-limb CRT composition and its reduction modulo other primes (ModRaise building blocks)."""
    mods = moduli_for(word_bits, 5, 1)
    h = Harness(be, word_bits, mods)
    rng = np.random.default_rng(14)
    p0, p1 = 1, 2
    x = np.stack([rand_limbs(rng, mods, [p0, p1]) for _ in range(2)])   # 2 polynomials x 2 limbs
    x[1, 0, :4] = mods[p0] - 1
    x[1, 1, :4] = mods[p1] - 1
    d0, d1 = h.up(x[:, 0]), h.up(x[:, 1])
    lo, hi = h.new(2, N), h.new(2, N)
    h.ctx.resolve2(h.p(lo), h.p(hi), h.p(d0), h.p(d1), p0, p1, count=2)
    glo, ghi = h.down(lo), h.down(hi)
    shift = 64 if word_bits == 64 else 32
    for k in range(2):
        wlo, whi = oracle.resolve2(mods[p0], mods[p1], x[k, 0], x[k, 1])
        if word_bits == 64:
            assert np.array_equal(glo[k], wlo) and np.array_equal(ghi[k], whi)
        else:
            assert np.array_equal(glo[k] | (ghi[k] << np.uint64(32)), wlo) and not whi.any()
    # big-integer spot check of the CRT property
    for c in (0, 1, 2, 3, N - 1):
        v = (int(ghi[1, c]) << shift) | int(glo[1, c])
        assert v < mods[p0] * mods[p1] and v % mods[p0] == int(x[1, 0, c]) and v % mods[p1] == int(x[1, 1, c])
    # reduce the first composite modulo every prime of the context
    idx = list(range(len(mods)))
    out = h.new(len(idx), N)
    lo0, hi0 = h.up(glo[0]), h.up(ghi[0])
    h.ctx.mod2(h.p(out), h.p(lo0), h.p(hi0), idx)
    got = h.down(out)
    wlo, whi = oracle.resolve2(mods[p0], mods[p1], x[0, 0], x[0, 1])
    for i, p in enumerate(idx):
        assert np.array_equal(got[i], oracle.mod2(mods[p], wlo, whi))
    assert np.array_equal(got[p0], x[0, 0]) and np.array_equal(got[p1], x[0, 1])


def make_keyswitch_inputs(rng, prm: params.CkksParams):
    all_idx = prm.q_idx + prm.p_idx
    c0 = rand_limbs(rng, prm.moduli, prm.q_idx)
    c1 = rand_limbs(rng, prm.moduli, prm.q_idx)
    evk = np.stack([np.stack([rand_limbs(rng, prm.moduli, all_idx) for _ in range(2)]) for _ in range(prm.dnum)])
    return c0, c1, evk


def small_params(word_bits, L, K, dnum):
    if word_bits == 32:
        return params.config_ref28(LOGN, L, K, dnum, total=L + K)
    q = params.ntt_primes_below(60, 1, LOGN) + params.ntt_primes_below(50, L - 1, LOGN)
    p = params.ntt_primes_below(60, K + 1, LOGN)[1:]
    return params.CkksParams(LOGN, 64, q + p[::-1], L, K, dnum)


def case_keyswitch(be, word_bits, L, K, dnum, bconv_mode, round_mode):
    prm = small_params(word_bits, L, K, dnum)
    h = Harness(be, word_bits, prm.moduli)
    rng = np.random.default_rng(13)
    c0, c1, evk = make_keyswitch_inputs(rng, prm)
    ks = _capi.KeySwitch(h.ctx, prm.q_idx, prm.p_idx, dnum, bconv_mode, round_mode)
    assert ks.workspace_bytes > 0
    d_c1, d_evk = h.up(c1), h.up(evk)
    o0, o1 = h.new(L, N), h.new(L, N)
    ks.apply(h.p(o0), h.p(o1), h.p(d_c1), h.p(d_evk))
    w0, w1 = h.orc.keyswitch(bconv_mode, round_mode, prm.q_idx, prm.p_idx, dnum, c1, evk)
    assert np.array_equal(h.down(o0), w0), "key switch c0 differs"
    assert np.array_equal(h.down(o1), w1), "key switch c1 differs"
    # HRot
    elt = be.lib.galois_elt_from_step(5, LOGN)
    d_c0 = h.up(c0)
    ks.hrot(h.p(o0), h.p(o1), h.p(d_c0), h.p(d_c1), h.p(d_evk), elt)
    w0, w1 = h.orc.hrot(bconv_mode, round_mode, prm.q_idx, prm.p_idx, dnum, elt, c0, c1, evk)
    assert np.array_equal(h.down(o0), w0), "HRot c0 differs"
    assert np.array_equal(h.down(o1), w1), "HRot c1 differs"
    # in place (outputs = inputs): the library rotates into its workspace first instead of folding the
    # rotation into the key switch's reads
    i0, i1 = h.up(c0), h.up(c1)
    ks.hrot(h.p(i0), h.p(i1), h.p(i0), h.p(i1), h.p(d_evk), elt)
    assert np.array_equal(h.down(i0), w0) and np.array_equal(h.down(i1), w1), "in-place HRot differs"
    # hoisted rotations: one ModUp, several rotations with pre-permuted keys
    ks.hoisted_begin(h.p(d_c1))
    for step in (1, -2):
        e2 = be.lib.galois_elt_from_step(step, LOGN)
        k0, k1 = h.orc.keyswitch(bconv_mode, round_mode, prm.q_idx, prm.p_idx, dnum, c1, evk)
        k0 = np.stack([oracle.ew("add", prm.moduli[p], k0[i], c0[i]) for i, p in enumerate(prm.q_idx)])
        w0 = np.stack([oracle.apply_galois_ntt(e2, LOGN, k0[i]) for i in range(L)])
        w1 = np.stack([oracle.apply_galois_ntt(e2, LOGN, k1[i]) for i in range(L)])
        ks.hoisted_rotate(h.p(o0), h.p(o1), h.p(d_c0), h.p(d_c1), h.p(d_evk), e2)
        assert np.array_equal(h.down(o0), w0) and np.array_equal(h.down(o1), w1), "hoisted rotation differs"
    # the last one again with the outputs on top of the inputs (separate automorphism pass)
    i0, i1 = h.up(c0), h.up(c1)
    ks.hoisted_rotate(h.p(i0), h.p(i1), h.p(i0), h.p(i1), h.p(d_evk), e2)
    assert np.array_equal(h.down(i0), w0) and np.array_equal(h.down(i1), w1), "in-place hoisted rotation differs"
    # HMult + relinearise, with and without rescale
    b0, b1 = rand_limbs(rng, prm.moduli, prm.q_idx), rand_limbs(rng, prm.moduli, prm.q_idx)
    d_b0, d_b1 = h.up(b0), h.up(b1)
    ks.hmult(h.p(o0), h.p(o1), h.p(d_c0), h.p(d_c1), h.p(d_b0), h.p(d_b1), h.p(d_evk), False)
    w0, w1 = h.orc.hmult_relin(bconv_mode, round_mode, False, prm.q_idx, prm.p_idx, dnum, c0, c1, b0, b1, evk)
    assert np.array_equal(h.down(o0), w0) and np.array_equal(h.down(o1), w1), "HMult differs"
    if L >= 2:
        r0, r1 = h.new(L - 1, N), h.new(L - 1, N)
        ks.hmult(h.p(r0), h.p(r1), h.p(d_c0), h.p(d_c1), h.p(d_b0), h.p(d_b1), h.p(d_evk), True)
        w0, w1 = h.orc.hmult_relin(bconv_mode, round_mode, True, prm.q_idx, prm.p_idx, dnum, c0, c1, b0, b1, evk)
        assert np.array_equal(h.down(r0), w0) and np.array_equal(h.down(r1), w1), "HMult+rescale differs"
    ks.close()


def case_keyswitch_rescale(be, word_bits, L, K, dnum, bconv_mode, round_mode):
    """Key switch with the PMU pre-additions and 1 / 2 rescale levels inside the ModDown, and the
    HMult that folds its rescale into the relinearisation's ModDown."""
    prm = small_params(word_bits, L, K, dnum)
    h = Harness(be, word_bits, prm.moduli)
    rng = np.random.default_rng(17)
    c0, c1, evk = make_keyswitch_inputs(rng, prm)
    a0, a1 = rand_limbs(rng, prm.moduli, prm.q_idx), rand_limbs(rng, prm.moduli, prm.q_idx)
    ks = _capi.KeySwitch(h.ctx, prm.q_idx, prm.p_idx, dnum, bconv_mode, round_mode)
    d_c1, d_evk, d_a0, d_a1 = h.up(c1), h.up(evk), h.up(a0), h.up(a1)
    for r in (0, 1, 2):
        if L - r < 1:
            continue
        o0, o1 = h.new(L - r, N), h.new(L - r, N)
        ks.apply_rescale(h.p(o0), h.p(o1), h.p(d_c1), h.p(d_evk), r, h.p(d_a0), h.p(d_a1))
        w0, w1 = h.orc.keyswitch_rescale(bconv_mode, round_mode, prm.q_idx, prm.p_idx, dnum, r, c1, evk, a0, a1)
        assert np.array_equal(h.down(o0), w0) and np.array_equal(h.down(o1), w1), "key switch with %d rescale levels differs" % r
        ks.apply_rescale(h.p(o0), h.p(o1), h.p(d_c1), h.p(d_evk), r)          # without pre-additions
        w0, w1 = h.orc.keyswitch_rescale(bconv_mode, round_mode, prm.q_idx, prm.p_idx, dnum, r, c1, evk)
        assert np.array_equal(h.down(o0), w0) and np.array_equal(h.down(o1), w1)
    if L >= 2:
        d_c0 = h.up(c0)
        r0, r1 = h.new(L - 1, N), h.new(L - 1, N)
        ks.hmult(h.p(r0), h.p(r1), h.p(d_c0), h.p(d_c1), h.p(d_a0), h.p(d_a1), h.p(d_evk), 2)
        w0, w1 = h.orc.hmult_relin_fused(bconv_mode, round_mode, prm.q_idx, prm.p_idx, dnum, c0, c1, a0, a1, evk)
        assert np.array_equal(h.down(r0), w0) and np.array_equal(h.down(r1), w1), "HMult with the fused rescale differs"
    ks.close()


def case_bsgs(be, word_bits, L, K, dnum, bconv_mode, round_mode, g=3, n_giant=3, r=0, missing=((1, 2),),
              prm=None, zero_first=True):
    """cerium_bsgs_apply against the oracle's restatement of the reference lowering: hoisted baby steps,
    plaintext products summed per giant step, giant-step key switches accumulated in the extended basis,
    one ModDown (with r rescale levels).  `missing` lists absent diagonals (giant, baby)."""
    prm = prm or small_params(word_bits, L, K, dnum)
    L, K, dnum = prm.L, prm.K, prm.dnum
    h = Harness(be, word_bits, prm.moduli)
    rng = np.random.default_rng(19)
    c0, c1, _ = make_keyswitch_inputs(rng, prm)
    all_idx = prm.q_idx + prm.p_idx
    key = lambda: np.stack([np.stack([rand_limbs(rng, prm.moduli, all_idx) for _ in range(2)]) for _ in range(dnum)])  # noqa: E731
    baby_elts = [1] + [be.lib.galois_elt_from_step(j, LOGN) for j in range(1, g)]
    giant_elts = [1 if (i == 0 and zero_first) else be.lib.galois_elt_from_step(g * i + (0 if zero_first else g), LOGN)
                  for i in range(n_giant)]
    baby_keys = [None] + [key() for _ in range(1, g)]
    giant_keys = [None if e == 1 else key() for e in giant_elts]
    present = np.ones((n_giant, g), dtype=np.uint8)
    for (i, j) in missing:
        if i < n_giant and j < g:
            present[i, j] = 0
    pts = np.stack([np.stack([rand_limbs(rng, prm.moduli, prm.q_idx) for _ in range(g)]) for _ in range(n_giant)])
    # oracle: baby steps as the hoisted rotations define them, then the lowering
    baby = [np.stack([c0, c1])]
    for j in range(1, g):
        k0, k1 = h.orc.keyswitch(bconv_mode, round_mode, prm.q_idx, prm.p_idx, dnum, c1, baby_keys[j])
        k0 = np.stack([oracle.ew("add", prm.moduli[p], k0[i], c0[i]) for i, p in enumerate(prm.q_idx)])
        baby.append(np.stack([np.stack([oracle.apply_galois_ntt(baby_elts[j], LOGN, k[i]) for i in range(L)]) for k in (k0, k1)]))
    zero_key = np.zeros_like(key())
    w0, w1 = h.orc.bsgs(bconv_mode, round_mode, prm.q_idx, prm.p_idx, dnum, r, np.stack(baby), pts, present, giant_elts,
                        np.stack([zero_key if k is None else k for k in giant_keys]))
    # device
    ks = _capi.KeySwitch(h.ctx, prm.q_idx, prm.p_idx, dnum, bconv_mode, round_mode)
    d_c0, d_c1 = h.up(c0), h.up(c1)
    d_pts = [[h.up(pts[i, j]) if present[i, j] else None for j in range(g)] for i in range(n_giant)]
    d_bk = [None] + [h.up(baby_keys[j]) for j in range(1, g)]    # taken as the pre-permuted keys, as the oracle does above
    d_gk = [None if k is None else h.up(k) for k in giant_keys]
    work = h.new(ks.bsgs_work_limbs(g, n_giant), N)
    o0, o1 = h.new(L - r, N), h.new(L - r, N)
    for _ in range(2):                                          # twice: the plan's accumulators are reused
        ks.bsgs_apply(h.p(o0), h.p(o1), h.p(d_c0), h.p(d_c1), g, n_giant,
                      [h.p(t) if t is not None else 0 for row in d_pts for t in row],
                      [h.p(t) if t is not None else 0 for t in d_bk], baby_elts,
                      [h.p(t) if t is not None else 0 for t in d_gk], giant_elts, r, h.p(work))
        assert np.array_equal(h.down(o0), w0), "BSGS c0 differs"
        assert np.array_equal(h.down(o1), w1), "BSGS c1 differs"
    ks.close()


def case_errors(be, word_bits=64):
    """Error behaviour of the boundary: status codes and messages instead of exceptions or faults."""
    import pytest
    mods = moduli_for(word_bits, 2, 0)
    with pytest.raises(_capi.CeriumError) as e:
        _capi.Context(be.lib, [mods[0], mods[0]], word_bits)
    assert e.value.code == _capi.ERR_INVALID
    with pytest.raises(_capi.CeriumError):
        _capi.Context(be.lib, [mods[0] + 2], word_bits)          # not prime / not 1 mod 2N
    with pytest.raises(_capi.CeriumError) as e:
        _capi.Context(be.lib, mods, word_bits, logn=15)
    assert e.value.code == _capi.ERR_UNSUPPORTED
    h = Harness(be, word_bits, mods)
    buf = h.new(2, N)
    with pytest.raises(_capi.CeriumError):
        h.ctx.ntt_forward(h.p(buf), h.p(buf), [0, 5])             # unknown prime index
    with pytest.raises(_capi.CeriumError):
        h.ctx.ntt_forward(0, h.p(buf), [0])                       # null pointer
    with pytest.raises(_capi.CeriumError):
        h.ctx.ntt_forward(h.p(buf) + 8, h.p(buf), [0])            # misaligned
    with pytest.raises(_capi.CeriumError):
        h.ctx.automorph(h.p(buf), h.p(buf), 5, 1)                 # aliasing
    with pytest.raises(_capi.CeriumError):
        h.ctx.automorph(h.p(buf), h.p(buf) + N * h.ctx.word_bytes, 4, 1)  # even Galois element
    with pytest.raises(_capi.CeriumError):
        _capi.KeySwitch(h.ctx, [0, 1], [1], 1)                    # prime used twice
    with pytest.raises(_capi.CeriumError):
        _capi.KeySwitch(h.ctx, [0], [1], 2)                       # dnum > L
    with pytest.raises(_capi.CeriumError):
        h.ctx.double_rescale(h.p(buf), h.p(buf), [0, 1], 1, h.p(buf))            # fewer than 3 limbs
    with pytest.raises(_capi.CeriumError):
        h.ctx.rescale_local(h.p(buf), h.p(buf), [0], 0, h.p(buf), 1)             # local prime = dropped prime
    with pytest.raises(_capi.CeriumError):
        _capi.KeySwitch(h.ctx, [0], [1], 1, lifted=True)                         # a lifted plan needs L >= 4
    ks = _capi.KeySwitch(h.ctx, [0], [1], 1)
    with pytest.raises(_capi.CeriumError):
        ks.mod_raise(h.p(buf), h.p(buf), h.p(buf), h.p(buf), 0, 1, h.p(buf))     # not a lifted plan
