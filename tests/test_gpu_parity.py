"""Parity tests proper: the CUDA build, called through the C ABI on cuda:0, against the CPU
oracle on the same seeded inputs (bit-exact: integer work, canonical residues both sides)."""
import numpy as np
import pytest

from cerium_b200 import _capi, params
from tests import parity_cases as pc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def be():
    from tests.backends import CudaBackend
    return CudaBackend()


@pytest.mark.parametrize("word_bits", [32, 64])
def test_ntt(be, word_bits):
    pc.case_ntt(be, word_bits, n_limbs=6, sixty=2)


def test_ntt_fp_extremes(be):
    pc.case_ntt_fp_extremes(be)


@pytest.mark.parametrize("word_bits", [32, 64])
def test_ntt_pointer_tables(be, word_bits):
    pc.case_ntt_ptrs(be, word_bits)


@pytest.mark.parametrize("word_bits", [32, 64])
def test_ewise_and_tensor(be, word_bits):
    pc.case_ewise(be, word_bits)


@pytest.mark.parametrize("word_bits", [32, 64])
def test_automorph(be, word_bits):
    pc.case_automorph(be, word_bits)


@pytest.mark.parametrize("word_bits,n_in,n_out,mode", [
    (64, 1, 3, _capi.BCONV_LAZY), (64, 5, 35, _capi.BCONV_LAZY), (64, 5, 35, _capi.BCONV_EXACT),
    (64, 8, 4, _capi.BCONV_EXACT), (64, 24, 6, _capi.BCONV_LAZY), (64, 48, 16, _capi.BCONV_EXACT),
    (32, 5, 30, _capi.BCONV_LAZY), (32, 18, 12, _capi.BCONV_LAZY), (32, 48, 16, _capi.BCONV_LAZY),
    (32, 13, 51, _capi.BCONV_LAZY), (32, 16, 47, _capi.BCONV_EXACT), (32, 17, 34, _capi.BCONV_LAZY), (32, 28, 28, _capi.BCONV_LAZY),
    (32, 32, 8, _capi.BCONV_LAZY), (32, 33, 8, _capi.BCONV_LAZY),
])
def test_bconv(be, word_bits, n_in, n_out, mode):
    pc.case_bconv(be, word_bits, n_in, n_out, mode)


@pytest.mark.parametrize("word_bits", [32, 64])
def test_sud(be, word_bits):
    pc.case_sud(be, word_bits)


@pytest.mark.parametrize("word_bits", [32, 64])
def test_reference_launcher_tables(be, word_bits):
    pc.case_sud_ptrs(be, word_bits)
    pc.case_bconv_ptrs(be, word_bits)


def test_u32_widest_primes(be):
    pc.case_u32_widest_primes(be)


@pytest.mark.parametrize("word_bits,round_mode", [
    (64, _capi.ROUND_FLOOR), (64, _capi.ROUND_HALF), (32, _capi.ROUND_FLOOR), (32, _capi.ROUND_HALF)])
def test_rescale(be, word_bits, round_mode):
    pc.case_rescale(be, word_bits, round_mode, L=6, n_polys=3)   # one pair and a single


@pytest.mark.parametrize("word_bits,L,K,dnum,bm,rm", [
    (64, 4, 2, 2, _capi.BCONV_LAZY, _capi.ROUND_FLOOR),
    (64, 6, 1, 6, _capi.BCONV_EXACT, _capi.ROUND_HALF),    # one digit per limb, one special prime
    (64, 7, 3, 3, _capi.BCONV_EXACT, _capi.ROUND_HALF),    # ragged digits 3, 2, 2
    (64, 9, 3, 3, _capi.BCONV_LAZY, _capi.ROUND_HALF),
    (32, 8, 4, 2, _capi.BCONV_LAZY, _capi.ROUND_FLOOR),
    (32, 6, 2, 3, _capi.BCONV_EXACT, _capi.ROUND_FLOOR),
    (32, 5, 1, 5, _capi.BCONV_LAZY, _capi.ROUND_FLOOR),    # one-limb digits, 32-bit
    (32, 12, 12, 1, _capi.BCONV_EXACT, _capi.ROUND_HALF),  # the reference examples' shape: conversions of 12 inputs
    (32, 24, 13, 2, _capi.BCONV_LAZY, _capi.ROUND_FLOOR),  # two digits of 12 limbs, 13 extension limbs
])
def test_keyswitch_hrot_hmult(be, word_bits, L, K, dnum, bm, rm):
    pc.case_keyswitch(be, word_bits, L, K, dnum, bm, rm)


@pytest.mark.parametrize("word_bits,L,K,dnum,bm,rm", [
    (64, 7, 3, 3, _capi.BCONV_EXACT, _capi.ROUND_HALF),
    (64, 6, 1, 6, _capi.BCONV_EXACT, _capi.ROUND_HALF),
    (64, 9, 3, 3, _capi.BCONV_LAZY, _capi.ROUND_FLOOR),
    (32, 8, 4, 2, _capi.BCONV_LAZY, _capi.ROUND_FLOOR),
    (32, 6, 2, 3, _capi.BCONV_EXACT, _capi.ROUND_HALF),
])
def test_keyswitch_with_fused_rescale(be, word_bits, L, K, dnum, bm, rm):
    pc.case_keyswitch_rescale(be, word_bits, L, K, dnum, bm, rm)


@pytest.mark.parametrize("word_bits,L,K,dnum,bm,rm,g,n_giant,r", [
    (64, 7, 3, 3, _capi.BCONV_EXACT, _capi.ROUND_HALF, 3, 3, 0),
    (64, 7, 3, 3, _capi.BCONV_EXACT, _capi.ROUND_HALF, 4, 6, 2),     # two groups of giant steps, double rescale level
    (64, 5, 2, 3, _capi.BCONV_LAZY, _capi.ROUND_FLOOR, 1, 3, 1),     # no baby rotation at all
    (32, 8, 4, 2, _capi.BCONV_LAZY, _capi.ROUND_FLOOR, 3, 5, 1),
])
def test_bsgs(be, word_bits, L, K, dnum, bm, rm, g, n_giant, r):
    pc.case_bsgs(be, word_bits, L, K, dnum, bm, rm, g=g, n_giant=n_giant, r=r)


def test_bsgs_every_giant_step_rotated(be):
    pc.case_bsgs(be, 64, 5, 2, 3, _capi.BCONV_EXACT, _capi.ROUND_HALF, g=2, n_giant=2, r=0, missing=(), zero_first=False)


@pytest.mark.parametrize("word_bits,bm,rm", [(64, _capi.BCONV_EXACT, _capi.ROUND_HALF), (64, _capi.BCONV_LAZY, _capi.ROUND_FLOOR), (32, _capi.BCONV_LAZY, _capi.ROUND_FLOOR)])
def test_mod_raise(be, word_bits, bm, rm):
    pc.case_mod_raise(be, word_bits, bm, rm)


@pytest.mark.parametrize("word_bits", [32, 64])
def test_double_rescale(be, word_bits):
    pc.case_double_rescale(be, word_bits)


@pytest.mark.parametrize("word_bits", [32, 64])
def test_resolve_and_mod(be, word_bits):
    pc.case_resolve_mod(be, word_bits)


def test_error_codes(be):
    pc.case_errors(be)


def test_ntt_full_batch_properties(be):
    """The benchmark's NTT shape (48 limbs x 8 polynomials, 50-bit primes): the oracle checks a
    sample of limbs; size-independent properties cover the rest (round trip = identity,
    linearity of the transform)."""
    mods = params.config_ntt(16, 48)
    h = pc.Harness(be, 64, mods)
    torch = be.torch
    idx = [l for _ in range(8) for l in range(48)]
    g = torch.Generator(device="cuda").manual_seed(1234)
    q = torch.tensor([mods[i] for i in idx], dtype=torch.int64, device="cuda").view(-1, 1)
    x = torch.randint(0, 1 << 49, (len(idx), pc.N), dtype=torch.int64, device="cuda", generator=g) % q
    y = torch.randint(0, 1 << 49, (len(idx), pc.N), dtype=torch.int64, device="cuda", generator=g) % q
    fx, fy, fs = torch.empty_like(x), torch.empty_like(x), torch.empty_like(x)
    h.ctx.ntt_forward(fx.data_ptr(), x.data_ptr(), idx)
    h.ctx.ntt_forward(fy.data_ptr(), y.data_ptr(), idx)
    s = (x + y) % q
    h.ctx.ntt_forward(fs.data_ptr(), s.data_ptr(), idx)
    assert torch.equal(fs, (fx + fy) % q), "NTT is not linear"
    assert bool((fx >= 0).all()) and bool((fx < q).all()), "NTT output is not canonical"
    back = torch.empty_like(x)
    h.ctx.ntt_inverse(back.data_ptr(), fx.data_ptr(), idx)
    assert torch.equal(back, x), "iNTT(NTT(x)) != x"
    sample = [0, 47, 48 * 3 + 17, 48 * 7 + 47]
    want = h.orc.ntt_forward(be.to_host(x[sample].contiguous()), [idx[i] for i in sample])
    assert np.array_equal(be.to_host(fx[sample].contiguous()), want)


def test_host_pipeline_matches_direct_calls(be):
    """The three-stream host pipeline returns, per submitted operation, what the direct call returns
    (ring of 3 slots, 7 operations, so every slot is reused)."""
    import numpy as np
    from cerium_b200.host_pipeline import HostPipeline
    torch = be.torch
    import oracle
    mods = pc.moduli_for(64, 4, 1)
    ctx = _capi.Context(be.lib, mods, 64)
    idx = [0, 1, 2, 3]
    rng = np.random.default_rng(7)

    def op(ins, outs, stream):
        ctx.ntt_forward(outs[0].data_ptr(), ins[0].data_ptr(), idx, stream=stream)

    pipe = HostPipeline(torch, [(4, pc.N)], [(4, pc.N)], op)
    hosts, slots = [], []
    for k in range(7):
        x = np.stack([rng.integers(0, mods[i], size=pc.N, dtype=np.uint64) for i in idx])
        h = torch.from_numpy(x.view(np.int64)).pin_memory()
        hosts.append((x, h))
        slot = pipe.submit([h])
        if k >= 2:
            # read the result of operation k - 2 while k and k - 1 are in flight
            got = pipe.wait((k - 2) % 3)[0].numpy().view(np.uint64).copy()
            slots.append((k - 2, got))
    pipe.drain()
    for k in (5, 6):
        slots.append((k, pipe.host_out[k % 3][0].numpy().view(np.uint64).copy()))
    orc = oracle.OracleContext(pc.LOGN, mods)
    for k, got in slots:
        assert np.array_equal(got, orc.ntt_forward(hosts[k][0], idx)), "operation %d" % k
