"""Kernel sources compiled for the host (tests/emu) against the oracle: checks the index
arithmetic of every kernel and the host orchestration without a GPU.  These are not the
parity tests proper (those run the CUDA build, tests/test_gpu_parity.py)."""
import pytest

from cerium_b200 import _capi
from tests import parity_cases as pc
from tests.backends import EmuBackend


@pytest.fixture(scope="module")
def be():
    return EmuBackend()


@pytest.mark.parametrize("word_bits", [32, 64])
def test_ntt(be, word_bits):
    pc.case_ntt(be, word_bits, n_limbs=2)


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
    (64, 1, 3, _capi.BCONV_LAZY), (64, 3, 5, _capi.BCONV_LAZY), (64, 3, 5, _capi.BCONV_EXACT),
    (64, 6, 2, _capi.BCONV_EXACT), (64, 10, 3, _capi.BCONV_LAZY),
    (32, 5, 4, _capi.BCONV_LAZY), (32, 9, 3, _capi.BCONV_EXACT), (32, 13, 5, _capi.BCONV_LAZY),
    (32, 16, 3, _capi.BCONV_EXACT), (32, 17, 2, _capi.BCONV_LAZY), (32, 32, 2, _capi.BCONV_LAZY), (32, 33, 2, _capi.BCONV_LAZY),
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


@pytest.mark.parametrize("word_bits,round_mode", [(64, _capi.ROUND_FLOOR), (64, _capi.ROUND_HALF), (32, _capi.ROUND_FLOOR)])
def test_rescale(be, word_bits, round_mode):
    pc.case_rescale(be, word_bits, round_mode, L=3, n_polys=3)   # one pair and a single


@pytest.mark.parametrize("word_bits,L,K,dnum,bm,rm", [
    (64, 4, 2, 2, _capi.BCONV_LAZY, _capi.ROUND_FLOOR),
    (64, 3, 1, 3, _capi.BCONV_EXACT, _capi.ROUND_HALF),
    (64, 5, 2, 3, _capi.BCONV_EXACT, _capi.ROUND_HALF),   # ragged digits: sizes 2, 2, 1
    (32, 4, 2, 2, _capi.BCONV_LAZY, _capi.ROUND_FLOOR),
    (32, 3, 1, 3, _capi.BCONV_LAZY, _capi.ROUND_FLOOR),   # one-limb digits: raise without converters
    (32, 12, 12, 1, _capi.BCONV_EXACT, _capi.ROUND_HALF), # the reference examples' shape: one digit of 12 limbs, 12 extension
                                                          # limbs - conversions of 12 inputs (register path for 9 to 32 inputs)
])
def test_keyswitch_hrot_hmult(be, word_bits, L, K, dnum, bm, rm):
    pc.case_keyswitch(be, word_bits, L, K, dnum, bm, rm)


@pytest.mark.parametrize("word_bits,L,K,dnum,bm,rm", [
    (64, 4, 2, 2, _capi.BCONV_EXACT, _capi.ROUND_HALF),
    (32, 3, 1, 3, _capi.BCONV_LAZY, _capi.ROUND_FLOOR),
])
def test_keyswitch_with_fused_rescale(be, word_bits, L, K, dnum, bm, rm):
    pc.case_keyswitch_rescale(be, word_bits, L, K, dnum, bm, rm)


@pytest.mark.parametrize("word_bits,L,K,dnum,bm,rm,g,n_giant,r", [
    (64, 3, 2, 2, _capi.BCONV_EXACT, _capi.ROUND_HALF, 2, 2, 0),
    (32, 3, 1, 3, _capi.BCONV_LAZY, _capi.ROUND_FLOOR, 2, 3, 1),
])
def test_bsgs(be, word_bits, L, K, dnum, bm, rm, g, n_giant, r):
    pc.case_bsgs(be, word_bits, L, K, dnum, bm, rm, g=g, n_giant=n_giant, r=r, missing=((1, 1),))


@pytest.mark.parametrize("word_bits,bm,rm", [(64, _capi.BCONV_EXACT, _capi.ROUND_HALF), (32, _capi.BCONV_LAZY, _capi.ROUND_FLOOR)])
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
