"""The C-ABI library loads on a machine without a GPU and exports every symbol that
include/cerium_b200.h declares; the ctypes table covers the same set.  No compute call is made."""
import ctypes
import os
import re

import pytest

from cerium_b200 import _capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "cerium_b200.h")).read()
    return sorted(set(re.findall(r"CERIUM_API[^;(]*?\b(cerium_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    syms = declared_symbols()
    for must in ("cerium_context_create", "cerium_ntt_forward", "cerium_ntt_inverse", "cerium_ntt_forward_ptrs",
                 "cerium_sud", "cerium_bconv_apply", "cerium_ewise", "cerium_tensor", "cerium_automorph",
                 "cerium_keyswitch_apply", "cerium_keyswitch_sharded_begin", "cerium_keyswitch_sharded_finish",
                 "cerium_hrot", "cerium_hmult", "cerium_rescale"):
        assert must in syms


def test_library_exports_every_declared_symbol():
    if not os.path.exists(_capi.LIB_PATH):
        from cerium_b200 import build
        build.build()
    dll = ctypes.CDLL(_capi.LIB_PATH)
    for name in declared_symbols():
        assert hasattr(dll, name), "libcerium_b200.so does not export %s" % name
    assert sorted(_capi.SIGNATURES) == declared_symbols()


def test_no_cpu_path_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    lib = _capi.load()
    from cerium_b200 import params
    with pytest.raises(_capi.CeriumError) as e:
        _capi.Context(lib, params.ntt_primes_below(50, 2, 16), 64)
    assert e.value.code == _capi.ERR_CUDA and "no CPU path" in e.value.message
    assert lib.dll.cerium_version() >= 100
