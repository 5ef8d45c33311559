"""The bootstrap operator list (cerium_b200/bootstrap.py) on the GPU, every step through the C ABI,
against the same list evaluated on the CPU oracle (tests/bootstrap_checker.py): ModRaise, a
CoeffToSlot BSGS stage with the rescale folded in, conjugation, the Chebyshev polynomial with its 16
HMults per part and a double-angle step, a SlotToCoeff stage - at a reduced shape (11 levels, 2 x 2
BSGS stages) so that the checker finishes in seconds.  Bit-exact on every limb of the result.
Structure after benchmarks/bootstrap_32K/bootstrap.py:299-358."""
import zlib

import numpy as np
import pytest

from cerium_b200 import _capi, bootstrap as bs, params
from tests import parity_cases as pc

pytestmark = pytest.mark.gpu


def test_bootstrap_operator_list_matches_the_checker():
    import torch
    from tests.backends import CudaBackend
    from tests.bootstrap_checker import OracleEvaluator
    be = CudaBackend()
    shape = bs.BootstrapShape(top=11, stages=1, baby=2, giant=2, double_angle=1)
    assert shape.levels_used == 10
    K, dnum = 3, 4
    q = params.ntt_primes_below(60, 1, pc.LOGN) + params.ntt_primes_below(50, shape.top, pc.LOGN)
    p = params.ntt_primes_below(60, K + 1, pc.LOGN)[1:]
    moduli = q + p
    q_idx, p_idx = list(range(shape.top + 1)), list(range(shape.top + 1, shape.top + 1 + K))

    def make_np(tag, lead, idx):
        rng = np.random.default_rng(zlib.crc32(repr(tag).encode()))
        return pc.rand_limbs(rng, moduli, list(idx) * int(np.prod(lead, dtype=np.int64) or 1)).reshape(tuple(lead) + (len(idx), pc.N)) \
            if lead else pc.rand_limbs(rng, moduli, idx)

    def make_dev(tag, lead, idx):
        return be.to_dev(make_np(tag, lead, idx))

    bm, rm = _capi.BCONV_EXACT, _capi.ROUND_HALF
    elt = lambda step: be.lib.galois_elt_from_step(step, pc.LOGN)  # noqa: E731
    m_cpu = bs.BootstrapMaterial(moduli, q_idx, p_idx, dnum, shape, make_np, elt)
    m_gpu = bs.BootstrapMaterial(moduli, q_idx, p_idx, dnum, shape, make_dev, elt)
    rng = np.random.default_rng(1)
    ct2 = [pc.rand_limbs(rng, moduli, q_idx[:2]), pc.rand_limbs(rng, moduli, q_idx[:2])]
    want = bs.bootstrap(OracleEvaluator(m_cpu, bm, rm), shape, ct2)
    ctx = _capi.Context(be.lib, moduli, 64)
    ev = bs.GpuEvaluator(torch, _capi, ctx, m_gpu, bm, rm)
    got = bs.bootstrap(ev, shape, [be.to_dev(ct2[0]), be.to_dev(ct2[1])])
    torch.cuda.synchronize()
    assert got.level == want.level == shape.top - shape.levels_used
    assert np.array_equal(be.to_host(got.c0[:got.level].contiguous()), want.c0), "bootstrap c0 differs from the checker"
    assert np.array_equal(be.to_host(got.c1[:got.level].contiguous()), want.c1), "bootstrap c1 differs from the checker"
    n = ev.count.n
    assert n["bsgs"] == 2 and n["hmult"] == 2 * (7 + 2 + 7 + 1) and n["mod_raise"] == 1 and n["pt_mac"] == 2
