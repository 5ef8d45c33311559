"""cerium_rescale_static: the rescale entry point for callers that cannot allocate device memory
(arena-only runtimes, plug-ins without an allocation budget, latency-critical sections).  Its
scratch is a fixed array inside the library, so the test drives it through the C ABI twice in a
row - the second call finds the first call's leftovers in the array - and expects both results
to equal cerium_rescale with a caller-provided scratch and the CPU oracle's rescale, bit for bit
(integer work)."""
import numpy as np
import pytest

from cerium_b200 import _capi
from tests import parity_cases as pc

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("word_bits,round_mode", [(64, _capi.ROUND_FLOOR), (64, _capi.ROUND_HALF), (32, _capi.ROUND_FLOOR)])
def test_rescale_static_matches_rescale_twice(word_bits, round_mode):
    from tests.backends import CudaBackend
    be = CudaBackend()
    L, n_polys = 5, 2
    mods = pc.moduli_for(word_bits, L, 1)
    if word_bits == 64:
        mods = mods[1:] + mods[:1]
    h = pc.Harness(be, word_bits, mods)
    q_idx = list(range(L))
    rng = np.random.default_rng(77)
    for call in range(2):
        x = np.stack([pc.rand_limbs(rng, mods, q_idx) for _ in range(n_polys)])
        dx = h.up(x)
        want = h.new(n_polys, L - 1, pc.N)
        scratch = h.new(n_polys, pc.N)
        h.ctx.rescale(h.p(want), h.p(dx), q_idx, n_polys, h.p(scratch), round_mode)
        got = h.new(n_polys, L - 1, pc.N)
        h.ctx.rescale_static(h.p(got), h.p(dx), q_idx, n_polys, round_mode)
        assert np.array_equal(h.down(got), h.down(want)), "call %d differs from cerium_rescale" % call
        orc = np.stack([h.orc.rescale(round_mode, q_idx, x[p]) for p in range(n_polys)])
        assert np.array_equal(h.down(got), orc), "call %d differs from the oracle" % call
        # a single polynomial uses only the first slot of the built-in scratch
        got1 = h.new(1, L - 1, pc.N)
        h.ctx.rescale_static(h.p(got1), h.p(dx), q_idx, 1, round_mode)
        assert np.array_equal(h.down(got1)[0], h.down(want)[0])
    # more polynomials than the built-in scratch holds: refused, nothing launched
    big = h.new(3, L, pc.N)
    out3 = h.new(3, L - 1, pc.N)
    with pytest.raises(_capi.CeriumError) as e:
        h.ctx.rescale_static(h.p(out3), h.p(big), q_idx, 3, round_mode)
    assert e.value.code == _capi.ERR_UNSUPPORTED and "2 polynomials" in e.value.message
