"""On-disk containers of the reference runtime (cerium/runtime/io/generator.cpp:503-564, 737-860):
byte layout, round trips and the assembly of a key-switch key from its per-digit entries."""
import struct

import numpy as np
import pytest

from cerium_b200 import containers as ct


def _limbs(rng, ids, n):
    return [(i, rng.integers(0, 1 << 28, size=n, dtype=np.uint32)) for i in ids]


def test_evalkey_bytes_follow_the_reference_layout(tmp_path):
    n = 4
    c = ct.Container("evalkeys", n, [97, 193, 257])
    c0 = [(0, np.array([1, 2, 3, 4], dtype=np.uint32)), (2, np.array([5, 6, 7, 8], dtype=np.uint32))]
    c1 = [(0, np.array([9, 10, 11, 12], dtype=np.uint32)), (2, np.array([13, 14, 15, 16], dtype=np.uint32))]
    c.entries["1:2:1:5:[0]"] = ct.Entry("1:2:1:5:[0]", [c0, c1])
    path = tmp_path / "evk.bin"
    ct.write(str(path), c)
    raw = path.read_bytes()
    want = b"Cerium::Evalkeys\n\0" + struct.pack("<QQ", 4, 3) + struct.pack("<3Q", 97, 193, 257)
    want += struct.pack("<QQ", 1, 4 * 16)                       # one entry, 16 words of payload
    want += struct.pack("<Q", 12) + b"1:2:1:5:[0]\0" + struct.pack("<Q", 2)
    for limbs in (c0, c1):
        for lid, data in limbs:
            want += struct.pack("<Q", lid) + data.tobytes()
    assert raw == want


@pytest.mark.parametrize("kind,n_polys", [("evalkeys", 2), ("ciphertexts", 2), ("plaintexts", 1)])
def test_round_trip(tmp_path, kind, n_polys):
    rng = np.random.default_rng(5)
    n = 64
    c = ct.Container(kind, n, [268042241, 268271617, 268369921])
    for name, ids in (("a", [0, 1, 2]), ("b(3)", [2, 0])):
        c.entries[name] = ct.Entry(name, [_limbs(rng, ids, n) for _ in range(n_polys)])
    path = str(tmp_path / "c.bin")
    ct.write(path, c)
    back = ct.read(path)
    assert (back.kind, back.n, back.primes) == (kind, n, c.primes)
    assert list(back.entries) == ["a", "b(3)"]
    for name, e in c.entries.items():
        for p in range(n_polys):
            assert [l for l, _ in back.entries[name].polys[p]] == [l for l, _ in e.polys[p]]
            for (_, x), (_, y) in zip(back.entries[name].polys[p], e.polys[p]):
                assert np.array_equal(x, y)
    assert np.array_equal(back.entries["b(3)"].stack(0, [0, 2]),
                          np.stack([dict(c.entries["b(3)"].polys[0])[0], dict(c.entries["b(3)"].polys[0])[2]]))


def test_evalkey_tensor_orders_digits_and_limbs(tmp_path):
    """A rotation key of three digits over limbs {0..5} + extension {63, 62}, written digit by digit in
    scrambled order, comes back as [digit][c0, c1][Q limbs, extension limbs][n]."""
    rng = np.random.default_rng(6)
    n, order = 32, [0, 1, 2, 3, 4, 5, 63, 62]
    key = rng.integers(0, 1 << 28, size=(3, 2, len(order), n), dtype=np.uint32)
    digits = {0: [0, 3], 1: [1, 4], 2: [2, 5]}          # the reference's strided digit split
    c = ct.Container("evalkeys", n, list(range(64)))
    for d in (2, 0, 1):
        name = "1:6:2:7:[%s]" % ",".join(str(x) for x in digits[d])
        scr = list(rng.permutation(len(order)))
        c.entries[name] = ct.Entry(name, [[(order[k], key[d, p, k]) for k in scr] for p in range(2)])
    c.entries["0:6:2:0:[0,3]"] = ct.Entry("0:6:2:0:[0,3]", [_limbs(rng, order, n), _limbs(rng, order, n)])
    path = str(tmp_path / "k.bin")
    ct.write(path, c)
    back = ct.read(path)
    assert ct.parse_evalkey_id("1:6:2:7:[1,4]") == (1, 6, 2, 7, [1, 4])
    assert np.array_equal(ct.evalkey_tensor(back, 1, 6, 2, 7, order), key)
    with pytest.raises(KeyError):
        ct.evalkey_tensor(back, 2, 6, 2, 7, order)
    with pytest.raises(KeyError):
        ct.evalkey_tensor(back, 1, 6, 2, 7, order + [61])


def test_malformed_files_are_refused(tmp_path):
    rng = np.random.default_rng(7)
    c = ct.Container("ciphertexts", 16, [97])
    c.entries["x"] = ct.Entry("x", [_limbs(rng, [0], 16), _limbs(rng, [0], 16)])
    path = tmp_path / "c.bin"
    ct.write(str(path), c)
    raw = path.read_bytes()
    (tmp_path / "short.bin").write_bytes(raw[:-3])
    with pytest.raises(ValueError, match="truncated"):
        ct.read(str(tmp_path / "short.bin"))
    (tmp_path / "long.bin").write_bytes(raw + b"\0")
    with pytest.raises(ValueError, match="trailing"):
        ct.read(str(tmp_path / "long.bin"))
    (tmp_path / "bad.bin").write_bytes(b"Cerium::Nothing\n\0" + raw[20:])
    with pytest.raises(ValueError, match="header"):
        ct.read(str(tmp_path / "bad.bin"))
    with pytest.raises(ValueError, match="polynomials"):
        ct.write(str(tmp_path / "w.bin"), ct.Container("plaintexts", 16, [97], {"x": c.entries["x"]}))


def test_key_from_a_container_drives_a_rotation(tmp_path):
    """A rotation key written digit by digit in the reference's file layout, read back and stacked by
    evalkey_tensor, gives the oracle's HRot when handed to the library (CPU build of the library sources)."""
    from cerium_b200 import _capi
    from tests import parity_cases as pc
    from tests.backends import EmuBackend
    be = EmuBackend()
    L, K, dnum = 4, 2, 2
    prm = pc.small_params(32, L, K, dnum)
    order = prm.q_idx + prm.p_idx
    h = pc.Harness(be, 32, prm.moduli)
    rng = np.random.default_rng(44)
    c0, c1, evk = pc.make_keyswitch_inputs(rng, prm)
    ks = _capi.KeySwitch(h.ctx, prm.q_idx, prm.p_idx, dnum, _capi.BCONV_LAZY, _capi.ROUND_FLOOR)
    # digit d owns the Q limbs d, d + dnum, ... (the reference's strided split)
    c = ct.Container("evalkeys", pc.N, [int(m) for m in prm.moduli])
    for d in reversed(range(dnum)):
        name = "1:%d:%d:5:[%s]" % (L, K, ",".join(str(prm.q_idx[i]) for i in range(d, L, dnum)))
        c.entries[name] = ct.Entry(name, [[(order[k], evk[d, p, k].astype(np.uint32)) for k in range(len(order))]
                                          for p in range(2)])
    path = str(tmp_path / "evk.bin")
    ct.write(path, c)
    key = ct.evalkey_tensor(ct.read(path), 1, L, K, 5, order)
    assert key.shape == (dnum, 2, L + K, pc.N) and np.array_equal(key, evk.astype(np.uint32))
    elt = be.lib.galois_elt_from_step(5, pc.LOGN)
    d_c0, d_c1, d_evk = h.up(c0), h.up(c1), h.up(key.astype(np.uint64))
    o0, o1 = h.new(L, pc.N), h.new(L, pc.N)
    ks.hrot(h.p(o0), h.p(o1), h.p(d_c0), h.p(d_c1), h.p(d_evk), elt)
    w0, w1 = h.orc.hrot(_capi.BCONV_LAZY, _capi.ROUND_FLOOR, prm.q_idx, prm.p_idx, dnum, elt, c0, c1, evk)
    assert np.array_equal(h.down(o0), w0) and np.array_equal(h.down(o1), w1)
