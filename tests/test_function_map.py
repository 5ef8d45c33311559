"""The reference runtime's plugin contract: a copy of function_map_shim.so installed as function_map_<p>.so
answers __GET_FUNCTION_MAP__ / __GET_FUNCTION_MAP_CUGRAPH__ with libcerium_b200.so's launchers of the
reference's signatures (cerium/runtime/execution/device_utils.cu:33-113) for the ntt / int / sud / bco
records of the partition's functions<p> file (cerium/compiler/backend/cuda_kernel.cc:1707-1916).

CPU tests: the maps, through a driver that loads the plugin as the reference does.  GPU tests: the
launchers themselves, stream and graph variants, against the oracle."""
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest

from cerium_b200 import _capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# records in the producer's layout (only .id and .type matter to the plugin)
FUNCTIONS = """function3 {
  .id: 3
  .type: int
  .outputs: r1
  .inputs: r0
  .bases: 0 1 2
}
function4 {
  .id: 4
  .type: bco
  .outputs: b0(3)
  .inputs: b0(0) b0(1) b0(2)
  .base_conv: <b0: 0 1 2 : 3 4>
}
function5 {
  .id: 5
  .type: ntt
  .outputs: r2
  .inputs: r1
}
function9 {
  .id: 9
  .type: generic
  .outputs: r3
  .inputs: r2 r1
}
function11 {
  .id: 11
  .type: sud
  .outputs: r4
  .inputs: r3 r2
  .sud: 3 4
}
"""

FAKE_PLUGIN = r"""
#include <cstdint>
#include <unordered_map>
typedef std::unordered_map<uint32_t, void*> M;
static void generated_9() {}
static void generated_5() {}
static M stream_map, graph_map;
const M& a() asm("__GET_FUNCTION_MAP__");
const M& b() asm("__GET_FUNCTION_MAP_CUGRAPH__");
const M& a() { stream_map[9] = (void*)&generated_9; stream_map[5] = (void*)&generated_5; return stream_map; }
const M& b() { graph_map[9] = (void*)&generated_9; return graph_map; }
"""


def _ensure_lib():
    from cerium_b200 import build
    if not os.path.exists(_capi.LIB_PATH) or not os.path.exists(build.SHIM_LIB):
        build.build()


# a second partition whose record 3 is a base conversion, not an inverse transform
FUNCTIONS_P1 = """function3 {
  .id: 3
  .type: bco
  .outputs: b0(3)
  .inputs: b0(0)
}
function7 {
  .id: 7
  .type: sud
  .outputs: r4
  .inputs: r3 r2
}
"""


def _run_driver(tmp_path, with_generated=False, two_partitions=False, preload=False, drop_functions=False):
    _ensure_lib()
    from cerium_b200 import plugin
    drv = str(tmp_path / "driver")
    subprocess.run(["g++", "-O1", "-std=c++17", os.path.join(ROOT, "tests", "function_map_driver.cpp"), "-o", drv, "-ldl"],
                   check=True)
    d = tmp_path / "prog" / "main"
    d.mkdir(parents=True)
    (d / "functions0").write_text(FUNCTIONS)
    if two_partitions:
        (d / "functions1").write_text(FUNCTIONS_P1)
    if with_generated:
        (tmp_path / "gen.cpp").write_text(FAKE_PLUGIN)
        subprocess.run(["g++", "-shared", "-fPIC", "-std=c++17", str(tmp_path / "gen.cpp"), "-o",
                        str(d / "function_map_0.so")], check=True)
    written = plugin.install(str(d))
    assert [os.path.basename(w) for w in written] == ["function_map_%d.so" % p for p in range(2 if two_partitions else 1)]
    assert os.path.exists(d / "function_map_0.orig.so") == with_generated
    assert plugin.install(str(d)) == written                   # installing twice changes nothing
    assert os.path.exists(d / "function_map_0.orig.so") == with_generated
    if drop_functions:
        os.remove(d / "functions0")
    cmd = [drv] + (["--preload", _capi.LIB_PATH] if preload else []) + written
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    maps = [{"stream": {}, "graph": {}} for _ in written]
    launchers, errors = {}, []
    for line in r.stdout.split("\n"):
        f = line.split()
        if len(f) == 4 and f[0].isdigit():
            maps[int(f[0])][f[1]][int(f[2])] = f[3]
        elif len(f) == 4 and f[0] == "launcher":
            launchers[(f[1], f[2])] = f[3]
        elif f and f[0] == "error":
            errors.append(line)
    return maps, launchers, errors


def test_plugin_maps_transform_records(tmp_path):
    maps, launchers, errors = _run_driver(tmp_path)
    assert not errors
    for kind in ("stream", "graph"):
        m = maps[0][kind]
        assert sorted(m) == [3, 4, 5, 11]          # the generic record has no launcher here
        assert m[3] == launchers[(kind, "int")]
        assert m[4] == launchers[(kind, "bco")]
        assert m[5] == launchers[(kind, "ntt")]
        assert m[11] == launchers[(kind, "sud")]
    assert len(set(launchers.values())) == 8 and "(nil)" not in launchers.values()


def test_plugin_keeps_generated_launchers_of_other_records(tmp_path):
    maps, launchers, errors = _run_driver(tmp_path, with_generated=True)
    assert not errors
    m = maps[0]
    assert sorted(m["stream"]) == [3, 4, 5, 9, 11] and sorted(m["graph"]) == [3, 4, 5, 9, 11]
    assert m["stream"][9] not in launchers.values()       # record 9 (generic) is the generated plugin's
    assert m["stream"][5] == launchers[("stream", "ntt")]  # record 5 (ntt) is overridden


@pytest.mark.parametrize("preload", [False, True])
def test_partitions_loaded_into_one_process_keep_their_own_maps(tmp_path, preload):
    """The runtime loads function_map_0.so, function_map_1.so, ... into one process
    (cerium/runtime/execution/function.cpp:171-177): id 3 is an inverse transform in partition 0 and a
    base conversion in partition 1, and each plugin must answer with its own record's launcher - also
    when the host program already holds the library under its real name."""
    maps, launchers, errors = _run_driver(tmp_path, two_partitions=True, preload=preload)
    assert not errors
    for kind in ("stream", "graph"):
        assert sorted(maps[0][kind]) == [3, 4, 5, 11]
        assert sorted(maps[1][kind]) == [3, 7]
        assert maps[0][kind][3] == launchers[(kind, "int")]
        assert maps[1][kind][3] == launchers[(kind, "bco")]
        assert maps[1][kind][7] == launchers[(kind, "sud")]


def test_plugin_reports_a_missing_functions_file(tmp_path):
    maps, launchers, errors = _run_driver(tmp_path, drop_functions=True)
    assert len(errors) == 2 and all("cannot open" in e and "functions0" in e for e in errors)
    lib = _capi.load()
    assert lib.dll.cerium_function_map_get(str(tmp_path / "nope").encode(), None, 0) is None
    assert b"cannot open" in lib.dll.cerium_function_map_error()
    assert lib.dll.cerium_function_map_size(str(tmp_path / "nope").encode(), 0) == -1


# ---------------------------------------------------------------------------------------------
# GPU: call the launchers the way execute_ntt / execute_int / execute_sud / execute_bco do
# ---------------------------------------------------------------------------------------------

_VP, _SZ = C.c_void_p, C.c_size_t
NTT_T = C.CFUNCTYPE(None, C.POINTER(_VP), _VP, _VP, _VP, _SZ, _VP, _VP)
SUD_T = C.CFUNCTYPE(None, C.POINTER(_VP), _VP, _VP, _VP, _SZ, _VP, _VP, _VP, _VP, _VP)
BCO_T = C.CFUNCTYPE(None, C.POINTER(_VP), _VP, _VP, _VP, _VP, _VP, _VP, _VP, _VP, _SZ, _SZ)
NTT_G = C.CFUNCTYPE(None, C.POINTER(_VP), C.POINTER(_VP), C.POINTER(_VP), _VP, _VP, _VP, _SZ, _VP, _VP)
SUD_G = C.CFUNCTYPE(None, C.POINTER(_VP), C.POINTER(_VP), C.POINTER(_VP), _VP, _VP, _VP, _SZ, _VP, _VP, _VP, _VP, _VP)
BCO_G = C.CFUNCTYPE(None, C.POINTER(_VP), C.POINTER(_VP), _VP, _VP, _VP, _VP, _VP, _VP, _VP, _VP, _SZ, _SZ)


class _Graph:
    """A CUDA graph the launchers add their nodes to, built and run through cuda-python."""

    def __init__(self):
        from cuda.bindings import runtime as rt
        self.rt = rt
        err, self.g = rt.cudaGraphCreate(0)
        assert err == rt.cudaError_t.cudaSuccess
        self.handle = _VP(int(self.g))

    def run(self):
        rt = self.rt
        err, ex = rt.cudaGraphInstantiate(self.g, 0)
        assert err == rt.cudaError_t.cudaSuccess, err
        (err,) = rt.cudaGraphLaunch(ex, 0)
        assert err == rt.cudaError_t.cudaSuccess, err
        (err,) = rt.cudaStreamSynchronize(0)
        assert err == rt.cudaError_t.cudaSuccess, err
        rt.cudaGraphExecDestroy(ex)
        rt.cudaGraphDestroy(self.g)


@pytest.mark.gpu
@pytest.mark.parametrize("graph", [False, True])
def test_launchers_match_the_oracle(tmp_path, graph):
    import torch
    from tests import parity_cases as pc
    from tests.backends import CudaBackend
    import oracle
    be = CudaBackend()
    mods = pc.moduli_for(32, 8)
    h = pc.Harness(be, 32, mods)
    lib = h.ctx.lib
    fpath = tmp_path / "functions0"
    fpath.write_text(FUNCTIONS)
    fp = str(fpath).encode()
    assert lib.dll.cerium_function_map_size(fp, 0) == 4
    assert lib.dll.cerium_function_map_bind(h.ctx.h, torch.cuda.current_device()) == 0
    try:
        look = lambda kid: lib.dll.cerium_function_map_lookup(fp, 1 if graph else 0, kid)
        rng = np.random.default_rng(91)
        N = pc.N
        lb = N * 4
        t64 = lambda v: be.to_dev(np.array(v, dtype=np.uint64))
        stream = _VP(0)
        # --- ntt (record 5) then int (record 3) on ragged pointer tables
        idx = [2, 0, 5]
        x = pc.rand_limbs(rng, mods, idx)
        dx, dy, dz = h.up(x), h.new(3, N), h.new(3, N)
        ins, mid, outs = (t64([h.p(t) + i * lb for i in range(3)]) for t in (dx, dy, dz))
        bases = be.to_dev(np.array(idx, dtype=np.uint32))
        if graph:
            g, n0, n1 = _Graph(), _VP(), _VP()
            NTT_G(look(5))(C.byref(g.handle), C.byref(n0), C.byref(n1), be.ptr(mid), be.ptr(ins), be.ptr(bases), 3, None, None)
            assert n0.value and n1.value and n0.value != n1.value
            g.run()
        else:
            NTT_T(look(5))(C.byref(stream), be.ptr(mid), be.ptr(ins), be.ptr(bases), 3, None, None)
        assert np.array_equal(h.down(dy), h.orc.ntt_forward(x, idx))
        if graph:
            g, n0, n1 = _Graph(), _VP(), _VP()
            NTT_G(look(3))(C.byref(g.handle), C.byref(n0), C.byref(n1), be.ptr(outs), be.ptr(mid), be.ptr(bases), 3, None, None)
            g.run()
        else:
            NTT_T(look(3))(C.byref(stream), be.ptr(outs), be.ptr(mid), be.ptr(bases), 3, None, None)
        assert np.array_equal(h.down(dz), x)
        # --- sud (record 11): two inputs per entry, factors per prime of the context
        minuend, coeff = pc.rand_limbs(rng, mods, idx), pc.rand_limbs(rng, mods, idx)
        fac = [int(rng.integers(1, m)) for m in mods]
        want = np.stack([h.orc.sud(p, minuend[i], coeff[i], fac[p]) for i, p in enumerate(idx)])
        dm, dc, do = h.up(minuend), h.up(coeff), h.new(3, N)
        pair = np.empty(6, dtype=np.uint64)
        pair[0::2] = [h.p(dm) + i * lb for i in range(3)]
        pair[1::2] = [h.p(dc) + i * lb for i in range(3)]
        d_pair, d_outs = be.to_dev(pair), t64([h.p(do) + i * lb for i in range(3)])
        d_fac = be.to_dev(np.array(fac, dtype=np.uint32))
        if graph:
            g, n0, n1 = _Graph(), _VP(), _VP()
            SUD_G(look(11))(C.byref(g.handle), C.byref(n0), C.byref(n1), be.ptr(d_outs), be.ptr(d_pair), be.ptr(bases), 3,
                            None, None, be.ptr(d_fac), None, None)
            g.run()
        else:
            SUD_T(look(11))(C.byref(stream), be.ptr(d_outs), be.ptr(d_pair), be.ptr(bases), 3, None, None, be.ptr(d_fac),
                            None, None)
        assert np.array_equal(h.down(do), want)
        # --- bco (record 4): two conversions 3 -> 5, everything from device tables
        in_idx, out_idx = [0, 1, 2], [3, 4, 5, 6, 7]
        qs, ps = [mods[i] for i in in_idx], [mods[j] for j in out_idx]
        Q = qs[0] * qs[1] * qs[2]
        F = [[pow(Q // q % q, -1, q) % pj * (Q // q % pj) % pj for q in qs] for pj in ps]
        d_F = be.to_dev(np.array(F, dtype=np.uint32).reshape(-1))
        d_ps = be.to_dev(np.array(ps, dtype=np.uint32))
        xs = [pc.rand_limbs(rng, mods, in_idx) for _ in range(2)]
        d_xs, d_os = [h.up(v) for v in xs], [h.new(5, N) for _ in range(2)]
        smem = ((3 * 5 // 32 + 1) * 32 + 256 * 3) * 4               # Evaluator::fn_bco's size
        tabs = [t64([h.p(o) for o in d_os]), t64([5, 5]), t64([h.p(v) for v in d_xs]), t64([3, 3]),
                t64([be.ptr(d_F)] * 2), t64([be.ptr(d_ps)] * 2)]   # held until the results are read back
        args = tuple(be.ptr(t) for t in tabs) + (None, None, smem, 2)
        if graph:
            g, n0 = _Graph(), _VP()
            BCO_G(look(4))(C.byref(g.handle), C.byref(n0), *args)
            assert n0.value
            g.run()
        else:
            BCO_T(look(4))(C.byref(stream), *args)
        for v, o in zip(xs, d_os):
            assert np.array_equal(h.down(o), oracle.bconv(oracle.BCONV_LAZY, qs, v, ps))
    finally:
        lib.dll.cerium_function_map_bind(None, torch.cuda.current_device())
