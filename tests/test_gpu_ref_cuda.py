"""On a GPU: the reference's own CUDA kernels (oracle/_ref/libref_cuda.so), the product's 32-bit
kernels and the CPU oracle agree modulo q on the same inputs."""
import numpy as np
import pytest

import oracle
from cerium_b200 import _capi
from tests import ref_cuda

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not ref_cuda.available(), reason="oracle/_ref/libref_cuda.so not built")]

N = 1 << 16


@pytest.fixture(scope="module")
def env():
    import importlib.util, os
    from tests.backends import CudaBackend
    here = os.path.dirname(os.path.abspath(__file__))
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(here, "golden", "make_ref_cuda_golden.py"))
    G = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(G)
    be = CudaBackend()
    return be, G, ref_cuda.RefCuda(G.PRIMES), _capi.Context(be.lib, G.PRIMES, 32), oracle.OracleContext(16, G.PRIMES)


def _canon(t, mods):
    return t.cpu().numpy().view(np.uint32) % np.array(mods, dtype=np.uint32)[:, None]


@pytest.mark.parametrize("name", ["ntt_fwd", "ntt_inv"])
def test_ntt_three_way(env, name):
    be, G, ref, ctx, octx = env
    torch = be.torch
    _, _, d = G.CASES[name]
    x = G.case_inputs(name)["x"]
    dx = torch.from_numpy(x.view(np.int32)).cuda()
    r = torch.zeros_like(dx)
    o = torch.zeros_like(dx)
    ref.ntt(r.data_ptr(), dx.data_ptr(), d["bases"], inverse=d["inverse"])
    (ctx.ntt_inverse if d["inverse"] else ctx.ntt_forward)(o.data_ptr(), dx.data_ptr(), d["bases"])
    torch.cuda.synchronize()
    mods = [G.PRIMES[b] for b in d["bases"]]
    want = (octx.ntt_inverse if d["inverse"] else octx.ntt_forward)(x.astype(np.uint64), d["bases"]).astype(np.uint32)
    assert np.array_equal(_canon(r, mods), want), "oracle differs from the reference CUDA kernel"
    assert np.array_equal(o.cpu().numpy().view(np.uint32), want), "product differs from the oracle"


@pytest.mark.parametrize("name", ["bconv_5_35", "bconv_5_30", "bconv_18_12"])
def test_bconv_three_way(env, name):
    be, G, ref, ctx, octx = env
    torch = be.torch
    _, _, d = G.CASES[name]
    x = G.case_inputs(name)["x"]
    dx = torch.from_numpy(x.view(np.int32)).cuda()
    r = torch.zeros((len(d["out_idx"]), N), dtype=torch.int32, device="cuda")
    o = torch.zeros_like(r)
    ref.bconv(r.data_ptr(), dx.data_ptr(), d["in_idx"], d["out_idx"])
    bc = _capi.BaseConverter(ctx, d["in_idx"], d["out_idx"], _capi.BCONV_LAZY)
    bc.apply(o.data_ptr(), dx.data_ptr())
    torch.cuda.synchronize()
    mods = [G.PRIMES[j] for j in d["out_idx"]]
    want = oracle.bconv(oracle.BCONV_LAZY, [G.PRIMES[i] for i in d["in_idx"]], x.astype(np.uint64), mods).astype(np.uint32)
    assert np.array_equal(_canon(r, mods), want), "oracle differs from the reference CUDA kernel"
    assert np.array_equal(o.cpu().numpy().view(np.uint32), want), "product differs from the oracle"


def test_sud_three_way(env):
    be, G, ref, ctx, octx = env
    torch = be.torch
    _, _, d = G.CASES["sud"]
    inp = G.case_inputs("sud")
    in1 = torch.from_numpy(inp["in1"].view(np.int32)).cuda()
    in2 = torch.from_numpy(inp["in2"].view(np.int32)).cuda()
    r = torch.zeros_like(in1)
    o = torch.zeros_like(in1)
    f = G.sud_factors(d["divide"])
    ref.sud(r.data_ptr(), in1.data_ptr(), in2.data_ptr(), d["bases"], f)
    work = in2.clone()
    ctx.sud(o.data_ptr(), in1.data_ptr(), work.data_ptr(), d["bases"], d["divide"])
    torch.cuda.synchronize()
    mods = [G.PRIMES[b] for b in d["bases"]]
    want = np.stack([octx.sud(b, inp["in1"][i].astype(np.uint64), inp["in2"][i].astype(np.uint64), f[b])
                     for i, b in enumerate(d["bases"])]).astype(np.uint32)
    assert np.array_equal(_canon(r, mods), want), "oracle differs from the reference CUDA kernel"
    assert np.array_equal(o.cpu().numpy().view(np.uint32), want), "product differs from the oracle"


def test_timing_against_reference_kernels(env, capsys):
    """Times the reference's kernels and the product's 32-bit kernels on identical inputs (384 limb
    transforms, the seven 5 -> 35 conversions of one key switch) and prints one JSON object; run
    with `-s` to see it.  Only the agreement of the outputs is asserted."""
    import json
    be, G, ref, ctx, octx = env
    torch = be.torch

    def timed(fn, iters=20):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / iters

    P = G.PRIMES
    idx = [l for _ in range(8) for l in range(48)]
    gen = torch.Generator(device="cuda").manual_seed(1)
    q = torch.tensor([P[i] for i in idx], dtype=torch.int64, device="cuda").view(-1, 1)
    x = (torch.randint(0, 1 << 40, (len(idx), N), dtype=torch.int64, device="cuda", generator=gen) % q).to(torch.int32)
    y, z = torch.empty_like(x), torch.empty_like(x)
    res = {}
    res["ours_ntt_fwd_384_ms"] = timed(lambda: ctx.ntt_forward(y.data_ptr(), x.data_ptr(), idx))
    res["ours_ntt_inv_384_ms"] = timed(lambda: ctx.ntt_inverse(y.data_ptr(), x.data_ptr(), idx))
    ref.ntt(z.data_ptr(), x.data_ptr(), idx, False, 3)
    res["ref_ntt_fwd_384_ms"] = ref.ntt(z.data_ptr(), x.data_ptr(), idx, False, 20) / 20
    ref.ntt(z.data_ptr(), x.data_ptr(), idx, True, 3)
    res["ref_ntt_inv_384_ms"] = ref.ntt(z.data_ptr(), x.data_ptr(), idx, True, 20) / 20
    in_idx = [0, 7, 14, 21, 28]
    out_idx = [i for i in range(35) if i % 7] + [63, 62, 61, 60, 59]
    xin = x[:35].contiguous()
    o_ref = torch.empty((7 * 35, N), dtype=torch.int32, device="cuda")
    o_ours = torch.empty_like(o_ref)
    ref.bconv(o_ref.data_ptr(), xin.data_ptr(), in_idx, out_idx, 7, 3)
    res["ref_bconv_5_35_x7_ms"] = ref.bconv(o_ref.data_ptr(), xin.data_ptr(), in_idx, out_idx, 7, 20) / 20
    bc = _capi.BaseConverter(ctx, in_idx, out_idx, _capi.BCONV_LAZY)
    outs = [o_ours.data_ptr() + d * 35 * N * 4 for d in range(7)]
    ins = [xin.data_ptr() + d * 5 * N * 4 for d in range(7)]
    res["ours_bconv_5_35_x7_one_launch_ms"] = timed(lambda: _capi.BaseConverter.apply_batch([bc] * 7, outs, ins))
    torch.cuda.synchronize()
    mods = np.array([P[j] for j in out_idx] * 7, dtype=np.uint32)[:, None]
    assert np.array_equal(o_ref.cpu().numpy().view(np.uint32) % mods, o_ours.cpu().numpy().view(np.uint32))
    # SuD tail over 70 limbs (two polynomials of 35), the reference launcher's tables on both sides
    sidx = [l for _ in range(2) for l in range(35)]
    fac = [(i * 2654435761 + 12345) % P[i] for i in range(len(P))]           # one residue per prime
    m1, c2 = x[:70].contiguous(), x[70:140].contiguous()
    for r_, l in enumerate(sidx):                                            # residues of the right primes
        m1[r_] = (x[r_ + 140].to(torch.int64) % P[l]).to(torch.int32)
        c2[r_] = (x[r_ + 210].to(torch.int64) % P[l]).to(torch.int32)
    s_ref, s_ours = torch.empty_like(m1), torch.empty_like(m1)
    ref.sud(s_ref.data_ptr(), m1.data_ptr(), c2.data_ptr(), sidx, fac, 3)
    res["ref_sud_70_ms"] = ref.sud(s_ref.data_ptr(), m1.data_ptr(), c2.data_ptr(), sidx, fac, 20) / 20
    lb = N * 4
    pair = np.empty(140, dtype=np.uint64)
    pair[0::2] = [m1.data_ptr() + i * lb for i in range(70)]
    pair[1::2] = [c2.data_ptr() + i * lb for i in range(70)]
    d_pair = be.to_dev(pair)
    d_outs = be.to_dev(np.array([s_ours.data_ptr() + i * lb for i in range(70)], dtype=np.uint64))
    d_bases = be.to_dev(np.array(sidx, dtype=np.uint32))
    d_fac = be.to_dev(np.array(fac, dtype=np.uint32))
    res["ours_sud_70_ms"] = timed(lambda: ctx.sud_ptrs(be.ptr(d_outs), be.ptr(d_pair), be.ptr(d_bases), 70, be.ptr(d_fac)))
    torch.cuda.synchronize()
    smods = np.array([P[l] for l in sidx], dtype=np.uint32)[:, None]
    assert np.array_equal(s_ref.cpu().numpy().view(np.uint32) % smods, s_ours.cpu().numpy().view(np.uint32))
    with capsys.disabled():
        print("\nREF_CUDA_TIMING " + json.dumps(res))
