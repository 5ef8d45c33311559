"""Multi-rank path on CPU: world_size 2 and 3 `gloo` process groups drive the library's limb-sharded
key switch / HRot / rescale and its limb collectives.  Compute runs on the emulation build
(tests/emu); the collectives go through the library's communicator with a caller-provided
transport over gloo (tests/host_transport.py); every rank's output limbs must equal the oracle's
single-device result."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, word_bits, L, K, dnum, bconv_mode, round_mode, ext_split, ret):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        os.environ["OMP_NUM_THREADS"] = "2"
        dist.init_process_group("gloo", rank=rank, world_size=world)
        import oracle
        from cerium_b200 import _capi, sharded
        from tests import parity_cases as pc
        from tests.backends import EmuBackend
        from tests.host_transport import GlooHostTransport
        be = EmuBackend()
        tr = GlooHostTransport()
        comm = _capi.Comm(be.lib, rank, world, transport=tr)
        prm = pc.small_params(word_bits, L, K, dnum)
        ctx = _capi.Context(be.lib, prm.moduli, word_bits)
        rng = np.random.default_rng(21)             # same inputs on every rank
        c0, c1, evk = pc.make_keyswitch_inputs(rng, prm)
        octx = oracle.OracleContext(pc.LOGN, prm.moduli)
        elt = be.lib.galois_elt_from_step(7, pc.LOGN)
        want_ks = octx.keyswitch(bconv_mode, round_mode, prm.q_idx, prm.p_idx, dnum, c1, evk)
        want_rot = octx.hrot(bconv_mode, round_mode, prm.q_idx, prm.p_idx, dnum, elt, c0, c1, evk)
        tdt = torch.int64 if word_bits == 64 else torch.int32
        ndt = np.int64 if word_bits == 64 else np.int32

        def t(a):
            return torch.from_numpy(np.ascontiguousarray(a).astype(np.uint64 if word_bits == 64 else np.uint32).view(ndt).copy())

        sk = sharded.ShardedKeySwitch(ctx, prm, comm, bconv_mode, round_mode, ext_split=ext_split)
        mine = sharded.local_limb_indices(L, rank, world)
        assert sk.n_local == len(mine) and sk.g == -(-L // world)
        assert sk.k_local == len(sharded.local_ext_indices(L, K, rank, world, ext_split))
        lc0, lc1 = sharded.shard_poly(t(c0), rank, world), sharded.shard_poly(t(c1), rank, world)
        levk = sharded.shard_key(t(evk), L, rank, world, ext_split)
        o0 = torch.zeros((max(len(mine), 1), pc.N), dtype=tdt)
        o1 = torch.zeros_like(o0)
        sk.keyswitch(o0, o1, lc1, levk)
        u = np.uint64 if word_bits == 64 else np.uint32
        ok = True
        if mine:
            ok &= np.array_equal(o0.numpy().view(u)[:len(mine)].astype(np.uint64), want_ks[0][mine])
            ok &= np.array_equal(o1.numpy().view(u)[:len(mine)].astype(np.uint64), want_ks[1][mine])
        sk.hrot(o0, o1, lc0, lc1, levk, elt)
        if mine:
            ok &= np.array_equal(o0.numpy().view(u)[:len(mine)].astype(np.uint64), want_rot[0][mine])
            ok &= np.array_equal(o1.numpy().view(u)[:len(mine)].astype(np.uint64), want_rot[1][mine])
        # rescale of the sharded rotation result against the one-device oracle
        rot = torch.stack([o0[:len(mine)], o1[:len(mine)]]) if mine else torch.zeros((2, 0, pc.N), dtype=tdt)
        assert tr.calls["allgather"] == (4 if ext_split else 2)     # one (two) exchange(s) per key switch
        res = sharded.sharded_rescale(ctx, comm, prm.q_idx, rot, round_mode)
        assert tr.calls["broadcast"] == 1
        keep = [i for i in mine if i != L - 1]
        for p_ in range(2):
            want_rs = octx.rescale(round_mode, prm.q_idx, want_rot[p_])
            if keep:
                ok &= np.array_equal(res[p_].numpy().view(u).astype(np.uint64), want_rs[keep])
        # the limb collectives on their own: AGS (reduce-scatter + mod) and ARD (all-reduce + mod) of
        # partial sums against the sum of all ranks' residues, DRM against the stacked blocks
        idx = [1, 0]
        parts = [pc.rand_limbs(np.random.default_rng(50 + r), prm.moduli, idx * world) for r in range(world)]
        total = sum(p_.astype(object) for p_ in parts)
        want_sum = np.stack([np.array([int(v) % prm.moduli[idx[b % 2]] for v in total[b]], dtype=np.uint64)
                             for b in range(2 * world)])
        wd = np.uint64 if word_bits == 64 else np.uint32
        buf = np.ascontiguousarray(parts[rank].astype(wd))
        red = np.zeros((2, pc.N), dtype=wd)
        comm.reducescatter_limbs(ctx, red.ctypes.data, buf.ctypes.data, idx)
        ok &= np.array_equal(red.astype(np.uint64), want_sum[2 * rank:2 * rank + 2])
        comm.allreduce_limbs(ctx, buf.ctypes.data, buf.ctypes.data, idx * world)
        ok &= np.array_equal(buf.astype(np.uint64), want_sum)
        gat = np.zeros((world, 2, pc.N), dtype=wd)
        comm.allgather_limbs(ctx, gat.ctypes.data, red.ctypes.data, 2)
        ok &= np.array_equal(gat.reshape(2 * world, pc.N).astype(np.uint64), want_sum)
        flag = torch.tensor([1 if ok else 0])
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        ret[rank] = int(flag.item())
        dist.destroy_process_group()
    except Exception as e:  # surfaced by the parent
        ret[rank] = "rank %d: %r" % (rank, e)
        raise


@pytest.mark.parametrize("world,word_bits,L,K,dnum,bm,rm,ext_split", [
    (2, 64, 5, 2, 3, 0, 0, False),   # ragged: ranks own 3 and 2 limbs, digits of size 2,2,1
    (2, 64, 4, 1, 4, 1, 1, False),   # one digit per limb, exact conversion with rounding
    (3, 32, 4, 2, 2, 0, 0, False),   # a rank with a single limb
    (2, 64, 5, 3, 3, 1, 1, True),    # extension limbs split 1 / 2, exact conversion with rounding
    (3, 64, 4, 2, 2, 0, 0, True),    # a rank without extension limbs
    (3, 32, 6, 3, 3, 1, 0, True),    # world = dnum: every rank's limbs belong to one digit
    (8, 64, 11, 5, 4, 1, 1, True),   # eight ranks as the benchmark runs them: 2,2,2,1,1,1,1,1 limbs, extension limbs on ranks 3..7 only
])
def test_sharded_keyswitch_matches_single_device(world, word_bits, L, K, dnum, bm, rm, ext_split):
    sys.path.insert(0, os.path.join(ROOT, "tests", "emu"))
    import build_emu
    build_emu.build()
    ctx = mp.get_context("spawn")
    mgr = ctx.Manager()
    ret = mgr.dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, word_bits, L, K, dnum, bm, rm, ext_split, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(600)
    for p in procs:
        if p.is_alive():
            p.terminate()
    assert all(p.exitcode == 0 for p in procs), dict(ret)
    assert all(ret.get(r) == 1 for r in range(world)), dict(ret)


def test_comm_split_on_a_callers_transport():
    """Groups of consecutive ranks exist for the NCCL transport only: a caller's transport gets its own
    communicator back for the full size and a clear refusal for a smaller one."""
    import pytest
    from cerium_b200 import _capi
    sys.path.insert(0, os.path.join(ROOT, "tests", "emu"))
    import build_emu
    lib = _capi.Library(build_emu.build())

    class Nothing:
        pass
    comm = _capi.Comm(lib, 1, 4, transport=Nothing())
    assert comm.split(4) == comm.h.value
    with pytest.raises(_capi.CeriumError) as e:
        comm.split(2)
    assert e.value.code == _capi.ERR_UNSUPPORTED and "sub-groups" in e.value.message
    with pytest.raises(_capi.CeriumError):
        comm.split(3)                                   # does not divide the number of ranks
    comm.close()


def test_local_limb_indices():
    from cerium_b200 import sharded
    assert sharded.local_limb_indices(35, 0, 8) == [0, 8, 16, 24, 32]
    assert sharded.local_limb_indices(35, 7, 8) == [7, 15, 23, 31]
    assert sorted(sum((sharded.local_limb_indices(35, r, 4) for r in range(4)), [])) == list(range(35))
