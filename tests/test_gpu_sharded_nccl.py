"""Limb-sharded HRot, rescale and the limb collectives over NCCL, one process per GPU (2, 4 and 8
ranks; each case is skipped when the machine has fewer GPUs): every rank's limbs must equal the
single-GPU result of the same ciphertext, bit for bit, with replicated and with split extension
limbs, at a small shape and at the benchmark's shape (L=35, K=5, dnum=7)."""
import os
import socket
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _worker(rank, world, port, ret):
    import numpy as np
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    sys.path.insert(0, ROOT)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from cerium_b200 import _capi, params, sharded
    from tests import parity_cases as pc
    lib = _capi.load()
    dev = torch.device("cuda", rank)
    comm = sharded.nccl_comm(lib, rank, world, rank)
    stream = torch.cuda.current_stream().cuda_stream
    ok = True

    def t(a):
        return torch.from_numpy(a.view(np.int64).copy()).to(dev)

    for prm, bm, rm in ((pc.small_params(64, 9, 3, 3), _capi.BCONV_LAZY, _capi.ROUND_FLOOR),
                        (params.config_hrot(pc.LOGN, 35, 5, 7), _capi.BCONV_EXACT, _capi.ROUND_HALF)):
        L = prm.L
        ctx = _capi.Context(lib, prm.moduli, 64, device=rank)
        rng = np.random.default_rng(5)                      # the same ciphertext and key on every rank
        c0, c1, evk = pc.make_keyswitch_inputs(rng, prm)
        elt = lib.galois_elt_from_step(11, pc.LOGN)
        # single-GPU result on this rank's device
        ks = _capi.KeySwitch(ctx, prm.q_idx, prm.p_idx, prm.dnum, bm, rm)
        f0 = torch.zeros((L, pc.N), dtype=torch.int64, device=dev)
        f1 = torch.zeros_like(f0)
        tc0, tc1, tevk = t(c0), t(c1), t(evk)
        ks.hrot(f0.data_ptr(), f1.data_ptr(), tc0.data_ptr(), tc1.data_ptr(), tevk.data_ptr(), elt, stream)
        ks.close()
        mine = sharded.local_limb_indices(L, rank, world)
        lc0, lc1 = sharded.shard_poly(tc0, rank, world), sharded.shard_poly(tc1, rank, world)
        o0 = torch.zeros((len(mine), pc.N), dtype=torch.int64, device=dev)
        o1 = torch.zeros_like(o0)
        for ext_split in (False, True):
            sk = sharded.ShardedKeySwitch(ctx, prm, comm, bm, rm, ext_split=ext_split)
            levk = sharded.shard_key(tevk, L, rank, world, ext_split)
            for _ in range(2):
                o0.zero_()
                o1.zero_()
                sk.hrot(o0, o1, lc0, lc1, levk, elt, stream)
            torch.cuda.synchronize()
            ok = ok and bool(torch.equal(o0, f0[mine]) and torch.equal(o1, f1[mine]))
            # in place on the inputs: the rotation goes through the workspace
            i0, i1 = lc0.clone(), lc1.clone()
            sk.hrot(i0, i1, i0, i1, levk, elt, stream)
            torch.cuda.synchronize()
            ok = ok and bool(torch.equal(i0, f0[mine]) and torch.equal(i1, f1[mine]))
            sk.ks.close()
        # sharded rescale (broadcast of the last limb) against the one-GPU rescale
        full = torch.stack([f0, f1])
        one = torch.empty((2, L - 1, pc.N), dtype=torch.int64, device=dev)
        scratch = torch.empty((2, pc.N), dtype=torch.int64, device=dev)
        ctx.rescale(one.data_ptr(), full.data_ptr(), prm.q_idx, 2, scratch.data_ptr(), rm, stream)
        res = sharded.sharded_rescale(ctx, comm, prm.q_idx, torch.stack([o0, o1]), rm, stream)
        torch.cuda.synchronize()
        keep = [i for i in mine if i != L - 1]
        ok = ok and bool(torch.equal(res, one[:, keep]))
        # AGS / ARD: sums of every rank's residues, reduced; DRM: the stacked blocks
        idx = [1, 0]
        q = torch.tensor([prm.moduli[i] for i in idx * world], dtype=torch.int64, device=dev).view(-1, 1)
        parts = [t(pc.rand_limbs(np.random.default_rng(50 + r), prm.moduli, idx * world)) for r in range(world)]
        want = sum(parts) % q                               # world * q < 2^63: the plain sum is exact
        buf = parts[rank].clone()
        red = torch.zeros((2, pc.N), dtype=torch.int64, device=dev)
        comm.reducescatter_limbs(ctx, red.data_ptr(), buf.data_ptr(), idx, stream)
        comm.allreduce_limbs(ctx, buf.data_ptr(), buf.data_ptr(), idx * world, stream)
        gat = torch.zeros((world, 2, pc.N), dtype=torch.int64, device=dev)
        comm.allgather_limbs(ctx, gat.data_ptr(), red.data_ptr(), 2, stream)
        torch.cuda.synchronize()
        ok = ok and bool(torch.equal(red, want[2 * rank:2 * rank + 2]) and torch.equal(buf, want)
                         and torch.equal(gat.view(2 * world, pc.N), want))
        del ctx
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    ret[rank] = int(flag.item())
    comm.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharded_hrot_nccl(world):
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(600)
    for p in procs:
        if p.is_alive():
            p.terminate()
    assert all(p.exitcode == 0 for p in procs) and all(ret.get(r) == 1 for r in range(world)), dict(ret)
