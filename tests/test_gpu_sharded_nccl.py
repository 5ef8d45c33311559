"""Limb-sharded HRot over NCCL on 2 GPUs (skipped with fewer): every rank's limbs must equal the
single-GPU result of the same ciphertext, bit for bit."""
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
    from cerium_b200 import _capi, sharded
    from tests import parity_cases as pc
    lib = _capi.load()
    L, K, dnum = 9, 3, 3
    prm = pc.small_params(64, L, K, dnum)
    ctx = _capi.Context(lib, prm.moduli, 64, device=rank)
    rng = np.random.default_rng(5)
    c0, c1, evk = pc.make_keyswitch_inputs(rng, prm)
    dev = torch.device("cuda", rank)

    def t(a):
        return torch.from_numpy(a.view(np.int64).copy()).to(dev)
    elt = lib.galois_elt_from_step(11, pc.LOGN)
    # single-GPU result on this rank's device
    ks = _capi.KeySwitch(ctx, prm.q_idx, prm.p_idx, dnum)
    f0, f1 = torch.zeros((L, pc.N), dtype=torch.int64, device=dev), torch.zeros((L, pc.N), dtype=torch.int64, device=dev)
    tc0, tc1, tevk = t(c0), t(c1), t(evk)
    ks.hrot(f0.data_ptr(), f1.data_ptr(), tc0.data_ptr(), tc1.data_ptr(), tevk.data_ptr(), elt,
            torch.cuda.current_stream().cuda_stream)
    sk = sharded.ShardedKeySwitch(lib, ctx, prm, rank, world, device=dev)
    mine = sharded.local_limb_indices(L, rank, world)
    o0 = torch.zeros((len(mine), pc.N), dtype=torch.int64, device=dev)
    o1 = torch.zeros_like(o0)
    for _ in range(2):
        sk.hrot(o0, o1, sharded.shard_poly(tc0, rank, world), sharded.shard_poly(tc1, rank, world),
                sharded.shard_key(tevk, L, rank, world), elt)
    torch.cuda.synchronize()
    ok = bool(torch.equal(o0, f0[mine]) and torch.equal(o1, f1[mine]))
    # sharded rescale (broadcast of the last limb) against the one-GPU rescale
    full = torch.stack([f0, f1])
    one = torch.empty((2, L - 1, pc.N), dtype=torch.int64, device=dev)
    scratch = torch.empty((2, pc.N), dtype=torch.int64, device=dev)
    ctx.rescale(one.data_ptr(), full.data_ptr(), prm.q_idx, 2, scratch.data_ptr(), _capi.ROUND_FLOOR,
                torch.cuda.current_stream().cuda_stream)
    res = sharded.sharded_rescale(ctx, prm.q_idx, torch.stack([o0, o1]), rank, world)
    torch.cuda.synchronize()
    keep = [i for i in mine if i != L - 1]
    ok = ok and bool(torch.equal(res, one[:, keep]))
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    ret[rank] = int(flag.item())
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_sharded_hrot_nccl_two_gpus():
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    for p in procs:
        if p.is_alive():
            p.terminate()
    assert all(p.exitcode == 0 for p in procs) and all(ret.get(r) == 1 for r in range(2)), dict(ret)
