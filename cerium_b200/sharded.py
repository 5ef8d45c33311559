"""Limb-sharded key switching over several GPUs (one process per GPU, ``torch.distributed``).

Restates the reference's input-broadcast key switching
(``cerium/compiler/backend/compiler_keyswitch.cc:253-432`` with ``current_partition_size > 1``):
Q-limb ``i`` lives on rank ``i % world``, extension limbs and their share of the work are
replicated, evaluation keys are sharded with the limbs, and the only exchange is one all-gather
of the coefficient-form limbs before base conversion (the DRM group,
``cerium/runtime/execution/evaluator.cpp:1154-1251``).  The gather lands in this GPU's own memory;
the conversion kernels then read local memory only.

Tensors may live on any device the loaded library computes on (CUDA tensors with the CUDA
build); the collective uses whatever backend the process group was created with.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from . import _capi
from .params import CkksParams


def local_limb_indices(L: int, rank: int, world: int) -> List[int]:
    """Global indices of the Q-limbs rank ``rank`` owns (round robin)."""
    return list(range(rank, L, world))


def shard_poly(poly: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """[L, N] -> this rank's limbs [n_local, N]."""
    return poly[local_limb_indices(poly.shape[0], rank, world)].contiguous()


def shard_key(evk: torch.Tensor, L: int, rank: int, world: int) -> torch.Tensor:
    """[dnum, 2, L+K, N] -> [dnum, 2, n_local+K, N]: the rank's Q-limbs and every extension limb."""
    idx = local_limb_indices(L, rank, world) + list(range(L, evk.shape[2]))
    return evk[:, :, idx].contiguous()


class ShardedKeySwitch:
    """Key switch / HRot on the limbs of one rank; every rank calls the same method in step."""

    def __init__(self, lib: _capi.Library, ctx: _capi.Context, prm: CkksParams, rank: int, world: int,
                 bconv_mode: int = _capi.BCONV_LAZY, round_mode: int = _capi.ROUND_FLOOR,
                 group: Optional[dist.ProcessGroup] = None, device: Optional[torch.device] = None):
        self.lib, self.ctx, self.prm = lib, ctx, prm
        self.rank, self.world, self.group = rank, world, group
        self.ks = _capi.KeySwitch(ctx, prm.q_idx, prm.p_idx, prm.dnum, bconv_mode, round_mode, rank, world)
        self.n_local = self.ks.local_limbs
        self.g = self.ks.gather_limbs
        self.dtype = torch.int64 if ctx.word_bits == 64 else torch.int32
        self.device = device if device is not None else torch.device("cpu")
        n = ctx.n
        self.send = torch.zeros((self.g, n), dtype=self.dtype, device=self.device)
        self.gathered = torch.zeros((world, self.g, n), dtype=self.dtype, device=self.device)
        self.rot = torch.zeros((2, max(self.n_local, 1), n), dtype=self.dtype, device=self.device)

    def _stream(self) -> int:
        return torch.cuda.current_stream().cuda_stream if self.device.type == "cuda" else 0

    def _all_gather(self):
        if self.world == 1:
            self.gathered.copy_(self.send.unsqueeze(0))
        else:
            dist.all_gather_into_tensor(self.gathered.view(-1), self.send.view(-1), group=self.group)

    def keyswitch(self, out0: torch.Tensor, out1: torch.Tensor, cpoly: torch.Tensor, evk: torch.Tensor,
                  add0: Optional[torch.Tensor] = None, add1: Optional[torch.Tensor] = None):
        """out0, out1, cpoly, add*: [n_local, N]; evk: [dnum, 2, n_local + K, N] (this rank's shard)."""
        s = self._stream()
        self.ks.sharded_begin(self.send.data_ptr(), cpoly.data_ptr() if self.n_local else 0, s)
        self._all_gather()
        self.ks.sharded_finish(out0.data_ptr() if self.n_local else 0, out1.data_ptr() if self.n_local else 0,
                               self.gathered.data_ptr(), cpoly.data_ptr() if self.n_local else 0, evk.data_ptr(),
                               add0.data_ptr() if add0 is not None else 0,
                               add1.data_ptr() if add1 is not None else 0, s)

    def hrot(self, out0: torch.Tensor, out1: torch.Tensor, c0: torch.Tensor, c1: torch.Tensor, evk: torch.Tensor,
             galois_elt: int):
        """Rotation of a sharded ciphertext: automorphism of the local limbs, key switch of the
        rotated c1, rotated c0 added to the first output (cerium/compiler/backend/compiler.cc:701-726)."""
        s = self._stream()
        if self.n_local:
            r0, r1 = self.rot[0, :self.n_local], self.rot[1, :self.n_local]
            self.ctx.automorph(r0.data_ptr(), c0.data_ptr(), galois_elt, self.n_local, s)
            self.ctx.automorph(r1.data_ptr(), c1.data_ptr(), galois_elt, self.n_local, s)
            self.keyswitch(out0, out1, r1, evk, add0=r0)
        else:
            self.keyswitch(out0, out1, c1, evk)


def sharded_rescale(ctx: _capi.Context, q_idx: List[int], local: torch.Tensor, rank: int, world: int,
                    round_mode: int = _capi.ROUND_FLOOR, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Rescale of a limb-sharded ciphertext (cerium/compiler/backend/compiler_rescale.cc:209-284 with
    ``current_partition_size > 1``): the owner of the last limb inverse-transforms it and broadcasts
    the coefficient-form residues, every rank divides its remaining limbs.

    local: [n_polys, n_local, N], this rank's limbs of every polynomial (round robin over q_idx).
    Returns [n_polys, n_local', N] with the last limb gone (n_local' = n_local - 1 on its owner).
    """
    L = len(q_idx)
    n_polys = local.shape[0]
    owner = (L - 1) % world
    mine = local_limb_indices(L, rank, world)
    stream = torch.cuda.current_stream().cuda_stream if local.device.type == "cuda" else 0
    last = torch.empty((n_polys, ctx.n), dtype=local.dtype, device=local.device)
    if rank == owner:
        src = local[:, -1].contiguous()                      # limb L-1 is the owner's last local limb
        ctx.ntt_inverse(last.data_ptr(), src.data_ptr(), [q_idx[L - 1]] * n_polys, stream=stream)
    if world > 1:
        dist.broadcast(last, src=owner, group=group)
    keep = [i for i in mine if i != L - 1]
    if not keep:
        return local[:, :0].contiguous()
    rest = local[:, :len(keep)].contiguous()
    out = torch.empty_like(rest)
    ctx.rescale_local(out.data_ptr(), rest.data_ptr(), [q_idx[i] for i in keep], q_idx[L - 1], last.data_ptr(),
                      n_polys, round_mode, stream)
    return out
