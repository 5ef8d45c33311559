"""Limb-sharded key switching over several GPUs: the Python face of the library's sharded calls.

One process per GPU.  Q-limb ``i`` lives on rank ``i % world``
(``cerium/compiler/backend/terms.h:672-685``); the K extension limbs are replicated
(``Term::Ext``) or, with ``ext_split``, continue the round robin (``Ext_Split`` / ``PaE_Split``,
``terms.h:623-790``); evaluation keys are sharded with the limbs.  The exchanges - the all-gather of
the coefficient-form limbs before base conversion (the reference's DRM group,
``cerium/compiler/backend/compiler_keyswitch.cc:323-335``,
``cerium/runtime/execution/evaluator.cpp:1154-1251``) and, with split extension limbs, the all-gather
of the accumulators' extension limbs before ModDown - run inside the library on a ``_capi.Comm``
(NCCL, or the caller's collectives); this module only slices tensors and forwards pointers.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from . import _capi
from .params import CkksParams


def local_limb_indices(L: int, rank: int, world: int) -> List[int]:
    """Global indices of the Q-limbs rank ``rank`` owns (round robin)."""
    return list(range(rank, L, world))


def local_ext_indices(L: int, K: int, rank: int, world: int, ext_split: bool) -> List[int]:
    """Indices (0..K-1) of the extension limbs rank ``rank`` computes."""
    if not ext_split or world == 1:
        return list(range(K))
    return [k for k in range(K) if (L + k) % world == rank]


def shard_poly(poly: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """[L, N] -> this rank's limbs [n_local, N]."""
    return poly[local_limb_indices(poly.shape[0], rank, world)].contiguous()


def shard_key(evk: torch.Tensor, L: int, rank: int, world: int, ext_split: bool = False) -> torch.Tensor:
    """[dnum, 2, L+K, N] -> [dnum, 2, n_local+k_local, N]: the rank's Q-limbs and its extension limbs."""
    K = evk.shape[2] - L
    idx = local_limb_indices(L, rank, world) + [L + k for k in local_ext_indices(L, K, rank, world, ext_split)]
    return evk[:, :, idx].contiguous()


def nccl_comm(lib: _capi.Library, rank: int, world: int, device: int, group=None) -> _capi.Comm:
    """An NCCL communicator of the library; the id travels over the caller's torch.distributed group."""
    import torch.distributed as dist
    box = [_capi.Comm.unique_id(lib) if rank == 0 else None]
    dist.broadcast_object_list(box, src=0, group=group)
    return _capi.Comm(lib, rank, world, device, nccl_id=box[0])


class ShardedKeySwitch:
    """Key switch / HRot on the limbs of one rank; every rank calls the same method in step."""

    def __init__(self, ctx: _capi.Context, prm: CkksParams, comm: _capi.Comm,
                 bconv_mode: int = _capi.BCONV_LAZY, round_mode: int = _capi.ROUND_FLOOR, ext_split: bool = False):
        self.ctx, self.prm, self.comm = ctx, prm, comm
        self.rank, self.world = comm.rank, comm.world
        self.ks = _capi.KeySwitch(ctx, prm.q_idx, prm.p_idx, prm.dnum, bconv_mode, round_mode, self.rank, self.world,
                                  ext_split=ext_split)
        self.n_local = self.ks.local_limbs
        self.k_local = self.ks.local_ext_limbs
        self.g = self.ks.gather_limbs

    @staticmethod
    def _p(t: Optional[torch.Tensor]) -> int:
        return t.data_ptr() if t is not None and t.numel() else 0

    def keyswitch(self, out0, out1, cpoly, evk, add0=None, add1=None, stream: int = 0):
        """out0, out1, cpoly, add*: [n_local, N]; evk: [dnum, 2, n_local + k_local, N] (this rank's shard)."""
        self.ks.sharded_apply(self.comm, self._p(out0), self._p(out1), self._p(cpoly), evk.data_ptr(),
                              self._p(add0), self._p(add1), stream)

    def hrot(self, out0, out1, c0, c1, evk, galois_elt: int, stream: int = 0):
        """Rotation of a sharded ciphertext (cerium/compiler/backend/compiler.cc:701-726 on every partition)."""
        self.ks.hrot_sharded(self.comm, self._p(out0), self._p(out1), self._p(c0), self._p(c1), evk.data_ptr(),
                             galois_elt, stream)


def sharded_rescale(ctx: _capi.Context, comm: _capi.Comm, q_idx: List[int], local: torch.Tensor,
                    round_mode: int = _capi.ROUND_FLOOR, stream: int = 0) -> torch.Tensor:
    """Rescale of a limb-sharded ciphertext (cerium/compiler/backend/compiler_rescale.cc:209-284 with several
    partitions).  local: [n_polys, n_local, N], this rank's limbs of every polynomial.  Returns
    [n_polys, n_local', N] with the last limb gone (n_local' = n_local - 1 on its owner)."""
    L = len(q_idx)
    n_polys = local.shape[0]
    keep = [i for i in local_limb_indices(L, comm.rank, comm.world) if i != L - 1]
    last = torch.empty((n_polys, ctx.n), dtype=local.dtype, device=local.device)
    out = torch.empty((n_polys, len(keep), ctx.n), dtype=local.dtype, device=local.device)
    ctx.rescale_sharded(comm, out.data_ptr() if keep else 0, local.data_ptr() if local.numel() else 0, q_idx,
                        n_polys, last.data_ptr(), round_mode, stream)
    return out
