"""Context-parallel decode across the GPUs of one node.

No counterpart in the upstream package (it is a single-device operator library).  Only one
shape needs an exchange: a single long sequence whose KV range is split over the ranks.  Each
rank attends to its own contiguous page range with the normal ``fmha_sail`` call (asking for
the LSE), then every rank all-gathers the per-rank (O, LSE) -- 33 KB per rank for 64 heads --
into its OWN memory with NCCL and runs the split-KV merge kernel with ``num_splits = world``.
Partials always land in local memory before a kernel reads them: no peer-memory loads.
"""
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from . import _lib
from ._lib import MSA_DT_F32


def shard_page_range(num_pages: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous, balanced split of ``num_pages`` logical pages: ``[begin, end)`` of ``rank``.
    The first ``num_pages % world`` ranks get one page more."""
    base, rem = divmod(num_pages, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def shard_units(num_units: int, rank: int, world: int):
    """Round-robin assignment of independent (batch item, KV-head group) units to ranks."""
    return list(range(rank, num_units, world))


def pack_partials(out_local: torch.Tensor, lse_local: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """What a rank contributes to the exchange: fp32 O ``[T, H, 128]`` and fp32 LSE ``[T, H]``."""
    return out_local.float().contiguous(), lse_local.float().contiguous()


def decode_allgather_merge(out_local: torch.Tensor, lse_local: torch.Tensor, group=None,
                           out: Optional[torch.Tensor] = None,
                           workspace: Optional[Tuple[torch.Tensor, torch.Tensor]] = None) -> torch.Tensor:
    """Combine per-rank attention results over disjoint key ranges.

    ``out_local [T, H, 128]`` (this rank's normalised output over ITS keys) and
    ``lse_local [T, H]`` (natural-log LSE over its keys; -inf if it saw none).  Returns the
    exact attention output over the union of all ranks' keys, replicated on every rank.
    """
    world = dist.get_world_size(group)
    T, H, D = out_local.shape
    po_l, pl_l = pack_partials(out_local, lse_local)
    if workspace is None:
        po = torch.empty(world, T, H, D, dtype=torch.float32, device=out_local.device)
        pl = torch.empty(world, T, H, dtype=torch.float32, device=out_local.device)
    else:
        po, pl = workspace
    dist.all_gather_into_tensor(po.view(-1), po_l.view(-1), group=group)     # flat views: rank-major layout
    dist.all_gather_into_tensor(pl.view(-1), pl_l.view(-1), group=group)
    if out is None:
        out = torch.empty(T, H, D, dtype=torch.bfloat16, device=out_local.device)
    _lib.check(_lib.lib.msa_lse_merge(
        po.data_ptr(), MSA_DT_F32, pl.data_ptr(), None, out.data_ptr(), None, world, T, H,
        out.stride(0), out.stride(1), 1.0, torch.cuda.current_stream().cuda_stream), "msa_lse_merge")
    return out
