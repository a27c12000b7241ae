"""Context-parallel decode across the GPUs of one node, and the sharding arithmetic.

No counterpart in the upstream package (it is a single-device operator library).  Only one
shape needs an exchange: a single long sequence whose KV range is split over the ranks.  Each
rank attends to its own contiguous page range with the normal ``fmha_sail`` call, asking for the
unrounded fp32 output and the LSE, which land side by side in one packed buffer
``[O: T*H*128 floats | LSE: T*H floats]`` -- 33 KB for one token and 64 heads.  ONE
``all_gather_into_tensor`` brings every rank's block into this rank's OWN memory, and the
split-KV merge kernel (``msa_lse_merge_ex`` with ``num_splits = world`` and the block size as the
split stride) produces the exact result on every rank.  Partials always land in local memory
before a kernel reads them: no peer-memory loads.
"""
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from . import _lib
from ._lib import MSA_DT_BF16, MSA_DT_F32

HEAD_DIM = 128


def shard_page_range(num_pages: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous, balanced split of ``num_pages`` logical pages: ``[begin, end)`` of ``rank``.
    The first ``num_pages % world`` ranks get one page more."""
    base, rem = divmod(num_pages, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def shard_units(num_units: int, rank: int, world: int, contiguous: bool = False) -> List[int]:
    """Assignment of independent (batch item, KV-head group) units to ranks: round-robin, or in
    contiguous balanced blocks (units of one batch item stay together, so that per-batch work such
    as the proxy pass is repeated on as few ranks as possible)."""
    if contiguous:
        begin, end = shard_page_range(num_units, rank, world)
        return list(range(begin, end))
    return list(range(rank, num_units, world))


class DecodeExchange:
    """Buffers and the two steps of the cross-rank combine for ``tokens`` query tokens x ``heads``.

    ``local_kwargs()`` are the ``out=`` / ``lse=`` arguments of this rank's ``fmha_sail`` call (fp32
    views into the packed block); ``allgather_merge()`` then runs the single collective and the merge.
    Everything is allocated once, here."""

    def __init__(self, tokens: int, heads: int, device, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.tokens, self.heads = tokens, heads
        rows = tokens * heads
        self.block = rows * (HEAD_DIM + 1)
        self.local = torch.empty(self.block, dtype=torch.float32, device=device)
        self.gathered = torch.empty(self.world * self.block, dtype=torch.float32, device=device)
        self.o_local = self.local[:rows * HEAD_DIM].view(tokens, heads, HEAD_DIM)
        self.lse_local = self.local[rows * HEAD_DIM:].view(tokens, heads)

    def local_kwargs(self):
        return {"out": self.o_local, "lse": self.lse_local}

    def allgather_merge(self, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """All-gather the packed (O, LSE) blocks and merge them into ``out`` (bf16 ``[T, H, 128]``)."""
        dist.all_gather_into_tensor(self.gathered, self.local, group=self.group)
        return self.merge_gathered(out)

    def merge_gathered(self, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        rows = self.tokens * self.heads
        if out is None:
            out = torch.empty(self.tokens, self.heads, HEAD_DIM, dtype=torch.bfloat16, device=self.local.device)
        lse_ptr = self.gathered.data_ptr() + rows * HEAD_DIM * 4
        _lib.check(_lib.lib.msa_lse_merge_ex(
            self.gathered.data_ptr(), MSA_DT_F32, lse_ptr, None, out.data_ptr(), MSA_DT_BF16, None,
            self.world, self.tokens, self.heads, self.block, self.block, out.stride(0), out.stride(1), 1.0,
            torch.cuda.current_stream().cuda_stream), "msa_lse_merge_ex")
        return out


def decode_allgather_merge(out_local: torch.Tensor, lse_local: torch.Tensor, group=None,
                           out: Optional[torch.Tensor] = None,
                           exchange: Optional[DecodeExchange] = None) -> torch.Tensor:
    """Combine per-rank attention results over disjoint key ranges.

    ``out_local [T, H, 128]`` (this rank's normalised output over ITS keys, fp32 or bf16) and
    ``lse_local [T, H]`` (natural-log LSE over its keys; -inf if it saw none).  Returns the
    exact attention output over the union of all ranks' keys, replicated on every rank.
    Convenience form of ``DecodeExchange`` for results that already exist: they are copied into
    the packed block first.  A step that runs every iteration should let ``fmha_sail`` write into
    ``DecodeExchange.local_kwargs()`` instead."""
    T, H, _ = out_local.shape
    ex = exchange if exchange is not None else DecodeExchange(T, H, out_local.device, group)
    ex.o_local.copy_(out_local)
    ex.lse_local.copy_(lse_local)
    return ex.allgather_merge(out)
