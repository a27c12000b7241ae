"""World-size-2 check (gloo, CPU) of the context-parallel decode exchange: each rank attends to
its own page range, the ranks all-gather their packed (O, LSE) blocks and merge.  The GPU code path does the same with
NCCL and the merge kernel; here the oracle stands in for both kernels so that the host-side logic
(page-range sharding, gather layout, merge semantics incl. a rank that owns no key) is covered
without a GPU."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def _worker(rank, world, port, kv_len, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "msa-for-sail_b200", "python"))
    from msa_for_sail import dist as mdist
    from oracle import msa_oracle as orc
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = torch.Generator().manual_seed(5)
    hq, hk, page = 8, 2, 128
    q = torch.randn(1, hq, 128, generator=g)
    k = torch.randn(kv_len, hk, 128, generator=g)
    v = torch.randn(kv_len, hk, 128, generator=g)
    n_pages = (kv_len + page - 1) // page
    p0, p1 = mdist.shard_page_range(n_pages, rank, world)
    s, e = p0 * page, min(kv_len, p1 * page)
    if e > s:
        o, lse = orc.attention(q, k[s:e], v[s:e], [1], [e - s], hq, hk, causal=False, return_lse=True)
    else:                                            # this rank owns no key
        o, lse = torch.zeros(1, hq, 128), torch.full((1, hq), -float("inf"))
    # the packed block of the exchange: [O: T*H*128 floats | LSE: T*H floats], one collective
    ex = mdist.DecodeExchange(1, hq, torch.device("cpu"))
    ex.o_local.copy_(o); ex.lse_local.copy_(lse)
    dist.all_gather_into_tensor(ex.gathered, ex.local)
    blocks = ex.gathered.view(world, ex.block)          # what the merge kernel is pointed at: split stride = block
    po = blocks[:, :hq * 128].reshape(world, 1, hq, 128)
    pl = blocks[:, hq * 128:].reshape(world, 1, hq)
    merged = orc.lse_merge(po, pl)
    full = orc.attention(q, k, v, [1], [kv_len], hq, hk, causal=False)
    ok = torch.allclose(merged, full, atol=1e-5, rtol=1e-5)
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        ret.put(bool(ok))


def _run(world, kv_len, port):
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, kv_len, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert ret.get(timeout=10) is True


def test_context_parallel_decode_two_ranks():
    _run(2, 1000, 29731)


def test_context_parallel_decode_rank_without_keys():
    _run(2, 100, 29732)          # one page only: rank 1 gets an empty range


def test_shard_helpers():
    sys.path.insert(0, os.path.join(ROOT, "msa-for-sail_b200", "python"))
    from msa_for_sail import dist as mdist
    for n, w in ((8192, 8), (10, 4), (3, 8), (0, 2)):
        ranges = [mdist.shard_page_range(n, r, w) for r in range(w)]
        assert ranges[0][0] == 0 and ranges[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
        assert max(e - s for s, e in ranges) - min(e - s for s, e in ranges) <= 1
    assert sorted(sum((mdist.shard_units(32, r, 8) for r in range(8)), [])) == list(range(32))
    for n, w in ((32, 8), (16, 4), (256, 8), (16, 2), (5, 2)):
        blocks = [mdist.shard_units(n, r, w, contiguous=True) for r in range(w)]
        assert sum(blocks, []) == list(range(n))            # contiguous, in rank order, nothing lost
