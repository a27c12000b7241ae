"""Multi-GPU check of the context-parallel decode: each rank runs `fmha_sail` over its own page
range, writing its unrounded fp32 (O, LSE) into the packed exchange block; one NCCL all-gather and the
merge kernel combine them; compared with the oracle over the whole sequence.  Runs with 2, 4 and 8
ranks where the box has that many GPUs (skipped otherwise)."""
import os
import sys

import pytest
import torch

from conftest import ROOT

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "msa-for-sail_b200", "python"))
    import torch.distributed as dist
    import msa_for_sail as msa
    from msa_for_sail import dist as mdist
    from oracle import msa_oracle as orc
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    g = torch.Generator().manual_seed(9)
    hq, hk, page, n_pages = 16, 2, 128, 37 * world
    kv_len = n_pages * page
    q = torch.randn(1, hq, 128, generator=g).to(torch.bfloat16)
    kp = torch.randn(n_pages, hk, page, 128, generator=g).to(torch.bfloat16)
    vp = torch.randn(n_pages, hk, page, 128, generator=g).to(torch.bfloat16)
    p0, p1 = mdist.shard_page_range(n_pages, rank, world)
    table = torch.arange(p1 - p0, dtype=torch.int32, device=dev)
    lens = (torch.tensor([1], dtype=torch.int32), torch.tensor([(p1 - p0) * page], dtype=torch.int32))
    errs = []
    for splits in (-1, 1):              # split-KV (the merge writes fp32 itself) and unsplit (converted from bf16)
        plan = msa.fmha_sail_plan(*lens, hq, num_kv_heads=hk, page_size=page, causal=False, num_kv_splits=splits)
        ex = mdist.DecodeExchange(1, hq, dev)
        msa.fmha_sail(q.to(dev), kp[p0:p1].to(dev), vp[p0:p1].to(dev), plan, kv_indices=table, **ex.local_kwargs())
        merged = ex.allgather_merge()
        torch.cuda.synchronize()
        k = kp.permute(0, 2, 1, 3).reshape(kv_len, hk, 128); v = vp.permute(0, 2, 1, 3).reshape(kv_len, hk, 128)
        ref = orc.attention(q, k, v, [1], [kv_len], hq, hk, causal=False)
        errs.append((merged.float().cpu() - ref).abs().max().item())
        # the convenience form on results that already exist
        merged2 = mdist.decode_allgather_merge(ex.o_local.clone(), ex.lse_local.clone())
        errs.append((merged2.float() - merged.float()).abs().max().item())
    dist.barrier()
    dist.destroy_process_group()
    ret.put((rank, max(errs)))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_context_parallel_decode_nccl(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, 29741 + world, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    errs = dict(ret.get(timeout=10) for _ in range(world))
    assert max(errs.values()) <= 2e-2, errs
