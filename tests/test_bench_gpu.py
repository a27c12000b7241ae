"""bench.py on the GPU at reduced sizes: the end-to-end legs (chunked prefill from pinned host
memory, three streams) must produce what the single device-resident call produces, and the parity
samples that every timed workload ends with must pass -- on the K distribution of the sparse
prefill configuration (per-page mean offsets), on the e4m3 decode pipeline with per-head scales,
and on the paged decode."""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "msa-for-sail_b200", "python"))

pytestmark = pytest.mark.gpu


def test_prefill_end_to_end_step_matches_the_resident_step():
    import bench
    import msa_for_sail as msa
    dev = torch.device("cuda:0")
    wl = bench.setup_prefill(msa, dev, 7, b=2, ql=2048, kl=2048, hq=16, hk=2)
    wl["step"]()
    r = wl["parity"]()                   # the device-timed step (random permutation of the pool) against the oracle
    assert r["rows"] >= 64 and r["max_abs"] <= 2e-2
    wl["e2e_ref_step"]()                 # one resident call on the cache layout of the end-to-end leg
    wl["e2e_step"]()
    wl["e2e_step"]()                     # buffers are reused step after step
    torch.cuda.synchronize()
    out, out_h = wl["results"]
    ref = out.float().cpu()
    got = out_h.float()
    assert torch.isfinite(got).all()
    # bf16 outputs of the same rows computed with the same key tiles: max-abs 2e-2 as everywhere else
    assert (got - ref).abs().max().item() <= 2e-2
    cos = torch.nn.functional.cosine_similarity(got.flatten(), ref.flatten(), dim=0).item()
    assert cos >= 0.9999


def test_msa_prefill_end_to_end_step_matches_the_resident_step():
    """Chunked sparse prefill (row chunks with growing kv_len) selects the same pages and gives the
    same output as the whole sequence in one call; K carries one N(0, 2) offset per (page, head)."""
    import bench
    import msa_for_sail as msa
    dev = torch.device("cuda:0")
    wl = bench.setup_msa_prefill(msa, dev, 11, b=2, t=8192, hq=16, hk=2, topk=8)
    wl["step"]()
    r = wl["parity"]()
    assert r["topk_exact"] and r["rows"] >= 64
    wl["e2e_step"]()
    wl["e2e_step"]()
    torch.cuda.synchronize()
    out, out_h = wl["results"]
    ref, got = out.float().cpu(), out_h.float()
    assert torch.isfinite(got).all()
    assert (got - ref).abs().max().item() <= 2e-2
    assert torch.nn.functional.cosine_similarity(got.flatten(), ref.flatten(), dim=0).item() >= 0.9999


@pytest.mark.parametrize("hq,hk,topk", [(64, 8, 16), (16, 2, 8)])
def test_msa_prefill_parity_sample_with_page_offsets(hq, hk, topk):
    """The sparse prefill pipeline at the head counts of the target configuration, shorter sequences."""
    import bench
    import msa_for_sail as msa
    wl = bench.setup_msa_prefill(msa, torch.device("cuda:0"), 5, b=2, t=4096, hq=hq, hk=hk, topk=topk)
    wl["step"]()
    r = wl["parity"]()
    assert r["topk_exact"] and r["max_abs"] <= 2e-2 and r["cos"] >= 0.9999


def test_e4m3_prefill_workloads_parity_sample_and_end_to_end():
    """The e4m3 variants of the dense and the sparse prefill workloads at reduced sizes: parity sample of the
    timed step, and the chunked end-to-end leg against the resident call."""
    import bench
    import msa_for_sail as msa
    dev = torch.device("cuda:0")
    wl = bench.setup_prefill(msa, dev, 9, b=2, ql=2048, kl=2048, hq=16, hk=2, fp8=True)
    wl["step"]()
    r = wl["parity"]()
    assert r["rows"] >= 64 and r["cos"] >= 0.999
    wl["e2e_ref_step"](); wl["e2e_step"](); wl["e2e_step"]()
    torch.cuda.synchronize()
    out, out_h = wl["results"]
    assert torch.nn.functional.cosine_similarity(out_h.float().flatten(), out.float().cpu().flatten(), dim=0).item() >= 0.9999
    del wl
    wl = bench.setup_msa_prefill(msa, dev, 10, b=2, t=4096, hq=64, hk=8, topk=16, fp8=True)
    wl["step"]()
    r = wl["parity"]()
    assert r["topk_exact"] and r["cos"] >= 0.999
    wl["e2e_step"](); wl["e2e_step"]()
    torch.cuda.synchronize()
    out, out_h = wl["results"]
    assert torch.isfinite(out_h.float()).all()
    assert torch.nn.functional.cosine_similarity(out_h.float().flatten(), out.float().cpu().flatten(), dim=0).item() >= 0.9999


@pytest.mark.parametrize("fp8", [True, False])
def test_msa_decode_parity_sample(fp8):
    """The decode pipeline in the shape of the target configuration (many batch items, 1 024-page
    sequences, top-16, 4 requested splits; e4m3 cache with one scale per KV head), smaller batch."""
    import bench
    import msa_for_sail as msa
    wl = bench.setup_msa_decode(msa, torch.device("cuda:0"), 6, b=8, kl=131072, hq=64, hk=8, topk=16, splits=4, fp8=fp8)
    wl["step"]()
    wl["e2e_step"]()
    r = wl["parity"]()
    assert r["topk_exact"] and r["rows"] == 8 * 64
    assert msa.api.last_status() == 0


def test_paged_decode_parity_sample():
    import bench
    import msa_for_sail as msa
    wl = bench.setup_decode(msa, torch.device("cuda:0"), 8, b=1, kl=65536, hq=64, hk=8)
    wl["step"]()
    r = wl["parity"]()
    assert r["rows"] == 64 and r["lse_max_abs"] <= 2e-2
