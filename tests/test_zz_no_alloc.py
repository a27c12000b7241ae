"""The allocation-free split-KV entry point (msa_fmha_fwd_split_static) against the regular
split path (msa_fmha_fwd + msa_lse_merge with a caller-owned workspace) and against the CPU oracle.

The entry point is for embedders that must not allocate device memory when they call into the
library (an engine whose own pool owns the device heap, a sandboxed plugin host): its per-split
scratch is a fixed array inside the library.  Two calls in a row, with different shapes, check
that what the first call left in that shared array does not leak into the second result.
Collected last on purpose (file name), and self-contained so it also passes alone.
"""
import ctypes

import pytest
import torch

from helpers import BF16_COS, BF16_MAX_ABS, check_out, gen, randn_bf16
from oracle import msa_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _params_from_plan(L, plan, q, k, v, out, lse):
    """Hand-built argument struct for a ragged, unpaged, dense call (same fields the Python API fills)."""
    p = L.MsaFmhaParams()
    p.q, p.k, p.v, p.out, p.lse = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr()
    p.q_stride_tok, p.q_stride_head = q.stride(0), q.stride(1)
    p.k_stride_tok, p.k_stride_head = k.stride(0), k.stride(1)
    p.v_stride_tok, p.v_stride_head = v.stride(0), v.stride(1)
    p.out_stride_tok, p.out_stride_head = out.stride(0), out.stride(1)
    p.qo_start = plan["qo_segment_offsets"].data_ptr()
    p.kv_start = plan["kv_segment_offsets"].data_ptr()
    p.kv_len = plan["kv_segment_lens"].data_ptr()
    p.qo_offset = plan["qo_offset"].data_ptr()
    p.work, p.num_work = plan["work"].data_ptr(), plan["num_work"]
    p.kv_extent = k.shape[0]
    p.total_q, p.num_qo_heads, p.num_kv_heads = q.shape[0], q.shape[1], k.shape[1]
    p.batch = plan["batch_size"]
    p.block_m, p.pack, p.page_size = plan["qo_tile_size"], plan["pack_factor"], 0
    p.num_splits = plan["num_kv_splits"]
    p.q_dtype = p.kv_dtype = L.MSA_DT_BF16
    p.flags = L.FLAG_OUT_O
    p.sm_scale, p.out_scale = 1.0 / 128 ** 0.5, 1.0
    return p


def _one_round(api, L, seed, kv_lens, hq, hk, splits, pass_spr=True):
    g = gen(seed)
    n = len(kv_lens)
    q_h = randn_bf16(g, n, hq, 128)
    k_h = randn_bf16(g, sum(kv_lens), hk, 128)
    v_h = randn_bf16(g, sum(kv_lens), hk, 128)
    q, k, v = q_h.to(DEV), k_h.to(DEV), v_h.to(DEV)
    lens = torch.ones(n, dtype=torch.int32)
    plan = api.fmha_sail_plan(lens, torch.tensor(kv_lens, dtype=torch.int32), hq, num_kv_heads=hk,
                              num_kv_splits=splits)
    pl = plan[3]
    assert pl["num_kv_splits"] > 1 and pl["workspace_o"] is not None       # the regular path uses scratch
    lse_ref = torch.empty(n, hq, dtype=torch.float32, device=DEV)
    out_ref, _ = api.fmha_sail(q, k, v, plan, lse=lse_ref)

    out = torch.full((n, hq, 128), 7.0, dtype=torch.bfloat16, device=DEV)
    lse = torch.full((n, hq), 7.0, dtype=torch.float32, device=DEV)
    p = _params_from_plan(L, pl, q, k, v, out, lse)
    spr = pl["num_kv_splits_per_row"]
    torch.cuda.synchronize()
    free0, alloc0 = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
    rc = L.lib.msa_fmha_fwd_split_static(ctypes.byref(p), spr.data_ptr() if pass_spr else None,
                                         torch.cuda.current_stream().cuda_stream)
    assert rc == 0, L.lib.msa_status_string(rc)
    torch.cuda.synchronize()
    # the call takes no device memory, neither from the driver nor from torch's pool
    assert torch.cuda.memory_allocated() == alloc0
    if getattr(_one_round, "warm", False):               # the first call on a device resolves the array's address
        assert torch.cuda.mem_get_info()[0] >= free0
    _one_round.warm = True
    ones = [1] * n
    check_out(out, orc.attention(q_h, k_h, v_h, ones, kv_lens, hq, hk), "static scratch vs oracle")
    a, b = out.float().cpu(), out_ref.float().cpu()
    assert torch.isfinite(a).all()
    assert (a - b).abs().max().item() <= BF16_MAX_ABS
    cos = torch.nn.functional.cosine_similarity(a.reshape(-1).double(), b.reshape(-1).double(), dim=0).item()
    assert cos >= BF16_COS
    assert torch.allclose(lse.cpu(), lse_ref.cpu(), atol=1e-4, rtol=1e-4)


def test_static_scratch_matches_regular_split_path_twice():
    import msa_for_sail as api
    from msa_for_sail import _lib as L
    _one_round(api, L, 1, [3000, 700, 2000, 129], 16, 2, 4)     # fills a large part of the scratch
    _one_round(api, L, 2, [1500, 260], 8, 2, 3)                 # smaller problem on the stale scratch


def test_static_scratch_ignores_slots_no_work_item_wrote():
    """Without splits_per_row the merge looks at all S slots of every token.  The 129-key sequence
    has one key tile, hence one work item per head group: its other slots are written by nobody in
    this call and still hold the partials of the larger call before it.  They must count as empty."""
    import msa_for_sail as api
    from msa_for_sail import _lib as L
    _one_round(api, L, 3, [4000, 3000, 2500, 3500], 16, 2, 4)
    _one_round(api, L, 4, [129, 1800, 140], 16, 2, 4, pass_spr=False)


def test_static_scratch_rejects_oversize_and_foreign_workspace():
    import msa_for_sail as api
    from msa_for_sail import _lib as L
    p = L.MsaFmhaParams()
    dummy = torch.zeros(64, dtype=torch.float32, device=DEV)
    for f in ("q", "k", "v", "out", "qo_start", "kv_start", "kv_len", "qo_offset"):
        setattr(p, f, dummy.data_ptr())
    p.flags, p.block_m, p.pack = L.FLAG_OUT_O, 16, 1
    p.num_qo_heads = p.num_kv_heads = 64
    p.num_splits, p.total_q = 8, 64                      # 8 * 64 * 64 = 32768 rows > 16384
    assert L.lib.msa_fmha_fwd_split_static(ctypes.byref(p), None, None) == -4
    p.num_splits = 1
    p.partial_o = dummy.data_ptr()                       # caller-provided scratch is refused here
    assert L.lib.msa_fmha_fwd_split_static(ctypes.byref(p), None, None) == -1
