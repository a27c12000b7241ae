"""Graph-safe planning: plan + run captured in one CUDA graph, replayed after the length tensors
and the page table were updated in place (upstream graph_safe mode, api.py:916-941 and the
usage described in allocate_graph_workspace, api.py:383-447)."""
import os
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path.insert(0, os.path.join(ROOT, "msa-for-sail_b200", "python"))
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)

from helpers import check_out, gen, randn_bf16, random_blocks   # noqa: E402
from oracle import msa_oracle as orc                          # noqa: E402

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _i32(x, device="cpu"):
    return torch.tensor(x, dtype=torch.int32, device=device)


def _state(g, kv_lens, n_pool):
    """A page table for these lengths over a fixed pool of `n_pool` pages."""
    pages = sum((kl + 127) // 128 for kl in kv_lens)
    return torch.randperm(n_pool, generator=g)[:pages].to(torch.int32)


@pytest.mark.parametrize("splits", [1, 3])
def test_dense_decode_plan_and_run_in_one_graph(splits):
    import msa_for_sail as api
    g = gen(2024 + splits)
    batch, hq, hk, n_pool, max_kv = 3, 16, 2, 64, 2048
    states = [[1000, 300, 2000], [1500, 128, 777], [64, 2048, 1]]
    kp = randn_bf16(g, n_pool, hk, 128, 128); vp = randn_bf16(g, n_pool, hk, 128, 128)
    q = randn_bf16(g, batch, hq, 128)
    qd, kd, vd = q.to(DEV), kp.to(DEV), vp.to(DEV)
    qo_lens = _i32([1] * batch, DEV)
    kv_lens = _i32(states[0], DEV)
    qo_off = torch.full((batch,), -1, dtype=torch.int32, device=DEV)      # -1: kv_len - qo_len
    table_dev = torch.zeros(batch * (max_kv // 128), dtype=torch.int32, device=DEV)
    out = torch.empty(batch, hq, 128, dtype=torch.bfloat16, device=DEV)
    ws = api.allocate_graph_workspace(batch, hq, num_kv_heads=hk, max_qo_len=1, page_size=128, num_kv_splits=splits)

    def step():
        plan = api.fmha_sail_plan(qo_lens, kv_lens, hq, num_kv_heads=hk, page_size=128, num_kv_splits=splits,
                                  qo_offset=qo_off, given_workspace=ws, max_total_q=batch, graph_safe=True,
                                  max_qo_len_override=1, qo_len_uniform_override=True, max_kv_len_override=max_kv)
        api.fmha_sail(qd, kd, vd, plan, kv_indices=table_dev, out=out)

    def load(state_lens, table):
        kv_lens.copy_(_i32(state_lens))
        table_dev[:table.numel()].copy_(table)

    def reference(state_lens, table):
        k = orc.paged_to_contiguous(kp, table, state_lens, 128)
        v = orc.paged_to_contiguous(vp, table, state_lens, 128)
        return orc.attention(q, k, v, [1] * batch, state_lens, hq, hk)

    tables = [_state(g, s, n_pool) for s in states]
    load(states[0], tables[0])
    step()                                                    # eager warm-up (creates the status word etc.)
    torch.cuda.synchronize()
    check_out(out, reference(states[0], tables[0]), "graph-safe eager")

    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    for lens, table in zip(states, tables):
        load(lens, table)
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        check_out(out, reference(lens, table), f"graph-safe replay {lens}")
    from msa_for_sail import api as api_mod
    assert api_mod.last_status() == 0


def test_sparse_decode_plan_and_run_in_one_graph():
    import msa_for_sail as api
    g = gen(777)
    batch, hq, hk, kbn, n_pool, max_kv = 2, 16, 2, 4, 80, 4096
    states = [[3000, 1000], [700, 4096]]
    kp = randn_bf16(g, n_pool, hk, 128, 128); vp = randn_bf16(g, n_pool, hk, 128, 128)
    q = randn_bf16(g, batch, hq, 128)
    qd, kd, vd = q.to(DEV), kp.to(DEV), vp.to(DEV)
    qo_lens = _i32([1] * batch, DEV)
    kv_lens = _i32(states[0], DEV)
    qo_off = torch.full((batch,), -1, dtype=torch.int32, device=DEV)
    table_dev = torch.zeros(batch * (max_kv // 128), dtype=torch.int32, device=DEV)
    bi_dev = torch.full((batch, hk, kbn), -1, dtype=torch.int32, device=DEV)
    out = torch.empty(batch, hq, 128, dtype=torch.bfloat16, device=DEV)
    ws = api.allocate_graph_workspace(batch, hq, num_kv_heads=hk, max_qo_len=1, page_size=128, kv_block_num=kbn,
                                      num_kv_splits=2)

    def step():
        plan = api.fmha_sail_plan(qo_lens, kv_lens, hq, num_kv_heads=hk, page_size=128, kv_block_num=kbn,
                                  num_kv_splits=2, qo_offset=qo_off, given_workspace=ws, max_total_q=batch,
                                  graph_safe=True, max_qo_len_override=1, qo_len_uniform_override=True,
                                  max_kv_len_override=max_kv)
        api.fmha_sail(qd, kd, vd, plan, kv_indices=table_dev, kv_block_indexes=bi_dev, out=out)

    tables = [_state(g, s, n_pool) for s in states]
    blocks = [random_blocks(g, [1] * batch, s, [kl - 1 for kl in s], hk, kbn) for s in states]

    def load(i):
        kv_lens.copy_(_i32(states[i]))
        table_dev[:tables[i].numel()].copy_(tables[i])
        bi_dev.copy_(blocks[i])

    load(0)
    step()
    torch.cuda.synchronize()
    check_out(out, orc.sparse_attention(q, kp, vp, [1] * batch, states[0], tables[0], blocks[0], hq), "sparse graph-safe eager")
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    for i in (1, 0):
        load(i)
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        check_out(out, orc.sparse_attention(q, kp, vp, [1] * batch, states[i], tables[i], blocks[i], hq),
                  f"sparse graph-safe replay {i}")
    from msa_for_sail import api as api_mod
    assert api_mod.last_status() == 0


@pytest.mark.parametrize("causal,paged", [(True, True), (False, True), (True, False)])
def test_plan_device_fills_what_its_header_says(causal, paged):
    """msa_plan_device against a direct evaluation of the formulas in include/msa_b200.h."""
    import ctypes
    import numpy as np
    from msa_for_sail import _lib
    rng = np.random.default_rng(5 + causal + 2 * paged)
    batch, hq, hk, pack, block_m, S, page = 7, 16, 2, 8, 16, 3, 128 if paged else 0
    ql = rng.integers(0, 3, batch).astype(np.int32)           # 0, 1 or 2 tokens: 2 * 8 rows fill the 16-row tile
    kl = rng.integers(1, 3000, batch).astype(np.int32)
    off_in = np.where(rng.random(batch) < 0.5, -1, rng.integers(0, 2500, batch)).astype(np.int32)
    max_total_q = int(ql.sum()) + 3
    groups = hq // pack
    dev = lambda a: torch.from_numpy(a).to(DEV)
    d_ql, d_kl, d_off = dev(ql), dev(kl), dev(off_in)
    z = lambda n: torch.full((n,), -7, dtype=torch.int32, device=DEV)
    qo_start, kv_start, kv_len_out, off_out = z(batch + 1), z(batch + 1), z(batch), z(batch)
    indptr, token_batch, spr = z(batch + 1), z(max_total_q), z(max_total_q)
    work = z(batch * groups * S * 8)
    a = _lib.MsaPlanDeviceArgs()
    a.qo_len, a.kv_len, a.qo_offset_in = d_ql.data_ptr(), d_kl.data_ptr(), d_off.data_ptr()
    a.qo_start, a.kv_start, a.kv_len_out, a.qo_offset_out = (qo_start.data_ptr(), kv_start.data_ptr(),
                                                             kv_len_out.data_ptr(), off_out.data_ptr())
    a.kv_page_indptr = indptr.data_ptr() if paged else None
    a.token_batch, a.splits_per_row, a.work = token_batch.data_ptr(), spr.data_ptr(), work.data_ptr()
    a.batch, a.num_qo_heads, a.num_kv_heads, a.block_m, a.pack, a.num_splits = batch, hq, hk, block_m, pack, S
    a.page_size, a.causal, a.noncausal_offset, a.max_total_q, a.row_tiles = page, int(causal), 4000, max_total_q, 1
    assert _lib.lib.msa_plan_device(ctypes.byref(a), torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    exp_off = np.where(off_in < 0, kl - ql, off_in) if causal else np.full(batch, 4000)
    assert np.array_equal(qo_start.cpu().numpy(), np.concatenate([[0], np.cumsum(ql)]))
    assert np.array_equal(kv_start.cpu().numpy(), np.concatenate([[0], np.cumsum(kl)]))
    assert np.array_equal(kv_len_out.cpu().numpy(), kl) and np.array_equal(off_out.cpu().numpy(), exp_off)
    if paged:
        assert np.array_equal(indptr.cpu().numpy(), np.concatenate([[0], np.cumsum((kl + 127) // 128)]))
    tb = token_batch.cpu().numpy()
    assert np.array_equal(tb[:ql.sum()], np.repeat(np.arange(batch), ql)) and (tb[ql.sum():] == 0).all()
    sp = spr.cpu().numpy()
    assert (sp[:ql.sum()] == S).all() and (sp[ql.sum():] == 0).all()     # padding rows: no splits to merge
    w = work.cpu().numpy().reshape(batch, groups, S, 8)
    for b in range(batch):
        nrows = min(block_m, int(ql[b]) * pack)
        vis = max(0, min(int(kl[b]), (nrows - 1) // pack + int(exp_off[b]) + 1)) if nrows > 0 else 0
        nt = (vis + 127) // 128
        chunk = max(1, -(-nt // S))
        for g in range(groups):
            for s in range(S):
                it = w[b, g, s]
                assert (it[0], it[1], it[2], it[5], it[6]) == (b, g * pack, 0, s, nrows)
                assert (it[3], it[4]) == (min(nt, s * chunk), min(nt, (s + 1) * chunk))


@pytest.mark.parametrize("splits", [1, 2])
def test_chunked_prefill_plan_and_run_in_one_graph(splits):
    """Several row tiles per batch item, ragged query lengths that change between replays:
    splits = 1 takes the tcgen05 prefill kernel, splits = 2 the generic kernel with a merge."""
    import msa_for_sail as api
    g = gen(99 + splits)
    batch, hq, hk, n_pool, max_kv, max_qo = 2, 4, 2, 40, 2048, 300
    max_total_q = batch * max_qo
    states = [([300, 120], [1000, 700]), ([100, 300], [2048, 300]), ([1, 257], [5, 1500])]
    kp = randn_bf16(g, n_pool, hk, 128, 128); vp = randn_bf16(g, n_pool, hk, 128, 128)
    q = randn_bf16(g, max_total_q, hq, 128)
    qd, kd, vd = q.to(DEV), kp.to(DEV), vp.to(DEV)
    qo_lens = _i32(states[0][0], DEV)
    kv_lens = _i32(states[0][1], DEV)
    qo_off = torch.full((batch,), -1, dtype=torch.int32, device=DEV)
    table_dev = torch.zeros(batch * (max_kv // 128), dtype=torch.int32, device=DEV)
    out = torch.zeros(max_total_q, hq, 128, dtype=torch.bfloat16, device=DEV)
    ws = api.allocate_graph_workspace(batch, hq, num_kv_heads=hk, max_qo_len=max_qo, page_size=128,
                                      num_kv_splits=splits)

    def step():
        plan = api.fmha_sail_plan(qo_lens, kv_lens, hq, num_kv_heads=hk, page_size=128, num_kv_splits=splits,
                                  qo_offset=qo_off, given_workspace=ws, max_total_q=max_total_q, graph_safe=True,
                                  max_qo_len_override=max_qo, qo_len_uniform_override=False,
                                  max_kv_len_override=max_kv)
        api.fmha_sail(qd, kd, vd, plan, kv_indices=table_dev, out=out)

    tables = [_state(g, s[1], n_pool) for s in states]

    def load(i):
        qo_lens.copy_(_i32(states[i][0])); kv_lens.copy_(_i32(states[i][1]))
        table_dev[:tables[i].numel()].copy_(tables[i])

    def check(i, name):
        ql, kl = states[i]
        n = sum(ql)
        k = orc.paged_to_contiguous(kp, tables[i], kl, 128)
        v = orc.paged_to_contiguous(vp, tables[i], kl, 128)
        check_out(out[:n], orc.attention(q[:n], k, v, ql, kl, hq, hk), name)
        if splits > 1:                                   # rows past the last token are merged from nothing
            assert (out[n:] == 0).all(), f"{name}: padded rows are not zero"

    load(0)
    step()
    torch.cuda.synchronize()
    check(0, "prefill graph-safe eager")
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    for i in (1, 2, 0):
        load(i)
        out.fill_(3.0)                                   # every real row, and with splits the padding, is rewritten
        graph.replay()
        torch.cuda.synchronize()
        check(i, f"prefill graph-safe replay {i}")
    from msa_for_sail import api as api_mod
    assert api_mod.last_status() == 0
