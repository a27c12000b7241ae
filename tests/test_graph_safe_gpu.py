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
