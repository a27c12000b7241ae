"""Seeded chaos suite: random ragged / paged / sparse batches through the public API against the
CPU oracle, after the upstream chaos cases (tests/regression/test_correctness.py:564-1134: random
batch size, query / key lengths and causal offsets per item, items ordered by query length so that
`split_prefill_decode` can cut the batch, a random choice of that flag, five head configurations,
four `kv_block_num`s).  Sizes are bounded so that the oracle for all 210 cases stays under a minute;
a failure names the family and the seed that reproduces it.
"""
import random

import pytest
import torch

from helpers import (BF16_COS, BF16_MAX_ABS, FP8_COS, check_out, check_score, gen, make_paged, randn_bf16,
                     random_blocks)
from oracle import msa_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"
HEADS = [(2, 2), (4, 1), (8, 2), (16, 2), (8, 8)]       # (query heads, KV heads)
SEEDS_PER_FAMILY = 70


def _i32(x):
    return torch.tensor(x, dtype=torch.int32)


def _shape(rng, q_budget, max_kv):
    """Batch of 1-6 items: query lengths out of a shared budget (or all short), key lengths between the
    query length and 64x it, an offset that keeps every row inside the keys; shortest query first."""
    b = rng.randint(1, 6)
    small_q = rng.random() < 0.5
    ql, kl, off = [], [], []
    left = q_budget
    for i in range(b):
        cap = 24 if small_q else max(1, min(left - (b - 1 - i), q_budget // 2))
        q = rng.randint(1, cap)
        left -= q
        k = rng.randint(q, min(max_kv, q * 64))
        ql.append(q); kl.append(k); off.append(rng.randint(0, k - q))
    order = sorted(range(b), key=lambda i: ql[i])
    return [ql[i] for i in order], [kl[i] for i in order], [off[i] for i in order]


def _ragged_case(api, seed):
    rng = random.Random(seed)
    hq, hk = HEADS[seed % len(HEADS)]
    ql, kl, off = _shape(rng, 384, 3000)
    g = gen(seed)
    q = randn_bf16(g, sum(ql), hq, 128); k = randn_bf16(g, sum(kl), hk, 128); v = randn_bf16(g, sum(kl), hk, 128)
    want_ms = rng.random() < 0.4
    plan = api.fmha_sail_plan(_i32(ql), _i32(kl), hq, num_kv_heads=hk, qo_offset=_i32(off),
                              split_prefill_decode=rng.random() < 0.5, output_maxscore=want_ms,
                              num_kv_splits=rng.choice([-1, -1, 1, 3]))
    out, ms = api.fmha_sail(q.to(DEV), k.to(DEV), v.to(DEV), plan, check_input_valid=True)
    check_out(out, orc.attention(q, k, v, ql, kl, hq, hk, qo_offset=off), f"ragged seed {seed}")
    if want_ms:
        check_score(ms, orc.tile_max_score(q, k, ql, kl, hk, ms.shape[1], qo_offset=off), f"ragged ms seed {seed}")
        _, ms2 = api.fmha_sail(q.to(DEV), k.to(DEV), v.to(DEV), plan, output_o=False)     # score-only mode
        check_score(ms2, orc.tile_max_score(q, k, ql, kl, hk, ms2.shape[1], qo_offset=off), f"ragged score-only seed {seed}")


def _paged_case(api, seed):
    rng = random.Random(1000 + seed)
    hq, hk = HEADS[seed % len(HEADS)]
    ql, kl, off = _shape(rng, 384, 3000)
    page = rng.choice([128, 128, 128, 64, 16])
    nhd = rng.random() < 0.3
    fp8 = page == 128 and rng.random() < 0.2
    g = gen(1000 + seed)
    q = randn_bf16(g, sum(ql), hq, 128)
    kp, vp, table = make_paged(g, kl, hk, page, nhd=nhd)
    if fp8:
        k8, kf = orc.quantize_e4m3(kp); v8, vf = orc.quantize_e4m3(vp)
        kd, vd, kp, vp = k8.to(DEV), v8.to(DEV), kf, vf
    else:
        kd, vd = kp.to(DEV), vp.to(DEV)
    plan = api.fmha_sail_plan(_i32(ql), _i32(kl), hq, num_kv_heads=hk, qo_offset=_i32(off), page_size=page,
                              split_prefill_decode=rng.random() < 0.5, use_fp8_kvcache=fp8,
                              num_kv_splits=rng.choice([-1, -1, 1, 4]))
    out, _ = api.fmha_sail(q.to(DEV), kd, vd, plan, kv_indices=table.to(DEV), check_input_valid=True)
    k = orc.paged_to_contiguous(kp, table, kl, page, nhd=nhd)
    v = orc.paged_to_contiguous(vp, table, kl, page, nhd=nhd)
    ref = orc.attention(q, k, v, ql, kl, hq, hk, qo_offset=off)
    check_out(out, ref, f"paged seed {seed} page {page} nhd {nhd} fp8 {fp8}",
              cos_min=FP8_COS if fp8 else BF16_COS, max_abs=0.1 if fp8 else BF16_MAX_ABS)


def _sparse_case(api, seed):
    rng = random.Random(2000 + seed)
    hq, hk = HEADS[seed % len(HEADS)]
    kbn = [4, 8, 16, 32][(seed // len(HEADS)) % 4]
    ql, kl, off = _shape(rng, 256, 6000)
    g = gen(2000 + seed)
    q = randn_bf16(g, sum(ql), hq, 128)
    kp, vp, table = make_paged(g, kl, hk, 128)
    bi = random_blocks(g, ql, kl, off, hk, kbn)
    plan = api.fmha_sail_plan(_i32(ql), _i32(kl), hq, num_kv_heads=hk, qo_offset=_i32(off), page_size=128,
                              kv_block_num=kbn, num_kv_splits=rng.choice([-1, 1, 2, 4]))
    from msa_for_sail import api as api_mod
    force = rng.random() < 0.5                       # both sparse paths: page-major and per-token
    old = api_mod._FORCE_SPARSE_TC
    api_mod._FORCE_SPARSE_TC = force
    try:
        out, _ = api.fmha_sail(q.to(DEV), kp.to(DEV), vp.to(DEV), plan, kv_indices=table.to(DEV),
                               kv_block_indexes=bi.to(DEV), check_input_valid=True)
    finally:
        api_mod._FORCE_SPARSE_TC = old
    ref = orc.sparse_attention(q, kp, vp, ql, kl, table, bi, hq, qo_offset=off)
    check_out(out, ref, f"sparse seed {seed} kbn {kbn} page-major {force}")


@pytest.mark.parametrize("family", ["ragged", "paged", "sparse"])
def test_chaos(family):
    import msa_for_sail as api
    run = {"ragged": _ragged_case, "paged": _paged_case, "sparse": _sparse_case}[family]
    for seed in range(SEEDS_PER_FAMILY):
        run(api, seed)
    torch.cuda.synchronize()
    assert api.api.last_status() == 0
