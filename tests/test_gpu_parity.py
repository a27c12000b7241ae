"""GPU parity tests: the CUDA path (through the C ABI, via the drop-in Python API) against the
CPU oracle on identical seeded inputs, and against the committed upstream golden fixtures.

Tolerances: top-k indices bit-exact; bf16 outputs max-abs <= 2e-2 and cosine >= 0.9999;
e4m3 operands cosine >= 0.999; max_score within 1e-2 relative.
"""
import math
import os

import numpy as np
import pytest
import torch

from conftest import from_bf16_bits, load_golden
from helpers import (FP8_COS, check_out, check_score, gen, make_paged, randn_bf16, random_blocks)
from oracle import msa_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _api():
    import msa_for_sail
    return msa_for_sail


def _i32(x):
    return torch.tensor(x, dtype=torch.int32)


@pytest.fixture(params=["tcgen05", "mma"])
def kernel_path(request):
    """Run a dense test twice: with the tcgen05 prefill kernel wherever the shape is eligible
    (forced even when the planner would rather split KV), and on the generic mma.sync kernel."""
    from msa_for_sail import api
    old = (api._USE_TC, api._FORCE_TC)
    api._USE_TC = api._FORCE_TC = api._USE_DECODE_TC = request.param == "tcgen05"
    yield request.param
    api._USE_TC, api._FORCE_TC = old
    api._USE_DECODE_TC = True


@pytest.fixture(params=["page-major", "token-major"])
def sparse_path(request):
    """Sparse tests run on the page-major tcgen05 path (forced even for tiny inputs) and on the
    token-major mma.sync path."""
    from msa_for_sail import api
    old = (api._USE_SPARSE_TC, api._FORCE_SPARSE_TC)
    api._USE_SPARSE_TC = api._FORCE_SPARSE_TC = request.param == "page-major"
    api._USE_DECODE_TC = request.param == "page-major"      # token-major run also covers the mma.sync decode kernel
    yield request.param
    api._USE_SPARSE_TC, api._FORCE_SPARSE_TC = old
    api._USE_DECODE_TC = True


@pytest.fixture(autouse=True)
def _no_kernel_timeouts():
    yield
    from msa_for_sail import api
    torch.cuda.synchronize()
    assert api.last_status() == 0, "a kernel reported a bounded-wait timeout"


# ---------------------------------------------------------------------------
# top-k
# ---------------------------------------------------------------------------

def test_topk_golden_distributions_bitexact():
    api = _api()
    z = load_golden("topk_dist.npz")
    for kind in sorted(k[:-3] for k in z.files if k.endswith("_in")):
        m = from_bf16_bits(z[kind + "_in"])
        for dt in (torch.bfloat16, torch.float32):
            got = api.sparse_topk_select(m.to(dt).to(DEV), 16, num_valid_pages=m.shape[1])
            assert np.array_equal(got.cpu().numpy(), z[kind + "_out"]), (kind, dt)


@pytest.mark.parametrize("H,K,T,nvp,topk,fb,fe,dt", [
    (4, 256, 8, 200, 16, 3, 2, torch.float32),
    (4, 256, 8, 200, 16, 8, 8, torch.bfloat16),
    (4, 512, 4, 400, 16, 4, 3, torch.float32),
    (2, 2048, 16, 2000, 16, 2, 3, torch.float32),
    (1, 256, 4096, 256, 16, 0, 0, torch.float32),
    (1, 1024, 32, 1024, 16, 0, 0, torch.float32),
    (8, 128, 33, 77, 8, 0, 0, torch.float32),
    (2, 128, 65, 128, 4, 1, 1, torch.bfloat16),
    (2, 384, 40, 300, 32, 2, 2, torch.float32),
    (3, 128, 5, 9, 16, 0, 0, torch.float32),       # nvp <= topk: identity + -1 padding
    (3, 128, 5, 16, 16, 0, 0, torch.bfloat16),
    (2, 128, 7, 17, 16, 0, 0, torch.float32),
    # more than 2048 rows: the thread-per-row kernel (fewer rows take the CTA-per-row kernel)
    (4, 256, 1024, 200, 16, 3, 2, torch.float32),
    (2, 2048, 1100, 2000, 16, 2, 3, torch.float32),
    (2, 384, 1200, 300, 32, 2, 2, torch.float32),
    (8, 128, 300, 77, 8, 0, 0, torch.float32),
    (2, 128, 1500, 128, 4, 1, 1, torch.bfloat16),
    # CTA-per-row kernel with more than 2048 pages (32 keys per thread)
    (1, 4096, 8, 4000, 16, 1, 1, torch.float32),
    (1, 8192, 4, 8192, 32, 0, 0, torch.bfloat16),
    (2, 2304, 3, 2100, 8, 0, 2, torch.float32),
])
def test_topk_matches_oracle(H, K, T, nvp, topk, fb, fe, dt):
    api = _api()
    g = gen(H * 1000 + K + T)
    m = torch.randn(H, K, T, generator=g)
    m[:, nvp:, :] = -float("inf")
    m[:, :fb, :] = -1e10
    if fe:
        m[:, nvp - fe:nvp, :] = -1e10
    # quantise scores so that ties are common
    m = torch.where(torch.isinf(m), m, (m * 4).round() / 4).to(dt)
    ref = orc.topk_select(m.float(), topk, nvp, fb, fe)
    got = api.sparse_topk_select(m.to(DEV), topk, num_valid_pages=nvp, force_begin_blocks=fb,
                                 force_end_blocks=fe)
    assert got.dtype == torch.int32 and tuple(got.shape) == (T, H, topk)
    assert torch.equal(got.cpu(), ref)
    out = torch.empty_like(got)
    got2 = api.sparse_topk_select(m.to(DEV), topk, num_valid_pages=nvp, output=out,
                                  force_begin_blocks=fb, force_end_blocks=fe)
    assert got2.data_ptr() == out.data_ptr() and torch.equal(out, got)


@pytest.mark.parametrize("H,K,T,nvp,topk,fb,fe,dt", [
    (1, 256, 40000, 256, 16, 0, 0, torch.float32),     # the sparse-prefill shape: 256 pages, top-16
    (1, 256, 37900, 200, 16, 2, 3, torch.float32),     # just enough token blocks, forced pages
    (2, 384, 19000, 300, 16, 0, 0, torch.bfloat16),    # more pages than the bound pass looks at, bf16 scores
    (4, 768, 9500, 700, 32, 1, 2, torch.float32),      # top-32 (no group-maxima bound)
    (2, 128, 19012, 128, 8, 0, 1, torch.float32),      # top-8, a ragged last token block
    (2, 128, 19012, 100, 4, 1, 0, torch.bfloat16),     # top-4
    (1, 1280, 38000, 1100, 16, 0, 0, torch.bfloat16),  # long rows
])
def test_topk_large_inputs_match_oracle(H, K, T, nvp, topk, fb, fe, dt):
    """Prefill-sized inputs (tens of thousands of tokens; fp32 scores on two-register keys, bf16 scores without
    forced pages on one-word keys): quantised scores (ties everywhere), a causal -inf tail per token, signed
    zeros and NaNs sprinkled in."""
    api = _api()
    g = gen(7 * H + K + T)
    m = torch.randn(H, K, T, generator=g)
    m = (m * 4).round() / 4                                            # many exact ties, +0.0 and -0.0 both occur
    # causal shape: token t sees pages <= t * nvp / T (at least one); the rest is -inf
    vis = (torch.arange(T) * nvp // T + 1).view(1, 1, T)
    m = torch.where(torch.arange(K).view(1, K, 1) < vis, m, torch.tensor(-float("inf")))
    m[:, nvp:, :] = -float("inf")
    nan_at = torch.rand(H, K, T, generator=g) < 0.001
    m = torch.where(nan_at & ~torch.isinf(m), torch.tensor(float("nan")), m).to(dt)
    ref = orc.topk_select(m.float(), topk, nvp, fb, fe)
    got = api.sparse_topk_select(m.to(DEV), topk, num_valid_pages=nvp, force_begin_blocks=fb, force_end_blocks=fe)
    assert torch.equal(got.cpu(), ref)


def test_topk_large_inputs_golden_distributions_bitexact():
    """The upstream tie distributions (and the signed-zero / NaN ones), repeated along the token axis
    to a prefill-sized input."""
    api = _api()
    z = load_golden("topk_dist.npz")
    for kind in sorted(k[:-3] for k in z.files if k.endswith("_in")):
        m = from_bf16_bits(z[kind + "_in"])                            # [4, 512, 8]
        rep = 1200
        big = m.repeat(1, 1, rep)                                      # token t of the copy = token t % 8
        want = torch.from_numpy(z[kind + "_out"]).repeat(rep, 1, 1)
        for dt in (torch.bfloat16, torch.float32):
            got = api.sparse_topk_select(big.to(dt).to(DEV), 16, num_valid_pages=m.shape[1])
            assert torch.equal(got.cpu(), want), (kind, dt)


def test_topk_causal_minus_inf_rows():
    """Rows with fewer than k finite scores take -inf pages in ascending index order, never -1."""
    api = _api()
    H, K, T = 1, 128, 64
    m = torch.full((H, K, T), -float("inf"))
    g = gen(5)
    for t in range(T):
        m[0, :t // 2 + 1, t] = torch.randn(t // 2 + 1, generator=g)
    got = api.sparse_topk_select(m.to(DEV), 16, num_valid_pages=40).cpu()
    assert torch.equal(got, orc.topk_select(m, 16, 40))
    assert (got >= 0).all()


# ---------------------------------------------------------------------------
# split merge
# ---------------------------------------------------------------------------

def test_lse_merge_matches_oracle():
    import ctypes
    from msa_for_sail import _lib
    g = gen(11)
    S, T, H = 5, 37, 6
    po = torch.randn(S, T, H, 128, generator=g)
    pl = torch.randn(S, T, H, generator=g) * 3
    pl[1, :, 2] = -float("inf"); po[1, :, 2] = float("nan")
    pl[:, 3, 1] = -float("inf")
    spr = torch.randint(1, S + 1, (T,), generator=g, dtype=torch.int32)
    ref_rows = []
    for t in range(T):
        s = int(spr[t])
        ref_rows.append(orc.lse_merge(po[:s, t:t + 1], pl[:s, t:t + 1], out_scale=0.5, return_lse=True))
    ref_o = torch.cat([r[0] for r in ref_rows]); ref_l = torch.cat([r[1] for r in ref_rows])
    out = torch.empty(T, H, 128, dtype=torch.bfloat16, device=DEV)
    lse = torch.empty(T, H, dtype=torch.float32, device=DEV)
    pod, pld, sprd = po.to(DEV), pl.to(DEV), spr.to(DEV)
    rc = _lib.lib.msa_lse_merge(pod.data_ptr(), _lib.MSA_DT_F32, pld.data_ptr(), sprd.data_ptr(), out.data_ptr(),
                                lse.data_ptr(), S, T, H, out.stride(0), out.stride(1), 0.5,
                                torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    check_out(out, ref_o, "merge")
    # bf16 partials (the sparse prefill path stores them that way)
    pob = po.to(torch.bfloat16)
    pob[1, :, 2] = 0          # a NaN bf16 partial behind a -inf LSE must still be ignored: keep NaN there
    pob[1, :, 2] = float("nan")
    ref_rows = [orc.lse_merge(pob[:int(spr[t]), t:t + 1].float(), pl[:int(spr[t]), t:t + 1], out_scale=0.5)
                for t in range(T)]
    pobd = pob.to(DEV)
    rc = _lib.lib.msa_lse_merge(pobd.data_ptr(), _lib.MSA_DT_BF16, pld.data_ptr(), sprd.data_ptr(), out.data_ptr(),
                                None, S, T, H, out.stride(0), out.stride(1), 0.5,
                                torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    check_out(out, torch.cat(ref_rows), "merge-bf16")
    l = lse.cpu()
    assert torch.equal(torch.isinf(l), torch.isinf(ref_l))
    fin = ~torch.isinf(ref_l)
    assert torch.allclose(l[fin], ref_l[fin], atol=1e-4, rtol=1e-4)


# ---------------------------------------------------------------------------
# dense attention
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("name", ["prefill", "chunked", "decode", "offset"])
def test_dense_golden(name, kernel_path):
    api = _api()
    z = load_golden(f"attn_{name}.npz")
    b, ql, kl, hq, hk, off = [int(x) for x in z["meta"]]
    q = from_bf16_bits(z["q"]).reshape(b * ql, hq, 128).to(DEV)
    k = from_bf16_bits(z["k"]).reshape(b * kl, hk, 128).to(DEV)
    v = from_bf16_bits(z["v"]).reshape(b * kl, hk, 128).to(DEV)
    plan = api.fmha_sail_plan(_i32([ql] * b), _i32([kl] * b), hq, num_kv_heads=hk, qo_offset=off)
    out, ms = api.fmha_sail(q, k, v, plan, check_input_valid=True)
    assert ms is None
    check_out(out, torch.from_numpy(z["o"]), name)


@pytest.mark.parametrize("qo_lens,kv_lens,hq,hk,splits", [
    ([200, 1, 77, 128], [200, 300, 500, 128], 8, 2, 1),
    ([513, 40], [700, 40], 4, 4, -1),
    ([1, 1, 1], [1000, 17, 129], 16, 2, 4),          # decode, packed GQA, fixed splits
    ([1, 1], [3000, 2500], 8, 1, -1),                # decode, adaptive splits
    ([3, 2, 4], [260, 128, 131], 8, 2, -1),          # short chunks, packed rows > 16
    ([0, 5, 3], [64, 0, 70], 4, 2, 1),               # empty q, empty kv
    ([300], [300], 2, 1, 3),                         # prefill with forced splits
    ([1000, 257, 640], [1000, 1300, 640], 8, 2, 1),  # multi-tile prefill, tails, chunked prefill
    ([2048], [2048], 2, 2, 1),
])
def test_dense_ragged_matches_oracle(qo_lens, kv_lens, hq, hk, splits, kernel_path):
    api = _api()
    g = gen(sum(qo_lens) + sum(kv_lens) + hq)
    q = randn_bf16(g, sum(qo_lens), hq, 128)
    k = randn_bf16(g, max(1, sum(kv_lens)), hk, 128)[:sum(kv_lens)]
    v = randn_bf16(g, max(1, sum(kv_lens)), hk, 128)[:sum(kv_lens)]
    ref, ref_lse = orc.attention(q, k, v, qo_lens, kv_lens, hq, hk, return_lse=True)
    plan = api.fmha_sail_plan(_i32(qo_lens), _i32(kv_lens), hq, num_kv_heads=hk, num_kv_splits=splits)
    lse = torch.full((sum(qo_lens), hq), 7.0, dtype=torch.float32, device=DEV)
    out, _ = api.fmha_sail(q.to(DEV), k.to(DEV), v.to(DEV), plan, check_input_valid=True, lse=lse)
    check_out(out, ref, "ragged")
    l = lse.cpu()
    assert torch.equal(torch.isinf(l), torch.isinf(ref_lse))
    fin = ~torch.isinf(ref_lse)
    assert torch.allclose(l[fin], ref_lse[fin], atol=2e-3, rtol=1e-3)


@pytest.mark.parametrize("page_size,nhd,qo_lens,kv_lens,hq,hk,splits", [
    (128, False, [256, 100], [256, 900], 8, 2, 1),
    (128, True, [130, 64], [400, 64], 4, 1, 1),
    (16, False, [90, 33], [100, 333], 4, 2, 1),
    (64, True, [1, 1, 1], [640, 100, 1], 8, 2, -1),
    (128, False, [1, 1, 1, 1], [2048, 1500, 128, 129], 16, 2, 4),
    (128, False, [700, 1500], [1211, 1500], 4, 2, 1),        # prefill over shuffled pages, tail page
    (128, True, [513], [2000], 4, 1, 1),
])
def test_dense_paged_matches_oracle(page_size, nhd, qo_lens, kv_lens, hq, hk, splits, kernel_path):
    api = _api()
    g = gen(page_size + sum(kv_lens))
    q = randn_bf16(g, sum(qo_lens), hq, 128)
    kp, vp, table = make_paged(g, kv_lens, hk, page_size, nhd=nhd)
    k = orc.paged_to_contiguous(kp, table, kv_lens, page_size, nhd)
    v = orc.paged_to_contiguous(vp, table, kv_lens, page_size, nhd)
    ref = orc.attention(q, k, v, qo_lens, kv_lens, hq, hk)
    plan = api.fmha_sail_plan(_i32(qo_lens), _i32(kv_lens), hq, num_kv_heads=hk, page_size=page_size,
                              num_kv_splits=splits)
    pre = torch.empty(sum(qo_lens), hq, 128, dtype=torch.bfloat16, device=DEV)
    out, _ = api.fmha_sail(q.to(DEV), kp.to(DEV), vp.to(DEV), plan, kv_indices=table.to(DEV), out=pre,
                           check_input_valid=True)
    assert out.data_ptr() == pre.data_ptr()
    check_out(out, ref, "paged")


def test_offset_override_and_noncausal(kernel_path):
    api = _api()
    g = gen(21)
    qo_lens, kv_lens, hq, hk = [50, 20], [300, 280], 4, 2
    q = randn_bf16(g, sum(qo_lens), hq, 128); k = randn_bf16(g, sum(kv_lens), hk, 128)
    v = randn_bf16(g, sum(kv_lens), hk, 128)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    plan = api.fmha_sail_plan(_i32(qo_lens), _i32(kv_lens), hq, num_kv_heads=hk)
    # tighter offsets at run time
    off = [100, 7]
    out, _ = api.fmha_sail(qd, kd, vd, plan, q_offset_override=_i32(off).to(DEV))
    check_out(out, orc.attention(q, k, v, qo_lens, kv_lens, hq, hk, qo_offset=off), "override-tensor")
    out, _ = api.fmha_sail(qd, kd, vd, plan, q_offset_override=5)
    check_out(out, orc.attention(q, k, v, qo_lens, kv_lens, hq, hk, qo_offset=5), "override-int")
    # non-causal plan sees everything; an override on it restores causality
    plan_nc = api.fmha_sail_plan(_i32(qo_lens), _i32(kv_lens), hq, num_kv_heads=hk, causal=False)
    out, _ = api.fmha_sail(qd, kd, vd, plan_nc)
    check_out(out, orc.attention(q, k, v, qo_lens, kv_lens, hq, hk, causal=False), "non-causal")
    out, _ = api.fmha_sail(qd, kd, vd, plan_nc, q_offset_override=_i32(off).to(DEV))
    check_out(out, orc.attention(q, k, v, qo_lens, kv_lens, hq, hk, qo_offset=off), "nc+override")


def test_mixed_prefill_decode_split(kernel_path):
    api = _api()
    g = gen(31)
    qo_lens, kv_lens, hq, hk = [1, 2, 300, 200], [500, 64, 300, 777], 8, 2
    q = randn_bf16(g, sum(qo_lens), hq, 128); k = randn_bf16(g, sum(kv_lens), hk, 128)
    v = randn_bf16(g, sum(kv_lens), hk, 128)
    plan = api.fmha_sail_plan(_i32(qo_lens), _i32(kv_lens), hq, num_kv_heads=hk,
                              split_prefill_decode=True, output_maxscore=True)
    assert plan[0] is True and plan[1] == 2
    out, ms = api.fmha_sail(q.to(DEV), k.to(DEV), v.to(DEV), plan)
    check_out(out, orc.attention(q, k, v, qo_lens, kv_lens, hq, hk), "mixed")
    ref_ms = orc.tile_max_score(q, k, qo_lens, kv_lens, hk, ms.shape[1])
    check_score(ms, ref_ms, "mixed-ms")


# ---------------------------------------------------------------------------
# max score (Full / OnlyScore)
# ---------------------------------------------------------------------------

def test_maxscore_golden():
    api = _api()
    z = load_golden("maxscore_ragged.npz")
    hq, hk, mkt = [int(x) for x in z["meta"]]
    q = from_bf16_bits(z["q"]).to(DEV); k = from_bf16_bits(z["k"]).to(DEV)
    qo_lens, kv_lens = _i32(z["qo_lens"].tolist()), _i32(z["kv_lens"].tolist())
    plan = api.fmha_sail_plan(qo_lens, kv_lens, hq, num_kv_heads=hk, output_maxscore=True)
    assert plan[3]["max_k_tiles"] == mkt
    out, ms = api.fmha_sail(q, k, k, plan, output_o=False)
    assert out is None and tuple(ms.shape) == (hq, mkt, q.shape[0])
    assert torch.isinf(ms[:, 4:]).all()
    check_score(ms[:, :4], torch.from_numpy(z["ms"]), "golden-ms")
    plan2 = api.fmha_sail_plan(qo_lens, kv_lens, hq, num_kv_heads=hk, output_maxscore=True,
                               qo_offset=_i32(z["off"].tolist()))
    _, ms2 = api.fmha_sail(q, k, k, plan2, output_o=False)
    check_score(ms2[:, :4], torch.from_numpy(z["ms_off"]), "golden-ms-off")


@pytest.mark.parametrize("paged,qo_lens,kv_lens,hq,hk,full,ms_dtype", [
    (False, [300, 20], [300, 500], 4, 2, True, torch.float32),
    (True, [257], [1000], 2, 1, False, torch.float32),
    (True, [1, 1, 1], [1000, 130, 128], 8, 1, False, torch.float32),     # proxy decode, packed
    (True, [1, 1], [700, 256], 4, 4, True, torch.float32),
    (False, [140], [600], 2, 2, False, torch.bfloat16),
])
def test_maxscore_matches_oracle(paged, qo_lens, kv_lens, hq, hk, full, ms_dtype, kernel_path):
    api = _api()
    g = gen(sum(kv_lens) + hq * 7)
    q = randn_bf16(g, sum(qo_lens), hq, 128)
    if paged:
        kp, vp, table = make_paged(g, kv_lens, hk, 128)
        k = orc.paged_to_contiguous(kp, table, kv_lens, 128)
        v = orc.paged_to_contiguous(vp, table, kv_lens, 128)
        kw = dict(kv_indices=table.to(DEV)); kd, vd = kp.to(DEV), vp.to(DEV); ps = 128
    else:
        k = randn_bf16(g, sum(kv_lens), hk, 128); v = randn_bf16(g, sum(kv_lens), hk, 128)
        kw = {}; kd, vd = k.to(DEV), v.to(DEV); ps = -1
    plan = api.fmha_sail_plan(_i32(qo_lens), _i32(kv_lens), hq, num_kv_heads=hk, page_size=ps,
                              output_maxscore=True)
    mkt = plan[3]["max_k_tiles"]
    assert mkt == math.ceil(math.ceil(max(kv_lens) / 128) / 128) * 128
    out, ms = api.fmha_sail(q.to(DEV), kd, vd, plan, output_o=full, max_score_dtype=ms_dtype, **kw)
    ref_ms = orc.tile_max_score(q, k, qo_lens, kv_lens, hk, mkt)
    check_score(ms, ref_ms, "ms", bf16=(ms_dtype == torch.bfloat16))
    if full:
        check_out(out, orc.attention(q, k, v, qo_lens, kv_lens, hq, hk), "full-o")
    else:
        assert out is None


# ---------------------------------------------------------------------------
# sparse attention
# ---------------------------------------------------------------------------

def test_sparse_golden(sparse_path):
    api = _api()
    z = load_golden("sparse_small.npz")
    hq, hk, kbn, page = [int(x) for x in z["meta"]]
    q = from_bf16_bits(z["q"]).to(DEV)
    kp = from_bf16_bits(z["k_pages"]).to(DEV); vp = from_bf16_bits(z["v_pages"]).to(DEV)
    qo_lens = z["qo_lens"].tolist(); kv_lens = z["kv_lens"].tolist()
    blocks = z["blocks"]
    bi = torch.cat([torch.from_numpy(blocks[b]).unsqueeze(0).expand(qo_lens[b], hk, kbn)
                    for b in range(len(qo_lens))], 0).contiguous().to(torch.int32)
    n_pages = sum(x // page for x in kv_lens)
    plan = api.fmha_sail_plan(_i32(qo_lens), _i32(kv_lens), hq, num_kv_heads=hk, page_size=page,
                              kv_block_num=kbn)
    out, ms = api.fmha_sail(q, kp, vp, plan, kv_indices=torch.arange(n_pages, dtype=torch.int32, device=DEV),
                            kv_block_indexes=bi.to(DEV), check_input_valid=True)
    assert ms is None
    check_out(out, from_bf16_bits(z["o"]).float(), "sparse-golden")


@pytest.mark.parametrize("qo_lens,kv_lens,hq,hk,kbn,splits,fp8", [
    ([5, 9], [700, 1300], 8, 2, 4, 1, False),
    ([1, 1, 1], [2048, 1000, 129], 16, 2, 8, 2, False),      # decode, split
    ([1, 1], [4096, 3000], 8, 1, 16, 4, False),              # decode, 4 splits
    ([17], [2500], 4, 4, 16, -1, False),                     # h_r = 1
    ([3, 1], [1500, 640], 64, 2, 8, -1, False),              # h_r = 32 -> 64-row tile
    ([4, 1], [900, 2048], 8, 2, 8, 2, True),                 # all-e4m3 operands
    ([300, 77], [1500, 700], 8, 2, 8, 1, False),             # many tokens per page, tail pages
    ([200], [1100], 16, 1, 16, 1, False),                    # h_r = 16: 8 tokens per chunk
    ([500], [3000], 2, 2, 4, 1, False),                      # h_r = 1: 128 tokens per chunk
    ([1, 1, 1], [3000, 129, 5000], 64, 8, 16, 4, True),      # e4m3 decode, 8 rows per item, -1 padded lists
    ([1, 1, 1], [3000, 129, 5000], 64, 8, 16, 4, False),     # same on a bf16 cache
    ([2, 1], [1000, 4100], 32, 2, 8, 1, True),               # e4m3, 16 rows per item, two tokens
    ([40, 3], [6000, 4500], 8, 2, 32, 1, False),             # 32 selected pages per token
    ([300, 77], [1500, 700], 8, 2, 8, 1, True),              # e4m3 prefill: many tokens per page, tail pages
    ([200], [1100], 16, 1, 16, 1, True),                     # e4m3, h_r = 16
    ([500], [3000], 2, 2, 4, 1, True),                       # e4m3, h_r = 1
    ([600, 5], [2600, 900], 64, 8, 16, 1, True),             # e4m3, h_r = 8, more chunks than Q buffers per item
])
def test_sparse_matches_oracle(qo_lens, kv_lens, hq, hk, kbn, splits, fp8, sparse_path):
    api = _api()
    g = gen(sum(kv_lens) + kbn)
    q = randn_bf16(g, sum(qo_lens), hq, 128)
    kp, vp, table = make_paged(g, kv_lens, hk, 128)
    offs = [kv_lens[i] - qo_lens[i] for i in range(len(qo_lens))]
    bi = random_blocks(g, qo_lens, kv_lens, offs, hk, kbn)
    if fp8:
        q8, qf = orc.quantize_e4m3(q); k8, kf = orc.quantize_e4m3(kp); v8, vf = orc.quantize_e4m3(vp)
        ref = orc.sparse_attention(qf, kf, vf, qo_lens, kv_lens, table, bi, hq)
        qd, kd, vd = q8.to(DEV), k8.to(DEV), v8.to(DEV)
    else:
        ref = orc.sparse_attention(q, kp, vp, qo_lens, kv_lens, table, bi, hq)
        qd, kd, vd = q.to(DEV), kp.to(DEV), vp.to(DEV)
    plan = api.fmha_sail_plan(_i32(qo_lens), _i32(kv_lens), hq, num_kv_heads=hk, page_size=128,
                              kv_block_num=kbn, num_kv_splits=splits, use_fp8_kvcache=fp8)
    out, _ = api.fmha_sail(qd, kd, vd, plan, kv_indices=table.to(DEV), kv_block_indexes=bi.to(DEV),
                           check_input_valid=True)
    assert out.dtype == torch.bfloat16
    if fp8:
        check_out(out, ref, "sparse-fp8", cos_min=FP8_COS, max_abs=0.1)
    else:
        check_out(out, ref, "sparse")


def test_fp8_kv_with_bf16_q_and_per_head_scales():
    """Decode over an e4m3 KV cache quantised with one fp32 scale per KV head; q stays bf16."""
    api = _api()
    g = gen(77)
    qo_lens, kv_lens, hq, hk = [1, 1, 1], [1024, 700, 2000], 16, 2
    q = randn_bf16(g, 3, hq, 128)
    kp, vp, table = make_paged(g, kv_lens, hk, 128, dtype=torch.float32)
    ks = kp.abs().amax(dim=(0, 2, 3)) / 448.0; vs = vp.abs().amax(dim=(0, 2, 3)) / 448.0
    k8, kf = orc.quantize_e4m3(kp, ks.view(1, hk, 1, 1)); v8, vf = orc.quantize_e4m3(vp, vs.view(1, hk, 1, 1))
    k = orc.paged_to_contiguous(kf, table, kv_lens, 128); v = orc.paged_to_contiguous(vf, table, kv_lens, 128)
    ref = orc.attention(q, k, v, qo_lens, kv_lens, hq, hk)
    for splits in (1, 4):
        plan = api.fmha_sail_plan(_i32(qo_lens), _i32(kv_lens), hq, num_kv_heads=hk, page_size=128,
                                  num_kv_splits=splits, use_fp8_kvcache=True)
        out, _ = api.fmha_sail(q.to(DEV), k8.to(DEV), v8.to(DEV), plan, kv_indices=table.to(DEV),
                               k_scale=ks.to(DEV), v_scale=vs.to(DEV))
        check_out(out, ref, f"fp8kv-s{splits}", cos_min=FP8_COS, max_abs=0.1)


@pytest.mark.parametrize("paged,qo_lens,kv_lens,hq,hk", [
    (False, [1000, 257, 640], [1000, 1300, 640], 8, 2),     # multi-tile, tails, chunked prefill
    (True, [700, 1500], [1211, 1500], 4, 2),                # shuffled pages, tail page
    (True, [2048], [2048], 2, 1),
    (False, [130, 1, 0], [400, 900, 5], 2, 1),              # a decode row and an empty item in the same call
])
def test_fp8_prefill_matches_oracle(paged, qo_lens, kv_lens, hq, hk, kernel_path):
    """e4m3 q, k and v with per-tensor scales through the prefill kernels: O, LSE and the per-tile scores."""
    api = _api()
    g = gen(len(qo_lens) * 1000 + sum(kv_lens) + hq)
    q_s, k_s, v_s = 0.02, 0.015, 0.01
    q8, qf = orc.quantize_e4m3(randn_bf16(g, sum(qo_lens), hq, 128), q_s)
    if paged:
        kp, vp, table = make_paged(g, kv_lens, hk, 128, dtype=torch.float32)
        k8, kpf = orc.quantize_e4m3(kp, k_s); v8, vpf = orc.quantize_e4m3(vp, v_s)
        kf = orc.paged_to_contiguous(kpf, table, kv_lens, 128); vf = orc.paged_to_contiguous(vpf, table, kv_lens, 128)
        kw = dict(kv_indices=table.to(DEV))
    else:
        k8, kf = orc.quantize_e4m3(randn_bf16(g, sum(kv_lens), hk, 128), k_s)
        v8, vf = orc.quantize_e4m3(randn_bf16(g, sum(kv_lens), hk, 128), v_s)
        kw = {}
    ref, ref_lse = orc.attention(qf, kf, vf, qo_lens, kv_lens, hq, hk, return_lse=True)
    plan = api.fmha_sail_plan(_i32(qo_lens), _i32(kv_lens), hq, num_kv_heads=hk, page_size=128 if paged else -1,
                              num_kv_splits=1, use_fp8_kvcache=True, output_maxscore=True)
    lse = torch.full((sum(qo_lens), hq), 7.0, dtype=torch.float32, device=DEV)
    out, ms = api.fmha_sail(q8.to(DEV), k8.to(DEV), v8.to(DEV), plan, q_scale=q_s, k_scale=k_s, v_scale=v_s,
                            lse=lse, check_input_valid=True, **kw)
    check_out(out, ref, "fp8-prefill", cos_min=FP8_COS, max_abs=0.1)
    l = lse.cpu()
    fin = ~torch.isinf(ref_lse)
    assert torch.equal(torch.isinf(l), ~fin)
    assert torch.allclose(l[fin], ref_lse[fin], atol=2e-3, rtol=1e-3)
    ref_ms = orc.tile_max_score(qf, kf, qo_lens, kv_lens, hk, ms.shape[1])
    # the kernel reports raw e4m3 x e4m3 dot products; the scales are the caller's to apply
    check_score(ms.float() * (q_s * k_s), ref_ms, "fp8-prefill-ms")


def test_fp8_onlyscore():
    api = _api()
    g = gen(78)
    qo_lens, kv_lens, hq, hk = [130, 1], [400, 900], 2, 1
    q8, qf = orc.quantize_e4m3(randn_bf16(g, sum(qo_lens), hq, 128))
    k8, kf = orc.quantize_e4m3(randn_bf16(g, sum(kv_lens), hk, 128))
    plan = api.fmha_sail_plan(_i32(qo_lens), _i32(kv_lens), hq, num_kv_heads=hk, output_maxscore=True)
    out, ms = api.fmha_sail(q8.to(DEV), k8.to(DEV), k8.to(DEV), plan, output_o=False)
    assert out is None
    check_score(ms, orc.tile_max_score(qf, kf, qo_lens, kv_lens, hk, ms.shape[1]), "fp8-ms")


@pytest.mark.parametrize("fp8", [False, True])
def test_proxy_decode_scores_paged(fp8, kernel_path):
    """Score-only pass of a decode batch over a paged 1-head proxy cache (bf16 and e4m3)."""
    api = _api()
    g = gen(79 + fp8)
    qo_lens, kv_lens, hq, hk = [1, 1, 2], [1500, 128, 700], 4, 1
    q = randn_bf16(g, sum(qo_lens), hq, 128)
    kp, _, table = make_paged(g, kv_lens, hk, 128)
    if fp8:
        q8, qf = orc.quantize_e4m3(q); k8, kf = orc.quantize_e4m3(kp)
        qd, kd = q8.to(DEV), k8.to(DEV)
    else:
        qf, kf, qd, kd = q, kp, q.to(DEV), kp.to(DEV)
    k = orc.paged_to_contiguous(kf, table, kv_lens, 128)
    plan = api.fmha_sail_plan(_i32(qo_lens), _i32(kv_lens), hq, num_kv_heads=hk, page_size=128,
                              output_maxscore=True, use_fp8_kvcache=fp8)
    out, ms = api.fmha_sail(qd, kd, kd, plan, kv_indices=table.to(DEV), output_o=False)
    assert out is None
    check_score(ms, orc.tile_max_score(qf, k, qo_lens, kv_lens, hk, ms.shape[1]), "proxy-decode-ms")


@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("hq,qo_lens", [(1, [1, 1, 1]), (2, [1, 1, 2]), (4, [1, 1, 1]), (1, [3, 4, 1]), (3, [1, 1, 1])])
def test_proxy_scores_few_rows(fp8, hq, qo_lens):
    """Score-only pass whose work items have at most four rows: the matrix-vector kernel
    (ragged last pages, two-token items whose rows see different key limits)."""
    api = _api()
    g = gen(91 + fp8 + hq)
    kv_lens, hk = [1500, 128, 700], 1
    q = randn_bf16(g, sum(qo_lens), hq, 128)
    kp, _, table = make_paged(g, kv_lens, hk, 128)
    if fp8:
        q8, qf = orc.quantize_e4m3(q); k8, kf = orc.quantize_e4m3(kp)
        qd, kd = q8.to(DEV), k8.to(DEV)
    else:
        qf, kf, qd, kd = q, kp, q.to(DEV), kp.to(DEV)
    k = orc.paged_to_contiguous(kf, table, kv_lens, 128)
    plan = api.fmha_sail_plan(_i32(qo_lens), _i32(kv_lens), hq, num_kv_heads=hk, page_size=128,
                              output_maxscore=True, use_fp8_kvcache=fp8)
    out, ms = api.fmha_sail(qd, kd, kd, plan, kv_indices=table.to(DEV), output_o=False)
    assert out is None
    check_score(ms, orc.tile_max_score(qf, k, qo_lens, kv_lens, hk, ms.shape[1]), "proxy-few-rows-ms")


def test_sparse_page_major_global_index_kernels():
    """The counting sort has two implementations: a shared-memory histogram per CTA (page tables of up
    to 12 288 logical pages) and one global atomic per selection (longer tables).  A 1.6 M-token
    sequence whose 12 400 logical pages map onto a small physical pool takes the second."""
    api = _api()
    from msa_for_sail import api as api_mod
    g = gen(4242)
    n_logical, n_pool = 12400, 48
    qo_lens, kv_lens, hq, hk, kbn = [300], [n_logical * 128 - 50], 8, 2, 8
    q = randn_bf16(g, sum(qo_lens), hq, 128)
    kp = randn_bf16(g, n_pool, hk, 128, 128); vp = randn_bf16(g, n_pool, hk, 128, 128)
    table = torch.randint(0, n_pool, (n_logical,), generator=g).to(torch.int32)
    offs = [kv_lens[0] - qo_lens[0]]
    bi = random_blocks(g, qo_lens, kv_lens, offs, hk, kbn)
    ref = orc.sparse_attention(q, kp, vp, qo_lens, kv_lens, table, bi, hq)
    plan = api.fmha_sail_plan(_i32(qo_lens), _i32(kv_lens), hq, num_kv_heads=hk, page_size=128, kv_block_num=kbn)
    old = api_mod._FORCE_SPARSE_TC
    api_mod._FORCE_SPARSE_TC = True
    try:
        out, _ = api.fmha_sail(q.to(DEV), kp.to(DEV), vp.to(DEV), plan, kv_indices=table.to(DEV),
                               kv_block_indexes=bi.to(DEV))
        torch.cuda.synchronize()
    finally:
        api_mod._FORCE_SPARSE_TC = old
    check_out(out, ref, "sparse-global-index")


# ---------------------------------------------------------------------------
# the whole MSA pipeline (proxy max-score -> top-k -> sparse attention)
# ---------------------------------------------------------------------------

def test_msa_pipeline_cpu_reference_config(sparse_path):
    """BASELINE config 1: B=1, q=kv=4096, 16 q heads / 2 kv heads, 32 pages (shuffled table),
    1-head proxy, top-8 pages per token, sparse attention.  Indices bit-exact, O in tolerance."""
    api = _api()
    g = gen(0)
    T, hq, hk, page, topk = 4096, 16, 2, 128, 8
    n_pages = T // page
    q = randn_bf16(g, T, hq, 128)
    kp = randn_bf16(g, n_pages, hk, page, 128); vp = randn_bf16(g, n_pages, hk, page, 128)
    table = torch.randperm(n_pages, generator=g).to(torch.int32)
    q_proxy = q[:, :1].contiguous()
    k_proxy_pages = kp[:, :1].contiguous()
    lens = _i32([T])
    # stage 1: proxy pass, max score only
    plan1 = api.fmha_sail_plan(lens, lens, 1, num_kv_heads=1, page_size=page, output_maxscore=True)
    _, ms = api.fmha_sail(q_proxy.to(DEV), k_proxy_pages.to(DEV), k_proxy_pages.to(DEV), plan1,
                          kv_indices=table.to(DEV), output_o=False)
    k_proxy = orc.paged_to_contiguous(k_proxy_pages, table, [T], page)
    ref_ms = orc.tile_max_score(q_proxy, k_proxy, [T], [T], 1, ms.shape[1])
    check_score(ms, ref_ms, "pipeline-ms")
    # stage 2: top-k on the GPU scores must equal the oracle's top-k on the same scores
    idx = api.sparse_topk_select(ms, topk, num_valid_pages=n_pages)
    assert torch.equal(idx.cpu(), orc.topk_select(ms.cpu(), topk, n_pages))
    # stage 3: sparse attention over the selected pages (1-head proxy -> broadcast to kv heads)
    bi = idx.expand(T, hk, topk).contiguous()
    plan2 = api.fmha_sail_plan(lens, lens, hq, num_kv_heads=hk, page_size=page, kv_block_num=topk)
    out, _ = api.fmha_sail(q.to(DEV), kp.to(DEV), vp.to(DEV), plan2, kv_indices=table.to(DEV),
                           kv_block_indexes=bi)
    sub = torch.arange(0, T, 37)       # the oracle walks tokens in Python: check a strided sample
    ref = orc.sparse_attention(q[sub], kp, vp, [1] * len(sub), [T] * len(sub),
                               table.repeat(len(sub)), bi.cpu()[sub], hq,
                               qo_offset=[int(t) for t in sub])
    check_out(out[sub.to(DEV)], ref, "pipeline-o")


# ---------------------------------------------------------------------------
# parameter line -> reproducer
# ---------------------------------------------------------------------------

@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["Off", "OnlyScore", "Sparse"])
def test_param_line_reruns_through_the_reproducer(mode, capsys):
    """The '[MSA] --format=' line printed for a call is enough to run the same shape again."""
    import importlib.util
    from msa_for_sail import api as api_mod
    api = _api()
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "msa-for-sail_b200", "benchmarks",
                        "run_msa.py")
    spec = importlib.util.spec_from_file_location("run_msa", path)
    run_msa = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(run_msa)
    g = gen(31)
    qo_lens, kv_lens, hq, hk, kbn = [1, 3], [700, 1300], 8, 2, 4
    q = randn_bf16(g, sum(qo_lens), hq, 128)
    kp, vp, table = make_paged(g, kv_lens, hk, 128)
    kw = dict(kv_indices=table.to(DEV))
    plan_kw = dict(num_kv_heads=hk, page_size=128)
    if mode == "Sparse":
        offs = [kv_lens[i] - qo_lens[i] for i in range(2)]
        kw["kv_block_indexes"] = random_blocks(g, qo_lens, kv_lens, offs, hk, kbn).to(DEV)
        plan_kw["kv_block_num"] = kbn
    elif mode == "OnlyScore":
        plan_kw["output_maxscore"] = True
        kw["output_o"] = False
    else:
        kw["output_maxscore"] = False
    plan = api.fmha_sail_plan(_i32(qo_lens), _i32(kv_lens), hq, **plan_kw)
    old = api_mod._SHOW_PARAMS
    api_mod._SHOW_PARAMS = True
    try:
        api.fmha_sail(q.to(DEV), kp.to(DEV), vp.to(DEV), plan, **kw)
    finally:
        api_mod._SHOW_PARAMS = old
    lines = [ln for ln in capsys.readouterr().out.splitlines() if ln.startswith("[MSA] --format=")]
    assert len(lines) == 1
    cfg = run_msa.parse_format(lines[0])
    assert cfg["seqlen_q"] == qo_lens and cfg["seqlen_k"] == kv_lens and cfg["sparse_mode"] == mode
    assert cfg["num_qo_heads"] == hq and cfg["num_kv_heads"] == hk
    run_msa.build_and_run(cfg)
    assert "RAN OK" in capsys.readouterr().out
