"""The production entry points: `minfer.ops.fmha_sail_plan` -> `minfer.ops.fmha_sail` ->
`minfer.ops.sparse_topk_select` called through `tvm_ffi.get_global_func` with CUDA tensors (bf16 and
e4m3), checked against the CPU oracle.  The plan travels through tvm_ffi both ways (tuple -> Array,
dict -> Map, tensors by DLPack) exactly as a tvm_ffi caller sees it."""
import pytest
import torch

from helpers import FP8_COS, check_out, check_score, gen, randn_bf16
from oracle import msa_oracle as orc

tvm_ffi = pytest.importorskip("tvm_ffi")
pytestmark = pytest.mark.gpu
DEV = "cuda"


def _i32(x):
    return torch.tensor(x, dtype=torch.int32)


@pytest.mark.parametrize("fp8", [False, True])
def test_plan_run_topk_through_tvm_ffi(fp8):
    import msa_for_sail  # noqa: F401  (registers the global functions)
    plan_f = tvm_ffi.get_global_func("minfer.ops.fmha_sail_plan")
    run_f = tvm_ffi.get_global_func("minfer.ops.fmha_sail")
    topk_f = tvm_ffi.get_global_func("minfer.ops.sparse_topk_select")
    g = gen(31 + fp8)
    qo_lens, kv_lens, hq, hk = [200, 3], [700, 450], 8, 2
    q = randn_bf16(g, sum(qo_lens), hq, 128); k = randn_bf16(g, sum(kv_lens), hk, 128); v = randn_bf16(g, sum(kv_lens), hk, 128)
    if fp8:
        q8, qf = orc.quantize_e4m3(q); k8, kf = orc.quantize_e4m3(k); v8, vf = orc.quantize_e4m3(v)
        dq, dk, dv, q, k, v = q8.to(DEV), k8.to(DEV), v8.to(DEV), qf, kf, vf
    else:
        dq, dk, dv = q.to(DEV), k.to(DEV), v.to(DEV)
    # positional arguments only, as a tvm_ffi caller passes them: lengths, query heads, KV heads
    plan = plan_f(tvm_ffi.from_dlpack(_i32(qo_lens)), tvm_ffi.from_dlpack(_i32(kv_lens)), hq, hk)
    assert len(plan) == 5 and not plan[0]
    res = run_f(tvm_ffi.from_dlpack(dq), tvm_ffi.from_dlpack(dk), tvm_ffi.from_dlpack(dv), plan)
    out = torch.from_dlpack(res[0])
    assert out.is_cuda and out.dtype == torch.bfloat16 and res[1] is None
    ref = orc.attention(q, k, v, qo_lens, kv_lens, hq, hk)
    check_out(out, ref, "ffi dense", cos_min=FP8_COS if fp8 else 0.9999, max_abs=0.1 if fp8 else 2e-2)

    # page scores of the same batch through the Python API (a plan with keyword options), top-k through tvm_ffi
    plan_s = msa_for_sail.fmha_sail_plan(_i32(qo_lens), _i32(kv_lens), hq, num_kv_heads=hk, output_maxscore=True)
    _, ms = msa_for_sail.fmha_sail(dq, dk, dk, plan_s, output_o=False)
    check_score(ms, orc.tile_max_score(q, k, qo_lens, kv_lens, hk, ms.shape[1]), "ffi scores")
    nvp = 6
    sel = torch.from_dlpack(topk_f(tvm_ffi.from_dlpack(ms), 4, nvp))
    assert torch.equal(sel.cpu(), orc.topk_select(ms.cpu(), 4, nvp))
