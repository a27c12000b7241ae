"""Child process of test_checked_build_gpu.py: runs with MSA_BOUNDS_CHECK=1, i.e. on libmsa_b200_check.so (the
sources of the shipped library compiled with -DMSA_BOUNDS_CHECK -DMSA_DEBUG_HOOKS).

1. Valid inputs through the checked kernels: results match the oracle, the status word stays 0.
2. A page table entry that is out of range by contract but inside the allocation (the pool tensor passed to the
   library is a view of the first N pages of a pool of N + 4; the entry names page N + 1): the kernel clamps it and
   the status word comes back as STATUS_BOUNDS.  Nothing can leave the buffers even if the check were wrong.
3. A bounded wait that runs out: a test hook makes the TMA producer of the dense prefill kernel stop before its
   second K tile (issuing nothing after it) and shortens the poll limit.  The MMA warp's wait for that tile gives
   up, every role returns, TMEM is released, the status word says STATUS_TIMEOUT; while it is set the next launch
   returns at once without touching its output; last_status() clears it and the kernel works again.
Prints one line per part; exits non-zero on the first failure.
"""
import ctypes
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "msa-for-sail_b200", "python"))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import msa_for_sail as msa                      # noqa: E402
from msa_for_sail import _lib, api             # noqa: E402
from oracle import msa_oracle as orc           # noqa: E402
from helpers import check_out, gen, make_paged, randn_bf16, random_blocks   # noqa: E402

DEV = "cuda"
assert _lib.BOUNDS_CHECK and _lib.LIB_PATH.endswith("libmsa_b200_check.so")


def i32(x):
    return torch.tensor(x, dtype=torch.int32)


def part_valid():
    g = gen(1)
    # dense paged prefill (tcgen05 kernel), paged decode with splits, sparse decode, sparse prefill (page-major)
    qo, kv, hq, hk = [300, 2], [700, 900], 8, 2
    q = randn_bf16(g, sum(qo), hq, 128)
    kp, vp, table = make_paged(g, kv, hk, 128)
    k = orc.paged_to_contiguous(kp, table, kv, 128); v = orc.paged_to_contiguous(vp, table, kv, 128)
    plan = msa.fmha_sail_plan(i32(qo), i32(kv), hq, num_kv_heads=hk, page_size=128)
    out, _ = msa.fmha_sail(q.to(DEV), kp.to(DEV), vp.to(DEV), plan, kv_indices=table.to(DEV))
    check_out(out, orc.attention(q, k, v, qo, kv, hq, hk), "checked dense")
    qd = randn_bf16(g, 2, hq, 128)
    plan = msa.fmha_sail_plan(i32([1, 1]), i32(kv), hq, num_kv_heads=hk, page_size=128, num_kv_splits=3)
    out, _ = msa.fmha_sail(qd.to(DEV), kp.to(DEV), vp.to(DEV), plan, kv_indices=table.to(DEV))
    check_out(out, orc.attention(qd, k, v, [1, 1], kv, hq, hk), "checked decode")
    offs = [kv[i] - qo[i] for i in range(2)]
    bi = random_blocks(g, qo, kv, offs, hk, 4)
    plan = msa.fmha_sail_plan(i32(qo), i32(kv), hq, num_kv_heads=hk, page_size=128, kv_block_num=4)
    for force in (False, True):
        api._FORCE_SPARSE_TC = force
        out, _ = msa.fmha_sail(q.to(DEV), kp.to(DEV), vp.to(DEV), plan, kv_indices=table.to(DEV), kv_block_indexes=bi.to(DEV))
        check_out(out, orc.sparse_attention(q, kp, vp, qo, kv, table, bi, hq), f"checked sparse page-major={force}")
    api._FORCE_SPARSE_TC = False
    ms_plan = msa.fmha_sail_plan(i32([1, 1]), i32(kv), 1, num_kv_heads=1, page_size=128, output_maxscore=True)
    msa.fmha_sail(qd[:, :1].contiguous().to(DEV), kp[:, :1].contiguous().to(DEV), kp[:, :1].contiguous().to(DEV), ms_plan,
                  kv_indices=table.to(DEV), output_o=False)
    torch.cuda.synchronize()
    assert api.last_status() == _lib.STATUS_OK, "valid inputs must leave the status word at 0"
    print("valid inputs: ok, status 0")


def part_bad_page():
    g = gen(2)
    n, extra, hq, hk = 6, 4, 4, 1
    pool_k = randn_bf16(g, n + extra, hk, 128, 128).to(DEV); pool_v = randn_bf16(g, n + extra, hk, 128, 128).to(DEV)
    q = randn_bf16(g, 1, hq, 128).to(DEV)
    table = torch.arange(n, dtype=torch.int32)
    table[3] = n + 1                               # >= the extent the library is told (n), < the real allocation (n + 4)
    for rows, splits in ((1, 1), (200, 1)):        # decode kernel / prefill kernel
        qq = randn_bf16(g, rows, hq, 128).to(DEV) if rows > 1 else q
        plan = msa.fmha_sail_plan(i32([rows]), i32([n * 128]), hq, num_kv_heads=hk, page_size=128, num_kv_splits=splits)
        out, _ = msa.fmha_sail(qq, pool_k[:n], pool_v[:n], plan, kv_indices=table.to(DEV))
        torch.cuda.synchronize()
        assert torch.isfinite(out.float()).all()
        st = api.last_status()
        assert st == _lib.STATUS_BOUNDS, f"expected STATUS_BOUNDS, got {st}"
        assert api.last_status() == 0                 # reading it cleared it
    print("out-of-range page id: clamped, STATUS_BOUNDS reported and cleared")


def part_timeout():
    g = gen(3)
    qo, kv, hq, hk = [512], [512], 2, 1                   # 4 key tiles per CTA on the tcgen05 prefill kernel
    q = randn_bf16(g, 512, hq, 128); k = randn_bf16(g, 512, hk, 128); v = randn_bf16(g, 512, hk, 128)
    plan = msa.fmha_sail_plan(i32(qo), i32(kv), hq, num_kv_heads=hk)
    assert plan[3]["tc_preferred"], "this shape is expected on the tcgen05 prefill kernel"
    ref = orc.attention(q, k, v, qo, kv, hq, hk)
    _lib.lib.msa_debug_tc_stall.argtypes = [ctypes.c_int, ctypes.c_uint]
    _lib.lib.msa_debug_tc_stall(1, 1 << 14)
    out = torch.full((512, hq, 128), 7.0, dtype=torch.bfloat16, device=DEV)
    msa.fmha_sail(q.to(DEV), k.to(DEV), v.to(DEV), plan, out=out)
    torch.cuda.synchronize()                               # returns: every wait in the kernel is bounded
    _lib.lib.msa_debug_tc_stall(-1, 0)
    st = api.last_status(reset=False)
    assert st == _lib.STATUS_TIMEOUT, f"expected STATUS_TIMEOUT, got {st}"
    out.fill_(7.0)
    msa.fmha_sail(q.to(DEV), k.to(DEV), v.to(DEV), plan, out=out)     # status still set: CTAs return after their prologue
    torch.cuda.synchronize()
    assert (out == 7.0).all(), "a launch while the status word is set must not run"
    assert api.last_status() == _lib.STATUS_TIMEOUT and api.last_status() == 0
    msa.fmha_sail(q.to(DEV), k.to(DEV), v.to(DEV), plan, out=out)
    torch.cuda.synchronize()
    check_out(out, ref, "after the timeout was cleared")
    assert api.last_status() == 0
    print("bounded wait ran out: STATUS_TIMEOUT, next launch skipped, cleared, kernel works again")


if __name__ == "__main__":
    part_valid()
    part_bad_page()
    part_timeout()
    print("CHECKED_BUILD_OK")
