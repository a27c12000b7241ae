"""CPU-side checks of the C ABI: the library loads, exports every symbol the header declares,
struct sizes agree with the binding, argument validation answers before any CUDA call, and the
native host planner covers every tile exactly once."""
import ctypes
import os
import re

import numpy as np
import pytest

from conftest import ROOT


def _lib():
    from msa_for_sail import _lib
    return _lib


def test_header_symbols_are_exported():
    L = _lib()
    hdr = open(os.path.join(ROOT, "include", "msa_b200.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    names = set(re.findall(r"\b(msa_[a-z0-9_]+)\s*\(", hdr))
    assert names, "no prototypes found"
    assert names == set(L.EXPORTS)
    for n in names:
        assert hasattr(L.lib, n), n
    assert L.lib.msa_build_arch() == 100


def test_struct_sizes_match():
    L = _lib()
    assert L.lib.msa_sizeof(0) == ctypes.sizeof(L.MsaFmhaParams)
    assert L.lib.msa_sizeof(1) == ctypes.sizeof(L.MsaWorkItem) == 32
    assert L.lib.msa_sizeof(2) == ctypes.sizeof(L.MsaPlanArgs)
    assert L.lib.msa_sizeof(3) == ctypes.sizeof(L.MsaPlanDeviceArgs)
    assert L.lib.msa_sizeof(99) == -1


def test_bad_arguments_are_rejected_without_touching_the_gpu():
    L = _lib()
    assert L.lib.msa_fmha_fwd(None, None) == -1
    p = L.MsaFmhaParams()
    assert L.lib.msa_fmha_fwd(ctypes.byref(p), None) == -1          # no output requested
    p.flags = L.FLAG_OUT_O
    assert L.lib.msa_fmha_fwd(ctypes.byref(p), None) == -1          # null tensors
    assert L.lib.msa_topk_select(None, 2, None, 1, 128, 1, 16, 1, 0, 0, None) == -1
    assert L.lib.msa_lse_merge(None, 2, None, None, None, None, 1, 1, 1, 0, 0, 1.0, None) == -1
    assert b"bad argument" in L.lib.msa_status_string(-1)
    with pytest.raises(RuntimeError):
        L.check(-2, "x")


def _plan(L, qo, kv, off, hq, hk, bm, pack, splits, sms=148):
    a_q, a_k, a_o = (np.asarray(x, np.int32) for x in (qo, kv, off))
    args = L.MsaPlanArgs(a_q.ctypes.data, a_k.ctypes.data, a_o.ctypes.data, len(qo), hq, hk, bm, pack,
                         splits, sms, 0)
    cap = 1 << 16
    work = np.empty((cap, 8), np.int32)
    spr = np.zeros(max(1, sum(qo)), np.int32)
    ms = ctypes.c_int32(0)
    n = L.lib.msa_plan_dense(ctypes.byref(args), work.ctypes.data, cap, spr.ctypes.data, ctypes.byref(ms))
    assert n >= 0
    return work[:n], spr, ms.value


@pytest.mark.parametrize("qo,kv,hq,hk,bm,pack,splits", [
    ([300, 1, 77], [300, 500, 900], 8, 2, 128, 1, 1),
    ([300, 1, 77], [300, 500, 900], 8, 2, 128, 1, 4),
    ([1, 1, 1, 1], [4096, 100, 5000, 128], 16, 2, 16, 8, -128),
    ([3, 2], [200, 300], 12, 2, 16, 6, 2),            # pack 6: 12 rows per item
    ([0, 4], [10, 0], 4, 4, 64, 1, -128),
    ([8192] * 2, [8192] * 2, 4, 1, 128, 1, -128),
])
def test_host_planner_covers_every_tile_once(qo, kv, hq, hk, bm, pack, splits):
    L = _lib()
    off = [k - q for q, k in zip(qo, kv)]
    work, spr, max_splits = _plan(L, qo, kv, off, hq, hk, bm, pack, splits)
    bm_eff = (bm // pack) * pack
    seen = {}
    for b, h0, r0, tb, te, sp, nr, _ in work.tolist():
        assert tb <= te and 0 < nr <= bm_eff and h0 % pack == 0
        seen.setdefault((b, h0, r0), []).append((tb, te, sp))
    tok0 = 0
    for b in range(len(qo)):
        rows = qo[b] * pack
        for r0 in range(0, rows, bm_eff):
            nrows = min(bm_eff, rows - r0)
            i_max = (r0 + nrows - 1) // pack
            want = max(0, -(-min(kv[b], i_max + off[b] + 1) // 128))
            for g in range(hq // pack):
                parts = sorted(seen.pop((b, g * pack, r0)))
                assert parts[0][0] == 0 and parts[-1][1] == want
                for x, y in zip(parts, parts[1:]):
                    assert x[1] == y[0]
                assert [p[2] for p in sorted(parts, key=lambda p: p[2])] == list(range(len(parts)))
                assert len(parts) <= max_splits
                for i in range(r0 // pack, i_max + 1):
                    assert spr[tok0 + i] == len(parts)
                if splits >= 1:
                    assert len(parts) <= splits
        tok0 += qo[b]
    assert not seen, "planner emitted items outside the problem"
    # longest first
    lens = [te - tb for _, _, _, tb, te, _, _, _ in work.tolist()]
    assert lens == sorted(lens, reverse=True)


def test_planner_reports_capacity():
    L = _lib()
    a = np.asarray([1000], np.int32)
    args = L.MsaPlanArgs(a.ctypes.data, a.ctypes.data, a.ctypes.data, 1, 8, 8, 128, 1, 1, 148, 0)
    work = np.empty((2, 8), np.int32)
    assert L.lib.msa_plan_dense(ctypes.byref(args), work.ctypes.data, 2, None, None) == -4


def test_api_surface_matches_upstream_names():
    import inspect
    import msa_for_sail as m
    for name in ("fmha_sail_plan", "fmha_sail", "sparse_topk_select", "allocate_graph_workspace"):
        assert callable(getattr(m, name))
    sig = inspect.signature(m.fmha_sail)
    assert list(sig.parameters)[:9] == ["q", "k", "v", "plan_info", "kv_indices", "kv_block_indexes",
                                        "q_offset_override", "out", "max_score"]
    sig = inspect.signature(m.sparse_topk_select)
    assert list(sig.parameters) == ["max_score", "topk", "num_valid_pages", "output",
                                    "force_begin_blocks", "force_end_blocks"]
    sig = inspect.signature(m.allocate_graph_workspace)
    assert list(sig.parameters) == ["batch_size", "num_qo_heads", "num_kv_heads", "max_qo_len", "page_size",
                                    "kv_block_num", "num_kv_splits", "device", "output_maxscore",
                                    "use_fp8_kvcache"]


def _valid_params(L):
    """A well-formed ragged dense call whose pointers are fake but aligned: every check below
    fails on the argument it breaks, before anything would touch the device."""
    p = L.MsaFmhaParams()
    fake = 0x1000
    for f in ("q", "k", "v", "out", "qo_start", "kv_start", "kv_len", "qo_offset", "work"):
        setattr(p, f, fake)
    p.q_stride_tok, p.q_stride_head = 8 * 128, 128
    p.k_stride_tok = p.v_stride_tok = 2 * 128
    p.k_stride_head = p.v_stride_head = 128
    p.out_stride_tok, p.out_stride_head = 8 * 128, 128
    p.total_q, p.num_qo_heads, p.num_kv_heads, p.batch = 4, 8, 2, 1
    p.num_work, p.block_m, p.pack, p.page_size, p.num_splits = 1, 16, 4, 0, 1
    p.q_dtype = p.kv_dtype = L.MSA_DT_BF16
    p.flags = L.FLAG_OUT_O
    p.sm_scale, p.out_scale = 0.1, 1.0
    return p


BROKEN = [
    ("kv_len", None, -1), ("q", None, -1), ("qo_offset", None, -1), ("v", None, -1),
    ("pack", 0, -1), ("pack", 3, -1), ("num_kv_heads", 0, -1), ("num_kv_heads", 3, -1),
    ("block_m", 48, -1), ("out_stride_tok", 8 * 128 + 4, -1), ("q", 0x1008, -1),
    ("kv_start", None, -1), ("q_dtype", 7, -2), ("kv_dtype", 2, -2), ("flags", 0, -1),
]


@pytest.mark.parametrize("field,value,code", BROKEN)
def test_fmha_entry_points_reject_bad_arguments_on_the_host(field, value, code):
    """msa_fmha_fwd and msa_fmha_fwd_split_static share one argument check; both must answer
    with an error code (never launch) for each broken argument."""
    L = _lib()
    for static in (False, True):
        p = _valid_params(L)
        if static:
            p.num_splits = 2
        setattr(p, field, value)
        if static:
            rc = L.lib.msa_fmha_fwd_split_static(ctypes.byref(p), None, None)
        else:
            rc = L.lib.msa_fmha_fwd(ctypes.byref(p), None)
        assert rc == code, (field, value, static, rc)


def test_sparse_and_paged_argument_rules():
    L = _lib()
    for static in (False, True):
        call = (lambda p: L.lib.msa_fmha_fwd_split_static(ctypes.byref(p), None, None)) if static else \
               (lambda p: L.lib.msa_fmha_fwd(ctypes.byref(p), None))
        p = _valid_params(L)                      # paged without a page table
        p.page_size = 128
        assert call(p) == -1
        p = _valid_params(L)                      # sparse on pages that are not 128 keys
        p.flags = L.FLAG_OUT_O | L.FLAG_SPARSE
        p.page_size, p.kv_page_indptr, p.kv_indices = 64, 0x1000, 0x1000
        p.kv_block_indexes, p.token_batch, p.kv_block_num = 0x1000, 0x1000, 4
        assert call(p) == -2
        p.page_size, p.token_batch = 128, None     # sparse without the token -> batch map
        assert call(p) == -1
        p.token_batch, p.pack = 0x1000, 2          # sparse must fold the whole head group
        assert call(p) == -1
    p = _valid_params(L)                          # the static entry owns its scratch and has a size limit
    p.num_splits, p.partial_o = 2, 0x1000
    assert L.lib.msa_fmha_fwd_split_static(ctypes.byref(p), None, None) == -1
    p = _valid_params(L)
    p.num_splits, p.total_q, p.num_qo_heads, p.num_kv_heads, p.pack = 8, 64, 64, 64, 1
    assert L.lib.msa_fmha_fwd_split_static(ctypes.byref(p), None, None) == -4


def test_shipped_library_exports_no_debug_hooks():
    """Tracing / test hooks exist only in builds with -DMSA_DEBUG_HOOKS."""
    import subprocess
    L = _lib()
    out = subprocess.run(["nm", "-D", "--defined-only", L.LIB_PATH], capture_output=True, text=True).stdout
    names = {ln.split()[-1] for ln in out.splitlines() if ln.strip()}
    assert not [n for n in names if n.startswith("msa_debug")], names
    assert set(L.EXPORTS) <= names
