"""FMHA varlen attention API for B200: plan + run, page top-k selection.

Same public surface as the upstream ``msa_for_sail.api`` (``fmha_sail_plan``
api.py:1480-1579, ``fmha_sail`` 1581-1728, ``sparse_topk_select`` 1736-1848,
``allocate_graph_workspace`` 383-447): same names, argument meaning, return
shapes and error behaviour.  Underneath, the upstream per-variant JIT is
replaced by one prebuilt C-ABI library of sm_100a kernels (see ``_lib``).
"""

import ctypes
import math
import os
from typing import Optional, Tuple, Union

import numpy as np
import torch

from . import _lib
from ._lib import FLAG_OUT_O, FLAG_OUT_SCORE, FLAG_SPARSE, MSA_DT_BF16, MSA_DT_E4M3, MSA_DT_F32

__all__ = [
    "fmha_sail_plan", "fmha_sail", "sparse_topk_select",
    "_fmha_sail_plan", "_fmha_sail",
    "allocate_graph_workspace",
]

KV_TILE = 128
_USE_TC = True                          # route eligible prefill shapes to the tcgen05 kernel
_FORCE_TC = False                       # ... even when the planner would rather split KV
_USE_DECODE_TC = True                   # tcgen05 decode kernel for short-query bf16 shapes
_USE_SPARSE_TC = True                   # page-major (KV-outer) tcgen05 path for sparse prefill
_FORCE_SPARSE_TC = False                # ... even when few tokens share a page
_STATUS = {}


def _status_word(device):
    """Per-device int32 status word the kernels report bounded-wait timeouts into."""
    idx = torch.device(device).index or 0
    if idx not in _STATUS:
        _STATUS[idx] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
    return _STATUS[idx]


def last_status(device=None, reset=True):
    """Read (synchronously) the device status word: 0 = ok, 1 = a kernel wait timed out, 2 = (bounds-checked
    build) a kernel found an out-of-range index in one of the caller's tables and clamped it."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    w = _status_word(device)
    v = int(w.item())
    if reset and v:
        w.zero_()
    return v
_SHOW_PARAMS = os.environ.get("MSA_SHOW_PARAMS", os.environ.get("PPU_LIB_SHOW_PARAMS", "0")) not in ("", "0")
_PACK_FACTORS = (2, 4, 6, 8, 16)       # upstream jit.py _PACK_FACTORS
_NUM_SMS = {}


def _num_sms(device):
    idx = torch.device("cuda", device if isinstance(device, int) else torch.device(device).index or 0).index
    if idx not in _NUM_SMS:
        _NUM_SMS[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _NUM_SMS[idx]


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _dt_code(dtype):
    if dtype == torch.bfloat16:
        return MSA_DT_BF16
    if dtype == torch.float8_e4m3fn:
        return MSA_DT_E4M3
    if dtype == torch.float32:
        return MSA_DT_F32
    raise ValueError(f"unsupported dtype {dtype}")


def _prefill_qlen_threshold(sparse):
    return 32 if sparse else 128


def _detect_paged_kv_layout(shape, page_size_hint):
    """HND ``[pages,Hkv,ps,D]`` vs NHD ``[pages,ps,Hkv,D]`` (upstream api.py:455-469).
    Returns (is_nhd, num_kv_heads, page_size); HND is tested first."""
    if len(shape) != 4:
        raise ValueError(
            f"paged K/V must be 4D ([pages,Hkv,ps,D] HND or [pages,ps,Hkv,D] NHD), "
            f"got shape {tuple(shape)}")
    if page_size_hint is not None and page_size_hint > 0:
        if shape[2] == page_size_hint:
            return False, int(shape[1]), int(shape[2])
        if shape[1] == page_size_hint:
            return True, int(shape[2]), int(shape[1])
        raise ValueError(
            f"cannot infer paged KV layout: neither dim1 nor dim2 of shape={tuple(shape)} "
            f"equals page_size={page_size_hint}; expected [pages,Hkv,ps,D] (HND) "
            f"or [pages,ps,Hkv,D] (NHD)")
    return False, int(shape[1]), int(shape[2])


def _compute_pack_factor(max_qo_len, num_qo_heads, num_kv_heads):
    """Query heads folded into the row dimension for short queries (upstream api.py:308-318).
    Here the whole KV-head group is folded whenever the queries are short."""
    if num_kv_heads == -1:
        num_kv_heads = num_qo_heads
    h_r = num_qo_heads // num_kv_heads
    if h_r <= 1 or max_qo_len <= 0 or max_qo_len > 32:
        return 1
    return h_r


def _block_m(rows):
    return 16 if rows <= 16 else (64 if rows <= 64 else 128)


class PlanInfo(dict):
    """Execution plan returned by the planner; pass it unchanged to ``fmha_sail``."""


# ----------------------------------------------------------------------------
# workspace arena (graph-safe callers hand in one fixed uint8 tensor)
# ----------------------------------------------------------------------------

class _Arena:
    def __init__(self, buf, device):
        self.buf, self.off, self.device = buf, 0, device

    def take(self, numel, dtype):
        item = torch.empty(0, dtype=dtype).element_size()
        if self.buf is None:
            return torch.empty(numel, dtype=dtype, device=self.device)
        self.off = (self.off + 255) & ~255
        end = self.off + numel * item
        if end > self.buf.numel():
            raise ValueError(
                f"given_workspace too small: {self.buf.numel()} bytes < required {end} bytes. "
                f"Re-allocate with allocate_graph_workspace(...).")
        out = self.buf[self.off:end].view(dtype)
        self.off = end
        return out


def _workspace_bytes(batch, total_q, num_qo_heads, splits, sparse):
    meta = (5 * (batch + 1) + 2 * total_q) * 4 + 256 * 8
    work = 0 if sparse else 2 * max(1, total_q) * num_qo_heads * max(1, splits) * 32   # both work lists
    part = 0 if splits <= 1 else splits * total_q * num_qo_heads * (128 + 1) * 4
    return meta + work + part + 4096


def allocate_graph_workspace(batch_size, num_qo_heads, num_kv_heads=-1,
                             max_qo_len=1, page_size=128, kv_block_num=-1,
                             num_kv_splits=1, device=None,
                             output_maxscore=False, use_fp8_kvcache=False):
    """Pre-allocate a fixed-address workspace for CUDA Graph capture
    (upstream api.py:383-447).  Pass the result as ``given_workspace`` to
    ``fmha_sail_plan``; sized for the worst case ``batch_size * max_qo_len`` tokens."""
    device = torch.cuda.current_device() if device is None else device
    is_sparse = kv_block_num > 0 and page_size > 0
    splits = num_kv_splits if num_kv_splits >= 1 else 128
    if is_sparse:
        splits = min(splits, kv_block_num)
    total = _workspace_bytes(batch_size, batch_size * max_qo_len, num_qo_heads, splits, is_sparse)
    return torch.empty(total, dtype=torch.uint8, device=device)


# ----------------------------------------------------------------------------
# planner
# ----------------------------------------------------------------------------

def _to_int_list(t):
    if isinstance(t, torch.Tensor):
        return [int(x) for x in t.detach().cpu().reshape(-1).tolist()]
    return [int(x) for x in t]


def _fmha_sail_plan(
    qo_segment_lens: torch.Tensor,
    kv_segment_lens: torch.Tensor,
    num_qo_heads: int,
    num_kv_heads: int = -1,
    qo_offset: Optional[Union[int, torch.Tensor]] = None,
    num_kv_splits: int = -1,
    page_size: int = -1,
    output_maxscore: bool = False,
    kv_block_num: int = -1,
    usable_SM_count: int = -1,
    causal: bool = True,
    sparse_kernel_mode: str = 'auto',
    use_fp8_kvcache: bool = False,
    device=None,
    stream=None,
    given_workspace=None,
    max_total_q: int = -1,
    graph_safe: bool = False,
    max_qo_len_override: int = -1,
    qo_len_uniform_override: Optional[bool] = None,
    max_kv_len_override: int = -1,
):
    """Internal planner (upstream ``_fmha_sail_plan``, api.py:889-1217).

    Lengths are read on the host; the work list is produced by the native
    host planner ``msa_plan_dense`` and uploaded once.  The plan owns its
    metadata tensors (no buffer is shared between two live plans)."""
    device = torch.cuda.current_device() if device is None else device
    dev = torch.device("cuda", device) if isinstance(device, int) else torch.device(device)

    if graph_safe:
        if max_qo_len_override <= 0:
            raise ValueError("graph_safe=True requires max_qo_len_override > 0")
        if qo_len_uniform_override is None:
            raise ValueError("graph_safe=True requires qo_len_uniform_override")
        if given_workspace is None:
            raise ValueError("graph_safe=True requires given_workspace (pre-allocated)")
        if max_total_q <= 0:
            raise ValueError("graph_safe=True requires max_total_q > 0")
        if (output_maxscore or not causal) and max_kv_len_override <= 0:
            raise ValueError(
                "graph_safe=True requires max_kv_len_override > 0 "
                "when output_maxscore=True or causal=False")
        if isinstance(qo_offset, int):
            raise ValueError(
                "graph_safe=True requires qo_offset as a CUDA tensor; an int "
                "triggers an in-capture allocation")

    if graph_safe:
        on_dev = (isinstance(qo_segment_lens, torch.Tensor) and qo_segment_lens.is_cuda
                  and isinstance(kv_segment_lens, torch.Tensor) and kv_segment_lens.is_cuda
                  and (qo_offset is None or (isinstance(qo_offset, torch.Tensor) and qo_offset.is_cuda)))
        hkv_ = num_qo_heads if num_kv_heads == -1 else num_kv_heads
        if on_dev:
            return _fmha_sail_plan_device(
                qo_segment_lens, kv_segment_lens, num_qo_heads, hkv_, qo_offset, num_kv_splits, page_size,
                output_maxscore, kv_block_num, usable_SM_count, causal, use_fp8_kvcache, dev, given_workspace,
                max_total_q, max_qo_len_override, bool(qo_len_uniform_override), max_kv_len_override)
        # host-resident lengths: planned on the host below, which reads them

    qo_lens = _to_int_list(qo_segment_lens)
    kv_lens = _to_int_list(kv_segment_lens)
    batch = len(qo_lens)
    assert len(kv_lens) == batch, "qo_segment_lens and kv_segment_lens must have the same length"
    max_qo = max(qo_lens) if qo_lens else 0
    qo_len_uniform = batch > 0 and min(qo_lens) == max_qo
    if max_qo_len_override > 0 and not graph_safe:
        assert max_qo_len_override == max_qo, (
            f"max_qo_len_override={max_qo_len_override} != actual max(qo_lens)={max_qo}")
    if qo_len_uniform_override is not None and not graph_safe:
        assert qo_len_uniform_override == qo_len_uniform, (
            f"qo_len_uniform_override={qo_len_uniform_override} != actual={qo_len_uniform}")

    orig_num_qo_heads = num_qo_heads
    hkv = num_qo_heads if num_kv_heads == -1 else num_kv_heads
    assert num_qo_heads % hkv == 0, (
        f"num_qo_heads ({num_qo_heads}) must be divisible by num_kv_heads ({hkv})")
    h_r = num_qo_heads // hkv
    is_sparse = kv_block_num > 0 and page_size > 0
    total_q = sum(qo_lens)
    max_kv = max(kv_lens) if kv_lens else 0
    if max_kv_len_override > 0:
        max_kv = max(max_kv, max_kv_len_override) if not graph_safe else max_kv_len_override

    # causal offsets (upstream prepare_plan_metadata.cuh:120-130)
    if not causal:
        offs = [max_kv] * batch
    elif qo_offset is None:
        offs = [kv_lens[i] - qo_lens[i] for i in range(batch)]
    elif isinstance(qo_offset, int):
        offs = [qo_offset] * batch
    else:
        offs = _to_int_list(qo_offset)
        assert len(offs) == batch, f"qo_offset must be [batch_size={batch}], got {len(offs)}"
        offs = [kv_lens[i] - qo_lens[i] if o < 0 else o for i, o in enumerate(offs)]

    if is_sparse:
        pack = h_r
        block_m = _block_m(h_r)
    else:
        pack = _compute_pack_factor(max_qo, num_qo_heads, hkv)
        block_m = _block_m(max_qo * pack)
    num_sms = _num_sms(dev)
    if usable_SM_count > 0:
        num_sms = min(num_sms, usable_SM_count)

    arena = _Arena(given_workspace, dev)

    def upload(values, n=None):
        a = np.asarray(values, dtype=np.int32)
        t = arena.take(a.size if n is None else n, torch.int32)
        if a.size:
            t[:a.size].copy_(torch.from_numpy(a), non_blocking=False)
        return t

    qo_start = np.zeros(batch + 1, np.int32); qo_start[1:] = np.cumsum(qo_lens)
    kv_start = np.zeros(batch + 1, np.int32); kv_start[1:] = np.cumsum(kv_lens)
    info = PlanInfo()
    info["qo_segment_offsets"] = upload(qo_start)
    info["kv_segment_offsets"] = upload(kv_start)
    info["qo_segment_lens"] = upload(qo_lens)
    info["kv_segment_lens"] = upload(kv_lens)
    info["qo_offset"] = upload(offs)
    if page_size > 0:
        indptr = np.zeros(batch + 1, np.int32)
        indptr[1:] = np.cumsum([(k + page_size - 1) // page_size for k in kv_lens])
        info["kv_page_indptr"] = upload(indptr)
    else:
        info["kv_page_indptr"] = None

    work = None
    num_work = 0
    splits_per_row = None
    if is_sparse:
        items = total_q * hkv
        if num_kv_splits >= 1:
            # an explicit count is an upper bound: once the (token, KV head) items alone give every
            # SM a CTA, further splitting only adds per-CTA prologue/epilogue latency and a merge
            # pass (the result does not depend on the split count)
            splits = min(num_kv_splits, kv_block_num)
            while splits > 1 and items * (splits // 2) >= num_sms:
                splits //= 2
        else:
            splits = 1
            while splits * 2 <= min(kv_block_num, 8) and items * splits < 2 * num_sms:
                splits *= 2
        info["token_batch"] = upload(np.repeat(np.arange(batch, dtype=np.int32), qo_lens))
        pages_per = [(kl + page_size - 1) // page_size for kl in kv_lens]
        info["page_batch"] = upload(np.repeat(np.arange(batch, dtype=np.int32), pages_per))
        info["num_logical_pages"] = int(sum(pages_per))
        info["sparse_ws"] = None
        # page-major path pays off once several tokens share a page
        info["sparse_tc_preferred"] = (sum(pages_per) > 0 and total_q * kv_block_num >= 8 * sum(pages_per)
                                       and total_q >= 256)
    else:
        info["token_batch"] = None
        a_q = np.asarray(qo_lens, np.int32); a_k = np.asarray(kv_lens, np.int32); a_o = np.asarray(offs, np.int32)
        args = _lib.MsaPlanArgs(
            a_q.ctypes.data, a_k.ctypes.data, a_o.ctypes.data, batch, num_qo_heads, hkv, block_m, pack,
            num_kv_splits if num_kv_splits >= 1 else -128, num_sms, 0)
        cap = 1024
        spr = np.ones(max(1, total_q), np.int32)
        max_splits = _lib._i32(1)
        while True:
            host = np.empty((cap, 8), np.int32)
            n = _lib.lib.msa_plan_dense(ctypes.byref(args), host.ctypes.data, cap, spr.ctypes.data,
                                        ctypes.byref(max_splits))
            if n == -4:
                cap *= 4
                continue
            _lib.check(n, "msa_plan_dense")
            break
        num_work = n
        splits = int(max_splits.value)
        work = arena.take(max(1, n) * 8, torch.int32)
        if n:
            work[:n * 8].copy_(torch.from_numpy(host[:n].reshape(-1)))
        info["_work_host"] = host[:n]
        if splits > 1:
            splits_per_row = upload(spr[:total_q])
        # second work list in 256-row items for the tcgen05 prefill kernel (q and k both bf16 or
        # both e4m3, unsplit, one query head per row tile, ragged K/V or 128-key pages)
        info["work_tc"], info["num_work_tc"] = None, 0
        info["tc_preferred"] = False
        if pack == 1 and max_qo > 128 and page_size in (-1, 0, 128):
            args_tc = _lib.MsaPlanArgs(
                a_q.ctypes.data, a_k.ctypes.data, a_o.ctypes.data, batch, num_qo_heads, hkv, 256, 1,
                1, num_sms, 0)
            cap_tc = max(16, (total_q // 256 + batch) * num_qo_heads)
            host_tc = np.empty((cap_tc, 8), np.int32)
            n_tc = _lib.check(_lib.lib.msa_plan_dense(ctypes.byref(args_tc), host_tc.ctypes.data, cap_tc,
                                                      None, None), "msa_plan_dense")
            if n_tc:
                wt = arena.take(n_tc * 8, torch.int32)
                wt.copy_(torch.from_numpy(host_tc[:n_tc].reshape(-1)))
                info["work_tc"], info["num_work_tc"] = wt, n_tc
                # with far too few items to fill the GPU the split-KV plan of the generic kernel wins
                # (a 256-row tcgen05 item runs about three times as fast as the same rows there)
                info["tc_preferred"] = splits == 1 or n_tc * 2 >= num_sms

    if splits > 1:
        info["workspace_o"] = arena.take(splits * total_q * orig_num_qo_heads * 128, torch.float32)
        info["workspace_lse"] = arena.take(splits * total_q * orig_num_qo_heads, torch.float32)
    else:
        info["workspace_o"] = None
        info["workspace_lse"] = None

    max_k_tiles = math.ceil(math.ceil(max_kv / KV_TILE) / 128) * 128 if output_maxscore else -1
    if output_maxscore and orig_num_qo_heads * max_k_tiles * total_q > (1 << 31):
        print("Too huge setting to output maxscore!")
        max_k_tiles = -1

    info.update({
        "qo_tile_size": block_m,
        "kv_tile_size": KV_TILE,
        "work": work,
        "num_work": num_work,
        "num_kv_splits": splits,
        "num_kv_splits_per_row": splits_per_row,
        "max_qo_len": max_qo,
        "predicted_speedup": 1.0,
        "max_k_tiles": max_k_tiles,
        "pack_factor": pack,
        "orig_num_qo_heads": orig_num_qo_heads,
        "num_kv_heads": hkv,
        "kv_heads_given": num_kv_heads != -1,
        "qo_len_uniform": qo_len_uniform,
        "graph_safe": graph_safe,
        "page_size": page_size,
        "kv_block_num": kv_block_num if is_sparse else -1,
        "is_sparse": is_sparse,
        "total_qo_len": total_q,
        "batch_size": batch,
        "causal": causal,
        "_host": {"qo_lens": qo_lens, "kv_lens": kv_lens, "qo_offset": offs},
    })
    return info


def _fmha_sail_plan_device(qo_segment_lens, kv_segment_lens, num_qo_heads, hkv, qo_offset, num_kv_splits,
                           page_size, output_maxscore, kv_block_num, usable_SM_count, causal, use_fp8_kvcache,
                           dev, given_workspace, max_total_q, max_qo, qo_len_uniform, max_kv_len_override):
    """Graph-safe planner (upstream graph_safe mode, api.py:916-941): the lengths stay on the GPU.

    Everything that sizes a launch comes from the arguments -- batch, ``max_qo_len_override`` (the
    row tiles per batch item), a fixed split count, ``max_total_q`` -- and one kernel
    (``msa_plan_device``) fills the metadata and the fixed-size work list inside
    ``given_workspace``.  No host read of device memory and no allocation, so the call can be
    captured in a CUDA graph together with ``fmha_sail`` and replayed after the length tensors (and
    the page table) have been updated in place."""
    batch = int(qo_segment_lens.shape[0])
    assert kv_segment_lens.shape[0] == batch, "qo_segment_lens and kv_segment_lens must have the same length"
    for name, t in (("qo_segment_lens", qo_segment_lens), ("kv_segment_lens", kv_segment_lens), ("qo_offset", qo_offset)):
        if t is not None and (t.dtype != torch.int32 or not t.is_contiguous()):
            raise ValueError(f"graph_safe=True requires {name} as a contiguous int32 CUDA tensor")
    h_r = num_qo_heads // hkv
    is_sparse = kv_block_num > 0 and page_size > 0
    if is_sparse:
        pack, block_m = h_r, _block_m(h_r)
        splits = min(num_kv_splits, kv_block_num) if num_kv_splits >= 1 else 1
        num_sms = _num_sms(dev)
        if usable_SM_count > 0:
            num_sms = min(num_sms, usable_SM_count)
        while splits > 1 and max_total_q * hkv * (splits // 2) >= num_sms:
            splits //= 2
    else:
        pack = _compute_pack_factor(max_qo, num_qo_heads, hkv)
        block_m = _block_m(max_qo * pack)
        splits = num_kv_splits if num_kv_splits >= 1 else 1
    groups = num_qo_heads // pack
    bm_eff = (block_m // pack) * pack
    row_tiles = max(1, -(-(max_qo * pack) // bm_eff))
    # long bf16 queries on 128-key pages (or ragged K/V): also a list of 256-row items for the tcgen05
    # prefill kernel, one query head per row tile, unsplit
    want_tc = (not is_sparse and pack == 1 and max_qo > 128 and page_size in (-1, 0, 128)
               and splits == 1)
    arena = _Arena(given_workspace, dev)
    info = PlanInfo()
    info["qo_segment_offsets"] = arena.take(batch + 1, torch.int32)
    info["kv_segment_offsets"] = arena.take(batch + 1, torch.int32)
    info["qo_segment_lens"] = qo_segment_lens
    info["kv_segment_lens"] = arena.take(batch, torch.int32)
    info["qo_offset"] = arena.take(batch, torch.int32)
    info["kv_page_indptr"] = arena.take(batch + 1, torch.int32) if page_size > 0 else None
    info["token_batch"] = arena.take(max_total_q, torch.int32) if is_sparse else None
    splits_per_row = arena.take(max_total_q, torch.int32) if splits > 1 else None
    n_items = 0 if is_sparse else batch * row_tiles * groups * splits
    work = arena.take(max(1, n_items) * 8, torch.int32) if not is_sparse else None
    tc_tiles = max(1, -(-max_qo // 256))
    n_items_tc = batch * tc_tiles * num_qo_heads if want_tc else 0
    work_tc = arena.take(n_items_tc * 8, torch.int32) if want_tc else None
    if splits > 1:
        info["workspace_o"] = arena.take(splits * max_total_q * num_qo_heads * 128, torch.float32)
        info["workspace_lse"] = arena.take(splits * max_total_q * num_qo_heads, torch.float32)
    else:
        info["workspace_o"] = info["workspace_lse"] = None
    max_kv = max_kv_len_override
    a = _lib.MsaPlanDeviceArgs()
    a.qo_len, a.kv_len, a.qo_offset_in = qo_segment_lens.data_ptr(), kv_segment_lens.data_ptr(), _ptr(qo_offset)
    a.qo_start, a.kv_start = info["qo_segment_offsets"].data_ptr(), info["kv_segment_offsets"].data_ptr()
    a.kv_len_out, a.qo_offset_out = info["kv_segment_lens"].data_ptr(), info["qo_offset"].data_ptr()
    a.kv_page_indptr, a.token_batch = _ptr(info["kv_page_indptr"]), _ptr(info["token_batch"])
    a.splits_per_row, a.work = _ptr(splits_per_row), _ptr(work)
    a.batch, a.num_qo_heads, a.num_kv_heads = batch, num_qo_heads, hkv
    a.block_m, a.pack, a.num_splits = block_m, pack, splits
    a.page_size, a.causal, a.noncausal_offset = page_size, int(bool(causal)), max(0, max_kv)
    a.max_total_q, a.row_tiles = max_total_q, row_tiles
    _lib.check(_lib.lib.msa_plan_device(ctypes.byref(a), _stream()), "msa_plan_device")
    if want_tc:
        t = _lib.MsaPlanDeviceArgs()
        t.qo_len, t.kv_len, t.qo_offset_in = a.qo_len, a.kv_len, a.qo_offset_in
        t.work = work_tc.data_ptr()
        t.batch, t.num_qo_heads, t.num_kv_heads = batch, num_qo_heads, hkv
        t.block_m, t.pack, t.num_splits, t.row_tiles = 256, 1, 1, tc_tiles
        t.page_size, t.causal, t.noncausal_offset, t.max_total_q = page_size, a.causal, a.noncausal_offset, 0
        _lib.check(_lib.lib.msa_plan_device(ctypes.byref(t), _stream()), "msa_plan_device")

    max_k_tiles = math.ceil(math.ceil(max_kv / KV_TILE) / 128) * 128 if output_maxscore else -1
    info.update({
        "qo_tile_size": block_m, "kv_tile_size": KV_TILE, "work": work, "num_work": n_items,
        "work_tc": work_tc, "num_work_tc": n_items_tc, "tc_preferred": want_tc,
        "page_batch": None, "num_logical_pages": 0, "sparse_tc_preferred": False, "sparse_ws": None,
        "num_kv_splits": splits, "num_kv_splits_per_row": splits_per_row, "max_qo_len": max_qo,
        "predicted_speedup": 1.0, "max_k_tiles": max_k_tiles, "pack_factor": pack,
        "orig_num_qo_heads": num_qo_heads, "num_kv_heads": hkv, "qo_len_uniform": qo_len_uniform,
        "graph_safe": True, "page_size": page_size, "kv_block_num": kv_block_num if is_sparse else -1,
        "is_sparse": is_sparse, "total_qo_len": max_total_q, "batch_size": batch, "causal": causal,
        "_host": None,
    })
    return info


# ----------------------------------------------------------------------------
# input validation (upstream _validate_fmha_inputs, api.py:471-768)
# ----------------------------------------------------------------------------

def _validate_fmha_inputs(q, k, v, plan, is_paged, kv_is_nhd, num_kv_heads, page_size,
                          kv_indices, kv_block_indexes, qo_offset):
    host = plan["_host"]
    qo_lens, kv_lens = host["qo_lens"], host["kv_lens"]
    batch = len(qo_lens)
    num_qo_heads = q.shape[1]
    assert q.dim() == 3, f"q must be [total_qo_len, num_qo_heads, head_dim], got {q.shape}"
    assert num_qo_heads % num_kv_heads == 0, (
        f"num_qo_heads ({num_qo_heads}) must be divisible by num_kv_heads ({num_kv_heads})")
    assert sum(qo_lens) == q.shape[0], (
        f"sum(qo_segment_lens)={sum(qo_lens)} != q.shape[0]={q.shape[0]}")
    if is_paged:
        assert k.dim() == 4 and v.dim() == 4, "paged K/V must be 4D"
        assert sorted([k.shape[1], k.shape[2]]) == sorted([num_kv_heads, page_size]), (
            f"paged K dims 1/2 must be {{Hkv={num_kv_heads}, page_size={page_size}}}, got {k.shape}")
        assert v.shape[:3] == k.shape[:3], (
            f"paged V must use the same layout as K, got K={tuple(k.shape)} V={tuple(v.shape)}")
        for name, t in (("K", k), ("V", v)):
            assert t.stride(3) == 1, f"paged {name} head_dim must be contiguous (stride(-1)==1)"
            if not kv_is_nhd:
                assert t.stride(2) == t.shape[3], (
                    f"paged {name} HND requires contiguous in-page tokens (stride(2)==head_dim)")
    else:
        assert sum(kv_lens) == k.shape[0], (
            f"sum(kv_segment_lens)={sum(kv_lens)} != k.shape[0]={k.shape[0]}")
    if qo_offset is not None:
        assert qo_offset.dim() == 1 and qo_offset.shape[0] == batch, (
            f"qo_offset must be [batch_size={batch}], got {qo_offset.shape}")
    pages_per = [(kl + page_size - 1) // page_size for kl in kv_lens] if is_paged else []
    if kv_indices is not None:
        assert is_paged, "kv_indices provided but K/V are not paged (4D)"
        kvi = kv_indices.cpu()
        if kv_block_indexes is None:
            assert kvi.numel() == sum(pages_per), (
                f"kv_indices length {kvi.numel()} != sum(ceil(kv_segment_lens/page_size))={sum(pages_per)}")
        if kvi.numel():
            assert (kvi >= 0).all() and (kvi < k.shape[0]).all(), (
                f"kv_indices has values outside [0, {k.shape[0]})")
    if kv_block_indexes is not None:
        assert is_paged, "sparse mode requires paged KV (kv_indices)"
        assert kv_indices is not None, "sparse mode requires kv_indices"
        assert kv_block_indexes.dim() == 3, (
            f"kv_block_indexes must be [total_qo_len, H_kv, KVBlockNum], got {kv_block_indexes.shape}")
        assert kv_block_indexes.shape[0] == q.shape[0]
        assert kv_block_indexes.shape[1] == num_kv_heads
        bi = kv_block_indexes.cpu()
        valid = bi != -1
        assert ((bi >= 0) | (bi == -1)).all(), "kv_block_indexes must contain only non-negative indices or -1"
        assert (valid[:, :, :-1] >= valid[:, :, 1:]).all(), "kv_block_indexes: -1 padding must be at the end"
        tok_batch = torch.repeat_interleave(torch.arange(batch), torch.tensor(qo_lens))
        n_pages = torch.tensor(pages_per)[tok_batch].view(-1, 1, 1)
        assert (bi[valid] < n_pages.expand_as(bi)[valid]).all(), (
            "kv_block_indexes: index out of range for batch page count")
        both = valid[:, :, :-1] & valid[:, :, 1:]
        if both.any():
            assert (bi[:, :, 1:][both] > bi[:, :, :-1][both]).all(), (
                "kv_block_indexes: must be strictly ascending")
    # plan coverage: every (batch, head group, row tile) exactly once per split, split ranges
    # contiguous from 0 (upstream tests/integration/test_plan_correctness.py:58-190)
    work = plan.get("_work_host")
    if work is not None and len(work):
        seen = {}
        for b, h0, r0, tb, te, sp, nr, _ in work.tolist():
            assert 0 <= b < batch and tb <= te
            seen.setdefault((b, h0, r0), []).append((tb, te, sp))
        pack, bm = plan["pack_factor"], plan["qo_tile_size"]
        bm_eff = (bm // pack) * pack
        groups = plan["orig_num_qo_heads"] // pack
        for b in range(batch):
            for r0 in range(0, qo_lens[b] * pack, bm_eff):
                for g in range(groups):
                    parts = sorted(seen.get((b, g * pack, r0), []))
                    assert parts, f"plan misses work item (batch={b}, head0={g * pack}, row0={r0})"
                    assert parts[0][0] == 0
                    for x, y in zip(parts, parts[1:]):
                        assert x[1] == y[0], f"gap/overlap at split boundary of {(b, g * pack, r0)}"
                    assert sorted(s[2] for s in parts) == list(range(len(parts)))


# ----------------------------------------------------------------------------
# run
# ----------------------------------------------------------------------------

def _scale_arg(x, device, hkv):
    """A scale is a float, or an fp32 tensor with one value per KV head."""
    if x is None:
        return 1.0, None
    if isinstance(x, torch.Tensor):
        if x.numel() == 1:
            return float(x.item()), None
        assert x.numel() == hkv, f"per-head scale must have {hkv} entries, got {x.numel()}"
        return 1.0, x.to(device=device, dtype=torch.float32).contiguous()
    return float(x), None


def _show_params(q, plan, is_paged, page_size, sm_scale, output_o, max_score, kv_block_indexes):
    """Print the call's shape as one '[MSA] --format=...' line (upstream
    csrc/msa_profiling_interface.hpp:99-157, enabled by PPU_LIB_SHOW_PARAMS=1);
    ``benchmarks/run_msa.py`` re-runs a call from such a line."""
    host = plan["_host"]
    if host is None:
        return
    if kv_block_indexes is not None:
        mode = "Sparse"
    elif max_score is not None:
        mode = "Full" if output_o else "OnlyScore"
    else:
        mode = "Off"
    lst = lambda v: "[" + ",".join(str(int(x)) for x in v) + "]"
    fields = [("dtype", "fp8" if q.dtype == torch.float8_e4m3fn else "bf16"), ("batch_size", plan["batch_size"]),
              ("seqlen_q", lst(host["qo_lens"])), ("seqlen_k", lst(host["kv_lens"])), ("qo_offset", lst(host["qo_offset"])),
              ("num_qo_heads", plan["orig_num_qo_heads"]), ("num_kv_heads", plan["num_kv_heads"]),
              ("head_dim_qk", 128), ("head_dim_vo", 128), ("num_kv_splits", plan["num_kv_splits"]),
              ("is_paged", int(is_paged)), ("page_size", page_size if is_paged else 0), ("causal", int(plan["causal"])),
              ("sm_scale", f"{sm_scale:.6f}"), ("sparse_mode", mode),
              ("kv_block_num", plan["kv_block_num"] if plan["is_sparse"] else 0)]
    print("[MSA] --format=" + ",".join(f"{k}:{v}" for k, v in fields) + ".", flush=True)


def _fmha_sail(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    plan_info,
    kv_indices: Optional[torch.Tensor] = None,
    kv_block_indexes: Optional[torch.Tensor] = None,
    q_offset_override: Optional[Union[int, torch.Tensor]] = None,
    out: Optional[torch.Tensor] = None,
    max_score: Optional[torch.Tensor] = None,
    sm_scale: Optional[float] = None,
    q_scale=None,
    k_scale=None,
    v_scale=None,
    o_scale=None,
    output_maxscore: bool = True,
    output_o: bool = True,
    check_input_valid: bool = False,
    max_score_dtype: Optional[torch.dtype] = None,
    lse: Optional[torch.Tensor] = None,
) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
    """Internal runner (upstream ``_fmha_sail``, api.py:1221-1477).

    Extension over upstream: ``lse`` -- a preallocated fp32 ``[total_q, Hq]``
    buffer that receives the natural-log LSE of every row; ``k_scale`` /
    ``v_scale`` may be fp32 tensors with one entry per KV head; bf16 ``q`` may
    be combined with e4m3 ``k``/``v``; a preallocated ``out`` may be fp32 (the
    unrounded result, what a rank hands to a cross-GPU merge: written by the
    split-KV merge directly, converted from the bf16 result otherwise)."""
    if not q.is_cuda:
        raise RuntimeError("fmha_sail needs CUDA tensors (there is no CPU path)")
    nnz_qo, num_qo_heads, head_dim_qk = q.shape
    plan_page = plan_info.get("page_size", -1)
    if kv_indices is None:
        nnz_kv, num_kv_heads, head_dim_vo = v.shape
        is_paged, kv_is_nhd, page_size = False, False, 0
    else:
        kv_is_nhd, num_kv_heads, page_size = _detect_paged_kv_layout(k.shape, plan_page)
        head_dim_vo = v.shape[3]
        is_paged = True
    if head_dim_qk != 128 or head_dim_vo != 128:
        raise ValueError("fmha_sail supports head_dim 128 only")

    max_k_tiles = plan_info["max_k_tiles"]
    is_fp8_q = q.dtype == torch.float8_e4m3fn
    is_fp8_kv = k.dtype == torch.float8_e4m3fn
    if is_fp8_q and not is_fp8_kv:
        raise ValueError(
            f"fmha_sail fp8 mode requires q/k to share the same dtype, got q={q.dtype}, k={k.dtype}")
    if is_fp8_kv and v is not None and output_o and v.dtype != k.dtype:
        raise ValueError("FP8 K requires V to use float8_e4m3fn as well")
    if is_fp8_q and kv_block_indexes is not None:
        if not is_paged or page_size != 128:
            raise ValueError("Sparse FP8 requires paged KV with page_size=128 and head_dim=128")

    if max_score_dtype is None:
        max_score_dtype = max_score.dtype if max_score is not None else torch.float32
    if max_score_dtype not in (torch.float32, torch.bfloat16):
        raise ValueError(
            f"fmha_sail max_score_dtype must be torch.float32 or torch.bfloat16, got {max_score_dtype}")
    if max_score is not None and max_score.dtype != max_score_dtype:
        raise ValueError(
            f"max_score buffer dtype {max_score.dtype} does not match max_score_dtype {max_score_dtype}")

    plan = plan_info
    batch = plan["batch_size"]
    if plan["_host"] is None:                 # planned on the device: total_qo_len is the bound max_total_q
        if nnz_qo > plan["total_qo_len"]:
            raise ValueError(f"plan allows at most {plan['total_qo_len']} query tokens, q has {nnz_qo}")
    elif plan["total_qo_len"] != nnz_qo:
        raise ValueError(f"plan was made for {plan['total_qo_len']} query tokens, q has {nnz_qo}")
    if plan["orig_num_qo_heads"] != num_qo_heads:
        raise ValueError("plan head counts do not match q / k")
    if plan["num_kv_heads"] != num_kv_heads:
        # A plan made without num_kv_heads does not pin the KV head count (upstream takes it from K's shape at
        # run time, api.py:1275-1290): such a plan has one query head per work item, which fits any grouping.
        if plan.get("kv_heads_given", True) or plan["pack_factor"] != 1 or plan["is_sparse"] or num_qo_heads % num_kv_heads:
            raise ValueError("plan head counts do not match q / k")
    if plan["is_sparse"] != (kv_block_indexes is not None):
        raise ValueError("plan sparse mode (kv_block_num) does not match kv_block_indexes")
    if (plan_page > 0) != is_paged:
        raise ValueError("plan page_size does not match the K/V layout (kv_indices given?)")

    qo_offset = plan["qo_offset"] if q_offset_override is None else q_offset_override
    if isinstance(qo_offset, int):
        if plan.get("graph_safe", False):
            raise ValueError(
                "graph_safe=True requires q_offset_override as a CUDA tensor; "
                "an int triggers an in-capture torch.full_like allocation")
        qo_offset = torch.full_like(plan["qo_segment_lens"], qo_offset)
    else:
        assert qo_offset.device == plan["qo_segment_lens"].device
        if qo_offset.dtype != torch.int32:
            qo_offset = qo_offset.to(torch.int32)

    if check_input_valid and plan["_host"] is not None:
        _validate_fmha_inputs(q, k, v, plan, is_paged, kv_is_nhd, num_kv_heads, page_size,
                              kv_indices, kv_block_indexes, qo_offset)

    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(head_dim_qk)
    q_s, _ = _scale_arg(q_scale, q.device, num_kv_heads)
    k_s, k_head = _scale_arg(k_scale, q.device, num_kv_heads)
    v_s, v_head = _scale_arg(v_scale, q.device, num_kv_heads)
    o_s, _ = _scale_arg(o_scale, q.device, num_kv_heads)

    assert output_o or output_maxscore

    if not output_maxscore or max_k_tiles == -1:
        max_score = None
        output_o = True
    elif max_score is None and max_k_tiles > 0:
        max_score = torch.full((num_qo_heads, max_k_tiles, nnz_qo), -float("inf"),
                               dtype=max_score_dtype, device=q.device)
    if kv_block_indexes is not None and max_score is not None:
        raise ValueError("sparse mode computes O only: plan it without output_maxscore")
    if max_score is not None and max_score_dtype == torch.bfloat16 and output_o:
        raise ValueError(
            "max_score_dtype=torch.bfloat16 requires OnlyScore mode "
            "(output_maxscore=True, output_o=False, no kv_block_indexes)")

    if not output_o:
        out = None
    elif out is None:
        out = torch.empty(nnz_qo, num_qo_heads, head_dim_vo, device=q.device, dtype=torch.bfloat16)
    else:
        assert out.dtype in (torch.bfloat16, torch.float32) and out.shape == (nnz_qo, num_qo_heads, head_dim_vo)
        assert out.stride(2) == 1

    if nnz_qo == 0:
        return out, max_score

    p = _lib.MsaFmhaParams()
    p.q, p.k = q.data_ptr(), k.data_ptr()
    p.v = v.data_ptr() if output_o else None
    p.q_stride_tok, p.q_stride_head = q.stride(0), q.stride(1)
    assert q.stride(2) == 1, "q head_dim must be contiguous"
    if is_paged:
        if kv_is_nhd:
            p.k_stride_page, p.k_stride_tok, p.k_stride_head = k.stride(0), k.stride(1), k.stride(2)
            p.v_stride_page, p.v_stride_tok, p.v_stride_head = v.stride(0), v.stride(1), v.stride(2)
        else:
            p.k_stride_page, p.k_stride_head, p.k_stride_tok = k.stride(0), k.stride(1), k.stride(2)
            p.v_stride_page, p.v_stride_head, p.v_stride_tok = v.stride(0), v.stride(1), v.stride(2)
        assert k.stride(3) == 1 and v.stride(3) == 1, "paged K/V head_dim must be contiguous"
        assert kv_indices.dtype == torch.int32 and kv_indices.is_cuda
        p.kv_indices = kv_indices.data_ptr()
        p.kv_page_indptr = plan["kv_page_indptr"].data_ptr()
        p.page_size = page_size
    else:
        p.k_stride_page = p.v_stride_page = 0
        p.k_stride_tok, p.k_stride_head = k.stride(0), k.stride(1)
        p.v_stride_tok, p.v_stride_head = v.stride(0), v.stride(1)
        assert k.stride(2) == 1 and v.stride(2) == 1, "K/V head_dim must be contiguous"
        p.kv_start = plan["kv_segment_offsets"].data_ptr()
        p.page_size = 0
    p.qo_start = plan["qo_segment_offsets"].data_ptr()
    p.kv_len = plan["kv_segment_lens"].data_ptr()
    p.qo_offset = qo_offset.data_ptr()
    splits = plan["num_kv_splits"]
    use_tc = (plan.get("work_tc") is not None and kv_block_indexes is None
              and q.dtype == k.dtype and k.dtype in (torch.bfloat16, torch.float8_e4m3fn)
              and page_size in (0, 128) and _USE_TC and (plan["tc_preferred"] or _FORCE_TC))
    use_split = output_o and splits > 1 and not use_tc
    kernel_out = out                             # what the attention kernel itself writes (bf16)
    if lse is not None:
        assert lse.dtype == torch.float32 and lse.is_contiguous() and lse.shape == (nnz_qo, num_qo_heads)
    if use_split:
        p.partial_o = plan["workspace_o"].data_ptr()
        p.partial_lse = plan["workspace_lse"].data_ptr()
        p.num_splits = splits
    else:
        p.num_splits = 1
        p.lse = _ptr(lse)
    if max_score is not None:
        assert max_score.is_contiguous() and max_score.shape == (num_qo_heads, max_k_tiles, nnz_qo)
        p.max_score = max_score.data_ptr()
        p.max_score_dtype = _dt_code(max_score.dtype)
        p.max_k_tiles = max_k_tiles
    if kv_block_indexes is not None:
        assert kv_block_indexes.dtype == torch.int32 and kv_block_indexes.is_cuda
        assert kv_block_indexes.dim() == 3 and kv_block_indexes.shape[0] == nnz_qo
        assert kv_block_indexes.stride(2) == 1
        if kv_block_indexes.shape[1] != num_kv_heads:
            raise ValueError(
                f"kv_block_indexes must be [total_qo_len, H_kv={num_kv_heads}, KVBlockNum], "
                f"got {tuple(kv_block_indexes.shape)}")
        p.kv_block_indexes = kv_block_indexes.data_ptr()
        p.kbi_stride_tok, p.kbi_stride_head = kv_block_indexes.stride(0), kv_block_indexes.stride(1)
        p.kv_block_num = kv_block_indexes.shape[2]
        p.token_batch = plan["token_batch"].data_ptr()
        g = num_qo_heads // num_kv_heads
        if (_USE_SPARSE_TC and (plan["sparse_tc_preferred"] or _FORCE_SPARSE_TC) and q.dtype == k.dtype
                and k.dtype in (torch.bfloat16, torch.float8_e4m3fn) and page_size == 128 and 128 % g == 0 and p.kv_block_num <= 32
                and plan["num_logical_pages"] > 0):
            need = _lib.lib.msa_sparse_workspace_bytes(nnz_qo, num_qo_heads, num_kv_heads, p.kv_block_num,
                                                       plan["num_logical_pages"])
            ws = plan.get("sparse_ws")
            if ws is None or ws.numel() < need or ws.device != q.device:
                ws = torch.empty(need, dtype=torch.uint8, device=q.device)
                plan["sparse_ws"] = ws
            p.sparse_ws, p.sparse_ws_bytes = ws.data_ptr(), ws.numel()
            p.page_batch = plan["page_batch"].data_ptr()
            p.num_logical_pages = plan["num_logical_pages"]
            use_split = False                     # the page-major path merges its own partials
            p.partial_o = p.partial_lse = None
            p.num_splits = 1
            p.lse = _ptr(lse)
    else:
        p.work = _ptr(plan["work"])
        p.num_work = plan["num_work"]
    if out is not None and out.dtype == torch.float32:
        # the split path's merge writes fp32 itself; an unsplit kernel writes bf16, converted below
        kernel_out = None if use_split else torch.empty(out.shape, dtype=torch.bfloat16, device=out.device)
    if kernel_out is not None:
        p.out = kernel_out.data_ptr()
        p.out_stride_tok, p.out_stride_head = kernel_out.stride(0), kernel_out.stride(1)
    p.k_scale_head, p.v_scale_head = _ptr(k_head), _ptr(v_head)
    p.total_q, p.num_qo_heads, p.num_kv_heads, p.batch = nnz_qo, num_qo_heads, num_kv_heads, batch
    p.block_m, p.pack = plan["qo_tile_size"], plan["pack_factor"]
    p.kv_extent = k.shape[0]
    if use_tc:
        p.work, p.num_work, p.block_m = plan["work_tc"].data_ptr(), plan["num_work_tc"], 256
    p.status = _status_word(q.device).data_ptr()
    rows = plan["max_qo_len"] * plan["pack_factor"] if kv_block_indexes is None else plan["pack_factor"]
    dt_ok = (q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16) or k.dtype == torch.float8_e4m3fn
    if (_USE_DECODE_TC and not use_tc and output_o != (max_score is not None) and dt_ok
            and page_size == 128 and 0 < rows <= 128
            and plan["pack_factor"] == num_qo_heads // num_kv_heads and 128 % plan["pack_factor"] == 0):
        p.decode_rows = rows
    p.q_dtype, p.kv_dtype = _dt_code(q.dtype), _dt_code(k.dtype)
    p.flags = (FLAG_OUT_O if output_o else 0) | (FLAG_OUT_SCORE if max_score is not None else 0) | \
              (FLAG_SPARSE if kv_block_indexes is not None else 0)
    p.sm_scale = float(q_s * k_s * sm_scale)
    p.out_scale = float(v_s * o_s)

    if _SHOW_PARAMS:
        _show_params(q, plan, is_paged, page_size, float(sm_scale), output_o, max_score, kv_block_indexes)
    stream = _stream()
    _lib.check(_lib.lib.msa_fmha_fwd(ctypes.byref(p), stream), "msa_fmha_fwd")

    if use_split:
        spr = plan["num_kv_splits_per_row"]
        _lib.check(_lib.lib.msa_lse_merge_ex(
            plan["workspace_o"].data_ptr(), MSA_DT_F32, plan["workspace_lse"].data_ptr(), _ptr(spr),
            out.data_ptr(), _dt_code(out.dtype), _ptr(lse), splits, nnz_qo, num_qo_heads, 0, 0,
            out.stride(0), out.stride(1), float(v_s * o_s), stream), "msa_lse_merge_ex")
    elif kernel_out is not None and kernel_out is not out:
        out.copy_(kernel_out)
    return out, max_score


def _decode_prefix(qo_segment_lens, sparse):
    """Length of the leading run of short-query (decode) batch items when the batch also holds a
    long-query (prefill) item, else 0.  Items are expected decode-first, as upstream's mixed
    batches are (api.py:1555-1575)."""
    long_items = (qo_segment_lens > _prefill_qlen_threshold(sparse)).nonzero(as_tuple=False)
    return int(long_items[0, 0].item()) if long_items.numel() else 0


def fmha_sail_plan(
    qo_segment_lens: torch.Tensor,
    kv_segment_lens: torch.Tensor,
    *args,
    qo_offset: Optional[Union[int, torch.Tensor]] = None,
    split_prefill_decode=False,
    **kwargs
):
    """Build a reusable execution plan for ``fmha_sail`` (upstream api.py:1480-1579).

    Returns ``(has_mixed_prefill, split, batch_size, decode_plan, prefill_plan)``;
    pass the tuple unchanged as ``plan_info`` to ``fmha_sail``.  Options
    (forwarded to ``_fmha_sail_plan``): ``num_kv_heads``, ``num_kv_splits``,
    ``page_size``, ``output_maxscore``, ``kv_block_num``, ``usable_SM_count``,
    ``causal``, ``use_fp8_kvcache``, ``device``, ``stream``, ``given_workspace``,
    ``max_total_q``, ``graph_safe`` and the ``*_override`` hints.  With
    ``split_prefill_decode`` a decode-first batch is planned as two sub-batches, each with
    the tile shape that suits it.
    """
    graph_safe = bool(kwargs.get("graph_safe", False))
    if isinstance(qo_offset, int):
        if graph_safe:
            raise ValueError(
                "graph_safe=True requires qo_offset as a CUDA tensor; an int "
                "triggers an in-capture torch.full_like allocation")
        qo_offset = torch.full_like(qo_segment_lens, qo_offset)
    batch_size = int(qo_segment_lens.shape[0])
    cut = 0
    if split_prefill_decode and not graph_safe and batch_size:
        cut = _decode_prefix(qo_segment_lens, kwargs.get("kv_block_num", -1) > 0)
    pieces = [slice(0, batch_size)] if cut == 0 else [slice(0, cut), slice(cut, batch_size)]
    plans = [_fmha_sail_plan(qo_segment_lens[s], kv_segment_lens[s], *args,
                             qo_offset=None if qo_offset is None else qo_offset[s], **kwargs) for s in pieces]
    return (cut > 0, cut, batch_size, plans[0], plans[1] if cut else None)


def _run_sub_batches(parts, q, k, v, kv_indices, kv_block_indexes, q_offset_override, out, max_score, kwargs):
    """Run consecutive sub-batches, each with its own plan, over slices of one call's tensors.

    ``parts``: ``[(plan, first batch item, one past the last)]`` in batch order.  Query tokens,
    page-table entries (paged) or keys (ragged) of the sub-batches follow one another in the
    inputs, so every sub-call sees plain slices; O and the LSE are written straight into slices of
    the combined buffers, per-tile scores are copied into a combined ``max_score`` (the
    sub-batches' tile counts differ)."""
    nnz_qo, num_qo_heads = q.shape[0], q.shape[1]
    paged = kv_indices is not None
    lse = kwargs.pop("lse", None)
    want_o = kwargs.get("output_o", True)
    if want_o and out is None:
        out = torch.empty(nnz_qo, num_qo_heads, v.shape[-1], device=q.device, dtype=torch.bfloat16)
    tok = kv = 0
    scores = []
    for plan, b0, b1 in parts:
        n_tok = plan["total_qo_len"]
        kv_lens = plan["_host"]["kv_lens"]
        ps = plan["page_size"]
        n_kv = sum(-(-kl // ps) for kl in kv_lens) if paged else sum(kv_lens)
        rows, span = slice(tok, tok + n_tok), slice(kv, kv + n_kv)
        off = q_offset_override[b0:b1] if isinstance(q_offset_override, torch.Tensor) else q_offset_override
        _, ms = _fmha_sail(
            q[rows], k if paged else k[span], v if paged else v[span], plan,
            kv_indices=kv_indices[span] if paged else None,
            kv_block_indexes=None if kv_block_indexes is None else kv_block_indexes[rows],
            q_offset_override=off, out=out[rows] if want_o else None, max_score=None,
            lse=None if lse is None else lse[rows], **kwargs)
        scores.append((rows, ms))
        tok += n_tok
        kv += n_kv
    if all(ms is None for _, ms in scores):
        return (out if want_o else None), None
    tiles = max(ms.shape[1] for _, ms in scores if ms is not None)
    dtype = next(ms.dtype for _, ms in scores if ms is not None)
    if max_score is None:
        max_score = torch.full((num_qo_heads, tiles, nnz_qo), -float("inf"), dtype=dtype, device=q.device)
    else:
        max_score.fill_(-float("inf"))
    for rows, ms in scores:
        if ms is not None:
            max_score[:, :ms.shape[1], rows] = ms
    return (out if want_o else None), max_score


def fmha_sail(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    plan_info,
    kv_indices: Optional[torch.Tensor] = None,
    kv_block_indexes: Optional[torch.Tensor] = None,
    q_offset_override: Optional[Union[int, torch.Tensor]] = None,
    out: Optional[torch.Tensor] = None,
    max_score: Optional[torch.Tensor] = None,
    **kwargs
) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
    """Run dense, paged or sparse FMHA using a precomputed plan (upstream api.py:1581-1728).

    ``q [total_q, Hq, 128]`` bf16 / e4m3; ``k``/``v`` ragged ``[total_kv, Hkv, 128]`` or
    paged ``[pages, Hkv, page, 128]`` (HND) / ``[pages, page, Hkv, 128]`` (NHD) with the flat
    int32 page table ``kv_indices``; ``kv_block_indexes [total_q, Hkv, kv_block_num]`` int32
    (ascending logical pages, -1 padded) selects sparse mode.  Runtime options: ``sm_scale``,
    ``q_scale``, ``k_scale``, ``v_scale``, ``o_scale``, ``output_maxscore``, ``output_o``,
    ``max_score_dtype``, ``check_input_valid``.  Returns ``(out, max_score)``; either may be
    ``None`` when that output is disabled.
    """
    mixed, cut, batch_size, first, second = plan_info
    if not mixed:
        return _fmha_sail(q, k, v, first, out=out, max_score=max_score, kv_indices=kv_indices,
                          kv_block_indexes=kv_block_indexes, q_offset_override=q_offset_override,
                          **kwargs)
    return _run_sub_batches([(first, 0, cut), (second, cut, batch_size)], q, k, v, kv_indices, kv_block_indexes,
                            q_offset_override, out, max_score, dict(kwargs))


# ============================================================================
# Sparse TopK Select
# ============================================================================

def sparse_topk_select(
    max_score: torch.Tensor,
    topk: int,
    num_valid_pages: Optional[int] = None,
    output: Optional[torch.Tensor] = None,
    force_begin_blocks: int = 0,
    force_end_blocks: int = 0,
) -> torch.Tensor:
    r"""Select top-k KV-tile indices per (qo_head, token) row (upstream api.py:1736-1848).

    ``max_score``: ``(num_qo_heads, max_k_tiles, total_qo_len)`` contiguous fp32 or bf16.
    Returns ``(total_qo_len, num_qo_heads, topk)`` int32, ascending by tile index, ``-1`` at
    the tail when fewer than ``topk`` pages exist.  Ranking is (score desc, index asc), so the
    result is deterministic for both dtypes.  ``topk`` may be 4, 8, 16 (upstream: 16 only) or 32.
    """
    if not isinstance(max_score, torch.Tensor) or max_score.dim() != 3:
        raise AssertionError(f"max_score must be 3D, got {getattr(max_score, 'shape', None)}")
    assert max_score.dtype in (torch.float32, torch.bfloat16), \
        f"max_score must be float32 or bfloat16, got {max_score.dtype}"
    assert max_score.is_contiguous(), "max_score must be contiguous"
    assert topk in (4, 8, 16, 32), f"topk must be 4, 8, 16 or 32, got {topk}"
    if not max_score.is_cuda:
        raise RuntimeError("sparse_topk_select needs a CUDA tensor (there is no CPU path)")
    num_qo_heads, max_k_tiles, total_qo_len = max_score.shape
    nvp = max_k_tiles if num_valid_pages is None else int(num_valid_pages)
    assert 0 < nvp <= max_k_tiles, f"num_valid_pages={nvp} must be in (0, max_k_tiles={max_k_tiles}]"
    fb, fe = int(force_begin_blocks), int(force_end_blocks)
    assert fb >= 0 and fe >= 0, (
        f"force_begin_blocks={fb} and force_end_blocks={fe} must be non-negative")
    assert fb + fe <= topk, (
        f"force_begin_blocks({fb}) + force_end_blocks({fe}) = {fb + fe} exceeds topk={topk}")
    shape = (total_qo_len, num_qo_heads, topk)
    if output is None:
        output = torch.empty(shape, dtype=torch.int32, device=max_score.device)
    else:
        assert output.dtype == torch.int32 and output.is_contiguous() and tuple(output.shape) == shape
    if total_qo_len == 0 or num_qo_heads == 0:
        return output
    _lib.check(_lib.lib.msa_topk_select(
        max_score.data_ptr(), _dt_code(max_score.dtype), output.data_ptr(),
        num_qo_heads, max_k_tiles, total_qo_len, topk, nvp, fb, fe, _stream()), "msa_topk_select")
    return output
