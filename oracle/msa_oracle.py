"""CPU oracle for the MSA attention hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain fp32 torch on CPU tensors, the PyTorch
references that the upstream project's own tests compare its kernels against.
It is the checker: only the test-suite, the smoke entry and the CPU-baseline
legs of the benchmark may import it.  Nothing in the shipped package does, and
the shipped package has no CPU fallback.

Parity status: PINNED.  Every function below is checked against outputs of the
upstream reference functions themselves (imported from the upstream tree by
``tests/golden/make_golden.py``, results committed as ``tests/golden/*.npz``)
by ``tests/test_oracle_golden.py``.

Upstream functions restated (paths are relative to the upstream project root):

* ``attention``          <- ``tests/ref_attn.py:24-81`` (``_mha_ref_single`` /
                            ``sdpa_ref_new``): fp32 matmul, mask
                            ``row + offset < col`` -> -inf, softmax, fp32 PV.
* ``tile_max_score``     <- ``tests/regression/test_onlyscore_correctness.py:32-76``
                            (``ref_tile_max_score``): raw q.k per 128-key tile,
                            causal -> -inf, max; layout ``[head, tile, token]``.
* ``sparse_attention``   <- ``tests/regression/test_sparse_attn.py:50-79``
                            (``sparse_ref``): gather selected logical pages,
                            mask on ORIGINAL key positions, softmax, PV.
* ``topk_select``        <- contract pinned by
                            ``tests/smoke/test_sparse_topk_forced.py:266-275``
                            (stable sort: score desc, index asc; emitted
                            ascending by index) and the forced-page / padding
                            rules of ``python/msa_for_sail/csrc/include/
                            sparse_topk_select.cuh:823-957,1410-1430``.
* ``lse_merge``          <- ``python/msa_for_sail/csrc/include/
                            sm80_fmha_reduction.hpp:133-215`` (weights
                            ``exp(lse_s - max)``; -inf LSE => weight 0 and the
                            partial is ignored).
* ``paged_to_contiguous``<- ``tests/regression/test_correctness.py:336-350``.
"""

from __future__ import annotations

import math
from typing import List, Optional, Sequence

import numpy as np
import torch

KV_TILE = 128  # max_score granularity: one value per 128 keys
FLT_MAX = float(np.finfo(np.float32).max)


def _as_list(x) -> List[int]:
    if isinstance(x, torch.Tensor):
        return [int(v) for v in x.reshape(-1).tolist()]
    return [int(v) for v in x]


# ---------------------------------------------------------------------------
# dense / ragged attention
# ---------------------------------------------------------------------------

def attention_single(q, k, v, h_q, h_k, causal=True, qo_offset=0, sm_scale=None,
                     return_lse=False, q_chunk=None):
    """One batch item.  q [q_len, h_q, d], k/v [kv_len, h_k, d] -> o [q_len, h_q, d] fp32.

    Same arithmetic as upstream ``_mha_ref_single`` but evaluated one KV head
    group at a time so that million-token keys fit in host memory (upstream
    materialises the GQA-expanded K and V in fp32).  Heads are grouped as
    ``(h_k, gqa_ratio)`` flattened into ``h_q``.
    Rows with no visible key give NaN in upstream (softmax of all -inf); here
    they are returned as 0 with LSE = -inf, which the upstream tests accept.
    """
    q_len, kv_len = q.shape[0], k.shape[0]
    d_v = v.shape[-1]
    g = h_q // h_k
    scale = (1.0 / math.sqrt(q.shape[-1])) if sm_scale is None else float(sm_scale)
    off = 0 if qo_offset is None else int(qo_offset)
    o = torch.zeros((q_len, h_q, d_v), dtype=torch.float32)
    lse = torch.full((q_len, h_q), -float("inf"), dtype=torch.float32)
    if q_len == 0 or kv_len == 0:
        return (o, lse) if return_lse else o
    if q_chunk is None:
        q_chunk = max(1, (1 << 24) // max(1, kv_len * g))
    col = torch.arange(kv_len)
    for hk in range(h_k):
        k_t = k[:, hk].float().t().contiguous()          # [d, kv_len]
        v_f = v[:, hk].float()                           # [kv_len, d_v]
        for s in range(0, q_len, q_chunk):
            e = min(s + q_chunk, q_len)
            q_c = q[s:e, hk * g:(hk + 1) * g].float()    # [qc, g, d]
            scores = (q_c.reshape(-1, q_c.shape[-1]) @ k_t) * scale   # [qc*g, kv]
            scores = scores.view(e - s, g, kv_len)
            if causal:
                row = torch.arange(s, e) + off
                invalid = row.unsqueeze(1) < col.unsqueeze(0)
                scores = scores.masked_fill(invalid.unsqueeze(1), -float("inf"))
            m = scores.max(dim=-1, keepdim=True).values
            m_safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
            p = torch.exp(scores - m_safe)
            l = p.sum(dim=-1, keepdim=True)
            out = (p.reshape(-1, kv_len) @ v_f).view(e - s, g, d_v)
            inv = torch.where(l > 0, 1.0 / l, torch.zeros_like(l))
            o[s:e, hk * g:(hk + 1) * g] = out * inv
            lse[s:e, hk * g:(hk + 1) * g] = torch.where(
                l > 0, m_safe + torch.log(l), torch.full_like(l, -float("inf"))).squeeze(-1)
    return (o, lse) if return_lse else o


def attention(q, k, v, qo_lens, kv_lens, h_q, h_k, causal=True, qo_offset=None,
              sm_scale=None, return_lse=False):
    """Ragged batch.  q [sum qo, h_q, d], k/v [sum kv, h_k, d] (fp32/bf16 CPU).

    ``qo_offset``: None -> bottom-right aligned (``kv - qo``), an int, or one
    value per batch item; row i sees key j iff ``i + offset >= j``.
    """
    qo_lens, kv_lens = _as_list(qo_lens), _as_list(kv_lens)
    outs, lses = [], []
    qs = ks = 0
    for b, (ql, kl) in enumerate(zip(qo_lens, kv_lens)):
        if qo_offset is None:
            off = kl - ql
        elif isinstance(qo_offset, int):
            off = qo_offset
        else:
            off = _as_list(qo_offset)[b]
        r = attention_single(q[qs:qs + ql], k[ks:ks + kl], v[ks:ks + kl], h_q, h_k,
                             causal=causal, qo_offset=off, sm_scale=sm_scale, return_lse=True)
        outs.append(r[0]); lses.append(r[1])
        qs += ql; ks += kl
    o = torch.cat(outs, 0) if outs else torch.zeros((0, h_q, v.shape[-1]))
    if return_lse:
        return o, (torch.cat(lses, 0) if lses else torch.zeros((0, h_q)))
    return o


# ---------------------------------------------------------------------------
# paged KV helpers
# ---------------------------------------------------------------------------

def paged_to_contiguous(pages, kv_indices, kv_lens, page_size, nhd=False):
    """Follow the flat page table and crop each sequence to its length.

    pages: HND ``[P, h_k, page, d]`` or NHD ``[P, page, h_k, d]``.
    Returns ragged ``[sum kv, h_k, d]``.
    """
    kv_lens = _as_list(kv_lens)
    idx = _as_list(kv_indices)
    outs, p0 = [], 0
    for kl in kv_lens:
        n = (kl + page_size - 1) // page_size
        sel = pages[torch.tensor(idx[p0:p0 + n], dtype=torch.long)] if n else pages[:0]
        if not nhd:
            sel = sel.permute(0, 2, 1, 3)                 # [n, page, h_k, d]
        outs.append(sel.reshape(n * page_size, sel.shape[2], sel.shape[3])[:kl])
        p0 += n
    return torch.cat(outs, 0)


# ---------------------------------------------------------------------------
# per-tile max score (proxy / indexer pass)
# ---------------------------------------------------------------------------

def tile_max_score(q, k, qo_lens, kv_lens, num_kv_heads, max_k_tiles, causal=True,
                   qo_offset=None):
    """``[h_q, max_k_tiles, total_q]`` fp32; raw (unscaled) q.k, -inf where masked/absent."""
    total_q, h_q, _ = q.shape
    g = h_q // num_kv_heads
    qo_lens, kv_lens = _as_list(qo_lens), _as_list(kv_lens)
    res = torch.full((h_q, max_k_tiles, total_q), -float("inf"), dtype=torch.float32)
    qs = ks = 0
    for b, (ql, kl) in enumerate(zip(qo_lens, kv_lens)):
        off = (kl - ql) if qo_offset is None else (
            qo_offset if isinstance(qo_offset, int) else _as_list(qo_offset)[b])
        n_tiles = (kl + KV_TILE - 1) // KV_TILE
        if ql and kl:
            qf = q[qs:qs + ql].float()                                    # [ql, h_q, d]
            kf = k[ks:ks + kl].float()                                    # [kl, h_k, d]
            s = torch.einsum("qhgd,khd->hgqk", qf.view(ql, num_kv_heads, g, -1), kf)
            s = s.reshape(h_q, ql, kl)
            if causal:
                qp = torch.arange(ql).unsqueeze(1) + off
                kp = torch.arange(kl).unsqueeze(0)
                s = s.masked_fill((qp < kp).unsqueeze(0), -float("inf"))
            pad = n_tiles * KV_TILE - kl
            if pad:
                s = torch.nn.functional.pad(s, (0, pad), value=-float("inf"))
            res[:, :n_tiles, qs:qs + ql] = s.view(h_q, ql, n_tiles, KV_TILE).max(-1).values.permute(0, 2, 1)
        qs += ql; ks += kl
    return res


# ---------------------------------------------------------------------------
# sparse (selected pages) attention
# ---------------------------------------------------------------------------

def sparse_attention(q, k_pages, v_pages, qo_lens, kv_lens, kv_indices, kv_block_indexes,
                     h_q, page_size=128, qo_offset=None, sm_scale=None, nhd=False,
                     return_lse=False):
    """Attention of each token over its own selected logical pages.

    q ``[T, h_q, d]``; pages HND ``[P, h_k, page, d]`` (or NHD); ``kv_indices``
    flat page table; ``kv_block_indexes [T, h_k, kbn]`` int, logical page
    numbers within the sequence, ascending, -1 padded.  Keys are masked by
    their ORIGINAL position ``page * page_size + j`` (causal and ``< kv_len``).
    Rows with nothing visible -> 0 (LSE -inf).
    """
    T = q.shape[0]
    h_k = k_pages.shape[2] if nhd else k_pages.shape[1]
    g = h_q // h_k
    d_v = v_pages.shape[-1]
    scale = (1.0 / math.sqrt(q.shape[-1])) if sm_scale is None else float(sm_scale)
    qo_lens, kv_lens = _as_list(qo_lens), _as_list(kv_lens)
    idx = torch.as_tensor(np.asarray(_as_list(kv_indices)), dtype=torch.long)
    bi = kv_block_indexes.to(torch.long).cpu()
    o = torch.zeros((T, h_q, d_v), dtype=torch.float32)
    lse = torch.full((T, h_q), -float("inf"), dtype=torch.float32)
    t = 0; p0 = 0
    for b, (ql, kl) in enumerate(zip(qo_lens, kv_lens)):
        off = (kl - ql) if qo_offset is None else (
            qo_offset if isinstance(qo_offset, int) else _as_list(qo_offset)[b])
        n_pages = (kl + page_size - 1) // page_size
        for i in range(ql):
            for hk in range(h_k):
                blocks = [int(x) for x in bi[t, hk].tolist() if x >= 0]
                if not blocks:
                    continue
                phys = idx[p0 + torch.tensor(blocks)]
                if nhd:
                    kg = k_pages[phys, :, hk].float().reshape(-1, k_pages.shape[-1])
                    vg = v_pages[phys, :, hk].float().reshape(-1, d_v)
                else:
                    kg = k_pages[phys, hk].float().reshape(-1, k_pages.shape[-1])
                    vg = v_pages[phys, hk].float().reshape(-1, d_v)
                pos = (torch.tensor(blocks).unsqueeze(1) * page_size
                       + torch.arange(page_size).unsqueeze(0)).reshape(-1)
                s = (q[t, hk * g:(hk + 1) * g].float() @ kg.t()) * scale      # [g, n]
                bad = (pos > i + off) | (pos >= kl)
                s = s.masked_fill(bad.unsqueeze(0), -float("inf"))
                m = s.max(-1, keepdim=True).values
                ms = torch.where(torch.isinf(m), torch.zeros_like(m), m)
                p = torch.exp(s - ms)
                l = p.sum(-1, keepdim=True)
                inv = torch.where(l > 0, 1.0 / l, torch.zeros_like(l))
                o[t, hk * g:(hk + 1) * g] = (p @ vg) * inv
                lse[t, hk * g:(hk + 1) * g] = torch.where(
                    l > 0, ms + torch.log(l), torch.full_like(l, -float("inf"))).squeeze(-1)
            t += 1
        p0 += n_pages
    return (o, lse) if return_lse else o


# ---------------------------------------------------------------------------
# top-k page selection
# ---------------------------------------------------------------------------

def _ord_key(x: torch.Tensor) -> torch.Tensor:
    """Integer key of an fp32 score, as int64, whose order is the order a stable descending
    ``torch.sort`` gives the scores: the upstream ``float_to_ord`` map
    (``sparse_topk_select.cuh:186-196``) with the two cases in which bit order and value order
    differ folded in -- -0.0 and +0.0 compare equal (one key), every NaN ranks above +inf and all
    NaNs tie (one key)."""
    x = x.contiguous() + 0.0                                  # -0.0 + 0.0 = +0.0
    bits = x.view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    neg = (bits >> 31) & 1
    key = torch.where(neg == 1, (~bits) & 0xFFFFFFFF, bits | 0x80000000)
    return torch.where(torch.isnan(x), torch.full_like(key, 0xFFFFFFFF), key)


def topk_select(max_score, topk, num_valid_pages=None, force_begin_blocks=0,
                force_end_blocks=0):
    """``[H, K, T]`` scores -> ``[T, H, topk]`` int32.

    Per (head, token) row, over pages ``[0, nvp)``: pages ``[0, fb)`` and
    ``[nvp - fe, nvp)`` rank as FLT_MAX; pick the ``topk`` best by
    (key desc, index asc); emit ascending by index.  ``nvp <= topk`` gives the
    identity list ``[0..nvp)`` padded with -1.
    """
    H, K, T = max_score.shape
    nvp = K if num_valid_pages is None else int(num_valid_pages)
    out = torch.full((T, H, topk), -1, dtype=torch.int32)
    if nvp <= topk:
        out[:, :, :nvp] = torch.arange(nvp, dtype=torch.int32)
        return out
    s = max_score[:, :nvp, :].float().clone()
    fe_start = nvp - force_end_blocks if force_end_blocks <= nvp else 0
    if force_begin_blocks:
        s[:, :force_begin_blocks, :] = FLT_MAX
    if force_end_blocks:
        s[:, fe_start:nvp, :] = FLT_MAX
    key = _ord_key(s)                                       # [H, nvp, T] int64
    # composite key: higher ord first, lower index first among equals
    comp = key * (1 << 20) + ((1 << 20) - 1 - torch.arange(nvp).view(1, nvp, 1))
    sel = comp.topk(topk, dim=1).indices                    # [H, topk, T]
    sel = sel.sort(dim=1).values
    out[:] = sel.permute(2, 0, 1).to(torch.int32)
    return out


# ---------------------------------------------------------------------------
# split-KV merge
# ---------------------------------------------------------------------------

def lse_merge(partial_o, partial_lse, out_scale=1.0, return_lse=False):
    """partial_o ``[S, T, H, D]`` (each already normalised), partial_lse ``[S, T, H]``
    natural-log LSE (-inf = split saw nothing, its partial is ignored even if it
    holds NaN/garbage).  Returns ``[T, H, D]`` fp32 (and the merged LSE)."""
    po = partial_o.float()
    pl = partial_lse.float()
    mx = pl.max(dim=0, keepdim=True).values
    mx_safe = torch.where(torch.isinf(mx), torch.zeros_like(mx), mx)
    w = torch.where(torch.isinf(pl) & (pl < 0), torch.zeros_like(pl), torch.exp(pl - mx_safe))
    sw = w.sum(0)
    po = torch.where((w == 0).unsqueeze(-1), torch.zeros_like(po), po)
    acc = (w.unsqueeze(-1) * po).sum(0)
    inv = torch.where(sw > 0, 1.0 / sw, torch.zeros_like(sw))
    o = acc * inv.unsqueeze(-1) * out_scale
    if return_lse:
        lse = torch.where(sw > 0, mx_safe.squeeze(0) + torch.log(sw),
                          torch.full_like(sw, -float("inf")))
        return o, lse
    return o


# ---------------------------------------------------------------------------
# fp8 helpers
# ---------------------------------------------------------------------------

def quantize_e4m3(x: torch.Tensor, scale=None):
    """Plain cast (scale None) or per-kv-head scaled cast to float8_e4m3fn.
    Returns (fp8 tensor, de-quantised fp32 tensor)."""
    if scale is None:
        q8 = x.float().to(torch.float8_e4m3fn)
        return q8, q8.float()
    q8 = (x.float() / scale).clamp(-448, 448).to(torch.float8_e4m3fn)
    return q8, q8.float() * scale
