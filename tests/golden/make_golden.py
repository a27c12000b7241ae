#!/usr/bin/env python3
"""Generate the golden fixtures in this directory from the UPSTREAM reference.

Run once, in a container that has the upstream tree checked out (path given by
``--reference`` or the environment variable ``MSA_REFERENCE_DIR``); the resulting ``*.npz`` files are
committed so that the test-suite never needs the upstream tree.

Every expected value here is produced by the upstream project's own PyTorch
reference code, imported unmodified and executed on CPU tensors:

* ``tests/ref_attn.py``                              ``sdpa_ref_new``
* ``tests/regression/test_onlyscore_correctness.py`` ``ref_tile_max_score``
* ``tests/regression/test_sparse_attn.py``           ``sparse_ref``
* the top-k contract of ``tests/smoke/test_sparse_topk_forced.py:266-275``
  (stable descending sort, first k, re-sorted ascending) evaluated with the
  same torch calls on that file's seven score distributions (shrunk to K=512), plus two more
  that the contract implies but the file does not exercise: zeros of both signs, and NaN.

bf16 tensors are stored as their uint16 bit patterns.
"""
import argparse
import importlib
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def bf16_bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("MSA_REFERENCE_DIR"), required="MSA_REFERENCE_DIR" not in os.environ,
                    help="directory of the upstream checkout")
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.reference, "tests"))
    sys.path.insert(0, os.path.join(args.reference, "tests", "regression"))
    ref_attn = importlib.import_module("ref_attn")
    onlyscore = importlib.import_module("test_onlyscore_correctness")
    sparse_mod = importlib.import_module("test_sparse_attn")

    # ---------------- dense attention (uniform batch; sdpa_ref_new wants 4-D) --------
    g = torch.Generator().manual_seed(0)
    cases = []
    for name, (b, ql, kl, hq, hk, off) in {
        "prefill": (2, 96, 96, 4, 2, None),
        "chunked": (2, 40, 300, 8, 1, None),
        "decode": (3, 1, 257, 8, 2, None),
        "offset": (1, 64, 200, 4, 4, 17),
    }.items():
        q = torch.randn(b, ql, hq, 128, generator=g).to(torch.bfloat16)
        k = torch.randn(b, kl, hk, 128, generator=g).to(torch.bfloat16)
        v = torch.randn(b, kl, hk, 128, generator=g).to(torch.bfloat16)
        qo_off = (kl - ql) if off is None else off
        o = ref_attn.sdpa_ref_new(q, k, v, hq, hk, causal=True, qo_offset=qo_off)
        cases.append(name)
        np.savez_compressed(
            os.path.join(HERE, f"attn_{name}.npz"),
            q=bf16_bits(q), k=bf16_bits(k), v=bf16_bits(v), o=o.numpy(),
            meta=np.array([b, ql, kl, hq, hk, qo_off], dtype=np.int64))

    # ---------------- per-tile max score (ragged) -------------------------------------
    g = torch.Generator().manual_seed(1)
    qo_lens = torch.tensor([37, 5, 130], dtype=torch.int32)
    kv_lens = torch.tensor([300, 129, 130], dtype=torch.int32)
    hq, hk = 4, 2
    q = torch.randn(int(qo_lens.sum()), hq, 128, generator=g).to(torch.bfloat16)
    k = torch.randn(int(kv_lens.sum()), hk, 128, generator=g).to(torch.bfloat16)
    max_k_tiles = 128
    ms = onlyscore.ref_tile_max_score(q, k, qo_lens, kv_lens, hk, max_k_tiles, causal=True)
    off_t = torch.tensor([100, 124, 0], dtype=torch.int32)
    ms_off = onlyscore.ref_tile_max_score(q, k, qo_lens, kv_lens, hk, max_k_tiles, causal=True,
                                          qo_offset_tensor=off_t)
    np.savez_compressed(
        os.path.join(HERE, "maxscore_ragged.npz"),
        q=bf16_bits(q), k=bf16_bits(k), qo_lens=qo_lens.numpy(), kv_lens=kv_lens.numpy(),
        ms=ms[:, :4].numpy(), ms_off=ms_off[:, :4].numpy(), off=off_t.numpy(),
        meta=np.array([hq, hk, max_k_tiles], dtype=np.int64))

    # ---------------- sparse attention (paged, shuffled table) ------------------------
    g = torch.Generator().manual_seed(2)
    page = 128
    qo_l = [3, 2]
    kv_l = [5 * page, 7 * page]
    hq, hk, kbn = 4, 2, 3
    n_pages = sum(x // page for x in kv_l)
    k_pages = torch.randn(n_pages, hk, page, 128, generator=g).to(torch.bfloat16)
    v_pages = torch.randn(n_pages, hk, page, 128, generator=g).to(torch.bfloat16)
    q = torch.randn(sum(qo_l), hq, 128, generator=g).to(torch.bfloat16)
    # upstream sparse_ref indexes pages as page_off + blk (identity page table) and
    # takes one block list per (batch, kv_head) shared by the batch's tokens
    per_batch_blocks = [[[0, 2, 4], [1, 3, 4]], [[0, 5, 6], [2, 3, 6]]]
    indptr = [0, 5, 12]
    qo_offsets = [kv_l[i] - qo_l[i] for i in range(2)]
    o = sparse_mod.sparse_ref(q, k_pages, v_pages, qo_l, indptr, per_batch_blocks, hq, hk, page,
                              qo_offsets, 128, torch.device("cpu"))
    np.savez_compressed(
        os.path.join(HERE, "sparse_small.npz"),
        q=bf16_bits(q), k_pages=bf16_bits(k_pages), v_pages=bf16_bits(v_pages),
        o=bf16_bits(o), qo_lens=np.array(qo_l), kv_lens=np.array(kv_l),
        blocks=np.array(per_batch_blocks, dtype=np.int32),
        meta=np.array([hq, hk, kbn, page], dtype=np.int64))

    # ---------------- top-k contract on the upstream tie-break distributions ----------
    H, K, T, topk, seed = 4, 512, 8, 16, 42

    def build(kind):
        gg = torch.Generator().manual_seed(seed)
        if kind == "randn":
            return torch.randn(H, K, T, generator=gg)
        order = torch.rand(H, K, T, generator=gg).argsort(dim=1)
        if kind in ("tie32", "tie64"):
            n_tie = 25 if kind == "tie32" else 50
            m = torch.full((H, K, T), float("-inf"))
            m.scatter_(1, order[:, :7, :], 2.0)
            m.scatter_(1, order[:, 7:7 + n_tie, :], -1.0)
            return m
        if kind == "uniform-sea-random":
            m = torch.full((H, K, T), float("-inf"))
            m.scatter_(1, order[:, :7, :], 2.0)
            return m
        if kind == "uniform-sea-prefix":
            m = torch.full((H, K, T), float("-inf"))
            m[:, :7, :] = torch.randn(H, 7, T, generator=gg)
            return m
        if kind == "zero-sea":
            m = torch.zeros(H, K, T)
            m.scatter_(1, order[:, :7, :], 2.0)
            return m
        if kind == "nonuniform-sea":
            m = torch.ones(H, K, T)
            m[:, 1::2, :] = 1.0078125
            m.scatter_(1, order[:, :7, :], 2.0)
            return m
        # two distributions beyond the upstream file's seven, evaluated with the same stable-sort calls:
        if kind == "signed-zero-sea":                # -0.0 and +0.0 compare equal: they tie, the lower index wins
            sign = torch.rand(H, K, T, generator=gg) < 0.5
            m = torch.where(sign, torch.tensor(-0.0), torch.tensor(0.0))
            m.scatter_(1, order[:, :7, :], 2.0)
            m.scatter_(1, order[:, 7:40, :], -1.0)
            return m
        if kind == "nan-sprinkled":                  # torch orders NaN above every number, NaNs tie among themselves
            m = torch.randn(H, K, T, generator=gg)
            m.scatter_(1, order[:, :5, :], float("nan"))
            return m
        raise ValueError(kind)

    kinds = ["randn", "tie32", "tie64", "uniform-sea-random", "uniform-sea-prefix",
             "zero-sea", "nonuniform-sea", "signed-zero-sea", "nan-sprinkled"]
    blob = {}
    for kind in kinds:
        m = build(kind).to(torch.bfloat16)          # bf16 path is the exact-index contract
        _, order = m.float().sort(dim=1, descending=True, stable=True)
        ref = order[:, :topk, :].sort(dim=1).values.permute(2, 0, 1)
        blob[kind.replace("-", "_") + "_in"] = bf16_bits(m)
        blob[kind.replace("-", "_") + "_out"] = ref.numpy().astype(np.int32)
    np.savez_compressed(os.path.join(HERE, "topk_dist.npz"), **blob)
    print("wrote fixtures to", HERE)


if __name__ == "__main__":
    main()
