"""Case builders and comparison helpers shared by the GPU parity tests."""
import math

import numpy as np
import torch

from conftest import cosine
from oracle import msa_oracle as orc

BF16_MAX_ABS = 2e-2      # bf16 outputs: max-abs error bound
BF16_COS = 0.9999        # bf16 outputs: cosine bound
FP8_COS = 0.999          # e4m3 operands: cosine bound
SCORE_REL = 1e-2         # max_score: relative bound


def gen(seed):
    return torch.Generator().manual_seed(seed)


def randn_bf16(g, *shape, scale=1.0):
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16)


def make_paged(g, kv_lens, h_k, page_size, nhd=False, extra_pages=3, scale=1.0, dtype=torch.bfloat16):
    """Random K/V page pools + a shuffled flat page table covering every sequence."""
    pages_per = [(kl + page_size - 1) // page_size for kl in kv_lens]
    n_pages = sum(pages_per) + extra_pages
    shape = (n_pages, page_size, h_k, 128) if nhd else (n_pages, h_k, page_size, 128)
    k = (torch.randn(*shape, generator=g) * scale).to(dtype)
    v = (torch.randn(*shape, generator=g) * scale).to(dtype)
    table = torch.randperm(n_pages, generator=g)[:sum(pages_per)].to(torch.int32)
    return k, v, table


def check_out(o, ref, name, cos_min=BF16_COS, max_abs=BF16_MAX_ABS):
    o = o.float().cpu()
    ref = ref.float()
    assert o.shape == ref.shape, (name, o.shape, ref.shape)
    assert torch.isfinite(o).all(), f"{name}: non-finite output"
    c = cosine(o, ref)
    err = (o - ref).abs().max().item() if o.numel() else 0.0
    assert c >= cos_min, f"{name}: cosine {c:.6f} < {cos_min}"
    if max_abs is not None:
        assert err <= max_abs, f"{name}: max-abs {err:.4f} > {max_abs}"
    return c, err


def check_score(ms, ref, name, rel=SCORE_REL, bf16=False):
    ms = ms.float().cpu()
    assert ms.shape == ref.shape, (name, ms.shape, ref.shape)
    inf_ref = torch.isinf(ref) & (ref < 0)
    assert torch.equal(torch.isinf(ms) & (ms < 0), inf_ref), f"{name}: -inf pattern differs"
    fin = ~inf_ref
    if fin.any():
        a, b = ms[fin], ref[fin]
        if bf16:
            b = b.to(torch.bfloat16).float()
            ulp = torch.pow(2.0, torch.floor(torch.log2(b.abs().clamp_min(1e-30))) - 7)
            assert ((a - b).abs() <= ulp.clamp_min(1e-2)).all(), f"{name}: bf16 max_score off by > 1 ulp"
        else:
            tol = rel * b.abs().clamp_min(1.0)
            bad = (a - b).abs() > tol
            assert not bad.any(), f"{name}: max_score rel err {((a - b).abs() / b.abs().clamp_min(1.0)).max():.4g}"


def random_blocks(g, qo_lens, kv_lens, offsets, h_k, kbn, page_size=128, pad_prob=0.3):
    """Per-token ascending logical page lists, -1 padded: [T, h_k, kbn] int32.  Pages are drawn
    from those at least partly visible to the token (plus, sometimes, one future page)."""
    rows = []
    for b, (ql, kl) in enumerate(zip(qo_lens, kv_lens)):
        n_pages = (kl + page_size - 1) // page_size
        for i in range(ql):
            vis = min(n_pages, (i + offsets[b]) // page_size + 2)
            vis = max(1, min(vis, n_pages))
            per_head = []
            for _ in range(h_k):
                n = min(kbn, vis)
                if torch.rand(1, generator=g).item() < pad_prob:
                    n = max(1, int(torch.randint(1, n + 1, (1,), generator=g).item()))
                sel = torch.randperm(vis, generator=g)[:n].sort().values.tolist()
                per_head.append(sel + [-1] * (kbn - n))
            rows.append(per_head)
    return torch.tensor(rows, dtype=torch.int32).reshape(-1, h_k, kbn)
