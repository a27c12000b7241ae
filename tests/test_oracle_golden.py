"""Pin the CPU oracle against outputs of the upstream reference functions
(fixtures written by tests/golden/make_golden.py)."""
import numpy as np
import torch

from conftest import from_bf16_bits, load_golden
from oracle import msa_oracle as orc


def _attn_case(name):
    z = load_golden(f"attn_{name}.npz")
    b, ql, kl, hq, hk, off = [int(x) for x in z["meta"]]
    q = from_bf16_bits(z["q"]).reshape(b * ql, hq, 128)
    k = from_bf16_bits(z["k"]).reshape(b * kl, hk, 128)
    v = from_bf16_bits(z["v"]).reshape(b * kl, hk, 128)
    o = orc.attention(q, k, v, [ql] * b, [kl] * b, hq, hk, causal=True, qo_offset=off)
    return o, torch.from_numpy(z["o"])


def test_attention_matches_upstream_sdpa_ref():
    for name in ("prefill", "chunked", "decode", "offset"):
        o, ref = _attn_case(name)
        assert o.shape == ref.shape
        assert torch.allclose(o, ref, atol=2e-5, rtol=1e-4), name


def test_tile_max_score_matches_upstream():
    z = load_golden("maxscore_ragged.npz")
    hq, hk, mkt = [int(x) for x in z["meta"]]
    q = from_bf16_bits(z["q"]); k = from_bf16_bits(z["k"])
    ms = orc.tile_max_score(q, k, z["qo_lens"], z["kv_lens"], hk, mkt, causal=True)
    ref = torch.from_numpy(z["ms"])
    assert torch.isinf(ms[:, 4:]).all()
    got = ms[:, :4]
    assert torch.equal(torch.isinf(got), torch.isinf(ref))
    fin = ~torch.isinf(ref)
    assert torch.allclose(got[fin], ref[fin], atol=1e-4, rtol=1e-5)
    ms2 = orc.tile_max_score(q, k, z["qo_lens"], z["kv_lens"], hk, mkt, causal=True,
                             qo_offset=[int(x) for x in z["off"]])[:, :4]
    ref2 = torch.from_numpy(z["ms_off"])
    assert torch.equal(torch.isinf(ms2), torch.isinf(ref2))
    fin = ~torch.isinf(ref2)
    assert torch.allclose(ms2[fin], ref2[fin], atol=1e-4, rtol=1e-5)


def test_sparse_attention_matches_upstream_sparse_ref():
    z = load_golden("sparse_small.npz")
    hq, hk, kbn, page = [int(x) for x in z["meta"]]
    q = from_bf16_bits(z["q"])
    kp = from_bf16_bits(z["k_pages"]); vp = from_bf16_bits(z["v_pages"])
    qo_lens = [int(x) for x in z["qo_lens"]]; kv_lens = [int(x) for x in z["kv_lens"]]
    blocks = z["blocks"]                       # [B, hk, kbn]
    bi = torch.cat([torch.from_numpy(blocks[b]).unsqueeze(0).expand(qo_lens[b], hk, kbn)
                    for b in range(len(qo_lens))], 0)
    n_pages = sum(x // page for x in kv_lens)
    o = orc.sparse_attention(q, kp, vp, qo_lens, kv_lens, list(range(n_pages)), bi, hq,
                             page_size=page)
    ref = from_bf16_bits(z["o"]).float()
    assert torch.allclose(o, ref, atol=1e-2, rtol=1e-2)     # upstream rounds to bf16
    assert (o.to(torch.bfloat16).float() - ref).abs().max() <= 2 ** -7 * ref.abs().max()


def test_topk_matches_upstream_contract():
    z = load_golden("topk_dist.npz")
    kinds = sorted(k[:-3] for k in z.files if k.endswith("_in"))
    assert len(kinds) == 9 and "signed_zero_sea" in kinds and "nan_sprinkled" in kinds
    for kind in kinds:
        m = from_bf16_bits(z[kind + "_in"]).float()
        got = orc.topk_select(m, 16, num_valid_pages=m.shape[1])
        assert np.array_equal(got.numpy(), z[kind + "_out"]), kind


def test_topk_edges():
    m = torch.randn(2, 128, 5)
    out = orc.topk_select(m, 16, num_valid_pages=9)
    assert out.shape == (5, 2, 16)
    assert (out[:, :, :9] == torch.arange(9, dtype=torch.int32)).all() and (out[:, :, 9:] == -1).all()
    m[:, 40:, :] = -float("inf")
    out = orc.topk_select(m, 16, num_valid_pages=100, force_begin_blocks=2, force_end_blocks=3)
    for t in range(5):
        for h in range(2):
            row = set(out[t, h].tolist())
            assert {0, 1, 97, 98, 99} <= row and -1 not in row


def test_lse_merge_equals_unsplit():
    g = torch.Generator().manual_seed(3)
    q = torch.randn(4, 4, 128, generator=g); k = torch.randn(300, 2, 128, generator=g)
    v = torch.randn(300, 2, 128, generator=g)
    full, lse_full = orc.attention(q, k, v, [4], [300], 4, 2, qo_offset=296, return_lse=True)
    parts, lses = [], []
    for s, e in ((0, 128), (128, 256), (256, 300)):
        # keys of a split keep their original positions: shift the offset
        o, l = orc.attention(q, k[s:e], v[s:e], [4], [e - s], 4, 2, qo_offset=296 - s, return_lse=True)
        parts.append(o); lses.append(l)
    parts.append(torch.full_like(parts[0], float("nan"))); lses.append(torch.full_like(lses[0], -float("inf")))
    o, l = orc.lse_merge(torch.stack(parts), torch.stack(lses), return_lse=True)
    assert torch.allclose(o, full, atol=1e-5, rtol=1e-5)
    assert torch.allclose(l, lse_full, atol=1e-5, rtol=1e-5)
