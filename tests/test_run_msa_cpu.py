"""The parameter-line format of the single-case reproducer (no GPU needed for the parser)."""
import importlib.util
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _mod():
    path = os.path.join(ROOT, "msa-for-sail_b200", "benchmarks", "run_msa.py")
    spec = importlib.util.spec_from_file_location("run_msa", path)
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


def test_parse_accepts_both_key_spellings_and_round_trips():
    m = _mod()
    emitted = ("[MSA] --format=dtype:bf16,batch_size:2,seqlen_q:[1,1],seqlen_k:[4096,700],qo_offset:[4095,699],"
               "num_heads:64,num_heads_kv:8,head_dim:128,head_dim_v:128,num_kv_splits:1,is_paged:1,page_size:128,"
               "causal:1,sm_scale:0.088388,sparse_mode:Sparse,topk:16.")
    cfg = m.parse_format(emitted)
    assert cfg["num_qo_heads"] == 64 and cfg["num_kv_heads"] == 8 and cfg["kv_block_num"] == 16
    assert cfg["seqlen_k"] == [4096, 700] and cfg["sparse_mode"] == "Sparse" and abs(cfg["sm_scale"] - 0.088388) < 1e-9
    assert m.parse_format(m.format_line(cfg)) == cfg
    assert "num_qo_heads:64" in m.format_line(cfg)


def test_defaults_and_work_model():
    m = _mod()
    cfg = m.parse_format("--format=seqlen_q:[2],seqlen_k:[256],num_qo_heads:4")
    assert cfg["num_kv_heads"] == 4 and cfg["sparse_mode"] == "Off" and cfg["is_paged"] == 1
    flops, nbytes = m.flops_and_bytes(cfg)
    # causal, offset 254: token 0 sees 255 keys, token 1 sees 256
    assert flops == 4 * (255 + 256) * 4 * 128
    assert nbytes == 2 * 4 * 128 * 2 + 256 * 4 * 128 * 2 * 2 + 2 * 4 * 128 * 2
    cfg2 = m.parse_format("--format=seqlen_q:[1],seqlen_k:[4096],num_qo_heads:8,num_kv_heads:1,kv_block_num:4")
    assert cfg2["sparse_mode"] == "Sparse"
    assert m.flops_and_bytes(cfg2)[0] == 8 * 512 * 4 * 128


def test_sweep_sections_enumerate_the_upstream_tables():
    m = _mod()
    rows = list(m.sweep_cases("prefill", seqs=(8192, 16384), tp=(1, 4)))
    assert [(c["num_qo_heads"], c["num_kv_heads"], c["seqlen_q"][0]) for _, c, _ in rows] == [
        (64, 4, 8192), (64, 4, 16384), (16, 1, 8192), (16, 1, 16384)]
    assert all(not c["is_paged"] and c["sparse_mode"] == "Off" and not mbu for _, c, mbu in rows)
    rows = list(m.sweep_cases("sparse_decode", decode_k=(8192,), decode_b=(32,), topk=8))
    assert [c["sparse_mode"] for _, c, _ in rows] == ["Off", "Sparse"] and all(mbu for _, _, mbu in rows)
    assert rows[1][1]["kv_block_num"] == 8 and rows[1][1]["seqlen_q"] == [8] * 32 and rows[1][1]["selection"] == "first"
    assert [len(list(m.sweep_cases(s_))) > 0 for s_ in m.SWEEP_SECTIONS] == [True] * 6
    assert m.TSV_HEADER[:4] == ["q_len", "kv_len", "dtype", "batch_size"] and len(m.TSV_HEADER) == 13 == len(m.TABLE)
    # a sparse row counts the keys it reads, a dense row the causal triangle
    sp = rows[1][1]
    assert m.sweep_work(sp)[0] == 32 * 64 * (8 * 8 * 128) * 256 * 2
    dn = list(m.sweep_cases("paged_prefill", seqs=(256,)))[0][1]
    assert m.sweep_work(dn)[0] == 64 * (256 * 256 - 256 * 255 // 2) * 256 * 2
