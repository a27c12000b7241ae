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
