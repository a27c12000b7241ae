#!/usr/bin/env python3
"""Re-run one `fmha_sail` call from its parameter line, optionally timed.

The parameter line is what the library prints for every `fmha_sail` call when the environment
variable ``MSA_SHOW_PARAMS=1`` (or the upstream name ``PPU_LIB_SHOW_PARAMS=1``) is set::

    [MSA] --format=dtype:bf16,batch_size:2,seqlen_q:[1,1],seqlen_k:[4096,700],qo_offset:[4095,699],\
num_qo_heads:64,num_kv_heads:8,head_dim_qk:128,head_dim_vo:128,num_kv_splits:1,is_paged:1,\
page_size:128,causal:1,sm_scale:0.088388,sparse_mode:Off,kv_block_num:0.

Same role and line format as the upstream tool (benchmarks/run_msa.py:1-69, emitter
csrc/msa_profiling_interface.hpp:99-157).  Upstream's emitter and parser disagree on some keys
(`num_heads` / `num_qo_heads`, `num_heads_kv` / `num_kv_heads`, `head_dim` / `head_dim_qk`,
`head_dim_v` / `head_dim_vo`, `topk` / `kv_block_num`): both spellings are accepted here.

Only the call's shape travels in the line, so the tensors are random.  sparse_mode: Off (O only),
Full (O and max_score), OnlyScore (max_score only), Sparse (O over kv_block_num selected pages).

    python run_msa.py --format "<line>"            # run once
    python run_msa.py --format "<line>" --bench    # time it; TFLOP/s and GB/s against the B200 peaks
    python run_msa.py --caselist cases.txt [--case_idx N]

``--sweep`` prints the tables of the upstream sweep benchmark (benchmarks/bench_sparse_attention_ops.py:
341-439): sections prefill (ragged dense, head presets TP1 64/4, TP2 32/2, TP4 16/1), paged_prefill,
sparse_prefill (the first top-k pages for every token), decode (4 query tokens, 64/4 heads), paged_decode,
sparse_decode (8 query tokens; a paged dense row and a sparse row per shape), with the upstream columns; ``-o``
writes the same rows tab-separated under the upstream header.  Each row is timed with a cold L2 (a 256 MB
buffer is rewritten before every iteration), median and standard deviation over the iterations.

    python run_msa.py --sweep [--sections prefill,sparse_decode] [--dtype bf16|fp8] [--seqs 8192,32768]
                      [--tp 1,2,4] [--decode-k 8192,65536] [--decode-b 32,64] [--topk 16] [-o sweep.tsv]
"""
import argparse
import json
import math
import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(os.path.dirname(HERE), "python"))

ALIASES = {"num_heads": "num_qo_heads", "num_heads_kv": "num_kv_heads", "head_dim": "head_dim_qk",
           "head_dim_v": "head_dim_vo", "topk": "kv_block_num"}
# nominal B200 figures, as upstream's table has them; --peaks takes measured ones
PEAKS = {"bf16_tflops": 2250.0, "fp8_tflops": 4500.0, "hbm_gbs": 8000.0}


def _value(text):
    text = text.strip()
    if text.startswith("["):
        return [int(x) for x in json.loads(text)]
    for conv in (int, float):
        try:
            return conv(text)
        except ValueError:
            pass
    return text


def parse_format(line):
    """'[MSA] --format=k:v,k:[..],k:v.' -> dict with the canonical key names."""
    body = re.sub(r"^.*?--format=", "", line).strip()
    if body.endswith("."):
        body = body[:-1]
    cfg = {}
    for key, val in re.findall(r"(\w+):(\[.*?\]|[^,]*?)(?=,\w+:|$)", body):
        cfg[ALIASES.get(key, key)] = _value(val)
    for need in ("seqlen_q", "seqlen_k", "num_qo_heads"):
        if need not in cfg:
            raise ValueError(f"parameter line has no '{need}': {line!r}")
    cfg.setdefault("num_kv_heads", cfg["num_qo_heads"])
    cfg.setdefault("dtype", "bf16")
    cfg.setdefault("batch_size", len(cfg["seqlen_q"]))
    cfg.setdefault("is_paged", 1)
    cfg.setdefault("page_size", 128)
    cfg.setdefault("causal", 1)
    cfg.setdefault("num_kv_splits", -1)
    cfg.setdefault("kv_block_num", 0)
    cfg.setdefault("sparse_mode", "Sparse" if cfg["kv_block_num"] > 0 else "Off")
    cfg.setdefault("head_dim_qk", 128)
    cfg.setdefault("head_dim_vo", 128)
    return cfg


def format_line(cfg):
    """The inverse of parse_format (what the library prints)."""
    def one(v):
        if isinstance(v, (list, tuple)):
            return "[" + ",".join(str(int(x)) for x in v) + "]"
        if isinstance(v, float):
            return f"{v:.6f}"
        return str(v)
    keys = ("dtype", "batch_size", "seqlen_q", "seqlen_k", "qo_offset", "num_qo_heads", "num_kv_heads", "head_dim_qk",
            "head_dim_vo", "num_kv_splits", "is_paged", "page_size", "causal", "sm_scale", "sparse_mode", "kv_block_num")
    return "[MSA] --format=" + ",".join(f"{k}:{one(cfg[k])}" for k in keys if k in cfg) + "."


def flops_and_bytes(cfg):
    """Algorithmic FLOPs and minimal HBM bytes of the call (upstream bench_utils.py:125-131)."""
    hq, hk = cfg["num_qo_heads"], cfg["num_kv_heads"]
    e = 1 if cfg["dtype"] in ("fp8", "e4m3") else 2
    sq, sk = cfg["seqlen_q"], cfg["seqlen_k"]
    offs = cfg.get("qo_offset") or [k - q for q, k in zip(sq, sk)]
    mode, kbn, page = cfg["sparse_mode"], cfg["kv_block_num"], cfg["page_size"]
    pairs = 0                                              # visible (query, key) pairs per head
    for q, k, o in zip(sq, sk, offs):
        for i in range(q):
            vis = min(k, i + o + 1) if cfg["causal"] else k
            pairs += min(vis, kbn * page) if mode == "Sparse" else max(vis, 0)
    per_pair = 2 * 128 if mode == "OnlyScore" else 4 * 128
    flops = hq * pairs * per_pair
    total_q = sum(sq)
    kv_tokens = total_q * kbn * page if mode == "Sparse" else sum(sk)
    kv_bytes = kv_tokens * hk * 128 * e * (1 if mode == "OnlyScore" else 2)
    nbytes = total_q * hq * 128 * e + kv_bytes + (0 if mode == "OnlyScore" else total_q * hq * 128 * 2)
    return flops, nbytes


def build_case(cfg):
    """Random tensors, plan and the call of one case: returns (callable, plan)."""
    import torch
    import msa_for_sail as msa
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(0)
    fp8 = cfg["dtype"] in ("fp8", "e4m3")
    dt = torch.float8_e4m3fn if fp8 else torch.bfloat16
    hq, hk = cfg["num_qo_heads"], cfg["num_kv_heads"]
    sq, sk = cfg["seqlen_q"], cfg["seqlen_k"]
    mode, kbn, page = cfg["sparse_mode"], cfg["kv_block_num"], cfg["page_size"]
    paged = bool(cfg["is_paged"])
    total_q = sum(sq)
    q = torch.randn(total_q, hq, 128, device=dev, generator=g, dtype=torch.bfloat16).to(dt)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32)
    kw = {}
    if paged:
        pages = [(k + page - 1) // page for k in sk]
        n_pages = sum(pages)
        k = torch.randn(n_pages, hk, page, 128, device=dev, generator=g, dtype=torch.bfloat16).to(dt)
        v = torch.randn(n_pages, hk, page, 128, device=dev, generator=g, dtype=torch.bfloat16).to(dt)
        kw["kv_indices"] = torch.randperm(n_pages, device=dev, generator=g).to(torch.int32)
    else:
        k = torch.randn(sum(sk), hk, 128, device=dev, generator=g, dtype=torch.bfloat16).to(dt)
        v = torch.randn(sum(sk), hk, 128, device=dev, generator=g, dtype=torch.bfloat16).to(dt)
    offs = cfg.get("qo_offset")
    plan = msa.fmha_sail_plan(i32(sq), i32(sk), hq, num_kv_heads=hk, page_size=page if paged else -1,
                              num_kv_splits=cfg["num_kv_splits"], causal=bool(cfg["causal"]),
                              qo_offset=i32(offs) if offs else None, use_fp8_kvcache=fp8,
                              output_maxscore=mode in ("Full", "OnlyScore"),
                              kv_block_num=kbn if mode == "Sparse" else -1)
    if mode == "Sparse" and cfg.get("selection") == "first":      # the sweep's choice: pages 0 .. k-1 for every token
        n_sel = min(kbn, min((kl + page - 1) // page for kl in sk))
        sel = torch.full((total_q, hk, kbn), -1, dtype=torch.int32, device=dev)
        sel[:, :, :n_sel] = torch.arange(n_sel, dtype=torch.int32, device=dev)
        kw["kv_block_indexes"] = sel
    elif mode == "Sparse":
        rows = []
        for b, (ql, kl) in enumerate(zip(sq, sk)):
            o = offs[b] if offs else kl - ql
            for i in range(ql):
                vis_pages = max(1, min((kl + page - 1) // page, (i + o) // page + 1))
                sel = torch.randperm(vis_pages, generator=torch.Generator().manual_seed(b * 131071 + i))[:kbn].sort().values
                rows.append(torch.cat([sel, torch.full((kbn - sel.numel(),), -1)]))
        kw["kv_block_indexes"] = torch.stack(rows).to(torch.int32).view(total_q, 1, kbn).expand(total_q, hk, kbn).contiguous().to(dev)
    if "sm_scale" in cfg:
        kw["sm_scale"] = float(cfg["sm_scale"])
    if mode == "OnlyScore":
        kw["output_o"] = False
    if mode in ("Off", "Sparse"):
        kw["output_maxscore"] = False

    def fn():
        return msa.fmha_sail(q, k, v, plan, **kw)

    return fn, plan


def build_and_run(cfg, bench=False, iters=20, peaks=None):
    import torch
    fn, _ = build_case(cfg)
    mode, fp8 = cfg["sparse_mode"], cfg["dtype"] in ("fp8", "e4m3")
    out, ms = fn()
    torch.cuda.synchronize()
    print(f"[run_msa] RAN OK [sparse_mode={mode}]: out={None if out is None else tuple(out.shape)} "
          f"max_score={None if ms is None else tuple(ms.shape)}")
    if not bench:
        return None
    for _ in range(3):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms_mean = e0.elapsed_time(e1) / iters
    flops, nbytes = flops_and_bytes(cfg)
    peaks = peaks or PEAKS
    tf, gb = flops / ms_mean / 1e9, nbytes / ms_mean / 1e6
    peak_tf = peaks["fp8_tflops" if fp8 else "bf16_tflops"]
    print(f"[run_msa] {ms_mean * 1e3:.1f} us  {tf:.1f} TFLOP/s (MFU {100 * tf / peak_tf:.1f} %)  "
          f"{gb:.1f} GB/s (MBU {100 * gb / peaks['hbm_gbs']:.1f} %)")
    return ms_mean


# ----------------------------------------------------------------------------------------------
# sweep tables
# ----------------------------------------------------------------------------------------------
SWEEP_SECTIONS = ("prefill", "paged_prefill", "sparse_prefill", "decode", "paged_decode", "sparse_decode")
TP_HEADS = {1: (64, 4), 2: (32, 2), 4: (16, 1)}            # head presets of the prefill sections
DECODE_HEADS = (64, 4)
TSV_HEADER = ["q_len", "kv_len", "dtype", "batch_size", "q_head", "kv_head", "head_dim", "latency_ms", "std_ms",
              "tflops", "gbs", "mfu_mbu_pct", "predicted_split_speedup_pct"]
TABLE = [("q_len", 8), ("kv_len", 8), ("dtype", 6), ("bsz", 5), ("h_q", 4), ("h_kv", 5), ("dim", 4), ("lat(ms)", 11),
         ("std(ms)", 9), ("TFLOPs", 10), ("GB/s", 10), ("MFU/MBU", 9), ("split%", 8)]


def sweep_cases(section, dtype="bf16", seqs=(8192, 16384, 32768, 65536, 131072), tp=(1, 2, 4),
                decode_k=(8192, 16384, 32768, 65536), decode_b=(32, 64, 128), topk=16, output_mode="o"):
    """The rows of one section: (table title, case dict, rated by bandwidth?)."""
    mode = {"o": "Off", "full": "Full", "maxscore": "OnlyScore"}[output_mode]

    def case(b, q, k, hq, hk, paged, sparse):
        return {"dtype": dtype, "batch_size": b, "seqlen_q": [q] * b, "seqlen_k": [k] * b, "qo_offset": [k - q] * b,
                "num_qo_heads": hq, "num_kv_heads": hk, "head_dim_qk": 128, "head_dim_vo": 128, "num_kv_splits": -1,
                "is_paged": int(paged), "page_size": 128, "causal": 1, "sparse_mode": "Sparse" if sparse else mode,
                "kv_block_num": topk if sparse else 0, "selection": "first"}

    if section == "prefill":
        for t in tp:
            hq, hk = TP_HEADS[t]
            for s_ in seqs:
                yield f"Prefill TP{t} (ragged dense, causal, {dtype})", case(1, s_, s_, hq, hk, False, False), False
    elif section in ("paged_prefill", "sparse_prefill"):
        hq, hk = TP_HEADS[1]
        sparse = section == "sparse_prefill"
        title = (f"Sparse Prefill TP1 (first top-K, page=128, topk={topk}, {dtype})" if sparse else
                 f"Paged Prefill TP1 (paged dense, causal, page=128, {dtype})")
        for s_ in seqs:
            yield title, case(1, s_, s_, hq, hk, True, sparse), False
    elif section in ("decode", "paged_decode"):
        hq, hk = DECODE_HEADS
        paged = section == "paged_decode"
        title = (f"Paged Decode (paged dense, MBU, page=128, h={hq}/{hk}, {dtype})" if paged else
                 f"Decode (ragged dense, MBU, h={hq}/{hk}, {dtype})")
        for b in decode_b:
            for k in decode_k:
                yield title, case(b, 4, k, hq, hk, paged, False), True
    elif section == "sparse_decode":
        hq, hk = DECODE_HEADS
        for b in decode_b:
            for k in decode_k:
                for sparse in (False, True):              # a paged dense row, then the sparse row of the same shape
                    yield (f"Sparse Decode (dense+sparse pairs, MBU, topk={topk}, {dtype})",
                           case(b, 8, k, hq, hk, True, sparse), True)
    else:
        raise ValueError(f"unknown section {section!r}; valid: {', '.join(SWEEP_SECTIONS)}")


def sweep_work(cfg):
    """FLOPs and bytes of a sweep row by the upstream sweep's own formulas
    (bench_sparse_attention_ops.py:135-140, 313-316): a sparse row counts the keys it reads, unmasked."""
    b, q, k = cfg["batch_size"], cfg["seqlen_q"][0], cfg["seqlen_k"][0]
    hq, hk = cfg["num_qo_heads"], cfg["num_kv_heads"]
    e = 1 if cfg["dtype"] in ("fp8", "e4m3") else 2
    if cfg["sparse_mode"] == "Sparse":
        k_eff = min(min(cfg["kv_block_num"], (k + 127) // 128) * 128, k)
        pairs = q * k_eff
    else:
        k_eff = k
        pairs = q * k - q * (q - 1) // 2
    flops = b * hq * pairs * (128 + 128) * 2
    nbytes = b * q * hq * 128 * e + b * k_eff * hk * 128 * e * 2 + b * q * hq * 128 * 2
    return flops, nbytes


def time_cold(fn, dry_ms=200, repeat_ms=1000):
    """Per-iteration CUDA-event times (ms) with the L2 rewritten before every iteration."""
    import torch
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    fn(); torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(); fn(); e1.record(); torch.cuda.synchronize()
    one = max(e0.elapsed_time(e1), 1e-3)
    for _ in range(max(1, int(dry_ms / one))):
        fn()
    n = max(5, min(2000, int(repeat_ms / one)))
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
    for a, b in evs:
        flush.zero_()
        a.record(); fn(); b.record()
    torch.cuda.synchronize()
    return [a.elapsed_time(b) for a, b in evs]


def run_sweep(args, peaks):
    import statistics
    sections = [x.strip() for x in args.sections.split(",") if x.strip()]
    if "all" in sections:
        sections = list(SWEEP_SECTIONS)
    ints = lambda text, default: [int(x) for x in text.split(",")] if text else list(default)
    kw = dict(dtype=args.dtype, seqs=ints(args.seqs, (8192, 16384, 32768, 65536, 131072)), tp=ints(args.tp, (1, 2, 4)),
              decode_k=ints(args.decode_k, (8192, 16384, 32768, 65536)), decode_b=ints(args.decode_b, (32, 64, 128)),
              topk=args.topk, output_mode=args.output_mode)
    tsv = open(args.output, "w") if args.output else None
    if tsv:
        tsv.write("\t".join(TSV_HEADER) + "\n")
    rule = "-" * (sum(w for _, w in TABLE) + len(TABLE) - 1)
    peak_tf = peaks["fp8_tflops" if args.dtype == "fp8" else "bf16_tflops"]
    for section in sections:
        last_title = None
        for title, cfg, by_bandwidth in sweep_cases(section, **kw):
            if title != last_title:
                print(f"\n{title}\n{rule}\n" + " ".join(f"{n:>{w}}" for n, w in TABLE) + f"\n{rule}", flush=True)
                last_title = title
            try:
                fn, plan = build_case(cfg)
                times = time_cold(fn, args.dry_run_ms, args.repeat_ms)
            except Exception as exc:                             # noqa: BLE001  (a row that does not fit is reported, the sweep goes on)
                sys.stderr.write(f"  row skipped ({cfg['seqlen_q'][0]} x {cfg['seqlen_k'][0]}, b={cfg['batch_size']}): {exc}\n")
                continue
            med, std = statistics.median(times), statistics.pstdev(times)
            flops, nbytes = sweep_work(cfg)
            tf, gb = flops / med / 1e9, nbytes / med / 1e6
            rate = gb / peaks["hbm_gbs"] if by_bandwidth else tf / peak_tf
            split = plan[3].get("predicted_speedup", 1.0)
            row = [cfg["seqlen_q"][0], cfg["seqlen_k"][0], args.dtype, cfg["batch_size"], cfg["num_qo_heads"],
                   cfg["num_kv_heads"], 128]
            cells = [str(x) for x in row] + [f"{med:.4f}", f"{std:.4f}", f"{tf:.2f}", f"{gb:.2f}", f"{rate * 100:.2f}%",
                                             f"{(split - 1) * 100:.2f}%"]
            print(" ".join(f"{c:>{w}}" for c, (_, w) in zip(cells, TABLE)), flush=True)
            if tsv:
                tsv.write("\t".join([str(x) for x in row] + [f"{med:.4f}", f"{std:.4f}", f"{tf:.4f}", f"{gb:.4f}",
                                                             f"{rate * 100:.4f}", f"{(split - 1) * 100:.4f}"]) + "\n")
                tsv.flush()
    if tsv:
        tsv.close()
def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--format", type=str, default=None, help="one '[MSA] --format=...' line")
    ap.add_argument("--caselist", type=str, default=None, help="file with one line per case")
    ap.add_argument("--case_idx", type=int, default=None, help="run only this line of --caselist")
    ap.add_argument("--bench", action="store_true", help="time the case")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--peaks", type=str, default=None, help="JSON file with bf16_tflops / fp8_tflops / hbm_gbs")
    ap.add_argument("--sweep", action="store_true", help="print the sweep tables instead of running single cases")
    ap.add_argument("--sections", type=str, default="all", help="comma-separated: " + ",".join(SWEEP_SECTIONS) + ",all")
    ap.add_argument("--dtype", choices=["bf16", "fp8"], default="bf16")
    ap.add_argument("--output_mode", choices=["full", "maxscore", "o"], default="o")
    ap.add_argument("--seqs", type=str, default=None, help="q = k lengths of the prefill sections")
    ap.add_argument("--tp", type=str, default=None, help="head presets of the prefill section: 1,2,4")
    ap.add_argument("--decode-k", dest="decode_k", type=str, default=None, help="KV lengths of the decode sections")
    ap.add_argument("--decode-b", dest="decode_b", type=str, default=None, help="batch sizes of the decode sections")
    ap.add_argument("--topk", type=int, default=16, choices=[4, 8, 16, 32])
    ap.add_argument("--dry-run-ms", dest="dry_run_ms", type=int, default=200)
    ap.add_argument("--repeat-ms", dest="repeat_ms", type=int, default=1000)
    ap.add_argument("--output", "-o", type=str, default=None, help="tab-separated copy of the sweep rows")
    args = ap.parse_args()
    if args.sweep:
        pk = dict(PEAKS)
        if args.peaks:
            with open(args.peaks) as f:
                raw = json.load(f)
            pk.update({k: raw[k] for k in PEAKS if k in raw})
        run_sweep(args, pk)
        return
    lines = []
    if args.format:
        lines.append(args.format)
    if args.caselist:
        with open(args.caselist) as f:
            cases = [ln.strip() for ln in f if "--format=" in ln]
        lines += cases if args.case_idx is None else [cases[args.case_idx]]
    if not lines:
        ap.error("give --format or --caselist")
    peaks = None
    if args.peaks:
        with open(args.peaks) as f:
            raw = json.load(f)
        peaks = dict(PEAKS)
        peaks.update({k: raw[k] for k in PEAKS if k in raw})
    for ln in lines:
        cfg = parse_format(ln)
        print(format_line(cfg))
        build_and_run(cfg, bench=args.bench, iters=args.iters, peaks=peaks)


if __name__ == "__main__":
    main()
