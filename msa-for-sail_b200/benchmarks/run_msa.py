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


def build_and_run(cfg, bench=False, iters=20, peaks=None):
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
    if mode == "Sparse":
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


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--format", type=str, default=None, help="one '[MSA] --format=...' line")
    ap.add_argument("--caselist", type=str, default=None, help="file with one line per case")
    ap.add_argument("--case_idx", type=int, default=None, help="run only this line of --caselist")
    ap.add_argument("--bench", action="store_true", help="time the case")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--peaks", type=str, default=None, help="JSON file with bf16_tflops / fp8_tflops / hbm_gbs")
    args = ap.parse_args()
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
