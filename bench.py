#!/usr/bin/env python3
"""Benchmark of the MSA attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

Headline workload = BASELINE config 3, the MSA sparse prefill pipeline: batch 2, q_len = kv_len =
32768, 64 query heads / 8 KV heads, head_dim 128, pages of 128 keys, 1-head proxy max-score pass ->
page top-k (16) -> sparse attention over the selected pages.  A step is one pass of the three
stages over the batch (plans are built once, as the upstream API intends).  The metric is effective
TFLOP/s: the causal-discounted QK FLOPs of the proxy pass plus the accessed-KV FLOPs of the sparse
stage (upstream bench_utils.attention_tflops, benchmarks/run_msa.py:149-163) per second.

The same JSON line carries, under "configs", full sub-records (value, step time, roofline, stages,
e2e, clocks, parity sample, CPU baseline) of the other BASELINE configurations: config 1 (the small
pipeline whose CPU baseline is the whole oracle pipeline), config 2 (dense paged causal prefill),
config 4 (MSA sparse decode over an e4m3 cache) and config 5 (1M-token paged decode).  With
--gpus N the (batch item, KV-head group) units of configs 2-4 are sharded over the ranks (no
collective) and the KV range of config 5 is split over them (NCCL all-gather of (O, LSE) + merge).

Every timed workload ends with a parity sample: rows of what the timed kernels wrote are compared
with the CPU oracle (top-k rows bit-exact); a miss fails the run.

Prints ONE JSON line (rank 0).  `--impl reference` times the CPU oracle port of the headline path
on the host cores over a bounded sample of the same workload.
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "msa-for-sail_b200", "python"))
sys.path.insert(0, ROOT)

D = 128
PAGE = 128


def attention_flops(batch, q_len, kv_len, h_q, causal=True):
    """Causal-discounted QK + PV FLOPs (upstream python/msa_for_sail/bench_utils.py:115-133)."""
    pairs = q_len * kv_len - (q_len * (q_len - 1) // 2 if causal else 0)
    return batch * h_q * pairs * (D + D) * 2


WORKLOADS = {
    # name: (kind, parameters)
    "msa_prefill_b2_s32768_h64kv8_top16": ("msa_prefill", dict(b=2, t=32768, hq=64, hk=8, topk=16)),      # config 3
    "msa_prefill_b1_s4096_h16kv2_top8": ("msa_prefill", dict(b=1, t=4096, hq=16, hk=2, topk=8, koff=0.0)),  # config 1
    "msa_prefill_b1_s8192_h32kv4_top16": ("msa_prefill", dict(b=1, t=8192, hq=32, hk=4, topk=16)),          # small: ncu
    "paged_prefill_b4_s8192_h64kv8": ("prefill", dict(b=4, ql=8192, kl=8192, hq=64, hk=8)),                 # config 2
    "paged_prefill_b2_s4096_h32kv4": ("prefill", dict(b=2, ql=4096, kl=4096, hq=32, hk=4)),                 # small: ncu
    # configs 2 and 3 with e4m3 Q, K, V (upstream's fp8 mode: same shapes, cache and queries cast to e4m3)
    "paged_prefill_e4m3_b4_s8192_h64kv8": ("prefill", dict(b=4, ql=8192, kl=8192, hq=64, hk=8, fp8=True)),
    "msa_prefill_e4m3_b2_s32768_h64kv8_top16": ("msa_prefill", dict(b=2, t=32768, hq=64, hk=8, topk=16, fp8=True)),
    "paged_prefill_e4m3_b2_s4096_h32kv4": ("prefill", dict(b=2, ql=4096, kl=4096, hq=32, hk=4, fp8=True)),       # small: ncu
    "msa_prefill_e4m3_b1_s8192_h32kv4_top16": ("msa_prefill", dict(b=1, t=8192, hq=32, hk=4, topk=16, fp8=True)), # small: ncu
    "msa_decode_e4m3_b32_kv131072_h64kv8_top16_split4": (
        "msa_decode", dict(b=32, kl=131072, hq=64, hk=8, topk=16, splits=4, fp8=True)),                     # config 4
    "msa_decode_bf16_b32_kv131072_h64kv8_top16_split4": (
        "msa_decode", dict(b=32, kl=131072, hq=64, hk=8, topk=16, splits=4, fp8=False)),
    "msa_decode_e4m3_b8_kv131072_h64kv8_top16_split4": (
        "msa_decode", dict(b=8, kl=131072, hq=64, hk=8, topk=16, splits=4, fp8=True)),                      # small: ncu
    "paged_decode_b1_kv1048576_h64kv8": ("decode", dict(b=1, kl=1048576, hq=64, hk=8)),                     # config 5
    "paged_decode_b1_kv131072_h64kv8": ("decode", dict(b=1, kl=131072, hq=64, hk=8)),                       # small: ncu
}
DEFAULT = "msa_prefill_b2_s32768_h64kv8_top16"
SUB_CONFIGS = [                       # sub-records of the default run, in BASELINE order
    ("config1", "msa_prefill_b1_s4096_h16kv2_top8"),
    ("config2", "paged_prefill_b4_s8192_h64kv8"),
    ("config4", "msa_decode_e4m3_b32_kv131072_h64kv8_top16_split4"),
    ("config5", "paged_decode_b1_kv1048576_h64kv8"),
    ("config2_e4m3", "paged_prefill_e4m3_b4_s8192_h64kv8"),
    ("config3_e4m3", "msa_prefill_e4m3_b2_s32768_h64kv8_top16"),
]
METRICS = {"prefill": ("prefill_effective_tflops", "TFLOP/s"), "msa_prefill": ("msa_prefill_effective_tflops", "TFLOP/s"),
           "msa_decode": ("msa_decode_kv_gbps", "GB/s"), "decode": ("decode_kv_gbps", "GB/s")}

# dram__bytes_read + dram__bytes_write per launch of the dominant kernel, from the ncu captures
# summarised under profiles/ (captured on the small variant and scaled by the units processed
# where the full workload is too large to capture with --set full)
TRAFFIC = {
    "paged_prefill_b4_s8192_h64kv8": (0.89e9, "scaled x8.0 from the b2_s4096_h32kv4 capture (111.5 MB)"),
    "paged_prefill_b2_s4096_h32kv4": (111.5e6, "captured"),
    "paged_decode_b1_kv1048576_h64kv8": (4.33e9, "scaled x8 from the kv131072 capture (541.7 MB)"),
    "paged_decode_b1_kv131072_h64kv8": (541.7e6, "captured"),
    "msa_prefill_b1_s8192_h32kv4_top16": (1.055e9, "captured (sparse_tc_kernel; sparse_merge_kernel: 1.155e9)"),
    "msa_prefill_b2_s32768_h64kv8_top16": (16.9e9, "scaled x16 from the b1_s8192_h32kv4 capture (sparse_tc_kernel; "
                                                    "sparse_merge_kernel: 18.5e9)"),
    "msa_prefill_e4m3_b1_s8192_h32kv4_top16": (0.976e9, "captured (sparse_tc_kernel<e4m3>: 62 MB read + 914 MB written)"),
    "msa_prefill_e4m3_b2_s32768_h64kv8_top16": (15.6e9, "scaled x16 from the e4m3 b1_s8192_h32kv4 capture (sparse_tc_kernel<e4m3>; "
                                                         "the merge kernel is the bf16 path's: 18.5e9)"),
    "paged_prefill_e4m3_b2_s4096_h32kv4": (59.2e6, "captured"),
    "paged_prefill_e4m3_b4_s8192_h64kv8": (0.47e9, "scaled x8.0 from the e4m3 b2_s4096_h32kv4 capture (59.2 MB)"),
    "msa_decode_e4m3_b8_kv131072_h64kv8_top16_split4": (138.1e6, "captured (score_gemv_kernel; decode_tc_kernel: 33.9e6)"),
    "msa_decode_e4m3_b32_kv131072_h64kv8_top16_split4": (552e6, "scaled x4 from the b8 capture (score_gemv_kernel; "
                                                               "decode_tc_kernel: 135e6)"),
}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"bf16": p["bf16_tflops"], "bf16_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                "hbm": p["hbm_gbs"], "src": "measured"}
    return {"bf16": 1590.0, "bf16_sustained": 1400.0, "hbm": 6650.0, "src": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc, self.index, self.first = [], None, index, 0

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
            t0 = time.time()
            while not self.rows and time.time() - t0 < 5.0:      # wait until the sampler is live
                time.sleep(0.01)
        except OSError:
            self.proc = None

    def mark(self):
        """Samples taken from now on belong to the timed region."""
        self.first = len(self.rows)

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        rows = self.rows[self.first:]
        clk = sorted(int(r[0]) for r in rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in rows if len(r) >= 6 for i in range(4) if r[2 + i] == "Active"})
        return {"sm_mhz": clk[len(clk) // 2] if clk else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(clk)}


class ParityError(RuntimeError):
    pass


def _cos(a, b):
    a, b = a.double().reshape(-1), b.double().reshape(-1)
    den = (a.norm() * b.norm()).item()
    return float((a @ b).item() / den) if den > 0 else 1.0


def _compare_rows(out, ref, cos_min, max_abs, what):
    """`out` [n, h, 128] against the oracle with the bounds the parity tests use: max-abs error and the
    cosine over the whole sample; the smallest per-row cosine is reported beside them.  Raises on a miss."""
    out, ref = out.float(), ref.float()
    if not torch.isfinite(out).all():
        raise ParityError(f"{what}: non-finite output")
    err = (out - ref).abs().max().item()
    cos = _cos(out, ref)
    num = (out.double() * ref.double()).sum(-1)
    den = out.double().norm(dim=-1) * ref.double().norm(dim=-1)
    row = torch.where(den > 0, num / den.clamp_min(1e-300), torch.ones_like(num))
    if err > max_abs or cos < cos_min:
        raise ParityError(f"{what}: max-abs {err:.4g} (limit {max_abs}), cosine {cos:.6f} (limit {cos_min})")
    return {"rows": int(out.shape[0] * out.shape[1]), "max_abs": err, "cos": cos, "cos_min_row": float(row.min().item())}


def _check_scores(ms, ref, what, rel=1e-2):
    """Per-page max scores: same -inf pattern, finite values within `rel` relative."""
    inf_ref = torch.isinf(ref) & (ref < 0)
    if not torch.equal(torch.isinf(ms) & (ms < 0), inf_ref):
        raise ParityError(f"{what}: -inf pattern of max_score differs from the oracle")
    fin = ~inf_ref
    e = ((ms[fin] - ref[fin]).abs() / ref[fin].abs().clamp_min(1.0)).max().item() if fin.any() else 0.0
    if e > rel:
        raise ParityError(f"{what}: max_score relative error {e:.4g} > {rel}")
    return e


# ----------------------------------------------------------------------------------------------
# sharding of the independent (batch item, KV-head group) units over the ranks
# ----------------------------------------------------------------------------------------------

def shard_shape(b, hq, hk, rank, world):
    """Contiguous block of the b * hk units for this rank -> (local batch, local query heads, local KV
    heads).  Whole batch items while there are enough of them, then KV-head groups of one item."""
    from msa_for_sail import dist as mdist
    units = mdist.shard_units(b * hk, rank, world, contiguous=True)
    if world == 1:
        return b, hq, hk
    n = len(units)
    if n == 0 or (b * hk) % world:
        return None                                  # the units do not divide over the ranks
    g = hq // hk
    if n % hk == 0:
        return n // hk, hq, hk
    if hk % n:
        return None                                  # a rank's units would straddle two batch items
    return 1, n * g, n


# ----------------------------------------------------------------------------------------------
# workloads: each builds HBM-resident inputs, returns a dict with the step closure, the
# algorithmic work of one step and a parity check of what the step wrote
# ----------------------------------------------------------------------------------------------

def _i32(x):
    return torch.tensor(x, dtype=torch.int32)


def setup_prefill(msa, dev, seed, b, ql, kl, hq, hk, fp8=False, **_):
    from oracle import msa_oracle as orc
    g = torch.Generator(device="cpu").manual_seed(seed)
    P = kl // PAGE                                            # pages per sequence
    pool = b * P
    dt = torch.float8_e4m3fn if fp8 else torch.bfloat16       # e4m3: plain casts (unit scales)
    esz = 1 if fp8 else 2
    q_h = (torch.randn(b * ql, hq, D, generator=g) * 0.5).to(torch.bfloat16).to(dt).pin_memory()
    k_h = (torch.randn(pool, hk, PAGE, D, generator=g) * 0.5).to(torch.bfloat16).to(dt).pin_memory()
    v_h = (torch.randn(pool, hk, PAGE, D, generator=g) * 0.5).to(torch.bfloat16).to(dt).pin_memory()
    # device-timed step: the page tables are one seeded random permutation of the whole pool
    table = torch.randperm(pool, generator=g).to(torch.int32).to(dev)
    q, k, v = q_h.to(dev), k_h.to(dev), v_h.to(dev)
    plan = msa.fmha_sail_plan(_i32([ql] * b), _i32([kl] * b), hq, num_kv_heads=hk, page_size=PAGE, use_fp8_kvcache=fp8)
    out = torch.empty(b * ql, hq, D, dtype=torch.bfloat16, device=dev)
    lse = torch.empty(b * ql, hq, dtype=torch.float32, device=dev)
    out_h = torch.empty(out.shape, dtype=out.dtype).pin_memory()

    def step():
        msa.fmha_sail(q, k, v, plan, kv_indices=table, out=out, lse=lse)

    # end to end: the inputs of a step start in pinned host memory.  One public-API call per row chunk of
    # a sequence (chunked prefill: chunk j attends to the keys of chunks 0..j), so that the copy-in of the
    # next chunk, the attention of this one and the copy-out of the previous one overlap (three streams;
    # every byte of Q, K, V still crosses PCIe inside the timed region, every byte of O comes back).  This
    # leg lays the cache out for streaming: every sequence owns a slab of P pages and its page table is
    # shuffled within groups of P / NCH pages, so that the pages a chunk adds are one contiguous host copy.
    NCH = 4 if (ql == kl and P % 4 == 0 and ql % (4 * 256) == 0) else 1     # row chunks per sequence
    gp = P // NCH
    local = torch.stack([torch.cat([torch.randperm(gp, generator=g) + j * gp for j in range(NCH)])
                         for _ in range(b)]).to(torch.int32)
    cq = ql // NCH
    plans = [msa.fmha_sail_plan(_i32([cq]), _i32([(j + 1) * cq]), hq, num_kv_heads=hk, page_size=PAGE, use_fp8_kvcache=fp8)
             for j in range(NCH)]
    local_dev = local.to(dev)
    table_e2e = (local + torch.arange(b, dtype=torch.int32).view(b, 1) * P).reshape(-1).to(dev)

    def e2e_ref_step():
        """The end-to-end leg's cache layout in one resident call (what its chunks must add up to)."""
        msa.fmha_sail(q, k, v, plan, kv_indices=table_e2e, out=out, lse=lse)

    qd, kd, vd, od = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v), torch.empty_like(out)
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    ev_in = [torch.cuda.Event() for _ in range(b * NCH)]
    ev_done = [torch.cuda.Event() for _ in range(b * NCH)]

    def e2e_step():
        cur = torch.cuda.current_stream()
        s_in.wait_stream(cur); s_out.wait_stream(cur)          # the previous step has released the buffers
        for i in range(b):
            rk = slice(i * P, (i + 1) * P)
            for j in range(NCH):
                n = i * NCH + j
                rq = slice(i * ql + j * cq, i * ql + (j + 1) * cq)
                rp = slice(i * P + j * gp, i * P + (j + 1) * gp)
                with torch.cuda.stream(s_in):
                    qd[rq].copy_(q_h[rq], non_blocking=True)
                    kd[rp].copy_(k_h[rp], non_blocking=True)
                    vd[rp].copy_(v_h[rp], non_blocking=True)
                    ev_in[n].record(s_in)
                cur.wait_event(ev_in[n])
                msa.fmha_sail(qd[rq], kd[rk], vd[rk], plans[j], kv_indices=local_dev[i, :(j + 1) * gp], out=od[rq])
                ev_done[n].record(cur)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_done[n])
                    out_h[rq].copy_(od[rq], non_blocking=True)
        cur.wait_stream(s_out)

    def parity():
        """64 (token, head) rows of the timed step's O and LSE: 4 (batch item, KV head) units x 2 tokens
        x the 8 heads of the group (fewer where the shard is smaller), dense causal oracle."""
        gsz = hq // hk
        gen = torch.Generator().manual_seed(seed + 1)
        units = [(int(torch.randint(0, b, (1,), generator=gen)), int(torch.randint(0, hk, (1,), generator=gen)))
                 for _ in range(4)]
        toks_per_unit = max(2, 64 // (4 * gsz))
        outs, refs, lses, lrefs = [], [], [], []
        for bi, kh in units:
            pages = table[bi * P:(bi + 1) * P].long()
            kc = k[pages, kh].reshape(P * PAGE, 1, D).to(torch.bfloat16).cpu()      # e4m3 values are exact in bf16
            vc = v[pages, kh].reshape(P * PAGE, 1, D).to(torch.bfloat16).cpu()
            pos = torch.randint(0, ql, (toks_per_unit,), generator=gen).tolist()
            pos[0] = ql - 1                                                    # the longest row of the sequence
            for i in pos:
                t = bi * ql + i
                qq = q[t:t + 1, kh * gsz:(kh + 1) * gsz].to(torch.bfloat16).cpu()
                o_ref, l_ref = orc.attention_single(qq, kc, vc, gsz, 1, True, i + kl - ql, return_lse=True)
                outs.append(out[t:t + 1, kh * gsz:(kh + 1) * gsz].cpu()); refs.append(o_ref)
                lses.append(lse[t:t + 1, kh * gsz:(kh + 1) * gsz].cpu()); lrefs.append(l_ref)
        r = _compare_rows(torch.cat(outs), torch.cat(refs), 0.999 if fp8 else 0.9999, 0.1 if fp8 else 2e-2, "dense prefill O")
        lerr = (torch.cat(lses) - torch.cat(lrefs)).abs().max().item()
        if lerr > 2e-2:
            raise ParityError(f"dense prefill LSE off by {lerr:.4g}")
        r["lse_max_abs"] = lerr
        return r

    nbytes = (q.numel() + k.numel() + v.numel()) * esz + out.numel() * 2
    return dict(step=step, e2e_step=e2e_step, e2e_ref_step=e2e_ref_step, results=(out, out_h), parity=parity,
                flops=attention_flops(b, ql, kl, hq), bytes=nbytes, unit="TFLOP/s", bound="tensor", launches=1, graph=False, tokens=b * ql,
                h2d=(q_h.numel() + k_h.numel() + v_h.numel()) * esz, d2h=out_h.numel() * 2,
                e2e_note=("chunked prefill through the public API, four row chunks per sequence; the copy-in of a chunk's Q "
                          "rows and K/V pages from pinned host memory, its attention and the copy-out of its O overlap "
                          "with the neighbouring chunks on three streams; this leg shuffles the page table within the "
                          "groups of pages a chunk adds (one contiguous host copy per chunk), the device-timed step uses "
                          "one random permutation of the whole pool"),
                l2="inputs larger than L2 (Q+K+V+O = %.2f GB per GPU)" % (nbytes / 1e9))


def setup_msa_prefill(msa, dev, seed, b, t, hq, hk, topk, koff=2.0, fp8=False, **_):
    """Configs 1 and 3: 1-head proxy max-score pass -> page top-k -> sparse attention on the selection.
    K = N(0,1) + one offset ~ N(0, koff) per (page, head), broadcast over the page's keys and head_dim."""
    from oracle import msa_oracle as orc
    g = torch.Generator(device=dev).manual_seed(seed)
    P = t // PAGE
    q = torch.randn(b * t, hq, D, device=dev, generator=g).to(torch.bfloat16)
    kp = (torch.randn(b * P, hk, PAGE, D, device=dev, generator=g)
          + math.sqrt(koff) * torch.randn(b * P, hk, 1, 1, device=dev, generator=g)).to(torch.bfloat16)
    vp = torch.randn(b * P, hk, PAGE, D, device=dev, generator=g).to(torch.bfloat16)
    if fp8:                                                   # plain casts (unit scales); the page offsets stay within range
        q, kp, vp = q.to(torch.float8_e4m3fn), kp.to(torch.float8_e4m3fn), vp.to(torch.float8_e4m3fn)
    esz = 1 if fp8 else 2
    wide = (lambda x: x.to(torch.bfloat16)) if fp8 else (lambda x: x)          # e4m3 values are exact in bf16
    table = torch.randperm(b * P, device=dev, generator=g).to(torch.int32)
    qx, kx = q[:, :1].contiguous(), kp[:, :1].contiguous()
    lens = _i32([t] * b)
    plan1 = msa.fmha_sail_plan(lens, lens, 1, num_kv_heads=1, page_size=PAGE, output_maxscore=True, use_fp8_kvcache=fp8)
    plan2 = msa.fmha_sail_plan(lens, lens, hq, num_kv_heads=hk, page_size=PAGE, kv_block_num=topk, use_fp8_kvcache=fp8)
    ms = torch.full((1, plan1[3]["max_k_tiles"], b * t), -float("inf"), device=dev)
    idx = torch.empty(b * t, 1, topk, dtype=torch.int32, device=dev)
    out = torch.empty(b * t, hq, D, dtype=torch.bfloat16, device=dev)

    def s_proxy():
        msa.fmha_sail(qx, kx, kx, plan1, kv_indices=table, output_o=False, max_score=ms)

    def s_topk():
        msa.sparse_topk_select(ms, topk, num_valid_pages=P, output=idx)

    def s_sparse():
        msa.fmha_sail(q, kp, vp, plan2, kv_indices=table, kv_block_indexes=idx.expand(b * t, hk, topk), out=out)

    def step():
        s_proxy(); s_topk(); s_sparse()

    pairs = t * t - t * (t - 1) // 2
    f_proxy = b * 1 * pairs * D * 2
    f_sparse = b * t * hq * (topk * PAGE) * (D + D) * 2          # accessed-KV FLOPs (upstream run_msa.py:159-163)
    out_h = torch.empty(out.shape, dtype=out.dtype).pin_memory()
    q_h = q.cpu().pin_memory()

    # end to end: Q starts in pinned host memory and O ends there; the KV cache is device-resident
    # state.  The pipeline runs as chunked prefill, NCH row chunks per sequence (chunk j attends to the
    # keys of chunks 0..j), so that the copy-in of the next chunk, the three stages of this one and the
    # copy-out of the previous one overlap on three streams.
    NCH = 8 if t % (8 * PAGE) == 0 and t // 8 >= 1024 else 1
    cq = t // NCH
    cplans = []
    for j in range(NCH):
        ln_q, ln_k = _i32([cq]), _i32([(j + 1) * cq])
        pa = msa.fmha_sail_plan(ln_q, ln_k, 1, num_kv_heads=1, page_size=PAGE, output_maxscore=True, use_fp8_kvcache=fp8)
        pb = msa.fmha_sail_plan(ln_q, ln_k, hq, num_kv_heads=hk, page_size=PAGE, kv_block_num=topk, use_fp8_kvcache=fp8)
        cplans.append((pa, pb, torch.full((1, pa[3]["max_k_tiles"], cq), -float("inf"), device=dev)))
    cidx = torch.empty(cq, 1, topk, dtype=torch.int32, device=dev)
    qd, od = torch.empty_like(q), torch.empty_like(out)
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    ev_in = [torch.cuda.Event() for _ in range(b * NCH)]
    ev_done = [torch.cuda.Event() for _ in range(b * NCH)]

    def e2e_step():
        cur = torch.cuda.current_stream()
        s_in.wait_stream(cur); s_out.wait_stream(cur)          # the previous step has released the buffers
        for i in range(b):
            for j in range(NCH):
                n = i * NCH + j
                rq = slice(i * t + j * cq, i * t + (j + 1) * cq)
                pages = (j + 1) * cq // PAGE
                tab = table[i * P:i * P + pages]
                pa, pb, cms = cplans[j]
                with torch.cuda.stream(s_in):
                    qd[rq].copy_(q_h[rq], non_blocking=True)
                    ev_in[n].record(s_in)
                cur.wait_event(ev_in[n])
                msa.fmha_sail(qd[rq][:, :1].contiguous(), kx, kx, pa, kv_indices=tab, output_o=False, max_score=cms)
                msa.sparse_topk_select(cms, topk, num_valid_pages=pages, output=cidx)
                msa.fmha_sail(qd[rq], kp, vp, pb, kv_indices=tab, kv_block_indexes=cidx.expand(cq, hk, topk), out=od[rq])
                ev_done[n].record(cur)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_done[n])
                    out_h[rq].copy_(od[rq], non_blocking=True)
        cur.wait_stream(s_out)

    def parity():
        """16 tokens (first and last of a sequence, some with fewer visible pages than top-k, the rest
        seeded random) x all query heads: the proxy scores of each token against the oracle, its top-k row
        bit-exact against the oracle's selection on the same scores, and its sparse attention rows."""
        gen = torch.Generator().manual_seed(seed + 2)
        n_tok = 16
        pos = torch.randint(0, t, (n_tok,), generator=gen)
        pos[0], pos[1], pos[2], pos[3] = 0, t - 1, min(t - 1, PAGE * topk // 2), min(t - 1, PAGE * topk + 5)
        seq = torch.randint(0, b, (n_tok,), generator=gen)
        toks = (seq * t + pos).tolist()
        # proxy scores: the token's query against the proxy cache of its sequence, per-page causal max
        ms_gpu = ms[0, :P][:, toks].t().contiguous().cpu()                     # [n_tok, P]
        ms_ref = torch.full_like(ms_gpu, -float("inf"))
        kseq = {}
        for j, tk in enumerate(toks):
            s, i = int(seq[j]), int(pos[j])
            if s not in kseq:
                kseq[s] = wide(kx[table[s * P:(s + 1) * P].long(), 0]).reshape(P * PAGE, D).float().cpu()
            sc = kseq[s][:i + 1] @ wide(qx[tk, 0]).float().cpu()
            npg = i // PAGE + 1
            sc = torch.nn.functional.pad(sc, (0, npg * PAGE - (i + 1)), value=-float("inf"))
            ms_ref[j, :npg] = sc.view(npg, PAGE).max(-1).values
        score_err = _check_scores(ms_gpu, ms_ref, "proxy pass")
        # top-k: the oracle's selection on the scores the GPU produced
        sel_ref = orc.topk_select(ms_gpu.t().contiguous().view(1, P, n_tok), topk, P)[:, 0]      # [n_tok, topk]
        sel_gpu = idx[toks, 0].cpu()
        topk_exact = bool(torch.equal(sel_gpu, sel_ref))
        if not topk_exact:
            raise ParityError("top-k rows differ from the oracle's selection")
        # sparse attention of the sampled tokens: one mini problem per token (its selected pages only)
        kc, vc, tabs = [], [], []
        for j, tk in enumerate(toks):
            s = int(seq[j])
            lp = sel_gpu[j].long()
            valid = lp >= 0
            phys = table[s * P + lp.clamp_min(0).to(dev)].long()
            kc.append(wide(kp[phys]).cpu()); vc.append(wide(vp[phys]).cpu())
            mini = torch.zeros(P, dtype=torch.int32)
            mini[lp[valid]] = (torch.arange(topk)[valid] + j * topk).to(torch.int32)
            tabs.append(mini)
        ref = orc.sparse_attention(wide(q[toks]).cpu(), torch.cat(kc), torch.cat(vc), [1] * n_tok, [t] * n_tok, torch.cat(tabs),
                                   sel_gpu.view(n_tok, 1, topk).expand(n_tok, hk, topk), hq,
                                   qo_offset=[int(x) for x in pos])
        r = _compare_rows(out[toks].cpu(), ref, 0.999 if fp8 else 0.9999, 0.1 if fp8 else 2e-2, "sparse prefill O")
        r.update(topk_exact=topk_exact, topk_rows=n_tok, score_rel_err=score_err)
        return r

    return dict(step=step, e2e_step=e2e_step, results=(out, out_h), parity=parity, flops=f_proxy + f_sparse, bytes=None,
                stages=dict(proxy=(s_proxy, f_proxy, "TFLOP/s"),
                            topk=(s_topk, ms[:, :P].numel() * 4 + idx.numel() * 4, "GB/s"),
                            sparse=(s_sparse, f_sparse, "TFLOP/s")),
                unit="TFLOP/s", bound="tensor", launches=7, graph=False, tokens=b * t,
                h2d=q_h.numel() * esz, d2h=out_h.numel() * 2,
                e2e_note=("chunked prefill through the public API, %d row chunk(s) per sequence: the copy-in of a chunk's Q "
                          "from pinned host memory, its proxy pass, top-k and sparse attention and the copy-out of its O "
                          "overlap with the neighbouring chunks on three streams; the KV cache is device-resident state" % NCH),
                l2=("inputs larger than L2 (Q+O = %.2f GB per GPU); the KV cache stays resident" % (2 * q.numel() * 2 / 1e9)
                    if 2 * q.numel() * 2 > 130e6 else
                    "L2 flushed between steps is NOT done: this small configuration (%.0f MB) exists for its CPU "
                    "baseline and parity, not for its GPU number" % (2 * q.numel() * 2 / 1e6)))


def setup_msa_decode(msa, dev, seed, b, kl, hq, hk, topk, splits, fp8, **_):
    """Config 4: proxy max-score over a 1-head proxy cache -> top-k -> sparse decode with split-KV."""
    from oracle import msa_oracle as orc
    g = torch.Generator(device=dev).manual_seed(seed)
    P = kl // PAGE
    kvdt = torch.float8_e4m3fn if fp8 else torch.bfloat16
    q = torch.randn(b, hq, D, device=dev, generator=g).to(torch.bfloat16)
    ks = vs = None
    kp = torch.empty(b * P, hk, PAGE, D, device=dev, dtype=kvdt)
    vp = torch.empty(b * P, hk, PAGE, D, device=dev, dtype=kvdt)
    if fp8:                                      # quantise with one fp32 scale per KV head (amax / 448), in slabs
        ks = torch.full((hk,), 5.5 / 448.0, device=dev); vs = torch.full((hk,), 5.5 / 448.0, device=dev)
    slab = 2048
    for s0 in range(0, b * P, slab):
        n = min(slab, b * P - s0)
        for dst, sc in ((kp, ks), (vp, vs)):
            x = torch.randn(n, hk, PAGE, D, device=dev, generator=g, dtype=torch.bfloat16)
            dst[s0:s0 + n] = (x.float() / sc.view(1, hk, 1, 1)).clamp(-448, 448).to(kvdt) if fp8 else x
    kx = torch.randn(b * P, 1, PAGE, D, device=dev, generator=g, dtype=torch.bfloat16).to(kvdt)
    qx = q[:, :1].contiguous().to(kvdt)
    table = torch.randperm(b * P, device=dev, generator=g).to(torch.int32)
    ql, kls = _i32([1] * b), _i32([kl] * b)
    plan1 = msa.fmha_sail_plan(ql, kls, 1, num_kv_heads=1, page_size=PAGE, output_maxscore=True, use_fp8_kvcache=fp8)
    plan2 = msa.fmha_sail_plan(ql, kls, hq, num_kv_heads=hk, page_size=PAGE, kv_block_num=topk,
                               num_kv_splits=splits, use_fp8_kvcache=fp8)
    ms = torch.full((1, plan1[3]["max_k_tiles"], b), -float("inf"), device=dev)
    idx = torch.empty(b, 1, topk, dtype=torch.int32, device=dev)
    bi = idx.expand(b, hk, topk)                 # every KV head uses the proxy head's pages: stride-0 view
    out = torch.empty(b, hq, D, dtype=torch.bfloat16, device=dev)
    kw = dict(k_scale=ks, v_scale=vs) if fp8 else {}

    def s_proxy():
        msa.fmha_sail(qx, kx, kx, plan1, kv_indices=table, output_o=False, max_score=ms)

    def s_topk():
        msa.sparse_topk_select(ms, topk, num_valid_pages=P, output=idx)

    def s_sparse():
        msa.fmha_sail(q, kp, vp, plan2, kv_indices=table, kv_block_indexes=bi, out=out, **kw)

    def step():
        s_proxy(); s_topk(); s_sparse()

    e = kp.element_size()
    by_sparse = b * hk * topk * PAGE * 2 * D * e + 2 * b * hq * D * 2     # unique pages + Q + O
    by_proxy = kx.numel() * kx.element_size() + ms[:, :P].numel() * 4
    q_h = q.cpu().pin_memory(); out_h = torch.empty(out.shape, dtype=out.dtype).pin_memory()

    def e2e_step():
        q.copy_(q_h, non_blocking=True)
        qx.copy_(q[:, :1])
        step()
        out_h.copy_(out, non_blocking=True)

    def parity():
        """Up to 8 batch items x all query heads (64 rows each): proxy scores, top-k row bit-exact,
        sparse decode output against the oracle on the de-quantised cache."""
        gen = torch.Generator().manual_seed(seed + 3)
        items = torch.randperm(b, generator=gen)[:min(b, 8)].tolist()
        n = len(items)
        ms_gpu = ms[0, :P][:, items].t().contiguous().cpu()
        ms_ref = torch.empty_like(ms_gpu)
        for j, it in enumerate(items):
            kk = kx[table[it * P:(it + 1) * P].long(), 0].reshape(P * PAGE, D).float().cpu()
            ms_ref[j] = (kk @ qx[it, 0].float().cpu()).view(P, PAGE).max(-1).values
        score_err = _check_scores(ms_gpu, ms_ref, "proxy pass")
        sel_ref = orc.topk_select(ms_gpu.t().contiguous().view(1, P, n), topk, P)[:, 0]
        sel_gpu = idx[items, 0].cpu()
        if not torch.equal(sel_gpu, sel_ref):
            raise ParityError("top-k rows differ from the oracle's selection")
        kc, vc, tabs = [], [], []
        for j, it in enumerate(items):
            phys = table[it * P + sel_gpu[j].long().to(dev)].long()
            kf, vf = kp[phys].float(), vp[phys].float()
            if fp8:
                kf, vf = kf * ks.view(1, hk, 1, 1), vf * vs.view(1, hk, 1, 1)
            kc.append(kf.cpu()); vc.append(vf.cpu())
            mini = torch.zeros(P, dtype=torch.int32)
            mini[sel_gpu[j].long()] = (torch.arange(topk) + j * topk).to(torch.int32)
            tabs.append(mini)
        ref = orc.sparse_attention(q[items].cpu(), torch.cat(kc), torch.cat(vc), [1] * n, [kl] * n, torch.cat(tabs),
                                   sel_gpu.view(n, 1, topk).expand(n, hk, topk), hq)
        r = _compare_rows(out[items].cpu(), ref, 0.999 if fp8 else 0.9999, 0.1 if fp8 else 2e-2, "sparse decode O")
        r.update(topk_exact=True, topk_rows=n, score_rel_err=score_err)
        return r

    return dict(step=step, e2e_step=e2e_step, parity=parity, flops=None, bytes=by_sparse + by_proxy,
                stages=dict(proxy=(s_proxy, by_proxy, "GB/s"), topk=(s_topk, ms[:, :P].numel() * 4, "GB/s"),
                            sparse=(s_sparse, by_sparse, "GB/s")),
                unit="GB/s", bound="hbm", launches=4, graph=True, tokens=b,
                h2d=q_h.numel() * 2, d2h=out_h.numel() * 2,
                e2e_note=("public API calls with pinned host tensors copied in and the result copied out each step; "
                          "the KV cache is device-resident state"),
                l2="every step streams %.0f MB (proxy cache + selected pages) of a %.1f GB cache: larger than L2" % (
                    (by_sparse + by_proxy) / 1e6, (kp.numel() + vp.numel()) * e / 1e9),
                extra_cfg=dict(num_kv_splits_used=plan2[3]["num_kv_splits"]))


def setup_decode(msa, dev, seed, b, kl, hq, hk, rank=0, world=1, **_):
    """Config 5: dense paged decode; with world > 1 this rank owns a contiguous slice of the pages."""
    import torch.distributed as dist
    from msa_for_sail import dist as mdist
    from oracle import msa_oracle as orc
    g = torch.Generator(device=dev).manual_seed(seed)
    p0, p1 = mdist.shard_page_range(kl // PAGE, rank, world)
    P = p1 - p0
    kl_local = P * PAGE
    q = torch.randn(b, hq, D, device=dev, generator=torch.Generator(device=dev).manual_seed(7)).to(torch.bfloat16)
    kp = torch.randn(b * P, hk, PAGE, D, device=dev, generator=g, dtype=torch.bfloat16)
    vp = torch.randn(b * P, hk, PAGE, D, device=dev, generator=g, dtype=torch.bfloat16)
    table = torch.randperm(b * P, device=dev, generator=g).to(torch.int32)
    plan = msa.fmha_sail_plan(_i32([1] * b), _i32([kl_local] * b), hq, num_kv_heads=hk, page_size=PAGE,
                              causal=(world == 1))
    out = torch.empty(b, hq, D, dtype=torch.bfloat16, device=dev)
    lse = torch.empty(b, hq, dtype=torch.float32, device=dev)
    merged = torch.empty_like(out)
    ex = mdist.DecodeExchange(b, hq, dev) if world > 1 else None

    # several ranks: this rank's unrounded fp32 (O, LSE) go straight into the packed exchange block
    okw = ex.local_kwargs() if world > 1 else dict(out=out, lse=lse)
    o_loc, l_loc = okw["out"], okw["lse"]

    def s_attn():
        msa.fmha_sail(q, kp, vp, plan, kv_indices=table, **okw)

    def s_exchange():
        ex.allgather_merge(out=merged)

    def step():
        s_attn()
        if world > 1:
            s_exchange()

    q_h = q.cpu().pin_memory(); out_h = torch.empty(out.shape, dtype=out.dtype).pin_memory()

    def e2e_step():
        q.copy_(q_h, non_blocking=True)
        step()
        out_h.copy_(merged if world > 1 else out, non_blocking=True)

    def parity():
        """All 64 rows (one token x 64 heads) against the dense oracle, one KV-head group at a time.  With
        several ranks each evaluates the oracle on its own key range; the per-rank (O, LSE) are gathered
        and merged with the oracle's merge, and compared with what the NCCL exchange + merge kernel gave."""
        gsz = hq // hk
        o_ref = torch.empty(b, hq, D); l_ref = torch.empty(b, hq)
        pages = table.long()
        for kh in range(hk):
            kc = kp[pages, kh].reshape(b * P * PAGE, 1, D).cpu()[:kl_local]
            vc = vp[pages, kh].reshape(b * P * PAGE, 1, D).cpu()[:kl_local]
            o_ref[:, kh * gsz:(kh + 1) * gsz], l_ref[:, kh * gsz:(kh + 1) * gsz] = orc.attention_single(
                q[:, kh * gsz:(kh + 1) * gsz].cpu(), kc, vc, gsz, 1, False, 0, return_lse=True)
        r = _compare_rows(o_loc.cpu(), o_ref, 0.9999, 2e-2, "paged decode O (this rank's keys)")
        lerr = (l_loc.cpu() - l_ref).abs().max().item()
        if lerr > 2e-2:
            raise ParityError(f"paged decode LSE off by {lerr:.4g}")
        r["lse_max_abs"] = lerr
        if world > 1:
            po = torch.empty(world, b, hq, D, device=dev); pl = torch.empty(world, b, hq, device=dev)
            dist.all_gather_into_tensor(po.view(-1), o_ref.to(dev).view(-1))
            dist.all_gather_into_tensor(pl.view(-1), l_ref.to(dev).view(-1))
            m_ref = orc.lse_merge(po.cpu(), pl.cpu())
            rm = _compare_rows(merged.cpu(), m_ref, 0.9999, 2e-2, "paged decode O merged over the ranks")
            r.update(merged_max_abs=rm["max_abs"], merged_cos=rm["cos"])
        return r

    nbytes = (kp.numel() + vp.numel()) * 2 + 2 * q.numel() * 2
    stages = dict(attention=(s_attn, nbytes, "GB/s"))
    if world > 1:
        stages["allgather_merge"] = (s_exchange, world * b * hq * (D + 1) * 4, "GB/s")
    return dict(step=step, e2e_step=e2e_step, parity=parity, flops=None, bytes=nbytes, stages=stages,
                unit="GB/s", bound="hbm", launches=2 + (1 if world > 1 else 0),
                graph=(world == 1), tokens=b, h2d=q_h.numel() * 2, d2h=out_h.numel() * 2,
                e2e_note=("public API call with the query copied in from pinned host memory and the result copied "
                          "out each step; the KV cache is device-resident state"),
                l2="inputs larger than L2 (K+V = %.2f GB per GPU)" % (nbytes / 1e9),
                extra_cfg=dict(kv_len_per_gpu=kl_local, num_kv_splits=plan[3]["num_kv_splits"]))


def total_work(kind, w):
    """Algorithmic work of one step of the WHOLE configuration, in the metric's unit numerator (TFLOP or
    GB): what `value` divides by the step time, whatever the number of ranks the units are spread over
    (work a rank repeats, such as the proxy pass of a sequence whose KV-head groups sit on several ranks,
    is not counted twice)."""
    if kind == "prefill":
        return attention_flops(w["b"], w["ql"], w["kl"], w["hq"]) / 1e12
    if kind == "msa_prefill":
        t = w["t"]
        pairs = t * t - t * (t - 1) // 2
        return (w["b"] * pairs * D * 2 + w["b"] * t * w["hq"] * w["topk"] * PAGE * (D + D) * 2) / 1e12
    if kind == "msa_decode":
        e = 1 if w["fp8"] else 2
        P = w["kl"] // PAGE
        sparse = w["b"] * w["hk"] * w["topk"] * PAGE * 2 * D * e + 2 * w["b"] * w["hq"] * D * 2
        proxy = w["b"] * P * PAGE * D * e + P * w["b"] * 4
        return (sparse + proxy) / 1e9
    return (w["b"] * w["kl"] * w["hk"] * 2 * D * 2 + 2 * w["b"] * w["hq"] * D * 2) / 1e9


SETUPS = {"prefill": setup_prefill, "msa_prefill": setup_msa_prefill, "msa_decode": setup_msa_decode,
          "decode": setup_decode}


def config_of(workload, world, graph=True):
    """The `config` object of a workload: a pure function of its name and the rank count, so that the
    CUDA arm and the CPU reference arm print the same one."""
    kind, w = WORKLOADS[workload]
    cfg = dict(workload=workload, **{k: v for k, v in w.items()})
    cfg["n_ranks"] = world
    if kind == "decode":
        cfg["sharding"] = ("KV page range split over the ranks, one NCCL all-gather of packed fp32 (O, LSE) + merge kernel"
                           if world > 1 else "single GPU")
    else:
        cfg["sharding"] = ("the %d independent (batch item, KV-head group) units in contiguous blocks over the ranks, "
                           "no collective" % (w["b"] * w["hk"]) if world > 1 else "single GPU")
    cfg["cuda_graph"] = bool(graph and kind in ("msa_decode", "decode") and (kind != "decode" or world == 1))
    cfg["l2"] = {"prefill": "inputs larger than L2: Q, K, V and O of a step are read / written once",
                 "msa_prefill": "inputs larger than L2: Q and O of a step are larger than L2, the KV cache stays resident",
                 "msa_decode": "every step streams the proxy cache and the selected pages of a cache far larger than L2",
                 "decode": "inputs larger than L2: every step streams the whole K and V of the sequence"}[kind]
    return cfg


# ----------------------------------------------------------------------------------------------
# CPU reference (oracle port) on a bounded sample of the same workload
# ----------------------------------------------------------------------------------------------

def _cpu_pipeline_fn(b, t, hq, hk, topk, koff, n_tok, gen):
    """One pass of the oracle pipeline (proxy scores -> top-k -> sparse attention) for `n_tok` tokens of
    one (sequence, KV-head group) unit -- or, with n_tok = None, for the whole configuration.
    Returns (callable, FLOPs of one call by the workload's formula, description)."""
    from oracle import msa_oracle as orc
    P = t // PAGE
    g = hq // hk
    whole = n_tok is None
    if whole:
        heads_q, heads_k, seqs, pos = hq, hk, b, torch.arange(t)
    else:
        heads_q, heads_k, seqs = g, 1, 1
        pos = torch.linspace(0, t - 1, n_tok).long()                           # spread over the causal triangle
    nt = len(pos)
    q = torch.randn(seqs * nt, heads_q, D, generator=gen).to(torch.bfloat16)
    kp = (torch.randn(seqs * P, heads_k, PAGE, D, generator=gen)
          + math.sqrt(koff) * torch.randn(seqs * P, heads_k, 1, 1, generator=gen)).to(torch.bfloat16)
    vp = torch.randn(seqs * P, heads_k, PAGE, D, generator=gen).to(torch.bfloat16)
    table = torch.randperm(seqs * P, generator=gen).to(torch.int32)
    qx, kx = q[:, :1], kp[:, :1]

    def fn():
        outs = []
        for s in range(seqs):
            kseq = kx[table[s * P:(s + 1) * P].long(), 0].reshape(t, D).float()
            sc = qx[s * nt:(s + 1) * nt, 0].float() @ kseq.t()                 # [nt, t] raw proxy scores
            sc = sc.masked_fill(pos.view(-1, 1) < torch.arange(t).view(1, -1), -float("inf"))
            ms = sc.view(nt, P, PAGE).max(-1).values.t().contiguous().view(1, P, nt)
            sel = orc.topk_select(ms, topk, P)                                  # [nt, 1, topk]
            outs.append(orc.sparse_attention(q[s * nt:(s + 1) * nt], kp, vp, [1] * nt, [t] * nt,
                                             table[s * P:(s + 1) * P].repeat(nt), sel.expand(nt, heads_k, topk),
                                             heads_q, qo_offset=[int(x) for x in pos]))
        return outs

    f_proxy = seqs * int((pos + 1).sum()) * D * 2
    f_sparse = seqs * nt * heads_q * topk * PAGE * (D + D) * 2
    what = (f"the whole pipeline: proxy scores of all {seqs * nt} tokens, top-{topk}, sparse attention of all "
            f"{heads_q} heads" if whole else
            f"one (sequence, KV-head group) unit of the pipeline: proxy scores, top-{topk} and sparse attention "
            f"({g} heads) of {nt} tokens spread over the {t}-token sequence")
    return fn, f_proxy + f_sparse, what


def cpu_reference_sample(workload, seconds_budget, threads):
    """Time the oracle on a bounded sample of the workload; returns (value in the workload's unit,
    seconds per sample, description)."""
    from oracle import msa_oracle as orc
    kind, w = WORKLOADS[workload]
    torch.set_num_threads(threads)
    gen = torch.Generator().manual_seed(0)
    hq, hk = w["hq"], w["hk"]
    g_heads = hq // hk
    units = w["b"] * hk
    if kind == "msa_prefill":
        whole = w["b"] * w["t"] <= 8192
        fn, flops, what = _cpu_pipeline_fn(w["b"], w["t"], hq, hk, w["topk"], w.get("koff", 2.0),
                                           None if whole else 256, gen)
        work = flops / 1e12
        tail = "" if whole else f"; {units} such units of {w['t']} tokens per step"
    elif kind == "prefill":
        ql, kl = w["ql"], w["kl"]
        rows = min(ql, 1024)
        q = (torch.randn(rows, g_heads, D, generator=gen) * 0.5).to(torch.bfloat16)
        k = (torch.randn(kl, 1, D, generator=gen) * 0.5).to(torch.bfloat16)
        v = (torch.randn(kl, 1, D, generator=gen) * 0.5).to(torch.bfloat16)
        off = kl - rows
        pairs = sum(min(kl, i + off + 1) for i in range(rows))
        fn = lambda: orc.attention_single(q, k, v, g_heads, 1, True, off)
        what = (f"one (batch item, KV-head group) unit: dense causal attention, last {rows} of {ql} query tokens x "
                f"{g_heads} heads over {kl} keys")
        work = g_heads * pairs * (D + D) * 2 / 1e12
        tail = f"; {units} such units per step"
    elif kind == "msa_decode":
        kl, topk = w["kl"], w["topk"]
        P = kl // PAGE
        q = torch.randn(1, g_heads, D, generator=gen).to(torch.bfloat16)
        kxs = torch.randn(kl, D, generator=gen).to(torch.bfloat16)
        kp = torch.randn(P, 1, PAGE, D, generator=gen).to(torch.bfloat16)
        vp = torch.randn(P, 1, PAGE, D, generator=gen).to(torch.bfloat16)
        table = torch.randperm(P, generator=gen).to(torch.int32)

        def fn():
            ms = (kxs.float() @ q[0, 0].float()).view(P, PAGE).max(-1).values.view(1, P, 1)
            sel = orc.topk_select(ms, topk, P)
            return orc.sparse_attention(q, kp, vp, [1], [kl], table, sel, g_heads)
        what = (f"one (batch item, KV-head group) unit of the pipeline: proxy scores over {kl} keys (bf16 on the CPU), "
                f"top-{topk}, sparse decode of {g_heads} heads over the selected pages")
        e = 1 if w["fp8"] else 2
        work = (kl * D * e + topk * PAGE * 2 * D * e) / 1e9       # bytes of the GPU workload's formula for this unit
        tail = f"; {units} such units per step (the proxy pass is shared by the {hk} groups of a batch item)"
    else:
        kl = w["kl"]
        keys = min(kl, 131072)
        q = torch.randn(1, g_heads, D, generator=gen).to(torch.bfloat16)
        k = torch.randn(keys, 1, D, generator=gen).to(torch.bfloat16)
        v = torch.randn(keys, 1, D, generator=gen).to(torch.bfloat16)
        fn = lambda: orc.attention_single(q, k, v, g_heads, 1, False, 0)
        work = keys * 2 * D * 2 / 1e9                     # GB of bf16 K+V the unit reads
        what = f"one KV-head group: one decode token x {g_heads} heads over {keys} of the {kl} keys"
        tail = f"; {hk * (kl // keys)} such samples per step"
    t0 = time.perf_counter(); fn(); first = time.perf_counter() - t0
    times = [first] if first > 1.0 else []           # a pass of seconds needs no separate warm-up
    t_end = time.perf_counter() + seconds_budget
    while len(times) < 3 or (time.perf_counter() < t_end and len(times) < 50):
        t0 = time.perf_counter(); fn(); times.append(time.perf_counter() - t0)
    times.sort()
    med = times[len(times) // 2]
    return work / med, med, f"{what}; fp32 torch on CPU, median of {len(times)}{tail}"


def run_reference(args, rank, world):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    kind, w = WORKLOADS[args.workload]
    metric, unit = METRICS[kind]
    vals = []
    for i in range(args.warmup + args.steps):
        v, med, sample = cpu_reference_sample(args.workload, 0.5, threads)
        if i >= args.warmup:
            vals.append((v, med))
    val = sum(x[0] for x in vals) / len(vals)
    ms = sum(x[1] for x in vals) / len(vals) * 1e3
    line = {
        "impl": "reference", "metric": metric, "value": val, "unit": unit, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong" if world > 1 else "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": config_of(args.workload, world, not args.no_graph),
        "cpu_baseline": {"value": val, "unit": unit, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": ("the upstream kernels need T-Head's PPU toolchain and cannot be built here: this arm times the CPU "
                 "oracle port of the same path on the host cores; each step is the bounded sample described in "
                 "cpu_baseline.sample"),
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------
# one measured workload -> one record
# ----------------------------------------------------------------------------------------------

def measure(msa, workload, args, rank, world, local_rank, dev, steps, warmup, with_cpu):
    import torch.distributed as dist
    kind, w = WORKLOADS[workload]
    metric, unit = METRICS[kind]
    params = dict(w)
    if kind == "decode":
        params.update(rank=rank, world=world)
    elif world > 1:
        shp = shard_shape(w["b"], w["hq"], w["hk"], rank, world)
        if shp is None:
            return {"skipped": f"the {w['b'] * w['hk']} (batch item, KV-head group) units of {workload} do not "
                               f"split evenly over {world} ranks"}, None
        params.update(b=shp[0], hq=shp[1], hk=shp[2])
    wl = SETUPS[kind](msa, dev, 1000 + rank, **params)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def graphed(fn):
        """Replay a short step from a CUDA graph, so that the host-side launch path is not what is timed."""
        if not wl["graph"] or args.no_graph:
            return fn, False
        try:
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                fn()
            return gr.replay, True
        except Exception as exc:                                   # noqa: BLE001
            sys.stderr.write(f"graph capture failed ({exc}); timing eager launches\n")
            torch.cuda.synchronize()
            return fn, False

    step, is_graph = graphed(wl["step"])
    stream = torch.cuda.current_stream()
    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(warmup):
        step()
    barrier()
    sampler.mark()
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    evs[0].record(stream)
    for i in range(steps):
        step()
        evs[i + 1].record(stream)
    barrier()
    clocks = sampler.stop()
    total_ms = evs[0].elapsed_time(evs[-1])
    step_ms = total_ms / steps
    if world > 1:
        t = torch.tensor([total_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    ms_per_step = total_ms / steps
    work = wl["flops"] / 1e12 if unit == "TFLOP/s" else wl["bytes"] / 1e9     # what THIS rank's step processes
    whole = total_work(kind, w)                         # the configuration's algorithmic work, all ranks together
    if world == 1 and abs(whole - work) > 1e-6 * whole:
        raise SystemExit(f"{workload}: work formulas disagree ({whole} vs {work})")
    value = whole / (ms_per_step * 1e-3)

    # parity sample of what the timed steps wrote (the eager step once more, so that the outputs are those
    # of the public-API call whether or not the timed loop replayed a graph)
    wl["step"]()
    torch.cuda.synchronize()
    status = msa.api.last_status()
    parity, parity_err = None, None
    try:
        if status:
            raise ParityError(f"device status word {status} (a bounded wait inside a kernel gave up)")
        parity = wl["parity"]()
    except ParityError as exc:
        parity_err = str(exc)
    if world > 1:
        bad = torch.tensor([1 if parity_err else 0], device=dev)
        dist.all_reduce(bad, op=dist.ReduceOp.MAX)
        if int(bad.item()) and not parity_err:
            parity_err = "a parity check failed on another rank"

    # per-stage device times of a pipeline workload
    stage_report = None
    if "stages" in wl:
        stage_report = {}
        for name, (fn, wk, s_unit) in wl["stages"].items():
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            n = max(5, min(steps, 20))
            run, _ = graphed(fn) if name != "allgather_merge" else (fn, False)
            st = torch.cuda.current_stream()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            e0.record(st)
            for _ in range(n):
                run()
            e1.record(st)
            barrier()
            ms = e0.elapsed_time(e1) / n
            if world > 1:
                tt = torch.tensor([ms], device=dev)
                dist.all_reduce(tt, op=dist.ReduceOp.MAX)
                ms = float(tt.item())
            stage_report[name] = {"ms": ms, "value_per_gpu": wk / (1e12 if s_unit == "TFLOP/s" else 1e9) / (ms * 1e-3),
                                  "unit": s_unit}

    e2e = None
    if not args.no_e2e:
        n_e2e = max(2, min(steps, 5 if kind in ("prefill", "msa_prefill") else 50))
        wl["e2e_step"]()
        barrier()
        st = torch.cuda.current_stream()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(st)
        for _ in range(n_e2e):
            wl["e2e_step"]()
        e1.record(st)
        barrier()
        e2e_ms = e0.elapsed_time(e1) / n_e2e
        if world > 1:
            t = torch.tensor([e2e_ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = float(t.item())
        try:
            numa = len([d for d in os.listdir("/sys/devices/system/node") if d.startswith("node") and d[4:].isdigit()])
        except OSError:
            numa = None
        e2e = {"value": whole / (e2e_ms * 1e-3), "unit": unit, "h2d_bytes_per_step": wl["h2d"],
               "d2h_bytes_per_step": wl["d2h"], "ms_per_step": e2e_ms, "steps": n_e2e, "note": wl["e2e_note"],
               "host_numa_nodes": numa,
               "host_binding": ("none: the host exposes one NUMA node, every rank's pinned buffers share its memory "
                                "controllers and PCIe root" if numa == 1 else
                                "none: ranks are not bound to the NUMA node of their GPU")}

    rec = None
    if rank == 0:
        pk = peaks()
        timed_s = total_ms * 1e-3
        if wl["bound"] == "tensor":
            burst = timed_s < 1.0
            f8x = 2.0 if w.get("fp8") else 1.0
            peak = f8x * (pk["bf16"] if burst else pk["bf16_sustained"])
            psrc = pk["src"] + (" cuBLAS bf16, burst figure: the timed region lasts %.2f s" % timed_s if burst else
                                " cuBLAS bf16, sustained figure: the timed region lasts %.2f s" % timed_s)
            if w.get("fp8"):
                psrc += "; x 2 for e4m3 (no fp8 GEMM was measured on this pool: twice the bf16 figure, as the nominal peaks are)"
        else:
            peak, psrc = pk["hbm"], pk["src"] + " (STREAM-style copy)"
        achieved = work / (step_ms * 1e-3)
        roof = {"bound": wl["bound"], "achieved": achieved, "peak": peak,
                "unit": "TFLOP/s" if wl["bound"] == "tensor" else "GB/s", "frac": achieved / peak,
                "traffic": TRAFFIC.get(workload, (None, None))[0] if world == 1 else None,
                "traffic_source": TRAFFIC.get(workload, (None, "not captured"))[1] if world == 1 else "single-GPU captures only",
                "peak_source": psrc, "step_ms": step_ms}
        if wl["bound"] == "tensor":
            roof["frac_of_burst_peak"] = achieved / (f8x * pk["bf16"])
            roof["frac_of_sustained_peak"] = achieved / (f8x * pk["bf16_sustained"])
        cfg = config_of(workload, world, not args.no_graph)
        rec = {
            "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong" if world > 1 else "weak", "vs_baseline": None,
            "dtype": "bf16" if not w.get("fp8") else "e4m3 cache and MMAs, fp32 accumulate", "data": "synthetic",
            "config": cfg, "roofline": roof, "clocks": clocks, "gpu_launches": steps * wl["launches"],
            "tokens_per_s": world * wl["tokens"] / (ms_per_step * 1e-3), "e2e": e2e,
            "parity_sample": parity if parity_err is None else {"failed": parity_err},
            "run": dict(cuda_graph_replay=is_graph, l2=wl["l2"], **wl.get("extra_cfg", {})),
        }
        if stage_report:
            rec["stages"] = stage_report
        if with_cpu and world == 1:
            threads = os.cpu_count() or 1
            v, med, sample = cpu_reference_sample(workload, args.cpu_seconds, threads)
            rec["cpu_baseline"] = {"value": v, "unit": unit, "cores": threads, "kind": "port", "sample": sample}
    del wl
    torch.cuda.empty_cache()
    return rec, parity_err


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS),
                    help="time this workload alone (default: the headline workload plus the sub-records of the other "
                         "BASELINE configurations)")
    ap.add_argument("--no-configs", action="store_true", help="headline workload only")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-seconds", type=float, default=5.0, help="CPU baseline budget per workload")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="do not replay decode steps from a CUDA graph")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    single = args.workload is not None
    headline = args.workload or DEFAULT
    if args.impl == "reference":
        args.workload = headline
        run_reference(args, rank, world)
        return
    args.warmup = max(args.warmup, 3)

    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    import msa_for_sail as msa

    failures = []
    line, err = measure(msa, headline, args, rank, world, local_rank, dev, args.steps, args.warmup,
                        not args.no_cpu_baseline)
    if err:
        failures.append(f"{headline}: {err}")
    if not single and not args.no_configs:
        subs = {}
        for label, name in SUB_CONFIGS:
            kind = WORKLOADS[name][0]
            # short steps need more of them for a stable mean and for the clock sampler to see the region
            steps = args.steps if kind in ("prefill", "msa_prefill") else max(args.steps, 200 if kind == "msa_decode" else 50)
            # (the e4m3 variants share the CPU baseline of configs 2 and 3: same algorithm, same shapes)
            rec, err = measure(msa, name, args, rank, world, local_rank, dev, steps, args.warmup,
                               not args.no_cpu_baseline and not label.endswith("_e4m3"))
            if err:
                failures.append(f"{name}: {err}")
            subs[label] = rec
        if rank == 0:
            line["configs"] = subs
    if rank == 0:
        if failures:
            line["parity_failed"] = failures
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    if failures:
        sys.stderr.write("PARITY FAILED: " + "; ".join(failures) + "\n")
        sys.exit(3)


if __name__ == "__main__":
    main()
