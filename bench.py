#!/usr/bin/env python3
"""Benchmark of the MSA attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

Default workload = BASELINE config 2: dense paged causal prefill, bf16, batch 4,
q_len = kv_len = 8192, 64 query heads / 8 KV heads, head_dim 128, page 128, page tables
seeded random permutations of a 256-page pool.  A step is one `fmha_sail` call over the
batch (the plan is built once, as the upstream API intends: "the plan ... can be reused
across layers").  The metric is effective TFLOP/s: causal-discounted algorithmic FLOPs
(upstream bench_utils.attention_tflops) per second.

Other workloads (--workload): the MSA sparse prefill pipeline (config 3: proxy max-score pass +
page top-k + sparse attention), the MSA sparse decode step over an e4m3 cache (config 4) and the
1M-token paged decode (config 5; with --gpus N the KV range is split over the ranks and the
partial (O, LSE) are combined by an NCCL all-gather + the merge kernel).

Prints ONE JSON line (rank 0).  `--impl reference` times the CPU oracle port of the same
path on the host cores over a bounded sample of the same workload.
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
    # kind, parameters
    "paged_prefill_b4_s8192_h64kv8": ("prefill", dict(b=4, ql=8192, kl=8192, hq=64, hk=8)),
    "paged_prefill_b2_s4096_h32kv4": ("prefill", dict(b=2, ql=4096, kl=4096, hq=32, hk=4)),          # small: ncu
    "msa_prefill_b2_s32768_h64kv8_top16": ("msa_prefill", dict(b=2, t=32768, hq=64, hk=8, topk=16)),
    "msa_prefill_b1_s8192_h32kv4_top16": ("msa_prefill", dict(b=1, t=8192, hq=32, hk=4, topk=16)),   # small: ncu
    "msa_decode_e4m3_b32_kv131072_h64kv8_top16_split4": (
        "msa_decode", dict(b=32, kl=131072, hq=64, hk=8, topk=16, splits=4, fp8=True)),
    "msa_decode_bf16_b32_kv131072_h64kv8_top16_split4": (
        "msa_decode", dict(b=32, kl=131072, hq=64, hk=8, topk=16, splits=4, fp8=False)),
    "msa_decode_e4m3_b8_kv131072_h64kv8_top16_split4": (
        "msa_decode", dict(b=8, kl=131072, hq=64, hk=8, topk=16, splits=4, fp8=True)),                # small: ncu
    "paged_decode_b1_kv1048576_h64kv8": ("decode", dict(b=1, kl=1048576, hq=64, hk=8)),
    "paged_decode_b1_kv131072_h64kv8": ("decode", dict(b=1, kl=131072, hq=64, hk=8)),               # small: ncu
}
DEFAULT = "paged_prefill_b4_s8192_h64kv8"

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


# ----------------------------------------------------------------------------------------------
# workloads: each builds HBM-resident inputs, returns a dict with the step closure and the
# algorithmic work of one step
# ----------------------------------------------------------------------------------------------

def _i32(x):
    return torch.tensor(x, dtype=torch.int32)


def setup_prefill(msa, dev, seed, b, ql, kl, hq, hk):
    g = torch.Generator(device="cpu").manual_seed(seed)
    P = kl // PAGE                                            # pages per sequence
    pool = b * P
    q_h = (torch.randn(b * ql, hq, D, generator=g) * 0.5).to(torch.bfloat16).pin_memory()
    k_h = (torch.randn(pool, hk, PAGE, D, generator=g) * 0.5).to(torch.bfloat16).pin_memory()
    v_h = (torch.randn(pool, hk, PAGE, D, generator=g) * 0.5).to(torch.bfloat16).pin_memory()
    # every sequence owns a slab of P pages; its page table is shuffled within groups of P / NCH pages, so
    # that the pages of the first j row chunks of a sequence are the first j groups of its slab
    NCH = 4 if (ql == kl and P % 4 == 0 and ql % (4 * 256) == 0) else 1     # row chunks per sequence (end to end)
    gp = P // NCH
    local = torch.stack([torch.cat([torch.randperm(gp, generator=g) + j * gp for j in range(NCH)])
                         for _ in range(b)]).to(torch.int32)
    table = (local + torch.arange(b, dtype=torch.int32).view(b, 1) * P).reshape(-1).to(dev)
    q, k, v = q_h.to(dev), k_h.to(dev), v_h.to(dev)
    plan = msa.fmha_sail_plan(_i32([ql] * b), _i32([kl] * b), hq, num_kv_heads=hk, page_size=PAGE)
    out = torch.empty(b * ql, hq, D, dtype=torch.bfloat16, device=dev)
    lse = torch.empty(b * ql, hq, dtype=torch.float32, device=dev)
    out_h = torch.empty(out.shape, dtype=out.dtype).pin_memory()

    def step():
        msa.fmha_sail(q, k, v, plan, kv_indices=table, out=out, lse=lse)

    # end to end: the inputs of a step start in pinned host memory.  One public-API call per row chunk of
    # a sequence (chunked prefill: chunk j attends to the keys of chunks 0..j, whose pages are the first
    # j + 1 groups of the slab), so that the copy-in of the next chunk, the attention of this one and the
    # copy-out of the previous one overlap (three streams; every byte of Q, K, V still crosses PCIe
    # inside the timed region, every byte of O comes back).
    cq = ql // NCH
    plans = [msa.fmha_sail_plan(_i32([cq]), _i32([(j + 1) * cq]), hq, num_kv_heads=hk, page_size=PAGE) for j in range(NCH)]
    local_dev = local.to(dev)
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

    nbytes = (q.numel() + k.numel() + v.numel() + out.numel()) * 2
    return dict(step=step, e2e_step=e2e_step, flops=attention_flops(b, ql, kl, hq), bytes=nbytes, results=(out, out_h),
                metric="prefill_effective_tflops", unit="TFLOP/s", bound="tensor", launches=1, graph=False,
                h2d=(q_h.numel() + k_h.numel() + v_h.numel()) * 2, d2h=out_h.numel() * 2,
                l2="inputs larger than L2 (Q+K+V+O = %.2f GB per GPU)" % (nbytes / 1e9),
                cfg=dict(batch_per_gpu=b, q_len=ql, kv_len=kl, num_qo_heads=hq, num_kv_heads=hk))


def setup_msa_prefill(msa, dev, seed, b, t, hq, hk, topk):
    """Config 3: 1-head proxy max-score pass -> page top-k -> sparse attention on the selection."""
    g = torch.Generator(device=dev).manual_seed(seed)
    P = t // PAGE
    q = torch.randn(b * t, hq, D, device=dev, generator=g).to(torch.bfloat16)
    kp = (torch.randn(b * P, hk, PAGE, D, device=dev, generator=g)
          + math.sqrt(2.0) * torch.randn(b * P, hk, 1, 1, device=dev, generator=g)).to(torch.bfloat16)
    vp = torch.randn(b * P, hk, PAGE, D, device=dev, generator=g).to(torch.bfloat16)
    table = torch.randperm(b * P, device=dev, generator=g).to(torch.int32)
    qx, kx = q[:, :1].contiguous(), kp[:, :1].contiguous()
    lens = _i32([t] * b)
    plan1 = msa.fmha_sail_plan(lens, lens, 1, num_kv_heads=1, page_size=PAGE, output_maxscore=True)
    plan2 = msa.fmha_sail_plan(lens, lens, hq, num_kv_heads=hk, page_size=PAGE, kv_block_num=topk)
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
        pa = msa.fmha_sail_plan(ln_q, ln_k, 1, num_kv_heads=1, page_size=PAGE, output_maxscore=True)
        pb = msa.fmha_sail_plan(ln_q, ln_k, hq, num_kv_heads=hk, page_size=PAGE, kv_block_num=topk)
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

    return dict(step=step, e2e_step=e2e_step, flops=f_proxy + f_sparse, bytes=None, results=(out, out_h),
                stages=dict(proxy=(s_proxy, f_proxy, "TFLOP/s"),
                            topk=(s_topk, ms[:, :P].numel() * 4 + idx.numel() * 4, "GB/s"),
                            sparse=(s_sparse, f_sparse, "TFLOP/s")),
                metric="msa_prefill_effective_tflops", unit="TFLOP/s", bound="tensor", launches=7, graph=False,
                h2d=q_h.numel() * 2, d2h=out_h.numel() * 2,
                l2="inputs larger than L2 (Q+O = %.2f GB per GPU); the KV cache stays resident" % (
                    2 * q.numel() * 2 / 1e9),
                cfg=dict(batch_per_gpu=b, q_len=t, kv_len=t, num_qo_heads=hq, num_kv_heads=hk, topk=topk,
                         proxy_heads=1))


def setup_msa_decode(msa, dev, seed, b, kl, hq, hk, topk, splits, fp8):
    """Config 4: proxy max-score over a 1-head proxy cache -> top-k -> sparse decode with split-KV."""
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

    return dict(step=step, e2e_step=e2e_step, flops=None, bytes=by_sparse + by_proxy,
                stages=dict(proxy=(s_proxy, by_proxy, "GB/s"), topk=(s_topk, ms[:, :P].numel() * 4, "GB/s"),
                            sparse=(s_sparse, by_sparse, "GB/s")),
                metric="msa_decode_kv_gbps", unit="GB/s", bound="hbm", launches=4, graph=True,
                h2d=q_h.numel() * 2, d2h=out_h.numel() * 2,
                l2="every step streams %.0f MB (proxy cache + selected pages) of a %.1f GB cache: larger than L2" % (
                    (by_sparse + by_proxy) / 1e6, (kp.numel() + vp.numel()) * e / 1e9),
                cfg=dict(batch_per_gpu=b, q_len=1, kv_len=kl, num_qo_heads=hq, num_kv_heads=hk, topk=topk,
                         num_kv_splits=splits, num_kv_splits_used=plan2[3]["num_kv_splits"],
                         kv_dtype="e4m3" if fp8 else "bf16", proxy_heads=1))


def setup_decode(msa, dev, seed, b, kl, hq, hk, rank=0, world=1):
    """Config 5: dense paged decode; with world > 1 this rank owns a contiguous slice of the pages."""
    from msa_for_sail import dist as mdist
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
    ws = (torch.empty(world, b, hq, D, dtype=torch.float32, device=dev),
          torch.empty(world, b, hq, dtype=torch.float32, device=dev))

    def step():
        msa.fmha_sail(q, kp, vp, plan, kv_indices=table, out=out, lse=lse)
        if world > 1:
            mdist.decode_allgather_merge(out, lse, out=merged, workspace=ws)

    q_h = q.cpu().pin_memory(); out_h = torch.empty(out.shape, dtype=out.dtype).pin_memory()

    def e2e_step():
        q.copy_(q_h, non_blocking=True)
        step()
        out_h.copy_(merged if world > 1 else out, non_blocking=True)

    nbytes = (kp.numel() + vp.numel()) * 2 + 2 * q.numel() * 2
    return dict(step=step, e2e_step=e2e_step, flops=None, bytes=nbytes,
                metric="decode_kv_gbps", unit="GB/s", bound="hbm", launches=2 + (1 if world > 1 else 0),
                graph=(world == 1), h2d=q_h.numel() * 2, d2h=out_h.numel() * 2,
                l2="inputs larger than L2 (K+V = %.2f GB per GPU)" % (nbytes / 1e9),
                cfg=dict(batch=b, q_len=1, kv_len=kl, kv_len_per_gpu=kl_local, num_qo_heads=hq, num_kv_heads=hk,
                         num_kv_splits=plan[3]["num_kv_splits"]))


SETUPS = {"prefill": setup_prefill, "msa_prefill": setup_msa_prefill, "msa_decode": setup_msa_decode,
          "decode": setup_decode}
METRICS = {"prefill": ("prefill_effective_tflops", "TFLOP/s"), "msa_prefill": ("msa_prefill_effective_tflops", "TFLOP/s"),
           "msa_decode": ("msa_decode_kv_gbps", "GB/s"), "decode": ("decode_kv_gbps", "GB/s")}


# ----------------------------------------------------------------------------------------------
# CPU reference (oracle port) on a bounded sample of the same workload
# ----------------------------------------------------------------------------------------------

def cpu_reference_sample(workload, seconds_budget, threads):
    """Time the oracle on one independent unit of the workload; returns (value in the workload's
    unit, seconds per sample, description)."""
    from oracle import msa_oracle as orc
    kind, w = WORKLOADS[workload]
    torch.set_num_threads(threads)
    gen = torch.Generator().manual_seed(0)
    hq, hk = w["hq"], w["hk"]
    g_heads = hq // hk
    if kind in ("prefill", "msa_prefill"):
        ql = w.get("ql", w.get("t")); kl = w.get("kl", w.get("t"))
        rows = min(ql, 1024)
        q = (torch.randn(rows, g_heads, D, generator=gen) * 0.5).to(torch.bfloat16)
        if kind == "prefill":
            k = (torch.randn(kl, 1, D, generator=gen) * 0.5).to(torch.bfloat16)
            v = (torch.randn(kl, 1, D, generator=gen) * 0.5).to(torch.bfloat16)
            off = kl - rows
            pairs = sum(min(kl, i + off + 1) for i in range(rows))
            fn = lambda: orc.attention_single(q, k, v, g_heads, 1, True, off)
            what = f"dense causal attention, last {rows} of {ql} query tokens x {g_heads} heads over {kl} keys"
        else:
            keys = w["topk"] * PAGE                       # the keys a token actually attends to
            k = torch.randn(keys, 1, D, generator=gen).to(torch.bfloat16)
            v = torch.randn(keys, 1, D, generator=gen).to(torch.bfloat16)
            pairs = rows * keys
            fn = lambda: orc.attention_single(q, k, v, g_heads, 1, False, 0)
            what = (f"attention of {rows} query tokens x {g_heads} heads over {keys} selected keys "
                    f"(one shared page list, gather not timed)")
        work = g_heads * pairs * (D + D) * 2 / 1e12
    else:
        kl = w["kl"]
        keys = w["topk"] * PAGE if kind == "msa_decode" else min(kl, 131072)
        q = torch.randn(1, g_heads, D, generator=gen).to(torch.bfloat16)
        k = torch.randn(keys, 1, D, generator=gen).to(torch.bfloat16)
        v = torch.randn(keys, 1, D, generator=gen).to(torch.bfloat16)
        fn = lambda: orc.attention_single(q, k, v, g_heads, 1, False, 0)
        work = keys * 2 * D * 2 / 1e9                     # GB of bf16 K+V the unit reads
        what = f"one decode token x {g_heads} heads over {keys} keys"
    fn()
    times = []
    t_end = time.perf_counter() + seconds_budget
    while len(times) < 3 or (time.perf_counter() < t_end and len(times) < 50):
        t0 = time.perf_counter(); fn(); times.append(time.perf_counter() - t0)
    times.sort()
    med = times[len(times) // 2]
    return work / med, med, (f"one (batch item, KV-head group) unit: {what}; fp32 torch on CPU, median of "
                             f"{len(times)}; {w['b'] * hk} such units per step")


def run_reference(args, rank):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    kind, w = WORKLOADS[args.workload]
    metric, unit = METRICS[kind]
    vals = []
    for i in range(args.warmup + args.steps):
        v, med, sample = cpu_reference_sample(args.workload, 1.0, threads)
        if i >= args.warmup:
            vals.append((v, med))
    val = sum(x[0] for x in vals) / len(vals)
    ms = sum(x[1] for x in vals) / len(vals) * 1e3
    line = {
        "impl": "reference", "metric": metric, "value": val, "unit": unit, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": dict(workload=args.workload, **w),
        "cpu_baseline": {"value": val, "unit": unit, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default=DEFAULT, choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="do not replay decode steps from a CUDA graph")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    args.warmup = max(args.warmup, 3)

    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    import msa_for_sail as msa

    kind, w = WORKLOADS[args.workload]
    strong = kind == "decode" and world > 1            # one sequence: its KV range is split over the ranks
    if kind == "decode":
        wl = SETUPS[kind](msa, dev, 1000 + rank, rank=rank, world=world, **w)
    else:
        wl = SETUPS[kind](msa, dev, 1000 + rank, **w)
    stream = torch.cuda.current_stream()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    step = wl["step"]
    graphed = False
    if wl["graph"] and not args.no_graph:
        # decode steps are a few tens of microseconds: replay them from a CUDA graph so that the
        # host-side launch path is not what gets measured
        try:
            for _ in range(3):
                step()
            torch.cuda.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                step()
            step, graphed = gr.replay, True
        except Exception as exc:                                   # noqa: BLE001
            sys.stderr.write(f"graph capture failed ({exc}); timing eager launches\n")
            torch.cuda.synchronize()
    stream = torch.cuda.current_stream()

    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(args.warmup):
        step()
    barrier()
    sampler.mark()
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    evs[0].record(stream)
    for i in range(args.steps):
        step()
        evs[i + 1].record(stream)
    barrier()
    clocks = sampler.stop()
    total_ms = evs[0].elapsed_time(evs[-1])
    per = sorted(evs[i].elapsed_time(evs[i + 1]) for i in range(args.steps))
    step_ms = sum(per) / len(per)
    if world > 1:
        t = torch.tensor([total_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    work = wl["flops"] / 1e12 if wl["unit"] == "TFLOP/s" else wl["bytes"] / 1e9
    value = world * work / (ms_per_step * 1e-3)        # strong scaling: every rank holds 1/world of the bytes

    # per-stage device times of a pipeline workload
    stage_report = None
    if "stages" in wl:
        stage_report = {}
        for name, (fn, wk, unit) in wl["stages"].items():
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            n = max(5, min(args.steps, 20))
            run = fn
            if wl["graph"] and not args.no_graph:
                try:
                    gs = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(gs):
                        fn()
                    run = gs.replay
                except Exception:                                  # noqa: BLE001
                    torch.cuda.synchronize()
            st = torch.cuda.current_stream()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(st)
            for _ in range(n):
                run()
            e1.record(st)
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / n
            stage_report[name] = {"ms": ms, "value": wk / (1e12 if unit == "TFLOP/s" else 1e9) / (ms * 1e-3),
                                  "unit": unit}

    e2e = None
    if not args.no_e2e:
        n_e2e = max(2, min(args.steps, 5 if kind in ("prefill", "msa_prefill") else 50))
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
        e2e = {"value": world * work / (e2e_ms * 1e-3), "unit": wl["unit"], "h2d_bytes_per_step": wl["h2d"],
               "d2h_bytes_per_step": wl["d2h"], "ms_per_step": e2e_ms, "steps": n_e2e,
               "note": ("chunked prefill through the public API, four row chunks per sequence; the copy-in of a chunk's Q "
                        "rows and K/V pages from pinned host memory, its attention and the copy-out of its O overlap "
                        "with the neighbouring chunks on three streams"
                        if kind == "prefill" else
                        "chunked prefill through the public API, eight row chunks per sequence: the copy-in of a chunk's Q "
                        "from pinned host memory, its proxy pass, top-k and sparse attention and the copy-out of its O "
                        "overlap with the neighbouring chunks on three streams; the KV cache is device-resident state"
                        if kind == "msa_prefill" else
                        "public API call with pinned host tensors copied in and the result copied out each step; "
                        "the KV cache is device-resident state")}

    if rank == 0:
        pk = peaks()
        if wl["bound"] == "tensor":
            peak, psrc = pk["bf16_sustained"], pk["src"] + " (sustained cuBLAS bf16: kernel timed inside a long loop)"
        else:
            peak, psrc = pk["hbm"], pk["src"] + " (STREAM-style copy)"
        achieved = work / (step_ms * 1e-3)
        line = {
            "metric": wl["metric"], "value": value, "unit": wl["unit"], "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong" if strong else "weak", "vs_baseline": None,
            "dtype": "bf16" if not w.get("fp8") else "e4m3 cache, fp16 math", "data": "synthetic",
            "config": dict(workload=args.workload, l2=wl["l2"], cuda_graph=graphed,
                           sharding=("KV page range split over ranks, NCCL all-gather of (O, LSE) + merge kernel"
                                     if strong else "independent (batch, KV-head group) units per GPU, no collective"),
                           **wl["cfg"]),
            "roofline": {"bound": wl["bound"], "achieved": achieved, "peak": peak,
                         "unit": "TFLOP/s" if wl["bound"] == "tensor" else "GB/s", "frac": achieved / peak,
                         "traffic": TRAFFIC.get(args.workload, (None, None))[0],
                         "traffic_source": TRAFFIC.get(args.workload, (None, "not captured"))[1],
                         "peak_source": psrc, "step_ms": step_ms},
            "clocks": clocks, "gpu_launches": args.steps * wl["launches"], "e2e": e2e,
        }
        if stage_report:
            line["stages"] = stage_report
        if not args.no_cpu_baseline and world == 1:
            threads = os.cpu_count() or 1
            v, med, sample = cpu_reference_sample(args.workload, 12.0, threads)
            line["cpu_baseline"] = {"value": v, "unit": wl["unit"], "cores": threads, "kind": "port", "sample": sample}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
