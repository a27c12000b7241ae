#!/usr/bin/env python3
"""Benchmark of the MSA attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

Default workload = BASELINE config 2: dense paged causal prefill, bf16, batch 4,
q_len = kv_len = 8192, 64 query heads / 8 KV heads, head_dim 128, page 128, page tables
seeded random permutations of a 256-page pool.  A step is one `fmha_sail` call over the
batch (the plan is built once, as the upstream API intends: "the plan ... can be reused
across layers").  The metric is effective TFLOP/s: causal-discounted algorithmic FLOPs
(upstream bench_utils.attention_tflops) per second.

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
    # name: (batch, q_len, kv_len, h_q, h_kv)
    "paged_prefill_b4_s8192_h64kv8": (4, 8192, 8192, 64, 8),
    "paged_prefill_b2_s4096_h32kv4": (2, 4096, 4096, 32, 4),      # small case for ncu captures (150 MB)
}
DEFAULT = "paged_prefill_b4_s8192_h64kv8"


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
        self.rows, self.proc, self.index = [], None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
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
        self.rows = self.rows[getattr(self, 'first', 0):]
        clk = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in self.rows if len(r) >= 6 for i in range(4) if r[2 + i] == "Active"})
        return {"sm_mhz": clk[len(clk) // 2] if clk else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(clk)}


def make_inputs(workload, device, seed):
    b, ql, kl, hq, hk = WORKLOADS[workload]
    g = torch.Generator(device="cpu").manual_seed(seed)
    pages_per = kl // PAGE
    pool = b * pages_per
    q = (torch.randn(b * ql, hq, D, generator=g) * 0.5).to(torch.bfloat16)
    k = (torch.randn(pool, hk, PAGE, D, generator=g) * 0.5).to(torch.bfloat16)
    v = (torch.randn(pool, hk, PAGE, D, generator=g) * 0.5).to(torch.bfloat16)
    table = torch.randperm(pool, generator=g).to(torch.int32)
    return q, k, v, table


def cpu_reference_sample(workload, seconds_budget, threads):
    """Time the oracle on ONE (batch item, KV-head group) unit of the workload, restricted to the
    last `rows` query tokens so the sample stays bounded; returns TFLOP/s over that sample."""
    from oracle import msa_oracle as orc
    b, ql, kl, hq, hk = WORKLOADS[workload]
    torch.set_num_threads(threads)
    g_heads = hq // hk
    rows = min(ql, 1024)
    gen = torch.Generator().manual_seed(0)
    q = (torch.randn(rows, g_heads, D, generator=gen) * 0.5).to(torch.bfloat16)
    k = (torch.randn(kl, 1, D, generator=gen) * 0.5).to(torch.bfloat16)
    v = (torch.randn(kl, 1, D, generator=gen) * 0.5).to(torch.bfloat16)
    off = kl - rows
    pairs = sum(min(kl, i + off + 1) for i in range(rows))
    flops = g_heads * pairs * (D + D) * 2
    orc.attention_single(q, k, v, g_heads, 1, True, off)           # warm-up
    times = []
    t_end = time.perf_counter() + seconds_budget
    while len(times) < 3 or (time.perf_counter() < t_end and len(times) < 20):
        t0 = time.perf_counter()
        orc.attention_single(q, k, v, g_heads, 1, True, off)
        times.append(time.perf_counter() - t0)
    times.sort()
    med = times[len(times) // 2]
    sample = (f"one (batch item, KV-head group) unit, last {rows} of {ql} query tokens x {g_heads} heads "
              f"over {kl} keys, fp32 torch on CPU, median of {len(times)}; {b * hk} such units per step")
    return flops / med / 1e12, med, sample


def run_reference(args, rank, world):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    wl = args.workload
    b, ql, kl, hq, hk = WORKLOADS[wl]
    vals = []
    for i in range(args.warmup + args.steps):
        tf, med, sample = cpu_reference_sample(wl, 2.0, threads)
        if i >= args.warmup:
            vals.append((tf, med))
    tf = sum(v[0] for v in vals) / len(vals)
    ms = sum(v[1] for v in vals) / len(vals) * 1e3
    line = {
        "impl": "reference", "metric": "prefill_effective_tflops", "value": tf, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl, "batch": b, "q_len": ql, "kv_len": kl, "num_qo_heads": hq,
                   "num_kv_heads": hk, "head_dim": D, "page_size": PAGE},
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
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
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    import msa_for_sail as msa

    wl = args.workload
    b, ql, kl, hq, hk = WORKLOADS[wl]
    q_h, k_h, v_h, table_h = make_inputs(wl, dev, seed=1000 + rank)
    q_h, k_h, v_h = q_h.pin_memory(), k_h.pin_memory(), v_h.pin_memory()
    q, k, v, table = q_h.to(dev), k_h.to(dev), v_h.to(dev), table_h.to(dev)
    lens = torch.full((b,), ql, dtype=torch.int32)
    kv_lens = torch.full((b,), kl, dtype=torch.int32)
    plan = msa.fmha_sail_plan(lens, kv_lens, hq, num_kv_heads=hk, page_size=PAGE)
    out = torch.empty(b * ql, hq, D, dtype=torch.bfloat16, device=dev)
    lse = torch.empty(b * ql, hq, dtype=torch.float32, device=dev)
    flops = attention_flops(b, ql, kl, hq)
    stream = torch.cuda.current_stream()

    def step():
        msa.fmha_sail(q, k, v, plan, kv_indices=table, out=out, lse=lse)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

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
    kernel_ms = sum(per) / len(per)                     # one launch per step: step time == kernel time
    if world > 1:
        t = torch.tensor([total_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    value = world * flops / (ms_per_step * 1e-3) / 1e12

    # end to end: host buffers in, host result out, through the public API
    e2e = None
    if not args.no_e2e:
        out_h = torch.empty(out.shape, dtype=out.dtype).pin_memory()
        n_e2e = max(2, min(args.steps, 5))

        def e2e_step():
            qd = q_h.to(dev, non_blocking=True); kd = k_h.to(dev, non_blocking=True)
            vd = v_h.to(dev, non_blocking=True)
            o, _ = msa.fmha_sail(qd, kd, vd, plan, kv_indices=table)
            out_h.copy_(o, non_blocking=True)

        e2e_step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(n_e2e):
            e2e_step()
        e1.record(stream)
        barrier()
        e2e_ms = e0.elapsed_time(e1) / n_e2e
        if world > 1:
            t = torch.tensor([e2e_ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = float(t.item())
        e2e = {"value": world * flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": q_h.numel() * 2 + k_h.numel() * 2 + v_h.numel() * 2,
               "d2h_bytes_per_step": out_h.numel() * 2, "ms_per_step": e2e_ms, "steps": n_e2e}

    if rank == 0:
        pk = peaks()
        peak = pk["bf16_sustained"]
        achieved = flops / (kernel_ms * 1e-3) / 1e12
        line = {
            "metric": "prefill_effective_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": wl, "batch_per_gpu": b, "global_batch": b * world, "q_len": ql, "kv_len": kl,
                       "num_qo_heads": hq, "num_kv_heads": hk, "head_dim": D, "page_size": PAGE,
                       "l2": "inputs larger than L2 (Q+K+V+O = %.2f GB per GPU)" % (
                           (q.numel() + k.numel() + v.numel() + out.numel()) * 2 / 1e9),
                       "sharding": "independent (batch, KV-head group) units per GPU, no collective"},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak, "traffic": None,
                         "peak_source": pk["src"] + " (sustained cuBLAS bf16, kernel timed inside a loop)",
                         "kernel_ms": kernel_ms},
            "clocks": clocks, "gpu_launches": args.steps, "e2e": e2e,
        }
        if not args.no_cpu_baseline and world == 1:
            threads = os.cpu_count() or 1
            tf, med, sample = cpu_reference_sample(wl, 12.0, threads)
            line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                                    "sample": sample}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
