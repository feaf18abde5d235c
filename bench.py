#!/usr/bin/env python
"""Benchmark of the KV-cache + decode-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One "step" = what one layer does for one decode step of every sequence of the batch: append one
K/V token per sequence (quantise-on-append for the quantised formats), then GQA attention of the
new query over the whole cache.  Default workload: BASELINE config 4 (16 sequences, past 32768,
block-32 int8 KV, 32 query / 8 KV heads, head_dim 128, f16 queries).  With N GPUs every rank runs
its own batch (sequences are independent: no collective on the data path; weak scaling).

Prints ONE JSON line: `value` = KV bytes read per second, summed over GPUs, with the inputs resident
in HBM; `e2e` = the same through the C ABI with host buffers (H2D of q / k_new / v_new and D2H of the
output inside the timed region); `roofline` = the decode kernel alone against the measured HBM
copy rate; `cpu_baseline` = the CPU restatement of tract's own algorithm on this box's host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# name -> (format, io dtype, sequences per GPU, past length (int or "ragged"), description)
WORKLOADS = {
    "cfg4-q8": ("q8_1", "f16", 16, 32768, "BASELINE config 4: batch 16, past 32768, Q8 block-32 KV (f16 scale + int8 codes)"),
    "cfg4-q4": ("q4_0", "f16", 16, 32768, "BASELINE config 4, 4-bit variant (Q4_0)"),
    "cfg4-f16": ("f16", "f16", 16, 32768, "config 4 shape with an unquantised f16 cache"),
    "cfg4-kivi8": ("kivi8", "f16", 16, 32768, "config 4 shape with tract's own KIVI int8 storage (QuantizedDynKeyValueCache)"),
    "cfg4-kivi4": ("kivi4", "f16", 16, 32768, "config 4 shape with tract's own KIVI int4 storage"),
    "cfg3-bf16": ("bf16", "bf16", 256, "ragged", "BASELINE config 3: 256 sequences, past ~ U[512,16384], bf16"),
    "cfg1-f32": ("f32", "f32", 1, 2048, "BASELINE config 1: batch 1, past 2048, f32"),
}
# prefill workloads: name -> (io dtype, sequences per GPU, past tokens, chunk tokens, description)
PREFILL = {
    "cfg2-prefill": ("f16", 1, 0, 512, "BASELINE config 2: 512-token chunk appended to an empty cache, causal Sdpa 512x512, f16"),
    "prefill-2k": ("f16", 1, 0, 2048, "config 2 geometry with a 2048-token chunk"),
    "prefill-8k": ("f16", 1, 0, 8192, "config 2 geometry with an 8192-token chunk"),
    "prefill-32k": ("f16", 1, 0, 32768, "config 2 geometry with a 32768-token chunk"),
    "prefill-chunked": ("f16", 8, 7680, 512, "8 sequences, a 512-token chunk after 7680 cached tokens"),
}
HQ, HKV, D = 32, 8, 128
OVERRIDE = {}  # --seqs / --past: smaller cases of a workload, for profiler captures
# DRAM traffic of the decode kernel per algorithmic byte (dram__bytes_read + dram__bytes_write over the K/V bytes of the
# launch), from the ncu captures summarised under profiles/ on a smaller case of the same workload (traffic grows in
# proportion to the tokens streamed, so it is scaled to the full launch by the units processed).
NCU_TRAFFIC_RATIO = {"q8_1": 1.018}
ROW_BYTES = {"f32": 512, "f16": 256, "bf16": 256, "q8_1": 128 + 8, "q4_0": 64 + 8,
             # KIVI: K = codes + 2 x D f32 parameters per 32 tokens, V = codes + 8 bytes per token; mean of K and V
             "kivi8": 128 + (32 + 8) // 2, "kivi4": 64 + (32 + 8) // 2}  # stored bytes per token-head (codes + scales)


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return json.load(open(p)), "measured"
    return {"hbm_gbs": 6650.0}, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines, self.t_mark = index, None, [], None

    def mark(self):
        """Start of the timed region: samples from 0.3 s before this point on are reported."""
        self.t_mark = time.time() - 0.3

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            def pump():
                for ln in self.proc.stdout:
                    self.lines.append((time.time(), ln))

            self.thread = threading.Thread(target=pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.06)
        self.proc.terminate()
        self.thread.join(timeout=2)
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ts, ln in self.lines:
            if self.t_mark is not None and ts < self.t_mark:
                continue
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 6 or not f[0].isdigit():
                continue
            sm.append(int(f[0]))
            mx = int(f[1])
            for n, val in zip(names, f[2:6]):
                if val == "Active":
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def draw_lengths(workload, rank):
    fmt, io, n_seq, past, _ = WORKLOADS[workload]
    if OVERRIDE.get("seqs"):
        n_seq = OVERRIDE["seqs"]
    if OVERRIDE.get("past"):
        past = OVERRIDE["past"]
    if past == "ragged":  # config 3: uniform integer in [512, 16384], seeded per rank
        g = np.random.Generator(np.random.Philox(key=1234 + rank))
        return [int(x) for x in g.integers(512, 16385, size=n_seq)]
    return [int(past)] * n_seq


def kv_bytes_per_step(workload, lens):
    """Algorithmic bytes: K and V of every cached token (past + the new one) read once."""
    fmt = WORKLOADS[workload][0]
    return 2 * HKV * ROW_BYTES[fmt] * sum(n + 1 for n in lens)


# ---------------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------------

def fill_cache(torch, cache, seqs, lens, io_dt, seed):
    """Pre-fills the past: N(0,1) with 1% of the elements multiplied by 20 (config 4's distribution)."""
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    order = sorted(range(len(seqs)), key=lambda i: lens[i])
    chunk = 4096
    done = 0
    while done < max(lens):
        live = [i for i in order if lens[i] > done]
        # sequences that still need tokens, grouped by how many they take in this round
        groups = {}
        for i in live:
            groups.setdefault(min(chunk, lens[i] - done), []).append(i)
        for n, idx in groups.items():
            for j in range(0, len(idx), 32):
                part = idx[j:j + 32]
                shape = (len(part), HKV, n, D)
                k = torch.randn(shape, generator=gen, device="cuda", dtype=torch.float32)
                v = torch.randn(shape, generator=gen, device="cuda", dtype=torch.float32)
                k = torch.where(torch.rand(shape, generator=gen, device="cuda") < 0.01, k * 20, k).to(io_dt)
                v = torch.where(torch.rand(shape, generator=gen, device="cuda") < 0.01, v * 20, v).to(io_dt)
                cache.append([seqs[i] for i in part], k, v)
        done += chunk
    torch.cuda.synchronize()


def run_ours(args, rank, world):
    import torch

    import tract_b200 as kv

    kv.lib()
    dev = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(dev)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{dev}"))
    fmt, io, n_seq, _, desc = WORKLOADS[args.workload]
    io_dt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[io]
    lens = draw_lengths(args.workload, rank)
    n_seq = len(lens)
    # a KIVI store cannot be truncated back after a step (finalised blocks are frozen), so its sequences grow by one
    # token per step and get head-room for every step this run makes
    grows = fmt.startswith("kivi")
    room = 128 + (4 * args.steps + 256 if grows else 0)
    cache = kv.KvCache(fmt, HKV, D, max_seqs=n_seq, max_seq_tokens=max(lens) + room, pool_tokens=sum(lens) + (room - 64) * n_seq)
    seqs = [cache.new_seq() for _ in range(n_seq)]
    fill_cache(torch, cache, seqs, lens, io_dt, seed=99 + rank)

    gen = torch.Generator(device="cuda")
    gen.manual_seed(7 + rank)
    q = torch.randn((n_seq, HQ, 1, D), generator=gen, device="cuda").to(io_dt)
    k_new = torch.randn((n_seq, HKV, 1, D), generator=gen, device="cuda").to(io_dt)
    v_new = torch.randn((n_seq, HKV, 1, D), generator=gen, device="cuda").to(io_dt)
    out = torch.empty_like(q)
    # host-side copy for the end-to-end leg: q | k | v of a step as the rows of one pinned buffer (what a fused q/k/v
    # projection leaves behind), one host-to-device copy per step; the cache calls take the three windows through strides
    hqkv = torch.cat([q, k_new, v_new], 1).cpu().pin_memory()
    dqkv = torch.empty((n_seq, HQ + 2 * HKV, 1, D), dtype=io_dt, device="cuda")
    dq, dk, dv = dqkv[:, :HQ], dqkv[:, HQ:HQ + HKV], dqkv[:, HQ + HKV:]
    hout = torch.empty_like(out, device="cpu").pin_memory()

    def step():
        cache.append_attend(seqs, k_new, v_new, q, causal=True, out=out)
        if not grows:
            for s, n in zip(seqs, lens):  # host bookkeeping only: keep the past length fixed from step to step
                cache.truncate(s, n)

    def step_e2e():
        dqkv.copy_(hqkv, non_blocking=True)
        cache.append_attend(seqs, dk, dv, dq, causal=True, out=out)
        hout.copy_(out, non_blocking=True)
        if not grows:
            for s, n in zip(seqs, lens):
                cache.truncate(s, n)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        barrier()
        ms = a.elapsed_time(b)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    sampler = ClockSampler(dev)
    if rank == 0:
        sampler.start()
    n_warm, t_w = 0, time.perf_counter()
    floor_s = 0.0 if (args.quick or grows) else 1.0
    while n_warm < max(args.warmup, 3) or time.perf_counter() - t_w < floor_s:  # >= W steps and >= 1 s under load
        step()
        n_warm += 1
        if n_warm % 16 == 0:
            torch.cuda.synchronize()
    sampler.mark()
    ms = timed(step, args.steps)
    clocks = sampler.stop() if rank == 0 else None
    for _ in range(3):
        step_e2e()
    ms_e2e = timed(step_e2e, args.steps)

    # per-kernel durations (event pairs inside the library), for the roofline of the decode kernel
    cache.profile(True)
    torch.cuda.synchronize()
    for _ in range(args.steps):
        step()
    recs = cache.profile_read()
    cache.profile(False)
    cache.check()
    per_kernel = {}
    for name, t in recs:
        per_kernel.setdefault(name, []).append(t)

    total_bytes = kv_bytes_per_step(args.workload, lens)
    if world > 1:
        t = torch.tensor([float(total_bytes), float(n_seq)], device="cuda", dtype=torch.float64)
        dist.all_reduce(t)
        all_bytes, all_seqs = float(t[0].item()), float(t[1].item())
    else:
        all_bytes, all_seqs = float(total_bytes), float(n_seq)
    result = None
    if rank == 0:
        pk, pk_kind = peaks()
        ms_step = ms / args.steps
        dec_ms = statistics.mean(per_kernel["decode"])
        achieved = total_bytes / (dec_ms * 1e-3) / 1e9
        h2d = hqkv.numel() * hqkv.element_size()
        d2h = hout.numel() * hout.element_size()
        result = {
            "metric": "decode-attn KV-read GB/s (sum over GPUs; per GPU = value / n_gpus)",
            "value": all_bytes / (ms_step * 1e-3) / 1e9,
            "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": {"q8_1": "int8 codes x f16 scale -> f32", "q4_0": "int4 codes x f16 scale -> f32"}.get(fmt, f"{fmt} -> f32"),
            "data": "synthetic",
            "config": {"workload": args.workload, "description": desc, "sequences_per_gpu": n_seq,
                       "past_tokens": lens[0] if len(set(lens)) == 1 else {"min": min(lens), "max": max(lens), "sum": sum(lens)},
                       "q_heads": HQ, "kv_heads": HKV, "head_dim": D, "io_dtype": io, "kv_format": fmt,
                       "parallelism": f"by-sequence x{world}, no collective",
                       "l2": "inputs larger than L2" if total_bytes > 2 * 126e6 else "working set fits L2 (warm)",
                       "kv_bytes_per_step_per_gpu": total_bytes},
            "tokens_per_s": all_seqs / (ms_step * 1e-3),
            "vs_nominal_8TBps_per_gpu": all_bytes / world / (ms_step * 1e-3) / 8e12,
            "e2e": {"value": all_bytes / (ms_e2e / args.steps * 1e-3) / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e / args.steps,
                    "tokens_per_s": all_seqs / (ms_e2e / args.steps * 1e-3)},
            "gpu_launches": len(recs),
            "kernels_ms": {k: statistics.mean(v) for k, v in per_kernel.items()},
            "roofline": {"bound": "hbm", "kernel": "kivi_decode_kernel" if fmt.startswith("kivi") else ("decode_kernel" if fmt == "f32" else "decode_mma_kernel"), "achieved": achieved, "peak": pk["hbm_gbs"],
                         "unit": "GB/s", "frac": achieved / pk["hbm_gbs"], "peak_kind": pk_kind,
                         "algorithmic_bytes": total_bytes,
                         "traffic": int(total_bytes * NCU_TRAFFIC_RATIO[fmt]) if fmt in NCU_TRAFFIC_RATIO else None,
                         "traffic_source": "profiles/decode_mma_q8_b8_p16384.md, scaled by tokens" if fmt in NCU_TRAFFIC_RATIO else None,
                         "frac_of_nominal_8TBps": achieved / 8000.0},
            "clocks": clocks,
        }
    cache.close()
    return result


def run_prefill(args, rank, world):
    """Prefill chunk: append S tokens per sequence, then causal attention of the S queries over the cache.
    Metric: causal-useful attention TFLOP/s (4 * Hq * D * sum over queries of visible keys)."""
    import torch

    import tract_b200 as kv

    dev = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(dev)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{dev}"))
    io, n_seq, past, S, desc = PREFILL[args.workload]
    io_dt = {"f16": torch.float16, "bf16": torch.bfloat16}[io]
    cache = kv.KvCache(io, HKV, D, max_seqs=n_seq, max_seq_tokens=past + S + 128)
    seqs = [cache.new_seq() for _ in range(n_seq)]
    if past:
        fill_cache(torch, cache, seqs, [past] * n_seq, io_dt, seed=11 + rank)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(3 + rank)
    mk = lambda h: (torch.randn((n_seq, h, S, D), generator=gen, device="cuda") * 0.5).to(io_dt)
    q, k_new, v_new = mk(HQ), mk(HKV), mk(HKV)
    out = torch.empty_like(q)
    hq, hk, hv = (t.cpu().pin_memory() for t in (q, k_new, v_new))
    hout = torch.empty_like(out, device="cpu").pin_memory()
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k_new), torch.empty_like(v_new)

    def step():
        cache.append(seqs, k_new, v_new)
        cache.attend(seqs, q, causal=True, out=out)
        for s in seqs:
            cache.truncate(s, past)

    def step_e2e():
        dq.copy_(hq, non_blocking=True), dk.copy_(hk, non_blocking=True), dv.copy_(hv, non_blocking=True)
        cache.append(seqs, dk, dv)
        cache.attend(seqs, dq, causal=True, out=out)
        hout.copy_(out, non_blocking=True)
        for s in seqs:
            cache.truncate(s, past)

    def timed(fn, steps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    sampler = ClockSampler(dev)
    if rank == 0:
        sampler.start()
    n_warm, t_w = 0, time.perf_counter()
    while n_warm < max(args.warmup, 3) or time.perf_counter() - t_w < (0.0 if args.quick else 1.0):
        step()
        n_warm += 1
        if n_warm % 8 == 0:
            torch.cuda.synchronize()
    sampler.mark()
    ms = timed(step, args.steps)
    clocks = sampler.stop() if rank == 0 else None
    for _ in range(3):
        step_e2e()
    ms_e2e = timed(step_e2e, args.steps)
    cache.profile(True)
    torch.cuda.synchronize()
    for _ in range(args.steps):
        step()
    recs = cache.profile_read()
    cache.profile(False)
    cache.check()
    per_kernel = {}
    for name, t in recs:
        per_kernel.setdefault(name, []).append(t)
    useful = 4.0 * HQ * D * n_seq * sum(past + i + 1 for i in range(S))  # causal-useful flops per step per GPU
    result = None
    if rank == 0:
        pk, pk_kind = peaks()
        ms_step = ms / args.steps
        k_ms = statistics.mean(per_kernel["prefill"])
        achieved = useful / (k_ms * 1e-3) / 1e12
        peak = pk.get("bf16_tflops", 1590.0)
        h2d = sum(t.numel() * t.element_size() for t in (hq, hk, hv))
        result = {
            "metric": "prefill causal-useful attention TFLOP/s (sum over GPUs)", "value": world * useful / (ms_step * 1e-3) / 1e12,
            "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": f"{io} operands, f32 accumulation",
            "data": "synthetic",
            "config": {"workload": args.workload, "description": desc, "sequences_per_gpu": n_seq, "past_tokens": past,
                       "chunk_tokens": S, "q_heads": HQ, "kv_heads": HKV, "head_dim": D, "io_dtype": io,
                       "parallelism": f"by-sequence x{world}, no collective",
                       "l2": "working set fits L2 (warm)" if (past + S) * n_seq * HKV * D * 4 < 100e6 else "inputs larger than L2",
                       "flops_per_step_per_gpu": useful},
            "tokens_per_s": world * n_seq * S / (ms_step * 1e-3),
            "e2e": {"value": world * useful / (ms_e2e / args.steps * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": hout.numel() * hout.element_size(), "ms_per_step": ms_e2e / args.steps},
            "gpu_launches": len(recs), "kernels_ms": {k: statistics.mean(v) for k, v in per_kernel.items()},
            "roofline": {"bound": "tensor", "kernel": "prefill_tc_kernel", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak, "peak_kind": pk_kind + " (bf16 cuBLAS burst)", "traffic": None,
                         "flops": "causal-useful (masked half of the diagonal tiles not counted)"},
            "clocks": clocks,
        }
    cache.close()
    return result


# ---------------------------------------------------------------------------------------------------
# CPU arm: the restatement of tract's own CPU algorithm (the Rust reference cannot be built here)
# ---------------------------------------------------------------------------------------------------

LINEAR = {
    # the Q4_0 linear layers of the BASELINE config 5 decoder shape (hidden 4096, FFN 14336), 8 sequences per GPU;
    # `layers` distinct weight matrices are walked per step so that the weights of a step exceed L2
    "q40-ffn-up": dict(n=14336, k=4096, m=8, layers=8, desc="FFN gate/up projection [14336 x 4096], Q4_0, 8 activation rows"),
    "q40-ffn-down": dict(n=4096, k=14336, m=8, layers=8, desc="FFN down projection [4096 x 14336], Q4_0, 8 activation rows"),
    "q40-attn-proj": dict(n=4096, k=4096, m=8, layers=32, desc="attention q / o projection [4096 x 4096], Q4_0, 8 activation rows"),
    "q40-gemv": dict(n=14336, k=4096, m=1, layers=8, desc="FFN gate/up projection, one activation row (GEMV)"),
    # a prompt pass: 512 activation rows through the same matrix (the many-rows kernel; bound by the per-block f32 scaling, not by HBM)
    "q40-ffn-up-m512": dict(n=14336, k=4096, m=512, layers=2, desc="FFN gate/up projection [14336 x 4096], Q4_0, 512 activation rows (prompt pass)"),
}


def run_linear(args, rank, world):
    """Q4_0 weights x int8-quantised activations (Q4_0::w4a8_gemm arithmetic): weight bytes per second against HBM."""
    import torch
    import torch.distributed as dist
    import tract_b200 as kv
    import oracle

    wl = LINEAR[args.workload]
    n, k, m, layers = wl["n"], wl["k"], wl["m"], wl["layers"]
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    g = torch.Generator(device="cpu").manual_seed(4242 + rank)
    # random blocks are valid Q4_0 weights: any nibbles, f16 scales drawn positive and small
    lins = []
    for _ in range(layers):
        blocks = torch.randint(0, 256, (n, k // 32, 18), dtype=torch.uint8, generator=g)
        scales = (torch.rand((n, k // 32), generator=g) * 0.05 + 0.001).to(torch.float16)
        blocks[:, :, :2] = scales.view(torch.uint8).reshape(n, k // 32, 2)
        lins.append(kv.Q40Linear(blocks.to(dev), max_m=m))
    a_host = torch.randn((m, k), generator=g).pin_memory()
    a_dev = a_host.to(dev)
    out = torch.empty((m, n), dtype=torch.float32, device=dev)
    out_host = torch.empty((m, n), dtype=torch.float32).pin_memory()
    weight_bytes = layers * n * (k // 32) * 18

    def launch_all():
        for lin in lins:
            lin.gemm(a_dev, out)

    # the step is launch bound from Python (2 launches per layer): replay it as a CUDA graph, as a decode loop would
    launch_all()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        launch_all()
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            launch_all()
    torch.cuda.synchronize()

    def step():
        graph.replay()

    def step_e2e():
        a_dev.copy_(a_host, non_blocking=True)
        step()
        out_host.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    sampler = ClockSampler(dev.index or 0)
    if rank == 0:
        sampler.start()
    for _ in range(max(args.warmup, 3)):
        step()
    sampler.mark()
    ms = timed(step, args.steps)
    clocks = sampler.stop() if rank == 0 else None
    ms_e2e = timed(step_e2e, max(10, args.steps // 10)) / max(10, args.steps // 10)
    lins[0].check()
    ms_step = ms / args.steps
    # the GEMM kernel alone, timed on the launching stream
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(20):
        step()
    e1.record()
    torch.cuda.synchronize()
    kern_ms = e0.elapsed_time(e1) / 20
    pk, pk_kind = peaks()
    value = world * weight_bytes / (ms_step * 1e-3) / 1e9
    achieved = weight_bytes / (kern_ms * 1e-3) / 1e9
    if rank == 0:
        line = {
            "metric": "Q4_0 weight-read GB/s (sum over GPUs)", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "u4 weights x s8 activations, s32 block dot products, f32 accumulation", "data": "synthetic",
            "config": {"workload": args.workload, "description": wl["desc"], "n": n, "k": k, "activation_rows": m, "layers_per_step": layers, "launch": "one CUDA graph replay per step",
                       "weight_bytes_per_step_per_gpu": weight_bytes, "parallelism": f"replicas x{world}, no collective",
                       "l2": "weights of one step exceed L2" if weight_bytes > 126e6 else "weights fit L2 (warm)"},
            "tokens_per_s": world * m * layers / (ms_step * 1e-3),
            "e2e": {"value": world * weight_bytes / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": m * k * 4,
                    "d2h_bytes_per_step": m * n * 4, "ms_per_step": ms_e2e},
            "gpu_launches": 2 * layers,
            "roofline": {"bound": "hbm", "kernel": ("q40_gemm_rows_kernel" if m > 24 else "q40_gemm_kernel") + " (+ activation quantiser)", "achieved": achieved, "peak": pk["hbm_gbs"],
                         "unit": "GB/s", "frac": achieved / pk["hbm_gbs"], "peak_kind": pk_kind, "traffic": None,
                         "algorithmic_bytes": weight_bytes},
            "clocks": clocks,
        }
        if not args.no_cpu_baseline:
            import time
            sc = np.random.default_rng(1).integers(0, 65535, (min(n, 512), k // 32)).astype(np.uint16) & 0x2fff
            pkd = np.random.default_rng(2).integers(0, 256, (min(n, 512), k // 2)).astype(np.uint8)
            a_np = a_host.numpy()
            thr = oracle.hardware_threads()
            t0 = time.perf_counter()
            reps = 0
            while time.perf_counter() - t0 < 5.0:
                oracle.w4a8_gemm(sc, pkd, a_np, threads=thr)
                reps += 1
            dt = (time.perf_counter() - t0) / reps
            line["cpu_baseline"] = {"value": min(n, 512) * (k // 32) * 18 / dt / 1e9, "unit": "GB/s", "cores": thr, "kind": "port",
                                    "sample": f"{min(n, 512)} of the {n} output rows of one layer, {m} activation rows, {reps} repetitions"}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


DECODER = {
    # BASELINE config 5: the Llama-3-8B shape, Q4_0 weights from a seed, 8 sequences per GPU (64 over 8 GPUs), caches at
    # 2048 tokens (filled with synthetic K / V: the prompt pass needs the large-M GEMM, which is not built), greedy steps
    "cfg5-decoder": dict(past=2048, seqs=8, kv="f16", desc="32-layer Llama-3-8B-shaped decoder, Q4_0 weights, f16 KV cache, 8 sequences x 2048 cached tokens, greedy decode"),
    "cfg5-decoder-q8kv": dict(past=2048, seqs=8, kv="q8_1", desc="the same with the int8 block-32 KV cache"),
    # the pp512 / tg128 methodology of the reference's llm bench (cli/src/llm.rs:47-139): a real prompt pass, then decode steps
    "cfg5-pp512": dict(past=0, prompt=512, seqs=8, kv="f16", desc="the same decoder: 512-token prompt pass through the model (timed), then greedy decode"),
}


def run_decoder(args, rank, world):
    import torch
    import torch.distributed as dist
    from tract_b200.decoder import Decoder, Shape

    wl = DECODER[args.workload]
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    sh = Shape()
    B, past = args.seqs or wl["seqs"], args.past or wl["past"]
    dec = Decoder(sh, n_seqs=B, max_tokens=past + wl.get("prompt", 0) + args.steps + max(args.warmup, 3) + 64, kv_format=wl["kv"], seed=100 + rank,
                  device=dev)
    pp = None
    if wl.get("prompt"):
        P = wl["prompt"]
        prompt = torch.randint(0, sh.vocab, (B, P), dtype=torch.int32)
        dec.prefill(prompt)  # warm-up (lazy allocations, attribute calls)
        torch.cuda.synchronize()
        dec.reset()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        dec.prefill(prompt)
        e1.record()
        torch.cuda.synchronize()
        pp = {"prompt_tokens": B * P, "ms": e0.elapsed_time(e1), "tokens_per_s": B * P / (e0.elapsed_time(e1) * 1e-3)}
        past = P
    else:
        dec.prefill_synthetic(past)
    tok_host = torch.randint(0, sh.vocab, (B,), dtype=torch.int32).pin_memory()
    out_host = torch.empty(B, dtype=torch.int32).pin_memory()
    dec.set_tokens(tok_host)

    def step():
        dec.step()

    def step_e2e():
        dec.tokens.copy_(tok_host, non_blocking=True)
        dec.step()
        out_host.copy_(dec.tokens, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def timed(fn, steps):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    sampler = ClockSampler(dev.index or 0)
    if rank == 0:
        sampler.start()
    for _ in range(max(args.warmup, 3)):
        step()
    sampler.mark()
    n_e2e = max(1, min(args.steps // 4, args.steps - 1))  # the steps are shared between the device-timed and the end-to-end loop
    n_dev = max(1, args.steps - n_e2e)
    ms = timed(step, n_dev) / n_dev
    clocks = sampler.stop() if rank == 0 else None
    ms_e2e = timed(step_e2e, n_e2e) / n_e2e
    # the hot-path share: one layer's cache kernels, timed by the library's own event pairs
    c0 = dec.layers[0]["cache"]
    c0.profile(True)
    torch.cuda.synchronize()
    dec.step()
    recs = dict()
    for name, t in c0.profile_read():
        recs.setdefault(name, []).append(t)
    c0.profile(False)
    dec.check()
    weight_bytes = sum(L[k].packed.numel() for L in dec.layers for k in ("wqkv", "wo", "wgu", "wd")) + dec.lm_head.packed.numel()
    kv_bytes = sh.n_layers * B * (past + args.steps // 2) * sh.n_kv_heads * sh.head_dim * 2 * (2 if wl["kv"] == "f16" else 1.0625)
    pk, pk_kind = peaks()
    if rank == 0:
        line = {
            "metric": "decode tokens/s of the full decoder (sum over GPUs)", "value": world * B / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "Q4_0 weights x int8 activations, f32 residual stream, 16-bit attention", "data": "synthetic",
            "config": {"workload": args.workload, "description": wl["desc"], "sequences_per_gpu": B, "cached_tokens": past,
                       "layers": sh.n_layers, "hidden": sh.hidden, "ffn": sh.ffn, "vocab": sh.vocab, "vocab_note": "assumed (not given by the config)",
                       "parallelism": f"by-sequence x{world}, no collective", "l2": "weights (4.2 GB) and caches exceed L2",
                       "weight_bytes_per_step": weight_bytes, "kv_bytes_per_step": kv_bytes,
                       "launch": "CUDA-graph segments between cache calls; cache calls from the host"},
            "e2e": {"value": world * B / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": B * 4, "d2h_bytes_per_step": B * 4,
                    "ms_per_step": ms_e2e},
            "gpu_launches": sh.n_layers * 10 + 6,  # per layer: 4 GEMMs, 3 quantising producers, append, decode, combine (which quantises for wo)
            "kernels_ms": {k: statistics.mean(v) for k, v in recs.items()},
            "prompt_pass": pp,
            "roofline": {"bound": "hbm", "kernel": "whole step (Q4_0 GEMMs dominate)", "achieved": (weight_bytes + kv_bytes) / (ms * 1e-3) / 1e9,
                         "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": (weight_bytes + kv_bytes) / (ms * 1e-3) / 1e9 / pk["hbm_gbs"],
                         "peak_kind": pk_kind, "traffic": None, "algorithmic_bytes": weight_bytes + kv_bytes},
            "clocks": clocks,
        }
        print(json.dumps(line))
    dec.close()
    if world > 1:
        dist.destroy_process_group()


def cpu_step_factory(workload, sample_seqs, sample_past, threads):
    """Returns (step_fn, bytes_per_step): one decode step of `sample_seqs` sequences on the CPU:
    quantise the new token, dequantise the whole cache (what QuantizedDynKvCacheState::eval does every
    step, quant_dyn_kv_cache.rs:483-495), then FlashSdpaOp over it."""
    import oracle

    fmt, io, _, _, _ = WORKLOADS[workload]
    g = np.random.Generator(np.random.Philox(key=5))
    T = sample_past + 1
    np_io = {"f32": np.float32, "f16": np.float16, "bf16": oracle.bfloat16}[io]
    k = g.standard_normal((sample_seqs, HKV, T, D), dtype=np.float32)
    v = g.standard_normal((sample_seqs, HKV, T, D), dtype=np.float32)
    q = g.standard_normal((sample_seqs, HQ, 1, D), dtype=np.float32).astype(np_io)
    if fmt == "q8_1":
        ks, _, kc = oracle.q8_1_quant(k)
        vs, _, vc = oracle.q8_1_quant(v)
    elif fmt == "q4_0":
        ks, kc = oracle.q4_0_quant(k)
        vs, vc = oracle.q4_0_quant(v)
    else:
        k, v = k.astype(np_io), v.astype(np_io)

    def step():
        if fmt == "q8_1":
            oracle.q8_1_quant(k[:, :, -1:])
            oracle.q8_1_quant(v[:, :, -1:])
            kd, vd = oracle.q8_1_dequant(ks, kc), oracle.q8_1_dequant(vs, vc)
        elif fmt == "q4_0":
            oracle.q4_0_quant(k[:, :, -1:])
            oracle.q4_0_quant(v[:, :, -1:])
            kd, vd = oracle.q4_0_dequant(ks, kc), oracle.q4_0_dequant(vs, vc)
        else:
            kd = oracle.dyn_kv_concat(k[:, :, :-1], k[:, :, -1:])
            vd = oracle.dyn_kv_concat(v[:, :, :-1], v[:, :, -1:])
        return oracle.flash_sdpa(q, kd, vd, causal=True, threads=threads)

    return step, 2 * HKV * ROW_BYTES[fmt] * sample_seqs * T


def cpu_baseline(workload, budget_s=12.0):
    import oracle

    threads = oracle.hardware_threads()
    fmt, io, n_seq, past, _ = WORKLOADS[workload]
    sample_past = 8192 if past == "ragged" else int(past)
    sample_seqs = max(1, min(n_seq, 2))
    step, nbytes = cpu_step_factory(workload, sample_seqs, sample_past, threads)
    step()
    t0 = time.perf_counter()
    n = 0
    while n < 2 or time.perf_counter() - t0 < budget_s:
        step()
        n += 1
        if n >= 50:
            break
    dt = (time.perf_counter() - t0) / n
    return {"value": nbytes / dt / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"{sample_seqs} of {n_seq} sequences, past {sample_past}, {n} steps of "
                      f"{dt * 1e3:.1f} ms (append-quantise 1 token, dequantise cache, flash attention)",
            "tokens_per_s": sample_seqs / dt}


def run_reference(args, rank, world):
    if rank != 0:
        return None
    import oracle

    threads = oracle.hardware_threads()
    if args.workload not in WORKLOADS:
        return {"impl": "reference", "unavailable": f"the CPU arm times the decode workloads only ({', '.join(sorted(WORKLOADS))}); "
                                                    f"the {args.workload} line carries its own cpu_baseline where it has one"}
    fmt, io, n_seq, past, desc = WORKLOADS[args.workload]
    sample_past = 8192 if past == "ragged" else int(past)
    sample_seqs = max(1, min(n_seq, 2))
    step, nbytes = cpu_step_factory(args.workload, sample_seqs, sample_past, threads)
    for _ in range(min(args.warmup, 1) or 1):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    val = nbytes / dt / 1e9
    sample = (f"each step = {sample_seqs} of {n_seq} sequences, past {sample_past}: append-quantise 1 token, "
              f"dequantise cache, flash attention, on {threads} host threads")
    return {"impl": "reference", "metric": "decode-attn KV-read GB/s (sum over GPUs; per GPU = value / n_gpus)",
            "value": val, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": 1, "ms_per_step": dt * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": args.workload, "description": desc, "kv_format": fmt, "io_dtype": io,
                       "q_heads": HQ, "kv_heads": HKV, "head_dim": D},
            "note": "tract is Rust and no cargo/rustc exists on this image: this arm times the CPU restatement of "
                    "tract's own algorithm (oracle/), the same code the parity tests check against",
            "tokens_per_s": sample_seqs / dt,
            "cpu_baseline": {"value": val, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="cfg4-q8", choices=sorted(WORKLOADS) + sorted(PREFILL) + sorted(LINEAR) + sorted(DECODER))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--quick", action="store_true", help="profiler runs: exactly W warm-up steps, no 1 s warm-up floor")
    ap.add_argument("--seqs", type=int, default=0, help="override sequences per GPU (profiling: smaller case)")
    ap.add_argument("--past", type=int, default=0, help="override the past length (profiling: smaller case)")
    args = ap.parse_args()
    OVERRIDE.update(seqs=args.seqs, past=args.past)
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    if args.impl == "reference":
        if args.steps > 10:
            args.steps = 10  # each CPU step takes seconds; keep the run within minutes
        r = run_reference(args, rank, world)
        if r:
            print(json.dumps(r))
        return
    if args.workload in LINEAR:
        run_linear(args, rank, world)
        return
    if args.workload in DECODER:
        if args.steps > 256:
            args.steps = 64  # the default step count is sized for the attention-only workloads
        run_decoder(args, rank, world)
        return
    if args.workload in PREFILL:
        r = run_prefill(args, rank, world)
        if rank == 0:
            print(json.dumps(r))
        return
    r = run_ours(args, rank, world)
    if rank == 0:
        if not args.no_cpu_baseline and world == 1:
            r["cpu_baseline"] = cpu_baseline(args.workload)
        elif world > 1:
            r["cpu_baseline"] = {"note": "timed at N=1 only"}
        print(json.dumps(r))
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


if __name__ == "__main__":
    main()
