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
copy rate; `cpu_baseline` = the CPU restatement of tract's own algorithm on this box's host cores;
`secondary` (default workload only) = short runs of the other configurations, each with its kernel time,
roofline fraction and end-to-end figure.

Timing: the K steps asked for are repeated R times back to back (R from a short calibration, so that the
timed region lasts at least `--min-seconds`) between one pair of CUDA events; ms_per_step = time / (K * R).
"""
from __future__ import annotations

import argparse
import json
import math
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
# prefill workloads: name -> (cache format, io dtype, sequences per GPU, past tokens, chunk tokens, description)
PREFILL = {
    "cfg2-prefill": ("f16", "f16", 1, 0, 512, "BASELINE config 2: 512-token chunk appended to an empty cache, causal Sdpa 512x512, f16"),
    "prefill-2k": ("f16", "f16", 1, 0, 2048, "config 2 geometry with a 2048-token chunk"),
    "prefill-8k": ("f16", "f16", 1, 0, 8192, "config 2 geometry with an 8192-token chunk"),
    "prefill-32k": ("f16", "f16", 1, 0, 32768, "config 2 geometry with a 32768-token chunk"),
    "prefill-chunked": ("f16", "f16", 8, 7680, 512, "8 sequences, a 512-token chunk after 7680 cached tokens"),
    "prefill-chunked-q8": ("q8_1", "f16", 8, 7680, 512, "8 sequences, a 512-token chunk after 7680 cached tokens, int8 block-32 KV cache"),
    "prefill-chunked-q4": ("q4_0", "f16", 8, 7680, 512, "8 sequences, a 512-token chunk after 7680 cached tokens, Q4_0 KV cache"),
    "prefill-chunked-kivi8": ("kivi8", "f16", 8, 7680, 512, "8 sequences, a 512-token chunk after 7680 cached tokens, KIVI int8 KV cache"),
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
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines, self.t_mark = index, None, [], None

    def mark(self):
        """Start of the timed region: samples from 0.1 s before this point on are reported."""
        self.t_mark = time.time() - 0.1

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


class Ctx:
    """One process per GPU: device, process group (NCCL, only for the timing barrier / max-over-ranks and the optional
    head-sharded all-gather), and the timing primitives every workload uses."""

    def __init__(self, rank, world):
        import torch

        self.torch, self.rank, self.world = torch, rank, world
        self.dev_index = int(os.environ.get("LOCAL_RANK", 0))
        torch.cuda.set_device(self.dev_index)
        self.dev = torch.device("cuda", self.dev_index)
        self.dist = None
        if world > 1:
            import torch.distributed as dist

            dist.init_process_group("nccl", device_id=self.dev)
            self.dist = dist

    def barrier(self):
        if self.dist:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, x):
        if not self.dist:
            return float(x)
        t = self.torch.tensor([float(x)], device=self.dev, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(self, *xs):
        if not self.dist:
            return [float(x) for x in xs]
        t = self.torch.tensor([float(x) for x in xs], device=self.dev, dtype=self.torch.float64)
        self.dist.all_reduce(t)
        return [float(v) for v in t.tolist()]

    def timed(self, fn, iters):
        """Milliseconds of `iters` calls of fn between two CUDA events on the current stream, a barrier and a device
        synchronisation on both sides, the maximum over the ranks."""
        torch = self.torch
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.barrier()
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        self.barrier()
        return self.max_over_ranks(a.elapsed_time(b))

    def measure(self, fn, steps, min_seconds, sampler=None, max_iters=None):
        """ms per step of fn: `steps` iterations repeated R times, R chosen from a calibration run of `steps` iterations
        (untimed, counted as warm-up) so that the timed region lasts at least min_seconds.  Returns (ms_per_step, R, timed_ms)."""
        cal = self.timed(fn, steps)
        reps = max(1, int(math.ceil(min_seconds * 1e3 / max(cal, 1e-3))))
        if max_iters:
            reps = max(1, min(reps, max_iters // steps))
        if sampler:
            sampler.mark()
        total = self.timed(fn, steps * reps)
        return total / (steps * reps), reps, total

    def close(self):
        if self.dist:
            self.dist.destroy_process_group()


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


def decode_config(workload, lens, world):
    """The `config` object of a decode workload: the same keys on our line and on the reference arm's."""
    fmt, io, _, _, desc = WORKLOADS[workload]
    total_bytes = kv_bytes_per_step(workload, lens)
    return {"workload": workload, "description": desc, "sequences_per_gpu": len(lens),
            "past_tokens": lens[0] if len(set(lens)) == 1 else {"min": min(lens), "max": max(lens), "sum": sum(lens)},
            "q_heads": HQ, "kv_heads": HKV, "head_dim": D, "io_dtype": io, "kv_format": fmt,
            "parallelism": f"by-sequence x{world}, no collective",
            "l2": "inputs larger than L2" if total_bytes > 2 * 126e6 else "working set fits L2 (warm)",
            "kv_bytes_per_step_per_gpu": total_bytes}


# ---------------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------------

def fill_cache(torch, cache, seqs, lens, io_dt, seed, n_kv=HKV, also=None):
    """Pre-fills the past: N(0,1) with 1% of the elements multiplied by 20 (config 4's distribution).  `also`: a second
    (cache, seqs, head slice) that receives the same tokens (the head-sharded check)."""
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
                shape = (len(part), n_kv, n, D)
                k = torch.randn(shape, generator=gen, device="cuda", dtype=torch.float32)
                v = torch.randn(shape, generator=gen, device="cuda", dtype=torch.float32)
                k = torch.where(torch.rand(shape, generator=gen, device="cuda") < 0.01, k * 20, k).to(io_dt)
                v = torch.where(torch.rand(shape, generator=gen, device="cuda") < 0.01, v * 20, v).to(io_dt)
                cache.append([seqs[i] for i in part], k, v)
                if also:
                    c2, s2, lo, hi = also
                    c2.append([s2[i] for i in part], k[:, lo:hi], v[:, lo:hi])
        done += chunk
    torch.cuda.synchronize()


def run_decode(ctx, workload, steps, warmup, min_seconds, quick=False, primary=True):
    """One decode workload on this rank's GPU.  Returns the full JSON line (rank 0; None elsewhere)."""
    torch = ctx.torch
    import tract_b200 as kv

    kv.lib()
    rank, world = ctx.rank, ctx.world
    fmt, io, n_seq, _, desc = WORKLOADS[workload]
    io_dt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[io]
    lens = draw_lengths(workload, rank)
    n_seq = len(lens)
    # a KIVI store cannot be truncated back after a step (finalised blocks are frozen), so its sequences grow by one
    # token per step: the run is held to a few hundred steps and the sequences get head-room for them
    grows = fmt.startswith("kivi")
    if grows:
        min_seconds = min(min_seconds, 0.15)
    room = 128 + (8192 if grows else 0)
    cache = kv.KvCache(fmt, HKV, D, max_seqs=n_seq, max_seq_tokens=max(lens) + room, pool_tokens=sum(lens) + (room - 64) * n_seq,
                       max_q_heads=HQ)
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
    out_e2e = torch.empty_like(q)
    hout = torch.empty_like(out, device="cpu").pin_memory()

    # one call into the library per step: append + attend, then (host bookkeeping only) the sequences go back to their
    # past length together, so that every step streams the same bytes
    back = None if grows else lens
    step = cache.prepared_step(seqs, k_new, v_new, q, out, rollback_to=back)
    core_e2e = cache.prepared_step(seqs, dk, dv, dq, out_e2e, rollback_to=back)

    def step_e2e():
        dqkv.copy_(hqkv, non_blocking=True)
        core_e2e()
        hout.copy_(out_e2e, non_blocking=True)

    sampler = ClockSampler(ctx.dev_index)
    if rank == 0 and primary:
        sampler.start()
    n_warm, t_w = 0, time.perf_counter()
    floor_s = 0.0 if (quick or grows or not primary) else 1.0
    while n_warm < max(warmup, 3) or time.perf_counter() - t_w < floor_s:  # >= W steps and >= 1 s under load
        step()
        n_warm += 1
        if n_warm % 16 == 0:
            torch.cuda.synchronize()
    cap = 2000 if grows else None  # a KIVI cache grows by one token per step: bounded by the head-room
    grown0 = cache.seq_len(seqs[0]) - lens[0]
    ms_step, reps, timed_ms = ctx.measure(step, steps, min_seconds, sampler, max_iters=cap)
    clocks = sampler.stop() if (rank == 0 and primary) else None
    for _ in range(3):
        step_e2e()
    grown1 = cache.seq_len(seqs[0]) - lens[0]
    ms_e2e, reps_e2e, _ = ctx.measure(step_e2e, steps, min_seconds, max_iters=cap)
    # the end-to-end leg drives the library through strided windows of one buffer: its result, read back on the host,
    # must be the device-resident result of the dense leg bit for bit (same inputs, same past)
    e2e_checked = None
    if not grows:
        step()
        step_e2e()
        torch.cuda.synchronize()
        e2e_checked = bool(torch.equal(hout, out.cpu()))
        if not e2e_checked:
            raise SystemExit(f"{workload}: the end-to-end output differs from the device-resident one")

    # per-kernel durations (event pairs inside the library), for the roofline of the decode kernel
    cache.profile(True)
    torch.cuda.synchronize()
    n_prof = min(max(steps, 20), 200)
    for _ in range(n_prof):
        step()
    recs = cache.profile_read()
    cache.profile(False)
    cache.check()
    per_kernel = {}
    for name, t in recs:
        per_kernel.setdefault(name, []).append(t)
    final_lens = [cache.seq_len(s) for s in seqs]

    # a KIVI cache has grown by one token per step: its figures use the mean length over each timed region
    total_bytes = bytes_e2e = kv_bytes_per_step(workload, lens)
    if grows:
        total_bytes = int(2 * HKV * ROW_BYTES[fmt] * sum(n + 1 + grown0 + steps + steps * reps / 2.0 for n in lens))
        bytes_e2e = int(2 * HKV * ROW_BYTES[fmt] * sum(n + 1 + grown1 + steps + steps * reps_e2e / 2.0 for n in lens))
    all_bytes, all_seqs, all_bytes_e2e = ctx.sum_over_ranks(total_bytes, n_seq, bytes_e2e)
    result = None
    if rank == 0:
        pk, pk_kind = peaks()
        dec_ms = statistics.median(per_kernel["decode"])
        dec_bytes = total_bytes if not grows else int(2 * HKV * ROW_BYTES[fmt] * sum(final_lens))
        achieved = dec_bytes / (dec_ms * 1e-3) / 1e9
        h2d = hqkv.numel() * hqkv.element_size()
        d2h = hout.numel() * hout.element_size()
        kernel = ("kivi_mma_kernel" if fmt.startswith("kivi") else ("decode_kernel" if fmt == "f32" else "decode_mma_kernel"))
        cfg = decode_config(workload, lens, world)
        cfg["timed_region"] = {"repeats_of_the_steps": reps, "ms": timed_ms, "min_seconds": min_seconds}
        result = {
            "metric": "decode-attn KV-read GB/s (sum over GPUs; per GPU = value / n_gpus)",
            "value": all_bytes / (ms_step * 1e-3) / 1e9,
            "unit": "GB/s",
            "n_gpus": world, "steps": steps, "warmup": max(warmup, 3), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": {"q8_1": "int8 codes x f16 scale -> f32", "q4_0": "int4 codes x f16 scale -> f32"}.get(fmt, f"{fmt} -> f32"),
            "data": "synthetic",
            "config": cfg,
            "tokens_per_s": all_seqs / (ms_step * 1e-3),
            "vs_nominal_8TBps_per_gpu": all_bytes / world / (ms_step * 1e-3) / 8e12,
            "e2e": {"value": all_bytes_e2e / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e,
                    "tokens_per_s": all_seqs / (ms_e2e * 1e-3), "output_equals_device_result": e2e_checked},
            "gpu_launches": steps * reps * 3,  # append, decode, combine per step, inside the timed region
            "kernels_ms": {k: statistics.median(v) for k, v in per_kernel.items()},
            "roofline": {"bound": "hbm", "kernel": kernel, "achieved": achieved, "peak": pk["hbm_gbs"],
                         "unit": "GB/s", "frac": achieved / pk["hbm_gbs"], "peak_kind": pk_kind,
                         "algorithmic_bytes": dec_bytes, "kernel_ms": dec_ms,
                         "traffic": int(total_bytes * NCU_TRAFFIC_RATIO[fmt]) if fmt in NCU_TRAFFIC_RATIO else None,
                         "traffic_source": "profiles/decode_mma_q8_b8_p16384.md, scaled by tokens" if fmt in NCU_TRAFFIC_RATIO else None,
                         "frac_of_nominal_8TBps": achieved / 8000.0},
            "clocks": clocks,
        }
        if clocks and clocks.get("sm_mhz"):
            # the product that stays put when two boxes differ only in the clock the power cap lets them hold
            result["roofline"]["kernel_ms_x_sm_mhz"] = dec_ms * clocks["sm_mhz"]
            result["ms_per_step_x_sm_mhz"] = ms_step * clocks["sm_mhz"]
    cache.close()
    del cache
    torch.cuda.empty_cache()
    return result


def run_prefill(ctx, workload, steps, warmup, min_seconds, quick=False, primary=True):
    """Prefill chunk: append S tokens per sequence, then causal attention of the S queries over the cache.
    Metric: causal-useful attention TFLOP/s (4 * Hq * D * sum over queries of visible keys)."""
    torch = ctx.torch
    import tract_b200 as kv

    rank, world = ctx.rank, ctx.world
    fmt, io, n_seq, past, S, desc = PREFILL[workload]
    io_dt = {"f16": torch.float16, "bf16": torch.bfloat16}[io]
    cache = kv.KvCache(fmt, HKV, D, max_seqs=n_seq, max_seq_tokens=past + S + 128, max_q_heads=HQ)
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
    if fmt.startswith("kivi"):
        # a KIVI store cannot be rolled back (a finalised key block does not come apart): the chunk is appended once, before
        # the timed region, and a step is the attention of its S queries over the past + S cached tokens
        cache.append(seqs, k_new, v_new)
        step = lambda: cache.attend(seqs, q, out=out)

        def step_e2e():
            dq.copy_(hq, non_blocking=True)
            cache.attend(seqs, dq, out=out)
            hout.copy_(out, non_blocking=True)
    else:
        back = [past] * n_seq
        step = cache.prepared_step(seqs, k_new, v_new, q, out, rollback_to=back)
        core_e2e = cache.prepared_step(seqs, dk, dv, dq, out, rollback_to=back)

        def step_e2e():
            dq.copy_(hq, non_blocking=True), dk.copy_(hk, non_blocking=True), dv.copy_(hv, non_blocking=True)
            core_e2e()
            hout.copy_(out, non_blocking=True)

    sampler = ClockSampler(ctx.dev_index)
    if rank == 0 and primary:
        sampler.start()
    n_warm, t_w = 0, time.perf_counter()
    while n_warm < max(warmup, 3) or time.perf_counter() - t_w < (0.0 if (quick or not primary) else 1.0):
        step()
        n_warm += 1
        if n_warm % 8 == 0:
            torch.cuda.synchronize()
    ms_step, reps, timed_ms = ctx.measure(step, steps, min_seconds, sampler)
    clocks = sampler.stop() if (rank == 0 and primary) else None
    for _ in range(3):
        step_e2e()
    ms_e2e, _, _ = ctx.measure(step_e2e, steps, min_seconds)
    cache.profile(True)
    torch.cuda.synchronize()
    for _ in range(min(max(steps, 10), 50)):
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
        k_name = "prefill" if "prefill" in per_kernel else "sdpa_dense"
        k_ms = statistics.median(per_kernel[k_name])
        achieved = useful / (k_ms * 1e-3) / 1e12
        peak = pk.get("bf16_tflops", 1590.0)
        kivi = fmt.startswith("kivi")
        h2d = sum(t.numel() * t.element_size() for t in ((hq,) if kivi else (hq, hk, hv)))
        result = {
            "metric": "prefill causal-useful attention TFLOP/s (sum over GPUs)", "value": world * useful / (ms_step * 1e-3) / 1e12,
            "unit": "TFLOP/s", "n_gpus": world, "steps": steps, "warmup": max(warmup, 3), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": f"{io} operands, f32 accumulation",
            "data": "synthetic",
            "config": {"workload": workload, "description": desc, "sequences_per_gpu": n_seq, "past_tokens": past,
                       "chunk_tokens": S, "q_heads": HQ, "kv_heads": HKV, "head_dim": D, "io_dtype": io, "kv_format": fmt,
                       "parallelism": f"by-sequence x{world}, no collective",
                       "l2": "working set fits L2 (warm)" if (past + S) * n_seq * HKV * D * 4 < 100e6 else "inputs larger than L2",
                       "flops_per_step_per_gpu": useful,
                       "step": "attention of the chunk's queries (the chunk is appended once, before the timed region)" if kivi
                               else "append the chunk, attention of its queries, roll the cache back",
                       "timed_region": {"repeats_of_the_steps": reps, "ms": timed_ms, "min_seconds": min_seconds}},
            "tokens_per_s": world * n_seq * S / (ms_step * 1e-3),
            "e2e": {"value": world * useful / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": hout.numel() * hout.element_size(), "ms_per_step": ms_e2e},
            "gpu_launches": steps * reps * (1 if kivi else 2), "kernels_ms": {k: statistics.median(v) for k, v in per_kernel.items()},
            "roofline": {"bound": "tensor", "kernel": ("prefill_tc_kernel" if fmt in ("f16", "bf16") else "attn_tc_kernel") if k_name == "prefill" else "sdpa_dense_kernel",
                         "achieved": achieved,
                         "peak": peak, "unit": "TFLOP/s", "kernel_ms": k_ms,
                         "frac": achieved / peak, "peak_kind": pk_kind + " (bf16 cuBLAS burst)", "traffic": None,
                         "flops": "causal-useful (masked half of the diagonal tiles not counted)"},
            "clocks": clocks,
        }
    cache.close()
    del cache
    torch.cuda.empty_cache()
    return result


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


def run_linear(ctx, workload, steps, warmup, no_cpu=False):
    """Q4_0 weights x int8-quantised activations (Q4_0::w4a8_gemm arithmetic): weight bytes per second against HBM."""
    torch = ctx.torch
    import tract_b200 as kv
    import oracle

    rank, world, dev = ctx.rank, ctx.world, ctx.dev
    wl = LINEAR[workload]
    n, k, m, layers = wl["n"], wl["k"], wl["m"], wl["layers"]
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

    sampler = ClockSampler(ctx.dev_index)
    if rank == 0:
        sampler.start()
    for _ in range(max(warmup, 3)):
        step()
    sampler.mark()
    ms = ctx.timed(step, steps)
    clocks = sampler.stop() if rank == 0 else None
    ms_e2e = ctx.timed(step_e2e, max(10, steps // 10)) / max(10, steps // 10)
    lins[0].check()
    ms_step = ms / steps
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
    if rank != 0:
        return None
    line = {
        "metric": "Q4_0 weight-read GB/s (sum over GPUs)", "value": value, "unit": "GB/s", "n_gpus": world, "steps": steps,
        "warmup": max(warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "u4 weights x s8 activations, s32 block dot products, f32 accumulation", "data": "synthetic",
        "config": {"workload": workload, "description": wl["desc"], "n": n, "k": k, "activation_rows": m, "layers_per_step": layers, "launch": "one CUDA graph replay per step",
                   "weight_bytes_per_step_per_gpu": weight_bytes, "parallelism": f"replicas x{world}, no collective",
                   "l2": "weights of one step exceed L2" if weight_bytes > 126e6 else "weights fit L2 (warm)"},
        "tokens_per_s": world * m * layers / (ms_step * 1e-3),
        "e2e": {"value": world * weight_bytes / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": m * k * 4,
                "d2h_bytes_per_step": m * n * 4, "ms_per_step": ms_e2e},
        "gpu_launches": 2 * layers * steps,
        "roofline": {"bound": "hbm", "kernel": ("q40_gemm_tc_kernel" if m >= 128 else "q40_gemm_rows_kernel" if m > 24 else "q40_gemm_kernel") + " (+ activation quantiser)", "achieved": achieved, "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": achieved / pk["hbm_gbs"], "peak_kind": pk_kind, "traffic": None,
                     "algorithmic_bytes": weight_bytes, "kernel_ms": kern_ms},
        "clocks": clocks,
    }
    if not no_cpu:
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
    return line


DECODER = {
    # BASELINE config 5: the Llama-3-8B shape, Q4_0 weights from a seed, 8 sequences per GPU (64 over 8 GPUs).
    # The stated shape: a real 2048-token prompt pass through the model, then 256 greedy steps
    "cfg5": dict(past=0, prompt=2048, seqs=8, kv="f16", greedy=256,
                 desc="BASELINE config 5: 32-layer Llama-3-8B-shaped decoder, Q4_0 weights, f16 KV cache, 8 sequences per GPU, "
                      "2048-token prompt pass, then 256 greedy decode steps"),
    # caches filled with synthetic K / V instead of a prompt pass (the decode steps alone)
    "cfg5-decoder": dict(past=2048, seqs=8, kv="f16", desc="32-layer Llama-3-8B-shaped decoder, Q4_0 weights, f16 KV cache, 8 sequences x 2048 cached tokens, greedy decode"),
    "cfg5-decoder-q8kv": dict(past=2048, seqs=8, kv="q8_1", desc="the same with the int8 block-32 KV cache"),
    # the pp512 / tg128 methodology of the reference's llm bench (cli/src/llm.rs:47-139): a real prompt pass, then decode steps
    "cfg5-pp512": dict(past=0, prompt=512, seqs=8, kv="f16", desc="the same decoder: 512-token prompt pass through the model (timed), then greedy decode"),
}


def run_decoder(ctx, workload, steps, warmup, seqs=0, past_override=0):
    torch = ctx.torch
    from tract_b200.decoder import Decoder, Shape

    rank, world, dev = ctx.rank, ctx.world, ctx.dev
    wl = DECODER[workload]
    sh = Shape()
    if wl.get("greedy"):
        steps = wl["greedy"]  # the configuration states its own step count
    B, past = seqs or wl["seqs"], past_override or wl["past"]
    dec = Decoder(sh, n_seqs=B, max_tokens=past + wl.get("prompt", 0) + 2 * steps + max(warmup, 3) + 64, kv_format=wl["kv"], seed=100 + rank,
                  device=dev)
    pp = None
    if wl.get("prompt"):
        P = wl["prompt"]
        prompt = torch.randint(0, sh.vocab, (B, P), dtype=torch.int32)
        dec.prefill(prompt[:, :64])  # warm-up on a short prompt (lazy allocations, attribute calls)
        torch.cuda.synchronize()
        dec.reset()
        ctx.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        dec.prefill(prompt)
        e1.record()
        ctx.barrier()
        pp_ms = ctx.max_over_ranks(e0.elapsed_time(e1))
        pp = {"prompt_tokens_per_gpu": B * P, "ms": pp_ms, "tokens_per_s": world * B * P / (pp_ms * 1e-3)}
        past = P
    else:
        dec.prefill_synthetic(past)
    tok_host = torch.randint(0, sh.vocab, (B,), dtype=torch.int32).pin_memory()
    out_host = torch.empty(B, dtype=torch.int32).pin_memory()
    if not wl.get("prompt"):
        dec.set_tokens(tok_host)

    def step():
        dec.step()

    def step_e2e():
        dec.tokens.copy_(tok_host, non_blocking=True)
        dec.step()
        out_host.copy_(dec.tokens, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    sampler = ClockSampler(ctx.dev_index)
    if rank == 0:
        sampler.start()
    for _ in range(max(warmup, 3)):
        step()
    sampler.mark()
    n_e2e = max(1, min(steps // 4, steps - 1))  # the steps are shared between the device-timed and the end-to-end loop
    n_dev = max(1, steps - n_e2e)
    ms = ctx.timed(step, n_dev) / n_dev
    clocks = sampler.stop() if rank == 0 else None
    ms_e2e = ctx.timed(step_e2e, n_e2e) / n_e2e
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
    kv_bytes = sh.n_layers * B * (past + max(warmup, 3) + n_dev // 2) * sh.n_kv_heads * sh.head_dim * 2 * (2 if wl["kv"] == "f16" else 1.0625)
    pk, pk_kind = peaks()
    line = None
    if rank == 0:
        line = {
            "metric": "decode tokens/s of the full decoder (sum over GPUs)", "value": world * B / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": steps, "warmup": max(warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "Q4_0 weights x int8 activations, f32 residual stream, 16-bit attention", "data": "synthetic",
            "config": {"workload": workload, "description": wl["desc"], "sequences_per_gpu": B, "cached_tokens": past,
                       "layers": sh.n_layers, "hidden": sh.hidden, "ffn": sh.ffn, "vocab": sh.vocab, "vocab_note": "assumed (not given by the config)",
                       "parallelism": f"by-sequence x{world}, no collective", "l2": "weights (4.2 GB) and caches exceed L2",
                       "weight_bytes_per_step": weight_bytes, "kv_bytes_per_step": kv_bytes,
                       "launch": "CUDA-graph segments between cache calls; cache calls from the host"},
            "e2e": {"value": world * B / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": B * 4, "d2h_bytes_per_step": B * 4,
                    "ms_per_step": ms_e2e},
            "gpu_launches": (sh.n_layers * 10 + 6) * n_dev,  # per layer: 4 GEMMs, 3 quantising producers, append, decode, combine (which quantises for wo)
            "kernels_ms": {k: statistics.mean(v) for k, v in recs.items()},
            "prompt_pass": pp,
            "roofline": {"bound": "hbm", "kernel": "whole step (Q4_0 GEMMs dominate)", "achieved": (weight_bytes + kv_bytes) / (ms * 1e-3) / 1e9,
                         "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": (weight_bytes + kv_bytes) / (ms * 1e-3) / 1e9 / pk["hbm_gbs"],
                         "peak_kind": pk_kind, "traffic": None, "algorithmic_bytes": weight_bytes + kv_bytes, "kernel_ms": ms},
            "clocks": clocks,
        }
    dec.close()
    del dec
    torch.cuda.empty_cache()
    return line


def run_sdpa(ctx, steps, warmup, min_seconds):
    """The lone Sdpa on dense tensors, over the shape list of the reference's own kernel bench (cuda/benches/cuda_flash.rs:84-110:
    batch 1, 32 query / 8 kv heads, head_dim 128, f16, causal; past + new tokens).  Metric: causal-useful attention TFLOP/s."""
    torch = ctx.torch
    import tract_b200 as kv

    shapes = [(0, 512), (0, 2048), (0, 8192), (2048, 1), (8192, 1)]  # (past, new tokens)
    rows = []
    for past, S in shapes:
        T = past + S
        gen = torch.Generator(device="cuda").manual_seed(5)
        mk = lambda h, n: (torch.randn((1, h, n, D), generator=gen, device="cuda") * 0.5).half()
        q, k, v = mk(HQ, S), mk(HKV, T), mk(HKV, T)
        fn = lambda: kv.sdpa(q, k, v, causal=True)
        for _ in range(max(warmup, 3)):
            fn()
        ms, reps, _ = ctx.measure(fn, max(steps // 4, 3), min_seconds)
        useful = 4.0 * HQ * D * sum(past + i + 1 for i in range(S))
        rows.append({"past": past, "new_tokens": S, "ms": ms, "tflops": useful / (ms * 1e-3) / 1e12})
    if ctx.rank != 0:
        return None
    pk, pk_kind = peaks()
    peak = pk.get("bf16_tflops", 1590.0)
    best = max(rows, key=lambda r: r["tflops"])
    return {"metric": "lone Sdpa causal-useful TFLOP/s (largest shape)", "value": best["tflops"], "unit": "TFLOP/s", "n_gpus": ctx.world,
            "steps": steps, "warmup": max(warmup, 3), "ms_per_step": best["ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f16 operands, f32 accumulation", "data": "synthetic",
            "config": {"workload": "sdpa-dense", "description": "lone Sdpa on dense [1, 32 | 8, T, 128] f16 tensors, causal", "shapes": rows,
                       "parallelism": f"replicas x{ctx.world}, no collective", "l2": "K/V of the larger shapes fit L2 (warm)"},
            "e2e": None, "gpu_launches": None,
            "roofline": {"bound": "tensor", "kernel": "sdpa kernel", "achieved": best["tflops"], "peak": peak, "unit": "TFLOP/s",
                         "frac": best["tflops"] / peak, "peak_kind": pk_kind + " (bf16 cuBLAS burst)", "traffic": None, "kernel_ms": best["ms"]}}


def run_head_sharded(ctx, steps, warmup):
    """The optional second axis (N >= 2): every rank holds Hkv / N kv heads of EVERY sequence of config 3 and the query heads
    that read them; one in-place NCCL all-gather of the attention outputs per step.  Every rank also holds the unsharded
    cache and checks the gathered output against it inside the run."""
    torch, dist = ctx.torch, ctx.dist
    import tract_b200 as kv
    from tract_b200 import sharding

    rank, world = ctx.rank, ctx.world
    if world < 2 or HKV % world:
        return None
    lens = draw_lengths("cfg3-bf16", 0)  # the same batch on every rank: the input is replicated
    B = len(lens)
    layer = sharding.HeadShardedAttention("bf16", HQ, HKV, D, max_seqs=B, max_seq_tokens=max(lens) + 128)
    full = kv.KvCache("bf16", HKV, D, max_seqs=B, max_seq_tokens=max(lens) + 128, pool_tokens=sum(lens) + 64 * B, max_q_heads=HQ)
    s_sh, s_full = [layer.new_seq() for _ in lens], [full.new_seq() for _ in lens]
    fill_cache(torch, full, s_full, lens, torch.bfloat16, seed=777, also=(layer.cache, s_sh, layer.kv_lo, layer.kv_hi))
    gen = torch.Generator(device="cuda").manual_seed(778)
    q = torch.randn((B, HQ, 1, D), generator=gen, device="cuda").bfloat16()
    buf = sharding.gather_buffer(torch, world, B, layer.q_hi - layer.q_lo, 1, D, q.dtype, q.device)
    want = full.attend(s_full, q, causal=True)
    got = layer.attend(s_sh, q, causal=True, buffer=buf)
    full.check(), layer.cache.check()
    diff = (got.float() - want.float()).abs().max().item()
    scale = want.float().pow(2).mean().sqrt().item()
    # a different split of the work (Hkv / N heads per launch): every element within one bf16 unit in the last place of
    # the unsharded result (2^-7 of its magnitude at most), small elements within 2e-3 of the tensor's scale
    ok = bool(((got.float() - want.float()).abs() <= want.float().abs() * 2.0 ** -7 + 2e-3 * scale).all().item())
    ok_all = ctx.sum_over_ranks(1.0 if ok else 0.0)[0] == world
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    att, gat = [], []
    for i in range(max(warmup, 3) + steps):
        ctx.barrier()
        ev[0].record()
        layer.cache.attend(s_sh, q[:, layer.q_lo:layer.q_hi], causal=True, out=buf[rank])
        ev[1].record()
        sharding.all_gather_heads(buf, rank)
        ev[2].record()
        torch.cuda.synchronize()
        if i >= max(warmup, 3):
            att.append(ev[0].elapsed_time(ev[1])), gat.append(ev[1].elapsed_time(ev[2]))
    a_ms, g_ms = ctx.max_over_ranks(statistics.median(att)), ctx.max_over_ranks(statistics.median(gat))
    layer.cache.close(), full.close()
    torch.cuda.empty_cache()
    if rank != 0:
        return None
    local_bytes = 2 * (HKV // world) * ROW_BYTES["bf16"] * sum(n + 1 for n in lens)
    return {"workload": "cfg3-bf16, kv heads split over the ranks", "parity_ok": bool(ok_all), "max_abs_diff": diff, "output_rms": scale,
            "attention_ms": a_ms, "all_gather_ms": g_ms, "all_gather_bytes_per_rank": B * (HQ // world) * D * 2,
            "kv_gbs_per_gpu": local_bytes / (a_ms * 1e-3) / 1e9, "collective": "one NCCL all_gather_into_tensor over local buffers (in place)"}


def brief(line):
    """The figures of a secondary workload: kernel time, roofline fraction, device-timed and end-to-end values."""
    if line is None:
        return None
    r = line.get("roofline") or {}
    out = {"value": line.get("value"), "unit": line.get("unit"), "ms_per_step": line.get("ms_per_step"),
           "kernel": r.get("kernel"), "kernel_ms": r.get("kernel_ms"), "roofline_frac": r.get("frac"), "bound": r.get("bound"),
           "e2e": (line.get("e2e") or {}).get("value"), "tokens_per_s": line.get("tokens_per_s")}
    if line.get("prompt_pass"):
        out["prompt_pass"] = line["prompt_pass"]
    if line.get("config", {}).get("shapes"):
        out["shapes"] = line["config"]["shapes"]
    return out


def run_secondary(ctx, args):
    """Short runs of the other configurations, for the `secondary` object of the default line."""
    sec = {}
    steps = max(5, min(args.steps, 20))

    def guarded(name, fn):
        t0 = time.perf_counter()
        try:
            r = fn()
            if ctx.rank == 0:
                sec[name] = brief(r) if not (isinstance(r, dict) and "parity_ok" in r) else r
                if sec[name] is not None:
                    sec[name]["wall_s"] = round(time.perf_counter() - t0, 1)
        except Exception as e:  # a secondary workload must not take the headline line down with it
            if ctx.rank == 0:
                sec[name] = {"error": f"{type(e).__name__}: {e}"[:300]}

    for wl in ("cfg4-q4", "cfg4-kivi8", "cfg4-kivi4", "cfg3-bf16", "cfg1-f32"):
        guarded(wl, lambda wl=wl: run_decode(ctx, wl, steps, 3, 0.2, quick=True, primary=False))
    for wl in ("cfg2-prefill", "prefill-8k", "prefill-chunked-q8"):
        guarded(wl, lambda wl=wl: run_prefill(ctx, wl, steps, 3, 0.2, quick=True, primary=False))
    guarded("sdpa-dense", lambda: run_sdpa(ctx, steps, 3, 0.05))
    if ctx.world >= 2:
        guarded("head_sharded", lambda: run_head_sharded(ctx, steps, 3))
    if not args.no_decoder:
        guarded("cfg5", lambda: run_decoder(ctx, "cfg5", 256, 3))
    return sec


# ---------------------------------------------------------------------------------------------------
# CPU arm: the restatement of tract's own CPU algorithm (the Rust reference cannot be built here)
# ---------------------------------------------------------------------------------------------------

def cpu_step_factory(workload, sample_seqs, sample_past, threads):
    """Returns (step_fn, bytes_per_step): one decode step of `sample_seqs` sequences on the CPU, as tract's CPU ops do it.
    Block formats: quantise the new token, dequantise the whole cache, FlashSdpaOp over it.  KIVI: the per-(batch, head)
    stores of QuantizedDynKvCacheState ingest the new token and rebuild the whole f32 cache (quant_dyn_kv_cache.rs:403-449,
    483-495), which Sdpa then reads.  Inputs: N(0,1) with 1 % of the elements multiplied by 20, as on the GPU arm."""
    import oracle

    fmt, io, _, _, _ = WORKLOADS[workload]
    g = np.random.Generator(np.random.Philox(key=5))
    T = sample_past + 1
    np_io = {"f32": np.float32, "f16": np.float16, "bf16": oracle.bfloat16}[io]

    def draw(shape):
        x = g.standard_normal(shape, dtype=np.float32)
        return np.where(g.random(shape, dtype=np.float32) < 0.01, x * np.float32(20), x)

    k, v = draw((sample_seqs, HKV, T, D)), draw((sample_seqs, HKV, T, D))
    q = g.standard_normal((sample_seqs, HQ, 1, D), dtype=np.float32).astype(np_io)
    if fmt == "q8_1":
        ks, _, kc = oracle.q8_1_quant(k)
        vs, _, vc = oracle.q8_1_quant(v)
    elif fmt == "q4_0":
        ks, kc = oracle.q4_0_quant(k)
        vs, vc = oracle.q4_0_quant(v)
    elif fmt.startswith("kivi"):
        bits = 8 if fmt == "kivi8" else 4
        kq, vq = oracle.QuantizedDynKeyValueCache(bits, True), oracle.QuantizedDynKeyValueCache(bits, False)
        kq.eval(k[:, :, :-1].astype(np_io)), vq.eval(v[:, :, :-1].astype(np_io))
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
        elif fmt.startswith("kivi"):  # the op's output: the whole cache, dequantised and cast to the model's type
            kd, vd = kq.eval(k[:, :, -1:].astype(np_io)), vq.eval(v[:, :, -1:].astype(np_io))
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
    lens = draw_lengths(args.workload, 0)
    sample_past = 8192 if past == "ragged" else int(lens[0])
    # each step walks a bounded sample of the batch: every sequence costs the same, so the rate does not depend on the count
    try:
        import psutil

        ram_gb = psutil.virtual_memory().available / 2**30
    except Exception:
        ram_gb = 16.0
    sample_seqs = max(1, min(len(lens), 4 if ram_gb > 24 else 2))
    step, nbytes = cpu_step_factory(args.workload, sample_seqs, sample_past, threads)
    steps = min(args.steps, 100)
    for _ in range(max(1, min(args.warmup, 3))):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    val = nbytes / dt / 1e9
    sample = (f"each step = {sample_seqs} of {len(lens)} sequences, past {sample_past}: append-quantise 1 token, "
              f"dequantise cache, flash attention, on {threads} host threads")
    cfg = decode_config(args.workload, lens, world)
    cfg["cpu_sample"] = sample
    return {"impl": "reference", "metric": "decode-attn KV-read GB/s (sum over GPUs; per GPU = value / n_gpus)",
            "value": val, "unit": "GB/s", "n_gpus": world, "steps": steps, "warmup": max(1, min(args.warmup, 3)), "ms_per_step": dt * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": cfg,
            "note": "tract is Rust and no cargo/rustc exists on this image: this arm times the CPU restatement of "
                    "tract's own algorithm (oracle/), the same code the parity tests check against",
            "tokens_per_s": sample_seqs / dt,
            "cpu_baseline": {"value": val, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="cfg4-q8", choices=sorted(WORKLOADS) + sorted(PREFILL) + sorted(LINEAR) + sorted(DECODER) + ["sdpa-dense"])
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true", help="only the workload named: no `secondary` object")
    ap.add_argument("--no-decoder", action="store_true", help="leave config 5 (the whole decoder) out of `secondary`")
    ap.add_argument("--min-seconds", type=float, default=0.5, help="least length of the timed region (the K steps are repeated)")
    ap.add_argument("--quick", action="store_true", help="profiler runs: exactly W warm-up steps, K timed steps, no repeats")
    ap.add_argument("--seqs", type=int, default=0, help="override sequences per GPU (profiling: smaller case)")
    ap.add_argument("--past", type=int, default=0, help="override the past length (profiling: smaller case)")
    args = ap.parse_args()
    OVERRIDE.update(seqs=args.seqs, past=args.past)
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    if args.impl == "reference":
        r = run_reference(args, rank, world)
        if r:
            print(json.dumps(r))
        return
    if args.quick:
        args.min_seconds = 0.0
    ctx = Ctx(rank, world)
    try:
        if args.workload in LINEAR:
            r = run_linear(ctx, args.workload, args.steps, args.warmup, args.no_cpu_baseline)
        elif args.workload in DECODER:
            r = run_decoder(ctx, args.workload, min(args.steps, 64) if args.steps > 256 else args.steps, args.warmup, args.seqs, args.past)
        elif args.workload in PREFILL:
            r = run_prefill(ctx, args.workload, args.steps, args.warmup, args.min_seconds, args.quick)
        elif args.workload == "sdpa-dense":
            r = run_sdpa(ctx, args.steps, args.warmup, args.min_seconds)
        else:
            r = run_decode(ctx, args.workload, args.steps, args.warmup, args.min_seconds, args.quick)
            default_run = args.workload == "cfg4-q8" and not (args.quick or args.no_secondary or args.seqs or args.past)
            sec = run_secondary(ctx, args) if default_run else None
            if rank == 0:
                if sec is not None:
                    r["secondary"] = sec
                if not args.no_cpu_baseline and world == 1:
                    r["cpu_baseline"] = cpu_baseline(args.workload)
                elif world > 1:
                    r["cpu_baseline"] = {"note": "timed at N=1 only"}
        if rank == 0 and r is not None:
            print(json.dumps(r), flush=True)
    finally:
        ctx.close()


if __name__ == "__main__":
    main()
