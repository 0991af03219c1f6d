#!/usr/bin/env python
"""Benchmark of the quantized-weight decode hot path on B200.

A step is one pass of the decode FFN projections of a dense 27B-class layer at batch 1:
quantize_q8(x[5120]) -> Q4_K gate matvec and Q4_K up matvec (5120 -> 17408, sharing the
quantized x), quantize_q8(h[17408]) -> Q6_K down matvec (17408 -> 5120).  The metric is the
reference's: repacked weight bytes streamed per second (GB/s).  Steps rotate over several
distinct copies of the layer's weights so that no launch finds its weights in L2.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

The K steps are replayed from CUDA graphs and timed as one round; the round is repeated until the
timed region lasts at least 50 ms, and `ms_per_step` is the median round (min and max beside it).

One GPU: the step is five launches with programmatic dependent launch.  With N > 1 (launched by
torch.distributed.run, one rank per GPU) the step is ONE cooperative launch per GPU (rc_ffn_decode_tp):
gate and up split by output rows, down by the matching columns, each rank streams its shard and the
ranks' partial outputs are summed through stores into peer memory; the row-sharded one-launch form and
the launch chain with peer gathers are timed beside it.  At N > 1 the line also carries the row-sharded
prefill GEMM that gathers its own output and the MoE layer with the experts spread over the ranks.
`--profile-case {mmqx,ffn}` runs a few launches of one kernel for a small ncu capture.
`--impl reference` times the reference's CPU path (dequantize to f32 + sequential-f32 row
dots, row-parallel over the host cores) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

Q4_K, Q6_K = 12, 14
HIDDEN, FFN = 5120, 17408
LAYER = [("gate", Q4_K, HIDDEN, FFN), ("up", Q4_K, HIDDEN, FFN), ("down", Q6_K, FFN, HIDDEN)]


def measured_peaks() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.lines: list[str] = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [s.strip() for s in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------- CPU arm


def cpu_layer_sample(seconds: float, threads: int):
    """Times the reference's CPU path (oracle port) on the layer's three matrices; returns
    (GB/s by the same byte count the GPU arm uses, description, seconds per layer)."""
    sys.path.insert(0, str(ROOT / "tests"))
    import oracle as ro
    from reinstinct_b200 import synth

    total_bytes, mats = 0, []
    for i, (_, t, in_dim, out_dim) in enumerate(LAYER):
        raw = synth.synth_blocks(t, in_dim, out_dim, seed=10 + i)
        x = synth.synth_activations(1, in_dim, seed=20 + i)
        mats.append((t, raw, x, in_dim, out_dim, np.empty(in_dim * out_dim, dtype=np.float32)))
        total_bytes += ro.repacked_len(t, in_dim, out_dim)
    times = []
    t_end = time.perf_counter() + seconds
    while not times or (time.perf_counter() < t_end and len(times) < 50):
        t0 = time.perf_counter()
        for t, raw, x, in_dim, out_dim, wf in mats:
            ro.cpu_path(t, raw, x, in_dim, out_dim, n_threads=threads, w_f32=wf, dequant=True)
        times.append(time.perf_counter() - t0)
    best = min(times)
    sample = (f"{len(times)} passes of the full layer (gate, up: Q4_K 5120->17408; down: Q6_K 17408->5120), "
              f"dequantize-to-f32 + sequential-f32 row dots, best pass {best * 1e3:.1f} ms")
    return total_bytes / best / 1e9, sample, best


def run_reference_arm(args):
    """The reference's CPU implementation of the path, all host threads, on rank 0 only.
    A step is one layer pass over the first `rows` output rows of each matrix, with `rows`
    chosen from a probe so that the whole run stays within a couple of minutes."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    sys.path.insert(0, str(ROOT / "tests"))
    import oracle as ro
    from reinstinct_b200 import synth

    def build(frac: float):
        total_bytes, mats = 0, []
        for i, (_, t, in_dim, out_dim) in enumerate(LAYER):
            rows = min(out_dim, max(32, int(out_dim * frac) // 32 * 32))
            raw = synth.synth_blocks(t, in_dim, rows, seed=10 + i)
            x = synth.synth_activations(1, in_dim, seed=20 + i)
            mats.append((t, raw, x, in_dim, rows, np.empty(in_dim * rows, dtype=np.float32)))
            total_bytes += ro.repacked_len(t, in_dim, rows)
        return total_bytes, mats

    def one_pass(mats):
        t0 = time.perf_counter()
        for t, raw, x, in_dim, rows, wf in mats:
            ro.cpu_path(t, raw, x, in_dim, rows, n_threads=threads, w_f32=wf, dequant=True)
        return time.perf_counter() - t0

    _, probe = build(1.0 / 16)
    one_pass(probe)
    t_probe = one_pass(probe) * 16  # estimate of a full layer pass
    budget_s = 100.0
    frac = min(1.0, budget_s / max(t_probe * (args.steps + args.warmup), 1e-9))
    total_bytes, mats = build(frac)
    times = []
    for it in range(args.warmup + args.steps):
        dt = one_pass(mats)
        if it >= args.warmup:
            times.append(dt)
    per_step_s = sum(times) / len(times)
    value = total_bytes / per_step_s / 1e9
    sample = (f"each step: dequantize-to-f32 + sequential-f32 row dots over the first {frac:.3f} of the output "
              f"rows of gate, up (Q4_K) and down (Q6_K), {total_bytes / 1e6:.1f} MB repacked, {threads} threads")
    full_layer_s = per_step_s * 176168960 / total_bytes
    line = {
        "impl": "reference", "metric": "q4k_decode_matvec_hbm_gbs", "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step_s * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "tok_per_s_per_layer": 1.0 / full_layer_s,
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus: int) -> dict:
    return {
        "workload": "config 2: dense-27B decode FFN, batch 1 (quantize x; Q4_K gate, up 5120->17408; SwiGLU+quantize; Q6_K down 17408->5120)",
        "bytes_per_step": 176168960,
        "l2": "weights rotate over 4 distinct layer copies (705 MB > 5x L2); every launch reads cold HBM",
        "parallelism": (f"row-shard x{n_gpus}; all-gather of the quantized intermediate and of down's output "
                        "(peer-memory push over NVLink, two alternating buffers)" if n_gpus > 1 else "single GPU"),
    }


# ------------------------------------------------------------------------------------- GPU arm

INT8_DENSE_PEAK_TOPS = 4500.0  # nominal B200 dense int8


def q4k_dram_traffic() -> tuple[int | None, str]:
    """DRAM bytes of one Q4_K 5120->17408 matvec launch, as the ncu summary kept beside the other
    profile summaries records it (dram__bytes_read.sum + dram__bytes_write.sum of one launch)."""
    import re

    f = ROOT / "profiles" / "matvec_q4k_5120x17408.md"
    try:
        m = re.search(r"dram bytes per launch \(read \+ write\)[^:]*:\s*([0-9,]+)", f.read_text())
        return int(m.group(1).replace(",", "")), "ncu summary of this kernel: dram__bytes_read.sum + dram__bytes_write.sum, one launch"
    except Exception:
        return None, "no ncu summary found"


def measured_tensor_peak() -> tuple[float, str]:
    """Burst bf16 GEMM throughput measured on this pool (the f16 kind runs at the same rate)."""
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["bf16_tflops"]), "measured bf16 burst"
        except Exception:
            pass
    return 1590.0, "fallback"


def moe_layer(rt, synth, torch, dev, timed):
    """Config 5: 256 experts, top-8 of 512 tokens, hidden 2048, expert FFN 512: router top-k, sort,
    gather, grouped gate+up GEMM (Q4_K [1024, 2048] per expert), SwiGLU + quantize, grouped down
    GEMM (Q6_K [2048, 512]), scatter, weighted combine; every step a launch of the library.
    HBM-bound: the figure of merit is expert-weight bytes / s.  The reported layer is the exact-integer
    route (BlockQ8 records into the per-sub-block tensor-core kernels); the f16-dequantized route, an
    approximation, rides beside it."""
    E, H, F, NT, K = 256, 2048, 512, 512, 8
    lib_tile = 8  # experts' worth of distinct blocks, tiled to 256 experts (bytes are what matter)

    def slab(t, in_dim, out_dim, seed):
        one = synth.synth_blocks(t, in_dim, out_dim * lib_tile, seed)
        return rt.GpuExpertTensor.from_bytes(np.tile(one, E // lib_tile), t, in_dim, out_dim, E, device=dev)

    gu, dn = slab(Q4_K, H, 2 * F, 91), slab(Q6_K, F, H, 92)
    logits = torch.from_numpy(synth.synth_router_logits(NT, E, 93)).to(dev)
    NE = NT * K
    ids = torch.empty(NT, K, dtype=torch.int32, device=dev)
    wts = torch.empty(NT, K, device=dev)
    x = torch.from_numpy(synth.synth_activations(NT, H, 94)).to(dev)
    moe = rt.MoeGroupedScratch.new(E, NE, device=dev)
    u8 = dict(dtype=torch.uint8, device=dev)
    xq, xg = torch.empty(NT * (H // 32) * 40, **u8), torch.empty(NE * (H // 32) * 40, **u8)
    hq = torch.empty(NE * (F // 32) * 40, **u8)
    y1 = torch.empty(NE, 2 * F, device=dev)
    y2, per_entry = torch.empty(NE, H, device=dev), torch.empty(NE, H, device=dev)
    out = torch.empty(NT, H, device=dev)

    def step(i):
        rt.launch_moe_topk(logits, ids, wts, E, K, NT)
        rt.launch_quantize_q8(x, xq, H, NT)
        rt.launch_moe_sort(moe, ids, NE)
        rt.launch_moe_gather_xq(moe, xq, xg, H // 32, K, NE)
        rt.launch_moe_grouped_gemm(moe, gu, xg, y1, H, 2 * F, NE)
        rt.launch_moe_act_q8(y1, hq, F, NE, rt.ACT_SWIGLU)
        rt.launch_moe_grouped_gemm(moe, dn, hq, y2, F, H, NE)
        rt.launch_moe_scatter_rows(moe, y2, per_entry, H, NE)
        rt.launch_moe_combine(per_entry, ids, wts, None, out, H, K, NT)

    gg = rt.MoeGroupedGemm(device=dev)

    def step_f16(i):
        rt.launch_moe_topk(logits, ids, wts, E, K, NT)
        rt.launch_moe_sort(moe, ids, NE)
        gg.gate_up(moe, gu, x, K, y1, NE)
        gg.down(moe, dn, y1, rt.ACT_SWIGLU, y2, NE)
        rt.launch_moe_scatter_rows(moe, y2, per_entry, H, NE)
        rt.launch_moe_combine(per_entry, ids, wts, None, out, H, K, NT)

    reps = 10
    us = timed(step, reps, 3) / reps * 1e3
    out_exact = out.clone()
    us_f16 = timed(step_f16, reps, 3) / reps * 1e3
    rel = float((out - out_exact).norm() / out_exact.norm())
    us_gu = timed(lambda i: rt.launch_moe_grouped_gemm(moe, gu, xg, y1, H, 2 * F, NE), reps, 3) / reps * 1e3
    us_dn = timed(lambda i: rt.launch_moe_grouped_gemm(moe, dn, hq, y2, F, H, NE), reps, 3) / reps * 1e3
    us_gu16 = timed(lambda i: gg.gate_up(moe, gu, x, K, y1, NE), reps, 3) / reps * 1e3
    us_dn16 = timed(lambda i: gg.down(moe, dn, y1, rt.ACT_SWIGLU, y2, NE), reps, 3) / reps * 1e3
    wbytes = gu.data.numel() + dn.data.numel()
    peak, _ = measured_peaks()

    # decode side of the same layer: one token, its 8 routed experts through the expert-indexed matvec
    # (gate+up then down).  Each call takes the next 8 experts of the slab, so every weight byte comes
    # from HBM (549 MB of experts > 4x L2).
    ids_dec = torch.arange(E, dtype=torch.int32, device=dev).reshape(E // K, K)
    xq1 = torch.empty((H // 32) * 40, **u8)
    hq1 = torch.empty(K * (F // 32) * 40, **u8)
    g1, d1 = torch.empty(1, K, 2 * F, device=dev), torch.empty(1, K, H, device=dev)
    rt.launch_quantize_q8(x[:1], xq1, H, 1)

    def decode_step(i):
        sel = ids_dec[i % (E // K)]
        rt.launch_moe_expert_matvec(gu, sel, xq1, g1, K, 1, H // 32, 0)
        rt.launch_moe_act_q8(g1, hq1, F, K, rt.ACT_SWIGLU)
        rt.launch_moe_expert_matvec(dn, sel, hq1, d1, K, 1, K * (F // 32), F // 32)

    for i in range(3):
        decode_step(i)
    torch.cuda.synchronize()
    g_dec = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g_dec):
        for i in range(E // K):
            decode_step(i)
    us_dec = timed(lambda i: g_dec.replay(), 4, 2) / (4 * (E // K)) * 1e3
    dec_bytes = (gu.bytes_per_expert + dn.bytes_per_expert) * K
    return {"workload": "config 5: 256 experts top-8, 512 tokens, hidden 2048, ffn 512 (548.9 MB of expert weights, 25.8 GOP)",
            "route": "exact integer block dots: quantize, sort, gather, grouped int8 / integer-f16 tensor-core GEMMs",
            "us_layer": us, "tok_per_s_per_layer": NT / (us * 1e-6), "tops": 2.0 * NE * (H * 2 * F + F * H) / us / 1e6,
            "us_gate_up": us_gu, "us_down": us_dn,
            "f16_dequantized_route": {"us_layer": us_f16, "us_gate_up": us_gu16, "us_down": us_dn16, "rel_l2_vs_exact_route": rel,
                                      "note": "opt-in approximation (rc_mmq_gemm_grouped_f32); not the reported figure"},
            "decode_1_token": {"us": us_dec, "expert_bytes": dec_bytes, "gbs": dec_bytes / us_dec / 1e3,
                               "frac_of_hbm_peak": dec_bytes / us_dec / 1e3 / peak,
                               "launches": "expert matvec (gate+up), SwiGLU+quantize, expert matvec (down)"},
            "roofline": {"bound": "hbm", "achieved": wbytes / us / 1e3, "peak": peak, "unit": "GB/s",
                         "frac": wbytes / us / 1e3 / peak, "note": "expert-weight bytes over the whole exact-route layer time"}}


def small_matvecs(rt, synth, torch, dev, timed):
    """Config 1 (Q8_0 4096 x 4096, batch 1) and config 3 (batch-4 verify matvec, 5120 x 5120, five formats):
    each over rotating weight copies larger than L2, replayed from a CUDA graph; GB/s of repacked weights."""
    peak, _ = measured_peaks()
    out = {}

    def one(t, in_dim, out_dim, n_rows, seed):
        w1 = rt.GpuMatvecTensor.from_bytes_matvec(synth.synth_blocks(t, in_dim, out_dim, seed), t, in_dim, out_dim, device=dev)
        n_copies = max(2, int(np.ceil(300e6 / w1.data.numel())))
        ws = [w1] + [rt.GpuMatvecTensor.from_repacked(w1.data.clone(), t, in_dim, out_dim, device=dev) for _ in range(n_copies - 1)]
        x = torch.from_numpy(synth.synth_activations(n_rows, in_dim, seed + 1)).to(dev)
        xq = torch.empty(n_rows * (in_dim // 32) * 40, dtype=torch.uint8, device=dev)
        rt.launch_quantize_q8(x, xq, in_dim, n_rows)
        y = torch.empty(n_rows, out_dim, device=dev)

        def sweep(i):
            for w in ws:
                if n_rows == 1:
                    rt.launch_matvec_xq8(w, xq, y)
                else:
                    rt.launch_matvec_batched(w, xq, y, n_rows)
        sweep(0)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            sweep(0)
        reps = 20
        us = timed(lambda i: g.replay(), reps, 3) * 1e3 / (reps * n_copies)
        nbytes = w1.data.numel()
        return {"us": us, "bytes": nbytes, "gbs": nbytes / us / 1e3, "frac_of_hbm_peak": nbytes / us / 1e3 / peak, "copies": n_copies}

    out["config1_q8_0"] = dict(workload="config 1: Q8_0 4096x4096 matvec, batch 1", **one(8, 4096, 4096, 1, 301))
    c3 = {}
    for name, t in (("Q4_0", 2), ("Q5_K", 13), ("Q6_K", 14), ("Q8_0", 8), ("IQ4_XS", 23)):
        c3[name] = one(t, 5120, 5120, 4, 310 + t)
    out["config3_batch4"] = {"workload": "config 3: batch-4 verify matvec, 5120x5120, five formats", "formats": c3}
    return out


def moe_expert_parallel(rt, synth, torch, dist, dev, timed, rank, world):
    """Config 5 sharded by experts over the ranks (N > 1): 256 experts split evenly, every rank routes its own 512 / N
    tokens (top-8); the routed BlockQ8 rows go to the owner of their expert, through the grouped gate+up GEMM there, and
    the results travel back.  Reported: the exchange done by the GPUs themselves (runtime.ExpertParallel: peer stores and
    two peer barriers per step, the whole step replayed from a CUDA graph of two steps).  Beside it: the same step with
    host-driven NCCL all-to-alls (eager).  value = tokens of all ranks per second through this gate+up stage."""
    from reinstinct_b200 import sharding as sh

    E, H, F, NT, K = 256, 2048, 512, 512, 8
    nt = NT // world
    e0, e1 = sh.expert_range(E, rank, world)
    one = synth.synth_blocks(Q4_K, H, 2 * F * 8, 91)
    n_local = e1 - e0
    gu = rt.GpuExpertTensor.from_bytes(np.tile(one, (n_local + 7) // 8)[: (n_local * one.size) // 8], Q4_K, H, 2 * F, n_local, device=dev)
    logits = torch.from_numpy(synth.synth_router_logits(NT, E, 93)[rank * nt:(rank + 1) * nt].copy()).to(dev)
    x = torch.from_numpy(synth.synth_activations(NT, H, 94)[rank * nt:(rank + 1) * nt].copy()).to(dev)
    ids = torch.empty(nt, K, dtype=torch.int32, device=dev)
    wts = torch.empty(nt, K, device=dev)
    u8 = dict(dtype=torch.uint8, device=dev)
    xq = torch.empty(nt * (H // 32) * 40, **u8)
    state = {}

    def step_host(i):
        # the routed rows travel as BlockQ8 records (2.56 KB instead of 8 KB of f32 per entry)
        rt.launch_moe_topk(logits, ids, wts, E, K, nt)
        rt.launch_quantize_q8(x, xq, H, nt)
        flat = ids.reshape(-1)
        plan = sh.plan_dispatch(flat, E)
        rows = xq.reshape(nt, (H // 32) * 40).repeat_interleave(K, dim=0).contiguous()
        rows_in = sh.dispatch_rows(rows, plan)
        ids_in = (sh.dispatch_rows(flat.to(torch.float32).reshape(-1, 1), plan).reshape(-1).to(torch.int32) - e0).contiguous()
        n_in = rows_in.shape[0]
        moe = rt.MoeGroupedScratch.new(n_local, n_in, device=dev)
        rt.launch_moe_sort(moe, ids_in, n_in)
        xg = torch.empty(n_in * (H // 32) * 40, **u8)
        rt.launch_moe_gather_xq(moe, rows_in.reshape(-1), xg, H // 32, 1, n_in)
        y_sorted = torch.empty(n_in, 2 * F, device=dev)
        rt.launch_moe_grouped_gemm(moe, gu, xg, y_sorted, H, 2 * F, n_in)
        y_in = torch.empty(n_in, 2 * F, device=dev)
        rt.launch_moe_scatter_rows(moe, y_sorted, y_in, 2 * F, n_in)
        state["y"] = sh.combine_rows(y_in, plan)
        state["n_in"] = n_in

    n_ent = nt * K
    ep = rt.ExpertParallel(gu, H, 2 * F, cap=n_ent, device=dev)
    out = torch.empty(n_ent, 2 * F, device=dev)

    def step_dev(i):
        rt.launch_moe_topk(logits, ids, wts, E, K, nt)
        rt.launch_quantize_q8(x, xq, H, nt)
        ep.step(ids.reshape(-1), xq, n_ent, K, out)

    # the whole layer: the owner also runs SwiGLU + quantize and the down GEMM, rows of the model width come back and
    # are combined with the routing weights at the source
    one_d = synth.synth_blocks(Q6_K, F, H * 8, 92)
    dn = rt.GpuExpertTensor.from_bytes(np.tile(one_d, (n_local + 7) // 8)[: (n_local * one_d.size) // 8], Q6_K, F, H, n_local, device=dev)
    ep_l = rt.ExpertParallel(gu, H, 2 * F, cap=n_ent, device=dev, down=dn, act=rt.ACT_SWIGLU)
    per_entry = torch.empty(n_ent, H, device=dev)
    y_layer = torch.empty(nt, H, device=dev)

    def step_layer(i):
        rt.launch_moe_topk(logits, ids, wts, E, K, nt)
        rt.launch_quantize_q8(x, xq, H, nt)
        ep_l.step(ids.reshape(-1), xq, n_ent, K, per_entry)
        rt.launch_moe_combine(per_entry, ids, wts, None, y_layer, H, K, nt)

    def graph_of_two(fn):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for i in range(2):
                fn(i)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(2):
                fn(i)
        return g

    # checked steps: both receive buffers against the host-driven result
    step_host(0)
    torch.cuda.synchronize()
    same = True
    for i in range(2):
        step_dev(i)
        torch.cuda.synchronize()
        same = same and bool(torch.equal(out, state["y"]))
    reps = 10
    g = graph_of_two(step_dev)
    us = timed(lambda i: g.replay(), reps, 3) / (2 * reps) * 1e3
    gl = graph_of_two(step_layer)
    us_layer = timed(lambda i: gl.replay(), reps, 3) / (2 * reps) * 1e3
    us_host = timed(step_host, 5, 3) / 5 * 1e3
    ep.close()
    ep_l.close()
    return {"workload": f"config 5, {E} experts over {world} ranks, {nt} tokens per rank, top-{K}",
            "us_layer": us_layer, "tok_per_s_layer": NT / (us_layer * 1e-6),
            "layer": "top-k, quantize, dispatch, [owner: sort, gather, gate_up GEMM, SwiGLU + quantize, down GEMM, scatter], return, combine",
            "us_step": us, "tok_per_s": NT / (us * 1e-6), "rows_received_rank0": state.get("n_in"),
            "step": "the gate_up stage alone (what the host-driven figure beside it covers)",
            "exchange": "rc_ep_plan / rc_ep_dispatch / rc_ep_return / rc_ep_collect: BlockQ8 rows and f32 results stored straight "
                        "into the owner's / the source's memory, two rc_peer_barrier per step, graph replay of two steps",
            "equals_host_driven_result": same,
            "us_step_host_driven_nccl": us_host}


def mmq_prefill_row_sharded(rt, synth, torch, dist, dev, timed, rank, world):
    """Config 4 sharded by output rows (N > 1): every rank holds rows [b, e) of the Q4_K 5120->17408 matrix
    (multiples of 32 rows) and runs the exact prefill GEMM of all 512 tokens against them; the kernel stores
    every finished tile into all ranks' [512, 17408] outputs (peer stores over NVLink, overlapped with the
    tiles still computing), and one handshake kernel ends the step.  Timed as the whole step, max over ranks;
    TOPS counts the whole 91.3 GOP.  The gathered result is checked against the unsharded call on rank 0."""
    from reinstinct_b200 import sharding as sh

    P = 512
    raw = synth.synth_blocks(Q4_K, HIDDEN, FFN, seed=77)
    shard, n_rows = sh.shard_raw_rows(raw, Q4_K, HIDDEN, FFN, rank, world)
    b0, _ = sh.row_shard_range(FFN, rank, world)
    w = rt.GpuMatvecTensor.from_bytes_matvec(shard.copy(), Q4_K, HIDDEN, n_rows, device=dev)
    x = torch.from_numpy(synth.synth_activations(P, HIDDEN, 78)).to(dev)
    gg = rt.GatheredPrefillGemm(P, FFN, HIDDEN, device=dev)
    gemm = rt.PrefillGemm(max_x=P * HIDDEN, device=dev)
    y_local = torch.empty((P, n_rows), dtype=torch.float32, device=dev)

    # one checked step
    k = gg.matmul(w, x, P, b0)
    got = torch.empty((P, FFN), dtype=torch.float32, device=dev)
    gg.read(k, got, P)
    torch.cuda.synchronize()
    same = None
    if rank == 0:
        w_full = rt.GpuMatvecTensor.from_bytes_matvec(raw, Q4_K, HIDDEN, FFN, device=dev)
        y_full = torch.empty((P, FFN), dtype=torch.float32, device=dev)
        gemm.matmul_into(y_full, w_full, x, P)
        torch.cuda.synchronize()
        same = bool(torch.equal(got, y_full))
        del w_full, y_full
    dist.barrier()

    reps = 10
    us = timed(lambda i: gg.matmul(w, x, P, b0), reps, 4) / reps * 1e3
    us_gemm = timed(lambda i: gemm.matmul_into(y_local, w, x, P), reps, 3) / reps * 1e3
    ops = 2.0 * P * HIDDEN * FFN
    out = {"workload": f"config 4 row-sharded: 512 tokens x Q4_K 5120->17408, {n_rows} rows on rank 0 of {world}",
           "us_step": us, "us_gemm_only": us_gemm, "tops": ops / (us * 1e-6) / 1e12,
           "gathered_equals_unsharded_bit_for_bit": same,
           "gather": f"tile stores into all {world} outputs from the GEMM's drain ({P * n_rows * 4 * (world - 1)} bytes outbound per rank) + rc_peer_barrier"}
    gg.close()
    return out


def mmq_prefill(rt, synth, torch, dev, timed):
    """Config 4: dense prefill GEMM, 512 tokens x Q4_K 5120->17408, through PrefillGemm (rc_matmul: exact
    integer block dots on tcgen05, integer-valued f16 operands, one accumulator tile per sub-block).
    TOPS = 2*P*K*N / t.  Beside it: the BlockQ8-input entry rc_mmq_gemm (kind::i8 kernel), the opt-in
    f16-dequantized approximation, and a scale-free int8 GEMM of the same shape by the vendor library as the
    attainable int8 rate of this box."""
    P = 512
    raw = synth.synth_blocks(Q4_K, HIDDEN, FFN, seed=77)
    w = rt.GpuMatvecTensor.from_bytes_matvec(raw, Q4_K, HIDDEN, FFN, device=dev)
    x = torch.from_numpy(synth.synth_activations(P, HIDDEN, 78)).to(dev)
    gemm = rt.PrefillGemm(max_x=P * HIDDEN, device=dev)
    y = torch.empty((P, FFN), dtype=torch.float32, device=dev)
    xq = torch.empty(P * (HIDDEN // 32) * 40, dtype=torch.uint8, device=dev)
    rt.launch_quantize_q8(x, xq, HIDDEN, P)
    ops = 2.0 * P * HIDDEN * FFN
    reps = 10
    ms_q = timed(lambda i: gemm.matmul_into(y, w, x, P), reps, 3) / reps
    y_exact = y.clone()
    ms_k = timed(lambda i: rt.launch_mmq_gemm(w, xq, y, P), reps, 3) / reps
    ms_f = timed(lambda i: gemm.matmul_f16_into(y, w, x, P), reps, 3) / reps
    rel_f16 = float((y - y_exact).norm() / y_exact.norm())
    attainable = None
    try:
        a8 = torch.randint(-127, 128, (P, HIDDEN), dtype=torch.int8, device=dev)
        b8 = torch.randint(-8, 8, (HIDDEN, FFN), dtype=torch.int8, device=dev)
        ms_i = timed(lambda i: torch._int_mm(a8, b8), reps, 3) / reps
        attainable = {"tops": ops / (ms_i * 1e-3) / 1e12, "us": ms_i * 1e3,
                      "how": "torch._int_mm (vendor int8 GEMM, int32 accumulation over the whole K, no block scales) on the same shape"}
        del a8, b8
    except Exception as e:  # a measurement aid only
        attainable = {"error": f"{type(e).__name__}: {e}"}
    tops_q = ops / (ms_q * 1e-3) / 1e12
    peak, peak_kind = measured_tensor_peak()
    return {"workload": "config 4: 512 tokens x Q4_K 5120->17408 (91.3 GOP)",
            "kernel": "activations_to_q16_kernel + mmqx_kernel<Q4_K> (tcgen05 kind::f16 on integer-valued operands: the f32 "
                      "accumulator tile of every 32-wide sub-block is the exact integer block dot; drained and scaled per sub-block)",
            "us_matmul_f32_in": ms_q * 1e3, "tops_matmul_f32_in": tops_q,
            "us_mmq_blockq8_in": ms_k * 1e3, "tops_mmq_blockq8_in": ops / (ms_k * 1e-3) / 1e12,
            "f16_dequantized_opt_in": {"us": ms_f * 1e3, "tops": ops / (ms_f * 1e-3) / 1e12, "rel_l2_vs_exact_route": rel_f16,
                                       "note": "rc_matmul_f16: an approximation without integer block dots; not the reported figure"},
            "roofline": {"bound": "tensor", "achieved": tops_q, "peak": peak, "unit": "TFLOP/s",
                         "frac": tops_q / peak, "peak_kind": peak_kind,
                         "frac_of_nominal_int8": tops_q / INT8_DENSE_PEAK_TOPS,
                         "attainable_int8": attainable,
                         "timed": "PrefillGemm call (rc_matmul), activation-image launch included"},
            "tok_per_s_per_layer_gate_only": P / (ms_q * 1e-3)}


def run_profile_case(args):
    """A few launches of ONE kernel on a workload small enough for a multi-pass ncu capture (the launches before the
    captured one run slowly under ncu, and multi-pass captures save and restore the device memory the kernel writes):
      mmqx  the exact prefill GEMM: 512 tokens x Q4_K 5120 -> 4736 rows (one wave of 148 tiles; K as in config 4)
      ffn   the decode FFN of config 2 as one cooperative launch (176 MB of weights per launch, two copies in turn)
    Prints a short JSON line; no timing claims are made from this mode."""
    import torch

    from reinstinct_b200 import runtime as rt
    from reinstinct_b200 import synth

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    rt.init(0)
    n = 0
    if args.profile_case == "mmqx":
        P, rows = 512, 4736
        w = rt.GpuMatvecTensor.from_bytes_matvec(synth.synth_blocks(Q4_K, HIDDEN, rows, seed=77), Q4_K, HIDDEN, rows, device=dev)
        x = torch.from_numpy(synth.synth_activations(P, HIDDEN, 78)).to(dev)
        gemm = rt.PrefillGemm(max_x=P * HIDDEN, device=dev)
        y = torch.empty((P, rows), dtype=torch.float32, device=dev)
        for _ in range(3):
            gemm.matmul_into(y, w, x, P)
            n += 1
    else:
        copies = [[rt.GpuMatvecTensor.from_bytes_matvec(synth.synth_blocks(t, i, o, seed=10 * c + k), t, i, o, device=dev)
                   for k, (_, t, i, o) in enumerate(LAYER)] for c in range(2)]
        x = torch.from_numpy(synth.synth_activations(1, HIDDEN, 5)).to(dev).reshape(-1)
        fused = [rt.FusedFfnDecode(ws[0], ws[1], ws[2], FFN, HIDDEN, device=dev) for ws in copies]
        for c in range(4):
            fused[c % 2].run(x)
            n += 1
    torch.cuda.synchronize()
    import ctypes

    st = ctypes.c_uint(0)
    rt._lib.load().rc_device_status(ctypes.byref(st))
    print(json.dumps({"profile_case": args.profile_case, "launches": n, "device_status": st.value}), flush=True)


def run_gpu_arm(args):
    import torch
    import torch.distributed as dist

    from reinstinct_b200 import runtime as rt
    from reinstinct_b200 import synth

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        # NCCL prints its version banner on stdout at the first communicator: keep stdout for the one JSON line
        sys.stdout.flush()
        keep = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=dev)
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(keep, 1)
            os.close(keep)
    rt.init(local)

    n_copies = 4  # even: the two gathered buffers of a peer all-gather alternate, a replayed graph must hold an even number of gathers
    # Row shards: rank r owns rows [r*out/world, (r+1)*out/world) of every matrix; shard sizes
    # are multiples of 32 so quantize-then-gather equals gather-then-quantize.
    shards = []
    for name, t, in_dim, out_dim in LAYER:
        assert out_dim % (32 * world) == 0
        shards.append((name, t, in_dim, out_dim // world))
    copies = []
    for c in range(n_copies):
        ws = []
        for i, (name, t, in_dim, out_local) in enumerate(shards):
            # seeds differ by copy, matrix and rank: every shard is distinct data
            raw = synth.synth_blocks(t, in_dim, out_local, seed=1000 * c + 10 * i + rank + 1)
            ws.append(rt.GpuMatvecTensor.from_bytes_matvec(raw, t, in_dim, out_local, device=dev))
        copies.append(ws)
    layer_bytes_local = sum(w.data.numel() for w in copies[0])
    layer_bytes_total = layer_bytes_local * world

    # the layer's input: one pinned host vector and its device copy
    in_host = torch.from_numpy(synth.synth_activations(1, HIDDEN, 5)).pin_memory()
    x_dev = torch.empty_like(in_host, device=dev)
    x_dev.copy_(in_host)
    xq = torch.empty((HIDDEN // 32) * 40, dtype=torch.uint8, device=dev)
    hq = torch.empty((FFN // 32) * 40, dtype=torch.uint8, device=dev)
    y_gu = torch.empty(2 * (FFN // world), device=dev)
    y_gate, y_up = y_gu[:FFN // world], y_gu[FFN // world:]
    y_down = torch.empty(HIDDEN // world, device=dev)
    g_gate = torch.empty(FFN, device=dev) if world > 1 else y_gate
    g_up = torch.empty(FFN, device=dev) if world > 1 else y_up
    yd_host = torch.empty(HIDDEN, dtype=torch.float32).pin_memory()
    use_fused = world > 1  # one GPU: the launch chain is the faster step; N > 1: one cooperative launch per GPU
    launches_per_step = 1 if use_fused else 5

    # The step is the decode FFN as the engine runs it (step_swiglu_ffn): quantize x, gate, up, SwiGLU+quantize,
    # down.  N > 1: gate and up stay sharded (the activation between them and down is elementwise); each rank
    # produces its 1/N of the quantized intermediate and the BlockQ8 shards are all-gathered (21.7 KB instead
    # of 2 x 68 KB of f32); down's output rows are all-gathered for the next layer.  The gathers are
    # rc_allgather_push (stores into peer memory over NVLink + a counter handshake, two alternating buffers),
    # so the whole sharded step replays from CUDA graphs.
    h_local = FFN // world
    hq_local = torch.empty((h_local // 32) * 40, dtype=torch.uint8, device=dev) if world > 1 else hq
    if world > 1:
        ga_h = rt.PeerAllGather(hq_local.numel())
        ga_y = rt.PeerAllGather(y_down.numel() * 4)

    # The step as ONE cooperative launch per GPU (rc_ffn_decode): quantize, gate and up rows, SwiGLU + quantize with the
    # records stored into every rank's intermediate buffer, the down rows stored into every rank's output; bounded
    # counter waits instead of launches between the phases.  One object per weight copy.
    fused = [rt.FusedFfnDecode(ws[0], ws[1], ws[2], FFN, HIDDEN, rank * h_local, rank * (HIDDEN // world), device=dev)
             for ws in copies]

    def step_fused(c: int):
        fused[c % n_copies].run(x_dev)

    def step_chain(c: int):
        """The same step as separate launches (five on one GPU, seven with the two peer gathers)."""
        ws = copies[c % n_copies]
        if world == 1:
            rt.launch_ffn_decode(ws[0], ws[1], ws[2], x_dev, xq, y_gate, y_up, hq, y_down)
            return
        rt.launch_quantize_q8(x_dev, xq, HIDDEN, 1)
        rt.launch_matvec_xq8(ws[0], xq, y_gate)
        rt.launch_matvec_xq8(ws[1], xq, y_up)
        rt.launch_swiglu_q8(y_gate, y_up, None, hq_local, h_local)
        ga_h.gather(hq_local)
        rt.launch_matvec_xq8(ws[2], ga_h.buffer_ptr, y_down)
        ga_y.gather(y_down)

    # checked steps: the fused launch against the launch chain (and, N > 1, the gathered records against
    # SwiGLU + quantize of the whole gathered vectors), on two copies so that both alternating buffers are used
    y_fused, y_chain = torch.empty(HIDDEN, device=dev), torch.empty(HIDDEN, device=dev)
    fused_rel = 0.0
    for c in range(2):
        step_chain(c)
        if world > 1:
            got = torch.empty_like(hq)
            ga_h.copy_out(got)
            ga_y.copy_out(y_chain)
            dist.all_gather_into_tensor(g_gate, y_gate)
            dist.all_gather_into_tensor(g_up, y_up)
            rt.launch_swiglu_q8(g_gate, g_up, None, hq, FFN)
            torch.cuda.synchronize()
            assert torch.equal(got, hq), "peer gather of the quantized intermediate differs from the local quantization"
        else:
            y_chain.copy_(y_down)
        step_fused(c)
        fused[c].read_y(y_fused)
        torch.cuda.synchronize()
        fused_rel = max(fused_rel, float((y_fused - y_chain).norm() / y_chain.norm()))
    assert fused_rel < 1e-3, f"fused FFN launch differs from the launch chain: {fused_rel}"
    step, step_other = (step_fused, step_chain) if use_fused else (step_chain, step_fused)

    # N > 1, the reported step: the tensor-parallel form (rc_ffn_decode_tp).  Gate and up by rows, down by the matching
    # COLUMNS in whole superblocks (17408 / 256 = 68 superblocks dealt out as evenly as they go), so the intermediate stays
    # on its rank and the one exchange is the sum of the partial outputs.  Its own weight shards (the same total bytes).
    tp = tp_rel = ms_rows = None
    if world > 1:
        from reinstinct_b200 import sharding as sh

        c0, c1 = sh.col_shard_range(FFN, rank, world, 256)
        n_loc = c1 - c0
        copies_tp = []
        for c in range(n_copies):
            shapes = ((Q4_K, HIDDEN, n_loc), (Q4_K, HIDDEN, n_loc), (Q6_K, n_loc, HIDDEN))
            copies_tp.append([rt.GpuMatvecTensor.from_bytes_matvec(synth.synth_blocks(t, i, o, seed=2000 * c + 10 * k + rank + 1), t, i, o, device=dev)
                              for k, (t, i, o) in enumerate(shapes)])
        tp = [rt.TensorParallelFfnDecode(ws[0], ws[1], ws[2], device=dev) for ws in copies_tp]
        tp_bytes = torch.tensor([float(sum(w.data.numel() for w in copies_tp[0]))], device=dev)
        dist.all_reduce(tp_bytes)
        layer_bytes_total = int(tp_bytes.item())

        def step_tp(c: int):
            tp[c % n_copies].run(x_dev)

        # checked steps: against the same shards through separate launches, partial outputs summed by NCCL
        yg_l, yu_l = torch.empty(n_loc, device=dev), torch.empty(n_loc, device=dev)
        hq_l = torch.empty((n_loc // 32) * 40, dtype=torch.uint8, device=dev)
        y_part, y_tp = torch.empty(HIDDEN, device=dev), torch.empty(HIDDEN, device=dev)
        tp_rel = 0.0
        for c in range(3):
            ws = copies_tp[c]
            rt.launch_ffn_decode(ws[0], ws[1], ws[2], x_dev, xq, yg_l, yu_l, hq_l, y_part)
            dist.all_reduce(y_part)
            step_tp(c)
            tp[c].read_y(y_tp)
            torch.cuda.synchronize()
            tp_rel = max(tp_rel, float((y_tp - y_part).norm() / y_part.norm()))
        # (a last-bit difference between the two forms' gate/up row sums moves a few quants of the intermediate across a
        # rounding boundary: the bar is the f32 tolerance of the reference's own kernel tests)
        worst = torch.tensor([tp_rel], device=dev)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)  # one decision for all ranks
        tp_rel = float(worst.item())
        step_rows = step
        if tp_rel < 1e-3:
            step = step_tp
        else:  # keep the row-sharded launch as the step and say so in the line
            print(f"bench: tensor-parallel launch differs from the launch chain + all-reduce by {tp_rel}; reporting the row-sharded launch",
                  file=sys.stderr, flush=True)
            for f in tp:
                f.close()
            tp = None
            layer_bytes_total = layer_bytes_local * world

    # End-to-end step through the host-side API with HOST buffers.  One GPU: runtime.launch_ffn_decode given the pinned
    # host input and output themselves (the quantizer reads x, the down matvec writes y across PCIe; no copy launches).
    # N > 1: x is uploaded by a copy node (every CTA reads it) and the launch writes the gathered output into the pinned host y.
    def step_e2e(c: int):
        if world == 1:
            ws = copies[c % n_copies]
            rt.launch_ffn_decode(ws[0], ws[1], ws[2], in_host, xq, y_gate, y_up, hq, yd_host)
        else:
            rt.copy_small(x_dev, in_host, HIDDEN * 4)  # every CTA reads x: one upload by a kernel (a memcpy node costs 9 us here)
            (tp or fused)[c % n_copies].run(x_dev, yd_host)  # the last phase writes the output to the host itself

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps: int, warmup: int) -> float:
        """Device time in ms of `steps` calls, max over ranks."""
        for i in range(warmup):
            fn(i)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(warmup + i)
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    def timed_rounds(round_fn, rounds: int, warm_rounds: int):
        """Per-round device times in ms (max over ranks per round): one event between consecutive rounds."""
        for i in range(warm_rounds):
            round_fn()
        barrier()
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(rounds + 1)]
        evs[0].record()
        for i in range(rounds):
            round_fn()
            evs[i + 1].record()
        barrier()
        ms = torch.tensor([evs[i].elapsed_time(evs[i + 1]) for i in range(rounds)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.cpu().numpy()

    # The decode loop is launch-bound from Python (8 us kernels), so the steps are replayed from CUDA graphs, as
    # the reference's engine replays its forward.  A round is EXACTLY --steps steps: graphs of L steps each, L the
    # largest of 4, 2, 1 that divides --steps (N > 1 needs an even L or a pair of graphs per parity; with L = 1 the
    # four graphs alternate parity by construction), replayed in cyclic order.
    K = max(1, args.steps)
    L = 4 if K % 4 == 0 else 2 if K % 2 == 0 else 1

    def build_graphs(step_fn):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for i in range(n_copies):  # warm-up outside capture (an even number of steps: parity is kept)
                step_fn(i)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graphs = []
        for g0 in range(0, n_copies, L):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for c in range(g0, g0 + L):
                    step_fn(c)
            graphs.append(g)
        return graphs

    def make_round(graphs):
        cursor = [0]

        def one_round():
            for _ in range(K // L):
                graphs[cursor[0] % len(graphs)].replay()
                cursor[0] += 1
        return one_round

    use_graph = not args.no_graph
    if use_graph:
        round_fn = make_round(build_graphs(step))
    else:
        cur = [0]

        def round_fn():
            for _ in range(K):
                step(cur[0])
                cur[0] += 1

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    # rounds: until the timed region lasts >= 50 ms (estimated from a probe round), at least 20
    probe = timed_rounds(round_fn, 3, max(1, (max(3, args.warmup) + K - 1) // K))
    est = float(np.median(probe))
    rounds = int(min(5000, max(20, np.ceil(50.0 / max(est, 1e-3)))))
    ms_rounds = timed_rounds(round_fn, rounds, 1)
    ms_per_step = float(np.median(ms_rounds)) / K
    value = layer_bytes_total / (ms_per_step * 1e-3) / 1e9
    # the same step the other way (one GPU: the single cooperative launch; N > 1: separate launches), for comparison
    if use_graph:
        other_round = make_round(build_graphs(step_other))
    else:
        cur_c = [0]

        def other_round():
            for _ in range(K):
                step_other(cur_c[0])
                cur_c[0] += 1
    ms_other = float(np.median(timed_rounds(other_round, max(20, rounds // 4), 2))) / K
    ms_chain, ms_fused = (ms_other, ms_per_step) if use_fused else (ms_per_step, ms_other)
    if world > 1:
        rows_round = make_round(build_graphs(step_rows)) if use_graph else None
        if rows_round is not None:
            ms_rows = float(np.median(timed_rounds(rows_round, max(20, rounds // 4), 2))) / K

    if use_graph:
        round_e2e = make_round(build_graphs(step_e2e))
    else:
        cur_e = [0]

        def round_e2e():
            for _ in range(K):
                step_e2e(cur_e[0])
                cur_e[0] += 1
    ms_e2e_rounds = timed_rounds(round_e2e, max(20, rounds // 2), 2)
    ms_e2e = float(np.median(ms_e2e_rounds)) / K
    e2e_value = layer_bytes_total / (ms_e2e * 1e-3) / 1e9
    e2e_check = None
    if world == 1:
        # the end-to-end call writes the same numbers the device-resident step does
        step(0)
        torch.cuda.synchronize()
        want = y_down.cpu()
        yd_host.zero_()
        step_e2e(0)
        torch.cuda.synchronize()
        e2e_check = bool(torch.equal(yd_host.reshape(-1), want.reshape(-1)))

    # dominant kernel alone: the Q4_K matvec over rotating copies, CUDA events on its stream
    q4k_bytes = copies[0][0].data.numel()
    mats = [copies[c][i] for c in range(n_copies) for i in (0, 1)]

    def q4k_only(i):
        for w in mats:
            rt.launch_matvec_xq8(w, xq, y_gate)
    if use_graph:
        gq = torch.cuda.CUDAGraph()
        q4k_only(0)
        torch.cuda.synchronize()
        with torch.cuda.graph(gq):
            q4k_only(0)

        def q4k_call():
            gq.replay()
    else:
        def q4k_call():
            q4k_only(0)
    q_rounds = timed_rounds(q4k_call, 200, 5)
    q4k_us = float(np.median(q_rounds)) * 1e3 / len(mats)
    clocks = sampler.stop() if rank == 0 else None

    # Q6_K down alone, for the per-format report
    q6_bytes = copies[0][2].data.numel()
    downs = [copies[c][2] for c in range(n_copies)]
    hq_src = hq if world == 1 else ga_h.buffer_ptr

    def q6_only():
        for w in downs:
            rt.launch_matvec_xq8(w, hq_src, y_down)
    q6_rounds = timed_rounds(q6_only, 100, 5)
    q6_us = float(np.median(q6_rounds)) * 1e3 / len(downs)

    mmq = moe = small = None
    if world == 1 and not args.skip_mmq:
        small = small_matvecs(rt, synth, torch, dev, timed)
        mmq = mmq_prefill(rt, synth, torch, dev, timed)
        moe = moe_layer(rt, synth, torch, dev, timed)

    moe_ep = mmq_rs = None
    if world > 1 and not args.skip_mmq:
        try:
            mmq_rs = mmq_prefill_row_sharded(rt, synth, torch, dist, dev, timed, rank, world)
        except Exception as e:  # the headline line must not depend on this extra
            mmq_rs = {"error": f"{type(e).__name__}: {e}"}
        try:
            moe_ep = moe_expert_parallel(rt, synth, torch, dist, dev, timed, rank, world)
        except Exception as e:
            moe_ep = {"error": f"{type(e).__name__}: {e}"}

    if rank == 0:
        peak, peak_kind = measured_peaks()
        achieved = q4k_bytes / (q4k_us * 1e-6) / 1e9
        traffic, traffic_src = q4k_dram_traffic()
        line = {
            "metric": "q4k_decode_matvec_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": K, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "rounds": rounds, "timed_region_ms": float(ms_rounds.sum()),
            "ms_per_step_min": float(ms_rounds.min()) / K, "ms_per_step_max": float(ms_rounds.max()) / K,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8 dp4a, f32 accumulate",
            "data": "synthetic", "config": workload_config(world),
            "e2e": {"value": e2e_value, "unit": "GB/s",
                    "h2d_bytes_per_step": HIDDEN * 4, "d2h_bytes_per_step": HIDDEN * 4,
                    "ms_per_step": ms_e2e, "ms_per_step_min": float(ms_e2e_rounds.min()) / K,
                    "ms_per_step_max": float(ms_e2e_rounds.max()) / K, "graph_replay": use_graph,
                    "how": ("runtime.launch_ffn_decode with the pinned host input and output as its x and y: the quantizer reads x "
                            "and the down matvec writes y across PCIe" if world == 1 else
                            "x uploaded by a copy kernel (rc_copy_small), the sharded launch whose last phase writes the summed output into the pinned host y"),
                    "equals_device_resident_step": e2e_check},
            "gpu_launches": launches_per_step * K * rounds,
            "step": ("one cooperative launch per GPU, tensor-parallel (rc_ffn_decode_tp: gate/up by rows, down by columns, partial "
                     "outputs summed in rank order)" if use_fused and tp is not None else
                     "one cooperative launch per GPU, all three projections by rows (rc_ffn_decode)" if use_fused else
                     "five launches (quantize, gate, up, SwiGLU + quantize, down) with programmatic dependent launch"),
            "ms_per_step_launch_chain": ms_chain, "ms_per_step_one_launch": ms_fused, "fused_vs_chain_rel_l2": fused_rel,
            "ms_per_step_one_launch_row_sharded": ms_rows, "tp_vs_chain_allreduce_rel_l2": tp_rel,
            "gather": "peer stores from inside the launch; arrival is read off the values" if world > 1 else None,
            "clocks": clocks,
            "roofline": {"bound": "hbm", "kernel": "matvec_rows_kernel<Q4_K,1,5> 5120->%d (the Q4_K decode matvec, timed alone)" % (FFN // world),
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": peak_kind, "us_per_launch": q4k_us, "bytes_per_launch": q4k_bytes,
                         "traffic": traffic if world == 1 else None, "traffic_source": traffic_src,
                         "fused_step": {"kernel": "ffn_tp_kernel<Q4_K,Q6_K>" if tp is not None else "ffn_decode_kernel<Q4_K,Q6_K>", "bytes_per_launch": layer_bytes_local,
                                        "us_per_launch": ms_fused * 1e3, "achieved": layer_bytes_local / (ms_fused * 1e-3) / 1e9,
                                        "frac": layer_bytes_local / (ms_fused * 1e-3) / 1e9 / peak}},
            "per_kernel": {"q4k_gate_up_gbs": achieved, "q6k_down_gbs": q6_bytes / (q6_us * 1e-6) / 1e9,
                           "q6k_us": q6_us},
            "tok_per_s_per_layer": 1e3 / ms_per_step,
            "graph_replay": use_graph, "graph_steps": L if use_graph else 0,
        }
        if small is not None:
            line.update(small)
        if mmq is not None:
            line["mmq_prefill"] = mmq
        if moe is not None:
            line["moe_grouped"] = moe
        if moe_ep is not None:
            line["moe_expert_parallel"] = moe_ep
        if mmq_rs is not None:
            line["mmq_prefill_row_sharded"] = mmq_rs
        if world == 1 and not args.no_cpu_baseline:
            v, sample, _ = cpu_layer_sample(seconds=12.0, threads=os.cpu_count() or 1)
            line["cpu_baseline"] = {"value": v, "unit": "GB/s", "cores": os.cpu_count() or 1, "kind": "port",
                                    "sample": sample}
        print(json.dumps(line), flush=True)
    for f in fused + (tp or []):
        f.close()
    if world > 1:
        ga_h.close()
        ga_y.close()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=30)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--skip-mmq", action="store_true", help="leave the prefill GEMM, MoE and small-matvec sections out")
    ap.add_argument("--profile-case", choices=["mmqx", "ffn"], help="run a few launches of one kernel on a small case (for ncu) and exit")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.profile_case:
        run_profile_case(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
