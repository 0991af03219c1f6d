#!/usr/bin/env python
"""Benchmark of the quantized-weight decode hot path on B200.

A step is one pass of the decode FFN projections of a dense 27B-class layer at batch 1:
quantize_q8(x[5120]) -> Q4_K gate matvec and Q4_K up matvec (5120 -> 17408, sharing the
quantized x), quantize_q8(h[17408]) -> Q6_K down matvec (17408 -> 5120).  The metric is the
reference's: repacked weight bytes streamed per second (GB/s).  Steps rotate over several
distinct copies of the layer's weights so that no launch finds its weights in L2.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

With N > 1 (launched by torch.distributed.run, one rank per GPU) every matrix is split by
output rows, each rank streams its shard, and the shards' outputs are all-gathered.
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


def moe_layer(rt, synth, torch, dev, timed):
    """Config 5: 256 experts, top-8 of 512 tokens, hidden 2048, expert FFN 512: router top-k, sort,
    gather, grouped gate+up GEMM (Q4_K [1024, 2048] per expert), SwiGLU + quantize, grouped down
    GEMM (Q6_K [2048, 512]), scatter, weighted combine; every step a launch of the library.
    HBM-bound: the figure of merit is expert-weight bytes / s."""
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

    # The same layer through the grouped GEMM that takes f32 activations (f16 operands, whole-K
    # accumulation): the gather, the activation and both quantizations happen inside its prologue.
    gg = rt.MoeGroupedGemm(device=dev)

    def step_f32(i):
        rt.launch_moe_topk(logits, ids, wts, E, K, NT)
        rt.launch_moe_sort(moe, ids, NE)
        gg.gate_up(moe, gu, x, K, y1, NE)
        gg.down(moe, dn, y1, rt.ACT_SWIGLU, y2, NE)
        rt.launch_moe_scatter_rows(moe, y2, per_entry, H, NE)
        rt.launch_moe_combine(per_entry, ids, wts, None, out, H, K, NT)

    reps = 10
    us_i8 = timed(step, reps, 3) / reps * 1e3
    out_i8 = out.clone()
    us_f32 = timed(step_f32, reps, 3) / reps * 1e3
    rel = float((out - out_i8).norm() / out_i8.norm())
    us = min(us_i8, us_f32)
    us_gu = timed(lambda i: rt.launch_moe_grouped_gemm(moe, gu, xg, y1, H, 2 * F, NE), reps, 3) / reps * 1e3
    us_dn = timed(lambda i: rt.launch_moe_grouped_gemm(moe, dn, hq, y2, F, H, NE), reps, 3) / reps * 1e3
    us_gu32 = timed(lambda i: gg.gate_up(moe, gu, x, K, y1, NE), reps, 3) / reps * 1e3
    us_dn32 = timed(lambda i: gg.down(moe, dn, y1, rt.ACT_SWIGLU, y2, NE), reps, 3) / reps * 1e3
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

    # replayed from a CUDA graph of one pass over all 32 expert groups, as a decode loop would be
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
            "us_layer": us, "tok_per_s_per_layer": NT / (us * 1e-6), "tops": 2.0 * NE * (H * 2 * F + F * H) / us / 1e6,
            "us_layer_blockq8_route": us_i8, "us_layer_f32_route": us_f32, "rel_l2_between_routes": rel,
            "us_gate_up": us_gu, "us_down": us_dn, "us_gate_up_f32_route": us_gu32, "us_down_f32_route": us_dn32,
            "decode_1_token": {"us": us_dec, "expert_bytes": dec_bytes, "gbs": dec_bytes / us_dec / 1e3,
                               "frac_of_hbm_peak": dec_bytes / us_dec / 1e3 / peak,
                               "launches": "expert matvec (gate+up), SwiGLU+quantize, expert matvec (down)"},
            "roofline": {"bound": "hbm", "achieved": wbytes / us / 1e3, "peak": peak, "unit": "GB/s",
                         "frac": wbytes / us / 1e3 / peak, "note": "expert-weight bytes over the whole layer time"}}


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
        "l2": "weights rotate over 3 distinct layer copies (528 MB > 4x L2); every launch reads cold HBM",
        "parallelism": (f"row-shard x{n_gpus}; all-gather of the quantized intermediate and of down's output "
                        "(peer-memory push over NVLink, or NCCL with --nccl-gather)" if n_gpus > 1 else "single GPU"),
    }


# ------------------------------------------------------------------------------------- GPU arm

# DRAM bytes of one Q4_K 5120->17408 matvec launch, from the ncu capture summarised in
# profiles/matvec_q4k_5120x17408.md (algorithmic bytes: 51,527,680).
Q4K_DRAM_TRAFFIC_BYTES = 51_566_000
INT8_DENSE_PEAK_TOPS = 4500.0  # nominal B200 dense int8; no measured int8 figure is supplied


def measured_tensor_peak() -> tuple[float, str]:
    """Burst bf16 GEMM throughput measured on this pool (the f16 kind runs at the same rate)."""
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["bf16_tflops"]), "measured bf16 burst"
        except Exception:
            pass
    return 1590.0, "fallback"


def moe_expert_parallel(rt, synth, torch, dist, dev, timed, rank, world):
    """Config 5 sharded by experts over the ranks (N > 1): 256 experts split evenly, every rank routes its
    own 512 / N tokens (top-8), the routed activation rows go to the owner of their expert by NCCL
    all-to-all (counts first), through the grouped gate+up GEMM there, and the results travel back.  The
    collectives are host-driven (eager NCCL), so the step is timed eagerly; value = tokens of all ranks per
    second through this gate+up stage."""
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
    gg = rt.MoeGroupedGemm(device=dev)
    state = {}

    def step(i):
        rt.launch_moe_topk(logits, ids, wts, E, K, nt)
        flat = ids.reshape(-1)
        plan = sh.plan_dispatch(flat, E)
        rows_in = sh.dispatch_rows(x.repeat_interleave(K, dim=0).contiguous(), plan)
        ids_in = (sh.dispatch_rows(flat.to(torch.float32).reshape(-1, 1), plan).reshape(-1).to(torch.int32) - e0).contiguous()
        n_in = rows_in.shape[0]
        moe = rt.MoeGroupedScratch.new(n_local, n_in, device=dev)
        rt.launch_moe_sort(moe, ids_in, n_in)
        y_sorted = torch.empty(n_in, 2 * F, device=dev)
        gg.gate_up(moe, gu, rows_in, 1, y_sorted, n_in)
        y_in = torch.empty(n_in, 2 * F, device=dev)
        rt.launch_moe_scatter_rows(moe, y_sorted, y_in, 2 * F, n_in)
        state["y"] = sh.combine_rows(y_in, plan)
        state["n_in"] = n_in

    reps = 5
    us = timed(step, reps, 3) / reps * 1e3
    return {"workload": f"config 5 gate+up stage, {E} experts over {world} ranks, {nt} tokens per rank, top-{K}",
            "us_step": us, "tok_per_s": NT / (us * 1e-6), "rows_received_rank0": state.get("n_in"),
            "collectives": "NCCL all_to_all_single: counts, rows, expert ids, results (eager, host-driven)"}


def mmq_prefill_row_sharded(rt, synth, torch, dist, dev, timed, rank, world):
    """Config 4 sharded by output rows (N > 1): every rank holds rows [b, e) of the Q4_K 5120->17408 matrix
    (multiples of 32 rows), runs the prefill GEMM of all 512 tokens against them, and the [512, e - b]
    outputs are all-gathered (NCCL all_gather_into_tensor, eager) into [N, 512, widest shard]; no other
    exchange.  Timed as the whole step, max over ranks; TOPS counts the whole 91.3 GOP."""
    from reinstinct_b200 import sharding as sh

    P = 512
    raw = synth.synth_blocks(Q4_K, HIDDEN, FFN, seed=77)
    shard, n_rows = sh.shard_raw_rows(raw, Q4_K, HIDDEN, FFN, rank, world)
    w = rt.GpuMatvecTensor.from_bytes_matvec(shard.copy(), Q4_K, HIDDEN, n_rows, device=dev)
    x = torch.from_numpy(synth.synth_activations(P, HIDDEN, 78)).to(dev)
    gemm = rt.PrefillGemm(max_x=P * HIDDEN, device=dev)
    widest = max(e - b for b, e in (sh.row_shard_range(FFN, r, world) for r in range(world)))
    y = torch.zeros((P, widest), dtype=torch.float32, device=dev)
    y_local = y if n_rows == widest else torch.empty((P, n_rows), dtype=torch.float32, device=dev)
    gathered = torch.empty((world * P, widest), dtype=torch.float32, device=dev)

    def step(i):
        gemm.matmul_into(y_local, w, x, P)
        if y_local is not y:
            y[:, :n_rows] = y_local
        dist.all_gather_into_tensor(gathered, y)

    def gemm_only(i):
        gemm.matmul_into(y_local, w, x, P)

    reps = 10
    us = timed(step, reps, 3) / reps * 1e3
    us_gemm = timed(gemm_only, reps, 3) / reps * 1e3
    ops = 2.0 * P * HIDDEN * FFN
    return {"workload": f"config 4 row-sharded: 512 tokens x Q4_K 5120->17408, {n_rows} rows on rank 0 of {world}",
            "us_step": us, "us_gemm_only": us_gemm, "tops": ops / (us * 1e-6) / 1e12,
            "gather": f"NCCL all_gather_into_tensor of {P * widest * 4} bytes per rank (eager)"}


def mmq_prefill(rt, synth, torch, dev, timed):
    """Config 4: dense prefill GEMM, 512 tokens x Q4_K 5120->17408, through PrefillGemm (f32
    activations in: f16 image + tcgen05 kind::f16 GEMM) and through the int8 entry point given
    BlockQ8 records (exact integer dots).  TOPS = 2*P*K*N / t."""
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
    ms_k = timed(lambda i: rt.launch_mmq_gemm(w, xq, y, P), reps, 3) / reps
    ms_q = timed(lambda i: gemm.matmul_into(y, w, x, P), reps, 3) / reps
    tops_q = ops / (ms_q * 1e-3) / 1e12
    peak, peak_kind = measured_tensor_peak()
    return {"workload": "config 4: 512 tokens x Q4_K 5120->17408 (91.3 GOP)",
            "kernel": "activations_to_f16_kernel + mmqd_kernel<Q4_K,512> (tcgen05 kind::f16, f32 accumulator in tensor "
                      "memory over the whole K; TMA-fed raw weights, bulk-copied activation image)",
            "us_matmul_f32_in": ms_q * 1e3, "tops_matmul_f32_in": tops_q,
            "us_mmq_blockq8_in": ms_k * 1e3, "tops_mmq_blockq8_in": ops / (ms_k * 1e-3) / 1e12,
            "note": "matmul_f32_in = PrefillGemm (two launches, both timed); mmq_blockq8_in = mmq_kernel<Q4_K,128,16,2> "
                    "(tcgen05 kind::i8, exact integer dots, one accumulator drain per 32-wide sub-block)",
            "roofline": {"bound": "tensor", "achieved": tops_q, "peak": peak, "unit": "TFLOP/s",
                         "frac": tops_q / peak, "peak_kind": peak_kind,
                         "frac_of_nominal_int8": tops_q / INT8_DENSE_PEAK_TOPS,
                         "timed": "PrefillGemm call, activation-image launch included"},
            "tok_per_s_per_layer_gate_only": P / (ms_q * 1e-3)}


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
        dist.init_process_group("nccl", device_id=dev)
    rt.init(local)

    n_copies = 3
    # Row shards: rank r owns rows [r*out/world, (r+1)*out/world) of every matrix; shard sizes
    # are multiples of 32 so quantize-then-gather equals gather-then-quantize.
    shards = []
    for name, t, in_dim, out_dim in LAYER:
        assert out_dim % (32 * world) == 0
        shards.append((name, t, in_dim, out_dim // world))
    copies = []
    layer_bytes_local = 0
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
    # gate | up outputs side by side (this rank's rows)
    y_gu = torch.empty(2 * (FFN // world), device=dev)
    y_gate, y_up = y_gu[:FFN // world], y_gu[FFN // world:]
    y_down = torch.empty(HIDDEN // world, device=dev)
    g_gate = torch.empty(FFN, device=dev) if world > 1 else y_gate
    g_up = torch.empty(FFN, device=dev) if world > 1 else y_up
    g_down = torch.empty(HIDDEN, device=dev) if world > 1 else y_down
    yd_host = torch.empty(HIDDEN, dtype=torch.float32).pin_memory()
    launches_per_step = 5

    # The intermediate h = silu(gate) * up is made and quantized in one launch (rc_swiglu_q8), so the
    # step is the decode FFN as the engine runs it: quantize x, gate, up, SwiGLU+quantize, down.
    # N > 1: gate and up stay sharded (the activation between them and down is elementwise); each
    # rank produces its 1/N of the quantized intermediate and the BlockQ8 shards are all-gathered (21.7 KB
    # instead of 2 x 68 KB of f32); down's output rows are all-gathered for the next layer.  The
    # gathers are rc_allgather_push (stores into peer memory over NVLink + a counter handshake),
    # so the whole sharded step replays from one CUDA graph; --nccl-gather uses NCCL instead.
    h_local = FFN // world
    hq_local = torch.empty((h_local // 32) * 40, dtype=torch.uint8, device=dev) if world > 1 else hq
    push = world > 1 and not args.nccl_gather
    if push:
        ga_h = rt.PeerAllGather(hq_local.numel())
        ga_y = rt.PeerAllGather(y_down.numel() * 4)
        hq_in, y_full = ga_h.buffer_ptr, ga_y
    else:
        hq_in = hq

    def step(c: int):
        ws = copies[c % n_copies]
        rt.launch_quantize_q8(x_dev, xq, HIDDEN, 1)
        rt.launch_matvec_xq8(ws[0], xq, y_gate)
        rt.launch_matvec_xq8(ws[1], xq, y_up)
        rt.launch_swiglu_q8(y_gate, y_up, None, hq_local, h_local)
        if world > 1:
            if push:
                ga_h.gather(hq_local)
            else:
                dist.all_gather_into_tensor(hq, hq_local)
        rt.launch_matvec_xq8(ws[2], hq_in, y_down)
        if world > 1:
            if push:
                ga_y.gather(y_down)
            else:
                dist.all_gather_into_tensor(g_down, y_down)

    if push:
        # one checked step: the gathered BlockQ8 must equal SwiGLU+quantize of the whole gathered vectors
        step(0)
        got = torch.empty_like(hq)
        ga_h.copy_out(got)
        dist.all_gather_into_tensor(g_gate, y_gate)
        dist.all_gather_into_tensor(g_up, y_up)
        rt.launch_swiglu_q8(g_gate, g_up, None, hq, FFN)
        torch.cuda.synchronize()
        assert torch.equal(got, hq), "peer gather of the quantized intermediate differs from the local quantization"

    # End-to-end step: the layer's input comes from pinned host memory and its output goes back there,
    # both inside the step.
    def step_e2e(c: int):
        x_dev.copy_(in_host, non_blocking=True)
        step(c)
        if push:
            ga_y.copy_out(yd_host)
        else:
            yd_host.copy_(g_down, non_blocking=True)

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

    # The decode loop is launch-bound from Python (8 us kernels), so the steps are replayed
    # from a CUDA graph, as the reference's engine replays its forward (graph of n_copies steps).
    # (Replaying NCCL collectives captured together with these launches hung on 2 GPUs, so with
    # --nccl-gather the steps are launched eagerly and are bound by host launch latency.)
    use_graph = (world == 1 or push) and not args.no_graph
    if use_graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for i in range(3):
                step(i)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for c in range(n_copies):
                step(c)

        def run_steps(i):
            graph.replay()
        steps_per_call = n_copies
    else:
        run_steps = step
        steps_per_call = 1

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    calls = max(1, (args.steps + steps_per_call - 1) // steps_per_call)
    steps_timed = calls * steps_per_call
    ms = timed(run_steps, calls, max(3, (args.warmup + steps_per_call - 1) // steps_per_call))
    ms_per_step = ms / steps_timed
    value = layer_bytes_total / (ms_per_step * 1e-3) / 1e9

    # end to end: host buffers in, host buffers out, copies inside the timed region.  Like the
    # device-resident steps, a user replays this from a CUDA graph (pinned-memory copies are
    # ordinary graph nodes): n_copies steps per graph, every one with its own uploads and downloads.
    if use_graph:
        for i in range(2):
            step_e2e(i)
        torch.cuda.synchronize()
        graph_e2e = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph_e2e):
            for c in range(n_copies):
                step_e2e(c)
        e2e_calls = max(1, (args.steps + n_copies - 1) // n_copies)
        ms_e2e = timed(lambda i: graph_e2e.replay(), e2e_calls, 3)
        e2e_steps = e2e_calls * n_copies
    else:
        ms_e2e = timed(step_e2e, args.steps, max(3, args.warmup))
        e2e_steps = args.steps
    e2e_value = layer_bytes_total / (ms_e2e / e2e_steps * 1e-3) / 1e9

    # The same step with no copy nodes: pinned host memory is addressable from the device, so the first
    # kernel reads x and the last one writes y straight across PCIe (single GPU; reported beside e2e).
    zero_copy = None
    if world == 1 and use_graph:
        def step_zc(c: int):
            ws = copies[c % n_copies]
            rt.launch_quantize_q8(in_host, xq, HIDDEN, 1)
            rt.launch_matvec_xq8(ws[0], xq, y_gate)
            rt.launch_matvec_xq8(ws[1], xq, y_up)
            rt.launch_swiglu_q8(y_gate, y_up, None, hq, FFN)
            rt.launch_matvec_xq8(ws[2], hq, yd_host)
        yd_host.zero_()
        step(0)
        torch.cuda.synchronize()
        want = y_down.cpu()
        step_zc(0)
        torch.cuda.synchronize()
        if torch.equal(yd_host.reshape(-1), want.reshape(-1)):
            graph_zc = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph_zc):
                for c in range(n_copies):
                    step_zc(c)
            calls = max(1, (args.steps + n_copies - 1) // n_copies)
            ms_zc = timed(lambda i: graph_zc.replay(), calls, 3) / (calls * n_copies)
            zero_copy = {"value": layer_bytes_total / (ms_zc * 1e-3) / 1e9, "ms_per_step": ms_zc,
                         "note": "x read and y written in pinned host memory by the kernels themselves"}

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

        def q4k_call(i):
            gq.replay()
    else:
        q4k_call = q4k_only
    reps = max(20, args.steps // 2)
    ms_q = timed(q4k_call, reps, 5)
    q4k_us = ms_q * 1e3 / (reps * len(mats))
    clocks = sampler.stop() if rank == 0 else None

    clocks = clocks  # sampled over the layer, e2e and Q4_K regions above
    # Q6_K down alone, for the per-format report
    q6_bytes = copies[0][2].data.numel()
    downs = [copies[c][2] for c in range(n_copies)]

    def q6_only(i):
        for w in downs:
            rt.launch_matvec_xq8(w, hq, y_down)
    ms_6 = timed(q6_only, reps, 5)
    q6_us = ms_6 * 1e3 / (reps * len(downs))

    mmq = moe = None
    if world == 1 and not args.skip_mmq:
        mmq = mmq_prefill(rt, synth, torch, dev, timed)
        moe = moe_layer(rt, synth, torch, dev, timed)

    moe_ep = None
    if world > 1 and not args.skip_mmq:
        try:
            moe_ep = moe_expert_parallel(rt, synth, torch, dist, dev, timed, rank, world)
        except Exception as e:  # the headline line must not depend on this extra
            moe_ep = {"error": f"{type(e).__name__}: {e}"}

    mmq_rs = None
    if world > 1 and not args.skip_mmq:
        try:
            mmq_rs = mmq_prefill_row_sharded(rt, synth, torch, dist, dev, timed, rank, world)
        except Exception as e:
            mmq_rs = {"error": f"{type(e).__name__}: {e}"}

    if rank == 0:
        peak, peak_kind = measured_peaks()
        achieved = q4k_bytes / (q4k_us * 1e-6) / 1e9
        line = {
            "metric": "q4k_decode_matvec_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": steps_timed, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8 dp4a, f32 accumulate",
            "data": "synthetic", "config": workload_config(world),
            "e2e": {"value": e2e_value, "unit": "GB/s",
                    "h2d_bytes_per_step": HIDDEN * 4, "d2h_bytes_per_step": HIDDEN * 4,
                    "ms_per_step": ms_e2e / e2e_steps, "graph_replay": use_graph, "zero_copy": zero_copy},
            "gpu_launches": (launches_per_step + (2 if push else 0)) * steps_timed,
            "gather": ("peer-push" if push else "nccl") if world > 1 else None,
            "clocks": clocks,
            "roofline": {"bound": "hbm", "kernel": "matvec_rows_kernel<Q4_K,1,5> 5120->%d" % (FFN // world),
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": peak_kind, "us_per_launch": q4k_us, "bytes_per_launch": q4k_bytes,
                         "traffic": Q4K_DRAM_TRAFFIC_BYTES if world == 1 else None,
                         "traffic_source": "profiles/matvec_q4k_5120x17408.md (ncu dram__bytes_read.sum + dram__bytes_write.sum, one launch)"},
            "per_kernel": {"q4k_gate_up_gbs": achieved, "q6k_down_gbs": q6_bytes / (q6_us * 1e-6) / 1e9,
                           "q6k_us": q6_us},
            "tok_per_s_per_layer": 1e3 / ms_per_step,
            "graph_replay": use_graph,
        }
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
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=30)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--nccl-gather", action="store_true", help="N > 1: gather with NCCL instead of rc_allgather_push")
    ap.add_argument("--skip-mmq", action="store_true", help="leave the config-4 prefill GEMM section out")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
