"""Shared case builders for the CPU and GPU parity tests (test infrastructure)."""
from __future__ import annotations

import struct

import numpy as np

import oracle as ro
from reinstinct_b200 import synth
from reinstinct_b200.synth import Lcg


def f16b(v) -> np.ndarray:
    return np.frombuffer(struct.pack("<H", ro.f32_to_f16(float(np.float32(v)))), dtype=np.uint8)


def lcg_case(t: int, in_dim: int, out_dim: int, seed: int, inc: int = 1442695040888963407) -> np.ndarray:
    """Weights the way the reference's kernel tests build them: every byte from the LCG, then
    tame f16 scales written at the format's d / dmin offsets
    (src/runtime/kernels.rs:3031-3045, 3141-3152; src/runtime/prefill.rs:604-626)."""
    bw, bb = ro.block_weights(t), ro.block_bytes(t)
    n = out_dim * (in_dim // bw)
    raw = Lcg(seed, inc).bytes(n * bb).reshape(n, bb).copy()
    for blk in range(n):
        d = (np.float32(blk % 29) - np.float32(14.0)) * np.float32(0.003)
        off = 208 if t == ro.Q6_K else 0
        raw[blk, off:off + 2] = f16b(d)
        if t in (ro.Q4_K, ro.Q5_K):
            raw[blk, 2:4] = f16b((np.float32(blk % 17) - np.float32(8.0)) * np.float32(0.0015))
    return raw.reshape(-1)


def lcg_x(n: int, seed: int) -> np.ndarray:
    return Lcg(seed).activations(n)


def f32_path(t: int, raw: np.ndarray, x: np.ndarray, in_dim: int, out_dim: int) -> np.ndarray:
    """dequantize_to_f32 + cpu::ops::matvec, the reference tests' oracle."""
    return ro.cpu_path(t, raw, x, in_dim, out_dim, n_threads=4)


def synth_case(t: int, in_dim: int, out_dim: int, n_rows: int, seed: int, signed: bool = True):
    raw = synth.synth_blocks(t, in_dim, out_dim, seed, signed_scales=signed)
    x = synth.synth_activations(n_rows, in_dim, seed + 1000)
    return raw, x
