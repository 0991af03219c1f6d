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


def iq3s_planes(in_dim: int, out_dim: int, seed: int):
    """Planes of an IQ3_S-tagged tensor as src/quant/iq3_s.rs:216-260 writes them — the IQ4_XS layout:
    16 nibble bytes per (row, sub-block) (weight k low, k + 16 high, nibble n = (v + 15) / 2), then one
    fp16 `db` per (row, sub-block); the padding sub-block of a power-of-two row stays zero.  Returns the
    planes and the f64 weights db * (2n - 15) they stand for."""
    rng = np.random.default_rng(seed)
    n_sub, nsp = in_dim // 32, ro.nsp(in_dim)
    nib = np.zeros((out_dim, nsp, 16), dtype=np.uint8)
    nib[:, :n_sub] = rng.integers(0, 256, (out_dim, n_sub, 16), dtype=np.uint8)
    # db = d * (1 + 2 * scale4): spread over the 1..31 range of the sub-scale, both signs
    db = (rng.uniform(2e-4, 2e-3, (out_dim, n_sub)) * (1 + 2 * rng.integers(0, 16, (out_dim, n_sub)))
          * rng.choice([-1.0, 1.0], (out_dim, n_sub))).astype(np.float16)
    sc = np.zeros((out_dim, nsp), dtype=np.float16)
    sc[:, :n_sub] = db
    planes = np.concatenate([nib.reshape(-1), sc.reshape(-1).view(np.uint8)])
    n = np.concatenate([nib[:, :n_sub] & 15, nib[:, :n_sub] >> 4], axis=2).astype(np.float64)  # weights 0..15, 16..31
    w = (db.astype(np.float64)[:, :, None] * (2.0 * n - 15.0)).reshape(out_dim, in_dim)
    return planes, w
