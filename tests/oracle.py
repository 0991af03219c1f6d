"""ctypes wrapper of the CPU oracle (oracle/libro_oracle.so).  Test infrastructure only."""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

ORACLE_DIR = Path(__file__).resolve().parent.parent / "oracle"
LIB_PATH = ORACLE_DIR / "libro_oracle.so"

Q4_0, Q8_0, Q4_K, Q5_K, Q6_K, IQ4_XS = 2, 8, 12, 13, 14, 23
ALL_TYPES = (Q4_0, Q8_0, Q4_K, Q5_K, Q6_K, IQ4_XS)
NAMES = {Q4_0: "q4_0", Q8_0: "q8_0", Q4_K: "q4_k", Q5_K: "q5_k", Q6_K: "q6_k", IQ4_XS: "iq4_xs"}

_lib = None


def build() -> Path:
    src = [ORACLE_DIR / "ro_oracle.c", ORACLE_DIR / "ro_oracle.h"]
    if not LIB_PATH.exists() or any(s.stat().st_mtime > LIB_PATH.stat().st_mtime for s in src):
        subprocess.run(["make", "-C", str(ORACLE_DIR)], check=True, capture_output=True)
    return LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(str(LIB_PATH))
        sz, vp, i = C.c_size_t, C.c_void_p, C.c_int
        L.ro_f16_to_f32.restype = C.c_float
        L.ro_f16_to_f32.argtypes = [C.c_uint16]
        L.ro_f32_to_f16.restype = C.c_uint16
        L.ro_f32_to_f16.argtypes = [C.c_float]
        L.ro_bf16_to_f32.restype = C.c_float
        L.ro_bf16_to_f32.argtypes = [C.c_uint16]
        for name in ("ro_block_bytes", "ro_block_weights"):
            getattr(L, name).restype = sz
            getattr(L, name).argtypes = [i]
        L.ro_nsp.restype = sz
        L.ro_nsp.argtypes = [sz]
        L.ro_repacked_len.restype = sz
        L.ro_repacked_len.argtypes = [i, sz, sz]
        L.ro_dequantize.restype = i
        L.ro_dequantize.argtypes = [i, vp, vp, sz]
        L.ro_repack.restype = i
        L.ro_repack.argtypes = [i, vp, sz, sz, vp]
        L.ro_quantize_q8.restype = None
        L.ro_quantize_q8.argtypes = [vp, vp, sz, sz]
        L.ro_dequantize_q8.restype = None
        L.ro_dequantize_q8.argtypes = [vp, vp, sz, sz]
        L.ro_matvec_q8.restype = i
        L.ro_matvec_q8.argtypes = [i, vp, vp, sz, sz, sz, sz, sz, vp, vp, vp]
        L.ro_matvec_f32.restype = None
        L.ro_matvec_f32.argtypes = [vp, vp, sz, sz, vp, i]
        L.ro_cpu_path.restype = i
        L.ro_cpu_path.argtypes = [i, vp, vp, sz, sz, sz, vp, vp, i, i]
        L.ro_moe_sort.restype = None
        L.ro_moe_sort.argtypes = [vp, sz, sz, sz, vp, vp, vp, vp]
        L.ro_router_topk.restype = None
        L.ro_router_topk.argtypes = [vp, sz, sz, sz, vp, vp]
        for name in ("ro_dequantize_q3_k", "ro_q3k_to_q6k", "ro_dequantize_iq4_nl", "ro_quantize_q8_0"):
            getattr(L, name).restype = None
            getattr(L, name).argtypes = [vp, vp, sz]
        L.ro_rmsnorm_q8.restype = None
        L.ro_rmsnorm_q8.argtypes = [vp, vp, vp, vp, vp, vp, sz, sz, C.c_float]
        L.ro_sigmoid_mul_q8.restype = None
        L.ro_sigmoid_mul_q8.argtypes = [vp, vp, vp, sz]
        L.ro_rmsnorm_gated_q8.restype = None
        L.ro_rmsnorm_gated_q8.argtypes = [vp, vp, vp, vp, vp, sz, sz, C.c_float]
        L.ro_swiglu_q8.restype = None
        L.ro_swiglu_q8.argtypes = [vp, vp, vp, vp, sz]
        L.ro_kernel_type.restype = i
        L.ro_kernel_type.argtypes = [i]
        L.ro_repack_any.restype = i
        L.ro_repack_any.argtypes = [i, vp, sz, sz, vp]
        L.ro_moe_act_q8.restype = None
        L.ro_moe_act_q8.argtypes = [vp, vp, sz, sz, i, vp]
        L.ro_moe_combine.restype = None
        L.ro_moe_combine.argtypes = [vp, vp, vp, vp, vp, sz, sz, sz]
        L.ro_grouped_q8.restype = i
        L.ro_grouped_q8.argtypes = [i, vp, sz, vp, sz, vp, sz, sz, vp, vp]
        _lib = L
    return _lib


def _p(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def f16_to_f32(bits: int) -> float:
    return float(lib().ro_f16_to_f32(bits))


def f32_to_f16(v: float) -> int:
    return int(lib().ro_f32_to_f16(C.c_float(v)))


def block_bytes(t: int) -> int:
    return lib().ro_block_bytes(t)


def block_weights(t: int) -> int:
    return lib().ro_block_weights(t)


def nsp(in_dim: int) -> int:
    return lib().ro_nsp(in_dim)


def repacked_len(t: int, in_dim: int, out_dim: int) -> int:
    return lib().ro_repacked_len(t, in_dim, out_dim)


def dequantize(t: int, blocks: np.ndarray, n_weights: int) -> np.ndarray:
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    out = np.empty(n_weights, dtype=np.float32)
    assert lib().ro_dequantize(t, _p(blocks), _p(out), n_weights) == 0
    return out


def repack(t: int, blocks: np.ndarray, in_dim: int, out_dim: int) -> np.ndarray:
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    n = repacked_len(t, in_dim, out_dim)
    assert n > 0, "unsupported shape"
    out = np.empty(n, dtype=np.uint8)
    assert lib().ro_repack(t, _p(blocks), in_dim, out_dim, _p(out)) == 0
    return out


def quantize_q8(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    x2 = x.reshape(-1, x.shape[-1])
    n_vec, in_dim = x2.shape
    out = np.empty(n_vec * (in_dim // 32) * 40, dtype=np.uint8)
    lib().ro_quantize_q8(_p(x2), _p(out), in_dim, n_vec)
    return out


def dequantize_q8(xq: np.ndarray, in_dim: int, n_vec: int) -> np.ndarray:
    out = np.empty((n_vec, in_dim), dtype=np.float32)
    lib().ro_dequantize_q8(_p(np.ascontiguousarray(xq)), _p(out), in_dim, n_vec)
    return out


def matvec_q8(t: int, w: np.ndarray, xq: np.ndarray, in_dim: int, out_dim: int, n_rows: int = 1,
              want_idots: bool = False):
    """Returns (y32 [n_rows,out], y64 [n_rows,out], idots [n_rows,out,n_sub,2] or None)."""
    w = np.ascontiguousarray(w, dtype=np.uint8)
    xq = np.ascontiguousarray(xq, dtype=np.uint8)
    y32 = np.empty((n_rows, out_dim), dtype=np.float32)
    y64 = np.empty((n_rows, out_dim), dtype=np.float64)
    idots = np.empty((n_rows, out_dim, in_dim // 32, 2), dtype=np.int32) if want_idots else None
    rc = lib().ro_matvec_q8(t, _p(w), _p(xq), in_dim, out_dim, n_rows, 0, out_dim, _p(y32), _p(y64), _p(idots))
    assert rc == 0
    return y32, y64, idots


def matvec_f32(x: np.ndarray, w: np.ndarray, in_dim: int, out_dim: int, n_threads: int = 1) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    y = np.empty(out_dim, dtype=np.float32)
    lib().ro_matvec_f32(_p(x), _p(w), in_dim, out_dim, _p(y), n_threads)
    return y


def cpu_path(t: int, blocks: np.ndarray, x: np.ndarray, in_dim: int, out_dim: int, n_threads: int = 1,
             w_f32: np.ndarray | None = None, dequant: bool = True) -> np.ndarray:
    """The reference's CPU path: dequantize to f32, then sequential-f32 row dots."""
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, in_dim)
    n_rows = x.shape[0]
    if w_f32 is None:
        w_f32 = np.empty(out_dim * in_dim, dtype=np.float32)
    y = np.empty((n_rows, out_dim), dtype=np.float32)
    rc = lib().ro_cpu_path(t, _p(np.ascontiguousarray(blocks)), _p(x), in_dim, out_dim, n_rows, _p(w_f32),
                           _p(y), n_threads, 1 if dequant else 0)
    assert rc == 0
    return y


def moe_sort(ids: np.ndarray, n_expert: int, bn: int):
    ids = np.ascontiguousarray(ids, dtype=np.int32).reshape(-1)
    n = ids.size
    count = np.zeros(n_expert, dtype=np.int32)
    eoff = np.zeros(n_expert + 1, dtype=np.int32)
    toff = np.zeros(n_expert + 1, dtype=np.int32)
    perm = np.full(max(n, 1), -1, dtype=np.int32)
    lib().ro_moe_sort(_p(ids), n, n_expert, bn, _p(count), _p(eoff), _p(toff), _p(perm))
    return count, eoff, toff, perm[:n]


def router_topk(logits: np.ndarray, n_used: int):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    n_tok, n_expert = logits.shape
    ids = np.empty((n_tok, n_used), dtype=np.int32)
    wts = np.empty((n_tok, n_used), dtype=np.float32)
    lib().ro_router_topk(_p(logits), n_tok, n_expert, n_used, _p(ids), _p(wts))
    return ids, wts


Q5_1 = 7    # the Q5_K kernel bodies with dsc = d, deff = -m (src/quant/q5_1.rs:11-20)
IQ3_S = 21  # kernel type only: IQ4_XS planes read through the codebook 2n - 15 (src/quant/iq3_s.rs:193-214)
Q3_K, IQ4_NL, BF16 = 11, 20, 30  # source-only types, relabelled onto Q6_K / IQ4_XS / Q8_0
SRC_BLOCK = {Q3_K: (256, 110), IQ4_NL: (32, 18), BF16: (1, 2)}  # weights, bytes per source block


def kernel_type(src_type: int) -> int:
    return lib().ro_kernel_type(src_type)


def dequantize_src(src_type: int, blocks: np.ndarray, n_weights: int) -> np.ndarray:
    """Direct decode of a source-only type (not through the relabelling)."""
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    out = np.empty(n_weights, dtype=np.float32)
    if src_type == Q3_K:
        lib().ro_dequantize_q3_k(_p(blocks), _p(out), n_weights)
    elif src_type == IQ4_NL:
        lib().ro_dequantize_iq4_nl(_p(blocks), _p(out), n_weights)
    elif src_type == BF16:
        out = (blocks.view(np.uint16).astype(np.uint32) << 16).view(np.float32)[:n_weights].copy()
    else:
        raise ValueError(src_type)
    return out


def q3k_to_q6k(blocks: np.ndarray, n_weights: int) -> np.ndarray:
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    out = np.empty(n_weights // 256 * 210, dtype=np.uint8)
    lib().ro_q3k_to_q6k(_p(blocks), _p(out), n_weights)
    return out


def quantize_q8_0(vals: np.ndarray) -> np.ndarray:
    vals = np.ascontiguousarray(vals, dtype=np.float32).reshape(-1)
    out = np.empty(vals.size // 32 * 34, dtype=np.uint8)
    lib().ro_quantize_q8_0(_p(vals), _p(out), vals.size)
    return out


def repack_any(src_type: int, blocks: np.ndarray, in_dim: int, out_dim: int) -> np.ndarray:
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    # IQ4_NL has no superblock: its planes (those of Q4_0) exist for any in_dim % 32 == 0
    n = repacked_len(Q4_0 if src_type == IQ4_NL else kernel_type(src_type), in_dim, out_dim)
    assert n > 0, "shape not allowed for the type"
    out = np.zeros(n, dtype=np.uint8)
    rc = lib().ro_repack_any(src_type, _p(blocks), in_dim, out_dim, _p(out))
    assert rc == 0, rc
    return out


def rmsnorm_q8(x: np.ndarray, w: np.ndarray, eps: float, add: np.ndarray | None = None):
    """x [n_vec, n] (+ add) -> (hidden f32, y f32, BlockQ8 bytes)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    n_vec, n = x.shape
    a = None if add is None else np.ascontiguousarray(add, dtype=np.float32)
    hid, y = np.empty_like(x), np.empty_like(x)
    out = np.zeros(n_vec * (n // 32) * 40, dtype=np.uint8)
    lib().ro_rmsnorm_q8(_p(x), _p(a), _p(np.ascontiguousarray(w, dtype=np.float32)), _p(hid), _p(y), _p(out), n, n_vec, eps)
    return hid, y, out


def sigmoid_mul_q8(x: np.ndarray, gate: np.ndarray):
    v = np.ascontiguousarray(x, dtype=np.float32).reshape(-1).copy()
    gate = np.ascontiguousarray(gate, dtype=np.float32).reshape(-1)
    out = np.zeros(v.size // 32 * 40, dtype=np.uint8)
    lib().ro_sigmoid_mul_q8(_p(v), _p(gate), _p(out), v.size)
    return v, out


def rmsnorm_gated_q8(x: np.ndarray, z: np.ndarray, w: np.ndarray, eps: float):
    x = np.ascontiguousarray(x, dtype=np.float32)
    n_heads, head_dim = x.shape
    y = np.empty_like(x)
    out = np.zeros(x.size // 32 * 40, dtype=np.uint8)
    lib().ro_rmsnorm_gated_q8(_p(x), _p(np.ascontiguousarray(z, dtype=np.float32)), _p(np.ascontiguousarray(w, dtype=np.float32)),
                              _p(y), _p(out), n_heads, head_dim, eps)
    return y, out


def swiglu_q8(gate: np.ndarray, up: np.ndarray):
    gate = np.ascontiguousarray(gate, dtype=np.float32).reshape(-1)
    up = np.ascontiguousarray(up, dtype=np.float32).reshape(-1)
    v = np.empty_like(gate)
    out = np.zeros(gate.size // 32 * 40, dtype=np.uint8)
    lib().ro_swiglu_q8(_p(gate), _p(up), _p(v), _p(out), gate.size)
    return v, out


def moe_act_q8(gu: np.ndarray, act: int):
    """gu f32 [n_slot, 2*ff] -> (BlockQ8 bytes [n_slot, ff/32, 40], f32 activations [n_slot, ff])."""
    gu = np.ascontiguousarray(gu, dtype=np.float32)
    n_slot, ff2 = gu.shape
    ff = ff2 // 2
    out = np.zeros((n_slot, ff // 32, 40), dtype=np.uint8)
    v = np.zeros((n_slot, ff), dtype=np.float32)
    lib().ro_moe_act_q8(_p(gu), _p(out), ff, n_slot, act, _p(v))
    return out, v


def moe_combine(experts: np.ndarray, ids: np.ndarray, weights: np.ndarray, expert_scale: np.ndarray | None):
    experts = np.ascontiguousarray(experts, dtype=np.float32)
    n_tok, n_used, hidden = experts.shape
    out = np.zeros((n_tok, hidden), dtype=np.float32)
    sc = None if expert_scale is None else np.ascontiguousarray(expert_scale, dtype=np.float32)
    lib().ro_moe_combine(_p(experts), _p(np.ascontiguousarray(ids, dtype=np.int32)),
                         _p(np.ascontiguousarray(weights, dtype=np.float32)), _p(sc), _p(out), hidden, n_used, n_tok)
    return out


def grouped_q8(t: int, slab: np.ndarray, bytes_per_expert: int, expert_off: np.ndarray, xq: np.ndarray,
               in_dim: int, out_dim: int):
    n_expert = expert_off.size - 1
    n_entries = int(expert_off[-1])
    y32 = np.zeros((n_entries, out_dim), dtype=np.float32)
    y64 = np.zeros((n_entries, out_dim), dtype=np.float64)
    rc = lib().ro_grouped_q8(t, _p(np.ascontiguousarray(slab)), bytes_per_expert,
                             _p(np.ascontiguousarray(expert_off, dtype=np.int32)), n_expert,
                             _p(np.ascontiguousarray(xq)), in_dim, out_dim, _p(y32), _p(y64))
    assert rc == 0
    return y32, y64


def rel_l2(a: np.ndarray, b: np.ndarray) -> float:
    """||a-b|| / ||b|| in f64 (src/runtime/kernels.rs:1588-1596 of the reference)."""
    a = np.asarray(a, dtype=np.float64).reshape(-1)
    b = np.asarray(b, dtype=np.float64).reshape(-1)
    return float(np.sqrt(np.sum((a - b) ** 2)) / max(np.sqrt(np.sum(b ** 2)), 1e-12))
