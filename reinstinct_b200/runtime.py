"""Host-side mirror of the reference's launch wrappers for the quantized-weight hot path.

Same names, argument meaning and error behaviour as the Rust runtime of the reference
(src/runtime/{gemma4,qwen35,prefill}.rs); every launch goes through the C ABI of
libreinstinct_cuda.so on the current torch CUDA stream.  torch supplies device memory and
streams only.  Errors from the library are raised as `RcError` carrying the code and the
message, like the reference's `Err("<ctx>: <message> (code N)")` (src/hip/mod.rs:19-22).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np
import torch

from . import _lib
from ._lib import ALL_TYPES, BLOCKQ8_BYTES, MATVEC_MAX_ROWS, RcError, check

__all__ = [
    "GpuMatvecTensor", "GpuExpertTensor", "PrefillGemm", "MoeGroupedScratch",
    "launch_quantize_q8", "launch_matvec", "launch_matvec_xq8", "launch_matvec_batched",
    "matvec_block_dots", "launch_mmq_gemm", "launch_moe_sort", "launch_moe_gather_xq",
    "launch_moe_grouped_gemm", "launch_moe_scatter_rows", "repacked_len", "init", "PeerAllGather",
    "PeerBuffers", "GatheredPrefillGemm", "launch_ffn_decode", "FusedFfnDecode", "MoeGroupedGemm", "launch_rmsnorm_q8", "launch_add_rmsnorm_q8", "launch_swiglu_q8",
    "launch_moe_expert_matvec", "launch_moe_gate_up_swiglu", "launch_moe_topk", "launch_moe_act_q8", "launch_moe_combine", "ACT_GEGLU", "ACT_SWIGLU",
]


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t) -> int:
    """Device address of a tensor; a plain int is taken as an address already (buffers that were
    not allocated by torch, e.g. PeerAllGather's)."""
    if t is None:
        return 0
    return t if isinstance(t, int) else t.data_ptr()


def init(device: int | None = None) -> None:
    """Loads the library and prepares `device` (rc_init); call before graph capture."""
    lib = _lib.load()
    dev = torch.cuda.current_device() if device is None else device
    check(lib.rc_init(dev), "rc_init")


def repacked_len(dtype: int, in_dim: int, out_dim: int) -> int:
    """quant::<fmt>::repacked_len (e.g. src/quant/q4_k.rs:98-102)."""
    n = _lib.load().rc_repacked_len(dtype, in_dim, out_dim)
    if n == 0:
        raise ValueError(f"unsupported dtype/shape: {dtype} in_dim={in_dim} out_dim={out_dim}")
    return n


@dataclass
class GpuMatvecTensor:
    """GpuMatvecTensor { data, dtype, in_dim, out_dim, repacked } (src/runtime/qwen35.rs:182-191)."""
    data: torch.Tensor  # uint8, device
    dtype: int
    in_dim: int
    out_dim: int
    repacked: bool = True

    @staticmethod
    def from_bytes_matvec(raw, dtype: int, in_dim: int, out_dim: int,
                          device: torch.device | str = "cuda") -> "GpuMatvecTensor":
        """from_bytes_matvec (src/runtime/qwen35.rs:251-331): on-disk GGUF rows -> repacked-v2
        planes.  The raw blocks are uploaded and repacked on the GPU (rc_repack_for_matvec).  Source-only
        types (Q3_K = 11, IQ4_NL = 20, BF16 = 30) come out tagged with the type they relabel onto
        (src/runtime/qwen35.rs:274-307)."""
        lib = _lib.load()
        ktype = lib.rc_kernel_type(dtype)
        need = lib.rc_ondisk_len(dtype, in_dim, out_dim)
        if need == 0:
            raise ValueError(f"from_bytes_matvec: unsupported dtype {dtype} or in_dim {in_dim}")
        raw_t = torch.as_tensor(np.frombuffer(raw, dtype=np.uint8) if not isinstance(raw, (np.ndarray, torch.Tensor)) else raw)
        raw_t = raw_t.reshape(-1)
        if raw_t.numel() < need:
            raise ValueError(f"from_bytes_matvec: {raw_t.numel()} bytes < {need} needed")
        raw_d = raw_t[:need].to(device, non_blocking=False).contiguous()
        out = torch.empty(repacked_len(ktype, in_dim, out_dim), dtype=torch.uint8, device=device)
        with torch.cuda.device(out.device):
            check(lib.rc_repack_for_matvec(_stream(), dtype, raw_d.data_ptr(), in_dim, out_dim,
                                           out.data_ptr()), "rc_repack_for_matvec")
            torch.cuda.current_stream().synchronize()
        return GpuMatvecTensor(out, ktype, in_dim, out_dim, True)

    @staticmethod
    def from_repacked(planes, dtype: int, in_dim: int, out_dim: int,
                      device: torch.device | str = "cuda") -> "GpuMatvecTensor":
        """Upload planes the caller has already repacked on the host, as the reference does with the
        output of `<fmt>::repack_for_matvec` (`DeviceBuf::from_slice(&p)`, src/runtime/qwen35.rs:309-317).
        The only way in for IQ3_S, whose planes are built by src/quant/iq3_s.rs:216-260."""
        need = repacked_len(dtype, in_dim, out_dim)
        if need == 0:
            raise ValueError(f"from_repacked: unsupported dtype {dtype} or in_dim {in_dim}")
        t = torch.as_tensor(planes).reshape(-1)
        if t.dtype != torch.uint8 or t.numel() < need:
            raise ValueError(f"from_repacked: need {need} uint8 bytes")
        return GpuMatvecTensor(t[:need].to(device).contiguous(), dtype, in_dim, out_dim, True)


@dataclass
class GpuExpertTensor:
    """GpuExpertTensor { data, dtype, in_dim, out_dim, bytes_per_expert, repacked }
    (src/runtime/qwen35.rs:387-436): every expert repacked separately into one slab."""
    data: torch.Tensor
    dtype: int
    in_dim: int
    out_dim: int
    bytes_per_expert: int
    n_expert: int
    repacked: bool = True

    @staticmethod
    def from_bytes(raw, dtype: int, in_dim: int, out_dim: int, n_expert: int,
                   device: torch.device | str = "cuda") -> "GpuExpertTensor":
        lib = _lib.load()
        per_src = lib.rc_ondisk_len(dtype, in_dim, out_dim)
        per_dst = repacked_len(dtype, in_dim, out_dim)
        raw_t = torch.as_tensor(raw).reshape(-1)
        if raw_t.numel() < per_src * n_expert:
            raise ValueError("GpuExpertTensor.from_bytes: raw buffer too small")
        raw_d = raw_t.to(device).contiguous()
        out = torch.empty(per_dst * n_expert, dtype=torch.uint8, device=device)
        with torch.cuda.device(out.device):
            for e in range(n_expert):
                check(lib.rc_repack_for_matvec(_stream(), dtype, raw_d.data_ptr() + e * per_src,
                                               in_dim, out_dim, out.data_ptr() + e * per_dst),
                      "rc_repack_for_matvec")
            torch.cuda.current_stream().synchronize()
        return GpuExpertTensor(out, dtype, in_dim, out_dim, per_dst, n_expert, True)

    @staticmethod
    def from_repacked(slab, dtype: int, in_dim: int, out_dim: int, n_expert: int,
                      device: torch.device | str = "cuda") -> "GpuExpertTensor":
        """Upload a slab of experts already repacked on the host, one after the other."""
        per = repacked_len(dtype, in_dim, out_dim)
        t = torch.as_tensor(slab).reshape(-1)
        if per == 0 or t.dtype != torch.uint8 or t.numel() < per * n_expert:
            raise ValueError("GpuExpertTensor.from_repacked: bad dtype, shape or slab size")
        return GpuExpertTensor(t[:per * n_expert].to(device).contiguous(), dtype, in_dim, out_dim, per, n_expert, True)


def launch_quantize_q8(x: torch.Tensor, out: torch.Tensor, in_dim: int, n_vec: int) -> None:
    """launch_quantize_q8(x, out, in_dim, n_vec) (src/runtime/gemma4.rs:1495-1506)."""
    assert x.dtype == torch.float32 and out.dtype == torch.uint8
    assert x.numel() >= in_dim * n_vec, "launch_quantize_q8: x too short"
    assert out.numel() >= (in_dim // 32) * BLOCKQ8_BYTES * n_vec, "launch_quantize_q8: out too short"
    check(_lib.load().rc_quantize_q8(_stream(), _ptr(x), _ptr(out), in_dim, n_vec), "rc_quantize_q8")


def launch_matvec_xq8(w: GpuMatvecTensor, xq8: torch.Tensor, y: torch.Tensor) -> None:
    """launch_matvec_xq8(w, xq8, y) (src/runtime/gemma4.rs:1526-1564)."""
    assert w.repacked, "launch_matvec_xq8 requires a repacked weight"
    assert isinstance(y, int) or (y.dtype == torch.float32 and y.numel() >= w.out_dim)
    check(_lib.load().rc_matvec(_stream(), w.dtype, _ptr(w.data), _ptr(xq8), _ptr(y), w.in_dim,
                                w.out_dim), "rc_matvec")


def launch_matvec(w: GpuMatvecTensor, x: torch.Tensor, y: torch.Tensor, xq8: torch.Tensor) -> None:
    """launch_matvec(w, x, y) (src/runtime/gemma4.rs:1508-1520): quantize into the engine's
    xq8 scratch, then the matvec."""
    assert w.repacked
    check(_lib.load().rc_matvec_f32(_stream(), w.dtype, _ptr(w.data), _ptr(x), _ptr(y), w.in_dim,
                                    w.out_dim, _ptr(xq8), xq8.numel()), "rc_matvec_f32")


def launch_matvec_batched(w: GpuMatvecTensor, xq8: torch.Tensor, y: torch.Tensor, n_rows: int) -> None:
    """The batched matvec launch of matmul_kquant_batched_into (src/runtime/prefill.rs:448-508)."""
    assert w.repacked
    check(_lib.load().rc_matvec_batched(_stream(), w.dtype, _ptr(w.data), _ptr(xq8), _ptr(y),
                                        w.in_dim, w.out_dim, n_rows), "rc_matvec_batched")


def matvec_block_dots(w: GpuMatvecTensor, xq8: torch.Tensor, n_rows: int) -> torch.Tensor:
    """Per-(activation row, weight row, sub-block) integers, int32 [n_rows][out][n_sub][2]."""
    out = torch.zeros((n_rows, w.out_dim, w.in_dim // 32, 2), dtype=torch.int32, device=w.data.device)
    check(_lib.load().rc_matvec_block_dots(_stream(), w.dtype, _ptr(w.data), _ptr(xq8), _ptr(out),
                                           w.in_dim, w.out_dim, n_rows), "rc_matvec_block_dots")
    return out


def launch_mmq_gemm(w: GpuMatvecTensor, xq8: torch.Tensor, y: torch.Tensor, p_rows: int) -> None:
    """The MMQ launch of matmul_mmq_into (src/runtime/prefill.rs:512-567)."""
    assert w.repacked
    check(_lib.load().rc_mmq_gemm(_stream(), w.dtype, _ptr(w.data), _ptr(xq8), _ptr(y), w.in_dim,
                                  w.out_dim, p_rows), "rc_mmq_gemm")


class PrefillGemm:
    """PrefillGemm (src/runtime/prefill.rs:215-567): Y = X . W^T for any row count, owning the
    int8 activation scratch.  The scratch grows on demand after a stream synchronize, which is
    only legal outside graph capture — pre-size with `max_x` as the reference does."""

    def __init__(self, max_x: int = 32, device: torch.device | str = "cuda"):
        self.device = torch.device(device)
        self.xq8 = torch.empty(max(max_x, 32) // 32 * BLOCKQ8_BYTES, dtype=torch.uint8, device=self.device)

    def _grow(self, n_bytes: int) -> None:
        if self.xq8.numel() < n_bytes:
            torch.cuda.current_stream().synchronize()  # the old buffer may still be in flight
            self.xq8 = torch.empty(n_bytes, dtype=torch.uint8, device=self.device)

    def matmul(self, w: GpuMatvecTensor, x: torch.Tensor, n_rows: int) -> torch.Tensor:
        dst = torch.empty((n_rows, w.out_dim), dtype=torch.float32, device=self.device)
        self.matmul_into(dst, w, x, n_rows)
        return dst

    def matmul_into(self, dst: torch.Tensor, w: GpuMatvecTensor, x: torch.Tensor, n_rows: int) -> None:
        if dst.numel() < n_rows * w.out_dim:
            raise ValueError(f"matmul_into: dst.len={dst.numel()} < n_rows*out_dim={n_rows * w.out_dim}")
        self.matmul_into_raw(dst.data_ptr(), w, x.data_ptr(), n_rows)

    def matmul_into_raw(self, dst_ptr: int, w: GpuMatvecTensor, x_ptr: int, n_rows: int) -> None:
        """matmul_into_raw (src/runtime/prefill.rs:343-437); the caller owns the bounds."""
        assert w.repacked, "only repacked weights are supported (no dequant->fp16 fallback)"
        lib = _lib.load()
        self._grow(lib.rc_matmul_scratch_bytes(w.in_dim, n_rows))
        check(lib.rc_matmul(_stream(), w.dtype, _ptr(w.data), x_ptr, dst_ptr, w.in_dim, w.out_dim,
                            n_rows, _ptr(self.xq8), self.xq8.numel()), "rc_matmul")

    def matmul_f16_into(self, dst: torch.Tensor, w: GpuMatvecTensor, x: torch.Tensor, n_rows: int) -> None:
        """The opt-in APPROXIMATE GEMM (rc_matmul_f16: operands dequantized and rounded once to f16,
        about 3e-4 relative L2 from matmul_into, no per-block integer dots).  No reference counterpart."""
        assert w.repacked
        if dst.numel() < n_rows * w.out_dim:
            raise ValueError(f"matmul_f16_into: dst.len={dst.numel()} < n_rows*out_dim={n_rows * w.out_dim}")
        lib = _lib.load()
        self._grow(lib.rc_matmul_scratch_bytes(w.in_dim, n_rows))
        check(lib.rc_matmul_f16(_stream(), w.dtype, _ptr(w.data), _ptr(x), _ptr(dst), w.in_dim, w.out_dim,
                                n_rows, _ptr(self.xq8), self.xq8.numel()), "rc_matmul_f16")

    def matmul_block_dots(self, w: GpuMatvecTensor, x: torch.Tensor, n_rows: int):
        """Debug: (y, idots) of the tensor-core route; idots int32 [n_rows][out_dim][in_dim / 32] is the tile
        the kernel drains per sub-block, before any f32 scaling (rc_matmul_block_dots)."""
        assert w.repacked
        lib = _lib.load()
        self._grow(lib.rc_matmul_scratch_bytes(w.in_dim, max(n_rows, MATVEC_MAX_ROWS + 1)))
        y = torch.empty((n_rows, w.out_dim), dtype=torch.float32, device=self.device)
        idots = torch.zeros((n_rows, w.out_dim, w.in_dim // 32), dtype=torch.int32, device=self.device)
        check(lib.rc_matmul_block_dots(_stream(), w.dtype, _ptr(w.data), _ptr(x), _ptr(y), _ptr(idots), w.in_dim,
                                       w.out_dim, n_rows, _ptr(self.xq8), self.xq8.numel()), "rc_matmul_block_dots")
        return y, idots

    def matmul_host(self, w: GpuMatvecTensor, x_host: torch.Tensor, y_host: torch.Tensor,
                    x_dev: torch.Tensor, y_dev: torch.Tensor, n_rows: int) -> None:
        """End-to-end call with HOST buffers (pinned): upload x, run, download y, all on the
        current stream; returns after the download is enqueued."""
        x_dev.copy_(x_host, non_blocking=True)
        self.matmul_into(y_dev, w, x_dev, n_rows)
        y_host.copy_(y_dev, non_blocking=True)


@dataclass
class MoeGroupedScratch:
    """MoeGroupedScratch (src/runtime/gemma4.rs:279-288): the sort outputs."""
    count: torch.Tensor
    cursor: torch.Tensor
    expert_off: torch.Tensor
    tile_off: torch.Tensor
    perm: torch.Tensor
    n_expert: int

    @staticmethod
    def new(n_expert: int, max_entries: int, device="cuda") -> "MoeGroupedScratch":
        i32 = dict(dtype=torch.int32, device=device)
        return MoeGroupedScratch(torch.zeros(n_expert, **i32), torch.zeros(n_expert, **i32),
                                 torch.zeros(n_expert + 1, **i32), torch.zeros(n_expert + 1, **i32),
                                 torch.zeros(max(max_entries, 1), **i32), n_expert)


def moe_tile_bn() -> int:
    return int(_lib.load().rc_moe_tile_bn())


def launch_moe_sort(moe: MoeGroupedScratch, ids: torch.Tensor, n_entries: int, bn: int | None = None) -> None:
    """launch_moe_sort (src/runtime/qwen35.rs:2892-2938)."""
    assert ids.dtype == torch.int32
    bn = moe_tile_bn() if bn is None else bn
    check(_lib.load().rc_moe_sort(_stream(), _ptr(ids), n_entries, moe.n_expert, bn, _ptr(moe.count),
                                  _ptr(moe.cursor), _ptr(moe.expert_off), _ptr(moe.tile_off),
                                  _ptr(moe.perm)), "rc_moe_sort")


def launch_moe_gather_xq(moe: MoeGroupedScratch, xq_src: torch.Tensor, xq_dst: torch.Tensor,
                         n_sub: int, n_used: int, n_entries: int) -> None:
    """launch_moe_gather_xq (src/runtime/qwen35.rs:2999-3013)."""
    check(_lib.load().rc_moe_gather_xq(_stream(), _ptr(xq_src), _ptr(moe.perm), _ptr(xq_dst), n_sub,
                                       n_used, n_entries), "rc_moe_gather_xq")


def launch_moe_scatter_rows(moe: MoeGroupedScratch, src: torch.Tensor, dst: torch.Tensor, dim: int,
                            n_entries: int) -> None:
    """launch_moe_scatter_rows (src/runtime/qwen35.rs:3016-3030)."""
    check(_lib.load().rc_moe_scatter_rows(_stream(), _ptr(src), _ptr(moe.perm), _ptr(dst), dim,
                                          n_entries), "rc_moe_scatter_rows")


def launch_moe_grouped_gemm(moe: MoeGroupedScratch, et: GpuExpertTensor, xq: torch.Tensor,
                            y: torch.Tensor, in_dim: int, out_dim: int, n_entries: int) -> None:
    """launch_moe_grouped_gemm (src/runtime/qwen35.rs:3036-3064)."""
    check(_lib.load().rc_mmq_gemm_grouped(_stream(), et.dtype, _ptr(et.data), et.bytes_per_expert,
                                          _ptr(moe.expert_off), _ptr(moe.tile_off), moe.n_expert,
                                          _ptr(xq), _ptr(y), in_dim, out_dim, n_entries),
          "rc_mmq_gemm_grouped")


class MoeGroupedGemm:
    """The grouped GEMM from f32 activations (rc_mmq_gemm_grouped_f32), owning its scratch like
    PrefillGemm owns its own.  `gate_up` gathers token rows through the sort's perm; `down` applies
    the gated activation to the gate_up output on the fly."""

    def __init__(self, device: torch.device | str = "cuda"):
        self.device = torch.device(device)
        self.scratch = torch.empty(16, dtype=torch.uint8, device=self.device)

    def _grow(self, n_bytes: int) -> None:
        if self.scratch.numel() < n_bytes:
            torch.cuda.current_stream().synchronize()
            self.scratch = torch.empty(n_bytes, dtype=torch.uint8, device=self.device)

    def _run(self, moe: "MoeGroupedScratch", et: GpuExpertTensor, x, index, div, row_stride, act, y, n_entries) -> None:
        lib = _lib.load()
        self._grow(lib.rc_mmq_gemm_grouped_scratch_bytes(et.in_dim, n_entries))
        check(lib.rc_mmq_gemm_grouped_f32(_stream(), et.dtype, _ptr(et.data), et.bytes_per_expert, _ptr(moe.expert_off),
                                          _ptr(moe.tile_off), moe.n_expert, _ptr(x), _ptr(index), div, row_stride, act,
                                          _ptr(y), et.in_dim, et.out_dim, n_entries, _ptr(self.scratch), self.scratch.numel()),
              "rc_mmq_gemm_grouped_f32")

    def gate_up(self, moe, et: GpuExpertTensor, x_tokens: torch.Tensor, n_used: int, y_sorted: torch.Tensor, n_entries: int) -> None:
        self._run(moe, et, x_tokens, moe.perm, n_used, et.in_dim, -1, y_sorted, n_entries)

    def down(self, moe, et: GpuExpertTensor, gate_up_sorted: torch.Tensor, act: int, y_sorted: torch.Tensor, n_entries: int) -> None:
        self._run(moe, et, gate_up_sorted, None, 1, 2 * et.in_dim, act, y_sorted, n_entries)


def launch_rmsnorm_q8(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, n: int, n_vec: int, eps: float) -> None:
    """launch_rmsnorm_q8 (kernels/rmsnorm_q8.cpp:38-103)."""
    check(_lib.load().rc_rmsnorm_q8(_stream(), _ptr(x), _ptr(w), _ptr(out), n, n_vec, eps), "rc_rmsnorm_q8")


def launch_add_rmsnorm_q8(hidden: torch.Tensor, add, w: torch.Tensor, y, out: torch.Tensor, n: int, n_vec: int,
                          eps: float) -> None:
    """launch_add_rmsnorm_q8 (kernels/qwen35_fused.cpp:66-118); add and y may be None."""
    check(_lib.load().rc_add_rmsnorm_q8(_stream(), _ptr(hidden), _ptr(add), _ptr(w), _ptr(y), _ptr(out), n, n_vec, eps),
          "rc_add_rmsnorm_q8")


def launch_swiglu_q8(gate: torch.Tensor, up: torch.Tensor, out, q8: torch.Tensor, n: int) -> None:
    """launch_swiglu_q8 (kernels/qwen35_fused.cpp:123-138); out may be None."""
    check(_lib.load().rc_swiglu_q8(_stream(), _ptr(gate), _ptr(up), _ptr(out), _ptr(q8), n), "rc_swiglu_q8")


def launch_sigmoid_mul_q8(x: torch.Tensor, gate: torch.Tensor, q8: torch.Tensor, n: int) -> None:
    """sigmoid_mul_q8_f32 (kernels/qwen35_fused.cpp:139-152); x is updated in place."""
    check(_lib.load().rc_sigmoid_mul_q8(_stream(), _ptr(x), _ptr(gate), _ptr(q8), n), "rc_sigmoid_mul_q8")


def launch_rmsnorm_gated_q8(x: torch.Tensor, z: torch.Tensor, w: torch.Tensor, y, q8: torch.Tensor, n_heads: int,
                            head_dim: int, eps: float) -> None:
    """rmsnorm_gated_q8_f32 (kernels/qwen35_fused.cpp:204-224); y may be None."""
    check(_lib.load().rc_rmsnorm_gated_q8(_stream(), _ptr(x), _ptr(z), _ptr(w), _ptr(y), _ptr(q8), n_heads, head_dim, eps),
          "rc_rmsnorm_gated_q8")


def launch_moe_expert_matvec(et: GpuExpertTensor, ids: torch.Tensor, xq8: torch.Tensor, y: torch.Tensor, n_used: int,
                             n_tok: int, xq_tok_stride: int, xq_slot_stride: int) -> None:
    """launch_moe_expert_matvec / launch_moe_down (src/runtime/qwen35.rs:3066-3139): decode-side
    routed-expert matvec, y [n_tok, n_used, out_dim]."""
    assert ids.dtype == torch.int32
    check(_lib.load().rc_moe_expert_matvec(_stream(), et.dtype, _ptr(et.data), et.bytes_per_expert, _ptr(ids), et.n_expert,
                                           _ptr(xq8), _ptr(y), et.in_dim, et.out_dim, n_used, n_tok, xq_tok_stride,
                                           xq_slot_stride), "rc_moe_expert_matvec")


def launch_moe_gate_up_swiglu(gate: GpuExpertTensor, up: GpuExpertTensor, ids: torch.Tensor, xq8: torch.Tensor,
                              y: torch.Tensor, n_used: int, n_tok: int, xq_tok_stride: int, xq_slot_stride: int) -> None:
    """launch_moe_gate_up_swiglu (src/runtime/qwen35.rs:3141-3167): y [n_tok, n_used, out_dim] = silu(gate) * up."""
    assert gate.dtype == up.dtype and gate.bytes_per_expert == up.bytes_per_expert and ids.dtype == torch.int32
    check(_lib.load().rc_moe_gate_up_swiglu(_stream(), gate.dtype, _ptr(gate.data), _ptr(up.data), gate.bytes_per_expert,
                                            _ptr(ids), gate.n_expert, _ptr(xq8), _ptr(y), gate.in_dim, gate.out_dim, n_used,
                                            n_tok, xq_tok_stride, xq_slot_stride), "rc_moe_gate_up_swiglu")


ACT_GEGLU, ACT_SWIGLU = 0, 1


def launch_moe_topk(logits: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, n_expert: int, n_used: int,
                    n_tok: int) -> None:
    """launch_moe_topk (src/runtime/gemma4.rs:1649-1670)."""
    assert logits.dtype == torch.float32 and ids.dtype == torch.int32 and weights.dtype == torch.float32
    check(_lib.load().rc_moe_topk(_stream(), _ptr(logits), n_tok, n_expert, n_used, _ptr(ids), _ptr(weights)),
          "rc_moe_topk")


def launch_moe_act_q8(gu: torch.Tensor, out: torch.Tensor, ff: int, n_slot: int, act: int = ACT_GEGLU) -> None:
    """launch_moe_geglu_q8 (src/runtime/gemma4.rs:1784-1800); act selects GeGLU or SwiGLU."""
    check(_lib.load().rc_moe_act_q8(_stream(), _ptr(gu), _ptr(out), ff, n_slot, act), "rc_moe_act_q8")


def launch_moe_combine(experts: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, expert_scale,
                       out: torch.Tensor, hidden: int, n_used: int, n_tok: int) -> None:
    """launch_moe_combine (src/runtime/gemma4.rs:1804-1823)."""
    check(_lib.load().rc_moe_combine(_stream(), _ptr(experts), _ptr(ids), _ptr(weights), _ptr(expert_scale),
                                     _ptr(out), hidden, n_used, n_tok), "rc_moe_combine")


def launch_ffn_decode(gate: GpuMatvecTensor, up: GpuMatvecTensor, down: GpuMatvecTensor, x, xq8: torch.Tensor,
                      y_gate: torch.Tensor, y_up: torch.Tensor, hq8: torch.Tensor, y) -> None:
    """step_swiglu_ffn (src/runtime/qwen35.rs:2694-2707): quantize x -> gate and up matvecs on the shared
    BlockQ8 -> SwiGLU + quantize in one launch -> down matvec; five launches on the current stream.  x and y
    may be PINNED HOST tensors: pinned memory is addressable from the device, so the first kernel reads the
    20 KB input and the last one writes the output across PCIe themselves and the step has no copy launches."""
    launch_quantize_q8(x, xq8, gate.in_dim, 1)
    launch_matvec_xq8(gate, xq8, y_gate)
    launch_matvec_xq8(up, xq8, y_up)
    launch_swiglu_q8(y_gate, y_up, None, hq8, gate.out_dim)
    launch_matvec_xq8(down, hq8, y)


class PeerBuffers:
    """`n_buffers` equal device buffers per rank plus the handshake words, allocated with rc_malloc and mapped
    into every rank of the group with CUDA IPC (one process per GPU on one box).  ptrs[k] is a ctypes array of
    every rank's k-th buffer (own one included), as the gather entry points take them."""

    def __init__(self, bytes_per_buffer: int, n_buffers: int = 2, group=None):
        import torch.distributed as dist

        lib = _lib.load()
        self.lib, self.bytes, self.n_buffers, self.group = lib, bytes_per_buffer, n_buffers, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self._stride = (bytes_per_buffer + 255) // 256 * 256
        data = self._stride * n_buffers
        flags = (self.world * 8 + 255) // 256 * 256
        base = C.c_void_p()
        check(lib.rc_malloc(C.byref(base), data + flags + 256), "rc_malloc")
        self._base = base.value
        check(lib.rc_memset_async(self._base, 0, data + flags + 256, _stream()), "rc_memset_async")
        torch.cuda.current_stream().synchronize()
        handle = (C.c_ubyte * 64)()
        check(lib.rc_ipc_get_handle(self._base, handle), "rc_ipc_get_handle")
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle), group=group)  # also orders the memset before any peer store
        self._opened = []
        bases = []
        for r, h in enumerate(handles):
            if r == self.rank:
                bases.append(self._base)
                continue
            p = C.c_void_p()
            hb = (C.c_ubyte * 64).from_buffer_copy(h)
            check(lib.rc_ipc_open_handle(hb, C.byref(p)), "rc_ipc_open_handle")
            self._opened.append(p.value)
            bases.append(p.value)
        self.ptrs = [(C.c_void_p * self.world)(*[b + k * self._stride for b in bases]) for k in range(n_buffers)]
        self.own = [self._base + k * self._stride for k in range(n_buffers)]
        self.flags = (C.c_void_p * self.world)(*[b + data for b in bases])
        self.epoch = self._base + data + flags
        dist.barrier(group=group)

    def barrier(self) -> None:
        """rc_peer_barrier on the current stream: returns once every rank's barrier of this call has run, i.e.
        once every store a peer issued before its barrier has landed here."""
        check(self.lib.rc_peer_barrier(_stream(), self.flags, self.epoch, self.rank, self.world), "rc_peer_barrier")

    def read(self, k: int, dst: torch.Tensor, n_bytes: int | None = None) -> None:
        """This rank's k-th buffer -> a torch tensor (device or pinned host), on the current stream."""
        kind = 3 if dst.is_cuda else 2
        check(self.lib.rc_memcpy_async(dst.data_ptr(), self.own[k], self.bytes if n_bytes is None else n_bytes, kind, _stream()),
              "rc_memcpy_async")

    def close(self) -> None:
        import torch.distributed as dist

        torch.cuda.current_stream().synchronize()
        dist.barrier(group=self.group)  # nobody unmaps while a peer may still store
        for p in self._opened:
            self.lib.rc_ipc_close_handle(p)
        self._opened = []
        if self._base:
            self.lib.rc_free(self._base)
            self._base = 0


def copy_small(dst, src, n_bytes: int) -> None:
    """rc_copy_small on the current stream: a few KB between pinned host and device memory (either way) by a kernel;
    in a replayed graph a memcpy node of that size costs three times as much."""
    check(_lib.load().rc_copy_small(_stream(), _ptr(dst), _ptr(src), n_bytes), "rc_copy_small")


class FusedFfnDecode:
    """step_swiglu_ffn (src/runtime/qwen35.rs:2694-2707) as ONE cooperative launch per GPU (rc_ffn_decode), row-sharded
    over the ranks of `group` (or a single GPU when torch.distributed is not initialised): this rank's `gate` and `up`
    hold rows [ffn_begin, ffn_begin + gate.out_dim) of the [ffn_total, in_dim] projections, `down` rows
    [out_begin, out_begin + down.out_dim) of [out_total, ffn_total].  After run(x) — on the stream — `self.y` (or the
    tensor given to run) holds all out_total outputs.  The exchange buffers and the work area belong to this object
    (one per layer shape); every rank makes the same sequence of run() calls."""

    def __init__(self, gate: GpuMatvecTensor, up: GpuMatvecTensor, down: GpuMatvecTensor, ffn_total: int, out_total: int,
                 ffn_begin: int = 0, out_begin: int = 0, group=None, device="cuda"):
        import torch.distributed as dist

        lib = _lib.load()
        self.lib, self.gate, self.up, self.down, self.group = lib, gate, up, down, group
        self.ffn_total, self.out_total, self.ffn_begin, self.out_begin = ffn_total, out_total, ffn_begin, out_begin
        h_bytes = (3 * ffn_total * 4 + 255) // 256 * 256
        total = h_bytes + (3 * out_total * 4 + 255) // 256 * 256
        self._h_off, self._y_off = 0, h_bytes
        multi = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
        if multi:
            self.peers = PeerBuffers(total, 1, group)
            self.rank, self.world = self.peers.rank, self.peers.world
            bases = [self.peers.ptrs[0][r] for r in range(self.world)]
            self._local = None
        else:
            self.peers, self.rank, self.world = None, 0, 1
            self._local = torch.empty(total, dtype=torch.uint8, device=device)
            bases = [self._local.data_ptr()]
        own = bases[self.rank]
        check(lib.rc_memset_async(own, 0xFF, total, _stream()), "rc_memset_async")  # "not arrived" everywhere
        torch.cuda.current_stream().synchronize()
        if multi:
            dist.barrier(group=group)  # no peer stores before every rank's fill is done
        self._h = (C.c_void_p * self.world)(*[b + self._h_off for b in bases])
        self._yp = (C.c_void_p * self.world)(*[b + self._y_off for b in bases])
        self._own_h = own + self._h_off
        self.y = torch.empty(out_total, dtype=torch.float32, device=device)
        self.work = torch.zeros(lib.rc_ffn_decode_work_bytes(gate.out_dim), dtype=torch.uint8, device=device)
        self.calls = 0

    def run(self, x, y=None) -> None:
        """x: f32 [in_dim] on the device or in pinned host memory.  y: where the finished output goes instead of self.y
        (a device tensor or a pinned host tensor: the last phase then writes across PCIe itself)."""
        g, d = self.gate, self.down
        out = self.y if y is None else y
        check(self.lib.rc_ffn_decode(_stream(), g.dtype, d.dtype, _ptr(g.data), _ptr(self.up.data), _ptr(d.data), _ptr(x), _ptr(out),
                                     g.in_dim, g.out_dim, self.ffn_total, self.ffn_begin, d.out_dim, self.out_total, self.out_begin,
                                     self.world, self.rank, self._h, self._yp, _ptr(self.work)), "rc_ffn_decode")
        self.calls += 1

    def read_y(self, dst: torch.Tensor) -> None:
        dst.copy_(self.y.reshape(dst.shape), non_blocking=True)

    def read_h(self, dst: torch.Tensor) -> None:
        """The f32 intermediate silu(gate) * up of the last run() (all ffn_total values), on the current stream."""
        kind = 3 if dst.is_cuda else 2
        src = self._own_h + (self.calls % 3) * self.ffn_total * 4
        check(self.lib.rc_memcpy_async(dst.data_ptr(), src, self.ffn_total * 4, kind, _stream()), "rc_memcpy_async")

    def close(self) -> None:
        if self.peers is not None:
            self.peers.close()


class TensorParallelFfnDecode:
    """step_swiglu_ffn (src/runtime/qwen35.rs:2694-2707) as ONE cooperative launch per GPU with the usual tensor-parallel
    split (rc_ffn_decode_tp): this rank's `gate` and `up` hold rows [b, b + n) of the [ffn_total, in_dim] projections and
    `down` the matching COLUMNS of the down projection as a tensor [out_total, n] of its own (sharding.shard_raw_cols).
    The intermediate stays on the rank; the ranks' partial outputs are summed in rank order.  After run(x) — on the
    stream — `self.y` (or the tensor given to run) holds all out_total outputs.  The exchange buffer and the work area
    belong to this object; every rank makes the same sequence of run() calls."""

    def __init__(self, gate: GpuMatvecTensor, up: GpuMatvecTensor, down: GpuMatvecTensor, group=None, device="cuda"):
        import torch.distributed as dist

        lib = _lib.load()
        assert down.in_dim == gate.out_dim == up.out_dim, "down must hold the columns that match this rank's gate/up rows"
        self.lib, self.gate, self.up, self.down, self.group = lib, gate, up, down, group
        self.out_total = down.out_dim
        multi = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
        world = dist.get_world_size(group) if multi else 1
        total = (3 * world * self.out_total * 4 + 255) // 256 * 256
        if multi:
            self.peers = PeerBuffers(total, 1, group)
            self.rank, self.world = self.peers.rank, self.peers.world
            bases = [self.peers.ptrs[0][r] for r in range(self.world)]
            self._local = None
        else:
            self.peers, self.rank, self.world = None, 0, 1
            self._local = torch.empty(total, dtype=torch.uint8, device=device)
            bases = [self._local.data_ptr()]
        check(lib.rc_memset_async(bases[self.rank], 0xFF, total, _stream()), "rc_memset_async")  # "not arrived" everywhere
        torch.cuda.current_stream().synchronize()
        if multi:
            dist.barrier(group=group)  # no peer stores before every rank's fill is done
        self._part = (C.c_void_p * self.world)(*bases)
        self.y = torch.empty(self.out_total, dtype=torch.float32, device=device)
        self.work = torch.zeros(lib.rc_ffn_decode_tp_work_bytes(gate.out_dim), dtype=torch.uint8, device=device)

    def run(self, x, y=None) -> None:
        """x: f32 [in_dim] on the device or in pinned host memory; y: where the output goes instead of self.y."""
        g, d = self.gate, self.down
        out = self.y if y is None else y
        check(self.lib.rc_ffn_decode_tp(_stream(), g.dtype, d.dtype, _ptr(g.data), _ptr(self.up.data), _ptr(d.data), _ptr(x), _ptr(out),
                                        g.in_dim, g.out_dim, self.out_total, self.world, self.rank, self._part, _ptr(self.work)),
              "rc_ffn_decode_tp")

    def read_y(self, dst: torch.Tensor) -> None:
        dst.copy_(self.y.reshape(dst.shape), non_blocking=True)

    def close(self) -> None:
        if self.peers is not None:
            self.peers.close()


class ExpertParallel:
    """Expert parallelism without the host (rc_ep_plan / rc_ep_dispatch / rc_ep_return / rc_ep_collect around the
    reference's own sort, gather, grouped GEMM and scatter launches, src/runtime/qwen35.rs:2892-3064): this rank owns
    the `experts.n_expert` experts [rank * n, (rank + 1) * n) of the layer, routes its own tokens, sends each routed
    BlockQ8 row to the owner of its expert by stores into peer memory and gets the result rows back the same way.
    `cap` >= the entries one rank routes per step (tokens x n_used).  step() is a fixed sequence of launches on the
    current stream (two peer barriers inside, no host involvement); the receive buffers alternate, so a captured graph
    must hold an even number of steps.  Without an initialised process group it runs as a world of one.
    With `down` (the owner's down-projection experts, [out_dim / 2 -> down.out_dim]) the owner runs the whole expert FFN
    on what it received — gate_up GEMM, gated activation + quantize, down GEMM (the sequence of the reference's MoE
    prefill, src/runtime/qwen35.rs:3036-3064 around moe_geglu_q8 / swiglu) — and rows of down.out_dim come back."""

    def __init__(self, experts: "GpuExpertTensor", in_dim: int, out_dim: int, cap: int, group=None, device="cuda",
                 down: "GpuExpertTensor | None" = None, act: int = ACT_SWIGLU):
        import torch.distributed as dist

        lib = _lib.load()
        self.lib, self.experts, self.in_dim, self.cap, self.group = lib, experts, in_dim, cap, group
        self.down, self.act, self.mid_dim = down, act, out_dim
        out_dim = down.out_dim if down is not None else out_dim
        self.out_dim = out_dim
        multi = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
        self.world = dist.get_world_size(group) if multi else 1
        self.rank = dist.get_rank(group) if multi else 0
        self.slots = self.world * cap
        self.row_bytes = in_dim // 32 * BLOCKQ8_BYTES
        al = lambda n: (n + 255) // 256 * 256
        rows_b, ids_b, ret_b = al(2 * self.slots * self.row_bytes), al(2 * self.slots * 4), al(self.slots * out_dim * 4)
        total = rows_b + ids_b + ret_b
        if multi:
            self.peers = PeerBuffers(total, 1, group)
            bases = [self.peers.ptrs[0][r] for r in range(self.world)]
            self._local = None
        else:
            self.peers = None
            self._local = torch.empty(total, dtype=torch.uint8, device=device)
            bases = [self._local.data_ptr()]
        own = bases[self.rank]
        check(lib.rc_memset_async(own + rows_b, 0xFF, ids_b, _stream()), "rc_memset_async")  # every slot unused
        torch.cuda.current_stream().synchronize()
        if multi:
            dist.barrier(group=group)
        arr = lambda off: (C.c_void_p * self.world)(*[b + off for b in bases])
        self._rows, self._ids, self._ret = arr(0), arr(rows_b), arr(rows_b + ids_b)
        self._own_rows, self._own_ids, self._own_ret = own, own + rows_b, own + rows_b + ids_b
        self.moe = MoeGroupedScratch.new(experts.n_expert, self.slots, device=device)
        self.xg = torch.empty(self.slots * self.row_bytes, dtype=torch.uint8, device=device)
        self.y_sorted = torch.empty(self.slots, self.mid_dim, dtype=torch.float32, device=device)
        if down is not None:
            self.hq = torch.empty(self.slots * (self.mid_dim // 2 // 32) * BLOCKQ8_BYTES, dtype=torch.uint8, device=device)
            self.y2_sorted = torch.empty(self.slots, out_dim, dtype=torch.float32, device=device)
        self.y_in = torch.empty(self.slots, out_dim, dtype=torch.float32, device=device)
        self.back = torch.empty(cap, dtype=torch.int32, device=device)
        self.buf = 0

    def step(self, ids: torch.Tensor, xq: torch.Tensor, n_entries: int, n_used: int, out: torch.Tensor) -> None:
        """ids: int32 [n_entries] global expert ids (entry e belongs to token e // n_used); xq: the tokens' BlockQ8 rows;
        out: f32 [n_entries, out_dim], entry order."""
        assert ids.dtype == torch.int32 and n_entries <= self.cap
        lib, st, b = self.lib, _stream(), self.buf
        n_local = self.experts.n_expert
        check(lib.rc_ep_plan(st, _ptr(ids), n_entries, n_local, self.cap, self.world, _ptr(self.back)), "rc_ep_plan")
        check(lib.rc_ep_dispatch(st, _ptr(ids), _ptr(self.back), _ptr(xq), n_entries, n_used, self.in_dim, n_local, self.cap,
                                 self.rank, self.world, b, self._rows, self._ids), "rc_ep_dispatch")
        if self.peers is not None:
            self.peers.barrier()
        ids_in = self._own_ids + b * self.slots * 4
        rows_in = self._own_rows + b * self.slots * self.row_bytes
        moe = self.moe
        check(lib.rc_moe_sort(st, ids_in, self.slots, n_local, moe_tile_bn(), _ptr(moe.count), _ptr(moe.cursor), _ptr(moe.expert_off),
                              _ptr(moe.tile_off), _ptr(moe.perm)), "rc_moe_sort")
        check(lib.rc_moe_gather_xq(st, rows_in, _ptr(moe.perm), _ptr(self.xg), self.in_dim // 32, 1, self.slots), "rc_moe_gather_xq")
        launch_moe_grouped_gemm(moe, self.experts, self.xg, self.y_sorted, self.in_dim, self.mid_dim, self.slots)
        if self.down is not None:
            ff = self.mid_dim // 2
            launch_moe_act_q8(self.y_sorted, self.hq, ff, self.slots, self.act)
            launch_moe_grouped_gemm(moe, self.down, self.hq, self.y2_sorted, ff, self.out_dim, self.slots)
            launch_moe_scatter_rows(moe, self.y2_sorted, self.y_in, self.out_dim, self.slots)
        else:
            launch_moe_scatter_rows(moe, self.y_sorted, self.y_in, self.out_dim, self.slots)
        check(lib.rc_ep_return(st, ids_in, _ptr(self.y_in), self.out_dim, self.cap, self.rank, self.world, self._ret), "rc_ep_return")
        if self.peers is not None:
            self.peers.barrier()
        check(lib.rc_ep_collect(st, _ptr(self.back), self._own_ret, _ptr(out), self.out_dim, n_entries), "rc_ep_collect")
        self.buf ^= 1

    def close(self) -> None:
        if self.peers is not None:
            self.peers.close()


class PeerAllGather:
    """All-gather of one small shard per rank by direct stores into the peers' memory
    (rc_allgather_push).  A call returns, on the stream, once every rank's shard of this call has arrived in
    the gathered buffer at `buffer_ptr` (`world * bytes_per_rank` bytes, rank r's shard at offset
    r * bytes_per_rank).  Consecutive calls ALTERNATE between two gathered buffers, so a fast rank's next
    push can never land under a slower rank's consumer of the previous call; read `buffer_ptr` after each
    call.  Safe to capture in a CUDA graph if the graph holds an even number of calls per object (a replay
    then starts on the same buffer as the capture did)."""

    def __init__(self, bytes_per_rank: int, group=None):
        assert bytes_per_rank % 16 == 0, "shards are copied in 16-byte units"
        self.bytes = bytes_per_rank
        self.peers = PeerBuffers(bytes_per_rank * _world(group), 2, group)
        self.rank, self.world = self.peers.rank, self.peers.world
        self.calls = 0
        self.buffer_ptr = self.peers.own[0]

    def gather(self, src) -> None:
        k = self.calls & 1
        p = self.peers
        check(p.lib.rc_allgather_push(_stream(), _ptr(src), self.bytes, p.ptrs[k], p.flags, p.epoch, self.rank, self.world),
              "rc_allgather_push")
        self.buffer_ptr = p.own[k]
        self.calls += 1

    def copy_out(self, dst: torch.Tensor) -> None:
        """The buffer of the latest call -> a torch tensor (device or pinned host), on the current stream."""
        self.peers.read((self.calls - 1) & 1 if self.calls else 0, dst, self.world * self.bytes)

    def close(self) -> None:
        self.peers.close()


def _world(group) -> int:
    import torch.distributed as dist

    return dist.get_world_size(group)


class GatheredPrefillGemm:
    """Row-sharded PrefillGemm whose kernel gathers its own output (rc_matmul_gather + rc_peer_barrier): every
    rank holds rows [row_begin, row_begin + w.out_dim) of an [out_total, in_dim] matrix, and after a call every
    rank's output buffer holds the whole [n_rows][out_total] f32 product, bit-identical to the unsharded
    rc_matmul.  Two output buffers alternate between calls (see PeerAllGather)."""

    def __init__(self, max_rows: int, out_total: int, in_dim: int, group=None, device="cuda"):
        self.out_total, self.max_rows = out_total, max_rows
        self.peers = PeerBuffers(max_rows * out_total * 4, 2, group)
        lib = _lib.load()
        self.scratch = torch.empty(lib.rc_matmul_scratch_bytes(in_dim, max(max_rows, MATVEC_MAX_ROWS + 1)), dtype=torch.uint8,
                                   device=device)
        self.calls = 0

    def matmul(self, w: GpuMatvecTensor, x: torch.Tensor, n_rows: int, row_begin: int, barrier: bool = True) -> int:
        """Returns the index of the output buffer this call fills."""
        assert w.repacked and n_rows <= self.max_rows
        k = self.calls & 1
        p = self.peers
        check(p.lib.rc_matmul_gather(_stream(), w.dtype, _ptr(w.data), _ptr(x), p.ptrs[k], p.world, self.out_total, row_begin,
                                     w.in_dim, w.out_dim, n_rows, _ptr(self.scratch), self.scratch.numel()), "rc_matmul_gather")
        if barrier:
            p.barrier()
        self.calls += 1
        return k

    def read(self, k: int, dst: torch.Tensor, n_rows: int) -> None:
        self.peers.read(k, dst, n_rows * self.out_total * 4)

    def close(self) -> None:
        self.peers.close()
