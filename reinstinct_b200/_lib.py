"""ctypes binding of libreinstinct_cuda.so (the C ABI in include/reinstinct_cuda.h).

The library holds the sm_100a kernels.  There is no other implementation behind these
functions: if the library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import re
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libreinstinct_cuda.so"
HEADER = PKG.parent / "include" / "reinstinct_cuda.h"

Q4_0, Q8_0, Q4_K, Q5_K, Q6_K, IQ4_XS = 2, 8, 12, 13, 14, 23
Q5_1 = 7    # MoE expert tensors: the Q5_K kernels with raw fp16 d, m per sub-block (src/quant/q5_1.rs)
IQ3_S = 21  # kernel type only: planes built by the caller (src/quant/iq3_s.rs:216-260), no device repack
ALL_TYPES = (Q4_0, Q8_0, Q4_K, Q5_K, Q6_K, IQ4_XS)
TYPE_NAMES = {Q4_0: "Q4_0", Q8_0: "Q8_0", Q4_K: "Q4_K", Q5_K: "Q5_K", Q6_K: "Q6_K", IQ4_XS: "IQ4_XS", IQ3_S: "IQ3_S", Q5_1: "Q5_1"}
BLOCKQ8_BYTES = 40
MATVEC_MAX_ROWS = 16


class RcError(RuntimeError):
    def __init__(self, code: int, what: str, msg: str):
        super().__init__(f"{what}: {msg} (code {code})")
        self.code = code


_lib = None

_vp, _u32, _sz, _i = C.c_void_p, C.c_uint32, C.c_size_t, C.c_int

_SIGNATURES = {
    "rc_init": (_i, [_i]),
    "rc_abi_version": (_i, []),
    "rc_error_string": (C.c_char_p, [_i]),
    "rc_repacked_n_sub_padded": (_sz, [_sz]),
    "rc_repacked_len": (_sz, [_i, _sz, _sz]),
    "rc_ondisk_len": (_sz, [_i, _sz, _sz]),
    "rc_repack_for_matvec": (_i, [_vp, _i, _vp, _sz, _sz, _vp]),
    "rc_quantize_q8": (_i, [_vp, _vp, _vp, _u32, _u32]),
    "rc_matvec": (_i, [_vp, _i, _vp, _vp, _vp, _u32, _u32]),
    "rc_matvec_batched": (_i, [_vp, _i, _vp, _vp, _vp, _u32, _u32, _u32]),
    "rc_matvec_f32": (_i, [_vp, _i, _vp, _vp, _vp, _u32, _u32, _vp, _sz]),
    "rc_matvec_f32_noalloc": (_i, [_vp, _i, _vp, _vp, _vp, _u32, _u32]),
    "rc_matvec_block_dots": (_i, [_vp, _i, _vp, _vp, _vp, _u32, _u32, _u32]),
    "rc_tune_matvec": (None, [_i, _i, _i]),
    "rc_tune_mmq": (None, [_i, _i]),
    "rc_device_status": (_i, [C.POINTER(C.c_uint)]),
    "rc_device_status_clear": (_i, [C.POINTER(C.c_uint)]),
    "rc_mmq_gemm": (_i, [_vp, _i, _vp, _vp, _vp, _u32, _u32, _u32]),
    "rc_matmul": (_i, [_vp, _i, _vp, _vp, _vp, _u32, _u32, _u32, _vp, _sz]),
    "rc_matmul_scratch_bytes": (_sz, [_u32, _u32]),
    "rc_matmul_f16": (_i, [_vp, _i, _vp, _vp, _vp, _u32, _u32, _u32, _vp, _sz]),
    "rc_matmul_block_dots": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _vp, _sz]),
    "rc_moe_sort": (_i, [_vp, _vp, _u32, _u32, _u32, _vp, _vp, _vp, _vp, _vp]),
    "rc_moe_tile_bn": (_u32, []),
    "rc_moe_gather_xq": (_i, [_vp, _vp, _vp, _vp, _u32, _u32, _u32]),
    "rc_moe_scatter_rows": (_i, [_vp, _vp, _vp, _vp, _u32, _u32]),
    "rc_mmq_gemm_grouped": (_i, [_vp, _i, _vp, _sz, _vp, _vp, _u32, _vp, _vp, _u32, _u32, _u32]),
    "rc_rmsnorm_q8": (_i, [_vp, _vp, _vp, _vp, _u32, _u32, C.c_float]),
    "rc_add_rmsnorm_q8": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, C.c_float]),
    "rc_sigmoid_mul_q8": (_i, [_vp, _vp, _vp, _vp, _sz]),
    "rc_rmsnorm_gated_q8": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, C.c_float]),
    "rc_swiglu_q8": (_i, [_vp, _vp, _vp, _vp, _vp, _sz]),
    "rc_kernel_type": (_i, [_i]),
    "rc_debug_read_trace": (_i, [_vp, C.c_size_t]),
    "rc_debug_read_prof": (_i, [_vp, C.c_size_t]),
    "rc_debug_read_ffn_trace": (_i, [_vp, C.c_size_t]),
    "rc_mmq_gemm_grouped_scratch_bytes": (_sz, [_u32, _u32]),
    "rc_mmq_gemm_grouped_f32": (_i, [_vp, _i, _vp, _sz, _vp, _vp, _u32, _vp, _vp, _u32, _sz, _i, _vp, _u32, _u32, _u32, _vp, _sz]),
    "rc_moe_gate_up_swiglu": (_i, [_vp, _i, _vp, _vp, _sz, _vp, _u32, _vp, _vp, _u32, _u32, _u32, _u32, _u32, _u32]),
    "rc_moe_expert_matvec": (_i, [_vp, _i, _vp, _sz, _vp, _u32, _vp, _vp, _u32, _u32, _u32, _u32, _u32, _u32]),
    "rc_moe_topk": (_i, [_vp, _vp, _u32, _u32, _u32, _vp, _vp]),
    "rc_moe_act_q8": (_i, [_vp, _vp, _vp, _u32, _u32, _i]),
    "rc_moe_combine": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32]),
    "rc_ipc_get_handle": (_i, [_vp, _vp]),
    "rc_ipc_open_handle": (_i, [_vp, C.POINTER(_vp)]),
    "rc_ipc_close_handle": (_i, [_vp]),
    "rc_allgather_push": (_i, [_vp, _vp, _sz, C.POINTER(_vp), C.POINTER(_vp), _vp, _u32, _u32]),
    "rc_ffn_decode_work_bytes": (_sz, [_u32]),
    "rc_ffn_decode": (_i, [_vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32, _u32, _u32, _u32, _u32,
                           C.POINTER(_vp), C.POINTER(_vp), _vp]),
    "rc_peer_barrier": (_i, [_vp, C.POINTER(_vp), _vp, _u32, _u32]),
    "rc_copy_small": (_i, [_vp, _vp, _vp, _sz]),
    "rc_ffn_decode_tp_work_bytes": (_sz, [_u32]),
    "rc_ffn_decode_tp": (_i, [_vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32, C.POINTER(_vp), _vp]),
    "rc_ep_plan": (_i, [_vp, _vp, _u32, _u32, _u32, _u32, _vp]),
    "rc_ep_dispatch": (_i, [_vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32, _u32, _u32, _u32, C.POINTER(_vp), C.POINTER(_vp)]),
    "rc_ep_return": (_i, [_vp, _vp, _vp, _u32, _u32, _u32, _u32, C.POINTER(_vp)]),
    "rc_ep_collect": (_i, [_vp, _vp, _vp, _vp, _u32, _u32]),
    "rc_allgather_push_logical": (_i, [_vp, C.POINTER(_vp), _sz, C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp), _u32]),
    "rc_matmul_gather": (_i, [_vp, _i, _vp, _vp, C.POINTER(_vp), _u32, _u32, _u32, _u32, _u32, _u32, _vp, _sz]),
    "rc_get_device_count": (_i, [C.POINTER(_i)]),
    "rc_set_device": (_i, [_i]),
    "rc_get_device": (_i, [C.POINTER(_i)]),
    "rc_device_get_name": (_i, [C.c_char_p, _i, _i]),
    "rc_device_total_mem": (_i, [C.POINTER(_sz), _i]),
    "rc_mem_get_info": (_i, [C.POINTER(_sz), C.POINTER(_sz)]),
    "rc_device_can_access_peer": (_i, [C.POINTER(_i), _i, _i]),
    "rc_device_enable_peer_access": (_i, [_i]),
    "rc_device_synchronize": (_i, []),
    "rc_malloc": (_i, [C.POINTER(_vp), _sz]),
    "rc_free": (_i, [_vp]),
    "rc_memcpy": (_i, [_vp, _vp, _sz, _i]),
    "rc_memcpy_async": (_i, [_vp, _vp, _sz, _i, _vp]),
    "rc_memcpy_peer_async": (_i, [_vp, _i, _vp, _i, _sz, _vp]),
    "rc_memset_async": (_i, [_vp, _i, _sz, _vp]),
    "rc_stream_create": (_i, [C.POINTER(_vp)]),
    "rc_stream_destroy": (_i, [_vp]),
    "rc_stream_synchronize": (_i, [_vp]),
    "rc_stream_wait_event": (_i, [_vp, _vp]),
    "rc_event_create": (_i, [C.POINTER(_vp)]),
    "rc_event_record": (_i, [_vp, _vp]),
    "rc_event_synchronize": (_i, [_vp]),
    "rc_event_elapsed_time": (_i, [C.POINTER(C.c_float), _vp, _vp]),
    "rc_event_destroy": (_i, [_vp]),
    "rc_stream_begin_capture": (_i, [_vp, _i]),
    "rc_stream_end_capture": (_i, [_vp, C.POINTER(_vp)]),
    "rc_graph_instantiate": (_i, [C.POINTER(_vp), _vp]),
    "rc_graph_launch": (_i, [_vp, _vp]),
    "rc_graph_destroy": (_i, [_vp]),
    "rc_graph_exec_destroy": (_i, [_vp]),
}


def declared_symbols() -> list[str]:
    """Every function name include/reinstinct_cuda.h declares."""
    text = HEADER.read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rc_[a-z0-9_]+)\s*\(", text)))


def load() -> C.CDLL:
    """Loads the library (once) and sets argument types.  Raises if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise FileNotFoundError(
            f"{LIB_PATH} is not built; run `python -m reinstinct_b200.build` (needs nvcc). "
            "There is no CPU implementation to fall back to.")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def error_string(code: int) -> str:
    return load().rc_error_string(code).decode()


def check(code: int, what: str) -> None:
    if code != 0:
        raise RcError(code, what, error_string(code))
