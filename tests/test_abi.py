"""The C-ABI library loads without a GPU and exports every symbol the header declares; the
host-only helpers agree with the oracle's layout arithmetic.  No compute call is made here."""
import ctypes as C

import pytest

import oracle as ro
from reinstinct_b200 import _lib


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    declared = _lib.declared_symbols()
    assert len(declared) >= 45
    missing = [s for s in declared if not hasattr(lib, s)]
    assert not missing, missing
    # the Python binding covers the whole header too
    assert sorted(_lib._SIGNATURES) == declared


def test_abi_version_and_error_strings():
    lib = _lib.load()
    assert lib.rc_abi_version() == 1
    assert _lib.error_string(0) == "success"
    for code in range(-8, 0):
        assert "unknown" not in _lib.error_string(code)
    assert "unknown" in _lib.error_string(-99)


@pytest.mark.parametrize("t", ro.ALL_TYPES)
@pytest.mark.parametrize("in_dim,out_dim", [(256, 1), (1024, 3), (2048, 384), (5120, 17408), (16384, 64)])
def test_layout_helpers_agree_with_oracle(t, in_dim, out_dim):
    lib = _lib.load()
    assert lib.rc_repacked_n_sub_padded(in_dim) == ro.nsp(in_dim)
    assert lib.rc_repacked_len(t, in_dim, out_dim) == ro.repacked_len(t, in_dim, out_dim)
    assert lib.rc_ondisk_len(t, in_dim, out_dim) == out_dim * (in_dim // ro.block_weights(t)) * ro.block_bytes(t)


def test_bad_shapes_and_types_are_rejected_before_any_launch():
    lib = _lib.load()
    assert lib.rc_repacked_len(_lib.Q4_K, 96, 4) == 0
    assert lib.rc_repacked_len(99, 256, 4) == 0
    # argument errors are reported before the device is touched
    assert lib.rc_quantize_q8(None, None, None, 33, 1) == -2
    assert lib.rc_matvec(None, 99, None, None, None, 256, 1) == -1
    assert lib.rc_matvec(None, _lib.Q4_K, None, None, None, 100, 1) == -2
    assert lib.rc_matvec(None, _lib.Q4_K, None, None, None, 256, 1) == -3
    assert lib.rc_matvec_batched(None, _lib.Q4_K, 16, 8, 4, 256, 1, 17) == -5
    assert lib.rc_matvec(None, _lib.Q4_K, 8, 8, 4, 256, 1) == -4
    # source-only tensor types relabel onto a kernel type; unsupported ones are refused
    assert lib.rc_kernel_type(11) == 14 and lib.rc_kernel_type(20) == 23 and lib.rc_kernel_type(30) == 8
    assert lib.rc_kernel_type(13) == 13 and lib.rc_kernel_type(10) == -1
    assert lib.rc_ondisk_len(11, 512, 3) == 660 and lib.rc_ondisk_len(30, 512, 3) == 3072 and lib.rc_ondisk_len(20, 384, 3) == 0
    assert lib.rc_repack_for_matvec(None, 10, 16, 256, 1, 16) == -1
    assert lib.rc_repack_for_matvec(None, 11, 16, 384, 1, 16) == -2
    # fused BlockQ8 producers
    assert lib.rc_rmsnorm_q8(None, 4, 4, 8, 48, 1, 1e-6) == -2
    assert lib.rc_rmsnorm_q8(None, None, 4, 8, 64, 1, 1e-6) == -3
    assert lib.rc_rmsnorm_q8(None, 4, 4, 4, 64, 1, 1e-6) == -4
    assert lib.rc_add_rmsnorm_q8(None, None, None, 4, None, 8, 64, 1, 1e-6) == -3
    assert lib.rc_add_rmsnorm_q8(None, None, None, None, None, None, 64, 0, 1e-6) == 0
    assert lib.rc_swiglu_q8(None, 4, 4, None, 8, 33) == -2
    assert lib.rc_swiglu_q8(None, 4, None, None, 8, 64) == -3
    assert lib.rc_swiglu_q8(None, None, None, None, None, 0) == 0
    assert lib.rc_sigmoid_mul_q8(None, 4, 4, 8, 40) == -2
    assert lib.rc_sigmoid_mul_q8(None, None, 4, 8, 64) == -3
    assert lib.rc_rmsnorm_gated_q8(None, 4, 4, 4, None, 8, 2, 2048, 1e-6) == -2
    assert lib.rc_rmsnorm_gated_q8(None, 4, None, 4, None, 8, 2, 128, 1e-6) == -3
    # MoE glue: expert and slot counts beyond what one warp per token holds, odd shapes
    assert lib.rc_moe_topk(None, 4, 1, 2000, 8, 4, 4) == -8
    assert lib.rc_moe_topk(None, 4, 1, 128, 33, 4, 4) == -8
    assert lib.rc_moe_topk(None, 4, 1, 4, 8, 4, 4) == -8
    assert lib.rc_moe_topk(None, None, 1, 128, 8, 4, 4) == -3
    assert lib.rc_moe_topk(None, None, 0, 128, 8, None, None) == 0
    assert lib.rc_moe_act_q8(None, 8, 8, 48, 1, 0) == -2
    assert lib.rc_moe_act_q8(None, 8, 8, 64, 1, 2) == -8
    assert lib.rc_moe_act_q8(None, 8, 4, 64, 1, 0) == -4
    assert lib.rc_moe_act_q8(None, None, None, 64, 0, 0) == 0
    assert lib.rc_moe_combine(None, 4, 4, 4, None, 4, 16, 0, 1) == -8
    assert lib.rc_moe_combine(None, None, 4, 4, None, 4, 16, 2, 1) == -3
    assert lib.rc_moe_gate_up_swiglu(None, _lib.Q4_K, 16, 16, 64, 4, 2, 8, 4, 512, 8, 2, 1, 16, 0) == -2   # in_dim % 1024
    assert lib.rc_moe_gate_up_swiglu(None, _lib.Q4_K, 16, None, 64, 4, 2, 8, 4, 1024, 8, 2, 1, 32, 0) == -3
    assert lib.rc_moe_expert_matvec(None, 99, 16, 64, 4, 2, 8, 4, 256, 8, 2, 1, 1, 0) == -1
    assert lib.rc_moe_expert_matvec(None, _lib.Q4_K, 16, 64, None, 2, 8, 4, 256, 8, 2, 1, 1, 0) == -3
    assert lib.rc_moe_expert_matvec(None, _lib.Q4_K, 16, 60, 4, 2, 8, 4, 256, 8, 2, 1, 1, 0) == -4
    assert lib.rc_moe_expert_matvec(None, _lib.Q4_K, 16, 64, 4, 0, 8, 4, 256, 8, 2, 1, 1, 0) == -8
    assert lib.rc_moe_expert_matvec(None, _lib.Q4_K, None, 64, None, 2, None, None, 256, 8, 2, 0, 1, 0) == 0
    assert lib.rc_matmul_scratch_bytes(5120, 4) == 4 * 160 * 40
