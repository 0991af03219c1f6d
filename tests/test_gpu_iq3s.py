"""GPU parity of the IQ3_S kernel type: the IQ4_XS planes read through the codebook 2n - 15
(src/runtime/qwen35.rs:281-286, src/quant/iq3_s.rs:193-214).  The planes are uploaded as the caller
built them (there is no device repack of the 110-byte blocks); every entry point that takes a
weight type is run once against the oracle."""
import ctypes

import numpy as np
import pytest
import torch

import cases
import oracle as ro

pytestmark = pytest.mark.gpu

T = ro.IQ3_S
F32_TOL = 1e-3      # the reference's GPU-vs-CPU bar (src/runtime/kernels.rs)
DEQ_EXPECTED = 6e-4  # f16-operand GEMM: two f16 roundings


def _status(lib) -> int:
    st = ctypes.c_uint(0)
    assert lib.rc_device_status(ctypes.byref(st)) == 0
    return st.value


def _xq(rt, x):
    n, in_dim = x.shape
    xq = torch.empty(n * (in_dim // 32) * 40, dtype=torch.uint8, device="cuda")
    rt.launch_quantize_q8(torch.from_numpy(x).cuda(), xq, in_dim, n)
    return xq


def test_repack_entry_refuses_iq3s(rt):
    lib = rt._lib.load()
    buf = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    assert lib.rc_repack_for_matvec(0, T, buf.data_ptr(), 256, 1, buf.data_ptr()) == -1  # RC_ERR_BAD_TYPE
    assert lib.rc_kernel_type(T) == T
    assert lib.rc_repacked_len(T, 512, 3) == ro.repacked_len(ro.IQ4_XS, 512, 3)


@pytest.mark.parametrize("in_dim,out_dim,n_rows", [(2048, 384, 1), (256, 37, 1), (5120, 1000, 1), (1024, 301, 2),
                                                   (512, 77, 7), (4096, 640, 16)])
def test_matvec_and_block_integers(rt, in_dim, out_dim, n_rows):
    planes, w = cases.iq3s_planes(in_dim, out_dim, seed=in_dim + n_rows)
    wt = rt.GpuMatvecTensor.from_repacked(planes, T, in_dim, out_dim)
    x = np.random.default_rng(out_dim).standard_normal((n_rows, in_dim)).astype(np.float32)
    xq = _xq(rt, x)
    y = torch.full((n_rows, out_dim), float("nan"), device="cuda")
    if n_rows == 1:
        rt.launch_matvec_xq8(wt, xq, y)
    else:
        rt.launch_matvec_batched(wt, xq, y, n_rows)
    torch.cuda.synchronize()
    _, y64, idots = ro.matvec_q8(T, planes, ro.quantize_q8(x), in_dim, out_dim, n_rows, want_idots=True)
    assert ro.rel_l2(y.cpu().numpy(), y64) < 1e-5
    assert ro.rel_l2(y.cpu().numpy(), x.astype(np.float64) @ w.T) < 2e-2   # int8 activations against the f32 ones
    assert np.array_equal(rt.matvec_block_dots(wt, xq, n_rows).cpu().numpy(), idots)


@pytest.mark.parametrize("in_dim,out_dim,p", [(1024, 300, 200), (256, 128, 17), (2048, 130, 513)])
def test_exact_integer_gemm(rt, in_dim, out_dim, p):
    """rc_mmq_gemm from BlockQ8 activations: the integer dots are exact, so the result matches the
    oracle to f32 summation order."""
    planes, _ = cases.iq3s_planes(in_dim, out_dim, seed=p)
    wt = rt.GpuMatvecTensor.from_repacked(planes, T, in_dim, out_dim)
    x = np.random.default_rng(p).standard_normal((p, in_dim)).astype(np.float32)
    y = torch.full((p, out_dim), float("nan"), device="cuda")
    rt.launch_mmq_gemm(wt, _xq(rt, x), y, p)
    torch.cuda.synchronize()
    assert _status(rt._lib.load()) == 0
    _, y64, _ = ro.matvec_q8(T, planes, ro.quantize_q8(x), in_dim, out_dim, p)
    assert ro.rel_l2(y.cpu().numpy(), y64) < 1e-5


@pytest.mark.parametrize("bn", [0, 128, 256, 512])
@pytest.mark.parametrize("in_dim,out_dim,p", [(1024, 300, 200), (512, 257, 600)])
def test_f16_operand_gemm(rt, bn, in_dim, out_dim, p):
    lib = rt._lib.load()
    planes, _ = cases.iq3s_planes(in_dim, out_dim, seed=bn + p)
    wt = rt.GpuMatvecTensor.from_repacked(planes, T, in_dim, out_dim)
    x = np.random.default_rng(bn + 1).standard_normal((p, in_dim)).astype(np.float32)
    lib.rc_tune_mmq(0, 32 | (bn << 8))
    try:
        y = torch.full((p, out_dim), float("nan"), device="cuda")
        rt.PrefillGemm().matmul_into(y, wt, torch.from_numpy(x).cuda(), p)
        torch.cuda.synchronize()
    finally:
        lib.rc_tune_mmq(0, 0)
    assert _status(lib) == 0
    _, y64, _ = ro.matvec_q8(T, planes, ro.quantize_q8(x), in_dim, out_dim, p)
    assert ro.rel_l2(y.cpu().numpy(), y64) < DEQ_EXPECTED < F32_TOL


def _experts(rt, in_dim, out_dim, n_expert, seed):
    parts = [cases.iq3s_planes(in_dim, out_dim, seed=seed + e)[0] for e in range(n_expert)]
    slab = np.concatenate(parts)
    return parts, slab, rt.GpuExpertTensor.from_repacked(slab, T, in_dim, out_dim, n_expert)


def test_expert_matvec_and_fused_gate_up(rt):
    in_dim, out_dim, n_expert, n_used, n_tok = 1024, 80, 6, 3, 4
    n_sub = in_dim // 32
    rng = np.random.default_rng(5)
    gparts, _, g = _experts(rt, in_dim, out_dim, n_expert, 100)
    uparts, _, u = _experts(rt, in_dim, out_dim, n_expert, 200)
    ids = rng.integers(0, n_expert, (n_tok, n_used)).astype(np.int32)
    ids_d = torch.from_numpy(ids).cuda()
    x = rng.standard_normal((n_tok, in_dim)).astype(np.float32)
    xq = _xq(rt, x)
    yg = torch.full((n_tok, n_used, out_dim), float("nan"), device="cuda")
    rt.launch_moe_expert_matvec(g, ids_d, xq, yg, n_used, n_tok, n_sub, 0)
    fused = torch.full((n_tok, n_used, out_dim), float("nan"), device="cuda")
    rt.launch_moe_gate_up_swiglu(g, u, ids_d, xq, fused, n_used, n_tok, n_sub, 0)
    torch.cuda.synchronize()
    xq_h = ro.quantize_q8(x).reshape(n_tok, -1)
    for tk in range(n_tok):
        for j in range(n_used):
            e = ids[tk, j]
            _, g64, _ = ro.matvec_q8(T, gparts[e], xq_h[tk], in_dim, out_dim, 1)
            _, u64, _ = ro.matvec_q8(T, uparts[e], xq_h[tk], in_dim, out_dim, 1)
            assert ro.rel_l2(yg[tk, j].cpu().numpy(), g64) < 1e-5
            want = g64 / (1.0 + np.exp(-g64)) * u64
            assert ro.rel_l2(fused[tk, j].cpu().numpy(), want) < 2e-5


def test_grouped_gemms(rt):
    """Expert-grouped GEMM, both routes: f32 token rows through the f16-operand kernel, BlockQ8 rows
    through the exact-integer one."""
    in_dim, out_dim, n_expert, n_tok, n_used = 1024, 304, 12, 48, 4
    rng = np.random.default_rng(8)
    n_entries = n_tok * n_used
    ids = rng.integers(0, n_expert - 2, n_entries, dtype=np.int32)
    ids[:70] = 3
    _, slab, et = _experts(rt, in_dim, out_dim, n_expert, 300)
    moe = rt.MoeGroupedScratch.new(n_expert, n_entries)
    rt.launch_moe_sort(moe, torch.from_numpy(ids).cuda(), n_entries)
    torch.cuda.synchronize()
    x = rng.standard_normal((n_tok, in_dim)).astype(np.float32)
    perm = moe.perm.cpu().numpy()[:n_entries]
    xs = x[perm // n_used]
    _, y64 = ro.grouped_q8(T, slab, et.bytes_per_expert, moe.expert_off.cpu().numpy(), ro.quantize_q8(xs), in_dim, out_dim)

    y = torch.full((n_entries, out_dim), float("nan"), device="cuda")
    rt.MoeGroupedGemm().gate_up(moe, et, torch.from_numpy(x).cuda(), n_used, y, n_entries)
    torch.cuda.synchronize()
    assert _status(rt._lib.load()) == 0
    assert ro.rel_l2(y.cpu().numpy(), y64) < DEQ_EXPECTED

    y2 = torch.full((n_entries, out_dim), float("nan"), device="cuda")
    rt.launch_moe_grouped_gemm(moe, et, _xq(rt, xs), y2, in_dim, out_dim, n_entries)
    torch.cuda.synchronize()
    assert _status(rt._lib.load()) == 0
    assert ro.rel_l2(y2.cpu().numpy(), y64) < 1e-5
