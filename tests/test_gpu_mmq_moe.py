"""GPU parity of the int8 MMQ GEMM (dense and expert-grouped), the expert sort and the
gather / scatter kernels, through the C ABI."""
import numpy as np
import pytest
import torch

import cases
import oracle as ro

pytestmark = pytest.mark.gpu

F32_TOL = 1e-3
DP4A_REL_L2_MAX = 1.5e-2


def quantize(rt, x: np.ndarray):
    n, in_dim = x.shape
    xq = torch.empty(n * (in_dim // 32) * 40, dtype=torch.uint8, device="cuda")
    rt.launch_quantize_q8(torch.from_numpy(x).cuda(), xq, in_dim, n)
    return xq


@pytest.mark.parametrize("t,seed", [(ro.Q4_K, 0x94940001), (ro.Q5_K, 0x95950001), (ro.Q6_K, 0x96960001)])
def test_mmq_reference_case_p70(rt, t, seed):
    """mmq_gemm_q4k_repacked_matches_matvec (src/runtime/kernels.rs:3171-3220): P=70 (not a
    tile multiple), out 384, in 2048, against per-row dequant + f32 matvec."""
    in_dim, out_dim, p = 2048, 384, 70
    raw = cases.lcg_case(t, in_dim, out_dim, seed)
    x = cases.lcg_x(p * in_dim, 0x2468ACE0).reshape(p, in_dim)
    w = rt.GpuMatvecTensor.from_bytes_matvec(raw, t, in_dim, out_dim)
    xq = quantize(rt, x)
    y = torch.full((p, out_dim), float("nan"), device="cuda")
    rt.launch_mmq_gemm(w, xq, y, p)
    torch.cuda.synchronize()
    got = y.cpu().numpy()
    _, y64, _ = ro.matvec_q8(t, ro.repack(t, raw, in_dim, out_dim), ro.quantize_q8(x), in_dim, out_dim, p)
    assert ro.rel_l2(got, y64) < F32_TOL
    assert ro.rel_l2(got, ro.cpu_path(t, raw, x, in_dim, out_dim, n_threads=8)) < DP4A_REL_L2_MAX


@pytest.mark.parametrize("t", ro.ALL_TYPES)
@pytest.mark.parametrize("p", [1, 17, 20, 24, 64, 129])
def test_mmq_all_formats_row_counts(rt, t, p):
    in_dim, out_dim = 1024, 259
    raw, x = cases.synth_case(t, in_dim, out_dim, p, seed=17 * t + p)
    w = rt.GpuMatvecTensor.from_bytes_matvec(raw, t, in_dim, out_dim)
    y = torch.full((p, out_dim), float("nan"), device="cuda")
    rt.launch_mmq_gemm(w, quantize(rt, x), y, p)
    torch.cuda.synchronize()
    _, y64, _ = ro.matvec_q8(t, ro.repack(t, raw, in_dim, out_dim), ro.quantize_q8(x), in_dim, out_dim, p)
    assert ro.rel_l2(y.cpu().numpy(), y64) < F32_TOL


@pytest.mark.parametrize("t", ro.ALL_TYPES)
@pytest.mark.parametrize("n_rows", [1, 4, 5, 16, 17, 20])
def test_matmul_dispatch_matches_oracle(rt, t, n_rows):
    """PrefillGemm::matmul_into across its dispatch boundaries (src/runtime/prefill.rs:579-682)."""
    in_dim, out_dim = 1024, 256
    raw, x = cases.synth_case(t, in_dim, out_dim, n_rows, seed=13 * t + n_rows)
    w = rt.GpuMatvecTensor.from_bytes_matvec(raw, t, in_dim, out_dim)
    gemm = rt.PrefillGemm(max_x=in_dim)  # grows on demand
    y = gemm.matmul(w, torch.from_numpy(x).cuda(), n_rows)
    torch.cuda.synchronize()
    _, y64, _ = ro.matvec_q8(t, ro.repack(t, raw, in_dim, out_dim), ro.quantize_q8(x), in_dim, out_dim, n_rows)
    got = y.cpu().numpy()
    assert ro.rel_l2(got, y64) < F32_TOL
    assert ro.rel_l2(got, ro.cpu_path(t, raw, x, in_dim, out_dim, n_threads=8)) < DP4A_REL_L2_MAX


@pytest.mark.parametrize("n_entries,n_expert", [(0, 4), (1, 1), (4096, 256), (777, 60), (100, 128), (5000, 1000)])
def test_moe_sort_bit_exact(rt, n_entries, n_expert):
    rng = np.random.default_rng(n_entries + n_expert)
    ids = rng.integers(0, n_expert, max(n_entries, 1), dtype=np.int32)[:n_entries]
    if n_entries > 10:
        ids[3] = -1
        ids[7] = n_expert
    bn = rt.moe_tile_bn()
    moe = rt.MoeGroupedScratch.new(n_expert, n_entries)
    rt.launch_moe_sort(moe, torch.from_numpy(ids).cuda() if n_entries else torch.zeros(1, dtype=torch.int32, device="cuda"), n_entries, bn)
    torch.cuda.synchronize()
    count, eoff, toff, perm = ro.moe_sort(ids, n_expert, bn)
    assert np.array_equal(moe.count.cpu().numpy(), count)
    assert np.array_equal(moe.cursor.cpu().numpy(), count)
    assert np.array_equal(moe.expert_off.cpu().numpy(), eoff)
    assert np.array_equal(moe.tile_off.cpu().numpy(), toff)
    assert np.array_equal(moe.perm.cpu().numpy()[:n_entries], perm)


def test_moe_gather_scatter_round_trip(rt):
    n_tok, n_used, n_expert, hidden = 37, 4, 16, 256
    n_entries, n_sub = n_tok * n_used, hidden // 32
    rng = np.random.default_rng(2)
    ids = rng.integers(0, n_expert, n_entries, dtype=np.int32)
    moe = rt.MoeGroupedScratch.new(n_expert, n_entries)
    rt.launch_moe_sort(moe, torch.from_numpy(ids).cuda(), n_entries)
    x = rng.standard_normal((n_tok, hidden)).astype(np.float32)
    xq = quantize(rt, x)
    g = torch.zeros(n_entries * n_sub * 40, dtype=torch.uint8, device="cuda")
    rt.launch_moe_gather_xq(moe, xq, g, n_sub, n_used, n_entries)
    src = torch.from_numpy(rng.standard_normal((n_entries, 96)).astype(np.float32)).cuda()
    dst = torch.zeros_like(src)
    rt.launch_moe_scatter_rows(moe, src, dst, 96, n_entries)
    src1 = src[:, :95].contiguous()   # a width that cannot use 16-byte stores
    dst1 = torch.zeros_like(src1)
    rt.launch_moe_scatter_rows(moe, src1, dst1, 95, n_entries)
    torch.cuda.synchronize()
    perm = moe.perm.cpu().numpy()
    xq_rows = xq.cpu().numpy().reshape(n_tok, -1)
    assert np.array_equal(g.cpu().numpy().reshape(n_entries, -1), xq_rows[perm // n_used])
    want = np.zeros((n_entries, 96), dtype=np.float32)
    want[perm] = src.cpu().numpy()
    assert np.array_equal(dst.cpu().numpy(), want)
    assert np.array_equal(dst1.cpu().numpy(), want[:, :95])


@pytest.mark.parametrize("t,in_dim,out_dim", [(ro.Q4_K, 2048, 96), (ro.Q6_K, 512, 200), (ro.Q5_K, 256, 64),
                                              (ro.Q8_0, 512, 64), (ro.Q4_0, 256, 40), (ro.IQ4_XS, 512, 72)])
def test_grouped_gemm_matches_oracle(rt, t, in_dim, out_dim):
    """Grouped GEMM over expert-sorted rows, with empty experts, experts with more rows than
    a tile, and padded strides (in_dim 2048 and 512 have power-of-two sub-block counts)."""
    n_expert, n_tok, n_used = 12, 48, 4
    n_entries, n_sub = n_tok * n_used, in_dim // 32
    rng = np.random.default_rng(t)
    ids = rng.integers(0, n_expert - 2, n_entries, dtype=np.int32)  # experts 10, 11 stay empty
    ids[:40] = 3                                                    # expert 3 spans several tiles
    raws = [cases.synth_case(t, in_dim, out_dim, 1, seed=100 * t + e)[0] for e in range(n_expert)]
    et = rt.GpuExpertTensor.from_bytes(np.concatenate(raws), t, in_dim, out_dim, n_expert)
    slab = np.concatenate([ro.repack(t, r, in_dim, out_dim) for r in raws])
    assert np.array_equal(et.data.cpu().numpy(), slab)
    x = rng.standard_normal((n_tok, in_dim)).astype(np.float32)
    moe = rt.MoeGroupedScratch.new(n_expert, n_entries)
    rt.launch_moe_sort(moe, torch.from_numpy(ids).cuda(), n_entries)
    xq = quantize(rt, x)
    g = torch.zeros(n_entries * n_sub * 40, dtype=torch.uint8, device="cuda")
    rt.launch_moe_gather_xq(moe, xq, g, n_sub, n_used, n_entries)
    y = torch.full((n_entries, out_dim), float("nan"), device="cuda")
    rt.launch_moe_grouped_gemm(moe, et, g, y, in_dim, out_dim, n_entries)
    torch.cuda.synchronize()
    eoff = moe.expert_off.cpu().numpy()
    _, y64 = ro.grouped_q8(t, slab, et.bytes_per_expert, eoff, g.cpu().numpy(), in_dim, out_dim)
    assert ro.rel_l2(y.cpu().numpy(), y64) < F32_TOL


@pytest.mark.parametrize("kind", [8, 16])
@pytest.mark.parametrize("t", ro.ALL_TYPES)
def test_mmq_both_tensor_core_kernels(rt, t, kind):
    """The int8-operand and the f16-operand tcgen05 kernels against the oracle, dense (a ragged
    200 x 300 problem over two token tiles) and grouped; Q6_K exists only in the f16 kernel (the
    int8 setting then runs the dp4a kernel)."""
    from reinstinct_b200 import _lib

    lib = _lib.load()
    lib.rc_tune_mmq(0, kind)
    try:
        in_dim, out_dim, p = 1024, 300, 200
        raw, x = cases.synth_case(t, in_dim, out_dim, p, seed=7 * t + kind)
        w = rt.GpuMatvecTensor.from_bytes_matvec(raw, t, in_dim, out_dim)
        y = torch.full((p, out_dim), float("nan"), device="cuda")
        rt.launch_mmq_gemm(w, quantize(rt, x), y, p)
        torch.cuda.synchronize()
        _, y64, _ = ro.matvec_q8(t, ro.repack(t, raw, in_dim, out_dim), ro.quantize_q8(x), in_dim, out_dim, p)
        assert ro.rel_l2(y.cpu().numpy(), y64) < F32_TOL
        st = __import__("ctypes").c_uint(0)
        assert lib.rc_device_status(__import__("ctypes").byref(st)) == 0 and st.value == 0
    finally:
        lib.rc_tune_mmq(0, 0)
