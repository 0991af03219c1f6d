"""GPU parity of Q5_1 expert tensors (src/runtime/qwen35.rs:421, src/quant/q5_1.rs): the device repack
byte for byte against the oracle, then every entry point that takes a weight type.  The kernels are the
Q5_K bodies with dsc = d, deff = -m (kernels/moe_matvec_q5k_repacked.cpp:86-91); in_dim only has to be a
multiple of 32."""
import ctypes

import numpy as np
import pytest
import torch

import cases
import oracle as ro

pytestmark = pytest.mark.gpu

T = ro.Q5_1
F32_TOL = 1e-3       # the reference's GPU-vs-CPU bar (src/runtime/kernels.rs)
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


@pytest.mark.parametrize("in_dim,out_dim", [(256, 5), (160, 23), (2048, 384), (1056, 130), (32, 1)])
def test_repack_matches_oracle(rt, in_dim, out_dim):
    raw, _ = cases.synth_case(T, in_dim, out_dim, 1, seed=in_dim + out_dim)
    w = rt.GpuMatvecTensor.from_bytes_matvec(raw, T, in_dim, out_dim)
    assert w.dtype == T
    np.testing.assert_array_equal(w.data.cpu().numpy(), ro.repack(T, raw, in_dim, out_dim))


@pytest.mark.parametrize("in_dim,out_dim,n_rows", [(2048, 384, 1), (160, 37, 1), (5120, 1000, 1), (1056, 301, 2),
                                                   (512, 77, 7), (4096, 640, 16), (96, 200, 5)])
def test_matvec_and_block_integers(rt, in_dim, out_dim, n_rows):
    raw, x = cases.synth_case(T, in_dim, out_dim, n_rows, seed=3 * in_dim + n_rows)
    wt = rt.GpuMatvecTensor.from_bytes_matvec(raw, T, in_dim, out_dim)
    xq = _xq(rt, x)
    y = torch.full((n_rows, out_dim), float("nan"), device="cuda")
    if n_rows == 1:
        rt.launch_matvec_xq8(wt, xq, y)
    else:
        rt.launch_matvec_batched(wt, xq, y, n_rows)
    torch.cuda.synchronize()
    planes = ro.repack(T, raw, in_dim, out_dim)
    _, y64, idots = ro.matvec_q8(T, planes, ro.quantize_q8(x), in_dim, out_dim, n_rows, want_idots=True)
    assert ro.rel_l2(y.cpu().numpy(), y64) < 1e-5
    assert ro.rel_l2(y.cpu().numpy(), ro.cpu_path(T, raw, x, in_dim, out_dim, n_threads=4)) < 2e-2
    assert np.array_equal(rt.matvec_block_dots(wt, xq, n_rows).cpu().numpy(), idots)


@pytest.mark.parametrize("in_dim,out_dim,p", [(1024, 300, 200), (160, 128, 17), (2048, 130, 513)])
def test_gemm_from_blockq8(rt, in_dim, out_dim, p):
    """rc_mmq_gemm: Q5_1 takes the dp4a passes (exact integer dots)."""
    raw, x = cases.synth_case(T, in_dim, out_dim, p, seed=p)
    wt = rt.GpuMatvecTensor.from_bytes_matvec(raw, T, in_dim, out_dim)
    y = torch.full((p, out_dim), float("nan"), device="cuda")
    rt.launch_mmq_gemm(wt, _xq(rt, x), y, p)
    torch.cuda.synchronize()
    assert _status(rt._lib.load()) == 0
    _, y64, _ = ro.matvec_q8(T, ro.repack(T, raw, in_dim, out_dim), ro.quantize_q8(x), in_dim, out_dim, p)
    assert ro.rel_l2(y.cpu().numpy(), y64) < 1e-5


@pytest.mark.parametrize("bn", [0, 128, 256, 512])
@pytest.mark.parametrize("in_dim,out_dim,p", [(1024, 300, 200), (1056, 257, 600), (160, 128, 40), (8192, 256, 64)])
def test_f16_operand_gemm(rt, bn, in_dim, out_dim, p):
    """rc_matmul beyond 16 rows: the tensor-core kernel, with the minima as extra K steps (+ m * xsum);
    in_dim 1056 and 160 leave the last group of eight sub-blocks partly empty, 8192 needs eight of them."""
    lib = rt._lib.load()
    raw, x = cases.synth_case(T, in_dim, out_dim, p, seed=bn + p)
    wt = rt.GpuMatvecTensor.from_bytes_matvec(raw, T, in_dim, out_dim)
    lib.rc_tune_mmq(0, 32 | (bn << 8))
    try:
        y = torch.full((p, out_dim), float("nan"), device="cuda")
        rt.PrefillGemm().matmul_into(y, wt, torch.from_numpy(x).cuda(), p)
        torch.cuda.synchronize()
    finally:
        lib.rc_tune_mmq(0, 0)
    assert _status(lib) == 0
    _, y64, _ = ro.matvec_q8(T, ro.repack(T, raw, in_dim, out_dim), ro.quantize_q8(x), in_dim, out_dim, p)
    assert ro.rel_l2(y.cpu().numpy(), y64) < DEQ_EXPECTED < F32_TOL


def _experts(rt, in_dim, out_dim, n_expert, seed):
    raws = [cases.synth_case(T, in_dim, out_dim, 1, seed=seed + e)[0] for e in range(n_expert)]
    parts = [ro.repack(T, r, in_dim, out_dim) for r in raws]
    return parts, np.concatenate(parts), rt.GpuExpertTensor.from_bytes(np.concatenate(raws), T, in_dim, out_dim, n_expert)


@pytest.mark.parametrize("in_dim", [1024, 1056])
def test_expert_matvec_down_and_fused_gate_up(rt, in_dim):
    """The three decode-side MoE kernels the reference runs Q5_1 experts on (qwen35.rs:3082, 3116); the
    fused gate + up kernel takes whole 1024-weight iterations only."""
    out_dim, n_expert, n_used, n_tok = 80, 6, 3, 4
    has_fused = in_dim % 1024 == 0
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
    if has_fused:
        rt.launch_moe_gate_up_swiglu(g, u, ids_d, xq, fused, n_used, n_tok, n_sub, 0)
    # down addressing: one activation row per (token, slot)
    xs = rng.standard_normal((n_tok * n_used, in_dim)).astype(np.float32)
    yd = torch.full((n_tok, n_used, out_dim), float("nan"), device="cuda")
    rt.launch_moe_expert_matvec(g, ids_d, _xq(rt, xs), yd, n_used, n_tok, n_used * n_sub, n_sub)
    torch.cuda.synchronize()
    xq_h = ro.quantize_q8(x).reshape(n_tok, -1)
    xs_h = ro.quantize_q8(xs).reshape(n_tok * n_used, -1)
    for tk in range(n_tok):
        for j in range(n_used):
            e = ids[tk, j]
            _, g64, _ = ro.matvec_q8(T, gparts[e], xq_h[tk], in_dim, out_dim, 1)
            _, u64, _ = ro.matvec_q8(T, uparts[e], xq_h[tk], in_dim, out_dim, 1)
            _, d64, _ = ro.matvec_q8(T, gparts[e], xs_h[tk * n_used + j], in_dim, out_dim, 1)
            assert ro.rel_l2(yg[tk, j].cpu().numpy(), g64) < 1e-5
            assert ro.rel_l2(yd[tk, j].cpu().numpy(), d64) < 1e-5
            want = g64 / (1.0 + np.exp(-g64)) * u64
            if has_fused:
                assert ro.rel_l2(fused[tk, j].cpu().numpy(), want) < 2e-5


@pytest.mark.parametrize("in_dim,out_dim", [(1024, 304), (1056, 128)])
def test_grouped_gemms(rt, in_dim, out_dim):
    """Expert-grouped GEMM (qwen35.rs:3045), both routes: f32 token rows through the f16-operand
    tensor-core kernel, BlockQ8 rows through the dp4a grouped kernel."""
    n_expert, n_tok, n_used = 12, 48, 4
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
