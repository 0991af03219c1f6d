"""GPU parity of the f16-operand dense GEMM behind rc_matmul (more than RC_MATVEC_MAX_ROWS rows): every
format, every token-tile width, ragged shapes, against the oracle's exact-integer formulation.  The
kernel rounds each dequantized weight and activation once to f16, so the bar is the reference's own f32
tolerance (1e-3 relative L2), not bit equality; the int8 kernel behind rc_mmq_gemm keeps the integer
dots exact."""
import ctypes

import numpy as np
import pytest
import torch

import cases
import oracle as ro

pytestmark = pytest.mark.gpu

F32_TOL = 1e-3          # src/runtime/kernels.rs GPU-vs-CPU bar of the reference's own kernel tests
EXPECTED = 5e-4         # what two f16 roundings give; a regression past this is a bug, not noise


def _status(lib) -> int:
    st = ctypes.c_uint(0)
    assert lib.rc_device_status(ctypes.byref(st)) == 0
    return st.value


def _oracle(t, raw, x, in_dim, out_dim, p):
    _, y64, _ = ro.matvec_q8(t, ro.repack(t, raw, in_dim, out_dim), ro.quantize_q8(x), in_dim, out_dim, p)
    return y64


@pytest.mark.parametrize("t", ro.ALL_TYPES)
@pytest.mark.parametrize("bn", [0, 128, 256, 512])
@pytest.mark.parametrize("in_dim,out_dim,p", [(1024, 300, 200), (256, 128, 17), (512, 257, 600), (2048, 130, 513)])
def test_deq_gemm_matches_oracle(rt, t, bn, in_dim, out_dim, p):
    """Ragged row and token counts (tiles partly outside the matrix, several tiles per CTA at the
    narrow widths), the smallest K of the K-quants (one superblock: the minima step is mostly padding)."""
    lib = rt._lib.load()
    raw, x = cases.synth_case(t, in_dim, out_dim, p, seed=7 * t + p)
    w = rt.GpuMatvecTensor.from_bytes_matvec(raw, t, in_dim, out_dim)
    lib.rc_tune_mmq(0, 32 | (bn << 8))
    try:
        y = torch.full((p, out_dim), float("nan"), device="cuda")
        rt.PrefillGemm().matmul_into(y, w, torch.from_numpy(x).cuda(), p)
        torch.cuda.synchronize()
    finally:
        lib.rc_tune_mmq(0, 0)
    assert _status(lib) == 0
    err = ro.rel_l2(y.cpu().numpy(), _oracle(t, raw, x, in_dim, out_dim, p))
    assert err < EXPECTED < F32_TOL


@pytest.mark.parametrize("t,in_dim,out_dim,p", [
    (ro.Q4_K, 4096, 130, 513),    # 4 ranges of K steps (minima steps included in the last one)
    (ro.Q6_K, 4096, 130, 513),
    (ro.Q4_K, 3072, 1300, 512),   # 11 row tiles: 3 ranges, uneven (99 steps over 3)
    (ro.Q8_0, 3072, 1300, 300),
])
def test_deq_gemm_k_split_three_and_four_ways(rt, t, in_dim, out_dim, p):
    """Few tiles, long K: the opt-in f16 route splits K into up to four ranges and adds the partial sums atomically
    (y zeroed first).  Parity with the oracle, and with the same call forced to one range (debug bit 64)."""
    lib = rt._lib.load()
    raw, x = cases.synth_case(t, in_dim, out_dim, p, seed=11 * t + p)
    w = rt.GpuMatvecTensor.from_bytes_matvec(raw, t, in_dim, out_dim)
    xd = torch.from_numpy(x).cuda()
    want = _oracle(t, raw, x, in_dim, out_dim, p)
    got = {}
    for name, kind in (("split", 32), ("one range", 32 | (64 << 20))):
        lib.rc_tune_mmq(0, kind)
        try:
            y = torch.full((p, out_dim), float("nan"), device="cuda")
            rt.PrefillGemm().matmul_into(y, w, xd, p)
            torch.cuda.synchronize()
        finally:
            lib.rc_tune_mmq(0, 0)
        assert _status(lib) == 0
        got[name] = y.cpu().numpy()
        assert ro.rel_l2(got[name], want) < EXPECTED, name
    assert ro.rel_l2(got["split"], got["one range"].astype(np.float64)) < 1e-5


@pytest.mark.parametrize("t", ro.ALL_TYPES)
def test_deq_gemm_many_tiles_per_cta(rt, t):
    """More tiles than SMs at the narrow width: the accumulator buffers and both rings wrap many times."""
    lib = rt._lib.load()
    in_dim, out_dim, p = 256, 128 * 40, 512
    raw, x = cases.synth_case(t, in_dim, out_dim, p, seed=31 * t)
    w = rt.GpuMatvecTensor.from_bytes_matvec(raw, t, in_dim, out_dim)
    want = _oracle(t, raw, x, in_dim, out_dim, p)
    for bn in (128, 512):
        lib.rc_tune_mmq(0, 32 | (bn << 8))
        try:
            y = torch.full((p, out_dim), float("nan"), device="cuda")
            rt.PrefillGemm().matmul_into(y, w, torch.from_numpy(x).cuda(), p)
            torch.cuda.synchronize()
        finally:
            lib.rc_tune_mmq(0, 0)
        assert _status(lib) == 0
        assert ro.rel_l2(y.cpu().numpy(), want) < EXPECTED


def test_deq_gemm_token_scale_range(rt):
    """Token rows of very different magnitude (1e-6 .. 1e4), an all-zero row and a row with one huge
    outlier: the per-token power-of-two scale keeps every row inside f16 range and precision."""
    t, in_dim, out_dim, p = ro.Q4_K, 1024, 256, 64
    raw, x = cases.synth_case(t, in_dim, out_dim, p, seed=99)
    scale = np.float32(10.0) ** np.linspace(-6, 4, p).astype(np.float32)
    x = (x * scale[:, None]).astype(np.float32)
    x[5] = 0.0
    x[9, 100] = 6.0e4
    w = rt.GpuMatvecTensor.from_bytes_matvec(raw, t, in_dim, out_dim)
    y = torch.full((p, out_dim), float("nan"), device="cuda")
    rt.PrefillGemm().matmul_into(y, w, torch.from_numpy(x).cuda(), p)
    torch.cuda.synchronize()
    got, want = y.cpu().numpy(), _oracle(t, raw, x, in_dim, out_dim, p)
    assert np.all(np.isfinite(got))
    assert np.all(got[5] == 0.0)
    for r in range(p):  # row by row: a global norm would hide the small rows
        if r != 5:
            assert ro.rel_l2(got[r], want[r]) < F32_TOL, r


def test_deq_gemm_agrees_with_exact_integer_kernel(rt):
    """The same call forced through the int8 kernel (exact integer dots) differs only by the f16 roundings."""
    lib = rt._lib.load()
    t, in_dim, out_dim, p = ro.Q5_K, 2048, 384, 96
    raw, x = cases.synth_case(t, in_dim, out_dim, p, seed=5)
    w = rt.GpuMatvecTensor.from_bytes_matvec(raw, t, in_dim, out_dim)
    xs = torch.from_numpy(x).cuda()
    ys = []
    for kind in (8, 32):
        lib.rc_tune_mmq(0, kind)
        try:
            ys.append(rt.PrefillGemm().matmul(w, xs, p).cpu().numpy())
        finally:
            lib.rc_tune_mmq(0, 0)
    assert ro.rel_l2(ys[0], _oracle(t, raw, x, in_dim, out_dim, p)) < 2e-6
    assert ro.rel_l2(ys[1], ys[0]) < EXPECTED


def test_scratch_bytes_cover_the_f16_image(rt):
    lib = rt._lib.load()
    for in_dim, n in ((5120, 512), (256, 17), (17408, 100)):
        n_sub = in_dim // 32
        ld = (n + 7) // 8 * 8
        image = (in_dim // 8 + (((n_sub + 7) // 8 + 3) // 4 * 4)) * ld * 16 + ld * 4
        assert lib.rc_matmul_scratch_bytes(in_dim, n) >= max(image, n * n_sub * 40)
    assert lib.rc_matmul_scratch_bytes(5120, 16) >= 16 * 160 * 40  # matvec range: BlockQ8 records only
