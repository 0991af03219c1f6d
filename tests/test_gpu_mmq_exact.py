"""GPU parity of the dense GEMM behind rc_matmul for more than RC_MATVEC_MAX_ROWS rows (the route
PrefillGemm::matmul_into_raw takes, src/runtime/prefill.rs:343-437 -> mmq_gemm_<fmt>_repacked_f32):
integer-valued f16 operands on the tensor cores, one accumulator tile per 32-wide sub-block.

Two bars.  The tile the kernel drains per (token, row, sub-block) is compared as INTEGERS with the
oracle's block dots (kernels/mmq_gemm_q4k_repacked.cpp:150-161 holds them in registers): bit-exact.
The f32 result is compared with the oracle's exact-integer formulation at the reference's f32 bar."""
import ctypes

import numpy as np
import pytest
import torch

import cases
import oracle as ro

pytestmark = pytest.mark.gpu

F32_TOL = 1e-3      # north-star bar for f32 outputs (relative L2 against the int8-path oracle)
EXPECTED = 2e-5     # what this route gives (f32 association + the 2^-16 minima split); beyond it is a bug

TYPES = list(ro.ALL_TYPES)


def _status(lib) -> int:
    st = ctypes.c_uint(0)
    assert lib.rc_device_status(ctypes.byref(st)) == 0
    return st.value


def _oracle(t, raw, x, in_dim, out_dim, p, want_idots=False):
    wrep = ro.repack(t, raw, in_dim, out_dim)
    _, y64, idots = ro.matvec_q8(t, wrep, ro.quantize_q8(x), in_dim, out_dim, p, want_idots=want_idots)
    return wrep, y64, idots


def _expected_tile(t, wrep, idots, in_dim, out_dim):
    """What the tensor-core accumulator holds per (token, row, sub-block): the block dot, times the
    integer sub-scale where the format has one (the f16 d / dmin stay outside)."""
    n_sub, nsp = in_dim // 32, ro.nsp(in_dim)
    q = out_dim * nsp
    i0, i1 = idots[..., 0].astype(np.int64), idots[..., 1].astype(np.int64)
    if t in (ro.Q4_K, ro.Q5_K):
        off = q * 16 + (q * 4 if t == ro.Q5_K else 0)
        sc = wrep[off:off + q * 2].reshape(out_dim, nsp, 2)[:, :n_sub, 0].astype(np.int64)
        return i0 * sc[None]
    if t == ro.Q6_K:
        off = q * 16 + q * 8
        s = wrep[off:off + q * 2].view(np.int8).reshape(out_dim, nsp, 2)[:, :n_sub].astype(np.int64)
        return i0 * s[None, :, :, 0] + i1 * s[None, :, :, 1]
    return i0


@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("in_dim,out_dim,p", [(2048, 384, 70), (768, 259, 129)])
def test_block_dots_bit_exact(rt, t, in_dim, out_dim, p):
    """The reference's own MMQ test shape (P = 70, out 384: src/runtime/kernels.rs:3171-3220; in_dim 2048
    is a power-of-two sub-block count, the padded stride) and a ragged 129 x 259 case (a token tile and a
    row tile each with one live element)."""
    lib = rt._lib.load()
    raw, x = cases.synth_case(t, in_dim, out_dim, p, seed=11 * t + p)
    w = rt.GpuMatvecTensor.from_bytes_matvec(raw, t, in_dim, out_dim)
    y, got = rt.PrefillGemm().matmul_block_dots(w, torch.from_numpy(x).cuda(), p)
    torch.cuda.synchronize()
    assert _status(lib) == 0
    wrep, y64, idots = _oracle(t, raw, x, in_dim, out_dim, p, want_idots=True)
    want = _expected_tile(t, wrep, idots, in_dim, out_dim)
    assert np.array_equal(got.cpu().numpy().astype(np.int64), want)
    assert ro.rel_l2(y.cpu().numpy(), y64) < EXPECTED < F32_TOL


@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("in_dim,out_dim,p", [(1024, 300, 200), (256, 128, 17), (512, 257, 600), (2048, 130, 513)])
def test_default_route_matches_oracle(rt, t, in_dim, out_dim, p):
    """rc_matmul as callers use it (no tuning switch): ragged row and token counts, the smallest K of the
    K-quants (one superblock), several token tiles."""
    lib = rt._lib.load()
    raw, x = cases.synth_case(t, in_dim, out_dim, p, seed=7 * t + p)
    w = rt.GpuMatvecTensor.from_bytes_matvec(raw, t, in_dim, out_dim)
    y = torch.full((p, out_dim), float("nan"), device="cuda")
    rt.PrefillGemm().matmul_into(y, w, torch.from_numpy(x).cuda(), p)
    torch.cuda.synchronize()
    assert _status(lib) == 0
    _, y64, _ = _oracle(t, raw, x, in_dim, out_dim, p)
    assert ro.rel_l2(y.cpu().numpy(), y64) < EXPECTED


@pytest.mark.parametrize("t", [ro.Q4_K, ro.Q5_K, ro.Q6_K, ro.Q8_0])
def test_long_k_more_minima_steps_than_ring_stages(rt, t):
    """K = 5120: twenty superblocks, so the block of minima steps (Q4_K, Q5_K) is several operand-ring cycles
    long and the two MMA issuers must not drift apart across it; several tiles per CTA on top (40 x 3 tiles
    would not do it: 60 x 3 = 180 tiles on 148 SMs)."""
    lib = rt._lib.load()
    in_dim, out_dim, p = 5120, 128 * 60 - 5, 300
    raw, x = cases.synth_case(t, in_dim, out_dim, p, seed=41 * t)
    w = rt.GpuMatvecTensor.from_bytes_matvec(raw, t, in_dim, out_dim)
    y = torch.full((p, out_dim), float("nan"), device="cuda")
    rt.PrefillGemm().matmul_into(y, w, torch.from_numpy(x).cuda(), p)
    torch.cuda.synchronize()
    assert _status(lib) == 0
    # the exact-integer batched matvec on a sample of tokens (the CPU oracle would take minutes at this size)
    sel = torch.arange(0, p, p // 16, device="cuda")[:16]
    xq = torch.empty(16 * (in_dim // 32) * 40, dtype=torch.uint8, device="cuda")
    rt.launch_quantize_q8(torch.from_numpy(x).cuda()[sel].contiguous(), xq, in_dim, 16)
    ye = torch.empty(16, out_dim, device="cuda")
    rt.launch_matvec_batched(w, xq, ye, 16)
    torch.cuda.synchronize()
    assert torch.isfinite(y).all()
    assert ro.rel_l2(y[sel].cpu().numpy(), ye.cpu().numpy().astype(np.float64)) < EXPECTED


@pytest.mark.parametrize("t", TYPES)
def test_many_tiles_per_cta(rt, t):
    """More tiles than SMs: every ring, the parked accumulator and the minima accumulator wrap across
    tiles inside one CTA.  The dump entry forces the tensor-core kernel whatever the cost model says."""
    lib = rt._lib.load()
    in_dim, out_dim, p = 256, 128 * 40, 512
    raw, x = cases.synth_case(t, in_dim, out_dim, p, seed=31 * t)
    w = rt.GpuMatvecTensor.from_bytes_matvec(raw, t, in_dim, out_dim)
    _, want, _ = _oracle(t, raw, x, in_dim, out_dim, p)
    y, _ = rt.PrefillGemm().matmul_block_dots(w, torch.from_numpy(x).cuda(), p)
    torch.cuda.synchronize()
    assert _status(lib) == 0
    assert ro.rel_l2(y.cpu().numpy(), want) < EXPECTED


def test_activation_range_and_zero_rows(rt):
    """Token rows of very different magnitude (1e-6 .. 1e4), an all-zero row and a row with one huge
    outlier: dx is an f32 scalar outside the integer product, so range never touches the operands."""
    lib = rt._lib.load()
    t, in_dim, out_dim, p = ro.Q4_K, 1024, 256, 64
    raw, x = cases.synth_case(t, in_dim, out_dim, p, seed=99)
    scale = np.float32(10.0) ** np.linspace(-6, 4, p).astype(np.float32)
    x = (x * scale[:, None]).astype(np.float32)
    x[5] = 0.0
    x[9, 17] = 3.0e7
    w = rt.GpuMatvecTensor.from_bytes_matvec(raw, t, in_dim, out_dim)
    y, _ = rt.PrefillGemm().matmul_block_dots(w, torch.from_numpy(x).cuda(), p)
    torch.cuda.synchronize()
    assert _status(lib) == 0
    _, y64, _ = _oracle(t, raw, x, in_dim, out_dim, p)
    got = y.cpu().numpy()
    assert np.all(got[5] == 0.0)
    for r in range(p):  # per row: a global norm would hide the small rows
        assert ro.rel_l2(got[r], y64[r]) < EXPECTED * 5, r


def test_result_is_reproducible_and_token_independent(rt):
    """No atomics, no K split: two runs are bit-identical, and a token's row does not depend on which
    other tokens share its tile."""
    t, in_dim, out_dim, p = ro.Q6_K, 1024, 640, 300
    raw, x = cases.synth_case(t, in_dim, out_dim, p, seed=5)
    w = rt.GpuMatvecTensor.from_bytes_matvec(raw, t, in_dim, out_dim)
    xd = torch.from_numpy(x).cuda()
    gemm = rt.PrefillGemm()
    y1, _ = gemm.matmul_block_dots(w, xd, p)
    y2, _ = gemm.matmul_block_dots(w, xd, p)
    perm = torch.randperm(p, device="cuda", generator=torch.Generator(device="cuda").manual_seed(3))
    y3, _ = gemm.matmul_block_dots(w, xd[perm].contiguous(), p)
    torch.cuda.synchronize()
    assert torch.equal(y1, y2)
    assert torch.equal(y3, y1[perm])


def test_scratch_rules(rt):
    """The route never depends on the scratch: a scratch that only holds the BlockQ8 records is an error
    for a shape that takes the tensor-core kernel, not a switch to other numerics."""
    lib = rt._lib.load()
    t, in_dim, out_dim, p = ro.Q4_K, 5120, 4096, 64
    raw, x = cases.synth_case(t, in_dim, out_dim, p, seed=1)
    w = rt.GpuMatvecTensor.from_bytes_matvec(raw, t, in_dim, out_dim)
    xd = torch.from_numpy(x).cuda()
    y = torch.empty(p, out_dim, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    small = torch.empty(p * (in_dim // 32) * 40, dtype=torch.uint8, device="cuda")
    rc = lib.rc_matmul(stream, t, w.data.data_ptr(), xd.data_ptr(), y.data_ptr(), in_dim, out_dim, p, small.data_ptr(), small.numel())
    assert rc == -6, lib.rc_error_string(rc)  # RC_ERR_SCRATCH_TOO_SMALL
    need = lib.rc_matmul_scratch_bytes(in_dim, p)
    big = torch.empty(need + 16, dtype=torch.uint8, device="cuda")
    rc = lib.rc_matmul(stream, t, w.data.data_ptr(), xd.data_ptr(), y.data_ptr(), in_dim, out_dim, p, big.data_ptr() + 8, need)
    assert rc == -4, lib.rc_error_string(rc)  # RC_ERR_MISALIGNED
    torch.cuda.synchronize()


def test_f16_route_is_opt_in_and_close(rt):
    """rc_matmul_f16 (operands dequantized to f16) is the named approximation: within the f32 bar of the
    exact route, and measurably not the same numbers."""
    t, in_dim, out_dim, p = ro.Q4_K, 2048, 512, 200
    raw, x = cases.synth_case(t, in_dim, out_dim, p, seed=21)
    w = rt.GpuMatvecTensor.from_bytes_matvec(raw, t, in_dim, out_dim)
    xd = torch.from_numpy(x).cuda()
    gemm = rt.PrefillGemm()
    y_exact, _ = gemm.matmul_block_dots(w, xd, p)
    y_f16 = torch.empty(p, out_dim, device="cuda")
    gemm.matmul_f16_into(y_f16, w, xd, p)
    torch.cuda.synchronize()
    err = ro.rel_l2(y_f16.cpu().numpy(), y_exact.cpu().numpy().astype(np.float64))
    assert 1e-5 < err < F32_TOL
