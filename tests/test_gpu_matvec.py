"""GPU parity of the decode / batched matvec family through the C ABI: per-block integer
dots bit-exact, f32 outputs within 1e-3 relative L2 of the int8-path oracle (f64 sums), and
within the reference's own 1.5e-2 of its f32 dequant path."""
import numpy as np
import pytest
import torch

import cases
import oracle as ro

pytestmark = pytest.mark.gpu

F32_TOL = 1e-3          # north-star tolerance against the int8-path oracle
DP4A_REL_L2_MAX = 1.5e-2  # src/runtime/kernels.rs:1601, against the f32 dequant path


def run_case(rt, t, raw, x, in_dim, out_dim, check_ints=True, f32_ref=True):
    n_rows = x.shape[0]
    w = rt.GpuMatvecTensor.from_bytes_matvec(raw, t, in_dim, out_dim)
    wq = ro.repack(t, raw, in_dim, out_dim)
    assert np.array_equal(w.data.cpu().numpy(), wq)
    xd = torch.from_numpy(x).cuda()
    xq = torch.empty(n_rows * (in_dim // 32) * 40, dtype=torch.uint8, device="cuda")
    rt.launch_quantize_q8(xd, xq, in_dim, n_rows)
    xq_ref = ro.quantize_q8(x)
    assert np.array_equal(xq.cpu().numpy(), xq_ref)
    y = torch.full((n_rows, out_dim), float("nan"), device="cuda")
    if n_rows == 1:
        rt.launch_matvec_xq8(w, xq, y)
    else:
        rt.launch_matvec_batched(w, xq, y, n_rows)
    torch.cuda.synchronize()
    y32, y64, idots = ro.matvec_q8(t, wq, xq_ref, in_dim, out_dim, n_rows, want_idots=check_ints)
    got = y.cpu().numpy()
    assert np.isfinite(got).all()
    e = ro.rel_l2(got, y64)
    assert e < F32_TOL, f"rel_l2 vs int8-path oracle {e:.3e}"
    if check_ints:
        gi = rt.matvec_block_dots(w, xq, n_rows).cpu().numpy()
        assert np.array_equal(gi, idots)
    if f32_ref:
        e32 = ro.rel_l2(got, ro.cpu_path(t, raw, x, in_dim, out_dim, n_threads=8))
        assert e32 < DP4A_REL_L2_MAX, f"rel_l2 vs f32 dequant path {e32:.3e}"
    return e


@pytest.mark.parametrize("t,seed,inc", [(ro.Q4_K, 0xD4A40001, 1442695040888963407),
                                        (ro.Q5_K, 0xD5A51234, 1), (ro.Q6_K, 0xD6A65678, 1)])
def test_reference_case_2048x384(rt, t, seed, inc):
    """matvec_q4k_repacked_matches_dequant_path (src/runtime/kernels.rs:3021-3118)."""
    raw = cases.lcg_case(t, 2048, 384, seed, inc)
    x = cases.lcg_x(2048, 0x13579BDF).reshape(1, -1)
    run_case(rt, t, raw, x, 2048, 384)


@pytest.mark.parametrize("t", [ro.Q4_K, ro.Q5_K, ro.Q6_K])
@pytest.mark.parametrize("in_dim", [5376, 8192, 16384, 21504])
def test_gemma_shapes_pad_path(rt, t, in_dim):
    """matvec_kquant_repacked_gemma_shapes_match_dequant (src/runtime/kernels.rs:3125-3168):
    8192 and 16384 have power-of-two sub-block counts (padded stride)."""
    raw, x = cases.synth_case(t, in_dim, 64, 1, seed=in_dim + t)
    run_case(rt, t, raw, x, in_dim, 64)


@pytest.mark.parametrize("t", ro.ALL_TYPES)
@pytest.mark.parametrize("n_rows", [1, 2, 3, 4, 5, 8, 15, 16])
def test_all_formats_all_row_counts(rt, t, n_rows):
    """Every dispatch boundary of matmul_into_matches_oracle_across_row_counts
    (src/runtime/prefill.rs:579-682), in_dim 1024 (padded stride), out 256 + a ragged tail."""
    raw, x = cases.synth_case(t, 1024, 259, n_rows, seed=31 * t + n_rows)
    run_case(rt, t, raw, x, 1024, 259)


@pytest.mark.parametrize("t", ro.ALL_TYPES)
def test_small_and_odd_shapes(rt, t):
    bw = ro.block_weights(t)
    for in_dim, out_dim, n_rows in [(bw, 1, 1), (bw, 3, 4), (bw * 3, 17, 2), (bw * 5, 1, 16)]:
        raw, x = cases.synth_case(t, in_dim, out_dim, n_rows, seed=in_dim + out_dim + t)
        # a handful of outputs is too few for a meaningful norm against the f32 path
        run_case(rt, t, raw, x, in_dim, out_dim, f32_ref=False)


@pytest.mark.parametrize("t", [ro.Q4_0, ro.Q8_0])
def test_in_dim_multiple_of_32_only(rt, t):
    """Q4_0 / Q8_0 accept any in_dim % 32 == 0 (the reference's dense MMQ silently assumes
    % 128, kernels/mmq_gemm_q8_0_repacked.cpp:87-109)."""
    raw, x = cases.synth_case(t, 32 * 7, 33, 3, seed=5 + t)
    run_case(rt, t, raw, x, 32 * 7, 33)


def test_config1_q8_0_4096(rt):
    raw, x = cases.synth_case(ro.Q8_0, 4096, 4096, 1, seed=1, signed=False)
    run_case(rt, ro.Q8_0, raw, x, 4096, 4096, check_ints=False)


@pytest.mark.parametrize("t,in_dim,out_dim", [(ro.Q4_K, 5120, 17408), (ro.Q6_K, 17408, 5120)])
def test_config2_layer_shapes(rt, t, in_dim, out_dim):
    raw, x = cases.synth_case(t, in_dim, out_dim, 1, seed=2 + t, signed=False)
    run_case(rt, t, raw, x, in_dim, out_dim, check_ints=False, f32_ref=(t == ro.Q4_K))


@pytest.mark.parametrize("t", [ro.Q4_0, ro.Q5_K, ro.Q6_K, ro.Q8_0, ro.IQ4_XS])
def test_config3_batch4_5120(rt, t):
    raw, x = cases.synth_case(t, 5120, 5120, 4, seed=3 + t, signed=False)
    run_case(rt, t, raw, x, 5120, 5120, check_ints=False)


def test_matvec_f32_wrapper_and_linearity(rt):
    """launch_matvec (quantize + matvec in one call) equals the two-step form, and the kernel
    is linear in the weights' super-scale: doubling d doubles y exactly (power of two)."""
    t, in_dim, out_dim = ro.Q6_K, 2048, 300
    raw, x = cases.synth_case(t, in_dim, out_dim, 1, seed=77)
    w = rt.GpuMatvecTensor.from_bytes_matvec(raw, t, in_dim, out_dim)
    xd = torch.from_numpy(x).cuda()
    xq = torch.empty((in_dim // 32) * 40, dtype=torch.uint8, device="cuda")
    y1 = torch.empty(out_dim, device="cuda")
    y2 = torch.empty(out_dim, device="cuda")
    rt.launch_matvec(w, xd, y1, xq)
    rt.launch_matvec_xq8(w, xq, y2)
    raw2 = raw.reshape(-1, 210).copy()
    d = raw2[:, 208:210].copy().view(np.float16).astype(np.float32) * 2
    raw2[:, 208:210] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    w2 = rt.GpuMatvecTensor.from_bytes_matvec(raw2.reshape(-1), t, in_dim, out_dim)
    y3 = torch.empty(out_dim, device="cuda")
    rt.launch_matvec_xq8(w2, xq, y3)
    torch.cuda.synchronize()
    assert torch.equal(y1, y2)
    assert torch.equal(y3, y1 * 2)


def test_argument_errors_leave_context_usable(rt):
    from reinstinct_b200 import _lib
    t, in_dim, out_dim = ro.Q4_K, 256, 8
    raw, x = cases.synth_case(t, in_dim, out_dim, 1, seed=9)
    w = rt.GpuMatvecTensor.from_bytes_matvec(raw, t, in_dim, out_dim)
    xq = torch.zeros(8 * 40, dtype=torch.uint8, device="cuda")
    y = torch.zeros(out_dim, device="cuda")
    with pytest.raises(_lib.RcError) as ei:
        rt.launch_matvec_batched(w, xq, y, 17)
    assert ei.value.code == -5
    bad = rt.GpuMatvecTensor(w.data, 99, in_dim, out_dim)
    with pytest.raises(_lib.RcError):
        rt.launch_matvec_xq8(bad, xq, y)
    rt.launch_matvec_xq8(w, xq, y)  # still works afterwards
    torch.cuda.synchronize()


@pytest.mark.parametrize("t", ro.ALL_TYPES)
def test_leftover_rows_of_a_mostly_empty_last_round(rt, t):
    """More rows than one-row-per-warp slots of the whole GPU, by a few: the leftover rows are dealt one per CTA and the
    CTA's warps take a group of the row each (matvec_rows_kernel's TAIL instantiation).  6144 columns are two groups in
    every format.  Against the oracle, row by row: the shared rows are the last ones."""
    props = torch.cuda.get_device_properties(0)
    slots = props.multi_processor_count * 4 * 8        # one-row warps resident at four CTAs of eight warps per SM
    in_dim, out_dim = 6144, slots + 164
    raw, x = cases.synth_case(t, in_dim, out_dim, 1, seed=900 + t)
    w = rt.GpuMatvecTensor.from_bytes_matvec(raw, t, in_dim, out_dim)
    xq_ref = ro.quantize_q8(x)
    xq = torch.from_numpy(xq_ref).cuda()
    y = torch.full((1, out_dim), float("nan"), device="cuda")
    rt.launch_matvec_xq8(w, xq, y)
    torch.cuda.synchronize()
    _, y64, _ = ro.matvec_q8(t, ro.repack(t, raw, in_dim, out_dim), xq_ref, in_dim, out_dim, 1)
    got = y.cpu().numpy().reshape(-1)
    want = np.asarray(y64, dtype=np.float64).reshape(-1)
    assert np.isfinite(got).all()
    assert ro.rel_l2(got[:slots], want[:slots]) < 1e-5
    assert ro.rel_l2(got[slots:], want[slots:]) < 1e-5   # the shared rows
    y2 = torch.empty_like(y)
    rt.launch_matvec_xq8(w, xq, y2)
    torch.cuda.synchronize()
    assert torch.equal(y, y2)
