"""GPU side of the relabelled source formats: rc_repack_for_matvec on Q3_K / IQ4_NL / BF16 rows gives
byte for byte the planes the oracle builds, and the tensors run on the kernels of the type they
relabel onto."""
import numpy as np
import pytest
import torch

import oracle as ro

pytestmark = pytest.mark.gpu


def _src_rows(t, in_dim, out_dim, seed):
    rng = np.random.default_rng(seed)
    if t == ro.BF16:
        f = (rng.standard_normal(in_dim * out_dim) * 0.05).astype(np.float32)
        f[:40] = 0.0
        return (f.view(np.uint32) >> 16).astype(np.uint16).view(np.uint8)
    wpb, bpb = ro.SRC_BLOCK[t]
    n_blocks = in_dim * out_dim // wpb
    raw = rng.integers(0, 256, n_blocks * bpb, dtype=np.uint8).reshape(n_blocks, bpb)
    d = np.array([ro.f32_to_f16(0.002 * (1 + (i % 37)) * (-1) ** i) for i in range(n_blocks)], dtype=np.uint16)
    d_off = 108 if t == ro.Q3_K else 0
    raw[:, d_off:d_off + 2] = d.view(np.uint8).reshape(-1, 2)
    return raw.reshape(-1)


@pytest.mark.parametrize("t", [ro.Q3_K, ro.IQ4_NL, ro.BF16])
@pytest.mark.parametrize("in_dim,out_dim", [(256, 7), (1024, 33), (2048, 64), (2816, 20)])
def test_repack_of_source_types_is_byte_exact(rt, t, in_dim, out_dim):
    raw = _src_rows(t, in_dim, out_dim, seed=in_dim + out_dim + t)
    w = rt.GpuMatvecTensor.from_bytes_matvec(raw, t, in_dim, out_dim)
    assert w.dtype == ro.kernel_type(t)
    want = ro.repack_any(t, raw, in_dim, out_dim)
    assert np.array_equal(w.data.cpu().numpy(), want)


@pytest.mark.parametrize("t", [ro.Q3_K, ro.IQ4_NL, ro.BF16])
@pytest.mark.parametrize("n_rows", [1, 4, 40])
def test_relabelled_tensor_runs_on_its_kernels(rt, t, n_rows):
    """Decode matvec, batched matvec and the prefill GEMM on a relabelled tensor against the f64
    product of its DIRECT decode with the dequantized activations (BF16: of its Q8_0 requantization)."""
    in_dim, out_dim = 1024, 96
    raw = _src_rows(t, in_dim, out_dim, seed=99 + t)
    w = rt.GpuMatvecTensor.from_bytes_matvec(raw, t, in_dim, out_dim)
    x = np.random.default_rng(t).standard_normal((n_rows, in_dim)).astype(np.float32)
    y = rt.PrefillGemm().matmul(w, torch.from_numpy(x).cuda(), n_rows)
    torch.cuda.synchronize()
    direct = ro.dequantize_src(t, raw, in_dim * out_dim)
    if t == ro.BF16:
        direct = ro.dequantize(ro.Q8_0, ro.quantize_q8_0(direct), in_dim * out_dim)
    xd = ro.dequantize_q8(ro.quantize_q8(x), in_dim, n_rows).reshape(n_rows, in_dim).astype(np.float64)
    want = xd @ direct.reshape(out_dim, in_dim).astype(np.float64).T
    assert ro.rel_l2(y.cpu().numpy(), want) < (1e-5 if n_rows <= 16 else 1e-3)


def test_source_type_arguments(rt):
    lib = rt._lib.load()
    assert lib.rc_kernel_type(11) == 14 and lib.rc_kernel_type(20) == 23 and lib.rc_kernel_type(30) == 8
    assert lib.rc_kernel_type(12) == 12 and lib.rc_kernel_type(10) == -1
    assert lib.rc_ondisk_len(11, 512, 3) == 3 * 2 * 110
    assert lib.rc_ondisk_len(20, 512, 3) == 3 * 16 * 18
    assert lib.rc_ondisk_len(30, 512, 3) == 3 * 512 * 2
    assert lib.rc_ondisk_len(11, 384, 3) == 0 and lib.rc_ondisk_len(20, 384, 3) == 0
    assert lib.rc_repack_for_matvec(None, 10, 16, 256, 1, 16) == -1
    assert lib.rc_repack_for_matvec(None, 11, 16, 384, 1, 16) == -2
