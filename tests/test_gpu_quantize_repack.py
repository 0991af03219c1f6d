"""GPU parity: quantize_q8 (bit-exact BlockQ8 bytes) and the on-device repack (bit-exact
planes), through the C ABI."""
import numpy as np
import pytest
import torch

import cases
import oracle as ro

pytestmark = pytest.mark.gpu


def _quantize(rt, x: np.ndarray) -> np.ndarray:
    n_vec, in_dim = x.shape
    xd = torch.from_numpy(x).cuda()
    out = torch.empty(n_vec * (in_dim // 32) * 40, dtype=torch.uint8, device="cuda")
    rt.launch_quantize_q8(xd, out, in_dim, n_vec)
    torch.cuda.synchronize()
    return out.cpu().numpy()


@pytest.mark.parametrize("n_vec,in_dim", [(1, 32), (1, 4096), (1, 5120), (4, 5120), (3, 17408), (70, 2048), (512, 5120)])
def test_quantize_q8_bit_exact(rt, n_vec, in_dim):
    x = np.random.default_rng(n_vec * 7 + in_dim).standard_normal((n_vec, in_dim)).astype(np.float32)
    assert np.array_equal(_quantize(rt, x), ro.quantize_q8(x))


def test_quantize_q8_edge_values(rt):
    x = np.random.default_rng(11).standard_normal((2, 512)).astype(np.float32)
    x[0, 0:32] = 0.0                      # amax == 0 -> d = 1, q = 0
    x[0, 32] = 3.0e38                     # near f32 max
    x[0, 64:96] = 1e-42                   # subnormal inputs
    x[1, 0] = 127.0
    x[1, 1:5] = [0.5, 1.5, 2.5, -0.5]     # ties -> even
    x[1, 5:32] = 0.0
    x[1, 100] = -0.0
    got = _quantize(rt, x)
    assert np.array_equal(got, ro.quantize_q8(x))
    q = got.reshape(-1, 40)[16, 8:].view(np.int8)
    assert list(q[:5]) == [127, 0, 2, 2, 0]


def test_quantize_q8_lcg_case(rt):
    """The activation stream of the reference's kernel tests (src/runtime/kernels.rs:3046-3049)."""
    x = cases.lcg_x(2048, 0x13579BDF).reshape(1, -1)
    assert np.array_equal(_quantize(rt, x), ro.quantize_q8(x))


def test_quantize_q8_rejects_bad_shapes(rt):
    x = torch.zeros(64, device="cuda")
    out = torch.zeros(80, dtype=torch.uint8, device="cuda")
    from reinstinct_b200 import _lib
    lib = _lib.load()
    assert lib.rc_quantize_q8(None, x.data_ptr(), out.data_ptr(), 48, 1) == -2
    assert lib.rc_quantize_q8(None, x.data_ptr(), out.data_ptr() + 4, 32, 1) == -4
    assert lib.rc_quantize_q8(None, x.data_ptr(), out.data_ptr(), 32, 0) == 0


@pytest.mark.parametrize("t", ro.ALL_TYPES)
@pytest.mark.parametrize("in_dim,out_dim", [(256, 1), (512, 3), (1024, 5), (2048, 384), (5120, 64), (8192, 7)])
def test_repack_bit_exact(rt, t, in_dim, out_dim):
    """rc_repack_for_matvec == quant::<fmt>::repack_for_matvec, including the pad sub-block of
    power-of-two rows (512, 1024, 2048, 8192 here) and odd out_dim."""
    raw = cases.lcg_case(t, in_dim, out_dim, seed=0xA5A5 + t + in_dim) if in_dim <= 1024 else \
        cases.synth_case(t, in_dim, out_dim, 1, seed=t + in_dim)[0]
    w = rt.GpuMatvecTensor.from_bytes_matvec(raw, t, in_dim, out_dim)
    assert np.array_equal(w.data.cpu().numpy(), ro.repack(t, raw, in_dim, out_dim))


def test_repack_iq4xs_subnormal_scale_truncates(rt):
    """d*(ls-32) in the binary16 subnormal range: the folded scale is truncated, not rounded,
    as src/quant/half.rs:70-74 does."""
    t, in_dim, out_dim = ro.IQ4_XS, 256, 4
    raw = cases.synth_case(t, in_dim, out_dim, 1, seed=3)[0].reshape(-1, 136).copy()
    for i, d in enumerate([3.1e-7, 9.0e-7, 2.3e-6, 6.0e-8]):
        raw[i, 0:2] = np.frombuffer(np.float16(d).tobytes(), dtype=np.uint8)
    raw = raw.reshape(-1)
    w = rt.GpuMatvecTensor.from_bytes_matvec(raw, t, in_dim, out_dim)
    assert np.array_equal(w.data.cpu().numpy(), ro.repack(t, raw, in_dim, out_dim))
