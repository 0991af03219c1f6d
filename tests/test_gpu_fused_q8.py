"""GPU parity of the fused BlockQ8 producers (rmsnorm_q8, add_rmsnorm_q8, swiglu_q8) through the C ABI."""
import numpy as np
import pytest
import torch

import oracle as ro

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,n_vec", [(32, 1), (2048, 1), (5120, 3), (17408, 2), (8192 + 64, 1)])
@pytest.mark.parametrize("with_add", [False, True])
def test_rmsnorm_q8_bit_exact(rt, n, n_vec, with_add):
    """Every arithmetic step is an IEEE operation in a fixed order, so the records, the f32 output and
    the updated residual all equal the oracle's bit for bit."""
    rng = np.random.default_rng(n + n_vec)
    x = (rng.standard_normal((n_vec, n)) * 2).astype(np.float32)
    add = rng.standard_normal((n_vec, n)).astype(np.float32)
    w = (rng.random(n) + 0.5).astype(np.float32)
    if n >= 64:
        x[0, 32:64] = 0.0
        add[0, 32:64] = 0.0           # an all-zero sub-block: d = 1, qs = 0
    eps = 1e-6
    hid_w, y_w, q_w = ro.rmsnorm_q8(x, w, eps, add if with_add else None)
    out = torch.zeros(n_vec * (n // 32) * 40, dtype=torch.uint8, device="cuda")
    wd = torch.from_numpy(w).cuda()
    if with_add:
        hid = torch.from_numpy(x).cuda()
        y = torch.full((n_vec, n), float("nan"), device="cuda")
        rt.launch_add_rmsnorm_q8(hid, torch.from_numpy(add).cuda(), wd, y, out, n, n_vec, eps)
        torch.cuda.synchronize()
        np.testing.assert_array_equal(hid.cpu().numpy().view(np.uint32), hid_w.view(np.uint32))
        np.testing.assert_array_equal(y.cpu().numpy().view(np.uint32), y_w.view(np.uint32))
    else:
        rt.launch_rmsnorm_q8(torch.from_numpy(x).cuda(), wd, out, n, n_vec, eps)
        torch.cuda.synchronize()
    np.testing.assert_array_equal(out.cpu().numpy(), q_w)


def test_add_rmsnorm_q8_without_add_or_y(rt):
    n = 1024
    rng = np.random.default_rng(3)
    x = rng.standard_normal((1, n)).astype(np.float32)
    w = np.ones(n, dtype=np.float32)
    hid = torch.from_numpy(x).cuda()
    out = torch.zeros((n // 32) * 40, dtype=torch.uint8, device="cuda")
    rt.launch_add_rmsnorm_q8(hid, None, torch.from_numpy(w).cuda(), None, out, n, 1, 1e-5)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(hid.cpu().numpy(), x)               # untouched
    np.testing.assert_array_equal(out.cpu().numpy(), ro.rmsnorm_q8(x, w, 1e-5)[2])


@pytest.mark.parametrize("n", [32, 4096, 17408 * 3])
def test_swiglu_q8_matches_oracle(rt, n):
    rng = np.random.default_rng(n)
    g = (rng.standard_normal(n) * 3).astype(np.float32)
    u = rng.standard_normal(n).astype(np.float32)
    v_w, q_w = ro.swiglu_q8(g, u)
    out = torch.full((n,), float("nan"), device="cuda")
    q8 = torch.zeros(n // 32 * 40, dtype=torch.uint8, device="cuda")
    rt.launch_swiglu_q8(torch.from_numpy(g).cuda(), torch.from_numpy(u).cuda(), out, q8, n)
    torch.cuda.synchronize()
    v = out.cpu().numpy()
    # expf differs by an ulp or two between the device and the host libm
    np.testing.assert_allclose(v, v_w, rtol=4e-6, atol=1e-9)
    # the records are the quantizer's for the device's own f32 values
    np.testing.assert_array_equal(q8.cpu().numpy(), ro.quantize_q8(v.reshape(1, -1)))
    a, b = q8.cpu().numpy().reshape(-1, 40)[:, 8:].view(np.int8).astype(int), q_w.reshape(-1, 40)[:, 8:].view(np.int8).astype(int)
    assert np.abs(a - b).max() <= 1 and (a != b).mean() < 2e-3


def test_fused_q8_feeds_the_matvec(rt):
    """rmsnorm_q8 output is consumed as-is by rc_matvec: same result as quantize_q8 of the oracle's y."""
    import cases
    t, in_dim, out_dim = ro.Q4_K, 2048, 128
    raw, x = cases.synth_case(t, in_dim, out_dim, 1, seed=8)
    w_norm = (np.random.default_rng(1).random(in_dim) + 0.5).astype(np.float32)
    wt = rt.GpuMatvecTensor.from_bytes_matvec(raw, t, in_dim, out_dim)
    xq = torch.zeros((in_dim // 32) * 40, dtype=torch.uint8, device="cuda")
    rt.launch_rmsnorm_q8(torch.from_numpy(x).cuda(), torch.from_numpy(w_norm).cuda(), xq, in_dim, 1, 1e-6)
    y = torch.empty(out_dim, device="cuda")
    rt.launch_matvec_xq8(wt, xq, y)
    torch.cuda.synchronize()
    _, _, q = ro.rmsnorm_q8(x, w_norm, 1e-6)
    _, y64, _ = ro.matvec_q8(t, ro.repack(t, raw, in_dim, out_dim), q, in_dim, out_dim, 1)
    assert ro.rel_l2(y.cpu().numpy(), y64) < 1e-5


@pytest.mark.parametrize("n", [32, 6144])
def test_sigmoid_mul_q8_matches_oracle(rt, n):
    rng = np.random.default_rng(n + 1)
    x = rng.standard_normal(n).astype(np.float32)
    g = (rng.standard_normal(n) * 3).astype(np.float32)
    v_w, q_w = ro.sigmoid_mul_q8(x, g)
    xd = torch.from_numpy(x.copy()).cuda()
    q8 = torch.zeros(n // 32 * 40, dtype=torch.uint8, device="cuda")
    rt.launch_sigmoid_mul_q8(xd, torch.from_numpy(g).cuda(), q8, n)
    torch.cuda.synchronize()
    v = xd.cpu().numpy()
    np.testing.assert_allclose(v, v_w, rtol=4e-6, atol=1e-9)                        # expf: device vs host libm
    np.testing.assert_array_equal(q8.cpu().numpy(), ro.quantize_q8(v.reshape(1, -1)))   # records of the device's own values


@pytest.mark.parametrize("n_heads,head_dim", [(1, 32), (16, 128), (48, 128), (3, 1024)])
def test_rmsnorm_gated_q8_matches_oracle(rt, n_heads, head_dim):
    rng = np.random.default_rng(n_heads * head_dim)
    x = (rng.standard_normal((n_heads, head_dim)) * 2).astype(np.float32)
    z = (rng.standard_normal((n_heads, head_dim)) * 2).astype(np.float32)
    w = (rng.random(head_dim) + 0.5).astype(np.float32)
    y_w, q_w = ro.rmsnorm_gated_q8(x, z, w, 1e-6)
    y = torch.full((n_heads, head_dim), float("nan"), device="cuda")
    q8 = torch.zeros(n_heads * head_dim // 32 * 40, dtype=torch.uint8, device="cuda")
    rt.launch_rmsnorm_gated_q8(torch.from_numpy(x).cuda(), torch.from_numpy(z).cuda(), torch.from_numpy(w).cuda(), y, q8,
                               n_heads, head_dim, 1e-6)
    torch.cuda.synchronize()
    yv = y.cpu().numpy()
    np.testing.assert_allclose(yv, y_w, rtol=4e-6, atol=1e-9)
    np.testing.assert_array_equal(q8.cpu().numpy(), ro.quantize_q8(yv.reshape(1, -1)))
    x64, z64 = x.astype(np.float64), z.astype(np.float64)
    ref = x64 / np.sqrt((x64 ** 2).mean(1, keepdims=True) + 1e-6) * w * (z64 / (1 + np.exp(-z64)))
    np.testing.assert_allclose(yv, ref, rtol=1e-5, atol=1e-6)
