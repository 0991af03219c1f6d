"""rc_matvec_f32_noalloc through the C ABI: the variant of rc_matvec_f32 for callers that cannot
provide (or allocate) the quantized-activation scratch.  It must give what rc_matvec_f32 gives
with a caller-owned scratch, on two calls in a row that share the library's fixed array — the
second with a shorter activation vector, so stale bytes of the first call sit behind it.
Collected last on purpose: a failure here cannot hide any other test's result."""
import ctypes as C

import numpy as np
import pytest
import torch

import cases
import oracle as ro

pytestmark = pytest.mark.gpu

F32_TOL = 1e-3  # the tolerance of the other matvec parity tests


def _both(rt, lib, t, in_dim, out_dim, seed):
    raw, x = cases.synth_case(t, in_dim, out_dim, 1, seed=seed)
    w = rt.GpuMatvecTensor.from_bytes_matvec(raw, t, in_dim, out_dim)
    xd = torch.from_numpy(x).cuda()
    stream = torch.cuda.current_stream().cuda_stream
    y_ref = torch.full((out_dim,), float("nan"), device="cuda")
    xq = torch.empty((in_dim // 32) * 40, dtype=torch.uint8, device="cuda")
    rt.launch_matvec(w, xd, y_ref, xq)
    y_new = torch.full((out_dim,), float("nan"), device="cuda")
    rc = lib.rc_matvec_f32_noalloc(stream, t, w.data.data_ptr(), xd.data_ptr(), y_new.data_ptr(), in_dim, out_dim)
    assert rc == 0, lib.rc_error_string(rc)
    torch.cuda.synchronize()
    a, b = y_new.cpu().numpy(), y_ref.cpu().numpy()
    assert np.isfinite(a).all()
    assert ro.rel_l2(a, b.astype(np.float64)) < F32_TOL
    # and against the CPU oracle, like every other matvec test
    _, y64, _ = ro.matvec_q8(t, ro.repack(t, raw, in_dim, out_dim), ro.quantize_q8(x), in_dim, out_dim, 1)
    assert ro.rel_l2(a, y64) < F32_TOL


def test_noalloc_matches_scratch_variant_twice(rt):
    from reinstinct_b200 import _lib

    lib = _lib.load()
    _both(rt, lib, ro.Q4_K, 5120, 640, seed=901)   # first call on the device: looks the array up
    _both(rt, lib, ro.Q6_K, 2048, 300, seed=902)   # second call: shorter x over the same array


def test_noalloc_rejects_oversize(rt):
    from reinstinct_b200 import _lib

    lib = _lib.load()
    big = 52416 + 32  # RC_NOALLOC_MAX_IN_DIM + one block
    one = torch.zeros(16, dtype=torch.uint8, device="cuda")
    rc = lib.rc_matvec_f32_noalloc(0, ro.Q8_0, one.data_ptr(), one.data_ptr(), one.data_ptr(), big, 1)
    assert rc == -9
    assert b"RC_NOALLOC_MAX_IN_DIM" in lib.rc_error_string(rc)
