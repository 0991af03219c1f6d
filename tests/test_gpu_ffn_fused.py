"""The decode FFN as one cooperative launch (rc_ffn_decode) against the five-launch chain it replaces
(step_swiglu_ffn, src/runtime/qwen35.rs:2694-2707: quantize, gate, up, swiglu_q8, down): the intermediate quantizes to
the chain's BlockQ8 records (up to the last bit of a row sum, where the two split a row over warps differently), the
outputs agree within f32 association and with the CPU oracle's exact integer dots, and repeat bit for bit.  A rank
whose peer never arrives runs into its bounded wait."""
import ctypes as C

import numpy as np
import pytest
import torch

import cases
import oracle as ro

pytestmark = pytest.mark.gpu

F32_TOL = 1e-3


def _status(lib, clear=False) -> int:
    st = C.c_uint(0)
    fn = lib.rc_device_status_clear if clear else lib.rc_device_status
    assert fn(C.byref(st)) == 0
    return st.value


def _records_close(a: torch.Tensor, b: torch.Tensor) -> bool:
    """BlockQ8 streams equal up to what a last-bit difference of the f32 inputs can do: d and xsum within 1e-5
    relative, quants off by at most one step in at most 1 % of the places."""
    ra, rb = a.cpu().numpy().reshape(-1, 40), b.cpu().numpy().reshape(-1, 40)
    fa, fb = ra[:, :8].copy().view(np.float32), rb[:, :8].copy().view(np.float32)
    if not np.allclose(fa, fb, rtol=1e-5, atol=1e-6):
        return False
    dq = np.abs(ra[:, 8:].view(np.int8).astype(np.int32) - rb[:, 8:].view(np.int8).astype(np.int32))
    return int(dq.max()) <= 1 and float((dq != 0).mean()) < 0.01


def _chain(rt, gate, up, down, xd, ffn, out):
    u8 = dict(dtype=torch.uint8, device="cuda")
    xq = torch.empty((gate.in_dim // 32) * 40, **u8)
    hq = torch.empty((ffn // 32) * 40, **u8)
    yg, yu, y = torch.empty(ffn, device="cuda"), torch.empty(ffn, device="cuda"), torch.empty(out, device="cuda")
    rt.launch_ffn_decode(gate, up, down, xd, xq, yg, yu, hq, y)
    return hq, y


@pytest.mark.parametrize("tg,td,hidden,ffn,out", [
    (ro.Q4_K, ro.Q6_K, 5120, 17408, 5120),   # config 2: one warp per down row
    (ro.Q4_K, ro.Q6_K, 1024, 2048, 640),     # a small shard-like shape: eight warps share a down row
    (ro.Q8_0, ro.Q8_0, 2048, 1024, 300),
    (ro.Q6_K, ro.Q6_K, 1024, 3072, 96),
    (ro.Q4_0, ro.Q4_0, 1024, 1024, 2000),
])
def test_fused_ffn_equals_the_launch_chain(rt, tg, td, hidden, ffn, out):
    lib = rt._lib.load()
    _status(lib, clear=True)
    gate = rt.GpuMatvecTensor.from_bytes_matvec(cases.synth_case(tg, hidden, ffn, 1, seed=1)[0], tg, hidden, ffn)
    up = rt.GpuMatvecTensor.from_bytes_matvec(cases.synth_case(tg, hidden, ffn, 1, seed=2)[0], tg, hidden, ffn)
    raw_d = cases.synth_case(td, ffn, out, 1, seed=3)[0]
    down = rt.GpuMatvecTensor.from_bytes_matvec(raw_d, td, ffn, out)
    fused = rt.FusedFfnDecode(gate, up, down, ffn, out)
    for rnd in range(3):  # the counters grow call by call
        x = cases.synth_case(tg, hidden, 8, 1, seed=10 + rnd)[1]
        xd = torch.from_numpy(x).cuda().reshape(-1)
        hq_ref, y_ref = _chain(rt, gate, up, down, xd, ffn, out)
        fused.run(xd)
        h = torch.empty(ffn, device="cuda")
        y = torch.empty_like(y_ref)
        fused.read_h(h)
        fused.read_y(y)
        hq = torch.empty_like(hq_ref)
        rt.launch_quantize_q8(h, hq, ffn, 1)   # the records the kernel formed from h in shared memory
        torch.cuda.synchronize()
        assert _status(lib) == 0
        # (the two may split a row over warps differently: a sum then differs in the last bit, and a quant may land
        # on the other side of a rounding boundary)
        assert _records_close(hq, hq_ref), f"round {rnd}: intermediate records differ"
        a, b = y.cpu().numpy(), y_ref.cpu().numpy().astype(np.float64)
        assert ro.rel_l2(a, b) < F32_TOL, rnd
        # the down projection against the CPU oracle on the fused kernel's OWN records: exact integer dots
        _, y64, _ = ro.matvec_q8(td, ro.repack(td, raw_d, ffn, out), hq.cpu().numpy(), ffn, out, 1)
        assert ro.rel_l2(a, y64) < 1e-5, rnd


def test_fused_ffn_config2_repeats_bit_for_bit(rt):
    """The order of additions depends on the shapes only: two objects, two calls each, one set of bits."""
    tg, td, hidden, ffn, out = ro.Q4_K, ro.Q6_K, 5120, 17408, 5120
    gate = rt.GpuMatvecTensor.from_bytes_matvec(cases.synth_case(tg, hidden, ffn, 1, seed=4)[0], tg, hidden, ffn)
    up = rt.GpuMatvecTensor.from_bytes_matvec(cases.synth_case(tg, hidden, ffn, 1, seed=5)[0], tg, hidden, ffn)
    down = rt.GpuMatvecTensor.from_bytes_matvec(cases.synth_case(td, ffn, out, 1, seed=6)[0], td, ffn, out)
    xd = torch.from_numpy(cases.synth_case(tg, hidden, 8, 1, seed=7)[1]).cuda().reshape(-1)
    _, y_ref = _chain(rt, gate, up, down, xd, ffn, out)
    outs = []
    for _ in range(2):
        fused = rt.FusedFfnDecode(gate, up, down, ffn, out)
        for _ in range(2):
            fused.run(xd)
            y = torch.empty_like(y_ref)
            fused.read_y(y)
            torch.cuda.synchronize()
            outs.append(y)
    assert all(torch.equal(outs[0], o) for o in outs[1:])
    assert ro.rel_l2(outs[0].cpu().numpy(), y_ref.cpu().numpy().astype(np.float64)) < 1e-5


def test_fused_ffn_absent_peer_runs_into_the_bounded_wait(rt):
    """Rank 0 of two whose peer never runs: its own half of the records arrives, the wait for the rest gives up
    after its limit, the status word says which wait, and the device stays usable."""
    lib = rt._lib.load()
    _status(lib, clear=True)
    tg, td, hidden, ffn, out = ro.Q4_K, ro.Q6_K, 1024, 2048, 256
    half = ffn // 2
    gate = rt.GpuMatvecTensor.from_bytes_matvec(cases.synth_case(tg, hidden, half, 1, seed=1)[0], tg, hidden, half)
    up = rt.GpuMatvecTensor.from_bytes_matvec(cases.synth_case(tg, hidden, half, 1, seed=2)[0], tg, hidden, half)
    down = rt.GpuMatvecTensor.from_bytes_matvec(cases.synth_case(td, ffn, out // 2, 1, seed=3)[0], td, ffn, out // 2)
    xd = torch.from_numpy(cases.synth_case(tg, hidden, 8, 1, seed=9)[1]).cuda().reshape(-1)
    mine = torch.full((3 * ffn * 4 + 3 * out * 4,), 0xFF, dtype=torch.uint8, device="cuda")
    absent = mine.clone()  # stands in for the peer's mapped buffers
    h_off, y_off = 0, 3 * ffn * 4
    arr = lambda off: (C.c_void_p * 2)(mine.data_ptr() + off, absent.data_ptr() + off)
    work = torch.zeros(lib.rc_ffn_decode_work_bytes(half), dtype=torch.uint8, device="cuda")
    y = torch.zeros(out, device="cuda")
    rc = lib.rc_ffn_decode(torch.cuda.current_stream().cuda_stream, tg, td, gate.data.data_ptr(), up.data.data_ptr(),
                           down.data.data_ptr(), xd.data_ptr(), y.data_ptr(), hidden, half, ffn, 0, out // 2, out, 0, 2, 0,
                           arr(h_off), arr(y_off), work.data_ptr())
    assert rc == 0, lib.rc_error_string(rc)
    torch.cuda.synchronize()
    st = _status(lib, clear=True)
    assert (st >> 20) & 0xF == 2, hex(st)      # the wait for the peers' share of the intermediate
    assert _status(lib) == 0
    # its own half of the intermediate did arrive, here and at the "peer" (the first call uses copy 1), the rest did not
    for buf in (mine, absent):
        h = buf[h_off:h_off + 3 * ffn * 4].view(torch.int32).reshape(3, ffn)
        assert bool((h[1, :half] != -1).all()) and bool((h[1, half:] == -1).all())
    assert float((torch.ones(4, device="cuda") * 3).sum()) == 12.0


@pytest.mark.parametrize("tg,td,hidden,ffn,out", [
    (ro.Q4_K, ro.Q6_K, 5120, 17408, 5120),   # config 2
    (ro.Q4_K, ro.Q6_K, 1024, 2304, 640),     # 72 sub-blocks: the last 1024-wide iteration of a down row is a quarter full
    (ro.Q4_K, ro.Q6_K, 1024, 6144, 4000),    # two full rounds of down rows, then 448 leftover rows walked by four warps each
    (ro.Q4_K, ro.Q6_K, 1024, 2048, 300),
    (ro.Q8_0, ro.Q8_0, 2048, 1056, 300),     # 33 sub-blocks
    (ro.Q6_K, ro.Q6_K, 1024, 256, 2000),     # one superblock per down row
    (ro.Q4_0, ro.Q4_0, 1024, 1024, 96),
])
def test_tensor_parallel_ffn_world_of_one_equals_the_launch_chain(rt, tg, td, hidden, ffn, out):
    """rc_ffn_decode_tp with one rank: the slice of the contraction is the whole of it.  Against the launch chain (f32
    association) and against the CPU oracle's exact integer dots on the chain's own records."""
    lib = rt._lib.load()
    _status(lib, clear=True)
    gate = rt.GpuMatvecTensor.from_bytes_matvec(cases.synth_case(tg, hidden, ffn, 1, seed=1)[0], tg, hidden, ffn)
    up = rt.GpuMatvecTensor.from_bytes_matvec(cases.synth_case(tg, hidden, ffn, 1, seed=2)[0], tg, hidden, ffn)
    raw_d = cases.synth_case(td, ffn, out, 1, seed=3)[0]
    down = rt.GpuMatvecTensor.from_bytes_matvec(raw_d, td, ffn, out)
    tp = rt.TensorParallelFfnDecode(gate, up, down)
    outs = []
    for rnd in range(4):  # the three copies of the partial buffer take turns
        x = cases.synth_case(tg, hidden, 8, 1, seed=10 + rnd % 2)[1]
        xd = torch.from_numpy(x).cuda().reshape(-1)
        hq_ref, y_ref = _chain(rt, gate, up, down, xd, ffn, out)
        tp.run(xd)
        y = torch.empty_like(y_ref)
        tp.read_y(y)
        torch.cuda.synchronize()
        assert _status(lib) == 0, rnd
        a = y.cpu().numpy()
        # (a last-bit difference between the two forms' gate/up row sums may move a quant of the intermediate across a
        # rounding boundary: 5e-4 allows a few such, a wrong block or scale would be 1e-2 and more)
        assert ro.rel_l2(a, y_ref.cpu().numpy().astype(np.float64)) < 5e-4, rnd
        _, y64, _ = ro.matvec_q8(td, ro.repack(td, raw_d, ffn, out), hq_ref.cpu().numpy(), ffn, out, 1)
        assert ro.rel_l2(a, y64) < 5e-4, rnd
        outs.append(y)
    assert torch.equal(outs[0], outs[2]) and torch.equal(outs[1], outs[3])  # same input, same bits
    tp.close()


def test_tensor_parallel_ffn_absent_peer_runs_into_the_bounded_wait(rt):
    """Rank 0 of two whose peer never runs: its own partial sums arrive in both partial buffers, the peer's never do,
    the read of the output rows gives up after its limit, the status word says which wait, the device stays usable."""
    lib = rt._lib.load()
    _status(lib, clear=True)
    tg, td, hidden, ffn, out = ro.Q4_K, ro.Q6_K, 1024, 2048, 256
    half = ffn // 2
    gate = rt.GpuMatvecTensor.from_bytes_matvec(cases.synth_case(tg, hidden, half, 1, seed=1)[0], tg, hidden, half)
    up = rt.GpuMatvecTensor.from_bytes_matvec(cases.synth_case(tg, hidden, half, 1, seed=2)[0], tg, hidden, half)
    down = rt.GpuMatvecTensor.from_bytes_matvec(cases.synth_case(td, half, out, 1, seed=3)[0], td, half, out)
    xd = torch.from_numpy(cases.synth_case(tg, hidden, 8, 1, seed=9)[1]).cuda().reshape(-1)
    mine = torch.full((3 * 2 * out * 4,), 0xFF, dtype=torch.uint8, device="cuda")
    absent = mine.clone()  # stands in for the peer's mapped buffer
    parts = (C.c_void_p * 2)(mine.data_ptr(), absent.data_ptr())
    work = torch.zeros(lib.rc_ffn_decode_tp_work_bytes(half), dtype=torch.uint8, device="cuda")
    y = torch.zeros(out, device="cuda")
    rc = lib.rc_ffn_decode_tp(torch.cuda.current_stream().cuda_stream, tg, td, gate.data.data_ptr(), up.data.data_ptr(),
                              down.data.data_ptr(), xd.data_ptr(), y.data_ptr(), hidden, half, out, 2, 0, parts, work.data_ptr())
    assert rc == 0, lib.rc_error_string(rc)
    torch.cuda.synchronize()
    st = _status(lib, clear=True)
    assert (st >> 20) & 0xF == 3, hex(st)      # the wait for the peers' partial sums
    assert _status(lib) == 0
    for buf in (mine, absent):                 # the first call uses copy 1: slot 0 (this rank) filled, slot 1 still empty
        p = buf.view(torch.int32).reshape(3, 2, out)
        assert bool((p[1, 0] != -1).all()) and bool((p[1, 1] == -1).all())
    assert float((torch.ones(4, device="cuda") * 3).sum()) == 12.0


def test_copy_small_moves_bytes_between_pinned_host_and_device(rt):
    """rc_copy_small: the kernel-side upload / download of a step's few KB (a memcpy node costs more in a replayed graph)."""
    lib = rt._lib.load()
    host = torch.arange(5120, dtype=torch.float32).pin_memory()
    dev = torch.zeros(5120, device="cuda")
    back = torch.zeros(5120, dtype=torch.float32).pin_memory()
    rt.copy_small(dev, host, 5120 * 4)
    rt.copy_small(back, dev, 5120 * 4)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        rt.copy_small(dev, host, 5120 * 4)
        rt.copy_small(back, dev, 5120 * 4)
    torch.cuda.synchronize()
    assert torch.equal(back, host) and torch.equal(dev.cpu(), host)
    host.mul_(2.0)
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(back, host)
    st = torch.cuda.current_stream().cuda_stream
    assert lib.rc_copy_small(st, dev.data_ptr(), host.data_ptr(), 20) == -2          # not a multiple of 16 bytes: RC_ERR_BAD_SHAPE
    assert lib.rc_copy_small(st, dev.data_ptr() + 4, host.data_ptr(), 16) == -4      # RC_ERR_MISALIGNED
    assert lib.rc_copy_small(st, 0, host.data_ptr(), 16) == -3                       # RC_ERR_NULL_POINTER
