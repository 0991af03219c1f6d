"""The multi-GPU code paths on ONE device: G logical ranks, as the reference tests its two-stage pipeline
with both stages on device 0 (tests/qwen35_pipeline.rs:8-10).  The push all-gather runs as one cooperative
launch with a CTA per rank (separate launches that wait on one another are never run on one GPU); the
row-sharded GEMM that gathers its own output runs shard after shard into G local output buffers; and the
bounded device wait is made to run out (a flag that nothing sets) to check the status word."""
import ctypes as C

import numpy as np
import pytest
import torch

import cases
import oracle as ro
from reinstinct_b200 import sharding as sh

pytestmark = pytest.mark.gpu


def _status(lib, clear=False) -> int:
    st = C.c_uint(0)
    fn = lib.rc_device_status_clear if clear else lib.rc_device_status
    assert fn(C.byref(st)) == 0
    return st.value


def _ptr_array(tensors):
    return (C.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


@pytest.mark.parametrize("world", [2, 4, 8])
def test_allgather_push_logical_ranks(rt, world):
    lib = rt._lib.load()
    _status(lib, clear=True)
    n_bytes = 21760 // 16 * 16 // world // 16 * 16 + 16  # about a BlockQ8 row of the 17408-wide intermediate per rank
    gathered = [torch.zeros(world * n_bytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
    flags = [torch.zeros(world, dtype=torch.int64, device="cuda") for _ in range(world)]
    epochs = [torch.zeros(1, dtype=torch.int64, device="cuda") for _ in range(world)]
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator(device="cuda").manual_seed(world)
    for rnd in range(3):  # new data every round over the same buffers and counters
        shards = [torch.randint(0, 256, (n_bytes,), dtype=torch.uint8, device="cuda", generator=g) for _ in range(world)]
        rc = lib.rc_allgather_push_logical(stream, _ptr_array(shards), n_bytes, _ptr_array(gathered), _ptr_array(flags),
                                           _ptr_array(epochs), world)
        assert rc == 0, lib.rc_error_string(rc)
        torch.cuda.synchronize()
        want = torch.cat(shards)
        for r in range(world):
            assert torch.equal(gathered[r], want), (rnd, r)
            assert int(epochs[r].item()) == rnd + 1
            assert bool((flags[r] == rnd + 1).all())
    assert _status(lib) == 0


@pytest.mark.parametrize("t", [ro.Q4_K, ro.Q6_K, ro.Q8_0])
@pytest.mark.parametrize("world", [2, 4])
def test_matmul_gather_logical_shards_equal_unsharded(rt, t, world):
    """Every logical rank runs its row shard through rc_matmul_gather with all G output buffers on this
    device: afterwards each buffer holds the unsharded product, bit for bit."""
    lib = rt._lib.load()
    in_dim, out_dim, p = 1024, 544, 70  # 17 units of 32 rows: uneven shards, partial tiles
    raw, x = cases.synth_case(t, in_dim, out_dim, p, seed=23 * t + world)
    xd = torch.from_numpy(x).cuda()
    w_full = rt.GpuMatvecTensor.from_bytes_matvec(raw, t, in_dim, out_dim)
    y_full, _ = rt.PrefillGemm().matmul_block_dots(w_full, xd, p)
    outs = [torch.full((p, out_dim), float("nan"), device="cuda") for _ in range(world)]
    scratch = torch.empty(lib.rc_matmul_scratch_bytes(in_dim, p), dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    for r in range(world):
        part, rows = sh.shard_raw_rows(raw, t, in_dim, out_dim, r, world)
        b, _ = sh.row_shard_range(out_dim, r, world)
        w = rt.GpuMatvecTensor.from_bytes_matvec(part.copy(), t, in_dim, rows)
        rc = lib.rc_matmul_gather(stream, t, w.data.data_ptr(), xd.data_ptr(), _ptr_array(outs), world, out_dim, b, in_dim, rows, p,
                                  scratch.data_ptr(), scratch.numel())
        assert rc == 0, lib.rc_error_string(rc)
    torch.cuda.synchronize()
    assert _status(lib) == 0
    for r in range(world):
        assert torch.equal(outs[r], y_full), r
    _, y64, _ = ro.matvec_q8(t, ro.repack(t, raw, in_dim, out_dim), ro.quantize_q8(x), in_dim, out_dim, p)
    assert ro.rel_l2(outs[0].cpu().numpy(), y64) < 2e-5


def test_peer_wait_runs_out_sets_status_and_clears(rt):
    """A rank whose peer never arrives: the wait gives up after its limit (200 ms), the kernel ends, the
    status word says so, the context stays usable, and rc_device_status_clear resets the word."""
    lib = rt._lib.load()
    _status(lib, clear=True)
    n_bytes = 256
    src = torch.arange(n_bytes, dtype=torch.uint8, device="cuda")
    mine = torch.zeros(2 * n_bytes, dtype=torch.uint8, device="cuda")
    absent = torch.zeros(2 * n_bytes, dtype=torch.uint8, device="cuda")  # stands in for the peer's mapped buffer
    flags = [torch.zeros(2, dtype=torch.int64, device="cuda") for _ in range(2)]
    epoch = torch.zeros(1, dtype=torch.int64, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.rc_allgather_push(stream, src.data_ptr(), n_bytes, _ptr_array([mine, absent]), _ptr_array(flags), epoch.data_ptr(), 0, 2)
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.equal(mine[:n_bytes], src)          # its own shard did arrive
    assert _status(lib) & 0x00FF0000                 # bit 16..23: the peer gather gave up
    assert _status(lib, clear=True) & 0x00FF0000     # read-and-clear returns it once more
    assert _status(lib) == 0
    # the barrier alone behaves the same, and the device is still usable afterwards
    rc = lib.rc_peer_barrier(stream, _ptr_array(flags), epoch.data_ptr(), 0, 2)
    assert rc == 0
    torch.cuda.synchronize()
    assert _status(lib, clear=True) & 0x00FF0000
    y = torch.ones(8, device="cuda") * 2
    assert float(y.sum()) == 16.0
