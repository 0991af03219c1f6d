"""GPU parity of the expert-grouped f16-operand GEMM (rc_mmq_gemm_grouped_f32) against the oracle's
exact-integer grouped GEMM: gate/up addressing (token rows gathered through the sort's perm) and down
addressing (gated activation of the gate_up output applied on the fly)."""
import ctypes

import numpy as np
import pytest
import torch

import cases
import oracle as ro

pytestmark = pytest.mark.gpu

EXPECTED = 6e-4   # two f16 roundings; the bar is the reference's 1e-3


def _status(lib) -> int:
    st = ctypes.c_uint(0)
    assert lib.rc_device_status(ctypes.byref(st)) == 0
    return st.value


def _setup(rt, t, in_dim, out_dim, n_expert, n_tok, n_used, seed):
    rng = np.random.default_rng(seed)
    n_entries = n_tok * n_used
    ids = rng.integers(0, max(n_expert - 2, 1), n_entries, dtype=np.int32)   # the last experts stay empty
    ids[:min(70, n_entries)] = min(3, n_expert - 1)                          # one expert spans several tiles
    raws = [cases.synth_case(t, in_dim, out_dim, 1, seed=100 * t + e)[0] for e in range(n_expert)]
    et = rt.GpuExpertTensor.from_bytes(np.concatenate(raws), t, in_dim, out_dim, n_expert)
    slab = np.concatenate([ro.repack(t, r, in_dim, out_dim) for r in raws])
    moe = rt.MoeGroupedScratch.new(n_expert, n_entries)
    rt.launch_moe_sort(moe, torch.from_numpy(ids).cuda(), n_entries)
    torch.cuda.synchronize()
    return rng, n_entries, et, slab, moe


@pytest.mark.parametrize("t", ro.ALL_TYPES)
@pytest.mark.parametrize("in_dim,out_dim", [(1024, 304), (256, 128)])
def test_grouped_gate_up_addressing(rt, t, in_dim, out_dim):
    n_expert, n_tok, n_used = 12, 48, 4
    rng, n_entries, et, slab, moe = _setup(rt, t, in_dim, out_dim, n_expert, n_tok, n_used, seed=t)
    x = rng.standard_normal((n_tok, in_dim)).astype(np.float32)
    y = torch.full((n_entries, out_dim), float("nan"), device="cuda")
    rt.MoeGroupedGemm().gate_up(moe, et, torch.from_numpy(x).cuda(), n_used, y, n_entries)
    torch.cuda.synchronize()
    assert _status(rt._lib.load()) == 0
    perm = moe.perm.cpu().numpy()[:n_entries]
    xq_sorted = ro.quantize_q8(x[perm // n_used])
    _, y64 = ro.grouped_q8(t, slab, et.bytes_per_expert, moe.expert_off.cpu().numpy(), xq_sorted, in_dim, out_dim)
    assert ro.rel_l2(y.cpu().numpy(), y64) < EXPECTED


@pytest.mark.parametrize("t", [ro.Q4_K, ro.Q6_K, ro.Q8_0])
@pytest.mark.parametrize("act", [0, 1])
def test_grouped_down_addressing_with_activation(rt, t, act):
    ff, hidden, n_expert, n_tok, n_used = 512, 192, 9, 40, 3
    rng, n_entries, et, slab, moe = _setup(rt, t, ff, hidden, n_expert, n_tok, n_used, seed=10 + t + act)
    gu = (rng.standard_normal((n_entries, 2 * ff)) * 2).astype(np.float32)   # gate_up output, sorted order
    y = torch.full((n_entries, hidden), float("nan"), device="cuda")
    rt.MoeGroupedGemm().down(moe, et, torch.from_numpy(gu).cuda(), act, y, n_entries)
    torch.cuda.synchronize()
    assert _status(rt._lib.load()) == 0
    aq, _ = ro.moe_act_q8(gu, act)
    _, y64 = ro.grouped_q8(t, slab, et.bytes_per_expert, moe.expert_off.cpu().numpy(), aq.reshape(-1), ff, hidden)
    assert ro.rel_l2(y.cpu().numpy(), y64) < EXPECTED


def test_grouped_many_tiles_per_cta(rt):
    """More tiles than SMs: 64 experts x 8 row tiles, the sixteen accumulator buffers wrap many times."""
    t, in_dim, out_dim, n_expert, n_tok, n_used = ro.Q4_K, 256, 1024, 64, 256, 4
    rng, n_entries, et, slab, moe = _setup(rt, t, in_dim, out_dim, n_expert, n_tok, n_used, seed=77)
    x = rng.standard_normal((n_tok, in_dim)).astype(np.float32)
    y = torch.full((n_entries, out_dim), float("nan"), device="cuda")
    rt.MoeGroupedGemm().gate_up(moe, et, torch.from_numpy(x).cuda(), n_used, y, n_entries)
    torch.cuda.synchronize()
    assert _status(rt._lib.load()) == 0
    perm = moe.perm.cpu().numpy()[:n_entries]
    _, y64 = ro.grouped_q8(t, slab, et.bytes_per_expert, moe.expert_off.cpu().numpy(), ro.quantize_q8(x[perm // n_used]),
                           in_dim, out_dim)
    assert ro.rel_l2(y.cpu().numpy(), y64) < EXPECTED


@pytest.mark.parametrize("t", [ro.Q4_K, ro.Q6_K])
def test_grouped_gate_up_with_dropped_entries(rt, t):
    """Ids outside the experts (and -1, the mark of an unused slot) are dropped by the
    sort: perm carries -1 for the slots past the routed total, and the f32 prologue must treat those as zero rows instead
    of reading a row at index 0xFFFFFFFF / n_used.  The kept entries equal the oracle's, nothing else is touched."""
    in_dim, out_dim, n_expert, n_tok, n_used = 512, 256, 8, 40, 2
    rng = np.random.default_rng(50 + t)
    n_entries = n_tok * n_used
    ids = rng.integers(0, n_expert, n_entries, dtype=np.int32)
    ids[::9] = -1
    ids[4::13] = n_expert + 3
    n_kept = int(((ids >= 0) & (ids < n_expert)).sum())
    raws = [cases.synth_case(t, in_dim, out_dim, 1, seed=200 * t + e)[0] for e in range(n_expert)]
    et = rt.GpuExpertTensor.from_bytes(np.concatenate(raws), t, in_dim, out_dim, n_expert)
    slab = np.concatenate([ro.repack(t, r, in_dim, out_dim) for r in raws])
    moe = rt.MoeGroupedScratch.new(n_expert, n_entries)
    rt.launch_moe_sort(moe, torch.from_numpy(ids).cuda(), n_entries)
    x = rng.standard_normal((n_tok, in_dim)).astype(np.float32)
    y = torch.full((n_entries, out_dim), float("nan"), device="cuda")
    rt.MoeGroupedGemm().gate_up(moe, et, torch.from_numpy(x).cuda(), n_used, y, n_entries)
    torch.cuda.synchronize()
    assert _status(rt._lib.load()) == 0
    expert_off = moe.expert_off.cpu().numpy()
    perm = moe.perm.cpu().numpy()[:n_entries]
    assert int(expert_off[n_expert]) == n_kept and (perm[:n_kept] >= 0).all() and (perm[n_kept:] == -1).all()
    _, y64 = ro.grouped_q8(t, slab, et.bytes_per_expert, expert_off, ro.quantize_q8(x[perm[:n_kept] // n_used]), in_dim, out_dim)
    got = y.cpu().numpy()
    assert np.isfinite(got[:n_kept]).all()
    assert ro.rel_l2(got[:n_kept], y64) < EXPECTED
    assert float((torch.ones(4, device="cuda") * 2).sum()) == 8.0   # the context is alive
