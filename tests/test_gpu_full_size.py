"""The benchmark's full-size configurations through size-independent properties (the oracle would take
minutes on them): exact linearity in a power of two, exact equivariance under token permutation, and
agreement of the tensor-core routes with the exact-integer batched matvec on a sample."""
import numpy as np
import pytest
import torch

import oracle as ro
from reinstinct_b200 import synth

pytestmark = pytest.mark.gpu


def test_config4_prefill_gemm_properties(rt):
    P, in_dim, out_dim, t = 512, 5120, 17408, ro.Q4_K
    raw = synth.synth_blocks(t, in_dim, out_dim, seed=77)
    w = rt.GpuMatvecTensor.from_bytes_matvec(raw, t, in_dim, out_dim)
    x = torch.from_numpy(synth.synth_activations(P, in_dim, 78)).cuda()
    gemm = rt.PrefillGemm()
    y = gemm.matmul(w, x, P)
    # doubling the activations doubles every output exactly: the quantizer's d doubles, q stays, the
    # token's power-of-two scale absorbs the factor, and the final multiply by its inverse is exact
    y2 = gemm.matmul(w, x * 2.0, P)
    assert torch.equal(y2, y * 2.0)
    # tokens are independent: permuting the rows of x permutes the rows of y bit for bit
    perm = torch.randperm(P, device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))
    yp = gemm.matmul(w, x[perm].contiguous(), P)
    assert torch.equal(yp, y[perm])
    # sixteen tokens through the exact-integer batched matvec
    sel = torch.arange(0, P, P // 16, device="cuda")[:16]
    xq = torch.empty(16 * (in_dim // 32) * 40, dtype=torch.uint8, device="cuda")
    rt.launch_quantize_q8(x[sel].contiguous(), xq, in_dim, 16)
    ye = torch.empty(16, out_dim, device="cuda")
    rt.launch_matvec_batched(w, xq, ye, 16)
    torch.cuda.synchronize()
    assert ro.rel_l2(y[sel].cpu().numpy(), ye.cpu().numpy()) < 1e-3
    assert torch.isfinite(y).all()


def test_config5_moe_grouped_gemm_against_expert_matvec(rt):
    """256 experts, top-8 of 512 tokens: every sorted entry's gate_up row equals the decode-side expert
    matvec of that token with that expert (exact-integer route: same per-block arithmetic), on both
    grouped routes within their bars."""
    E, H, F, NT, K, t = 256, 2048, 512, 512, 8, ro.Q4_K
    one = synth.synth_blocks(t, H, 2 * F * 8, 91)
    gu = rt.GpuExpertTensor.from_bytes(np.tile(one, E // 8), t, H, 2 * F, E)
    logits = torch.from_numpy(synth.synth_router_logits(NT, E, 93)).cuda()
    ids = torch.empty(NT, K, dtype=torch.int32, device="cuda")
    wts = torch.empty(NT, K, device="cuda")
    rt.launch_moe_topk(logits, ids, wts, E, K, NT)
    NE = NT * K
    x = torch.from_numpy(synth.synth_activations(NT, H, 94)).cuda()
    moe = rt.MoeGroupedScratch.new(E, NE)
    rt.launch_moe_sort(moe, ids, NE)
    n_sub = H // 32
    xq = torch.empty(NT * n_sub * 40, dtype=torch.uint8, device="cuda")
    rt.launch_quantize_q8(x, xq, H, NT)
    xg = torch.empty(NE * n_sub * 40, dtype=torch.uint8, device="cuda")
    rt.launch_moe_gather_xq(moe, xq, xg, n_sub, K, NE)
    y_sorted = torch.empty(NE, 2 * F, device="cuda")
    rt.launch_moe_grouped_gemm(moe, gu, xg, y_sorted, H, 2 * F, NE)
    y_entry = torch.empty(NT, K, 2 * F, device="cuda")
    rt.launch_moe_scatter_rows(moe, y_sorted, y_entry, 2 * F, NE)
    # decode-side route: token t, slot j -> expert ids[t][j], one activation row per token
    y_dec = torch.empty(NT, K, 2 * F, device="cuda")
    rt.launch_moe_expert_matvec(gu, ids, xq, y_dec, K, NT, n_sub, 0)
    y32 = torch.empty(NE, 2 * F, device="cuda")
    rt.MoeGroupedGemm().gate_up(moe, gu, x, K, y32, NE)
    y32_entry = torch.empty(NT, K, 2 * F, device="cuda")
    rt.launch_moe_scatter_rows(moe, y32, y32_entry, 2 * F, NE)
    torch.cuda.synchronize()
    ref = y_dec.cpu().numpy()
    assert ro.rel_l2(y_entry.cpu().numpy(), ref) < 1e-5      # both exact-integer: only the order of f32 additions differs
    assert ro.rel_l2(y32_entry.cpu().numpy(), ref) < 1e-3
    # every entry was produced: the sort's counts add up and no row kept its fill value
    assert int(moe.expert_off.cpu()[-1]) == NE
    assert torch.isfinite(y_entry).all() and torch.isfinite(y32_entry).all()
