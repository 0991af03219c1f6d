"""GPU parity of the MoE glue kernels (router top-k, gated activation + BlockQ8 quantizer, weighted
combine) through the C ABI, against the CPU oracle."""
import numpy as np
import pytest
import torch

import oracle as ro

pytestmark = pytest.mark.gpu


def _topk(rt, logits: np.ndarray, n_used: int):
    n_tok, n_expert = logits.shape
    ids = torch.full((n_tok, n_used), -7, dtype=torch.int32, device="cuda")
    wts = torch.full((n_tok, n_used), float("nan"), device="cuda")
    rt.launch_moe_topk(torch.from_numpy(logits).cuda(), ids, wts, n_expert, n_used, n_tok)
    torch.cuda.synchronize()
    return ids.cpu().numpy(), wts.cpu().numpy()


@pytest.mark.parametrize("n_tok,n_expert,n_used", [(1, 128, 8), (7, 128, 8), (33, 256, 8), (5, 64, 4), (3, 60, 6),
                                                     (2, 1024, 32), (9, 8, 2), (4, 8, 8), (512, 128, 8)])
def test_topk_matches_oracle(rt, n_tok, n_expert, n_used):
    rng = np.random.default_rng(n_tok * 1000 + n_expert + n_used)
    logits = (rng.standard_normal((n_tok, n_expert)) * 3.0).astype(np.float32)
    ids, wts = _topk(rt, logits, n_used)
    rids, rwts = ro.router_topk(logits, n_used)
    # The softmax sum is reduced in a different order, so probabilities may differ in the last
    # bits; selection only differs where two probabilities are that close.
    p = np.exp(logits.astype(np.float64) - logits.max(1, keepdims=True))
    p /= p.sum(1, keepdims=True)
    for t in range(n_tok):
        if not np.array_equal(ids[t], rids[t]):
            for k in np.nonzero(ids[t] != rids[t])[0]:
                assert abs(p[t, ids[t, k]] - p[t, rids[t, k]]) <= 4e-7 * p[t, rids[t, k]]
    assert (ids == rids).mean() > 0.999
    np.testing.assert_allclose(wts, rwts, rtol=2e-6, atol=0)
    np.testing.assert_allclose(wts.sum(1), 1.0, rtol=1e-5)


def test_topk_ties_nan_and_floor(rt):
    n_expert, n_used = 128, 8
    logits = np.zeros((4, n_expert), dtype=np.float32)
    logits[1, 5] = np.nan          # a NaN logit can never be chosen
    logits[1, 0] = np.nan
    logits[2] = -1e30              # equal after the max subtraction: uniform
    logits[3, 100:] = 50.0         # 28 equal winners: the lowest indices of them
    ids, wts = _topk(rt, logits, n_used)
    rids, rwts = ro.router_topk(logits, n_used)
    np.testing.assert_array_equal(ids, rids)
    np.testing.assert_array_equal(ids[0], np.arange(8))
    np.testing.assert_array_equal(ids[1], [1, 2, 3, 4, 6, 7, 8, 9])
    np.testing.assert_array_equal(ids[3], np.arange(100, 108))
    np.testing.assert_allclose(wts, rwts, rtol=2e-6)
    np.testing.assert_allclose(wts, 0.125, rtol=1e-6)


def test_topk_row_without_a_number_follows_the_reference(rt):
    """All logits of a token NaN: no probability is a number and no candidate ever wins.  The reference's scan then
    leaves its index at 0 (kernels/moe_topk.cpp: `float bv = -1.0f; int bi = 0;`), and so do the oracle and the kernel:
    ids stay inside the experts, the neighbouring rows are untouched."""
    logits = np.zeros((3, 64), dtype=np.float32)
    logits[1] = np.nan
    ids, wts = _topk(rt, logits, 4)
    rids, rwts = ro.router_topk(logits, 4)
    np.testing.assert_array_equal(ids, rids)
    np.testing.assert_array_equal(ids[1], 0)
    np.testing.assert_array_equal(wts[1], rwts[1])
    np.testing.assert_allclose(wts[[0, 2]], 0.25, rtol=1e-6)


def _unpack_q8(b: np.ndarray):
    b = np.ascontiguousarray(b).reshape(-1, 40)
    d = b[:, 0:4].copy().view(np.float32).reshape(-1)
    xs = b[:, 4:8].copy().view(np.float32).reshape(-1)
    qs = b[:, 8:].view(np.int8)
    return d, xs, qs


@pytest.mark.parametrize("act", [0, 1])
@pytest.mark.parametrize("ff,n_slot", [(32, 1), (704, 8), (768, 37), (1408, 64), (2048, 300)])
def test_act_q8_matches_oracle(rt, act, ff, n_slot):
    rng = np.random.default_rng(ff + n_slot + act)
    gu = (rng.standard_normal((n_slot, 2 * ff)) * 2.5).astype(np.float32)
    if n_slot > 1:
        gu[1, :32] = 0.0           # an all-zero sub-block: d = 1, qs = 0
    out = torch.zeros(n_slot * (ff // 32) * 40, dtype=torch.uint8, device="cuda")
    rt.launch_moe_act_q8(torch.from_numpy(gu).cuda(), out, ff, n_slot, act)
    torch.cuda.synchronize()
    d, xs, qs = _unpack_q8(out.cpu().numpy())
    ref, v = ro.moe_act_q8(gu, act)
    rd, rxs, rqs = _unpack_q8(ref)
    # tanhf / expf differ by a few ulp between the device and the host libm: the f32 fields
    # agree to that, and a rounding boundary may move single int8 values by one.
    np.testing.assert_allclose(d, rd, rtol=4e-6)
    np.testing.assert_allclose(xs, rxs, rtol=0, atol=4e-6 * np.abs(v).reshape(-1, 32).sum(1).max())
    diff = np.abs(qs.astype(np.int32) - rqs.astype(np.int32))
    assert diff.max() <= 1
    assert (diff != 0).mean() < 2e-3
    # and the dequantized activation stays within the format's own step of the f64 value
    g64, u64 = gu[:, :ff].astype(np.float64), gu[:, ff:].astype(np.float64)
    a64 = (0.5 * g64 * (1 + np.tanh(0.7978845608028654 * (g64 + 0.044715 * g64 ** 3)))) if act == 0 \
        else g64 / (1 + np.exp(-g64))
    want = (a64 * u64).reshape(-1, 32)
    assert np.all(np.abs(qs * d[:, None] - want) <= 0.5001 * d[:, None] + 1e-6)


def test_act_q8_feeds_grouped_gemm_layout(rt):
    """The output is the BlockQ8 stream rc_quantize_q8 writes for the same f32 values."""
    ff, n_slot = 1024, 19
    rng = np.random.default_rng(99)
    gu = rng.standard_normal((n_slot, 2 * ff)).astype(np.float32)
    gu[:, :ff] = 40.0              # gelu(40) = 40 and silu(40) = 40 exactly in f32: v = 40 * up
    v = (np.float32(40.0) * gu[:, ff:]).astype(np.float32)
    for act in (0, 1):
        out = torch.zeros(n_slot * (ff // 32) * 40, dtype=torch.uint8, device="cuda")
        rt.launch_moe_act_q8(torch.from_numpy(gu).cuda(), out, ff, n_slot, act)
        want = torch.zeros_like(out)
        rt.launch_quantize_q8(torch.from_numpy(v).cuda(), want, ff, n_slot)
        torch.cuda.synchronize()
        assert torch.equal(out, want)
        np.testing.assert_array_equal(out.cpu().numpy(), ro.quantize_q8(v).reshape(-1))


@pytest.mark.parametrize("n_tok,n_used,hidden,scaled", [(1, 8, 2816, True), (5, 8, 2048, True), (3, 4, 1000, False),
                                                         (130, 8, 257, True), (2, 1, 64, True)])
def test_combine_bit_exact(rt, n_tok, n_used, hidden, scaled):
    rng = np.random.default_rng(n_tok + hidden)
    n_expert = 128
    experts = rng.standard_normal((n_tok, n_used, hidden)).astype(np.float32)
    ids = rng.integers(0, n_expert, (n_tok, n_used)).astype(np.int32)
    wts = rng.random((n_tok, n_used)).astype(np.float32)
    sc = (rng.random(n_expert) + 0.5).astype(np.float32) if scaled else None
    out = torch.full((n_tok, hidden), float("nan"), device="cuda")
    rt.launch_moe_combine(torch.from_numpy(experts).cuda(), torch.from_numpy(ids).cuda(), torch.from_numpy(wts).cuda(),
                          None if sc is None else torch.from_numpy(sc).cuda(), out, hidden, n_used, n_tok)
    torch.cuda.synchronize()
    want = ro.moe_combine(experts, ids, wts, sc)
    np.testing.assert_array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32))
    w64 = wts.astype(np.float64) * (sc[ids].astype(np.float64) if scaled else 1.0)
    ref = np.einsum("tj,tjh->th", w64, experts.astype(np.float64))
    assert ro.rel_l2(out.cpu().numpy(), ref) < 1e-6


def test_moe_layer_glue_end_to_end(rt):
    """router -> sort -> gather -> gate_up GEMM -> activation+quantize -> down GEMM -> scatter ->
    combine, every step through the C ABI, against the oracle chain."""
    import cases
    t = ro.Q4_K
    n_tok, hidden, ff, n_expert, n_used = 24, 512, 256, 8, 2
    rng = np.random.default_rng(5)
    raw_gu = [cases.synth_case(t, hidden, 2 * ff, 1, seed=100 + e)[0] for e in range(n_expert)]
    raw_dn = [cases.synth_case(t, ff, hidden, 1, seed=200 + e)[0] for e in range(n_expert)]
    x = rng.standard_normal((n_tok, hidden)).astype(np.float32)
    logits = rng.standard_normal((n_tok, n_expert)).astype(np.float32)
    sc = (rng.random(n_expert) + 0.5).astype(np.float32)

    # oracle chain
    rids, rwts = ro.router_topk(logits, n_used)
    xq = ro.quantize_q8(x).reshape(n_tok, -1)
    exp_out = np.zeros((n_tok, n_used, hidden), dtype=np.float32)
    for tk in range(n_tok):
        for j in range(n_used):
            e = rids[tk, j]
            g32, _, _ = ro.matvec_q8(t, ro.repack(t, raw_gu[e], hidden, 2 * ff), xq[tk], hidden, 2 * ff, 1)
            aq, _ = ro.moe_act_q8(g32.reshape(1, -1), 0)
            d32, _, _ = ro.matvec_q8(t, ro.repack(t, raw_dn[e], ff, hidden), aq.reshape(-1), ff, hidden, 1)
            exp_out[tk, j] = d32.reshape(-1)
    want = ro.moe_combine(exp_out, rids, rwts, sc)

    # device chain
    gu_t = rt.GpuExpertTensor.from_bytes(np.concatenate(raw_gu), t, hidden, 2 * ff, n_expert)
    dn_t = rt.GpuExpertTensor.from_bytes(np.concatenate(raw_dn), t, ff, hidden, n_expert)
    ids = torch.empty((n_tok, n_used), dtype=torch.int32, device="cuda")
    wts = torch.empty((n_tok, n_used), device="cuda")
    rt.launch_moe_topk(torch.from_numpy(logits).cuda(), ids, wts, n_expert, n_used, n_tok)
    n_ent = n_tok * n_used
    moe = rt.MoeGroupedScratch.new(n_expert, n_ent)
    rt.launch_moe_sort(moe, ids, n_ent)
    xq_d = torch.empty(n_tok * (hidden // 32) * 40, dtype=torch.uint8, device="cuda")
    rt.launch_quantize_q8(torch.from_numpy(x).cuda(), xq_d, hidden, n_tok)
    xq_s = torch.empty(n_ent * (hidden // 32) * 40, dtype=torch.uint8, device="cuda")
    rt.launch_moe_gather_xq(moe, xq_d, xq_s, hidden // 32, n_used, n_ent)
    gu = torch.empty((n_ent, 2 * ff), device="cuda")
    rt.launch_moe_grouped_gemm(moe, gu_t, xq_s, gu, hidden, 2 * ff, n_ent)
    aq = torch.empty(n_ent * (ff // 32) * 40, dtype=torch.uint8, device="cuda")
    rt.launch_moe_act_q8(gu, aq, ff, n_ent, rt.ACT_GEGLU)
    dn = torch.empty((n_ent, hidden), device="cuda")
    rt.launch_moe_grouped_gemm(moe, dn_t, aq, dn, ff, hidden, n_ent)
    per_entry = torch.empty((n_tok, n_used, hidden), device="cuda")
    rt.launch_moe_scatter_rows(moe, dn, per_entry, hidden, n_ent)
    out = torch.empty((n_tok, hidden), device="cuda")
    rt.launch_moe_combine(per_entry, ids, wts, torch.from_numpy(sc).cuda(), out, hidden, n_used, n_tok)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(ids.cpu().numpy(), rids)
    assert ro.rel_l2(out.cpu().numpy(), want) < 1e-3


@pytest.mark.parametrize("t", ro.ALL_TYPES)
@pytest.mark.parametrize("n_tok,in_dim,out_dim", [(1, 2048, 192), (5, 1024, 80), (3, 256, 512)])
def test_expert_matvec_matches_plain_matvec(rt, t, n_tok, in_dim, out_dim):
    """Decode-side routed-expert matvec, gate/up addressing (one activation row per token) and down
    addressing (one per slot): identical bits to rc_matvec on the chosen expert's tensor, and the
    oracle's value."""
    import cases
    n_expert, n_used, n_sub = 6, 3, in_dim // 32
    rng = np.random.default_rng(1000 * t + n_tok)
    raws = [cases.synth_case(t, in_dim, out_dim, 1, seed=50 * t + e)[0] for e in range(n_expert)]
    et = rt.GpuExpertTensor.from_bytes(np.concatenate(raws), t, in_dim, out_dim, n_expert)
    singles = [rt.GpuMatvecTensor.from_bytes_matvec(r, t, in_dim, out_dim) for r in raws]
    ids = rng.integers(0, n_expert, (n_tok, n_used)).astype(np.int32)
    ids_d = torch.from_numpy(ids).cuda()
    for tok_stride, slot_stride in ((n_sub, 0), (n_used * n_sub, n_sub)):  # in BlockQ8 blocks, as the reference passes them
        n_x = n_tok if slot_stride == 0 else n_tok * n_used
        x = rng.standard_normal((n_x, in_dim)).astype(np.float32)
        xq = torch.empty(n_x * n_sub * 40, dtype=torch.uint8, device="cuda")
        rt.launch_quantize_q8(torch.from_numpy(x).cuda(), xq, in_dim, n_x)
        y = torch.full((n_tok, n_used, out_dim), float("nan"), device="cuda")
        rt.launch_moe_expert_matvec(et, ids_d, xq, y, n_used, n_tok, tok_stride, slot_stride)
        torch.cuda.synchronize()
        got = y.cpu().numpy()
        xq_h = ro.quantize_q8(x).reshape(n_x, -1)
        for tk in range(n_tok):
            for j in range(n_used):
                e, row = ids[tk, j], (tk * tok_stride + j * slot_stride) // n_sub
                one = torch.empty(out_dim, device="cuda")
                rt.launch_matvec_xq8(singles[e], xq[row * n_sub * 40:(row + 1) * n_sub * 40], one)
                torch.cuda.synchronize()
                _, y64, _ = ro.matvec_q8(t, ro.repack(t, raws[e], in_dim, out_dim), xq_h[row], in_dim, out_dim, 1)
                assert ro.rel_l2(got[tk, j], y64) < 1e-5
                assert ro.rel_l2(got[tk, j], one.cpu().numpy()) < 1e-6   # row splitting may differ: same terms, other order


def test_expert_matvec_bad_id_and_arguments(rt):
    import cases
    t, in_dim, out_dim, n_expert = ro.Q4_K, 512, 64, 3
    raws = [cases.synth_case(t, in_dim, out_dim, 1, seed=e)[0] for e in range(n_expert)]
    et = rt.GpuExpertTensor.from_bytes(np.concatenate(raws), t, in_dim, out_dim, n_expert)
    x = np.ones((1, in_dim), dtype=np.float32)
    xq = torch.empty((in_dim // 32) * 40, dtype=torch.uint8, device="cuda")
    rt.launch_quantize_q8(torch.from_numpy(x).cuda(), xq, in_dim, 1)
    ids = torch.tensor([[1, -1, 7, 2]], dtype=torch.int32, device="cuda")
    y = torch.full((1, 4, out_dim), float("nan"), device="cuda")
    rt.launch_moe_expert_matvec(et, ids, xq, y, 4, 1, in_dim // 32, 0)
    torch.cuda.synchronize()
    got = y.cpu().numpy()
    assert np.all(got[0, 1] == 0) and np.all(got[0, 2] == 0)
    assert np.all(np.isfinite(got)) and np.any(got[0, 0] != 0) and np.any(got[0, 3] != 0)


@pytest.mark.parametrize("t", ro.ALL_TYPES)
def test_gate_up_swiglu_equals_two_matvecs_and_activation(rt, t):
    """The fused decode kernel against two expert matvecs (same per-block arithmetic, same order) and
    the SiLU product in f32."""
    import cases
    n_expert, n_used, n_tok, in_dim, out_dim = 5, 3, 4, 2048, 96
    rng = np.random.default_rng(t)
    gates = [cases.synth_case(t, in_dim, out_dim, 1, seed=60 * t + e)[0] for e in range(n_expert)]
    ups = [cases.synth_case(t, in_dim, out_dim, 1, seed=70 * t + e)[0] for e in range(n_expert)]
    g = rt.GpuExpertTensor.from_bytes(np.concatenate(gates), t, in_dim, out_dim, n_expert)
    u = rt.GpuExpertTensor.from_bytes(np.concatenate(ups), t, in_dim, out_dim, n_expert)
    ids = torch.from_numpy(rng.integers(0, n_expert, (n_tok, n_used)).astype(np.int32)).cuda()
    x = rng.standard_normal((n_tok, in_dim)).astype(np.float32) * 0.1
    n_sub = in_dim // 32
    xq = torch.empty(n_tok * n_sub * 40, dtype=torch.uint8, device="cuda")
    rt.launch_quantize_q8(torch.from_numpy(x).cuda(), xq, in_dim, n_tok)
    y = torch.full((n_tok, n_used, out_dim), float("nan"), device="cuda")
    rt.launch_moe_gate_up_swiglu(g, u, ids, xq, y, n_used, n_tok, n_sub, 0)
    yg, yu = torch.empty_like(y), torch.empty_like(y)
    rt.launch_moe_expert_matvec(g, ids, xq, yg, n_used, n_tok, n_sub, 0)
    rt.launch_moe_expert_matvec(u, ids, xq, yu, n_used, n_tok, n_sub, 0)
    torch.cuda.synchronize()
    gv, uv = yg.cpu().numpy().astype(np.float64), yu.cpu().numpy().astype(np.float64)
    want = gv / (1 + np.exp(-gv)) * uv
    assert ro.rel_l2(y.cpu().numpy(), want) < 1e-5
