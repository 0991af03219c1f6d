"""Expert parallelism without the host (rc_ep_plan / rc_ep_dispatch / rc_ep_return / rc_ep_collect) as a world of one:
every kernel of the exchange runs, the placement is checked against its definition, and the layer's result equals the
reference's own launch sequence (sort, gather, grouped GEMM, scatter; src/runtime/qwen35.rs:2892-3064) bit for bit,
over alternating buffers, with dropped entries, and replayed from a CUDA graph."""
import numpy as np
import pytest
import torch

import cases
import oracle as ro

pytestmark = pytest.mark.gpu


def _layer(rt, t, hidden, out_dim, n_expert, seed):
    raws = [cases.synth_case(t, hidden, out_dim, 1, seed=seed + e)[0] for e in range(n_expert)]
    return rt.GpuExpertTensor.from_bytes(np.concatenate(raws), t, hidden, out_dim, n_expert)


def _plain(rt, et, ids, xq, hidden, out_dim, n_used, n_ent):
    moe = rt.MoeGroupedScratch.new(et.n_expert, n_ent)
    rt.launch_moe_sort(moe, ids, n_ent)
    xg = torch.empty(n_ent * (hidden // 32) * 40, dtype=torch.uint8, device="cuda")
    rt.launch_moe_gather_xq(moe, xq, xg, hidden // 32, n_used, n_ent)
    y_sorted = torch.zeros(n_ent, out_dim, device="cuda")
    rt.launch_moe_grouped_gemm(moe, et, xg, y_sorted, hidden, out_dim, n_ent)
    y = torch.zeros(n_ent, out_dim, device="cuda")
    rt.launch_moe_scatter_rows(moe, y_sorted, y, out_dim, n_ent)
    return y


@pytest.mark.parametrize("t", [ro.Q4_K, ro.Q6_K])
def test_world_of_one_equals_the_plain_sequence(rt, t):
    hidden, out_dim, n_expert, n_used, n_tok = 512, 256, 8, 2, 40
    et = _layer(rt, t, hidden, out_dim, n_expert, 500)
    n_ent = n_tok * n_used
    ep = rt.ExpertParallel(et, hidden, out_dim, cap=n_ent + 7)
    rng = np.random.default_rng(3)
    for rnd in range(4):  # both receive buffers, twice
        x = torch.from_numpy(rng.standard_normal((n_tok, hidden)).astype(np.float32)).cuda()
        xq = torch.empty(n_tok * (hidden // 32) * 40, dtype=torch.uint8, device="cuda")
        rt.launch_quantize_q8(x, xq, hidden, n_tok)
        ids_np = rng.integers(0, n_expert, size=n_ent).astype(np.int32)
        if rnd == 2:
            ids_np[::7] = -1  # dropped entries: no slot, zeros come back
        ids = torch.from_numpy(ids_np).cuda()
        out = torch.full((n_ent, out_dim), 7.0, device="cuda")
        ep.step(ids, xq, n_ent, n_used, out)
        want = _plain(rt, et, ids, xq, hidden, out_dim, n_used, n_ent)
        torch.cuda.synchronize()
        # placement: entry e sits at (owner 0) slot = number of earlier kept entries
        back = ep.back[:n_ent].cpu().numpy()
        kept = ids_np >= 0
        assert np.array_equal(back[kept], np.arange(kept.sum())) and np.all(back[~kept] == -1)
        assert torch.equal(out, want), f"round {rnd}"
        if rnd == 2:
            assert float(out[::7].abs().max()) == 0.0
    ep.close()


def test_two_steps_replay_from_a_graph(rt):
    t, hidden, out_dim, n_expert, n_used, n_tok = ro.Q4_K, 512, 256, 4, 2, 24
    et = _layer(rt, t, hidden, out_dim, n_expert, 600)
    n_ent = n_tok * n_used
    ep = rt.ExpertParallel(et, hidden, out_dim, cap=n_ent)
    rng = np.random.default_rng(4)
    x = torch.from_numpy(rng.standard_normal((n_tok, hidden)).astype(np.float32)).cuda()
    xq = torch.empty(n_tok * (hidden // 32) * 40, dtype=torch.uint8, device="cuda")
    ids = torch.from_numpy(rng.integers(0, n_expert, size=n_ent).astype(np.int32)).cuda()
    outs = [torch.empty(n_ent, out_dim, device="cuda") for _ in range(2)]
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        rt.launch_quantize_q8(x, xq, hidden, n_tok)
        for o in outs:
            ep.step(ids, xq, n_ent, n_used, o)  # warm-up outside capture (an even number of steps)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        rt.launch_quantize_q8(x, xq, hidden, n_tok)
        for o in outs:
            ep.step(ids, xq, n_ent, n_used, o)
    want = _plain(rt, et, ids, xq, hidden, out_dim, n_used, n_ent)
    for rep in range(3):
        x.copy_(torch.from_numpy(rng.standard_normal((n_tok, hidden)).astype(np.float32)))
        for o in outs:
            o.zero_()
        g.replay()
        want = _plain(rt, et, ids, xq, hidden, out_dim, n_used, n_ent)
        torch.cuda.synchronize()
        assert torch.equal(outs[0], want) and torch.equal(outs[1], want), rep
    ep.close()


def test_whole_expert_ffn_at_the_owner(rt):
    """With a down projection the owner runs gate_up GEMM, SwiGLU + quantize and the down GEMM on what it received;
    rows of the model width come back.  Equal to the same launches on one GPU, bit for bit."""
    t, td, hidden, ff, n_expert, n_used, n_tok = ro.Q4_K, ro.Q6_K, 512, 256, 8, 2, 40
    gu = _layer(rt, t, hidden, 2 * ff, n_expert, 700)
    dn = _layer(rt, td, ff, hidden, n_expert, 800)
    n_ent = n_tok * n_used
    ep = rt.ExpertParallel(gu, hidden, 2 * ff, cap=n_ent, down=dn, act=rt.ACT_SWIGLU)
    rng = np.random.default_rng(5)
    for rnd in range(2):
        x = torch.from_numpy(rng.standard_normal((n_tok, hidden)).astype(np.float32)).cuda()
        xq = torch.empty(n_tok * (hidden // 32) * 40, dtype=torch.uint8, device="cuda")
        rt.launch_quantize_q8(x, xq, hidden, n_tok)
        ids = torch.from_numpy(rng.integers(0, n_expert, size=n_ent).astype(np.int32)).cuda()
        out = torch.empty(n_ent, hidden, device="cuda")
        ep.step(ids, xq, n_ent, n_used, out)
        moe = rt.MoeGroupedScratch.new(n_expert, n_ent)
        rt.launch_moe_sort(moe, ids, n_ent)
        xg = torch.empty(n_ent * (hidden // 32) * 40, dtype=torch.uint8, device="cuda")
        rt.launch_moe_gather_xq(moe, xq, xg, hidden // 32, n_used, n_ent)
        y1 = torch.zeros(n_ent, 2 * ff, device="cuda")
        rt.launch_moe_grouped_gemm(moe, gu, xg, y1, hidden, 2 * ff, n_ent)
        hq = torch.empty(n_ent * (ff // 32) * 40, dtype=torch.uint8, device="cuda")
        rt.launch_moe_act_q8(y1, hq, ff, n_ent, rt.ACT_SWIGLU)
        y2 = torch.zeros(n_ent, hidden, device="cuda")
        rt.launch_moe_grouped_gemm(moe, dn, hq, y2, ff, hidden, n_ent)
        want = torch.zeros(n_ent, hidden, device="cuda")
        rt.launch_moe_scatter_rows(moe, y2, want, hidden, n_ent)
        torch.cuda.synchronize()
        assert torch.equal(out, want), rnd
    ep.close()
