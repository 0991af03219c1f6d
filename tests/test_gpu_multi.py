"""Two-GPU tests (skipped on a single-GPU box): the peer-memory all-gather and a row-sharded
matvec whose gathered output must equal the single-GPU result bit for bit."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, q):
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    for p in (str(root), str(root / "tests")):
        if p not in sys.path:
            sys.path.insert(0, p)
    import torch.distributed as dist

    import cases
    import oracle as ro
    from reinstinct_b200 import runtime as rt
    from reinstinct_b200 import sharding as sh

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        rt.init(rank)
        t, in_dim, out_dim = ro.Q4_K, 2048, 640
        raw, x = cases.synth_case(t, in_dim, out_dim, 1, seed=5)
        part, rows = sh.shard_raw_rows(raw, t, in_dim, out_dim, rank, world)
        w = rt.GpuMatvecTensor.from_bytes_matvec(part, t, in_dim, rows)
        xq = torch.empty((in_dim // 32) * 40, dtype=torch.uint8, device="cuda")
        rt.launch_quantize_q8(torch.from_numpy(x).cuda(), xq, in_dim, 1)
        y = torch.empty(rows, device="cuda")
        ga = rt.PeerAllGather(rows * 4)
        w_full = rt.GpuMatvecTensor.from_bytes_matvec(raw, t, in_dim, out_dim)
        y_full = torch.empty(out_dim, device="cuda")
        got = torch.empty(out_dim, device="cuda")
        lib = rt._lib.load()
        for rnd in range(5):  # new activations every round over the same (alternating) buffers and counters
            x = cases.synth_case(t, in_dim, out_dim, 1, seed=50 + rnd)[1]
            rt.launch_quantize_q8(torch.from_numpy(x).cuda(), xq, in_dim, 1)
            rt.launch_matvec_xq8(w, xq, y)
            ga.gather(y)
            ga.copy_out(got)
            # same kernel, same rows, same arithmetic as the unsharded launch
            rt.launch_matvec_xq8(w_full, xq, y_full)
            torch.cuda.synchronize()
            assert torch.equal(got, y_full), f"round {rnd}: gathered shards differ from the single-GPU launch"
        st = __import__("ctypes").c_uint(0)
        assert lib.rc_device_status(__import__("ctypes").byref(st)) == 0 and st.value == 0
        full32, _, _ = ro.matvec_q8(t, ro.repack(t, raw, in_dim, out_dim), ro.quantize_q8(x), in_dim, out_dim, 1)
        assert ro.rel_l2(got.cpu().numpy(), full32.astype(np.float64)) < 1e-3
        # the row-sharded prefill GEMM that gathers its own output: every rank ends with the whole product,
        # bit-identical to the unsharded call, on both of its alternating buffers
        P = 200
        xs = torch.from_numpy(cases.synth_case(t, in_dim, out_dim, P, seed=77)[1]).cuda()
        y_ref, _ = rt.PrefillGemm().matmul_block_dots(w_full, xs, P)
        gg = rt.GatheredPrefillGemm(P, out_dim, in_dim)
        b0, _ = sh.row_shard_range(out_dim, rank, world)
        y_all = torch.empty(P, out_dim, device="cuda")
        for rnd in range(3):
            k = gg.matmul(w, xs, P, b0)
            gg.read(k, y_all, P)
            torch.cuda.synchronize()
            assert torch.equal(y_all, y_ref), f"gathered GEMM round {rnd} differs from the unsharded product"
        assert lib.rc_device_status(__import__("ctypes").byref(st)) == 0 and st.value == 0
        gg.close()
        ga.close()
        # the decode FFN as one cooperative launch per GPU: gate/up rows and down rows sharded, the f32 intermediate
        # and the output rows stored straight into the peer's memory; every rank ends with the whole output, the two
        # ranks' copies bit-equal, and equal to the one-GPU launch chain within f32 association
        tg, td, hidden, ffn, out = ro.Q4_K, ro.Q6_K, 1024, 2048, 640
        raw_g, raw_u = (cases.synth_case(tg, hidden, ffn, 1, seed=s)[0] for s in (61, 62))
        raw_d = cases.synth_case(td, ffn, out, 1, seed=63)[0]
        full = [rt.GpuMatvecTensor.from_bytes_matvec(r, ty, i, o) for r, ty, i, o in
                ((raw_g, tg, hidden, ffn), (raw_u, tg, hidden, ffn), (raw_d, td, ffn, out))]
        pg, ng = sh.shard_raw_rows(raw_g, tg, hidden, ffn, rank, world)
        pu, _ = sh.shard_raw_rows(raw_u, tg, hidden, ffn, rank, world)
        pd, nd = sh.shard_raw_rows(raw_d, td, ffn, out, rank, world)
        f0, _ = sh.row_shard_range(ffn, rank, world)
        o0, _ = sh.row_shard_range(out, rank, world)
        fused = rt.FusedFfnDecode(rt.GpuMatvecTensor.from_bytes_matvec(pg, tg, hidden, ng),
                                  rt.GpuMatvecTensor.from_bytes_matvec(pu, tg, hidden, ng),
                                  rt.GpuMatvecTensor.from_bytes_matvec(pd, td, ffn, nd), ffn, out, f0, o0)
        u8 = dict(dtype=torch.uint8, device="cuda")
        xq2, hq2 = torch.empty((hidden // 32) * 40, **u8), torch.empty((ffn // 32) * 40, **u8)
        yg, yu, y_chain = (torch.empty(n, device="cuda") for n in (ffn, ffn, out))
        y_f = torch.empty(out, device="cuda")
        for rnd in range(4):
            xd = torch.from_numpy(cases.synth_case(tg, hidden, 8, 1, seed=70 + rnd)[1]).cuda().reshape(-1)
            rt.launch_ffn_decode(full[0], full[1], full[2], xd, xq2, yg, yu, hq2, y_chain)
            fused.run(xd)
            fused.read_y(y_f)
            torch.cuda.synchronize()
            assert lib.rc_device_status(__import__("ctypes").byref(st)) == 0 and st.value == 0, hex(st.value)
            assert ro.rel_l2(y_f.cpu().numpy(), y_chain.cpu().numpy().astype(np.float64)) < 1e-3, rnd
            both = [torch.empty_like(y_f) for _ in range(world)]
            dist.all_gather(both, y_f)
            assert all(torch.equal(both[0], b) for b in both[1:]), f"fused FFN round {rnd}: the ranks' outputs differ"
        fused.close()
        # the tensor-parallel form (gate/up by rows, down by the matching columns, partial outputs summed in rank order):
        # uneven column shards in whole superblocks
        ffn2 = 2304
        raw_g2, raw_u2 = (cases.synth_case(tg, hidden, ffn2, 1, seed=s)[0] for s in (64, 65))
        raw_d2 = cases.synth_case(td, ffn2, out, 1, seed=66)[0]
        full2 = [rt.GpuMatvecTensor.from_bytes_matvec(r, ty, i, o) for r, ty, i, o in
                 ((raw_g2, tg, hidden, ffn2), (raw_u2, tg, hidden, ffn2), (raw_d2, td, ffn2, out))]
        c0, c1 = sh.col_shard_range(ffn2, rank, world, 256)
        row_bytes = (hidden // 256) * 144
        g_part = np.asarray(raw_g2, dtype=np.uint8)[c0 * row_bytes:c1 * row_bytes]
        u_part = np.asarray(raw_u2, dtype=np.uint8)[c0 * row_bytes:c1 * row_bytes]
        d_part = sh.shard_raw_cols(raw_d2, td, ffn2, out, c0, c1)
        tp = rt.TensorParallelFfnDecode(rt.GpuMatvecTensor.from_bytes_matvec(g_part, tg, hidden, c1 - c0),
                                        rt.GpuMatvecTensor.from_bytes_matvec(u_part, tg, hidden, c1 - c0),
                                        rt.GpuMatvecTensor.from_bytes_matvec(d_part, td, c1 - c0, out))
        hq3 = torch.empty((ffn2 // 32) * 40, **u8)
        yg3, yu3 = torch.empty(ffn2, device="cuda"), torch.empty(ffn2, device="cuda")
        for rnd in range(4):
            xd = torch.from_numpy(cases.synth_case(tg, hidden, 8, 1, seed=80 + rnd)[1]).cuda().reshape(-1)
            rt.launch_ffn_decode(full2[0], full2[1], full2[2], xd, xq2, yg3, yu3, hq3, y_chain)
            tp.run(xd)
            tp.read_y(y_f)
            torch.cuda.synchronize()
            assert lib.rc_device_status(__import__("ctypes").byref(st)) == 0 and st.value == 0, hex(st.value)
            assert ro.rel_l2(y_f.cpu().numpy(), y_chain.cpu().numpy().astype(np.float64)) < 5e-4, rnd
            both = [torch.empty_like(y_f) for _ in range(world)]
            dist.all_gather(both, y_f)
            assert all(torch.equal(both[0], b) for b in both[1:]), f"tensor-parallel FFN round {rnd}: the ranks' outputs differ"
        tp.close()
        q.put((rank, "ok"))
    except Exception as e:  # report instead of leaving the peer waiting
        q.put((rank, f"{type(e).__name__}: {e}"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_gather_row_sharded_matvec_two_gpus():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert all(msg == "ok" for _, msg in results), results


def _moe_worker(rank: int, world: int, port: int, q):
    """Expert parallelism over two GPUs: rank g owns half of the experts, every rank routes its own
    tokens; routed activation rows travel to the owning rank by all-to-all (counts first), go through
    the grouped GEMM there and travel back.  Must equal the same layer computed with all experts on
    one GPU, bit for bit (same kernel, per-entry arithmetic independent of the tile an entry lands in)."""
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    for p in (str(root), str(root / "tests")):
        if p not in sys.path:
            sys.path.insert(0, p)
    import torch.distributed as dist

    import cases
    import oracle as ro
    from reinstinct_b200 import runtime as rt
    from reinstinct_b200 import sharding as sh

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        rt.init(rank)
        t, hidden, out_dim, n_expert, n_used, n_tok = ro.Q4_K, 512, 256, 8, 2, 24
        raws = [cases.synth_case(t, hidden, out_dim, 1, seed=300 + e)[0] for e in range(n_expert)]
        e0, e1 = sh.expert_range(n_expert, rank, world)
        et_local = rt.GpuExpertTensor.from_bytes(np.concatenate(raws[e0:e1]), t, hidden, out_dim, e1 - e0)
        et_all = rt.GpuExpertTensor.from_bytes(np.concatenate(raws), t, hidden, out_dim, n_expert)
        rng = np.random.default_rng(40 + rank)          # every rank has its own tokens
        x = torch.from_numpy(rng.standard_normal((n_tok, hidden)).astype(np.float32)).cuda()
        logits = torch.from_numpy(rng.standard_normal((n_tok, n_expert)).astype(np.float32)).cuda()
        ids = torch.empty(n_tok, n_used, dtype=torch.int32, device="cuda")
        wts = torch.empty(n_tok, n_used, device="cuda")
        rt.launch_moe_topk(logits, ids, wts, n_expert, n_used, n_tok)
        n_ent = n_tok * n_used
        gg = rt.MoeGroupedGemm()

        # one GPU, all experts: sorted GEMM, rows scattered back to entry order
        moe = rt.MoeGroupedScratch.new(n_expert, n_ent)
        rt.launch_moe_sort(moe, ids, n_ent)
        y_sorted = torch.empty(n_ent, out_dim, device="cuda")
        gg.gate_up(moe, et_all, x, n_used, y_sorted, n_ent)
        want = torch.empty(n_ent, out_dim, device="cuda")
        rt.launch_moe_scatter_rows(moe, y_sorted, want, out_dim, n_ent)
        torch.cuda.synchronize()

        # expert-parallel: entries (token row, expert id) go to the owner of the expert
        flat_ids = ids.reshape(-1)
        plan = sh.plan_dispatch(flat_ids, n_expert)
        rows = x.repeat_interleave(n_used, dim=0).contiguous()            # one row per entry
        rows_in = sh.dispatch_rows(rows, plan)
        ids_in = sh.dispatch_rows(flat_ids.to(torch.float32).reshape(-1, 1), plan).reshape(-1).to(torch.int32) - e0
        n_in = rows_in.shape[0]
        assert int(ids_in.min()) >= 0 and int(ids_in.max()) < e1 - e0
        moe_l = rt.MoeGroupedScratch.new(e1 - e0, n_in)
        rt.launch_moe_sort(moe_l, ids_in.contiguous(), n_in)
        y_l = torch.empty(n_in, out_dim, device="cuda")
        gg.gate_up(moe_l, et_local, rows_in, 1, y_l, n_in)                 # perm indexes the received rows
        y_in = torch.empty(n_in, out_dim, device="cuda")
        rt.launch_moe_scatter_rows(moe_l, y_l, y_in, out_dim, n_in)
        torch.cuda.synchronize()
        got = sh.combine_rows(y_in, plan)
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"expert-parallel result differs: rel {float((got - want).norm() / want.norm()):.3e}"

        # the same layer with the exchange done by the GPUs themselves (peer stores, two peer barriers per step, no
        # host in the loop), from BlockQ8 rows: equal to the reference's launch sequence on one GPU with all experts,
        # over both receive buffers
        xq = torch.empty(n_tok * (hidden // 32) * 40, dtype=torch.uint8, device="cuda")
        ep = rt.ExpertParallel(et_local, hidden, out_dim, cap=n_ent)
        for rnd in range(4):
            x2 = torch.from_numpy(np.random.default_rng(70 + 10 * rnd + rank).standard_normal((n_tok, hidden)).astype(np.float32)).cuda()
            rt.launch_quantize_q8(x2, xq, hidden, n_tok)
            moe2 = rt.MoeGroupedScratch.new(n_expert, n_ent)
            rt.launch_moe_sort(moe2, flat_ids.contiguous(), n_ent)
            xg = torch.empty(n_ent * (hidden // 32) * 40, dtype=torch.uint8, device="cuda")
            rt.launch_moe_gather_xq(moe2, xq, xg, hidden // 32, n_used, n_ent)
            ys = torch.zeros(n_ent, out_dim, device="cuda")
            rt.launch_moe_grouped_gemm(moe2, et_all, xg, ys, hidden, out_dim, n_ent)
            want2 = torch.zeros(n_ent, out_dim, device="cuda")
            rt.launch_moe_scatter_rows(moe2, ys, want2, out_dim, n_ent)
            got2 = torch.empty(n_ent, out_dim, device="cuda")
            ep.step(flat_ids.contiguous(), xq, n_ent, n_used, got2)
            torch.cuda.synchronize()
            assert torch.equal(got2, want2), f"device-driven expert parallelism, round {rnd}: differs from the one-GPU layer"
        st = __import__("ctypes").c_uint(0)
        assert rt._lib.load().rc_device_status(__import__("ctypes").byref(st)) == 0 and st.value == 0, hex(st.value)
        ep.close()
        q.put((rank, "ok"))
    except Exception as e:  # report instead of leaving the peer waiting
        q.put((rank, f"{type(e).__name__}: {e}"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_expert_parallel_grouped_gemm_two_gpus():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_moe_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert all(msg == "ok" for _, msg in results), results
