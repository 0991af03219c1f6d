"""World-size-2 tests of the multi-GPU host logic on CPU (gloo): row sharding + all-gather of
matvec outputs, and the expert-parallel dispatch / combine plan.  The per-rank compute is done by
the CPU oracle here (test infrastructure); on GPUs the same plumbing moves the kernels' outputs."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import cases
import oracle as ro
from reinstinct_b200 import sharding as sh


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, fn_name: str, q):
    import datetime

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    # a short collective timeout: a peer that is gone ends the next collective with an error, not a hang
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    try:
        globals()[fn_name](rank, world)
        q.put((rank, "ok"))
    except Exception as e:  # report, do not hang the peer
        q.put((rank, f"{type(e).__name__}: {e}"))
    finally:
        dist.destroy_process_group()


def _run(fn_name: str, world: int = 2):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fn_name, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert all(msg == "ok" for _, msg in results), results


def _row_shard_case(rank: int, world: int):
    for t, in_dim, out_dim, n_rows in [(ro.Q4_K, 1024, 320, 1), (ro.Q6_K, 512, 259, 3), (ro.Q8_0, 256, 40, 2)]:
        raw, x = cases.synth_case(t, in_dim, out_dim, n_rows, seed=out_dim + t)
        xq = ro.quantize_q8(x)
        full32, _, _ = ro.matvec_q8(t, ro.repack(t, raw, in_dim, out_dim), xq, in_dim, out_dim, n_rows)
        part, rows = sh.shard_raw_rows(raw, t, in_dim, out_dim, rank, world)
        b, e = sh.row_shard_range(out_dim, rank, world)
        assert rows == e - b
        if rows:
            y_local, _, _ = ro.matvec_q8(t, ro.repack(t, part, in_dim, rows), xq, in_dim, rows, n_rows)
        else:
            y_local = np.zeros((n_rows, 0), dtype=np.float32)
        got = sh.all_gather_rows(torch.from_numpy(np.ascontiguousarray(y_local)), out_dim).numpy()
        # every row is computed by exactly one rank with the same arithmetic: bit-identical
        assert np.array_equal(got, full32.reshape(n_rows, out_dim))


def _expert_parallel_case(rank: int, world: int):
    n_expert, n_tok, n_used, width = 13, 20, 3, 80
    rng = np.random.default_rng(100 + rank)
    ids = torch.from_numpy(rng.integers(0, n_expert, n_tok * n_used, dtype=np.int32))
    rows = torch.from_numpy(rng.integers(0, 256, (n_tok * n_used, width), dtype=np.uint8))
    plan = sh.plan_dispatch(ids, n_expert)
    assert sum(plan.send_counts) == n_tok * n_used
    got_rows = sh.dispatch_rows(rows, plan)
    got_ids = sh.dispatch_rows(ids.reshape(-1, 1), plan).reshape(-1)
    lo, hi = sh.expert_range(n_expert, rank, world)
    assert bool(((got_ids >= lo) & (got_ids < hi)).all()), "a row reached a rank that does not own its expert"
    # stand-in for the expert FFN: depends on the expert and on every byte of the row
    y = (got_rows.to(torch.float32).sum(dim=1, keepdim=True) * (got_ids.to(torch.float32).reshape(-1, 1) + 1.0)).repeat(1, 4)
    back = sh.combine_rows(y, plan)
    want = (rows.to(torch.float32).sum(dim=1, keepdim=True) * (ids.to(torch.float32).reshape(-1, 1) + 1.0)).repeat(1, 4)
    assert torch.equal(back, want)


def _rank_leaves_announced_case(rank: int, world: int):
    """A rank leaves between steps and says so in the rendezvous store: the other learns of it on the host
    before its next launch."""
    store = dist.distributed_c10d._get_default_store()
    t = torch.ones(4) * (rank + 1)
    dist.all_reduce(t)  # step 1: everybody is there
    assert float(t[0]) == sum(range(1, world + 1))
    if rank == world - 1:
        sh.announce_leave(store, rank)
        return  # leaves: no collective in flight
    import time
    for _ in range(200):  # the survivors poll the store before their next step
        if sh.departed_ranks(store, world):
            break
        time.sleep(0.02)
    with pytest.raises(sh.RankLeft) as e:
        sh.check_peers_alive(store, world)
    assert e.value.ranks == [world - 1]


def _rank_leaves_silently_case(rank: int, world: int):
    """A rank leaves between steps without a word: the survivor's next collective ends with an error within
    the process group's timeout."""
    t = torch.ones(4)
    dist.all_reduce(t)
    if rank == world - 1:
        return
    import time
    t0 = time.time()
    with pytest.raises(Exception):
        for _ in range(3):  # the peer's sockets may outlive it by one call
            dist.all_reduce(t)
            time.sleep(0.5)
    assert time.time() - t0 < 60


def test_row_shard_ranges_cover_everything():
    for out_dim in (17408, 5120, 259, 40, 31, 64):
        for world in (1, 2, 3, 4, 8):
            spans = [sh.row_shard_range(out_dim, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == out_dim
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            assert all(b % 32 == 0 for b, _ in spans)
    owners = sh.expert_owner(torch.arange(13), 13, 4)
    for r in range(4):
        lo, hi = sh.expert_range(13, r, 4)
        assert bool((owners[lo:hi] == r).all())


def test_column_shards_partition_the_contraction_and_sum_to_the_whole():
    """The tensor-parallel split of the down projection: whole blocks of the format per rank, uneven shares last; the
    ranks' partial products (CPU oracle, exact integer dots per block) add up to the unsharded row products."""
    t, in_dim, out_dim = ro.Q6_K, 2304, 24
    for world in (1, 2, 4, 8):
        ranges = [sh.col_shard_range(in_dim, r, world, 256) for r in range(world)]
        assert ranges[0][0] == 0 and ranges[-1][1] == in_dim
        assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
        sizes = [e - b for b, e in ranges]
        assert all(s % 256 == 0 for s in sizes) and max(sizes) - min(sizes) <= 256 and sizes == sorted(sizes)
    raw, x = cases.synth_case(t, in_dim, out_dim, 1, seed=21)
    xq = ro.quantize_q8(x)
    _, want, _ = ro.matvec_q8(t, ro.repack(t, raw, in_dim, out_dim), xq, in_dim, out_dim, 1)
    world = 4
    total = np.zeros(out_dim, dtype=np.float64)
    for r in range(world):
        b, e = sh.col_shard_range(in_dim, r, world, 256)
        part = sh.shard_raw_cols(raw, t, in_dim, out_dim, b, e)
        xq_part = np.asarray(xq).reshape(-1, 40)[b // 32:e // 32].reshape(-1)
        _, y, _ = ro.matvec_q8(t, ro.repack(t, part, e - b, out_dim), xq_part, e - b, out_dim, 1)
        total += np.asarray(y, dtype=np.float64).reshape(-1)
    assert ro.rel_l2(total, np.asarray(want, dtype=np.float64).reshape(-1)) < 1e-6
    with pytest.raises(ValueError):
        sh.shard_raw_cols(raw, t, in_dim, out_dim, 32, 288)


def test_row_sharded_matvec_two_ranks():
    _run("_row_shard_case")


def test_expert_parallel_dispatch_two_ranks():
    _run("_expert_parallel_case")


def test_rank_that_leaves_is_seen_in_the_store():
    _run("_rank_leaves_announced_case")


def test_rank_that_leaves_silently_ends_the_next_collective_with_an_error():
    _run("_rank_leaves_silently_case")
