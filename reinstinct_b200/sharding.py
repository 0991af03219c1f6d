"""Host-side sharding of the quantized-weight hot path across the GPUs of one box.

The reference has no collectives (its multi-GPU mode is layer pipelining over
hipMemcpyPeerAsync, src/runtime/pipeline.rs:1-19); the path itself shards in two natural ways:

  * matvec / batched matvec / dense MMQ split by OUTPUT ROWS.  Rows of every GGUF format are
    independent (src/runtime/qwen35.rs:247-250), so rank g takes on-disk rows
    [g*out/G, (g+1)*out/G), repacks them as a tensor of its own (nsp depends on in_dim only) and
    the outputs are all-gathered.  Shard sizes are kept multiples of 32 rows so that
    quantize-then-gather equals gather-then-quantize for a following layer.
  * MoE grouped GEMMs split by EXPERTS: rank g owns experts [g*E/G, (g+1)*E/G); tokens stay
    data-parallel and their routed BlockQ8 rows travel by all-to-all (counts first, then the
    rows), are sorted locally by expert, and the f32 results travel back the same way.

Everything here is plain torch + torch.distributed and works on any backend (NCCL on the GPUs,
gloo in the CPU tests); no kernel is launched from this file.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch
import torch.distributed as dist

from .synth import BLOCK_BYTES, BLOCK_WEIGHTS

ROW_MULTIPLE = 32


def row_shard_range(out_dim: int, rank: int, world: int, multiple: int = ROW_MULTIPLE) -> tuple[int, int]:
    """Rows [begin, end) of rank `rank`: units of `multiple` rows dealt out as evenly as
    possible, the remainder (out_dim % multiple) going to the last rank."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world {world}")
    units = out_dim // multiple
    base, extra = divmod(units, world)
    begin = (rank * base + min(rank, extra)) * multiple
    end = begin + (base + (1 if rank < extra else 0)) * multiple
    if rank == world - 1:
        end = out_dim
    return begin, end


def shard_raw_rows(raw, dtype: int, in_dim: int, out_dim: int, rank: int, world: int) -> tuple[np.ndarray, int]:
    """The on-disk bytes of this rank's rows and their count."""
    row_bytes = (in_dim // BLOCK_WEIGHTS[dtype]) * BLOCK_BYTES[dtype]
    raw = np.asarray(raw, dtype=np.uint8).reshape(-1)
    if raw.size < row_bytes * out_dim:
        raise ValueError("raw buffer shorter than out_dim rows")
    b, e = row_shard_range(out_dim, rank, world)
    return raw[b * row_bytes:e * row_bytes], e - b


def col_shard_range(in_dim: int, rank: int, world: int, block: int) -> tuple[int, int]:
    """Columns [begin, end) of rank `rank` when a contraction of in_dim columns is dealt out in whole blocks of `block`
    columns (the weight format's block: 256 for the K-quants, 32 otherwise), as evenly as possible, the ranks with the
    larger share last."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world {world}")
    if in_dim % block:
        raise ValueError("in_dim is not a whole number of blocks")
    units = in_dim // block
    base, extra = divmod(units, world)
    first_big = world - extra
    begin = (rank * base + max(0, rank - first_big)) * block
    end = begin + (base + (1 if rank >= first_big else 0)) * block
    return begin, end


def shard_raw_cols(raw, dtype: int, in_dim: int, out_dim: int, begin: int, end: int) -> np.ndarray:
    """The on-disk bytes of columns [begin, end) of every row (whole blocks), as a tensor [out_dim][end - begin] of its own."""
    bw, bb = BLOCK_WEIGHTS[dtype], BLOCK_BYTES[dtype]
    if begin % bw or end % bw or not 0 <= begin < end <= in_dim:
        raise ValueError("column range must be whole blocks inside the row")
    rows = np.asarray(raw, dtype=np.uint8).reshape(-1)[: out_dim * (in_dim // bw) * bb].reshape(out_dim, in_dim // bw, bb)
    return np.ascontiguousarray(rows[:, begin // bw:end // bw, :]).reshape(-1)


def all_gather_rows(y_local: torch.Tensor, out_dim: int, group=None) -> torch.Tensor:
    """[n_rows, out_local] shards (any sizes) -> [n_rows, out_dim] on every rank."""
    world = dist.get_world_size(group)
    n_rows = y_local.shape[0]
    sizes = [row_shard_range(out_dim, r, world) for r in range(world)]
    widest = max(e - b for b, e in sizes)
    padded = torch.zeros((n_rows, widest), dtype=y_local.dtype, device=y_local.device)
    padded[:, :y_local.shape[1]] = y_local
    flat = torch.empty((world * n_rows, widest), dtype=y_local.dtype, device=y_local.device)
    dist.all_gather_into_tensor(flat, padded.contiguous(), group=group)
    parts = flat.view(world, n_rows, widest)
    out = torch.empty((n_rows, out_dim), dtype=y_local.dtype, device=y_local.device)
    for r, (b, e) in enumerate(sizes):
        out[:, b:e] = parts[r, :, :e - b]
    return out


# ---- expert parallelism ---------------------------------------------------------------------


def expert_range(n_expert: int, rank: int, world: int) -> tuple[int, int]:
    base, extra = divmod(n_expert, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def expert_owner(expert_ids: torch.Tensor, n_expert: int, world: int) -> torch.Tensor:
    """Owning rank of every expert id (same split as expert_range)."""
    base, extra = divmod(n_expert, world)
    cut = extra * (base + 1)
    e = expert_ids.to(torch.int64)
    big = torch.div(e, base + 1, rounding_mode="floor")
    small = extra + torch.div(e - cut, max(base, 1), rounding_mode="floor")
    return torch.where(e < cut, big, small).to(torch.int64)


@dataclass
class DispatchPlan:
    """How this rank's routed entries travel: `order` sorts local entries (tok*n_used + slot) by
    destination rank (stable), `send_counts[r]` of them go to rank r, `recv_counts[r]` arrive
    from rank r."""
    order: torch.Tensor
    send_counts: list[int]
    recv_counts: list[int]


def plan_dispatch(ids: torch.Tensor, n_expert: int, group=None) -> DispatchPlan:
    """ids: int32 [n_tok_local * n_used].  Exchanges the per-rank counts (one small all-to-all)."""
    world = dist.get_world_size(group)
    dest = expert_owner(ids.reshape(-1), n_expert, world)
    order = torch.argsort(dest, stable=True)
    send = torch.bincount(dest, minlength=world).to(torch.int64)
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return DispatchPlan(order, [int(v) for v in send.tolist()], [int(v) for v in recv.tolist()])


def dispatch_rows(rows: torch.Tensor, plan: DispatchPlan, group=None) -> torch.Tensor:
    """rows [n_entries_local, width] in entry order -> the rows this rank's experts must process,
    grouped by source rank."""
    sendbuf = rows[plan.order].contiguous()
    recvbuf = torch.empty((sum(plan.recv_counts), rows.shape[1]), dtype=rows.dtype, device=rows.device)
    dist.all_to_all_single(recvbuf, sendbuf, plan.recv_counts, plan.send_counts, group=group)
    return recvbuf


def combine_rows(rows: torch.Tensor, plan: DispatchPlan, group=None) -> torch.Tensor:
    """Inverse of dispatch_rows for per-entry results: returns [n_entries_local, width] in the
    original entry order."""
    back = torch.empty((sum(plan.send_counts), rows.shape[1]), dtype=rows.dtype, device=rows.device)
    dist.all_to_all_single(back, rows.contiguous(), plan.send_counts, plan.recv_counts, group=group)
    out = torch.empty_like(back)
    out[plan.order] = back
    return out


# ---- failure detection on the host --------------------------------------------------------------
#
# A rank may only leave between steps, with none of its kernels or collectives in flight.  The others
# must learn of it on the host before their next launch: a device-side wait on a peer that is gone would
# merely run out (rc_device_status bit 16) after the step's outputs are already lost.


class RankLeft(RuntimeError):
    def __init__(self, ranks):
        super().__init__(f"ranks {sorted(ranks)} left the job")
        self.ranks = sorted(ranks)


def announce_leave(store, rank: int) -> None:
    """Called by a rank that is about to leave (between steps)."""
    store.set(f"reinstinct/left/{rank}", b"1")


def departed_ranks(store, world: int) -> list[int]:
    """Ranks that have announced their leave (a non-blocking look at the rendezvous store)."""
    return [r for r in range(world) if store.check([f"reinstinct/left/{r}"])]


def check_peers_alive(store, world: int) -> None:
    """Raises RankLeft if any rank has announced its leave; call before every sharded launch."""
    gone = departed_ranks(store, world)
    if gone:
        raise RankLeft(gone)
