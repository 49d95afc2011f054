"""Multi-GPU drivers for the sparse MLA backward: one process per GPU, `torch.distributed` for plumbing.

The reference has no distributed code.  The two shardings below are the ones its operator admits:
  * batch-sharded: sequences are independent (own q / kv / indices / dKV), so sequence b simply runs on
    rank b % world_size and nothing is exchanged;
  * query-sharded: one long sequence, queries split into contiguous blocks; kv is replicated, every
    rank accumulates a full-size fp32 partial dKV from its queries, and the partials are summed with a
    reduce-scatter (rank r ends up owning kv rows [r*s_kv/R, (r+1)*s_kv/R)).  dQ rows need no exchange.
The collective is a real exchange step of the algorithm (a sum over query shards), not decoration.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def sequences_of_rank(n_sequences: int, rank: int, world_size: int) -> List[int]:
    """Batch sharding: sequence ids owned by `rank` (round-robin)."""
    return [b for b in range(n_sequences) if b % world_size == rank]


def query_block(s_q: int, rank: int, world_size: int) -> Tuple[int, int]:
    """Query sharding: [start, stop) rows of the query dimension owned by `rank` (contiguous, balanced)."""
    base, rem = divmod(s_q, world_size)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def kv_rows_of_rank(s_kv: int, rank: int, world_size: int) -> Tuple[int, int]:
    """Rows of dKV a rank owns after the reduce-scatter; s_kv must divide evenly."""
    if s_kv % world_size:
        raise ValueError(f"s_kv={s_kv} must be divisible by world_size={world_size} for the reduce-scatter")
    n = s_kv // world_size
    return rank * n, (rank + 1) * n


def reduce_scatter_dkv(partial: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Sum the ranks' fp32 partial dKV [s_kv, 576]; returns this rank's row block [s_kv/R, 576]."""
    world = dist.get_world_size(group)
    if world == 1:
        return partial
    rank = dist.get_rank(group)
    r0, r1 = kv_rows_of_rank(partial.shape[0], rank, world)
    out = torch.empty((r1 - r0,) + tuple(partial.shape[1:]), dtype=partial.dtype, device=partial.device)
    if dist.get_backend(group) == "gloo":
        # gloo has no reduce_scatter_tensor: all-reduce, then keep the owned block
        full = partial.clone()
        dist.all_reduce(full, op=dist.ReduceOp.SUM, group=group)
        out.copy_(full[r0:r1])
    else:
        dist.reduce_scatter_tensor(out, partial, op=dist.ReduceOp.SUM, group=group)
    return out


def query_sharded_bwd(bwd_fn, q_blk, kv, dO_blk, lse_blk, O_blk, idx_blk, q_row0: int,
                      q_start_index_s: Optional[int], partial: Optional[torch.Tensor] = None,
                      group: Optional[dist.ProcessGroup] = None, **kw):
    """Backward of this rank's query block, then the dKV reduce-scatter.

    `bwd_fn` has the operator's signature (`mla_bwd`).  The causal bound is expressed relative to
    the query's global row, so the block's first row shifts it.  Returns (dQ block, owned dKV rows).
    """
    qs = None if q_start_index_s is None else q_start_index_s + q_row0
    if partial is None:
        partial = torch.empty(kv.shape, dtype=torch.float32, device=kv.device)
    dq, part = bwd_fn(q_blk, kv, dO_blk, lse_blk, O_blk, idx_blk, q_start_index_s=qs, out_dkv=partial, **kw)
    flat = part.reshape(part.shape[0], part.shape[-1])
    return dq, reduce_scatter_dkv(flat, group)
