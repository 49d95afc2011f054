"""Multi-GPU drivers for the sparse MLA backward: one process per GPU, `torch.distributed` for plumbing.

The reference has no distributed code.  The two shardings below are the ones its operator admits:
  * batch-sharded: sequences are independent (own q / kv / indices / dKV), so sequence b simply runs on
    rank b % world_size and nothing is exchanged;
  * query-sharded: one long sequence, queries split into contiguous blocks; kv is replicated, every
    rank accumulates a full-size fp32 partial dKV from its queries, and the partials are summed with a
    reduce-scatter (rank r ends up owning kv rows [r*s_kv/R, (r+1)*s_kv/R)).  dQ rows need no exchange.
The collective is a real exchange step of the algorithm (a sum over query shards), not decoration.  It comes in
two forms: NCCL's reduce-scatter (`reduce_scatter_dkv`), and `PullReducer`, a kernel of this library in which every
rank pulls its rows of the other ranks' partials over NVLink with plain loads, adds them in rank order and clears
what it has read, so that the next step starts from clean partials without a memset.
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


class PullReducer:
    """The ranks' partial dKV buffers in symmetric memory (every rank's buffer mapped into every process of the node)
    and the pull-reduce kernel `smla_dkv_pull_reduce` in place of NCCL's reduce-scatter.

    `partial` is this rank's [s_kv, 576] fp32 buffer: pass it to the operator as `out_dkv`.  With `zero_sources=True`
    every `reduce()` leaves all partials at zero again (each rank clears the rows it has read, in every rank's buffer),
    so the operator can run with `accumulate=True` and no memset; that saves a 151 MB local clear per step but sends as
    many zeros over NVLink as data was read, which costs more than it saves from four ranks up (the links are the
    bound) - hence off by default.  `reduce()` runs on the current stream between two cross-rank barriers of the
    symmetric-memory handle: every rank must call it once per step, like a collective.  torch provides the memory mapping and the
    barriers; the reduction itself is this library's kernel.  Two forms: plain peer loads (always available), and -
    where the symmetric memory also has an NVSwitch multicast mapping and `multimem=True` - `multimem.ld_reduce`, which
    lets the switch add the ranks' copies so that a rank receives only its reduced rows."""

    def __init__(self, s_kv: int, device, group: Optional[dist.ProcessGroup] = None, multimem: bool = False,
                 zero_sources: bool = False):
        import ctypes
        import torch.distributed._symmetric_memory as symm_mem
        from . import op
        group = group if group is not None else dist.group.WORLD
        self.world, self.rank, self.s_kv = dist.get_world_size(group), dist.get_rank(group), s_kv
        self.rows = kv_rows_of_rank(s_kv, self.rank, self.world)
        try:
            symm_mem.enable_symm_mem_for_group(group.group_name)     # needed by older torch releases, harmless later
        except Exception:
            pass
        self.partial = symm_mem.empty((s_kv, op.D_QK), dtype=torch.float32, device=device)
        self.partial.zero_()
        self.hdl = symm_mem.rendezvous(self.partial, group)
        offset = int(getattr(self.hdl, "offset", 0) or 0)
        ptrs = [int(p) + offset for p in self.hdl.buffer_ptrs]
        if ptrs[self.rank] != self.partial.data_ptr():
            raise RuntimeError("symmetric memory handle does not describe the partial buffer")
        self._ptrs = (ctypes.c_void_p * self.world)(*ptrs)
        mc = int(getattr(self.hdl, "multicast_ptr", 0) or 0)
        self.multicast_ptr = mc + offset if mc else 0
        self.multimem = bool(multimem and self.multicast_ptr)
        self.zero_sources = bool(zero_sources)
        self._lib = op.load_library()
        self._raise = op._raise_status

    def reduce(self, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Sum of all ranks' partials over this rank's rows [s_kv / R, 576] (and, with `zero_sources`, clear them)."""
        n = self.rows[1] - self.rows[0]
        if out is None:
            out = torch.empty(n, self.partial.shape[1], dtype=torch.float32, device=self.partial.device)
        stream = torch.cuda.current_stream().cuda_stream
        self.hdl.barrier(channel=0)            # every rank's backward has finished writing its partial
        z = 1 if self.zero_sources else 0
        if self.multimem:
            st = self._lib.smla_dkv_multimem_reduce(self.multicast_ptr, self.world, self.rank, self.s_kv, out.data_ptr(), z, stream)
        else:
            st = self._lib.smla_dkv_pull_reduce(self._ptrs, self.world, self.rank, self.s_kv, out.data_ptr(), z, stream)
        self._raise(self._lib, st, "smla_dkv_pull_reduce")
        self.hdl.barrier(channel=1)            # every rank has finished reading (and clearing) before anyone writes again
        return out


def query_sharded_bwd(bwd_fn, q_blk, kv, dO_blk, lse_blk, O_blk, idx_blk, q_row0: int,
                      q_start_index_s: Optional[int], partial: Optional[torch.Tensor] = None,
                      group: Optional[dist.ProcessGroup] = None, reducer: Optional[PullReducer] = None, **kw):
    """Backward of this rank's query block, then the sum of the ranks' partial dKV.

    `bwd_fn` has the operator's signature (`mla_bwd`).  The causal bound is expressed relative to
    the query's global row, so the block's first row shifts it.  With `reducer` the partial lives in symmetric
    memory and the sum is the library's NVLink pull-reduce; otherwise NCCL's reduce-scatter.
    Returns (dQ block, owned dKV rows).
    """
    qs = None if q_start_index_s is None else q_start_index_s + q_row0
    if reducer is not None:
        # partials the previous reduce() left clear are accumulated into; otherwise the operator clears them first
        dq, _ = bwd_fn(q_blk, kv, dO_blk, lse_blk, O_blk, idx_blk, q_start_index_s=qs, out_dkv=reducer.partial,
                       accumulate=reducer.zero_sources, **kw)
        return dq, reducer.reduce()
    if partial is None:
        partial = torch.empty(kv.shape, dtype=torch.float32, device=kv.device)
    dq, part = bwd_fn(q_blk, kv, dO_blk, lse_blk, O_blk, idx_blk, q_start_index_s=qs, out_dkv=partial, **kw)
    flat = part.reshape(part.shape[0], part.shape[-1])
    return dq, reduce_scatter_dkv(flat, group)
