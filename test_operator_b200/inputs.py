"""Seeded synthetic workloads for the sparse MLA backward.

The shapes (h_q, d_qk = 512 latent + 64 rope, d_v = 512, top-k) are those the reference
operator is written for (`mla_bwd/mla_bwd.cuh:44-56`, `mla_bwd/test_mla_bwd.py:154-160`).
No dataset is involved: values are bf16 N(0,1), index patterns follow the named workloads.
`o` and base-2 `lse` come from a chunked fp32 torch forward that runs on whatever device
the tensors live on (the same arithmetic as `dq_test/test_dq_phase.py:53-59`).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Optional

import torch

LOG2E = 1.4426950408889634
D_QK = 576
D_V = 512


@dataclass(frozen=True)
class Workload:
    name: str
    batch: int          # independent sequences
    s_q: int
    s_kv: int
    h_q: int
    topk: int
    index_mode: str     # "uniform" | "causal_offset" | "skewed" | "causal_prefix"
    invalid_frac: float = 0.0
    causal_base: int = 0            # causal_offset: query i draws from [0, min(s_kv, causal_base + i))
    recent_window: int = 4096       # skewed: half of the slots come from the last `recent_window` rows
    q_start_index_s: Optional[int] = None

    @property
    def flops(self) -> float:
        """Algorithmic work: 5504 FLOPs per (query, head, top-k slot), padding slots included
        (`mla_bwd/test_mla_bwd.py:125-135,143`)."""
        return 5504.0 * self.batch * self.s_q * self.h_q * self.topk


WORKLOADS: Dict[str, Workload] = {
    # CPU-runnable tiny case
    "tiny": Workload("tiny", 1, 64, 256, 16, 64, "uniform", invalid_frac=0.10),
    "head64": Workload("head64", 1, 4096, 8192, 64, 2048, "uniform"),
    "head128": Workload("head128", 1, 4096, 32768, 128, 2048, "causal_offset",
                        invalid_frac=0.05, causal_base=28672),
    "batch_sharded": Workload("batch_sharded", 8, 8192, 16384, 128, 2048, "uniform"),
    "query_sharded": Workload("query_sharded", 1, 16384, 65536, 128, 2048, "skewed",
                              invalid_frac=0.10),
    # the reference script's own case (`mla_bwd/test_mla_bwd.py:154-185`): causal prefix + s_kv sentinel
    "ref_script": Workload("ref_script", 1, 4096, 8192, 128, 2048, "causal_prefix", q_start_index_s=0),
}


def _distinct_rows(n_rows: int, k: int, limits: torch.Tensor, gen: torch.Generator, device) -> torch.Tensor:
    """Row i gets k distinct integers uniform in [0, limits[i]) (limits[i] >= k), via top-k of random keys."""
    out = torch.empty(n_rows, k, dtype=torch.int32, device=device)
    max_lim = int(limits.max().item())
    step = max(1, min(n_rows, (1 << 26) // max(max_lim, 1)))
    col = torch.arange(max_lim, device=device).unsqueeze(0)
    for r0 in range(0, n_rows, step):
        r1 = min(r0 + step, n_rows)
        keys = torch.rand(r1 - r0, max_lim, generator=gen, device=device)
        keys = torch.where(col < limits[r0:r1].unsqueeze(1), keys, torch.full_like(keys, -1.0))
        out[r0:r1] = keys.topk(k, dim=1).indices.to(torch.int32)
    return out


def make_indices(w: Workload, gen: torch.Generator, device) -> torch.Tensor:
    """int32 [s_q, topk] for one sequence of workload `w`."""
    s_q, s_kv, topk = w.s_q, w.s_kv, w.topk
    if w.index_mode == "uniform":
        lim = torch.full((s_q,), s_kv, dtype=torch.int64, device=device)
        idx = _distinct_rows(s_q, topk, lim, gen, device)
    elif w.index_mode == "causal_offset":
        lim = torch.clamp(w.causal_base + torch.arange(s_q, device=device), max=s_kv)
        idx = _distinct_rows(s_q, topk, lim, gen, device)
    elif w.index_mode == "skewed":
        half = topk // 2
        win = min(w.recent_window, s_kv)
        lim = torch.full((s_q,), win, dtype=torch.int64, device=device)
        recent = _distinct_rows(s_q, half, lim, gen, device) + (s_kv - win)
        # the other half: uniform over the rows outside the recent window, so that all slots stay distinct
        lim2 = torch.full((s_q,), s_kv - win, dtype=torch.int64, device=device)
        if s_kv - win >= topk - half:
            rest = _distinct_rows(s_q, topk - half, lim2, gen, device)
        else:
            rest = torch.full((s_q, topk - half), -1, dtype=torch.int32, device=device)
        idx = torch.cat([recent, rest], dim=1)
        perm = torch.rand(s_q, topk, generator=gen, device=device).argsort(dim=1)
        idx = torch.gather(idx, 1, perm)
    elif w.index_mode == "causal_prefix":
        # row t: min(t+1, topk) distinct values from [0, t], the rest = s_kv (out-of-range sentinel)
        idx = torch.full((s_q, topk), s_kv, dtype=torch.int32, device=device)
        n_small = min(s_q, topk)
        for t in range(n_small):
            idx[t, : t + 1] = torch.randperm(t + 1, generator=gen, device=device).to(torch.int32)
        if s_q > topk:
            lim = torch.arange(topk, s_q, device=device) + 1
            idx[topk:] = _distinct_rows(s_q - topk, topk, lim, gen, device)
    else:
        raise ValueError(w.index_mode)
    if w.invalid_frac > 0:
        drop = torch.rand(s_q, topk, generator=gen, device=device) < w.invalid_frac
        idx = torch.where(drop, torch.full_like(idx, -1), idx)
    return idx.contiguous()


@torch.no_grad()
def forward_o_lse(q, kv, indices, sm_scale: Optional[float] = None,
                  q_start_index_s: Optional[int] = None, chunk_s: int = 16):
    """fp32 torch forward on the tensors' device: returns (o bf16, lse fp32 in base-2 units)."""
    s_q, h_q, d_qk = q.shape
    s_kv = kv.shape[0]
    scale = sm_scale if sm_scale is not None else 1.0 / math.sqrt(d_qk)
    kf = kv.reshape(s_kv, d_qk)
    ok = (indices >= 0) & (indices < s_kv)
    if q_start_index_s is not None:
        pos = q_start_index_s + torch.arange(s_q, device=q.device).unsqueeze(1)
        ok = ok & (indices <= pos)
    safe = indices.clamp(0, s_kv - 1).long()
    o = torch.empty(s_q, h_q, D_V, dtype=torch.bfloat16, device=q.device)
    lse2 = torch.empty(s_q, h_q, dtype=torch.float32, device=q.device)
    ninf = torch.tensor(float("-inf"), device=q.device)
    pinf = torch.tensor(float("inf"), device=q.device)
    for s0 in range(0, s_q, chunk_s):
        s1 = min(s0 + chunk_s, s_q)
        kg = kf.index_select(0, safe[s0:s1].reshape(-1)).view(s1 - s0, -1, d_qk).float()
        p = torch.matmul(q[s0:s1].float(), kg.transpose(-2, -1))
        logits = torch.where(ok[s0:s1].unsqueeze(1), p, ninf) * scale
        l = torch.logsumexp(logits, dim=-1)
        l = torch.where(torch.isinf(l) & (l < 0), pinf, l)
        s = torch.exp(logits - l.unsqueeze(-1))
        o[s0:s1] = torch.matmul(s, kg[..., :D_V]).to(torch.bfloat16)
        lse2[s0:s1] = l * LOG2E
    return o, lse2


@torch.no_grad()
def make_sequence(w: Workload, seq: int = 0, device="cpu", seed: int = 42, with_forward: bool = True,
                  s_q_override: Optional[int] = None):
    """One sequence of workload `w`: dict(q, kv, dO, lse, O, indices).  `lse` is base-2.

    `s_q_override` keeps only the first rows of the query dimension (a bounded sample of
    the same workload: per-query cost does not depend on s_q).
    """
    gen = torch.Generator(device=device)
    gen.manual_seed(seed * 1000003 + seq * 7919 + sum(map(ord, w.name)))
    if s_q_override is not None and s_q_override < w.s_q:
        w = Workload(**{**w.__dict__, "s_q": s_q_override})
    q = torch.randn(w.s_q, w.h_q, D_QK, generator=gen, device=device, dtype=torch.float32).to(torch.bfloat16)
    kv = torch.randn(w.s_kv, D_QK, generator=gen, device=device, dtype=torch.float32).to(torch.bfloat16)
    dO = torch.randn(w.s_q, w.h_q, D_V, generator=gen, device=device, dtype=torch.float32).to(torch.bfloat16)
    indices = make_indices(w, gen, device)
    if with_forward:
        O, lse = forward_o_lse(q, kv, indices, q_start_index_s=w.q_start_index_s)
    else:
        # the reference script's synthetic stand-ins (`mla_bwd/test_mla_bwd.py:175-177`)
        lse = torch.randn(w.s_q, w.h_q, generator=gen, device=device) * 2.0 + 5.0
        O = torch.randn(w.s_q, w.h_q, D_V, generator=gen, device=device).to(torch.bfloat16)
    return dict(q=q, kv=kv, dO=dO, lse=lse.contiguous(), O=O, indices=indices,
                q_start_index_s=w.q_start_index_s)
