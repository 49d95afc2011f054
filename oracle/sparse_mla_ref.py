"""Oracle for the sparse MLA attention backward. TEST INFRASTRUCTURE ONLY.

This file restates, in plain fp32 PyTorch, the algorithm of the reference's own checker
(`mla_bwd/test_mla_bwd.py:18-90`, function `build_reference`) and of the forward used to
make `o`/`lse` (`dq_test/test_dq_phase.py:39-66`).  Nothing in the shipped package may
import it: only the tests, the smoke check and the CPU-baseline leg of the benchmark do,
and only as the checker or as the timed CPU baseline.

Parity pinning: the reference stores no golden vectors for this path (every test
regenerates seeded random inputs).  The restatement is therefore pinned against outputs
of the reference functions themselves, executed on CPU tensors: the backward by
`tests/golden/make_golden.py` (`build_reference` of `mla_bwd/test_mla_bwd.py`, bit-identical),
the forward and the natural-log-lse / query-start semantics by
`tests/golden/make_golden_fwd.py` (`build_reference` of `dq_test/test_dq_phase.py`);
the resulting vectors live in `tests/golden/*.npz`.

The functions are plain torch and run on whatever device their inputs live on: on CPU tensors they
are the CPU oracle (and the timed CPU baseline); on CUDA tensors the same fp32 arithmetic runs in
torch's own kernels, which lets the tests check every query of the full-size workloads in seconds,
as the reference's own script does (`mla_bwd/test_mla_bwd.py:93-112` builds its reference on the GPU).

Math contract (identical in the CUDA path):
    P      = Q . K_g^T                                  (K_g = kv rows gathered by `indices`)
    S      = exp2(P * sm_scale * log2(e) - lse2)        masked slots -> exactly 0
    Delta  = rowsum(O * dO)
    dP     = dO . V_g^T                                 (V = first d_v columns of kv)
    dS     = S * (dP - Delta) * sm_scale
    S, dS are rounded to bf16 (round-to-nearest-even) before the second-stage products
    dQ     = dS_bf16 . K_g
    dKV[idx, :d_v] += S_bf16^T . dO + dS_bf16^T . Q[:, :d_v]
    dKV[idx, d_v:] += dS_bf16^T . Q[:, d_v:]
A slot is valid when 0 <= idx < s_kv and, if a causal bound is given, idx <= q_start + row.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

LOG2E = 1.4426950408889634


def valid_mask(indices: torch.Tensor, s_kv: int, q_start_index_s: Optional[int]) -> torch.Tensor:
    """Boolean [s_q, topk]: which top-k slots take part.

    Follows `mla_bwd/test_mla_bwd.py:36,55-57` (range check and `idx <= query position`);
    `q_start_index_s=None` switches the causal term off, an int shifts the query position
    as `dq_test/test_dq_phase.py:48-49` does.
    """
    ok = (indices >= 0) & (indices < s_kv)
    if q_start_index_s is not None:
        pos = q_start_index_s + torch.arange(indices.shape[0], dtype=torch.int64, device=indices.device).unsqueeze(1)
        ok = ok & (indices.to(torch.int64) <= pos)
    return ok


def sparse_mla_fwd_ref(
    q: torch.Tensor,          # [s_q, h_q, d_qk] bf16
    kv: torch.Tensor,         # [s_kv, d_qk] bf16
    indices: torch.Tensor,    # [s_q, topk] int32
    d_v: int = 512,
    sm_scale: Optional[float] = None,
    q_start_index_s: Optional[int] = None,
    chunk_s: int = 8,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Forward that makes the backward's inputs: returns (o bf16 [s_q,h_q,d_v], lse fp32 natural log).

    Follows `dq_test/test_dq_phase.py:53-59`: logits = masked(P) * sm_scale, lse = logsumexp,
    o = softmax . V rounded to bf16.  A query with no valid slot gets lse = -inf there; this
    function returns lse = +inf for such rows so that every S becomes 0 downstream.
    """
    s_q, h_q, d_qk = q.shape
    s_kv = kv.shape[0]
    scale = sm_scale if sm_scale is not None else 1.0 / math.sqrt(d_qk)
    kf = kv.float()
    safe = indices.clamp(0, s_kv - 1).long()
    ok = valid_mask(indices, s_kv, q_start_index_s)
    dev = q.device
    o = torch.empty(s_q, h_q, d_v, dtype=torch.bfloat16, device=dev)
    lse = torch.empty(s_q, h_q, dtype=torch.float32, device=dev)
    neg_inf = torch.tensor(float("-inf"), device=dev)
    pos_inf = torch.tensor(float("inf"), device=dev)
    for s0 in range(0, s_q, chunk_s):
        s1 = min(s0 + chunk_s, s_q)
        kg = kf.index_select(0, safe[s0:s1].reshape(-1)).view(s1 - s0, -1, d_qk)
        p = torch.matmul(q[s0:s1].float(), kg.transpose(-2, -1))
        p = torch.where(ok[s0:s1].unsqueeze(1), p, neg_inf)
        logits = p * scale
        l = torch.logsumexp(logits, dim=-1)
        l = torch.where(torch.isinf(l) & (l < 0), pos_inf, l)
        s = torch.exp(logits - l.unsqueeze(-1))
        o[s0:s1] = torch.matmul(s, kg[..., :d_v]).to(torch.bfloat16)
        lse[s0:s1] = l
    return o, lse


def sparse_mla_bwd_ref(
    q: torch.Tensor,          # [s_q, h_q, d_qk] bf16
    kv: torch.Tensor,         # [s_kv, d_qk] bf16
    dO: torch.Tensor,         # [s_q, h_q, d_v] bf16
    lse: torch.Tensor,        # [s_q, h_q] fp32
    O: torch.Tensor,          # [s_q, h_q, d_v] bf16
    indices: torch.Tensor,    # [s_q, topk] int32
    sm_scale: Optional[float] = None,
    q_start_index_s: Optional[int] = 0,
    lse_is_base2: bool = True,
    chunk_s: int = 8,
    return_intermediates: bool = False,
):
    """fp32 backward; returns (dQ fp32 [s_q,h_q,d_qk], dKV fp32 [s_kv,d_qk]).

    Defaults reproduce `mla_bwd/test_mla_bwd.py:18-90` exactly: sm_scale = 1/sqrt(d_qk) (`:38`),
    base-2 lse (`:70`), causal bound with query start 0 (`:55-57`).  With
    `return_intermediates=True` also returns (delta fp32 [s_q,h_q], S bf16 and dS bf16 as
    [s_q, topk, h_q]) for stage-by-stage checks of the CUDA kernels.
    """
    s_q, h_q, d_qk = q.shape
    s_kv = kv.shape[0]
    topk = indices.shape[1]
    d_v = dO.shape[2]
    scale = float(sm_scale) if sm_scale is not None else 1.0 / (d_qk ** 0.5)
    # The reference multiplies by the truncated constant 1.44269504 (`:39`); keep it so
    # that the restatement is bit-identical to the reference on its own settings.
    scale_log2e = scale * 1.44269504
    lse2 = lse if lse_is_base2 else lse * LOG2E

    kf = kv.float()
    safe = indices.clamp(0, s_kv - 1).long()
    ok = valid_mask(indices, s_kv, q_start_index_s)

    dev = q.device
    dQ = torch.empty(s_q, h_q, d_qk, dtype=torch.float32, device=dev)
    dKV = torch.zeros(s_kv, d_qk, dtype=torch.float32, device=dev)
    if return_intermediates:
        delta_all = torch.empty(s_q, h_q, dtype=torch.float32, device=dev)
        S_all = torch.empty(s_q, topk, h_q, dtype=torch.bfloat16, device=dev)
        dS_all = torch.empty(s_q, topk, h_q, dtype=torch.bfloat16, device=dev)

    neg_inf = torch.tensor(float("-inf"), device=dev)
    for s0 in range(0, s_q, chunk_s):
        s1 = min(s0 + chunk_s, s_q)
        cs = s1 - s0
        qc = q[s0:s1].float()
        doc = dO[s0:s1].float()
        oc = O[s0:s1].float()
        flat = safe[s0:s1].reshape(-1)
        kg = kf.index_select(0, flat).view(cs, topk, d_qk)
        vg = kg[..., :d_v]
        okc = ok[s0:s1]

        p = torch.matmul(qc, kg.transpose(-2, -1))
        p = torch.where(okc.unsqueeze(1), p, neg_inf)
        dp = torch.matmul(doc, vg.transpose(-2, -1))
        delta = (oc * doc).sum(dim=-1)

        s = torch.exp2(p * scale_log2e - lse2[s0:s1].unsqueeze(-1))
        ds = s * (dp - delta.unsqueeze(-1)) * scale
        s_b = s.to(torch.bfloat16)
        ds_b = ds.to(torch.bfloat16)

        dQ[s0:s1] = torch.matmul(ds_b.float(), kg)

        # three separate products and (dV + dK_nope) as in `mla_bwd/test_mla_bwd.py:74-77`
        ds_t = ds_b.float().transpose(-2, -1)
        dv = torch.matmul(s_b.float().transpose(-2, -1), doc)
        dk_nope = torch.matmul(ds_t, qc[:, :, :d_v])
        dk_rope = torch.matmul(ds_t, qc[:, :, d_v:])
        dk = torch.cat([dv + dk_nope, dk_rope], dim=-1)
        sel = okc.reshape(-1)
        dKV.index_add_(0, flat[sel], dk.reshape(-1, d_qk)[sel])

        if return_intermediates:
            delta_all[s0:s1] = delta
            S_all[s0:s1] = s_b.transpose(-2, -1)
            dS_all[s0:s1] = ds_b.transpose(-2, -1)

    if return_intermediates:
        return dQ, dKV, delta_all, S_all, dS_all
    return dQ, dKV


def calc_diff(a: torch.Tensor, b: torch.Tensor) -> Tuple[float, float]:
    """(max abs diff, mean relative diff) exactly as `mla_bwd/test_mla_bwd.py:11-15`."""
    d = (a.float() - b.float()).abs()
    return d.max().item(), (d / (1e-4 + a.float().abs())).mean().item()


def cosine(a: torch.Tensor, b: torch.Tensor) -> float:
    a = a.double().flatten()
    b = b.double().flatten()
    den = (a.norm() * b.norm()).item()
    return 1.0 if den == 0 else (a @ b).item() / den
