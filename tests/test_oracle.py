"""CPU tests of the oracle: golden vectors made by the reference's own checker, and properties."""
import os

import numpy as np
import pytest
import torch

from oracle.sparse_mla_ref import (calc_diff, cosine, sparse_mla_bwd_ref, sparse_mla_fwd_ref,
                                   valid_mask)
from tests.golden.make_golden import CASES, input_digest, make_case_inputs
from test_operator_b200.inputs import LOG2E, WORKLOADS, forward_o_lse, make_sequence

GOLD = os.path.join(os.path.dirname(__file__), "golden")


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_matches_reference_golden(name):
    q, kv, dO, lse, O, idx = make_case_inputs(name)
    g = np.load(os.path.join(GOLD, f"{name}.npz"))
    assert str(g["digest"]) == input_digest([q, kv, dO, lse, O, idx]), "seeded inputs drifted"
    dq, dkv = sparse_mla_bwd_ref(q, kv, dO, lse, O, idx)
    # bit-identical where the BLAS is the one the vectors were made with; 1e-5 relative elsewhere
    for mine, ref in ((dq, g["dQ"]), (dkv, g["dKV"])):
        ref = torch.from_numpy(ref)
        tol = 1e-5 * ref.abs().max().item()
        assert (mine - ref).abs().max().item() <= tol


def test_invalid_slots_contribute_exactly_zero():
    q, kv, dO, lse, O, idx = make_case_inputs("ref_mixed_h64")
    dq, dkv = sparse_mla_bwd_ref(q, kv, dO, lse, O, idx, q_start_index_s=None)
    ok = valid_mask(idx, kv.shape[0], None)
    touched = torch.zeros(kv.shape[0], dtype=torch.bool)
    touched[idx[ok].long()] = True
    assert torch.all(dkv[~touched] == 0)
    # replacing invalid values by other invalid values changes nothing, bitwise
    idx2 = torch.where(ok, idx, torch.full_like(idx, -7))
    dq2, dkv2 = sparse_mla_bwd_ref(q, kv, dO, lse, O, idx2, q_start_index_s=None)
    assert torch.equal(dq, dq2) and torch.equal(dkv, dkv2)


def test_chunking_and_lse_base_do_not_matter():
    q, kv, dO, lse, O, idx = make_case_inputs("ref_mixed_h64")
    a = sparse_mla_bwd_ref(q, kv, dO, lse, O, idx, chunk_s=8)
    b = sparse_mla_bwd_ref(q, kv, dO, lse, O, idx, chunk_s=1)
    assert calc_diff(a[0], b[0])[0] < 1e-4 and calc_diff(a[1], b[1])[0] < 1e-3
    c = sparse_mla_bwd_ref(q, kv, dO, lse / LOG2E, O, idx, lse_is_base2=False)
    assert cosine(a[0], c[0]) > 0.99999 and cosine(a[1], c[1]) > 0.99999


def test_matches_autograd_of_dense_softmax():
    """With o/lse from the true forward, dQ and dKV are the gradients of sum(o*dO) (up to bf16 rounding)."""
    w = WORKLOADS["tiny"]
    d = make_sequence(w, device="cpu", seed=3)
    q, kv, dO, idx = d["q"], d["kv"], d["dO"], d["indices"]
    dq, dkv = sparse_mla_bwd_ref(q, kv, dO, d["lse"], d["O"], idx, q_start_index_s=None)
    qf = q.float().requires_grad_(True)
    kvf = kv.float().requires_grad_(True)
    ok = valid_mask(idx, w.s_kv, None)
    kg = kvf[idx.clamp(0, w.s_kv - 1).long()]                   # [s_q, topk, 576]
    p = torch.einsum("shd,std->sht", qf, kg) / (576 ** 0.5)
    p = p.masked_fill(~ok.unsqueeze(1), float("-inf"))
    o = torch.einsum("sht,stv->shv", torch.softmax(p, dim=-1), kg[..., :512])
    (o * dO.float()).sum().backward()
    assert cosine(dq, qf.grad) > 0.999
    assert cosine(dkv, kvf.grad) > 0.999


def test_forward_helpers_agree():
    w = WORKLOADS["tiny"]
    d = make_sequence(w, device="cpu", seed=5)
    o, lse = sparse_mla_fwd_ref(d["q"], d["kv"], d["indices"])
    assert torch.equal(o, d["O"])
    assert torch.allclose(lse * LOG2E, d["lse"], rtol=1e-6, atol=1e-6)


def test_workload_index_generators():
    for name in ("tiny", "head128", "query_sharded", "ref_script"):
        w = WORKLOADS[name]
        small = type(w)(**{**w.__dict__, "s_q": 8, "s_kv": min(w.s_kv, 8192), "topk": 64,
                           "causal_base": min(w.causal_base, 4096), "recent_window": 256})
        g = torch.Generator().manual_seed(1)
        idx = __import__("test_operator_b200.inputs", fromlist=["make_indices"]).make_indices(small, g, "cpu")
        assert idx.shape == (8, 64) and idx.dtype == torch.int32
        for r in range(8):
            v = idx[r][(idx[r] >= 0) & (idx[r] < small.s_kv)]
            assert v.unique().numel() == v.numel(), "valid indices of a query must be distinct"


@pytest.mark.parametrize("name", sorted(__import__("tests.golden.make_golden_fwd", fromlist=["FWD_CASES"]).FWD_CASES))
def test_forward_oracle_matches_reference_phase_test_golden(name):
    """o / lse of the restated forward, and S / dS / dQ of the restated backward fed with natural-log lse and a query
    start, against what the reference's phase-test checker (`dq_test/test_dq_phase.py:39-66`) produced."""
    from tests.golden.make_golden_fwd import make_fwd_case_inputs
    q, kv, dO, indices, q_start = make_fwd_case_inputs(name)
    g = np.load(os.path.join(GOLD, f"{name}.npz"))
    rows = torch.from_numpy(g["rows"]).long()
    o, lse = sparse_mla_fwd_ref(q, kv.squeeze(1), indices.squeeze(1), q_start_index_s=q_start)
    assert (lse - torch.from_numpy(g["lse"])).abs().max().item() <= 1e-4
    o_gold = torch.from_numpy(g["o_bits"]).view(torch.bfloat16)
    assert (o[rows].view(torch.int16) != o_gold.view(torch.int16)).float().mean().item() <= 1e-3
    dq, _, _, S, dS = sparse_mla_bwd_ref(q, kv.squeeze(1), dO, lse, o, indices.squeeze(1), q_start_index_s=q_start,
                                         lse_is_base2=False, return_intermediates=True)
    dq_gold = torch.from_numpy(g["dQ_bits"]).view(torch.bfloat16).float()
    assert calc_diff(dq_gold, dq[rows])[1] < 1e-2 and cosine(dq_gold, dq[rows]) > 0.9999
    # the reference keeps S / dS as [query, head, slot]; the oracle's intermediates are [query, slot, head]
    S_gold = torch.from_numpy(g["S_bits"]).view(torch.bfloat16).float().transpose(1, 2)
    dS_gold = torch.from_numpy(g["dS_bits"]).view(torch.bfloat16).float().transpose(1, 2)
    for mine, gold in ((S[rows].float(), S_gold), (dS[rows].float(), dS_gold)):
        err = (mine - gold).abs()
        assert torch.all(err <= 2 ** -7 * gold.abs() + 2e-4 * gold.abs().max())
