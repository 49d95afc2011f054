"""Forward kernel chain (logits -> softmax -> o = S.V) and the autograd wrapper against the CPU oracle.

Tolerances: o is bf16 and the probabilities pass through bf16 before the S.V product (the oracle keeps
them in fp32), so max-abs <= 2^-6 * max|o| and cosine >= 0.9999; lse (fp32, ex2.approx) to 2e-4 absolute.
"""
import pytest
import torch

from oracle.sparse_mla_ref import cosine, sparse_mla_bwd_ref, sparse_mla_fwd_ref
from test_operator_b200.inputs import LOG2E, WORKLOADS, Workload, make_sequence

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

CASES = [
    ("h16", 9, 256, 16, 64, 0.1),
    ("h64", 5, 512, 64, 256, 0.1),
    ("h128", 5, 512, 128, 256, 0.05),
    ("h128_ragged", 3, 300, 128, 96, 0.2),
    ("h128_long", 2, 4096, 128, 1024, 0.1),
]


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_forward_matches_oracle(case):
    from test_operator_b200 import op
    name, s_q, s_kv, h_q, topk, inv = case
    w = Workload(name, 1, s_q, s_kv, h_q, topk, "uniform", invalid_frac=inv)
    s = make_sequence(w, device="cpu", seed=23, with_forward=False)
    s["indices"][0, : topk // 2] = -1
    if s_q > 2:
        s["indices"][2] = s_kv + 1            # a query without any valid slot
    o_ref, lse_ref = sparse_mla_fwd_ref(s["q"], s["kv"], s["indices"], q_start_index_s=None)
    o, lse = op.mla_fwd(s["q"].to(DEV), s["kv"].to(DEV), s["indices"].to(DEV), q_start_index_s=None,
                        check_device_status=True)
    o, lse = o.float().cpu(), lse.cpu()
    fin = torch.isfinite(lse_ref)
    assert torch.equal(torch.isinf(lse), ~fin)
    assert torch.allclose(lse[fin], lse_ref[fin] * LOG2E, rtol=0, atol=2e-4)
    assert (o - o_ref.float()).abs().max().item() <= 2 ** -6 * o_ref.float().abs().max().item()
    assert cosine(o, o_ref) > 0.9999
    if s_q > 2:
        assert torch.all(o[2] == 0)


def test_forward_natural_log_and_causal():
    from test_operator_b200 import op
    w = Workload("fc", 1, 8, 64, 64, 64, "uniform")
    s = make_sequence(w, device="cpu", seed=5, with_forward=False)
    o_ref, lse_ref = sparse_mla_fwd_ref(s["q"], s["kv"], s["indices"], q_start_index_s=20)
    o, lse = op.mla_fwd(s["q"].to(DEV), s["kv"].to(DEV), s["indices"].to(DEV), q_start_index_s=20, lse_is_base2=False,
                        check_device_status=True)
    fin = torch.isfinite(lse_ref)
    assert torch.allclose(lse.cpu()[fin], lse_ref[fin], rtol=0, atol=2e-4)
    assert cosine(o.float().cpu(), o_ref) > 0.9999


def test_autograd_wrapper_round_trip():
    """sparse_mla(q, kv, idx).backward(dO): gradients equal the oracle backward fed with the oracle forward."""
    from test_operator_b200 import op
    w = Workload("ag", 1, 6, 512, 128, 128, "uniform", invalid_frac=0.1)
    s = make_sequence(w, device="cpu", seed=29)
    q = s["q"].to(DEV).requires_grad_(True)
    kv = s["kv"].to(DEV).requires_grad_(True)
    o = op.sparse_mla(q, kv, s["indices"].to(DEV), q_start_index_s=None)
    o.backward(s["dO"].to(DEV))
    dq_ref, dkv_ref = sparse_mla_bwd_ref(s["q"], s["kv"], s["dO"], s["lse"], s["O"], s["indices"], q_start_index_s=None)
    assert cosine(q.grad.float().cpu(), dq_ref) > 0.9995
    assert cosine(kv.grad.float().cpu(), dkv_ref) > 0.9995


def test_forward_full_size_query_subset():
    from test_operator_b200 import op
    w = WORKLOADS["head128"]
    s = make_sequence(w, device=DEV, seed=42, s_q_override=10, with_forward=False)
    o_ref, lse_ref = sparse_mla_fwd_ref(s["q"].cpu(), s["kv"].cpu(), s["indices"].cpu(), q_start_index_s=None)
    o, lse = op.mla_fwd(s["q"], s["kv"], s["indices"], q_start_index_s=None, check_device_status=True)
    assert torch.allclose(lse.cpu(), lse_ref * LOG2E, rtol=0, atol=3e-4)
    assert cosine(o.float().cpu(), o_ref) > 0.9999


@pytest.mark.parametrize("name", ["dqphase_full_topk_window", "dqphase_partial_causal_window"])
def test_forward_and_natural_log_backward_against_reference_phase_test_golden(name):
    """Vectors made by the reference's phase-test checker (`dq_test/test_dq_phase.py:39-66`, see
    tests/golden/make_golden_fwd.py): the forward's o / lse, and - fed with that natural-log lse, that o and the query
    start - the backward's S, dS (stage check) and dQ.  Its two cases: query start 63 and 0, [s_kv, 1, 576] kv and
    [s_q, 1, topk] indices, out-of-range sentinel s_kv."""
    import os
    import numpy as np
    from oracle.sparse_mla_ref import calc_diff
    from tests.golden.make_golden_fwd import make_fwd_case_inputs
    from test_operator_b200 import op
    q, kv, dO, indices, q_start = make_fwd_case_inputs(name)
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", f"{name}.npz"))
    rows = torch.from_numpy(g["rows"]).long()
    qd, kvd, dOd, idxd = q.to(DEV), kv.to(DEV), dO.to(DEV), indices.to(DEV)
    o, lse = op.mla_fwd(qd, kvd, idxd, q_start_index_s=q_start, lse_is_base2=False, check_device_status=True)
    assert torch.allclose(lse.cpu(), torch.from_numpy(g["lse"]), rtol=0, atol=2e-4)
    o_gold = torch.from_numpy(g["o_bits"]).view(torch.bfloat16).float()
    assert (o[rows.to(DEV)].float().cpu() - o_gold).abs().max().item() <= 2 ** -6 * o_gold.abs().max().item()
    assert cosine(o[rows.to(DEV)].float().cpu(), o_gold) > 0.9999
    # backward with the golden forward outputs (all 32 queries come from the restated forward, pinned bit for bit to
    # the reference on CPU; the stored rows are the ones compared)
    o_ref, lse_ref = sparse_mla_fwd_ref(q, kv.squeeze(1), indices.squeeze(1), q_start_index_s=q_start)
    ws = op.workspace_for(qd, kvd, idxd)
    dq = torch.empty_like(qd)
    dkv = torch.empty(kvd.shape, dtype=torch.float32, device=DEV)
    lay = op.run_stages(qd, kvd, dOd, lse_ref.to(DEV), o_ref.to(DEV), idxd, dq, dkv, ws, op.STAGE_ALL,
                        q_start_index_s=q_start, lse_is_base2=False)
    assert op.device_status(ws) == 0
    dq_gold = torch.from_numpy(g["dQ_bits"]).view(torch.bfloat16).float()
    mx, rel = calc_diff(dq_gold, dq[rows.to(DEV)].float().cpu())
    assert rel < 1e-2 and cosine(dq_gold, dq[rows.to(DEV)].float().cpu()) > 0.99999      # the phase test's own gate is rel < 1e-2
    S, dS = (m.cpu() for m in op.scratch_matrices(ws, lay))
    S_gold = torch.from_numpy(g["S_bits"]).view(torch.bfloat16).float().transpose(1, 2)      # [query, slot, head]
    dS_gold = torch.from_numpy(g["dS_bits"]).view(torch.bfloat16).float().transpose(1, 2)
    for mine, gold in ((S[rows, :64, :128].float(), S_gold), (dS[rows, :64, :128].float(), dS_gold)):
        err = (mine - gold).abs()
        assert torch.all(err <= 2 ** -7 * gold.abs() + 2e-4 * gold.abs().max())


def test_forward_over_packed_sequences_with_a_query_table():
    """Two sequences of different length packed along the first dimension, one forward call: the per-query table
    tells the kernels which kv rows a query may touch, its causal position and how many of its slots are in use."""
    from test_operator_b200 import op
    shapes = [(7, 200), (12, 333)]
    topk, h_q = 64, 64
    seqs = [make_sequence(Workload("fv", 1, sq, skv, h_q, topk, "uniform", invalid_frac=0.1), device="cpu", seed=70 + i,
                          with_forward=False) for i, (sq, skv) in enumerate(shapes)]
    q = torch.cat([s["q"] for s in seqs]).to(DEV)
    kv = torch.cat([s["kv"] for s in seqs]).to(DEV)
    idx = torch.cat([s["indices"] for s in seqs]).to(DEV)
    lens = torch.randint(1, topk + 1, (q.shape[0],), generator=torch.Generator().manual_seed(3), dtype=torch.int32)
    meta = op.query_meta_for([0, 7], [7, 12], [0, 200], [200, 333], DEV, 150, topk, lens)
    o, lse = op.mla_fwd(q, kv, idx, q_start_index_s=150, query_meta=meta, check_device_status=True)
    r0 = 0
    for s, (sq, skv) in zip(seqs, shapes):
        ii = s["indices"].clone()
        ii[torch.arange(topk)[None, :] >= lens[r0:r0 + sq, None].long()] = -1
        o_ref, lse_ref = sparse_mla_fwd_ref(s["q"], s["kv"], ii, q_start_index_s=150)
        fin = torch.isfinite(lse_ref)
        got = lse[r0:r0 + sq].cpu()
        assert torch.equal(torch.isinf(got), ~fin)
        assert torch.allclose(got[fin], lse_ref[fin] * LOG2E, rtol=0, atol=2e-4)
        assert cosine(o[r0:r0 + sq].float().cpu(), o_ref) > 0.9999
        r0 += sq


def test_forward_many_queries_repeats_bit_for_bit_and_matches_oracle():
    """More queries than SMs: every CTA of the logits kernels walks through several queries with its ring, accumulator
    buffers and counters running on, and four threads issue its UMMAs (two per tile stream, handing over through a
    counter).  o and lse must come out bit-identical in every run, and all queries are compared with the oracle
    (the same fp32 arithmetic on the GPU)."""
    from test_operator_b200 import op
    w = Workload("fwd_repeat", 1, 700, 1024, 128, 512, "uniform", invalid_frac=0.1)
    s = make_sequence(w, device=DEV, seed=78, with_forward=False)
    q, kv, idx = s["q"], s["kv"], s["indices"]
    first = None
    for _ in range(12):
        o, lse = op.mla_fwd(q, kv, idx, q_start_index_s=None, check_device_status=True)
        if first is None:
            first = (o.clone(), lse.clone())
        else:
            assert torch.equal(o.view(torch.int16), first[0].view(torch.int16))
            assert torch.equal(lse.view(torch.int32), first[1].view(torch.int32))
    o_ref, lse_ref = sparse_mla_fwd_ref(q, kv, idx, q_start_index_s=None)
    assert torch.allclose(first[1], lse_ref.to(first[1].device) * LOG2E, rtol=0, atol=3e-4)
    o_f, o_r = first[0].float(), o_ref.to(first[0].device).float()
    assert (o_f - o_r).abs().max().item() <= 2.0 ** -6 * o_r.abs().max().item()
    assert cosine(o_f.cpu(), o_r.cpu()) > 0.9999
