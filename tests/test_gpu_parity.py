"""GPU parity tests: the CUDA path (through the C ABI) against the CPU oracle and the golden vectors.

Tolerances (bf16 inputs, fp32 accumulation, dQ rounded to bf16, dKV summed by fp32 atomics in
arbitrary order): the reference's own gate `rel_diff < 0.01` (`mla_bwd/test_mla_bwd.py:191-193`),
tightened with cosine similarity >= 0.99999 and max-abs error <= 2^-7 * max|ref| for dQ (one bf16
rounding of the output) and <= 1e-3 * max|ref| for dKV.  Slots with an invalid index must
contribute exactly nothing (bit-exact checks below).
"""
import os

import numpy as np
import pytest
import torch

from oracle.sparse_mla_ref import calc_diff, cosine, sparse_mla_bwd_ref, valid_mask
from tests.golden.make_golden import CASES, make_case_inputs
from test_operator_b200.inputs import LOG2E, WORKLOADS, Workload, make_sequence

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
DEV = "cuda:0"


def _op():
    from test_operator_b200 import op
    return op


def _to_dev(*ts):
    return [t.to(DEV) for t in ts]


def _assert_close(dq, dkv, dq_ref, dkv_ref):
    dq = dq.float().cpu()
    dkv = dkv.float().cpu().reshape(dkv_ref.shape)
    dq_ref_b = dq_ref.bfloat16().float()
    mq, rq = calc_diff(dq_ref_b, dq)
    mk, rk = calc_diff(dkv_ref, dkv)
    assert rq < 0.01 and rk < 0.01, (rq, rk)
    assert cosine(dq_ref, dq) > 0.99999 and cosine(dkv_ref, dkv) > 0.99999
    assert mq <= 2 ** -7 * dq_ref.abs().max().item() + 1e-6, mq
    assert mk <= 1e-3 * dkv_ref.abs().max().item() + 1e-6, mk


def _run(seq, **kw):
    op = _op()
    d = _to_dev(seq["q"], seq["kv"], seq["dO"], seq["lse"], seq["O"], seq["indices"])
    kw.setdefault("q_start_index_s", seq.get("q_start_index_s"))
    return op.mla_bwd(*d, check_device_status=True, **kw)


@pytest.mark.parametrize("name", sorted(CASES))
def test_golden_vectors_made_by_the_reference(name):
    """Reference defaults (causal bound with query start 0, base-2 lse) against the reference's own outputs."""
    q, kv, dO, lse, O, idx = make_case_inputs(name)
    g = np.load(os.path.join(GOLD, f"{name}.npz"))
    dq, dkv = _op().mla_bwd(*_to_dev(q, kv, dO, lse, O, idx), check_device_status=True)
    _assert_close(dq, dkv, torch.from_numpy(g["dQ"]), torch.from_numpy(g["dKV"]))


CASES_SMALL = [
    # name, s_q, s_kv, h_q, topk, index mode, invalid fraction
    ("tiny_cfg", 64, 256, 16, 64, "uniform", 0.10),
    ("h64", 5, 512, 64, 256, "uniform", 0.10),
    ("h128", 5, 512, 128, 256, "uniform", 0.05),
    ("h128_ragged_topk", 3, 300, 128, 96, "uniform", 0.2),     # top-k not a multiple of any tile
    ("h32_small_topk", 4, 64, 32, 8, "uniform", 0.0),
    ("h8_one_query", 1, 40, 8, 40, "uniform", 0.3),
    ("h128_all_slots_invalid_some_rows", 6, 128, 128, 64, "uniform", 0.0),
    ("h128_skewed", 4, 2048, 128, 128, "skewed", 0.1),
    # more queries than the persistent recompute clusters / dkv CTAs of a B200: every CTA walks over several queries
    ("h128_many_queries", 401, 1024, 128, 256, "uniform", 0.1),
    ("h64_many_queries_two_tiles", 333, 700, 64, 300, "uniform", 0.05),
]


@pytest.mark.parametrize("case", CASES_SMALL, ids=[c[0] for c in CASES_SMALL])
def test_small_cases_against_oracle(case):
    name, s_q, s_kv, h_q, topk, mode, inv = case
    w = Workload(name, 1, s_q, s_kv, h_q, topk, mode, invalid_frac=inv, recent_window=256)
    seq = make_sequence(w, device="cpu", seed=17)
    if "all_slots_invalid" in name:
        seq["indices"][1] = -1
        seq["indices"][4] = s_kv + 5
    ref = sparse_mla_bwd_ref(seq["q"], seq["kv"], seq["dO"], seq["lse"], seq["O"], seq["indices"], q_start_index_s=None)
    dq, dkv = _run(seq)
    _assert_close(dq, dkv, *ref)
    if "all_slots_invalid" in name:
        assert torch.all(dq[1] == 0) and torch.all(dq[4] == 0)


def test_duplicate_indices_and_3d_layouts():
    """The same kv row twice in one query adds twice; kv [s_kv,1,576] / indices [s_q,1,topk] are accepted."""
    w = Workload("dup", 1, 4, 64, 64, 64, "uniform")
    seq = make_sequence(w, device="cpu", seed=3)
    seq["indices"][:, 32:] = seq["indices"][:, :32]
    seq["O"], lse = __import__("test_operator_b200.inputs", fromlist=["forward_o_lse"]).forward_o_lse(
        seq["q"], seq["kv"], seq["indices"])
    seq["lse"] = lse
    ref = sparse_mla_bwd_ref(seq["q"], seq["kv"], seq["dO"], seq["lse"], seq["O"], seq["indices"], q_start_index_s=None)
    op = _op()
    q, kv, dO, lse, O, idx = _to_dev(seq["q"], seq["kv"], seq["dO"], seq["lse"], seq["O"], seq["indices"])
    dq, dkv = op.mla_bwd(q, kv.unsqueeze(1), dO, lse, O, idx.unsqueeze(1), q_start_index_s=None, check_device_status=True)
    assert dkv.shape == (64, 1, 576)
    _assert_close(dq, dkv, *ref)


def test_invalid_slots_are_masked_bit_exactly():
    w = Workload("mask", 1, 6, 256, 128, 128, "uniform", invalid_frac=0.3)
    seq = make_sequence(w, device="cpu", seed=5)
    idx = seq["indices"]
    dq, dkv = _run(seq)
    ok = valid_mask(idx, w.s_kv, None)
    touched = torch.zeros(w.s_kv, dtype=torch.bool)
    touched[idx[ok].long()] = True
    raw = dkv.cpu().view(torch.int32)
    assert torch.all(raw[~touched] == 0), "rows no valid slot points at must stay +0.0 bitwise"
    # other invalid values in the unused slots: dQ bitwise identical
    seq2 = dict(seq)
    junk = torch.where(torch.arange(idx.numel()).view_as(idx) % 2 == 0, torch.full_like(idx, -12345),
                       torch.full_like(idx, w.s_kv + 77))
    seq2["indices"] = torch.where(ok, idx, junk)
    dq2, dkv2 = _run(seq2)
    assert torch.equal(dq.view(torch.int16), dq2.view(torch.int16))
    assert torch.allclose(dkv, dkv2, rtol=0, atol=1e-5 * dkv.abs().max().item())


def test_causal_bound_and_query_start():
    w = Workload("causal", 1, 8, 64, 64, 64, "uniform")
    seq = make_sequence(w, device="cpu", seed=9)
    for qs in (0, 20):
        ref = sparse_mla_bwd_ref(seq["q"], seq["kv"], seq["dO"], seq["lse"], seq["O"], seq["indices"], q_start_index_s=qs)
        dq, dkv = _run(seq, q_start_index_s=qs)
        _assert_close(dq, dkv, *ref)


def test_natural_log_lse_and_custom_scale():
    w = Workload("opts", 1, 4, 128, 64, 64, "uniform", invalid_frac=0.1)
    seq = make_sequence(w, device="cpu", seed=21)
    ref = sparse_mla_bwd_ref(seq["q"], seq["kv"], seq["dO"], seq["lse"] / LOG2E, seq["O"], seq["indices"],
                             q_start_index_s=None, lse_is_base2=False)
    seq_n = dict(seq)
    seq_n["lse"] = (seq["lse"] / LOG2E).contiguous()
    dq, dkv = _run(seq_n, lse_is_base2=False)
    _assert_close(dq, dkv, *ref)
    ref = sparse_mla_bwd_ref(seq["q"], seq["kv"], seq["dO"], seq["lse"] + 1.0, seq["O"], seq["indices"],
                             sm_scale=0.05, q_start_index_s=None)
    seq_s = dict(seq)
    seq_s["lse"] = seq["lse"] + 1.0
    dq, dkv = _run(seq_s, sm_scale=0.05)
    _assert_close(dq, dkv, *ref)


def test_stage_outputs_delta_s_ds():
    """Delta, and the bf16 S / dS the recompute kernel hands to the other two, against the oracle's."""
    op = _op()
    w = Workload("stages", 1, 3, 256, 128, 192, "uniform", invalid_frac=0.1)
    seq = make_sequence(w, device="cpu", seed=2)
    _, _, delta_ref, S_ref, dS_ref = sparse_mla_bwd_ref(seq["q"], seq["kv"], seq["dO"], seq["lse"], seq["O"],
                                                        seq["indices"], q_start_index_s=None, return_intermediates=True)
    q, kv, dO, lse, O, idx = _to_dev(seq["q"], seq["kv"], seq["dO"], seq["lse"], seq["O"], seq["indices"])
    assert torch.allclose(op.delta(O, dO).cpu(), delta_ref, rtol=1e-5, atol=1e-4)
    ws = op.workspace_for(q, kv, idx)
    dq = torch.empty_like(q)
    dkv = torch.empty(kv.shape, dtype=torch.float32, device=DEV)
    lay = op.run_stages(q, kv, dO, lse, O, idx, dq, dkv, ws, op.STAGE_DELTA | op.STAGE_RECOMPUTE, q_start_index_s=None)
    assert op.device_status(ws) == 0
    S, dS = (m.cpu() for m in op.scratch_matrices(ws, lay))
    assert torch.all(S[:, w.topk:] == 0) and torch.all(dS[:, w.topk:] == 0), "padding slots must be zero"
    # bf16 values may differ by one ulp where the fp32 value sits on a rounding boundary; dS additionally
    # carries the cancellation in (dP - Delta), so it gets an absolute term scaled by the tensor's range
    for mine, ref in ((S[:, :w.topk, :w.h_q], S_ref), (dS[:, :w.topk, :w.h_q], dS_ref)):
        err = (mine.float() - ref.float()).abs()
        assert torch.all(err <= 2 ** -7 * ref.float().abs() + 2e-4 * ref.float().abs().max())
        assert (err > 0).float().mean().item() < 0.05


def test_dq_is_deterministic_and_dkv_spread_is_small():
    w = Workload("det", 1, 8, 64, 128, 64, "uniform")   # 8 queries all hitting the same 64 rows: heavy contention
    seq = make_sequence(w, device="cpu", seed=4)
    a = _run(seq)
    b = _run(seq)
    assert torch.equal(a[0].view(torch.int16), b[0].view(torch.int16))
    spread = (a[1] - b[1]).abs().max().item()
    assert spread <= 1e-5 * a[1].abs().max().item()


def test_query_passes_and_accumulation_agree():
    """A small scratch budget (several passes over the queries) and accumulate-into-buffer give the same result."""
    op = _op()
    w = Workload("passes", 1, 7, 256, 64, 128, "uniform", invalid_frac=0.1)
    seq = make_sequence(w, device="cpu", seed=8)
    ref = sparse_mla_bwd_ref(seq["q"], seq["kv"], seq["dO"], seq["lse"], seq["O"], seq["indices"], q_start_index_s=None)
    dq, dkv = _run(seq, workspace_budget=3 * 128 * 64 * 4 + 4096)   # room for 2-3 queries per pass
    _assert_close(dq, dkv, *ref)
    d = _to_dev(seq["q"], seq["kv"], seq["dO"], seq["lse"], seq["O"], seq["indices"])
    acc = torch.zeros(w.s_kv, 576, dtype=torch.float32, device=DEV)
    dqs = []
    for r0, r1 in ((0, 3), (3, 7)):
        part = [d[0][r0:r1], d[1], d[2][r0:r1], d[3][r0:r1], d[4][r0:r1], d[5][r0:r1]]
        dq_p, _ = op.mla_bwd(*part, q_start_index_s=None, out_dkv=acc, accumulate=True, check_device_status=True)
        dqs.append(dq_p)
    _assert_close(torch.cat(dqs), acc, *ref)


def test_scaling_dO_by_two_scales_dQ_bit_exactly():
    w = Workload("lin", 1, 4, 256, 128, 128, "uniform")
    seq = make_sequence(w, device="cpu", seed=6)
    dq1, dkv1 = _run(seq)
    seq2 = dict(seq)
    seq2["dO"] = (seq["dO"].float() * 2).bfloat16()
    dq2, dkv2 = _run(seq2)
    assert torch.equal((dq1.float() * 2).bfloat16().view(torch.int16), dq2.view(torch.int16))
    assert torch.allclose(dkv1 * 2, dkv2, rtol=0, atol=1e-5 * dkv2.abs().max().item())


@pytest.mark.parametrize("name,n_check", [("head64", 12), ("head128", 12)])
def test_full_size_shapes_query_subset(name, n_check):
    """Full s_kv / h_q / top-k of the benchmark workloads; the query dimension is cut so the CPU oracle
    finishes in seconds (a query's dQ row and its dKV contribution do not depend on the other queries)."""
    w = WORKLOADS[name]
    seq = make_sequence(w, device=DEV, seed=42, s_q_override=n_check)
    cpu = {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in seq.items()}
    ref = sparse_mla_bwd_ref(cpu["q"], cpu["kv"], cpu["dO"], cpu["lse"], cpu["O"], cpu["indices"], q_start_index_s=None)
    dq, dkv = _run(cpu)
    _assert_close(dq, dkv, *ref)


def test_full_size_head128_properties():
    """Benchmark size (s_q 1024 of 4096 to bound test time, full everything else): properties that need no oracle."""
    op = _op()
    w = WORKLOADS["head128"]
    seq = make_sequence(w, device=DEV, seed=42, s_q_override=1024)
    q, kv, dO, lse, O, idx = (seq[k] for k in ("q", "kv", "dO", "lse", "O", "indices"))
    dq, dkv = op.mla_bwd(q, kv, dO, lse, O, idx, q_start_index_s=None, check_device_status=True)
    assert torch.isfinite(dq.float()).all() and torch.isfinite(dkv).all()
    # untouched kv rows stay exactly zero
    ok = (idx >= 0) & (idx < w.s_kv)
    touched = torch.zeros(w.s_kv, dtype=torch.bool, device=DEV)
    touched[idx[ok].long()] = True
    assert torch.all(dkv.view(torch.int32)[~touched] == 0)
    # the sum over two halves of the queries equals the whole (accumulation path, order-insensitive tolerance)
    acc = torch.zeros_like(dkv)
    for r0, r1 in ((0, 512), (512, 1024)):
        dq_p, _ = op.mla_bwd(q[r0:r1], kv, dO[r0:r1], lse[r0:r1], O[r0:r1], idx[r0:r1], q_start_index_s=None,
                             out_dkv=acc, accumulate=True, check_device_status=True)
        assert torch.equal(dq_p.view(torch.int16), dq[r0:r1].view(torch.int16))
    assert (acc - dkv).abs().max().item() <= 1e-4 * dkv.abs().max().item()
    # column sums of dKV for 32 queries against a dense torch evaluation on the GPU (no scatter involved there)
    n = 32
    dq_s, dkv_s = op.mla_bwd(q[:n], kv, dO[:n], lse[:n], O[:n], idx[:n], q_start_index_s=None, check_device_status=True)
    kg = kv[idx[:n].clamp(0, w.s_kv - 1).long()].float()                      # [n, topk, 576]
    p = torch.einsum("shd,std->sht", q[:n].float(), kg)
    s_ = torch.exp2(p * (576 ** -0.5) * LOG2E - lse[:n].unsqueeze(-1)) * ok[:n].unsqueeze(1)
    dp = torch.einsum("shv,stv->sht", dO[:n].float(), kg[..., :512])
    delta = (O[:n].float() * dO[:n].float()).sum(-1)
    ds = (s_ * (dp - delta.unsqueeze(-1)) * 576 ** -0.5).bfloat16().float()
    s_b = s_.bfloat16().float()
    want = torch.einsum("sht,shd->d", ds, q[:n].float())
    want[:512] += torch.einsum("sht,shv->v", s_b, dO[:n].float())
    got = dkv_s.sum(0)
    assert cosine(want.cpu(), got.cpu()) > 0.9999
    assert (want - got).abs().max().item() <= 1e-2 * want.abs().max().item()


def test_back_to_back_runs_repeat_bit_for_bit():
    """Twenty runs of a case with more queries than resident clusters (every cluster walks through several queries,
    the pipelines never drain in between): S, dS and dQ must come out bit-identical every time.  The hand-overs between
    the two CTAs of a cluster use relaxed cluster-scope arrivals (the release form costs hundreds of cycles per
    call); a stale read there would show up as a rare difference between runs."""
    op = _op()
    w = Workload("repeat", 1, 700, 1024, 128, 512, "uniform", invalid_frac=0.1)
    seq = make_sequence(w, device=DEV, seed=77)
    q, kv, dO, lse, O, idx = (seq[k] for k in ("q", "kv", "dO", "lse", "O", "indices"))
    ws = op.workspace_for(q, kv, idx)
    dq = torch.empty_like(q)
    dkv = torch.empty(kv.shape, dtype=torch.float32, device=DEV)
    first = None
    for _ in range(20):
        lay = op.run_stages(q, kv, dO, lse, O, idx, dq, dkv, ws, op.STAGE_ALL, q_start_index_s=None)
        S, dS = op.scratch_matrices(ws, lay)
        cur = (S.clone(), dS.clone(), dq.clone())
        if first is None:
            first = cur
        else:
            for a, b in zip(first, cur):
                assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    assert op.device_status(ws) == 0
    ref = sparse_mla_bwd_ref(q, kv, dO, lse, O, idx, q_start_index_s=None, chunk_s=16)
    _assert_close(dq, dkv, ref[0].cpu(), ref[1].cpu())


@pytest.mark.parametrize("h_q,topk,s_kv", [(128, 256, 300), (64, 96, 128), (16, 40, 64)])
def test_all_ones_known_answers(h_q, topk, s_kv):
    """All-ones inputs have exact integer answers, so a contraction that loses a K-step, a head or a key shows as a
    wrong integer (the reference pins its sub-steps the same way: `ds_unit_tests/ds_tmem/test_ds_tmem.py:61-66`,
    `ds_unit_tests/dkv_mma/test_dkv_mma.py:74-80`, `ds_unit_tests/dq_mma/test_dq_mma.py:69-74`).
    q = kv = dO = 1, O = 1/2, sm_scale = 1/16, lse = 576/16 (natural log):  P = 576, S = 1, dP = 512, Delta = 256,
    dS = (512 - 256)/16 = 16;  dQ = 16 x (valid slots of the query) in every element;  a dKV row touched by c slots holds
    c * h_q * 17 in its first 512 columns (S.dO + dS.Q) and c * h_q * 16 in the last 64 (dS.Q only)."""
    op = _op()
    s_q = 7
    g = torch.Generator().manual_seed(h_q + topk)
    idx = torch.stack([torch.randperm(s_kv, generator=g)[:topk] for _ in range(s_q)]).to(torch.int32)
    idx[torch.rand(s_q, topk, generator=g) < 0.25] = -1
    idx[3] = s_kv            # a query with no valid slot at all
    ones = lambda *shape: torch.ones(*shape, dtype=torch.bfloat16, device=DEV)
    q, kv, dO = ones(s_q, h_q, 576), ones(s_kv, 576), ones(s_q, h_q, 512)
    O = torch.full((s_q, h_q, 512), 0.5, dtype=torch.bfloat16, device=DEV)
    lse = torch.full((s_q, h_q), 576.0 / 16.0, dtype=torch.float32, device=DEV)
    dq, dkv = op.mla_bwd(q, kv, dO, lse, O, idx.to(DEV), sm_scale=1.0 / 16.0, q_start_index_s=None, lse_is_base2=False,
                         check_device_status=True)
    valid = (idx >= 0) & (idx < s_kv)
    n_valid = valid.sum(1)
    want_dq = (16.0 * n_valid).view(s_q, 1, 1).expand(s_q, h_q, 576)
    assert torch.equal(dq.float().cpu(), want_dq.float())
    count = torch.zeros(s_kv)
    count.index_add_(0, idx[valid].long(), torch.ones(int(valid.sum())))
    want_dkv = torch.cat([(count * h_q * 17.0).view(-1, 1).expand(s_kv, 512), (count * h_q * 16.0).view(-1, 1).expand(s_kv, 64)], 1)
    assert torch.equal(dkv.cpu(), want_dkv)
