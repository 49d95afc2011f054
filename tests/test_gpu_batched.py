"""Batched and variable-length entry points against the oracle run sequence by sequence."""
import pytest
import torch

from oracle.sparse_mla_ref import sparse_mla_bwd_ref
from tests.metrics import assert_backward_close
from test_operator_b200.inputs import Workload, make_sequence

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
KEYS = ("q", "kv", "dO", "lse", "O", "indices")


def _close(dq, dkv, dq_ref, dkv_ref):
    """Same tolerances as the single-sequence parity tests."""
    assert_backward_close(dq.cpu(), dkv.cpu().reshape(dkv_ref.shape), dq_ref, dkv_ref)


def test_batched_with_topk_length():
    from test_operator_b200 import op
    w = Workload("b", 1, 9, 320, 64, 96, "uniform", invalid_frac=0.1)
    seqs = [make_sequence(w, device="cpu", seed=31 + b) for b in range(3)]
    g = torch.Generator().manual_seed(5)
    lens = torch.randint(0, w.topk + 1, (3, w.s_q), generator=g, dtype=torch.int32)
    lens[0, 0] = 0                  # a query without any slot in use
    lens[1, :] = w.topk             # a sequence using every slot
    stacked = {k: torch.stack([s[k] for s in seqs]).to(DEV) for k in KEYS}
    dq, dkv = op.mla_bwd_batched(*[stacked[k] for k in KEYS], topk_length=lens.to(DEV), q_start_index_s=None)
    assert dq.shape == stacked["q"].shape and dkv.shape == stacked["kv"].shape and dkv.dtype == torch.float32
    for b, s in enumerate(seqs):
        idx = s["indices"].clone()
        idx[torch.arange(w.topk)[None, :] >= lens[b][:, None].long()] = -1
        dq_ref, dkv_ref = sparse_mla_bwd_ref(s["q"], s["kv"], s["dO"], s["lse"], s["O"], idx, q_start_index_s=None)
        _close(dq[b], dkv[b], dq_ref, dkv_ref)
    assert torch.all(dq[0, 0] == 0)


def test_varlen_sequences_of_different_length():
    from test_operator_b200 import op
    shapes = [(5, 200), (0, 0), (17, 333), (1, 64)]          # (queries, kv rows); the second sequence is empty
    topk, h_q = 48, 128
    seqs = []
    for i, (s_q, s_kv) in enumerate(shapes):
        if s_q:
            seqs.append(make_sequence(Workload("v", 1, s_q, s_kv, h_q, topk, "uniform", invalid_frac=0.1), device="cpu", seed=40 + i))
    cat = {k: torch.cat([s[k] for s in seqs]).to(DEV) for k in KEYS}
    cu_q, cu_kv = [0], [0]
    for s_q, s_kv in shapes:
        cu_q.append(cu_q[-1] + s_q)
        cu_kv.append(cu_kv[-1] + s_kv)
    dq, dkv = op.mla_bwd_varlen(*[cat[k] for k in KEYS], cu_q, torch.tensor(cu_kv), q_start_index_s=None)
    assert dq.shape == cat["q"].shape and dkv.shape == cat["kv"].shape
    it = iter(seqs)
    for i, (s_q, s_kv) in enumerate(shapes):
        if not s_q:
            continue
        s = next(it)
        dq_ref, dkv_ref = sparse_mla_bwd_ref(s["q"], s["kv"], s["dO"], s["lse"], s["O"], s["indices"], q_start_index_s=None)
        _close(dq[cu_q[i]:cu_q[i + 1]], dkv[cu_kv[i]:cu_kv[i + 1]], dq_ref, dkv_ref)


def test_varlen_rejects_bad_offsets():
    from test_operator_b200 import op
    s = make_sequence(Workload("v", 1, 4, 64, 16, 16, "uniform"), device="cpu", seed=3)
    dev = [s[k].to(DEV) for k in KEYS]
    with pytest.raises(RuntimeError):
        op.mla_bwd_varlen(*dev, [0, 3], [0, 64])            # does not cover q
    with pytest.raises(RuntimeError):
        op.mla_bwd_varlen(*dev, [0, 4], [0, 32, 64])        # lengths differ


def test_batched_large_enough_for_the_overlapped_schedule():
    """1200 packed queries: the per-query table and the two-stream schedule together (the small cases above run the
    kernels one after the other)."""
    from test_operator_b200 import op
    w = Workload("bl", 1, 400, 640, 128, 256, "uniform", invalid_frac=0.1)
    seqs = [make_sequence(w, device=DEV, seed=61 + b) for b in range(3)]
    stacked = {k: torch.stack([s[k] for s in seqs]) for k in KEYS}
    before = op.get_schedule()
    op.set_schedule(2, 0)
    try:
        dq, dkv = op.mla_bwd_batched(*[stacked[k] for k in KEYS], q_start_index_s=300, check_device_status=True)
        assert op.last_launch_count() == 1 + 3 * 2
    finally:
        op.set_schedule(*before)
    for b, s in enumerate(seqs):
        dq_ref, dkv_ref = sparse_mla_bwd_ref(*[s[k] for k in KEYS], q_start_index_s=300, chunk_s=16)
        assert_backward_close(dq[b], dkv[b], dq_ref, dkv_ref, f"sequence {b}")
