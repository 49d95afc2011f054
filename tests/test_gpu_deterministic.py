"""Reproducible dKV: the staged dKV kernel plus the segment sum over the index inverse (CSR by kv row) give the same
bits in every run, agree with the fp32-reduction path to the spread of its atomics, and with the oracle to the parity
tolerances - also when the staging buffer is small and the queries take several passes."""
import pytest
import torch

from oracle.sparse_mla_ref import sparse_mla_bwd_ref
from tests.metrics import assert_backward_close
from test_operator_b200.inputs import Workload, make_sequence

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
KEYS = ("q", "kv", "dO", "lse", "O", "indices")

CASES = [
    # heavy contention: 600 queries x 512 slots over 1024 rows, so every kv row collects about 300 contributions
    ("contended_h128", Workload("det128", 1, 600, 1024, 128, 512, "uniform", invalid_frac=0.1), None, 2 << 30),
    # several passes over the queries (staging for about 64 queries), skewed pattern, causal rule
    ("passes_h64", Workload("det64", 1, 300, 4096, 64, 320, "skewed", invalid_frac=0.1, recent_window=512), 3900, 64 * 512 * 2304),
    ("tiny_h16", Workload("det16", 1, 5, 64, 16, 40, "uniform", invalid_frac=0.3), None, 2 << 30),
]


@pytest.mark.parametrize("name,w,q_start,budget", CASES, ids=[c[0] for c in CASES])
def test_deterministic_dkv_repeats_bit_for_bit_and_matches(name, w, q_start, budget):
    from test_operator_b200 import op
    s = make_sequence(w, device=DEV, seed=51)
    args = [s[k] for k in KEYS]
    runs = [op.mla_bwd(*args, q_start_index_s=q_start, deterministic=True, staging_budget=budget, check_device_status=True)
            for _ in range(3)]
    for dq, dkv in runs[1:]:
        assert torch.equal(dq.view(torch.int16), runs[0][0].view(torch.int16))
        assert torch.equal(dkv.view(torch.int32), runs[0][1].view(torch.int32)), "dKV must repeat bit for bit"
    dq_a, dkv_a = op.mla_bwd(*args, q_start_index_s=q_start, check_device_status=True)       # fp32 reductions
    assert torch.equal(dq_a.view(torch.int16), runs[0][0].view(torch.int16))
    assert (dkv_a - runs[0][1]).abs().max().item() <= 1e-5 * dkv_a.abs().max().item()
    dq_ref, dkv_ref = sparse_mla_bwd_ref(*args, q_start_index_s=q_start, chunk_s=16)
    assert_backward_close(runs[0][0], runs[0][1], dq_ref, dkv_ref, name)
    # rows no valid slot points at stay +0.0 bitwise, as in the regular path
    idx = s["indices"]
    ok = (idx >= 0) & (idx < w.s_kv)
    if q_start is not None:
        ok &= idx <= q_start + torch.arange(w.s_q, device=DEV).unsqueeze(1)
    touched = torch.zeros(w.s_kv, dtype=torch.bool, device=DEV)
    touched[idx[ok].long()] = True
    assert torch.all(runs[0][1].view(torch.int32)[~touched] == 0)


def test_deterministic_accumulates_into_an_existing_buffer():
    from test_operator_b200 import op
    w = Workload("detacc", 1, 90, 512, 128, 256, "uniform", invalid_frac=0.1)
    s = make_sequence(w, device=DEV, seed=52)
    args = [s[k] for k in KEYS]
    whole = op.mla_bwd(*args, q_start_index_s=None, deterministic=True, check_device_status=True)[1]
    acc = torch.zeros_like(whole)
    for r0, r1 in ((0, 40), (40, 90)):
        part = [a[r0:r1] if i != 1 else a for i, a in enumerate(args)]
        op.mla_bwd(*part, q_start_index_s=None, deterministic=True, out_dkv=acc, accumulate=True, check_device_status=True)
    assert (acc - whole).abs().max().item() <= 1e-5 * whole.abs().max().item()
