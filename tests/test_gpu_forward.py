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
