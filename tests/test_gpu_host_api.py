"""Host-buffer entry point (pipelined copies) against the device entry point."""
import pytest
import torch

from test_operator_b200.inputs import Workload, make_sequence

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("q_start", [None, 40])
def test_host_entry_matches_device_entry(q_start):
    from test_operator_b200 import op
    w = Workload("host", 1, 37, 512, 64, 128, "uniform", invalid_frac=0.1)
    s = make_sequence(w, device="cpu", seed=19)
    host = [s[k].pin_memory() for k in ("q", "kv", "dO", "lse", "O", "indices")]
    dq_h, dkv_h = op.mla_bwd_host(*host, device="cuda:0", q_start_index_s=q_start, n_chunks=5)
    dev = [t.to("cuda:0") for t in host]
    dq_d, dkv_d = op.mla_bwd(*dev, q_start_index_s=q_start, check_device_status=True)
    from oracle.sparse_mla_ref import sparse_mla_bwd_ref
    from tests.metrics import assert_backward_close
    assert_backward_close(dq_d.cpu(), dkv_d.cpu(), *sparse_mla_bwd_ref(*host, q_start_index_s=q_start))
    assert not dq_h.is_cuda and not dkv_h.is_cuda
    assert torch.equal(dq_h.view(torch.int16), dq_d.cpu().view(torch.int16))
    assert (dkv_h - dkv_d.cpu()).abs().max().item() <= 1e-5 * dkv_d.abs().max().item()
