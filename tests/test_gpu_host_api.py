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


def test_reduction_rate_probe_adds_what_it_claims():
    """The probe's figure is bytes / time, so the bytes must be real: every launch adds exactly one to
    n_ctas x rows_per_cta x row_floats elements (whole rows, so every row holds one integer value)."""
    import ctypes
    from test_operator_b200 import op
    lib = op.load_library()
    n_rows, row_floats, rows_per_cta, n_ctas = 512, 576, 64, 7
    buf = torch.zeros(n_rows, row_floats, dtype=torch.float32, device="cuda:0")
    rc = lib.smla_reduction_rate_probe(ctypes.c_void_p(buf.data_ptr()), n_rows, row_floats, rows_per_cta, n_ctas,
                                       ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    assert buf.sum(dtype=torch.float64).item() == n_ctas * rows_per_cta * row_floats
    assert torch.equal(buf, buf[:, :1].expand_as(buf))
    assert lib.smla_reduction_rate_probe(None, n_rows, row_floats, rows_per_cta, n_ctas, None) == 1      # bad argument
    assert op.reduction_rate_gbs(4096, torch.device("cuda:0"), rows_per_cta=512) > 100.0
