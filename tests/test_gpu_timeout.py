"""The device-side timeout path, exercised without hanging anything.

Every wait inside the kernels (on an mbarrier or a shared-memory counter) is bounded: when its limit runs out it
records a code in the workspace's error word, raises the CTA's abort flag and returns, so the kernel ends normally and
the host reads SMLA_ERR_DEVICE_TIMEOUT - where the reference prints and carries on (`mla_bwd/mla_bwd.cu:814-818,
965-968`).  The self-test kernel waits, with a limit of a fraction of a millisecond, on a barrier nothing ever signals,
through the same three wait routines the kernels use.  Nothing here faults or hangs: the wait gives up by design.
"""
import pytest
import torch

from oracle.sparse_mla_ref import sparse_mla_bwd_ref
from tests.metrics import assert_backward_close
from test_operator_b200.inputs import Workload, make_sequence

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
KEYS = ("q", "kv", "dO", "lse", "O", "indices")


@pytest.mark.parametrize("which", [0, 1, 2], ids=["sleeping_wait", "spinning_wait", "counter_wait"])
def test_a_wait_that_runs_out_is_reported_and_the_workspace_stays_usable(which):
    from test_operator_b200 import op
    lib = op.load_library()
    w = Workload("after_timeout", 1, 5, 512, 128, 256, "uniform", invalid_frac=0.1)
    s = make_sequence(w, device=DEV, seed=3)
    args = [s[k] for k in KEYS]
    ws = op.workspace_for(s["q"], s["kv"], s["indices"])
    out = torch.full((3,), -1, dtype=torch.int64, device=DEV)
    limit = 200_000                                   # cycles: about 0.1 ms
    stream = torch.cuda.current_stream().cuda_stream
    assert op.device_status(ws) == 0
    assert lib.smla_selftest_wait_timeout(ws.ptr, which, limit, out.data_ptr(), stream) == 0
    # an ordinary call queued behind it on the same workspace must not erase the record
    dq, dkv = op.mla_bwd(*args, q_start_index_s=None, workspace=ws)
    assert op.device_status(ws) == 4                  # SMLA_ERR_DEVICE_TIMEOUT, kernel returned normally
    assert op.last_device_code() == 900 + 10 * which
    first, second, cycles = out.tolist()
    assert first == 0 and second == 0                 # the wait gave up; the next wait in the CTA returned at once
    assert limit <= cycles < 100 * limit
    assert op.device_status(ws) == 0                  # reported once, then cleared
    # and the results of the ordinary call are right
    dq_ref, dkv_ref = sparse_mla_bwd_ref(*args, q_start_index_s=None)
    assert_backward_close(dq, dkv, dq_ref, dkv_ref, "after a timeout")
    dq2, dkv2 = op.mla_bwd(*args, q_start_index_s=None, workspace=ws, check_device_status=True)
    assert torch.equal(dq.view(torch.int16), dq2.view(torch.int16))
