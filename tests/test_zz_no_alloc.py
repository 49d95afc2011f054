"""The allocation-free entry point (`smla_bwd_run_noalloc`) against the regular one.

This file sorts last on purpose: a run that stops at the first failure has then already run every
other test.  The entry point serves host code that may not allocate device memory (a plugin living
inside a framework that owns the whole GPU memory pool, or a loop that cannot afford the device-wide
synchronisation an allocation can cause); it draws its scratch from a 32 MiB array built into the
library.  Checked here, through the C ABI: same dQ bit for bit, same dKV up to the order of the fp32
atomics (1e-5 of the largest value, the tolerance the other dKV repeatability tests use), on two calls
in a row (the second call meets the scratch the first one left), with several passes over the query
dimension, and a clear refusal when even one query does not fit.
"""
import ctypes

import pytest
import torch

from test_operator_b200.inputs import Workload, make_sequence

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _params(op, t, dq, dkv, q_start):
    return op._make_params(t["q"], t["kv"], t["dO"], t["lse"], t["O"], t["indices"], dq, dkv, None, q_start, True)


def test_noalloc_entry_matches_regular_entry_twice_in_a_row():
    from test_operator_b200 import op
    lib = op.load_library()
    assert lib.smla_bwd_noalloc_capacity() == 32 << 20
    # h_q 128, topk 1024: 512 KiB of S/dS per query -> about 63 queries per pass, so 150 queries take 3 passes
    w = Workload("noalloc", 1, 150, 4096, 128, 1024, "uniform", invalid_frac=0.1)
    seq = make_sequence(w, device=DEV, seed=31)
    t = {k: v for k, v in seq.items() if torch.is_tensor(v)}
    stream = torch.cuda.current_stream().cuda_stream

    dq_ref, dkv_ref = op.mla_bwd(t["q"], t["kv"], t["dO"], t["lse"], t["O"], t["indices"], q_start_index_s=None,
                                 check_device_status=True)
    # the regular entry point is itself held to the oracle on this shape, so that "equal to it" means "right"
    from oracle.sparse_mla_ref import sparse_mla_bwd_ref
    from tests.metrics import assert_backward_close
    assert_backward_close(dq_ref, dkv_ref, *sparse_mla_bwd_ref(t["q"], t["kv"], t["dO"], t["lse"], t["O"], t["indices"],
                                                               q_start_index_s=None, chunk_s=16))
    for call in range(2):
        dq = torch.full_like(t["q"], float("nan"))
        dkv = torch.full(t["kv"].shape, float("nan"), dtype=torch.float32, device=DEV)
        p = _params(op, t, dq, dkv, None)
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        torch_before = torch.cuda.memory_allocated()
        st = lib.smla_bwd_run_noalloc(ctypes.byref(p), stream)
        assert st == 0, lib.smla_status_string(st)
        assert lib.smla_bwd_noalloc_status(stream) == 0
        if call == 1:
            # what the entry point is for: the device's free memory and torch's books are where they were (the first
            # call may still have made the driver load the kernels' code, so the second one is the one held to it)
            assert torch.cuda.mem_get_info()[0] == free_before
            assert torch.cuda.memory_allocated() == torch_before
        assert lib.smla_bwd_last_launch_count() >= 1 + 3 * 3      # Delta + three kernels per pass, three passes
        assert torch.equal(dq.view(torch.int16), dq_ref.view(torch.int16)), f"dQ differs on call {call}"
        assert (dkv - dkv_ref).abs().max().item() <= 1e-5 * dkv_ref.abs().max().item(), f"dKV differs on call {call}"


def test_noalloc_python_wrapper_validates_and_matches():
    from test_operator_b200 import op
    w = Workload("noalloc_py", 1, 40, 1024, 64, 256, "uniform", invalid_frac=0.1)
    seq = make_sequence(w, device=DEV, seed=32)
    t = {k: v for k, v in seq.items() if torch.is_tensor(v)}
    dq_ref, dkv_ref = op.mla_bwd(t["q"], t["kv"], t["dO"], t["lse"], t["O"], t["indices"], q_start_index_s=None,
                                 check_device_status=True)
    dq = torch.empty_like(t["q"])
    dkv = torch.empty(t["kv"].shape, dtype=torch.float32, device=DEV)
    op.mla_bwd_noalloc(t["q"], t["kv"], t["dO"], t["lse"], t["O"], t["indices"], dq, dkv, q_start_index_s=None)
    assert op.load_library().smla_bwd_noalloc_status(torch.cuda.current_stream().cuda_stream) == 0
    assert torch.equal(dq.view(torch.int16), dq_ref.view(torch.int16))
    assert (dkv - dkv_ref).abs().max().item() <= 1e-5 * dkv_ref.abs().max().item()
    with pytest.raises(RuntimeError):      # outputs of the wrong size or type never reach the kernels
        op.mla_bwd_noalloc(t["q"], t["kv"], t["dO"], t["lse"], t["O"], t["indices"], dq[:-1], dkv, q_start_index_s=None)
    with pytest.raises(RuntimeError):
        op.mla_bwd_noalloc(t["q"], t["kv"], t["dO"], t["lse"], t["O"], t["indices"], dq, dkv.double(), q_start_index_s=None)


def test_noalloc_entry_refuses_what_cannot_fit():
    from test_operator_b200 import op
    lib = op.load_library()
    # Delta alone (4 * s_q * h_q bytes) beyond 32 MiB: refused before anything is launched, pointers never touched
    p = op._Params(256, 256, 256, 256, 256, 256, 256, 256, 70000, 1024, 128, 64, 0.0, 0, 1)
    st = lib.smla_bwd_run_noalloc(ctypes.byref(p), None)
    assert st == 5
    assert b"built-in" in lib.smla_status_string(st)
    # one query's S/dS beyond 32 MiB (topk 70000 x 128 heads x 4 bytes)
    p = op._Params(256, 256, 256, 256, 256, 256, 256, 256, 4, 100000, 128, 70000, 0.0, 0, 1)
    assert lib.smla_bwd_run_noalloc(ctypes.byref(p), None) == 5
