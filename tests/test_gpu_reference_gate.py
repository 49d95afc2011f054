"""The reference's own end-to-end gate, through the extension module of the reference's name.

`mla_bwd/test_mla_bwd.py:149-207` builds S = 4096 queries, S_KV = 8192, 128 heads, top-k 2048, a causal-prefix index
pattern with the out-of-range sentinel S_KV, synthetic lse / O, calls `mla_bwd_cuda.mla_bwd(q, kv, dO, lse, O,
indices)` with exactly these six arguments and passes when both rel_diff figures are below 0.01
(`:93-112,191-193`; rel_diff = mean |a - b| / (1e-4 + |a|) with a = the operator's output, `:11-15`).  The same
steps run here against the `mla_bwd_cuda` module that `python setup.py build_ext --inplace` builds from this
repository, with the oracle (the restated `build_reference`) evaluated on the GPU over all queries.
"""
import pytest
import torch

from oracle.sparse_mla_ref import calc_diff, sparse_mla_bwd_ref

pytestmark = pytest.mark.gpu


def test_reference_gate_through_the_extension_module():
    from tests.conftest import import_extension
    mla_bwd_cuda = import_extension()        # the compiled extension; no Python stand-in exists
    assert mla_bwd_cuda.__file__.endswith(".so")
    S, B_H, D_Q, S_KV, B_TOPK, D_V = 4096, 128, 576, 8192, 2048, 512
    torch.manual_seed(42)
    q = torch.randn(S, B_H, D_Q, dtype=torch.bfloat16, device="cuda")
    kv = torch.randn(S_KV, D_Q, dtype=torch.bfloat16, device="cuda")
    dO = torch.randn(S, B_H, D_V, dtype=torch.bfloat16, device="cuda")
    lse = torch.randn(S, B_H, dtype=torch.float32, device="cuda") * 2.0 + 5.0
    O = torch.randn(S, B_H, D_V, dtype=torch.bfloat16, device="cuda")
    indices = torch.full((S, B_TOPK), S_KV, dtype=torch.int32, device="cuda")
    for t in range(S):
        n_valid = min(t + 1, B_TOPK)
        indices[t, :n_valid] = torch.randperm(t + 1, device="cuda")[:n_valid].to(torch.int32)

    dQ_ref, dKV_ref = sparse_mla_bwd_ref(q, kv, dO, lse, O, indices)          # defaults = the reference's settings
    dQ, dKV = mla_bwd_cuda.mla_bwd(q, kv, dO, lse, O, indices)
    torch.cuda.synchronize()
    mla_bwd_cuda.check_device_status(0)
    assert dQ.dtype == torch.bfloat16 and dQ.shape == q.shape
    assert dKV.dtype == torch.float32 and dKV.shape == kv.shape
    dq_max, dq_rel = calc_diff(dQ, dQ_ref.bfloat16())
    dkv_max, dkv_rel = calc_diff(dKV, dKV_ref)
    print(f"\nreference gate: dQ max_diff={dq_max:.3e} rel_diff={dq_rel:.3e}; dKV max_diff={dkv_max:.3e} rel_diff={dkv_rel:.3e}")
    assert dq_rel < 0.01 and dkv_rel < 0.01

    # the second call reuses the scratch the first one left (kept per device and stream): no new device memory
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    dQ2, dKV2 = mla_bwd_cuda.mla_bwd(q, kv, dO, lse, O, indices)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() - before == dQ2.numel() * 2 + dKV2.numel() * 4
    assert torch.equal(dQ.view(torch.int16), dQ2.view(torch.int16))
    mla_bwd_cuda.release_workspaces()


def test_extension_keywords_and_errors():
    from tests.conftest import import_extension
    mla_bwd_cuda = import_extension()
    from test_operator_b200 import op
    from test_operator_b200.inputs import Workload, make_sequence
    w = Workload("ext", 1, 6, 256, 64, 128, "uniform", invalid_frac=0.1)
    s = make_sequence(w, device="cuda", seed=12)
    args = [s[k] for k in ("q", "kv", "dO", "lse", "O", "indices")]
    a = mla_bwd_cuda.mla_bwd(*args, q_start_index_s=None)
    b = op.mla_bwd(*args, q_start_index_s=None, check_device_status=True)
    assert torch.equal(a[0].view(torch.int16), b[0].view(torch.int16))
    assert (a[1] - b[1]).abs().max().item() <= 1e-5 * b[1].abs().max().item()
    a3 = mla_bwd_cuda.mla_bwd(args[0], args[1].unsqueeze(1), *args[2:5], args[5].unsqueeze(1), sm_scale=0.05, q_start_index_s=3)
    assert a3[1].shape == (256, 1, 576)
    with pytest.raises(RuntimeError, match="contiguous"):
        mla_bwd_cuda.mla_bwd(args[0].transpose(0, 1), *args[1:])
    with pytest.raises(RuntimeError, match="dtype"):
        mla_bwd_cuda.mla_bwd(args[0], args[1], args[2], args[3].double(), args[4], args[5])
    with pytest.raises(RuntimeError, match="CUDA"):
        mla_bwd_cuda.mla_bwd(*[t.cpu() for t in args])
