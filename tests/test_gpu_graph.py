"""The whole backward is stream-ordered (no host synchronisation, no allocation inside the library), so a call with a
caller-owned workspace can be captured in a CUDA graph and replayed."""
import pytest
import torch

from test_operator_b200.inputs import Workload, make_sequence

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_backward_replays_from_a_cuda_graph():
    from test_operator_b200 import op
    w = Workload("graph", 1, 160, 1024, 128, 256, "uniform", invalid_frac=0.1)
    s = make_sequence(w, device="cpu", seed=23)
    q, kv, dO, lse, O, idx = (s[k].to(DEV) for k in ("q", "kv", "dO", "lse", "O", "indices"))
    ws = op.workspace_for(q, kv, idx)
    dkv = torch.empty(kv.shape, dtype=torch.float32, device=DEV)
    dq_eager, _ = op.mla_bwd(q, kv, dO, lse, O, idx, q_start_index_s=None, out_dkv=dkv, workspace=ws)   # also the warm-up
    dkv_eager = dkv.clone()
    torch.cuda.synchronize()

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            dq_g, _ = op.mla_bwd(q, kv, dO, lse, O, idx, q_start_index_s=None, out_dkv=dkv, workspace=ws)
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(2):
        dkv.fill_(7.0)          # the captured call clears dKV itself
        dq_g.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert op.device_status(ws) == 0
        assert torch.equal(dq_g.view(torch.int16), dq_eager.view(torch.int16))          # dQ is reproducible bit for bit
        assert (dkv - dkv_eager).abs().max().item() <= 1e-5 * dkv_eager.abs().max().item()   # fp32 atomics: order varies
