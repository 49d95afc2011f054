"""The overlapped schedule (dKV kernel of one part of the queries on a second stream beside the recompute and dQ
kernels of the next part) against the plain one-after-the-other schedule and against the oracle."""
import pytest
import torch

from oracle.sparse_mla_ref import sparse_mla_bwd_ref
from tests.metrics import assert_backward_close
from test_operator_b200.inputs import Workload, make_sequence

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
KEYS = ("q", "kv", "dO", "lse", "O", "indices")


@pytest.mark.parametrize("chunks,dkv_pairs", [(2, 0), (3, 24), (4, 40)])
def test_overlapped_schedule_matches_sequential_and_oracle(chunks, dkv_pairs):
    from test_operator_b200 import op
    # enough queries that every part keeps all clusters busy (the library falls back to fewer parts otherwise)
    w = Workload("sched", 1, 1400, 2048, 128, 256, "uniform", invalid_frac=0.1)
    s = make_sequence(w, device=DEV, seed=37)
    args = [s[k] for k in KEYS]
    before = op.get_schedule()
    try:
        op.set_schedule(0, 0)
        dq0, dkv0 = op.mla_bwd(*args, q_start_index_s=None, check_device_status=True)
        n0 = op.last_launch_count()
        op.set_schedule(chunks, dkv_pairs)
        for _ in range(2):
            dq1, dkv1 = op.mla_bwd(*args, q_start_index_s=None, check_device_status=True)
            n1 = op.last_launch_count()
            assert n1 == 1 + 3 * chunks and n0 == 4
            assert torch.equal(dq0.view(torch.int16), dq1.view(torch.int16))
            assert (dkv0 - dkv1).abs().max().item() <= 1e-5 * dkv0.abs().max().item()
        # several passes over the queries (small scratch) with parts inside every pass
        dq2, dkv2 = op.mla_bwd(*args, q_start_index_s=None, check_device_status=True,
                               workspace_budget=700 * 256 * 128 * 4 + (1 << 20))
        assert torch.equal(dq0.view(torch.int16), dq2.view(torch.int16))
        assert (dkv0 - dkv2).abs().max().item() <= 1e-5 * dkv0.abs().max().item()
    finally:
        op.set_schedule(*before)
    dq_ref, dkv_ref = sparse_mla_bwd_ref(*args, q_start_index_s=None, chunk_s=16)
    assert_backward_close(dq1, dkv1, dq_ref, dkv_ref, "overlapped")


def test_overlapped_schedule_replays_from_a_cuda_graph():
    """The overlapped schedule's second stream forks from and joins the caller's stream, so a capture of the caller's
    stream takes the whole call (the first call, which creates that stream, came before)."""
    from test_operator_b200 import op
    before = op.get_schedule()
    op.set_schedule(2, 0)
    try:
        _graph_replay_case(op, 128)
    finally:
        op.set_schedule(*before)


def test_default_schedule_follows_the_head_count():
    """Automatic (-1): two overlapped parts with 64 heads, the kernels one after the other with 128."""
    from test_operator_b200 import op
    before = op.get_schedule()
    op.set_schedule(-1, 0)
    try:
        for h_q, launches in ((64, 1 + 3 * 2), (128, 1 + 3)):
            w = Workload("sched_auto", 1, 1400, 2048, h_q, 256, "uniform", invalid_frac=0.1)
            s = make_sequence(w, device=DEV, seed=39)
            args = [s[k] for k in KEYS]
            dq, dkv = op.mla_bwd(*args, q_start_index_s=None, check_device_status=True)
            assert op.last_launch_count() == launches
            dq_ref, dkv_ref = sparse_mla_bwd_ref(*args, q_start_index_s=None, chunk_s=16)
            assert_backward_close(dq, dkv, dq_ref, dkv_ref, f"automatic schedule, {h_q} heads")
    finally:
        op.set_schedule(*before)


def _graph_replay_case(op, h_q):
    w = Workload("sched_graph", 1, 1400, 2048, h_q, 256, "uniform", invalid_frac=0.1)
    s = make_sequence(w, device=DEV, seed=38)
    args = [s[k] for k in KEYS]
    ws = op.workspace_for(s["q"], s["kv"], s["indices"])
    dkv = torch.empty(s["kv"].shape, dtype=torch.float32, device=DEV)
    dq_eager, _ = op.mla_bwd(*args, q_start_index_s=None, out_dkv=dkv, workspace=ws)
    assert op.last_launch_count() == 1 + 3 * op.get_schedule()[0]
    dkv_eager = dkv.clone()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            dq_g, _ = op.mla_bwd(*args, q_start_index_s=None, out_dkv=dkv, workspace=ws)
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(2):
        dkv.fill_(7.0)
        dq_g.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert op.device_status(ws) == 0
        assert torch.equal(dq_g.view(torch.int16), dq_eager.view(torch.int16))
        assert (dkv - dkv_eager).abs().max().item() <= 1e-5 * dkv_eager.abs().max().item()
