"""Query-sharded backward on 2 GPUs (needs two; skipped otherwise): queries split over the ranks, kv replicated, fp32
partial dKV per rank, summed by NCCL's reduce-scatter and by the library's NVLink pull-reduce kernel - both against
the oracle evaluated over ALL queries on each rank's own GPU.  Ranks are child processes; NVLS / multicast are
switched off in them (plain peer loads only)."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    import torch.distributed as dist
    from oracle.sparse_mla_ref import sparse_mla_bwd_ref
    from tests.metrics import error_figures
    from test_operator_b200 import op, sharding
    from test_operator_b200.inputs import Workload, make_sequence
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        # the long-context workload's pattern (half of the slots from the most recent rows, 10 % unused), cut down
        w = Workload("qs2", 1, 640, 8192, 128, 512, "skewed", invalid_frac=0.1, recent_window=1024)
        s = make_sequence(w, 0, device=dev, seed=7)                  # same seed: same tensors on every rank
        keys = ("q", "dO", "lse", "O", "indices")
        for q_start in (None, 7600):
            dq_ref, dkv_ref = sparse_mla_bwd_ref(s["q"], s["kv"], s["dO"], s["lse"], s["O"], s["indices"], q_start_index_s=q_start, chunk_s=16)
            r0, r1 = sharding.query_block(w.s_q, rank, world)
            k0, k1 = sharding.kv_rows_of_rank(w.s_kv, rank, world)
            blk = [s[k][r0:r1].contiguous() for k in keys]
            reducer = sharding.PullReducer(w.s_kv, dev, zero_sources=True)
            plain = sharding.PullReducer(w.s_kv, dev)       # partials cleared by the operator, not by the reduction
            for name, kw in (("nccl", {}), ("pull", {"reducer": reducer}), ("pull again", {"reducer": reducer}),
                             ("plain pull", {"reducer": plain}), ("plain pull again", {"reducer": plain})):
                dq, rows = sharding.query_sharded_bwd(op.mla_bwd, blk[0], s["kv"], blk[1], blk[2], blk[3], blk[4], r0, q_start,
                                                      check_device_status=True, **kw)
                torch.cuda.synchronize()
                fq = error_figures(dq_ref[r0:r1].bfloat16().float(), dq.float())
                fk = error_figures(dkv_ref[k0:k1], rows)
                assert fq["rel_diff"] < 0.01 and fq["cosine"] > 0.99999 and fq["max_abs"] <= 2 ** -7 * fq["max_ref"] + 1e-6, (name, fq)
                assert fk["rel_diff"] < 0.01 and fk["cosine"] > 0.99999 and fk["max_abs"] <= 2 ** -8 * fk["max_ref"] + 1e-6, (name, fk)
                if name.startswith("pull"):   # the fused-zero form
                    dist.barrier()
                    torch.cuda.synchronize()
                    assert torch.count_nonzero(reducer.partial).item() == 0, "the pull-reduce leaves every partial clear"
            del reducer, plain
        ret[rank] = "ok"
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_query_sharded_two_ranks_nccl_and_pull_reduce_against_oracle():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=600)
    for p in procs:
        if p.is_alive():
            p.terminate()
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert ret.get(0) == "ok" and ret.get(1) == "ok"
