#!/usr/bin/env python3
"""Benchmark of the sparse MLA attention backward (5504 FLOPs per query x head x top-k slot).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload NAME] [--s-q ROWS] [--stages MASK] [--schedule CHUNKS,DKV_PAIRS]

One JSON line on stdout (rank 0).  A step is one backward over the whole workload:
  N = 1   workload "head128"  (s_q 4096, s_kv 32768, h_q 128, top-k 2048), one sequence
  N > 1   workload "batch_sharded" (8 independent sequences of s_q 8192, s_kv 16384, h_q 128, top-k 2048)
          split round-robin over the ranks, no communication -> strong scaling; the same line then also carries a
          `query_sharded` block: the long sequence (s_q 16384, s_kv 65536) split by queries with an NCCL
          reduce-scatter of the fp32 partial dKV, timed as a whole, with the collective timed apart and the
          result checked against the unsharded operator.
`value` times the operator with inputs resident in HBM; `e2e` times it from pinned host buffers
(copies in and results out inside the timed region).  `--impl reference` times the reference's
CPU algorithm (the oracle port) on the host cores.  `--s-q` / `--stages` cut the workload down
for profiler captures and are reported in `config`.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from test_operator_b200.inputs import WORKLOADS, make_sequence  # noqa: E402

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
STAGE_NAMES = {2: "delta", 4: "recompute", 8: "dkv", 16: "dq"}
KERNEL_NAMES = {"recompute": "smla_recompute_pair_kernel", "dkv": "smla_dkv_pair_kernel", "dq": "smla_dq_kernel"}
# DRAM bytes (read + write) per query of each kernel at h_q 128 / top-k 2048, from the ncu captures summarised in
# profiles/ (296-query case, dram__bytes_read.sum + dram__bytes_write.sum divided by 296; every kernel's DRAM
# traffic grows in proportion to the number of queries).  They describe the kernels as captured there: a kernel
# change needs a new capture, and `roofline.traffic_source` names the summary the figure came from.
DRAM_BYTES_PER_QUERY_H128_TOPK2048 = {"recompute": 1.366e6, "dkv": 2.248e6, "dq": 0.722e6}
TRAFFIC_SOURCE = {"recompute": "profiles/smla_recompute_pair_kernel_head128_296q.txt",
                  "dkv": "profiles/smla_dkv_pair_kernel_head128_296q.txt", "dq": "profiles/smla_dq_kernel_head128_296q.txt"}
# share of the 5504 FLOPs per slot each kernel carries: recompute = P + dP, dkv = dV + dK, dq = dQ
STAGE_FLOP_SHARE = {4: (2 * 576 + 2 * 512) / 5504.0, 8: (2 * 512 + 2 * 576) / 5504.0, 16: 2 * 576 / 5504.0}
KEYS = ("q", "kv", "dO", "lse", "O", "indices")


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples of one GPU while the timed region runs."""
    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.t0 = self.t1 = None

    def mark_begin(self):
        self.t0 = time.time()

    def mark_end(self):
        self.t1 = time.time()

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        import datetime
        sm, smax, reasons = [], [], set()
        all_sm, all_max = [], []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                ts = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                clk, cmax = float(parts[1]), float(parts[2])
            except ValueError:
                continue
            all_sm.append(clk)
            all_max.append(cmax)
            # samples taken while the timed steps ran (the sampler starts earlier so that it is up to speed)
            if self.t0 is not None and self.t1 is not None and not (self.t0 - 0.05 <= ts <= self.t1 + 0.05):
                continue
            sm.append(clk)
            smax.append(cmax)
            for n, v in zip(names, parts[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:          # timed region shorter than the sampling period: fall back to every sample taken
            sm, smax = all_sm, all_max
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def _dist_setup(n_gpus: int):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, world, local


def _config(wname, w, s_q, sharding="none"):
    """The workload: the same keys and values for our arm and the reference arm (what is particular to an arm - kernel
    stages, schedule, the sample the CPU arm times - sits beside `config`, not in it)."""
    return {"workload": wname, "batch": w.batch, "s_q": s_q or w.s_q, "s_kv": w.s_kv, "h_q": w.h_q, "topk": w.topk,
            "d_qk": 576, "d_v": 512, "flops_per_slot": 5504, "q_start_index_s": w.q_start_index_s,
            "lse": "base 2, from the fp32 forward", "sharding": sharding,
            "l2": "inputs larger than L2 (no flush)"}


def _oracle_run(seq, w, n_queries: int, threads: int):
    """The CPU oracle on the first n_queries rows of `seq` (all top-k slots, full kv): (TFLOP/s, seconds, dQ, dKV)."""
    from oracle.sparse_mla_ref import sparse_mla_bwd_ref
    torch.set_num_threads(threads)
    cpu = {k: (v[:n_queries].cpu() if k in ("q", "dO", "lse", "O", "indices") else
               (v.cpu() if torch.is_tensor(v) else v)) for k, v in seq.items()}
    t0 = time.perf_counter()
    dq, dkv = sparse_mla_bwd_ref(cpu["q"], cpu["kv"], cpu["dO"], cpu["lse"], cpu["O"], cpu["indices"],
                                 q_start_index_s=cpu["q_start_index_s"])
    dt = time.perf_counter() - t0
    return 5504.0 * n_queries * w.h_q * w.topk / dt / 1e12, dt, dq, dkv


def _error_figures(ref, got):
    """max-abs error, the reference script's rel_diff (mean |a - b| / (1e-4 + |a|)), cosine similarity."""
    a, b = ref.double().flatten(), got.double().flatten()
    d = (a - b).abs()
    den = (a.norm() * b.norm()).item()
    return {"max_abs": d.max().item(), "rel_diff": (d / (1e-4 + a.abs())).mean().item(),
            "cosine": 1.0 if den == 0 else (a @ b).item() / den, "max_ref": a.abs().max().item()}


def run_reference(args):
    """The reference's own CPU implementation of the path, all host threads, bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wname = args.workload or ("head128" if args.gpus == 1 else "batch_sharded")
    w = WORKLOADS[wname]
    threads = os.cpu_count() or 1
    n_step = args.s_q or 32
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    seq = make_sequence(w, 0, device=dev, s_q_override=n_step)
    seq = {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in seq.items()}
    times = []
    for i in range(args.warmup + args.steps):
        _, dt, _, _ = _oracle_run(seq, w, n_step, threads)
        if i >= args.warmup:
            times.append(dt)
    ms = 1e3 * sum(times) / len(times)
    val = 5504.0 * n_step * w.h_q * w.topk / (ms * 1e-3) / 1e12
    sample = (f"{n_step} of {w.s_q} queries of sequence 0 per step, full kv and top-k: a rate, the cost of a query "
              f"does not depend on how many there are")
    print(json.dumps({
        "impl": "reference", "metric": "sparse_mla_bwd_tflops", "value": val, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": _config(wname, w, None, sharding="batch" if args.gpus > 1 else "none"),
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def _event_pair():
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def _query_sharded_block(op, sharding, dist, rank, world, dev, steps, warmup):
    """BASELINE config 5 at `world` GPUs: queries split in contiguous blocks, kv replicated, one fp32 partial dKV per
    rank, NCCL reduce-scatter.  Returns the block for the JSON line (rank 0) - timing of the whole step, of the
    collective alone, the one-GPU time of the same workload, and a check of the sharded result."""
    w = WORKLOADS["query_sharded"]
    full = make_sequence(w, 0, device=dev)                       # same seed on every rank: identical tensors
    qs = full["q_start_index_s"]
    r0, r1 = sharding.query_block(w.s_q, rank, world)
    mine = {k: full[k][r0:r1].contiguous() for k in ("q", "dO", "lse", "O", "indices")}
    kv = full["kv"]
    ws = op.workspace_for(mine["q"], kv, mine["indices"])
    partial = torch.empty(kv.shape, dtype=torch.float32, device=dev)

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    # ---- check, once, before timing: 64 queries of every rank's block through the sharded path, against the
    # unsharded operator over the same world * 64 queries on this GPU (dQ rows bit for bit, owned dKV rows to the
    # tolerance of fp32 sums taken in a different order)
    n_chk = 64
    sub = {k: mine[k][:n_chk].contiguous() for k in mine}
    dq_s, rows_s = sharding.query_sharded_bwd(op.mla_bwd, sub["q"], kv, sub["dO"], sub["lse"], sub["O"], sub["indices"],
                                              r0, qs, partial=partial, workspace=ws)
    starts = [sharding.query_block(w.s_q, r, world)[0] for r in range(world)]
    union = {k: torch.cat([full[k][a:a + n_chk] for a in starts]).contiguous() for k in mine}
    if qs is None:
        dq_u, dkv_u = op.mla_bwd(union["q"], kv, union["dO"], union["lse"], union["O"], union["indices"],
                                 q_start_index_s=None, workspace=ws)
    else:   # rows of the union are not consecutive queries: give every query its own position
        meta = torch.cat([op.query_meta_for([0], [n_chk], [0], [w.s_kv], dev, qs + a, w.topk) for a in starts])
        dq_u, dkv_u = op.mla_bwd(union["q"], kv, union["dO"], union["lse"], union["O"], union["indices"],
                                 q_start_index_s=qs, workspace=ws, query_meta=meta.contiguous())
    k0, k1 = sharding.kv_rows_of_rank(w.s_kv, rank, world)
    f = _error_figures(dkv_u.reshape(w.s_kv, -1)[k0:k1], rows_s)
    dq_equal = bool(torch.equal(dq_u[rank * n_chk:(rank + 1) * n_chk].view(torch.int16), dq_s.view(torch.int16)))
    chk = torch.tensor([f["max_abs"], f["max_ref"], 1.0 - f["cosine"], 0.0 if dq_equal else 1.0], dtype=torch.float64, device=dev)
    dist.all_reduce(chk, op=dist.ReduceOp.MAX)
    check = {"queries_per_rank": n_chk, "against": "the unsharded operator over the same queries on one GPU",
             "dkv_max_abs": chk[0].item(), "dkv_max_ref": chk[1].item(), "dkv_one_minus_cosine": chk[2].item(),
             "dq_bit_identical": chk[3].item() == 0.0, "ok": bool(chk[3].item() == 0.0 and chk[0].item() <= 1e-4 * chk[1].item())}
    del union, dq_u, dkv_u, sub

    def step(with_collective=True):
        if with_collective:
            return sharding.query_sharded_bwd(op.mla_bwd, mine["q"], kv, mine["dO"], mine["lse"], mine["O"], mine["indices"],
                                              r0, qs, partial=partial, workspace=ws)
        return op.mla_bwd(mine["q"], kv, mine["dO"], mine["lse"], mine["O"], mine["indices"],
                          q_start_index_s=None if qs is None else qs + r0, out_dkv=partial, workspace=ws)

    def timed(fn, n):
        barrier()
        a, b = _event_pair()
        a.record()
        for _ in range(n):
            fn()
        b.record()
        barrier()
        t = torch.tensor([a.elapsed_time(b) / n], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for _ in range(max(1, warmup)):
        step()
    ms = timed(step, steps)
    ms_compute = timed(lambda: step(False), steps)
    out_rows = torch.empty(k1 - k0, 576, dtype=torch.float32, device=dev)
    flat = partial.reshape(w.s_kv, 576)
    ms_coll = timed(lambda: dist.reduce_scatter_tensor(out_rows, flat, op=dist.ReduceOp.SUM), 10)
    # ---- the same step with the library's NVLink pull-reduce in place of NCCL (partials in symmetric memory, cleared by
    # the reduction itself, so the backward accumulates and no memset runs)
    pull = None
    try:
        reducer = sharding.PullReducer(w.s_kv, dev)
    except Exception as e:          # symmetric memory unavailable on this box: say so, NCCL figures stand
        pull = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
    else:
        def pull_step():
            return sharding.query_sharded_bwd(op.mla_bwd, mine["q"], kv, mine["dO"], mine["lse"], mine["O"], mine["indices"],
                                              r0, qs, reducer=reducer, workspace=ws)
        _, rows_nccl = step()
        ref_max = rows_nccl.abs().max().item()
        pull = {"max_ref": ref_max,
                "how": "smla_dkv_pull_reduce (plain peer loads) / smla_dkv_multimem_reduce (multimem.ld_reduce through the NVSwitch) "
                       "between two symmetric-memory barriers; fused_zero: the kernel also clears what it read in every rank's "
                       "buffer, so the backward accumulates and runs no memset"}
        variants = [("peer_loads", False, False), ("peer_loads_fused_zero", False, True)]
        if reducer.multicast_ptr:
            variants += [("multimem", True, False), ("multimem_fused_zero", True, True)]
        else:
            pull["multimem"] = {"unavailable": "the symmetric memory has no multicast mapping on this box"}
        for name, mm, fz in variants:
            reducer.multimem, reducer.zero_sources = mm, fz
            reducer.partial.zero_()
            barrier()
            _, rows_v = pull_step()
            torch.cuda.synchronize()
            d = torch.tensor([(rows_v - rows_nccl).abs().max().item()], dtype=torch.float64, device=dev)
            dist.all_reduce(d, op=dist.ReduceOp.MAX)
            pull_step()
            ms_v = timed(pull_step, steps)
            ms_v_coll = timed(lambda: reducer.reduce(out_rows), 10)
            pull[name] = {"ms_per_step": ms_v, "value": 5504.0 * w.s_q * w.h_q * w.topk / (ms_v * 1e-3) / 1e12,
                          "collective_ms": ms_v_coll, "max_abs_vs_nccl": d[0].item()}
        del reducer
    status = torch.tensor([op.device_status(ws)], dtype=torch.int64, device=dev)
    dist.all_reduce(status, op=dist.ReduceOp.MAX)
    # ---- the same workload on one GPU (rank 0 alone; the others wait): the base the scaling is measured against
    del mine, partial, ws
    base_ms = None
    if rank == 0:
        ws1 = op.workspace_for(full["q"], kv, full["indices"])
        a, b = _event_pair()
        for i in range(3):
            if i == 1:
                a.record()
            op.mla_bwd(*[full[k] for k in KEYS], q_start_index_s=qs, workspace=ws1)
        b.record()
        torch.cuda.synchronize()
        base_ms = a.elapsed_time(b) / 2
        if op.device_status(ws1) != 0:
            status[0] = 4
        del ws1
    barrier()
    flops = 5504.0 * w.s_q * w.h_q * w.topk
    blk = {"config": _config("query_sharded", w, None, sharding="query+reduce_scatter"),
           "ms_per_step": ms, "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
           "compute_ms": ms_compute, "collective_ms": ms_coll,
           "collective": f"ncclReduceScatter (torch reduce_scatter_tensor) of the {w.s_kv * 576 * 4 / 1e6:.0f} MB fp32 partial dKV, timed alone",
           "check": check, "pull_reduce": pull, "device_status": int(status.item())}
    if base_ms is not None:
        blk["scaling_base"] = {"ms_per_step": base_ms, "value": flops / (base_ms * 1e-3) / 1e12, "n_gpus": 1,
                               "speedup": base_ms / ms}
    return blk


def run_ours(args):
    from test_operator_b200 import op, sharding
    import torch.distributed as dist

    rank, world, local = _dist_setup(args.gpus)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the sparse MLA backward has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if args.schedule:
        c, d = (int(x) for x in args.schedule.split(","))
        op.set_schedule(c, d)
    wname = args.workload or ("head128" if world == 1 else "batch_sharded")
    w = WORKLOADS[wname]
    query_sharded = wname == "query_sharded" and world > 1
    stages = args.stages or op.STAGE_ALL

    # ---- this rank's share of the workload, resident in HBM -------------------------------------------
    if query_sharded:
        full = make_sequence(w, 0, device=dev, s_q_override=args.s_q)
        r0, r1 = sharding.query_block(full["q"].shape[0], rank, world)
        seqs = [{k: (v[r0:r1].contiguous() if k in ("q", "dO", "lse", "O", "indices") else v) for k, v in full.items()}]
        seqs[0]["row0"] = r0
        del full
        my_queries = r1 - r0
    else:
        ids = sharding.sequences_of_rank(w.batch, rank, world)
        seqs = [make_sequence(w, b, device=dev, s_q_override=args.s_q) for b in ids]
        my_queries = sum(s["q"].shape[0] for s in seqs)
    total_q = torch.tensor([my_queries], dtype=torch.int64, device=dev)
    if world > 1:
        dist.all_reduce(total_q)
    flops = 5504.0 * int(total_q.item()) * w.h_q * w.topk
    ws = op.workspace_for(seqs[0]["q"], seqs[0]["kv"], seqs[0]["indices"]) if seqs else None
    partial = torch.empty(seqs[0]["kv"].shape, dtype=torch.float32, device=dev) if query_sharded else None
    smclk = op.SMClock(dev)
    bad_status = []

    def check_status(where):
        if ws is not None and op.device_status(ws) != 0:
            bad_status.append(f"{where} (device code {op.last_device_code()})")

    launches = [0]

    def step():
        outs = []
        for s in seqs:
            if query_sharded:
                outs.append(sharding.query_sharded_bwd(op.mla_bwd, s["q"], s["kv"], s["dO"], s["lse"], s["O"],
                                                       s["indices"], s["row0"], s["q_start_index_s"],
                                                       partial=partial, workspace=ws))
            elif stages == op.STAGE_ALL:
                outs.append(op.mla_bwd(s["q"], s["kv"], s["dO"], s["lse"], s["O"], s["indices"],
                                       q_start_index_s=s["q_start_index_s"], workspace=ws))
            else:
                dq = torch.empty_like(s["q"])
                dkv = torch.empty(s["kv"].shape, dtype=torch.float32, device=dev)
                op.run_stages(s["q"], s["kv"], s["dO"], s["lse"], s["O"], s["indices"], dq, dkv, ws, stages,
                              q_start_index_s=s["q_start_index_s"])
            launches[0] += op.last_launch_count()
        return outs

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    sampler.start()
    for _ in range(args.warmup):
        step()
    barrier()
    check_status("warm-up")
    launches[0] = 0
    e0, e1 = _event_pair()
    barrier()
    sampler.mark_begin()
    smclk.begin()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    smclk.end()
    barrier()
    sampler.mark_end()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / args.steps
    step_mhz = smclk.mhz()
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    n_launch = launches[0]
    check_status("timed steps")

    # ---- per-kernel times (rank 0's first sequence), for the roofline of the dominant kernel -------------
    # Each kernel alone, with the SMs' own cycle counters around it: ms x MHz (cycles) is what can be compared between a
    # kernel timed alone at burst clocks and the same kernel inside a power-capped step.
    kernels = {}
    if seqs and not query_sharded:
        s = seqs[0]
        dq = torch.empty_like(s["q"])
        dkv = torch.zeros(s["kv"].shape, dtype=torch.float32, device=dev)
        nq = s["q"].shape[0]
        for bit, name in STAGE_NAMES.items():
            if not (stages & bit):
                continue
            ts, mhzs = [], []
            for i in range(4):
                a, b = _event_pair()
                smclk.begin()
                a.record()
                op.run_stages(s["q"], s["kv"], s["dO"], s["lse"], s["O"], s["indices"], dq, dkv, ws, bit,
                              q_start_index_s=s["q_start_index_s"])
                b.record()
                smclk.end()
                torch.cuda.synchronize()
                if i:
                    ts.append(a.elapsed_time(b))
                    mhzs.append(smclk.mhz())
            kms = sum(ts) / len(ts)
            entry = {"ms": kms}
            mh = [m for m in mhzs if m]
            if mh:
                entry["sm_mhz"] = sum(mh) / len(mh)
                entry["mcycles"] = kms * entry["sm_mhz"] * 1e-3
            if bit in STAGE_FLOP_SHARE:
                entry["tflops"] = STAGE_FLOP_SHARE[bit] * 5504.0 * nq * w.h_q * w.topk / (kms * 1e-3) / 1e12
            else:
                entry["gbs"] = 2.0 * nq * w.h_q * 512 * 2 / (kms * 1e-3) / 1e9
            kernels[name] = entry
        check_status("per-kernel timing")
    # the forward op of the same shapes (2176 FLOPs per slot: P and S.V), first sequence of this rank
    forward = None
    if seqs and not query_sharded and stages == op.STAGE_ALL and not args.no_forward:
        s = seqs[0]
        ts = []
        for i in range(4):
            a, b = _event_pair()
            a.record()
            op.mla_fwd(s["q"], s["kv"], s["indices"], q_start_index_s=s["q_start_index_s"], check_device_status=(i == 3))
            b.record()
            torch.cuda.synchronize()
            if i:
                ts.append(a.elapsed_time(b))
        fms = sum(ts) / len(ts)
        forward = {"ms": fms, "tflops": 2176.0 * s["q"].shape[0] * w.h_q * w.topk / (fms * 1e-3) / 1e12,
                   "flops_per_slot": 2176}
    peaks, peak_kind = load_peaks()
    roofline = None
    mm = {k: v for k, v in kernels.items() if "tflops" in v}
    if mm:
        dom = max(mm, key=lambda k: mm[k]["ms"])
        peak = float(peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))  # burst: kernel timed alone
        roofline = {"bound": "tensor", "kernel": KERNEL_NAMES[dom], "achieved": mm[dom]["tflops"], "peak": peak,
                    "unit": "TFLOP/s", "frac": mm[dom]["tflops"] / peak, "peak_kind": peak_kind + " burst",
                    "traffic": None}
        per_q = DRAM_BYTES_PER_QUERY_H128_TOPK2048.get(dom)
        if per_q is not None and w.h_q == 128 and w.topk == 2048:
            roofline["traffic"] = per_q * seqs[0]["q"].shape[0]
            roofline["traffic_source"] = TRAFFIC_SOURCE[dom] + " (296-query ncu capture, scaled by the number of queries)"
        # What bounds the dKV kernel is not the tensor pipe but the rate at which the chip takes fp32 reductions: every
        # (query, slot) adds 576 floats to a kv row.  The ceiling is measured here, on this GPU, with the same instruction
        # form on random rows of a dKV-sized buffer.
        if dom == "dkv" and rank == 0:
            try:
                ceiling = op.reduction_rate_gbs(w.s_kv, dev)
                red_bytes = float(seqs[0]["q"].shape[0]) * w.topk * 576 * 4
                red_gbs = red_bytes / (mm[dom]["ms"] * 1e-3) / 1e9
                roofline["reduction"] = {"bytes_per_launch": red_bytes, "achieved_gbs": red_gbs, "ceiling_gbs": ceiling,
                                         "frac": red_gbs / ceiling,
                                         "how": "ceiling: smla_reduction_rate_probe, red.global.add.f32 on random rows of a "
                                                "[s_kv, 576] fp32 buffer from all SMs, CUDA events, best of 3"}
            except Exception as e:      # a measurement aid must not take the line down
                roofline["reduction"] = {"error": str(e)[:200]}
        # the whole step against the same peak, and where its time goes in SM cycles
        step_tf = flops / (ms * 1e-3) / 1e12
        roofline["step"] = {"achieved_per_gpu": step_tf / world, "frac": step_tf / world / peak}
        if step_mhz and all("mcycles" in v for v in kernels.values()) and world == 1 and len(seqs) == 1:
            kc = sum(v["mcycles"] for v in kernels.values())
            roofline["step"].update({"sm_mhz": step_mhz, "mcycles": ms * step_mhz * 1e-3, "kernels_alone_mcycles": kc,
                                     "note": "mcycles = ms x mean SM MHz from the SMs' cycle counters: the step against the "
                                             "sum of its kernels timed one by one, in cycles (the clock differs)"})

    # ---- the same step back to back for about a second (one GPU): the power cap then sets the clock, so this is the
    # figure to hold against the sustained measured peak, as the short timed region is to the burst peak ---------
    sustained = None
    if world == 1 and seqs and stages == op.STAGE_ALL and not args.no_sustained:
        n_sus = max(20, int(1000.0 / max(ms, 1e-3)))
        s2 = ClockSampler(local)
        s2.start()
        torch.cuda.synchronize()
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        s2.mark_begin()
        evs[0].record()
        for i in range(n_sus):
            if i == n_sus // 2:
                evs[1].record()
                smclk.begin()
            step()
        evs[2].record()
        smclk.end()
        torch.cuda.synchronize()
        s2.mark_end()
        c2 = s2.stop()
        half_ms = evs[1].elapsed_time(evs[2]) / (n_sus - n_sus // 2)
        sus_peak = float(peaks.get("bf16_tflops_sustained", FALLBACK_PEAKS.get("bf16_tflops_sustained", 1400.0)))
        burst_peak = float(peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
        sus_val = flops / (half_ms * 1e-3) / 1e12
        sustained = {"steps": n_sus, "ms_per_step": half_ms, "value": sus_val, "unit": "TFLOP/s",
                     "timed": "second half of the steps", "clocks": c2, "sm_mhz_counters": smclk.mhz(),
                     "frac_of_sustained_peak": sus_val / sus_peak, "sustained_peak": sus_peak,
                     "short_run_frac_of_burst_peak": flops / (ms * 1e-3) / 1e12 / burst_peak, "burst_peak": burst_peak,
                     "peak_kind": peak_kind}
        check_status("sustained block")

    # ---- the reference script's timing recipe on our extension module ------------------------------------
    # `mla_bwd/test_mla_bwd.py:137-146` times the operator call with do_bench(rep=50, warmup=10): every call on its
    # own, the L2 flushed before it.  Same recipe here on the timed workload, through the compiled `mla_bwd_cuda`
    # module with positional arguments (the workload's causal start as the one keyword), beside the same calls
    # without the flush.
    ref_recipe = None
    if world == 1 and seqs and stages == op.STAGE_ALL and not args.no_ref_recipe:
        try:
            import mla_bwd_cuda
        except ImportError as e:      # not built: say so, the ctypes path above is the measured product
            ref_recipe = {"unavailable": f"mla_bwd_cuda extension not built ({e})"}
        else:
            s = seqs[0]
            fargs = [s[k] for k in KEYS]
            flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
            res = {}
            for label, do_flush in (("ms_l2_flushed", True), ("ms_back_to_back", False)):
                for _ in range(3):
                    mla_bwd_cuda.mla_bwd(*fargs, q_start_index_s=s["q_start_index_s"])
                ts = []
                for _ in range(20):
                    if do_flush:
                        flush.zero_()
                    a, b = _event_pair()
                    a.record()
                    mla_bwd_cuda.mla_bwd(*fargs, q_start_index_s=s["q_start_index_s"])
                    b.record()
                    torch.cuda.synchronize()
                    ts.append(a.elapsed_time(b))
                res[label] = sum(ts) / len(ts)
            mla_bwd_cuda.check_device_status(local)
            mla_bwd_cuda.release_workspaces()
            del flush
            res["tflops_l2_flushed"] = 5504.0 * s["q"].shape[0] * w.h_q * w.topk / (res["ms_l2_flushed"] * 1e-3) / 1e12
            res["how"] = ("mla_bwd_cuda.mla_bwd(q, kv, dO, lse, O, indices, q_start_index_s=...) allocating dQ and dKV per call, "
                          "scratch cached by the module; 20 calls each, CUDA events per call")
            ref_recipe = res

    # ---- end to end from pinned host buffers --------------------------------------------------------------
    e2e = None
    if seqs and not query_sharded and stages == op.STAGE_ALL and not args.no_e2e:
        host = []
        h2d = d2h = 0
        for s in seqs:
            hs = {k: (v.cpu().pin_memory() if torch.is_tensor(v) else v) for k, v in s.items()}
            host.append(hs)
            h2d += sum(v.numel() * v.element_size() for v in hs.values() if torch.is_tensor(v))
            d2h += s["q"].numel() * 2 + s["kv"].numel() * 4
        out_pinned = [(torch.empty(s["q"].shape, dtype=torch.bfloat16).pin_memory(),
                       torch.empty(s["kv"].shape, dtype=torch.float32).pin_memory()) for s in seqs]
        n_e2e = max(1, min(args.steps, 3))

        def e2e_step():
            for hs, (hq, hkv) in zip(host, out_pinned):
                op.mla_bwd_host(hs["q"], hs["kv"], hs["dO"], hs["lse"], hs["O"], hs["indices"], device=dev,
                                q_start_index_s=hs["q_start_index_s"], workspace=ws, out_dq=hq, out_dkv=hkv)

        e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(n_e2e):
            e2e_step()
        barrier()
        e_ms = 1e3 * (time.perf_counter() - t0) / n_e2e
        te = torch.tensor([e_ms], dtype=torch.float64, device=dev)
        hb = torch.tensor([h2d, d2h], dtype=torch.int64, device=dev)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
            dist.all_reduce(hb)
        e2e = {"value": flops / (float(te.item()) * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": float(te.item()),
               "h2d_bytes_per_step": int(hb[0].item()), "d2h_bytes_per_step": int(hb[1].item()), "steps": n_e2e}
        check_status("end-to-end block")
        del host, out_pinned

    # ---- scaling base and the query-sharded workload (N > 1) ----------------------------------------------
    scaling_base = None
    qs_block = None
    if world > 1 and not query_sharded and stages == op.STAGE_ALL and not args.s_q:
        # the same batch-sharded work on ONE GPU: rank 0 runs as many sequences as the whole job holds (its own first
        # sequence, repeated: all sequences have the same shapes and index statistics), the other ranks wait
        if rank == 0:
            s = seqs[0]
            a, b = _event_pair()
            for rep in range(2):
                if rep == 1:
                    a.record()
                for _ in range(w.batch):
                    op.mla_bwd(s["q"], s["kv"], s["dO"], s["lse"], s["O"], s["indices"],
                               q_start_index_s=s["q_start_index_s"], workspace=ws)
            b.record()
            torch.cuda.synchronize()
            bms = a.elapsed_time(b)
            scaling_base = {"ms_per_step": bms, "value": flops / (bms * 1e-3) / 1e12, "n_gpus": 1, "speedup": bms / ms,
                            "how": f"rank 0 alone, {w.batch} sequences of the workload's shape back to back"}
            check_status("scaling base")
        barrier()
        if not args.no_query_sharded:
            seqs = None          # free this rank's batch-sharded sequences and scratch first
            ws = None
            torch.cuda.empty_cache()
            qs_block = _query_sharded_block(op, sharding, dist, rank, world, dev, max(2, min(args.steps, 5)), 2)

    # ---- CPU baseline (rank 0, one GPU only): the oracle port on a bounded sample; its outputs are also the parity
    # check of the timed workload ---------------------------------------------------------------------------
    cpu_baseline = None
    parity = None
    if rank == 0 and world == 1 and seqs and not args.no_cpu:
        threads = os.cpu_count() or 1
        s = seqs[0]
        _oracle_run(s, w, 8, threads)                          # calibrate
        _, dt, _, _ = _oracle_run(s, w, 32, threads)           # second, warmed-up calibration
        nq_all = s["q"].shape[0]
        n = int(max(16, min(nq_all, 15.0 / max(dt / 32, 1e-4))))
        val, dt, dq_ref, dkv_ref = _oracle_run(s, w, n, threads)
        cpu_baseline = {"value": val, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                        "sample": f"first {n} of {nq_all} queries of sequence 0, full kv and top-k, {dt:.1f} s"}
        if stages == op.STAGE_ALL:
            sub = [s[k][:n].contiguous() if k != "kv" else s[k] for k in KEYS]
            runs = [op.mla_bwd(*sub, q_start_index_s=s["q_start_index_s"], workspace=ws) for _ in range(2)]
            torch.cuda.synchronize()
            check_status("parity block")
            (dq_a, dkv_a), (dq_b, dkv_b) = runs
            parity = {"queries": n, "of": nq_all, "against": "the CPU oracle outputs of the cpu_baseline sample (fp32 torch restatement of the reference's build_reference)",
                      "dQ": _error_figures(dq_ref.bfloat16().float(), dq_a.float().cpu()),
                      "dKV": _error_figures(dkv_ref, dkv_a.cpu().reshape(dkv_ref.shape)),
                      "dQ_run_to_run_bit_identical": bool(torch.equal(dq_a.view(torch.int16), dq_b.view(torch.int16))),
                      "dKV_run_to_run_max_spread": (dkv_a - dkv_b).abs().max().item(),
                      "gate": "rel_diff < 0.01 for both (mla_bwd/test_mla_bwd.py:191-193)"}
            parity["pass"] = bool(parity["dQ"]["rel_diff"] < 0.01 and parity["dKV"]["rel_diff"] < 0.01)

    if rank == 0:
        out = {
            "metric": "sparse_mla_bwd_tflops", "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong" if world > 1 else "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": _config(wname, w, args.s_q,
                              ("query+reduce_scatter" if query_sharded else "batch") if world > 1 else "none"),
            "stages": stages, "schedule": dict(zip(("chunks", "dkv_pairs"), op.get_schedule()),
                                                note="chunks -1: chosen from the head count (64 heads: two overlapped parts; "
                                                     "128: the kernels one after the other)"),
            "clocks": clocks, "gpu_launches": n_launch, "kernels": kernels,
            "device_status": "ok" if not bad_status else "TIMEOUT in: " + "; ".join(bad_status),
        }
        if step_mhz:
            out["sm_mhz_counters"] = step_mhz
        if forward:
            out["forward"] = forward
        if roofline:
            out["roofline"] = roofline
        if sustained:
            out["sustained"] = sustained
        if ref_recipe:
            out["ref_recipe"] = ref_recipe
        if e2e:
            out["e2e"] = e2e
        if scaling_base:
            out["scaling_base"] = scaling_base
        if qs_block:
            out["query_sharded"] = qs_block
        if cpu_baseline:
            out["cpu_baseline"] = cpu_baseline
        if parity:
            out["parity"] = parity
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()
    if bad_status:
        raise SystemExit("device reported a timed-out wait: results invalid (" + "; ".join(bad_status) + ")")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS))
    ap.add_argument("--s-q", dest="s_q", type=int, default=None, help="keep only the first rows of the query dimension")
    ap.add_argument("--stages", type=int, default=0, help="bit mask of kernels to run (profiling); 0 = all")
    ap.add_argument("--schedule", default=None, help="chunks,dkv_pairs (see smla_bwd_set_schedule); default: the library's")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-sustained", dest="no_sustained", action="store_true")
    ap.add_argument("--no-forward", dest="no_forward", action="store_true")
    ap.add_argument("--no-ref-recipe", dest="no_ref_recipe", action="store_true")
    ap.add_argument("--no-query-sharded", dest="no_query_sharded", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
