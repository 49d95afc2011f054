#!/usr/bin/env python3
"""Golden vectors for the forward (o, lse) and the natural-log-lse / query-start semantics, made by RUNNING the
reference's phase-test checker.

`dq_test/test_dq_phase.py:39-66` (`build_reference`) computes, in fp32 torch on whatever device its inputs live on,
o and lse (natural log) of the sparse attention forward and from them S, dS and dQ of the backward, with the causal
rule `idx <= q_start_index_s + row`.  The script imports that function from a checkout of the reference (the module
imports its CUDA extension `dq_phase_cuda` at the top, so a stub of that name is registered first), runs it on CPU on
the two cases of the reference's own test (`:98-99`: s_q 32, s_kv 256, top-k 64, 128 heads, query start 63 and 0) and
stores the outputs.  While doing so it checks the restated forward of `oracle/sparse_mla_ref.py` against it.

Usage:  python tests/golden/make_golden_fwd.py /path/to/reference_checkout
"""
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle.sparse_mla_ref import sparse_mla_bwd_ref, sparse_mla_fwd_ref  # noqa: E402

FWD_CASES = {
    # name: (s_q, s_kv, q_start_index_s)   -- the two cases of dq_test/test_dq_phase.py:98-99
    "dqphase_full_topk_window": (32, 256, 63),
    "dqphase_partial_causal_window": (32, 256, 0),
}
B_H, D_QK, D_V, TOPK = 128, 576, 512, 64
ROWS = [0, 1, 15, 31]      # query rows whose outputs are stored (all heads; keeps the fixtures near 1 MB per case)


def make_fwd_case_inputs(name):
    """Seeded CPU inputs in the style of the reference's build_inputs (`dq_test/test_dq_phase.py:22-36`): per row a
    random subset of the positions the causal rule admits, the rest filled with the out-of-range sentinel s_kv."""
    s_q, s_kv, q_start = FWD_CASES[name]
    g = torch.Generator().manual_seed(4321 + sum(map(ord, name)))
    q = torch.randn(s_q, B_H, D_QK, generator=g).to(torch.bfloat16)
    kv = torch.randn(s_kv, 1, D_QK, generator=g).to(torch.bfloat16)
    dO = torch.randn(s_q, B_H, D_V, generator=g).to(torch.bfloat16)
    indices = torch.full((s_q, 1, TOPK), s_kv, dtype=torch.int32)
    for t in range(s_q):
        max_valid = min(q_start + t + 1, s_kv)
        n_valid = min(max_valid, TOPK)
        indices[t, 0, :n_valid] = torch.randperm(max_valid, generator=g)[:n_valid].to(torch.int32)
    return q, kv, dO, indices, q_start


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else None
    if ref_root is None or not os.path.isdir(os.path.join(ref_root, "dq_test")):
        raise SystemExit("usage: make_golden_fwd.py /path/to/reference_checkout")
    sys.modules["dq_phase_cuda"] = types.ModuleType("dq_phase_cuda")   # stub: the script imports it at the top
    sys.path.insert(0, os.path.join(ref_root, "dq_test"))
    import test_dq_phase as ref

    torch.set_num_threads(4)
    for name in FWD_CASES:
        q, kv, dO, indices, q_start = make_fwd_case_inputs(name)
        o, lse, dQ, S, dS = ref.build_reference(q, kv, dO, indices, q_start)
        o_mine, lse_mine = sparse_mla_fwd_ref(q, kv.squeeze(1), indices.squeeze(1), q_start_index_s=q_start)
        d_lse = (lse - lse_mine).abs().max().item()
        n_o = (o.view(torch.int16) != o_mine.view(torch.int16)).sum().item()
        # usually bit-identical; the CPU BLAS does not always sum in the same order from run to run (threads), which
        # moves lse by a few 1e-5 and flips the rounding of a few values of o
        assert d_lse <= 1e-4, f"{name}: restated lse differs by {d_lse}"
        assert n_o <= 1e-3 * o.numel(), f"{name}: restated o differs in {n_o} bf16 values"
        dq_mine, _, _, S_mine, dS_mine = sparse_mla_bwd_ref(q, kv.squeeze(1), dO, lse, o, indices.squeeze(1), q_start_index_s=q_start,
                                                             lse_is_base2=False, return_intermediates=True)
        rel = ((dq_mine - dQ.float()).abs() / (1e-4 + dQ.float().abs())).mean().item()
        assert rel < 1e-2, f"{name}: restated dQ rel_diff {rel}"
        # bf16 tensors are stored as their bit patterns (int16): exact and half the size of fp32
        bits = lambda t: t[ROWS].contiguous().view(torch.int16).numpy()
        np.savez_compressed(os.path.join(HERE, f"{name}.npz"), rows=np.array(ROWS), lse=lse.numpy(),
                            o_bits=bits(o), dQ_bits=bits(dQ), S_bits=bits(S), dS_bits=bits(dS))
        print(f"{name}: wrote golden; restated forward: lse max diff {d_lse:.2e}, {n_o} of {o.numel()} bf16 values of o differ; "
              f"restated backward dQ rel_diff {rel:.2e}")


if __name__ == "__main__":
    main()
