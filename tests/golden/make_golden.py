#!/usr/bin/env python3
"""Generate the golden vectors under tests/golden/ by RUNNING the reference's own checker.

The reference keeps no stored vectors for the sparse MLA backward; its test regenerates
seeded inputs and calls `build_reference` (`mla_bwd/test_mla_bwd.py:18-90`).  That function
is device-agnostic torch code, so this script imports it from a checkout of the reference
(the module imports the CUDA extension at the top, so a stub module of that name is
registered first), runs it on CPU tensors, and stores inputs-by-seed + outputs.  While doing
so it asserts that the restatement in `oracle/sparse_mla_ref.py` is BIT-IDENTICAL to the
reference on the reference's own settings.

Usage:  python tests/golden/make_golden.py /path/to/reference_checkout
The checkout is needed only to regenerate; the tests read the committed .npz files.
"""
import hashlib
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle.sparse_mla_ref import sparse_mla_bwd_ref, sparse_mla_fwd_ref  # noqa: E402

CASES = {
    # name: (s_q, s_kv, h_q, topk, index style)
    "ref_prefix_h16": (16, 96, 16, 32, "prefix"),     # the reference script's index style: causal prefix + s_kv sentinel
    "ref_mixed_h128": (4, 160, 128, 64, "mixed"),     # -1, >= s_kv, and future (idx > row) entries mixed in
    "ref_mixed_h64": (6, 64, 64, 32, "mixed"),
}


def make_case_inputs(name):
    """Deterministic CPU inputs for a golden case (shared with tests/test_oracle.py)."""
    s_q, s_kv, h_q, topk, style = CASES[name]
    g = torch.Generator().manual_seed(1234 + sum(map(ord, name)))
    q = torch.randn(s_q, h_q, 576, generator=g).to(torch.bfloat16)
    kv = torch.randn(s_kv, 576, generator=g).to(torch.bfloat16)
    dO = torch.randn(s_q, h_q, 512, generator=g).to(torch.bfloat16)
    lse = torch.randn(s_q, h_q, generator=g) * 2.0 + 5.0
    O = torch.randn(s_q, h_q, 512, generator=g).to(torch.bfloat16)
    idx = torch.full((s_q, topk), s_kv, dtype=torch.int32)
    if style == "prefix":
        for t in range(s_q):
            n = min(t + 1, topk)
            idx[t, :n] = torch.randperm(t + 1, generator=g)[:n].to(torch.int32)
    else:
        for t in range(s_q):
            idx[t] = torch.randperm(s_kv, generator=g)[:topk].to(torch.int32)
        # make the first few rows of kv reachable under the causal rule, then sprinkle invalid values
        for t in range(s_q):
            n = min(t + 1, topk // 2)
            idx[t, :n] = torch.randperm(t + 1, generator=g)[:n].to(torch.int32)
        r = torch.rand(s_q, topk, generator=g)
        idx = torch.where(r < 0.1, torch.full_like(idx, -1), idx)
        idx = torch.where((r >= 0.1) & (r < 0.2), torch.full_like(idx, s_kv + 3), idx)
    return q, kv, dO, lse.contiguous(), O, idx.contiguous()


def input_digest(tensors):
    h = hashlib.sha256()
    for t in tensors:
        h.update(t.contiguous().view(torch.uint8).numpy().tobytes())
    return h.hexdigest()


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else None
    if ref_root is None or not os.path.isdir(os.path.join(ref_root, "mla_bwd")):
        raise SystemExit("usage: make_golden.py /path/to/reference_checkout")
    sys.modules["mla_bwd_cuda"] = types.ModuleType("mla_bwd_cuda")  # stub: the script imports it at top
    sys.path.insert(0, os.path.join(ref_root, "mla_bwd"))
    import test_mla_bwd as ref  # the reference's script

    torch.set_num_threads(4)
    for name in CASES:
        q, kv, dO, lse, O, idx = make_case_inputs(name)
        dq_ref, dkv_ref = ref.build_reference(q, kv, dO, lse, O, idx)
        dq_mine, dkv_mine = sparse_mla_bwd_ref(q, kv, dO, lse, O, idx)  # defaults = reference settings
        assert torch.equal(dq_ref, dq_mine), f"{name}: restated dQ is not bit-identical to the reference"
        assert torch.equal(dkv_ref, dkv_mine), f"{name}: restated dKV is not bit-identical to the reference"
        np.savez_compressed(
            os.path.join(HERE, f"{name}.npz"),
            dQ=dq_ref.numpy(), dKV=dkv_ref.numpy(),
            digest=np.array(input_digest([q, kv, dO, lse, O, idx])),
        )
        print(f"{name}: wrote golden (dQ {tuple(dq_ref.shape)}, dKV {tuple(dkv_ref.shape)}); restatement bit-identical")


if __name__ == "__main__":
    main()
