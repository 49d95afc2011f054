"""Index inverse (CSR by kv row) on the GPU against the numpy oracle: integer work, bit-exact."""
import numpy as np
import pytest
import torch

from oracle.index_inverse_ref import index_inverse_ref

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _indices(s_q, topk, s_kv, seed, invalid_frac=0.1, lo=None):
    g = np.random.default_rng(seed)
    idx = g.integers(0 if lo is None else lo, s_kv, size=(s_q, topk), dtype=np.int64)
    bad = g.random((s_q, topk)) < invalid_frac
    idx[bad] = g.choice(np.array([-1, s_kv, s_kv + 7, -(2 ** 31), 2 ** 31 - 1]), size=int(bad.sum()))
    return idx.astype(np.int32)


def _run(idx, s_kv, q_start):
    from test_operator_b200 import op
    row_ptr, entries = op.index_inverse(torch.from_numpy(idx).to(DEV), s_kv, q_start_index_s=q_start)
    torch.cuda.synchronize()
    return row_ptr.cpu().numpy(), entries.cpu().numpy()


# (s_q, topk, s_kv, causal start): one / two / three radix passes, ragged last block, keys of exactly 8 and 16 bits
CASES = [
    (3, 32, 200, None),          # one pass, a single partial block
    (64, 64, 255, None),         # largest s_kv whose keys (0..s_kv) fit 8 bits
    (64, 64, 256, None),         # two passes of 5 bits
    (257, 96, 5000, None),       # two passes, several blocks, ragged tail
    (300, 128, 65535, 100),      # 16-bit keys, causal bound cuts most slots of early queries
    (129, 2048, 70000, None),    # three passes
    (512, 64, 40, None),         # few rows: long segments, heavy duplicates
]


@pytest.mark.parametrize("s_q,topk,s_kv,q_start", CASES)
def test_index_inverse_matches_oracle(s_q, topk, s_kv, q_start):
    idx = _indices(s_q, topk, s_kv, seed=s_q + topk)
    row_ptr, entries = _run(idx, s_kv, q_start)
    ref_ptr, ref_entries = index_inverse_ref(idx, s_kv, q_start)
    assert np.array_equal(row_ptr, ref_ptr)
    assert np.array_equal(entries, ref_entries)


def test_index_inverse_full_size_properties():
    """head128 shape (4096 x 2048 slots over 32768 rows): oracle equality plus the properties any CSR must have."""
    s_q, topk, s_kv = 4096, 2048, 32768
    idx = _indices(s_q, topk, s_kv, seed=11, invalid_frac=0.05)
    row_ptr, entries = _run(idx, s_kv, None)
    assert row_ptr[0] == 0 and np.all(np.diff(row_ptr) >= 0)
    n_valid = int(((idx >= 0) & (idx < s_kv)).sum())
    assert row_ptr[-1] == n_valid
    assert np.array_equal(np.sort(entries), np.arange(s_q * topk, dtype=np.int32))      # a permutation
    rows_of_entries = idx.reshape(-1)[entries[:n_valid]]
    assert np.all(np.diff(rows_of_entries) >= 0)                                        # grouped by row
    assert np.array_equal(np.repeat(np.arange(s_kv), np.diff(row_ptr)), rows_of_entries)
    ref_ptr, ref_entries = index_inverse_ref(idx, s_kv, None)
    assert np.array_equal(row_ptr, ref_ptr) and np.array_equal(entries, ref_entries)
    again_ptr, again_entries = _run(idx, s_kv, None)
    assert np.array_equal(again_ptr, row_ptr) and np.array_equal(again_entries, entries)  # reproducible


def test_index_inverse_reproduces_dkv_touch_pattern():
    """Rows with an empty segment are exactly the rows the backward leaves at +0.0."""
    from test_operator_b200 import op
    from test_operator_b200.inputs import Workload, make_sequence
    w = Workload("t", 1, 33, 512, 64, 64, "uniform", invalid_frac=0.2)
    s = make_sequence(w, device=DEV, seed=9)
    _, dkv = op.mla_bwd(s["q"], s["kv"], s["dO"], s["lse"], s["O"], s["indices"], q_start_index_s=None)
    row_ptr, _ = op.index_inverse(s["indices"], w.s_kv, q_start_index_s=None)
    empty = (row_ptr[1:] == row_ptr[:-1])
    untouched = (dkv.view(w.s_kv, -1) == 0).all(dim=1)
    assert torch.equal(empty | untouched, untouched) and bool((untouched & ~empty).sum() == 0)


def test_index_inverse_empty_and_errors():
    from test_operator_b200 import op
    row_ptr, entries = op.index_inverse(torch.empty(0, 32, dtype=torch.int32, device=DEV), 100)
    assert entries.numel() == 0 and torch.all(row_ptr == 0) and row_ptr.numel() == 101
    with pytest.raises(RuntimeError):
        op.index_inverse(torch.zeros(4, 32, dtype=torch.int64, device=DEV), 100)
    with pytest.raises(RuntimeError):
        op.index_inverse(torch.zeros(4, 32, dtype=torch.int32, device=DEV), 0)
