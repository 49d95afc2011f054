"""CPU restatement of the index inverse (CSR by kv row).  TEST INFRASTRUCTURE ONLY: imported by tests/, never by
the product path.

The reference project has no such operator (parity unpinned against reference outputs: there are none); what is
pinned is the validity rule, which is the one of its kernel and checker (`mla_bwd/mla_bwd.cu:765-789`,
`mla_bwd/test_mla_bwd.py:41-47`): a slot counts iff `0 <= idx < s_kv` and, with a causal start, `idx <= start + q`.
The CSR itself is defined by a stable sort, which numpy provides directly.
"""
from __future__ import annotations

from typing import Optional, Tuple

import numpy as np


def index_inverse_ref(indices: np.ndarray, s_kv: int, q_start_index_s: Optional[int] = None) -> Tuple[np.ndarray, np.ndarray]:
    """indices [s_q, topk] int32 -> (row_ptr [s_kv + 1] int32, entries [s_q * topk] int32).

    entries = flat slot ids (q * topk + slot) sorted by (kv row, flat id), unused slots last in flat order."""
    idx = np.asarray(indices, dtype=np.int64).reshape(indices.shape[0], indices.shape[-1])
    s_q, topk = idx.shape
    valid = (idx >= 0) & (idx < s_kv)
    if q_start_index_s is not None:
        valid &= idx <= (q_start_index_s + np.arange(s_q, dtype=np.int64))[:, None]
    keys = np.where(valid, idx, s_kv).reshape(-1)
    entries = np.argsort(keys, kind="stable").astype(np.int32)
    counts = np.bincount(keys, minlength=s_kv + 1)[: s_kv + 1]
    row_ptr = np.zeros(s_kv + 1, dtype=np.int64)
    row_ptr[1:] = np.cumsum(counts[:s_kv])
    return row_ptr.astype(np.int32), entries


def index_inverse_loops(indices, s_kv: int, q_start_index_s: Optional[int] = None):
    """The same by plain loops (small cases only): checks the numpy form."""
    rows = [[] for _ in range(s_kv)]
    unused = []
    s_q, topk = len(indices), len(indices[0]) if len(indices) else 0
    for q in range(s_q):
        for s in range(topk):
            i = int(indices[q][s])
            ok = 0 <= i < s_kv and (q_start_index_s is None or i <= q_start_index_s + q)
            (rows[i] if ok else unused).append(q * topk + s)
    row_ptr, entries = [0], []
    for r in rows:
        entries += r
        row_ptr.append(len(entries))
    return np.array(row_ptr, dtype=np.int32), np.array(entries + unused, dtype=np.int32)
