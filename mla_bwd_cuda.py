"""Drop-in for the reference's extension module of the same name.

`mla_bwd(q, kv, dO, lse, O, indices) -> (dQ, dKV)` as `mla_bwd/mla_bwd.cu:1060-1063` exports it, so that
the reference's `mla_bwd/test_mla_bwd.py` runs unmodified with this repository on PYTHONPATH.
"""
from test_operator_b200.op import mla_bwd  # noqa: F401

__all__ = ["mla_bwd"]
