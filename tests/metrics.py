"""Error figures shared by the GPU tests; they work on tensors of any size on any device (chunked, fp64 sums)."""
import torch


def error_figures(ref: torch.Tensor, got: torch.Tensor, chunk: int = 1 << 24) -> dict:
    """max-abs error, the reference script's rel_diff (`mla_bwd/test_mla_bwd.py:11-15`: mean of
    |a - b| / (1e-4 + |a|) with a = reference), cosine similarity and max |ref|."""
    a = ref.reshape(-1)
    b = got.reshape(-1)
    assert a.numel() == b.numel()
    max_abs = 0.0
    rel_sum = dot = na = nb = 0.0
    max_ref = 0.0
    for i in range(0, a.numel(), chunk):
        x = a[i:i + chunk].double()
        y = b[i:i + chunk].double()
        d = (x - y).abs()
        max_abs = max(max_abs, d.max().item())
        rel_sum += (d / (1e-4 + x.abs())).sum().item()
        dot += (x * y).sum().item()
        na += (x * x).sum().item()
        nb += (y * y).sum().item()
        max_ref = max(max_ref, x.abs().max().item())
    den = (na * nb) ** 0.5
    return {"max_abs": max_abs, "rel_diff": rel_sum / max(a.numel(), 1), "cosine": 1.0 if den == 0 else dot / den,
            "max_ref": max_ref}


def assert_backward_close(dq, dkv, dq_ref, dkv_ref, what=""):
    """The reference's gate rel_diff < 0.01 (`mla_bwd/test_mla_bwd.py:191-193`), tightened with cosine > 0.99999,
    max-abs <= 2^-7 max|ref| for dQ (compared with the bf16-rounded reference: one rounding step of the output) and
    max-abs <= 2^-8 max|ref| for dKV.  Why 2^-8 and not less: oracle and kernel both round S and dS to bf16 before the
    second-stage products, but reach the fp32 value being rounded by different routes (exp2 vs ex2.approx, different
    summation order), so a value that sits on a rounding boundary can come out one bf16 step apart (the stage test
    bounds how many do).  One such entry moves one element of dKV by 2^-8 |S| |dO|, i.e. by 2^-8 of a term that can
    dominate that element when few queries touch the row; with thousands of queries per row the figure is far smaller
    (the full-size tests print it)."""
    fq = error_figures(dq_ref.bfloat16().float(), dq.float())
    fk = error_figures(dkv_ref.reshape(dkv.shape).float(), dkv.float())
    msg = f"{what} dQ {fq} dKV {fk}"
    assert fq["rel_diff"] < 0.01 and fk["rel_diff"] < 0.01, msg
    assert fq["cosine"] > 0.99999 and fk["cosine"] > 0.99999, msg
    assert fq["max_abs"] <= 2 ** -7 * fq["max_ref"] + 1e-6, msg
    assert fk["max_abs"] <= 2 ** -8 * fk["max_ref"] + 1e-6, msg
    return fq, fk
