"""CPU tests: the C-ABI library loads and exports what the header declares; host-side checks and sharding."""
import ctypes
import os
import re
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle.sparse_mla_ref import sparse_mla_bwd_ref
from test_operator_b200 import op, sharding
from test_operator_b200.inputs import Workload, make_sequence

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    lib = op.load_library()
    hdr = open(os.path.join(ROOT, "include", "smla_bwd.h")).read()
    names = set(re.findall(r"\b(smla_[a-z_0-9]+)\s*\(", hdr))
    assert {"smla_bwd_run", "smla_bwd_run_stages", "smla_bwd_delta", "smla_bwd_workspace_size"} <= names
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/smla_bwd.h but not exported"


def test_extension_module_is_compiled_code_and_checks_like_the_reference():
    """`python setup.py build_ext --inplace` (run by `__graft_entry__.build()`) leaves the module `mla_bwd_cuda` in the
    tree: a compiled extension exporting `mla_bwd`, as `mla_bwd/setup.py:61-78` / `mla_bwd/mla_bwd.cu:1060-1063` do."""
    mod = pytest.importorskip("mla_bwd_cuda")
    assert mod.__file__.endswith(".so") and callable(mod.mla_bwd)
    t = torch.zeros(2, 16, 576, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="CUDA tensor"):       # TORCH_CHECK -> RuntimeError (mla_bwd.cu:975-1015)
        mod.mla_bwd(t, t, t, t, t, t)


def test_struct_layout_matches_header_field_order():
    hdr = open(os.path.join(ROOT, "include", "smla_bwd.h")).read()
    body = hdr[hdr.index("typedef struct smla_bwd_params {"): hdr.index("} smla_bwd_params;")]
    fields = []
    for line in body.splitlines()[1:]:
        line = line.split("/*")[0].strip()
        if not line or line.startswith("*") or not line.endswith(";"):
            continue
        decl = line[:-1]
        for part in decl.split(","):
            fields.append(re.findall(r"([A-Za-z_0-9]+)$", part.strip())[0])
    assert fields == [f[0] for f in op._Params._fields_]


def _header_fields(struct_name):
    hdr = open(os.path.join(ROOT, "include", "smla_bwd.h")).read()
    body = hdr[hdr.index("typedef struct %s {" % struct_name): hdr.index("} %s;" % struct_name)]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = []
    for decl in body.split("{", 1)[1].split(";"):
        decl = decl.strip()
        if not decl:
            continue
        for part in decl.split(","):
            fields.append(re.findall(r"([A-Za-z_0-9]+)$", part.strip())[0])
    return fields


def test_other_struct_layouts_match_the_header():
    assert _header_fields("smla_bwd_params") == [f[0] for f in op._Params._fields_]
    assert _header_fields("smla_fwd_params") == [f[0] for f in op._FwdParams._fields_]
    assert _header_fields("smla_bwd_det_params") == [f[0] for f in op._DetParams._fields_]
    assert _header_fields("smla_bwd_workspace_layout") == [f[0] for f in op.WorkspaceLayout._fields_]


def test_new_entry_points_refuse_bad_arguments_without_a_gpu():
    lib = op.load_library()
    p = op._Params(0, 0, 0, 0, 0, 0, 0, 0, 64, 256, 16, 64, 0.0, 0, 1)
    assert lib.smla_bwd_staging_bytes_per_query(ctypes.byref(p)) == 256 * 576 * 4       # top-k padded to 256 slots
    assert lib.smla_bwd_run_deterministic(ctypes.byref(p), None, None, 0, None, 31) == 1
    assert lib.smla_bwd_set_schedule(1, 0) == 1 and lib.smla_bwd_set_schedule(-2, 0) == 1
    c, d = op.get_schedule()
    assert c == -1 and d == 0                                                        # the library's default: automatic
    assert lib.smla_dkv_pull_reduce(None, 2, 0, 64, None, 0, None) == 1
    assert lib.smla_dkv_multimem_reduce(None, 2, 0, 64, None, 0, None) == 1
    assert lib.smla_selftest_wait_timeout(None, 0, 1000, None, None) == 1
    assert lib.smla_bwd_workspace_init(None, None) == 1


def test_workspace_size_and_bad_arguments_without_a_gpu():
    lib = op.load_library()
    p = op._Params(0, 0, 0, 0, 0, 0, 0, 0, 4096, 32768, 128, 2048, 0.0, 0, 1)
    full = lib.smla_bwd_workspace_size(ctypes.byref(p), 1 << 40)
    assert full >= 4096 * 2048 * 128 * 4          # bf16 S and dS for every query
    small = lib.smla_bwd_workspace_size(ctypes.byref(p), 1 << 30)
    assert small <= (1 << 30) + (1 << 20) and small < full
    lay = op.WorkspaceLayout()
    assert lib.smla_bwd_get_workspace_layout(ctypes.byref(p), small, ctypes.byref(lay)) == 0
    assert 1 <= lay.q_chunk < 4096 and lay.topk_pad == 2048 and lay.h_pad == 128
    bad = op._Params(0, 0, 0, 0, 0, 0, 0, 0, 16, 64, 12, 32, 0.0, 0, 1)    # h_q not a multiple of 8
    assert lib.smla_bwd_workspace_size(ctypes.byref(bad), 0) == 0
    # null pointers are refused before any CUDA call
    assert lib.smla_bwd_run(ctypes.byref(p), None, 0, None) == 1
    assert lib.smla_bwd_run(ctypes.byref(p), ctypes.c_void_p(256), 1 << 20, None) == 1
    assert lib.smla_bwd_delta(None, None, None, 4, 16, None) == 1
    assert b"workspace" in lib.smla_status_string(3)


def test_operator_rejects_what_the_reference_rejects():
    w = Workload("v", 1, 2, 32, 16, 8, "uniform")
    s = make_sequence(w, device="cpu", seed=1)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        op.mla_bwd(s["q"], s["kv"], s["dO"], s["lse"], s["O"], s["indices"])
    with pytest.raises(RuntimeError):
        op._validate(s["q"].float(), s["kv"], s["dO"], s["lse"], s["O"], s["indices"])


def test_validate_shapes_on_meta_like_cpu_tensors(monkeypatch):
    """Shape / dtype / contiguity rules, exercised on CPU tensors by bypassing only the device check."""
    w = Workload("v", 1, 2, 32, 16, 8, "uniform")
    s = make_sequence(w, device="cpu", seed=1)
    monkeypatch.setattr(torch.Tensor, "is_cuda", property(lambda self: True))
    op._validate(s["q"], s["kv"], s["dO"], s["lse"], s["O"], s["indices"])
    op._validate(s["q"], s["kv"].unsqueeze(1), s["dO"], s["lse"], s["O"], s["indices"].unsqueeze(1))
    for bad in (
        dict(q=s["q"][:, :, :512].contiguous()),                      # wrong head dim
        dict(dO=s["dO"][:, :, :256].contiguous()),                    # wrong d_v
        dict(lse=s["lse"].double()),                                   # wrong dtype
        dict(indices=s["indices"].long()),
        dict(q=s["q"].transpose(0, 1)),                                # not contiguous
        dict(lse=s["lse"][:1]),                                        # wrong s_q
        dict(kv=torch.zeros(32, 2, 576, dtype=torch.bfloat16)),        # h_kv != 1
    ):
        args = {**{k: s[k] for k in ("q", "kv", "dO", "lse", "O", "indices")}, **bad}
        with pytest.raises(RuntimeError):
            op._validate(args["q"], args["kv"], args["dO"], args["lse"], args["O"], args["indices"])


def test_partition_helpers():
    assert sharding.sequences_of_rank(8, 1, 4) == [1, 5]
    blocks = [sharding.query_block(10, r, 4) for r in range(4)]
    assert blocks == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert sharding.kv_rows_of_rank(64, 3, 4) == (48, 64)
    with pytest.raises(ValueError):
        sharding.kv_rows_of_rank(10, 0, 4)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _query_sharded_worker(rank, world, port, q_start):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    w = Workload("qs", 1, 10, 64, 16, 16, "uniform", invalid_frac=0.1)
    s = make_sequence(w, device="cpu", seed=13)
    full_dq, full_dkv = sparse_mla_bwd_ref(s["q"], s["kv"], s["dO"], s["lse"], s["O"], s["indices"], q_start_index_s=q_start)

    def cpu_bwd(q, kv, dO, lse, O, idx, q_start_index_s=None, out_dkv=None, **kw):   # stands in for the CUDA operator
        dq, dkv = sparse_mla_bwd_ref(q, kv, dO, lse, O, idx, q_start_index_s=q_start_index_s)
        out_dkv.copy_(dkv)
        return dq.bfloat16(), out_dkv

    r0, r1 = sharding.query_block(w.s_q, rank, world)
    dq, mine = sharding.query_sharded_bwd(cpu_bwd, s["q"][r0:r1], s["kv"], s["dO"][r0:r1], s["lse"][r0:r1],
                                          s["O"][r0:r1], s["indices"][r0:r1], r0, q_start)
    k0, k1 = sharding.kv_rows_of_rank(w.s_kv, rank, world)
    assert torch.allclose(mine, full_dkv[k0:k1], rtol=1e-5, atol=1e-5)
    assert torch.equal(dq, full_dq[r0:r1].bfloat16())
    dist.destroy_process_group()


@pytest.mark.parametrize("q_start", [None, 30])
def test_query_sharded_reduce_scatter_two_ranks_gloo(q_start):
    port = _free_port()
    mp.spawn(_query_sharded_worker, args=(2, port, q_start), nprocs=2, join=True)


def test_index_inverse_oracle_forms_agree_and_abi_rejects_bad_shapes():
    import numpy as np
    from oracle.index_inverse_ref import index_inverse_ref, index_inverse_loops
    g = np.random.default_rng(3)
    for s_q, topk, s_kv, start in [(5, 8, 13, None), (9, 16, 7, 2), (1, 32, 300, None), (0, 4, 5, None)]:
        idx = g.integers(-3, s_kv + 3, size=(s_q, topk)).astype(np.int32)
        a_ptr, a_ent = index_inverse_ref(idx, s_kv, start)
        b_ptr, b_ent = index_inverse_loops(idx, s_kv, start)
        assert np.array_equal(a_ptr, b_ptr) and np.array_equal(a_ent, b_ent)
    lib = op.load_library()
    assert lib.smla_index_inverse_workspace_size(4096, 2048, 32768) >= 3 * 4096 * 2048 * 4
    assert lib.smla_index_inverse_workspace_size(4, 0, 10) == 0
    assert lib.smla_index_inverse_workspace_size(1 << 20, 1 << 12, 10) == 0      # s_q * topk needs more than 31 bits
    assert lib.smla_index_inverse(None, 4, 32, 0, 0, None, None, None, 0, None) == 1
    assert lib.smla_index_inverse(None, 4, 32, 10, 0, None, None, None, 0, None) == 1


def test_header_is_plain_c_and_links_from_a_c_program(tmp_path):
    """The boundary is a C ABI: the header compiles as C99 and a C program links the library and calls it (entry
    points that need no device: sizes, argument checks, the status text)."""
    import shutil
    import subprocess
    if shutil.which("gcc") is None:
        pytest.skip("no C compiler")
    lib = op.load_library()
    lib_dir = os.path.dirname(lib._name)
    src = tmp_path / "abi.c"
    src.write_text(r'''
#include <stdio.h>
#include <string.h>
#include "smla_bwd.h"
int main(void) {
    smla_bwd_params p;
    memset(&p, 0, sizeof p);
    p.s_q = 4096; p.s_kv = 32768; p.h_q = 128; p.topk = 2048; p.q_start_index_s = SMLA_NO_CAUSAL; p.lse_is_base2 = 1;
    size_t need = smla_bwd_workspace_size(&p, 0);
    if (need < (size_t)4096 * 2048 * 128 * 4) return 1;
    if (smla_bwd_run(&p, NULL, 0, NULL) != SMLA_ERR_BAD_ARG) return 2;
    if (smla_bwd_run_noalloc(NULL, NULL) != SMLA_ERR_BAD_ARG) return 3;
    if (smla_bwd_staging_bytes_per_query(&p) != (size_t)2048 * SMLA_D_QK * 4) return 4;
    printf("%s %zu\n", smla_status_string(SMLA_ERR_DEVICE_TIMEOUT), need);
    return 0;
}
''')
    exe = tmp_path / "abi"
    cmd = ["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe),
           "-L", lib_dir, "-lsmla_bwd", "-Wl,-rpath," + lib_dir]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True)
    assert run.returncode == 0, (run.returncode, run.stdout, run.stderr)
    assert "bounded wait" in run.stdout
