"""The hand-written sm_100a operator include (include/mask_b200_operator_sm100.inc) under the
reference's own Format-DSL host bridge: the bridge executable is the reference's translation unit
(its main, its packer, its cuSPARSE comparison with atol = rtol = 1e-3 over every element, its
JSON report) built by oracle/Makefile with the operator swapped in; only the included kernels are
ours.  Exit code 0 means the bridge's own verification passed."""
import json
import os
import subprocess

import pytest

from mask_b200 import generators as G
from tests import cases

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(ROOT, "oracle", "_ref")


def _exe(name):
    p = os.path.join(REF_DIR, name)
    if not os.path.exists(p):
        pytest.skip(f"{name} not built (needs a checkout of the reference: make -C oracle bridge)")
    return p


def _run(exe, mtx, out, n, policy, extra=()):
    cmd = [exe, "--filename", mtx, "--dataset", "t", "--result-json", out, "--n", str(n), "--warmup", "1", "--repeat", "2",
           "--execution-policy", policy, "--task-group-tiles", "16", *extra]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    rep = json.load(open(out)) if os.path.exists(out) else None
    return r, rep


def test_operator_declares_the_bridge_contract():
    src = open(os.path.join(ROOT, "include", "mask_b200_operator_sm100.inc")).read()
    for token in ("#define SPARSENE_GENERATED_REQUIRES_SINGLE_WARP 1", "#define SPARSENE_GENERATED_THREADS_PER_BLOCK 32",
                  "#define SPARSENE_GENERATED_SUPPORTS_TASK_MAPPING 1", "generated_kernel(", "generated_task_mapped_kernel(",
                  "generated_bound_task_kernel("):
        assert token in src


@pytest.mark.gpu
@pytest.mark.parametrize("tile_n,n", [(64, 128), (128, 256)])
@pytest.mark.parametrize("policy,extra", [("row", ()), ("strict_lb", ()), ("multi_bind", ()), ("auto", ("--max-tiles-per-segment", "0")),
                                          ("row", ("--max-tiles-per-segment", "0"))])
@pytest.mark.parametrize("name", ["hub_rows", "rmat10", "m33_empty_window", "stencil8"])
def test_bridge_accepts_the_sm100_operator(tmp_path, name, policy, extra, tile_n, n):
    exe = _exe(f"bridge_sm100_tn{tile_n}")
    m = cases.SMALL[name]()
    mtx = str(tmp_path / "m.mtx")
    G.write_matrix_market(m, mtx)
    r, rep = _run(exe, mtx, str(tmp_path / "out.json"), n, policy, extra)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert rep["correctness"]["passed"] is True and rep["correctness"]["mismatches"] == 0
    assert rep["shape"]["M"] == m.M and rep["shape"]["nnz"] == m.nnz
    if policy in ("strict_lb", "multi_bind"):
        assert rep["packed"]["execution_policy"] == policy and rep["packed"]["task_groups"] > 0


@pytest.mark.gpu
def test_same_result_quality_as_the_emitted_operator(tmp_path):
    """Same bridge, same matrix: the reference compiler's own operator and ours both pass, with
    errors of the same size against cuSPARSE (both round the two operands to TF32)."""
    ours, theirs = _exe("bridge_sm100_tn64"), _exe("bridge_refgen_tn64")
    m = cases.SMALL["rmat12u"]()
    mtx = str(tmp_path / "m.mtx")
    G.write_matrix_market(m, mtx)
    for policy in ("row", "strict_lb", "multi_bind"):
        r1, a = _run(ours, mtx, str(tmp_path / "a.json"), 128, policy)
        r2, b = _run(theirs, mtx, str(tmp_path / "b.json"), 128, policy)
        assert r1.returncode == 0 and r2.returncode == 0, (r1.stdout, r1.stderr, r2.stdout, r2.stderr)
        assert a["packed"] == b["packed"]
        assert a["correctness"]["max_abs_error"] <= 2.0 * b["correctness"]["max_abs_error"] + 1e-6
