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
    """Ours must pass the bridge's gate wherever the operator emitted by the reference's compiler
    passes it (very long rows can miss it for both: FP32 summation order against cuSPARSE), with
    an error of the same size."""
    exe, ref_exe = _exe(f"bridge_sm100_tn{tile_n}"), _exe("bridge_refgen_tn64")
    m = cases.SMALL[name]()
    mtx = str(tmp_path / "m.mtx")
    G.write_matrix_market(m, mtx)
    r, rep = _run(exe, mtx, str(tmp_path / "out.json"), n, policy, extra)
    r2, ref = _run(ref_exe, mtx, str(tmp_path / "ref.json"), n, policy, extra)
    assert r.returncode in (0, 2) and r2.returncode in (0, 2), r.stdout[-2000:] + r.stderr[-2000:]
    assert rep["shape"] == ref["shape"] and rep["shape"]["M"] == m.M and rep["shape"]["nnz"] == m.nnz
    assert rep["packed"] == ref["packed"]
    assert rep["correctness"]["nonfinite"] == 0
    assert rep["correctness"]["passed"] or not ref["correctness"]["passed"], (rep["correctness"], ref["correctness"])
    assert rep["correctness"]["max_abs_error"] <= 2.0 * ref["correctness"]["max_abs_error"] + 1e-4
    if policy in ("strict_lb", "multi_bind"):
        assert rep["packed"]["execution_policy"] == policy and rep["packed"]["task_groups"] > 0


@pytest.mark.gpu
@pytest.mark.parametrize("policy", ["row", "strict_lb", "multi_bind"])
def test_fast_tf32_switch_matches_the_emitted_operator(tmp_path, policy):
    """With SPARSENE_FAST_TF32 both operators issue one MMA per product; errors are then of TF32
    size for both."""
    ours, theirs = _exe("bridge_sm100_fast_tn64"), _exe("bridge_refgen_fast_tn64")
    m = cases.SMALL["rmat12u"]()
    mtx = str(tmp_path / "m.mtx")
    G.write_matrix_market(m, mtx)
    r1, a = _run(ours, mtx, str(tmp_path / "a.json"), 128, policy)
    r2, b = _run(theirs, mtx, str(tmp_path / "b.json"), 128, policy)
    assert r1.returncode in (0, 2) and r2.returncode in (0, 2)
    assert a["packed"] == b["packed"]
    assert a["correctness"]["nonfinite"] == 0
    assert a["correctness"]["max_abs_error"] <= 2.0 * b["correctness"]["max_abs_error"] + 1e-4


def _run_dtc(exe, mtx, n):
    env = dict(os.environ, SPARSENE_DISABLE_MTX_CACHE="1")
    r = subprocess.run([exe, "-filename", mtx, "-N", str(n), "-warmup", "1", "-repeat", "2"], capture_output=True, text=True,
                       timeout=300, env=env)
    out = {}
    for line in r.stdout.splitlines():
        if line.startswith("VERIFICATION"):
            out.update({kv.split("=")[0]: float(kv.split("=")[1]) for kv in line.split()[1:]})
        if line.startswith("mykernel_time:"):
            out["ms"] = float(line.split()[1])
    return r, out


def test_metcf_operator_declares_the_seam():
    src = open(os.path.join(ROOT, "include", "mask_b200_operator_metcf_sm100.inc")).read()
    for token in ("#define SPARSENE_GENERATED_TILE_B", "CHECK_CUDA2", "generated_kernel(float* dB_val, float* dC, int* dval_coo_idx_new"):
        assert token in src


@pytest.mark.gpu
@pytest.mark.parametrize("n", [128, 96, 48])      # the host program picks TILE_B = 64, 32, 16
@pytest.mark.parametrize("name", ["hub_rows", "rmat10", "m33_empty_window", "stencil8", "uniform512"])
def test_dtc_generated_seam_accepts_the_sm100_operator(tmp_path, name, n):
    """The reference's ME-TCF testbed (its main, packer, timing loop and cuSPARSE gate, atol = rtol
    = 1e-3) built with the hand-written operator include: exit code 0 = its verification passed;
    the same binary with the include kept in the reference tree is run beside it."""
    ours, theirs = _exe("dtc_generated_sm100"), _exe("dtc_generated_ref")
    m = cases.SMALL[name]()
    mtx = str(tmp_path / "m.mtx")
    G.write_matrix_market(m, mtx)
    r, a = _run_dtc(ours, mtx, n)
    r2, b = _run_dtc(theirs, mtx, n)
    assert "errors" in a and "ms" in a, r.stdout[-1500:] + r.stderr[-1500:]
    assert a["nonfinite"] == 0
    assert (r.returncode == 0 and a["errors"] == 0) or r2.returncode != 0, (a, b, r.stdout[-800:])
    assert a["max_abs_error"] <= 2.0 * b.get("max_abs_error", 0.0) + 1e-4


@pytest.mark.gpu
@pytest.mark.parametrize("name,n", [("hub_rows", 128), ("rmat10", 512), ("m33_empty_window", 64), ("stencil8", 256)])
def test_srbcrs_testbed_seam(tmp_path, name, n):
    """The reference's SR-BCRS testbed main (MatrixMarket reader, its own SR-BCRS packer, cuSPARSE
    check with atol = rtol = 1e-3) linked against libmask_b200.so through the replacement host
    program mask_b200/seams/sr_bcrs_host_program_16x8.cu: the seam sr_bcrs_test_tf32<16,64,8>."""
    exe = _exe("srbcrs_testbed_sm100")
    m = cases.SMALL[name]()
    mtx = str(tmp_path / "m.mtx")
    G.write_matrix_market(m, mtx)
    r = subprocess.run([exe, "-filename", mtx, "-N", str(n), "-warmup", "1", "-repeat", "2"], capture_output=True, text=True,
                       timeout=300)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-1500:]
    assert "correctness: PASS" in r.stdout and "mykernel_time:" in r.stdout


@pytest.mark.gpu
@pytest.mark.parametrize("name,n", [("hub_rows", 128), ("rmat10", 512), ("m33_empty_window", 48), ("stencil8", 96)])
def test_dtc_testbed_seam(tmp_path, name, n):
    """The reference's ME-TCF testbed main (its ME-TCF packer and cuSPARSE check) linked against
    libmask_b200.so through mask_b200/seams/dtc_host_program.cu: the seam
    dtc_spmm_test_val_sidx_bind_reorder<TILE_B>."""
    exe = _exe("dtc_testbed_sm100")
    m = cases.SMALL[name]()
    mtx = str(tmp_path / "m.mtx")
    G.write_matrix_market(m, mtx)
    r, a = _run_dtc(exe, mtx, n)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-1500:]
    assert a["errors"] == 0 and a["nonfinite"] == 0 and "ms" in a
