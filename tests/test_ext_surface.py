"""The reference-named Python modules (SRBCRSSpMM, DTCSpMM) and the caller-level callables:
CPU tests check names and host-side error behaviour, GPU tests call them the way the reference's
router does (end2end/gcn/external_backend_spmm.py:805-920) and compare with the oracle."""
import importlib
import os
import sys

import numpy as np
import pytest

from tests import cases

EXT = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "mask_b200", "ext")

# names the reference router resolves, first match wins (external_backend_spmm.py:632-763, 420-480)
SRBCRS_NAMES = ["preprocess_gpu", "preprocess_gpu_16x8", "run_SRBCRS", "run_SRBCRS_balance", "run_SRBCRS_16x8",
                "run_SRBCRS_16x8_balance", "preprocess_gpu_16x8_strict_lb", "run_SRBCRS_16x8_strict_lb",
                "preprocess_gpu_16x8_multi_binding", "run_SRBCRS_16x8_multi_binding",
                "run_SRBCRS_16x8_strict_lb_balance", "run_SRBCRS_16x8_multi_binding_balance"]
DTC_NAMES = ["preprocess_gpu", "run_DTCSpMM", "preprocess_gpu_strict_lb", "preprocess_gpu_multi_binding",
             "run_DTCSpMM_strict_lb", "run_DTCSpMM_multi_binding", "run_DTCSpMM_balance",
             "run_DTCSpMM_strict_lb_balance", "run_DTCSpMM_multi_binding_balance", "DTCSpMM_gcn"]


def _mod(name):
    if EXT not in sys.path:
        sys.path.insert(0, EXT)
    return importlib.import_module(name)


def test_modules_export_the_reference_names():
    sr, dt = _mod("SRBCRSSpMM"), _mod("DTCSpMM")
    for n in SRBCRS_NAMES:
        assert callable(getattr(sr, n)), n
    for n in DTC_NAMES:
        assert callable(getattr(dt, n)), n
    assert os.path.dirname(os.path.abspath(sr.__file__)) == EXT


def test_host_side_errors_without_gpu():
    import torch
    sr = _mod("SRBCRSSpMM")
    cpu_i = torch.zeros(4, dtype=torch.int32)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        sr.preprocess_gpu_16x8(cpu_i, cpu_i, torch.zeros(4), 3, 16, 8, cpu_i, cpu_i, cpu_i)
    with pytest.raises(RuntimeError, match="32x32"):
        sr.preprocess_gpu(cpu_i, cpu_i, torch.zeros(4), 3, 32, 32, cpu_i, cpu_i, cpu_i)
    with pytest.raises(RuntimeError, match="32x32"):
        sr.run_SRBCRS()
    from mask_b200 import spmm_backend
    spmm_backend.reset_backend_state()
    os.environ["SPARSENE_SPMM_BACKEND"] = "flashsparse"
    try:
        with pytest.raises(RuntimeError, match="not provided"):
            spmm_backend.spmm_external(None, None, None, None, 1, 1, 1)
    finally:
        del os.environ["SPARSENE_SPMM_BACKEND"]


def _dev(m):
    import torch
    return (torch.from_numpy(m.rowptr).cuda(), torch.from_numpy(m.colind).cuda(), torch.from_numpy(m.values).cuda())


@pytest.mark.gpu
@pytest.mark.parametrize("variant", ["16x8", "16x8_strict_lb", "16x8_multi_binding"])
def test_srbcrs_module_router_convention(oracle_mod, variant):
    import torch
    sr = _mod("SRBCRSSpMM")
    m = cases.SMALL["rmat10"]()
    rp, ci, va = _dev(m)
    W = (m.M + 15) // 16
    bp = torch.zeros(W, dtype=torch.int32, device="cuda")
    e2c = torch.zeros(m.nnz, dtype=torch.int32, device="cuda")
    e2r = torch.zeros(m.nnz, dtype=torch.int32, device="cuda")
    pre = {"16x8": sr.preprocess_gpu_16x8, "16x8_strict_lb": sr.preprocess_gpu_16x8_strict_lb,
           "16x8_multi_binding": sr.preprocess_gpu_16x8_multi_binding}[variant]
    runf = {"16x8": sr.run_SRBCRS_16x8, "16x8_strict_lb": sr.run_SRBCRS_16x8_strict_lb,
            "16x8_multi_binding": sr.run_SRBCRS_16x8_multi_binding}[variant]
    rwo, rowid, tile_id, tc_off, a2x, T = pre(ci, rp, va, m.M, 16, 8, bp, e2c, e2r)
    want = oracle_mod.pack_srbcrs(m.M, m.rowptr, m.colind, m.values)
    assert T == want["T"] and rowid.numel() == T and tc_off.numel() == 1 and a2x.numel() == 1
    assert np.array_equal(rwo.cpu().numpy(), want["val_soff"]) and np.array_equal(tile_id.cpu().numpy(), want["val_sidx"])
    obp, oe2c, oe2r = oracle_mod.edge_maps(m.M, m.rowptr, m.colind)
    assert np.array_equal(bp.cpu().numpy(), obp) and np.array_equal(e2c.cpu().numpy(), oe2c)
    assert np.array_equal(e2r.cpu().numpy(), oe2r)
    B = np.random.Generator(np.random.PCG64(5)).standard_normal((m.K, 64), dtype=np.float32)
    out = runf(torch.from_numpy(B).cuda(), rwo, tile_id, tc_off, a2x, m.M, m.nnz, "")
    assert isinstance(out, list) and out[0].shape == (m.M, 64)
    ref = oracle_mod.spmm_f32(m.M, m.rowptr, m.colind, m.values, B)
    absp = oracle_mod.spmm_abs_f64(m.M, m.rowptr, m.colind, m.values, B)
    assert oracle_mod.check_tolerance(out[0].cpu().numpy(), ref, absp)[0] == 0
    out_b = sr.run_SRBCRS_16x8_balance(torch.from_numpy(B).cuda(), rwo, tile_id, tc_off, a2x, m.M, "")
    assert torch.equal(out_b[0], sr.run_SRBCRS_16x8(torch.from_numpy(B).cuda(), rwo, tile_id, tc_off, a2x, m.M, m.nnz, "")[0])
    assert sr.run_SRBCRS_16x8(torch.zeros((m.K, 0), device="cuda"), rwo, tile_id, tc_off, a2x, m.M, m.nnz, "")[0].shape == (m.M, 0)
    with pytest.raises(RuntimeError, match="cache miss"):
        sr.run_SRBCRS_16x8(torch.from_numpy(B).cuda(), rwo.clone(), tile_id, tc_off, a2x, m.M, m.nnz, "")
    with pytest.raises(RuntimeError, match="blk_h"):
        sr.preprocess_gpu_16x8(ci, rp, va, m.M, 32, 32, bp, e2c, e2r)


@pytest.mark.gpu
def test_dtc_module_router_convention(oracle_mod):
    import torch
    dt = _mod("DTCSpMM")
    m = cases.SMALL["rmat10"]()
    rp, ci, va = _dev(m)
    W = (m.M + 15) // 16
    bp = torch.zeros(W, dtype=torch.int32, device="cuda")
    e2c = torch.zeros(m.nnz, dtype=torch.int32, device="cuda")
    e2r = torch.zeros(m.nnz, dtype=torch.int32, device="cuda")
    B = np.random.Generator(np.random.PCG64(6)).standard_normal((m.K, 32), dtype=np.float32)
    # reference behaviour: unit weights
    rwo, rowid, tile_id, coo_off, coo_idx, T = dt.preprocess_gpu(ci, rp, m.M, 16, 8, bp, e2c, e2r)
    want = oracle_mod.pack_metcf(m.M, m.rowptr, m.colind, np.ones_like(m.values))
    assert T == want["T"] and np.array_equal(coo_off.cpu().numpy(), want["val_coo_off"])
    assert np.array_equal(coo_idx.cpu().numpy(), want["val_coo_idx"]) and np.array_equal(tile_id.cpu().numpy(), want["val_sidx"])
    out = dt.run_DTCSpMM(torch.from_numpy(B).cuda(), rwo, tile_id, coo_off, coo_idx, m.M, m.nnz, "")[0]
    ones = np.ones_like(m.values)
    ref = oracle_mod.spmm_f32(m.M, m.rowptr, m.colind, ones, B)
    absp = oracle_mod.spmm_abs_f64(m.M, m.rowptr, m.colind, ones, B)
    assert oracle_mod.check_tolerance(out.cpu().numpy(), ref, absp)[0] == 0
    # with real values, through the strict_lb names
    rwo2, _, tile2, off2, idx2, _ = dt.preprocess_gpu_strict_lb(ci, rp, m.M, 16, 8, bp, e2c, e2r, values=va)
    out2 = dt.run_DTCSpMM_strict_lb(torch.from_numpy(B).cuda(), rwo2, tile2, off2, idx2, m.M, m.nnz, "")[0]
    ref2 = oracle_mod.spmm_f32(m.M, m.rowptr, m.colind, m.values, B)
    absp2 = oracle_mod.spmm_abs_f64(m.M, m.rowptr, m.colind, m.values, B)
    assert oracle_mod.check_tolerance(out2.cpu().numpy(), ref2, absp2)[0] == 0


@pytest.mark.gpu
def test_caller_level_callables(oracle_mod):
    import torch
    from mask_b200 import spmm_backend
    spmm_backend.reset_backend_state()
    m = cases.SMALL["hub_rows"]()
    rp, ci, va = _dev(m)
    B = np.random.Generator(np.random.PCG64(8)).standard_normal((m.K, 30), dtype=np.float32)  # N % 4 != 0: padded
    Bd = torch.from_numpy(B).cuda()
    ref = oracle_mod.spmm_f32(m.M, m.rowptr, m.colind, m.values, B)
    absp = oracle_mod.spmm_abs_f64(m.M, m.rowptr, m.colind, m.values, B)
    for fn in (spmm_backend.srbcrs_spmm, spmm_backend.dtc_spmm, spmm_backend.spmm_external):
        out = fn(rp.to(torch.int64), ci.to(torch.int64), va, Bd, m.M, 30, m.M)
        assert out.shape == (m.M, 30)
        assert oracle_mod.check_tolerance(out.cpu().numpy(), ref, absp)[0] == 0
    n_cached = len(spmm_backend._cache)
    spmm_backend.srbcrs_spmm(rp.to(torch.int64), ci.to(torch.int64), va, Bd, m.M, 30, m.M)
    assert len(spmm_backend._cache) > 0 and n_cached >= 2
    spmm_backend.reset_backend_state()
    assert not spmm_backend._cache


@pytest.mark.gpu
def test_dense_operand_layouts_like_the_reference(oracle_mod):
    """The reference extension makes `dense` contiguous itself and does not care how many rows it
    has beyond the matrix's columns; pattern-only graphs (values=None) multiply with unit weights."""
    import torch
    from mask_b200 import spmm_backend
    sr = _mod("SRBCRSSpMM")
    m = cases.SMALL["rmat10"]()
    rp, ci, va = _dev(m)
    W = (m.M + 15) // 16
    bp = torch.zeros(W, dtype=torch.int32, device="cuda")
    e2c = torch.zeros(m.nnz, dtype=torch.int32, device="cuda")
    e2r = torch.zeros(m.nnz, dtype=torch.int32, device="cuda")
    rwo, _, tile_id, tc_off, a2x, _ = sr.preprocess_gpu_16x8(ci, rp, va, m.M, 16, 8, bp, e2c, e2r)
    B = np.random.Generator(np.random.PCG64(15)).standard_normal((m.K + 40, 64), dtype=np.float32)
    ref = oracle_mod.spmm_f32(m.M, m.rowptr, m.colind, m.values, B[: m.K])
    absp = oracle_mod.spmm_abs_f64(m.M, m.rowptr, m.colind, m.values, B[: m.K])
    tall = torch.from_numpy(B).cuda()                                   # more rows than columns of A
    strided = torch.from_numpy(np.ascontiguousarray(B.T)).cuda().t()    # column-major storage
    assert not strided.is_contiguous()
    for d in (tall, strided):
        out = sr.run_SRBCRS_16x8(d, rwo, tile_id, tc_off, a2x, m.M, m.nnz, "")[0]
        assert oracle_mod.check_tolerance(out.cpu().numpy(), ref, absp)[0] == 0
    with pytest.raises(RuntimeError, match="rows"):
        sr.run_SRBCRS_16x8(tall[: m.K - 1], rwo, tile_id, tc_off, a2x, m.M, m.nnz, "")
    spmm_backend.reset_backend_state()
    ones = np.ones_like(m.values)
    out = spmm_backend.srbcrs_spmm(rp, ci, None, tall[: m.K], m.M, 64, m.M)
    ref1 = oracle_mod.spmm_f32(m.M, m.rowptr, m.colind, ones, B[: m.K])
    absp1 = oracle_mod.spmm_abs_f64(m.M, m.rowptr, m.colind, ones, B[: m.K])
    assert oracle_mod.check_tolerance(out.cpu().numpy(), ref1, absp1)[0] == 0
    spmm_backend.reset_backend_state()
