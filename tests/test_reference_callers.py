"""The reference project's own callers, unmodified, on this library's modules.

``end2end/gcn/external_backend_spmm.py`` (the router: loads an extension module by name from a
search path, resolves entry points per variant, caches the preprocess result, pads N to a tile
width; :500-601, :632-763, :805-920) and ``end2end/gcn/eva_gcn_sparsene.py`` (the GCN driver:
``SpMMBackend``, ``ReplaceableSpMMFunction`` with its transposed product in backward, the model;
:189-345) are imported from a checkout of the reference -- ``$MASK_REF``, else a folder
``reference`` beside this repository -- and pointed at ``mask_b200/ext`` with the router's own
environment switches.  Nothing of the reference is edited or copied.  Skipped where no checkout
is present."""
import importlib
import os
import sys

import numpy as np
import pytest

from tests import cases

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXT = os.path.join(ROOT, "mask_b200", "ext")
REF = os.environ.get("MASK_REF") or os.path.join(os.path.dirname(ROOT), "reference")
GCN_DIR = os.path.join(REF, "end2end", "gcn")

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not os.path.isfile(os.path.join(GCN_DIR, "external_backend_spmm.py")),
                                 reason="needs a checkout of the reference project (MASK_REF)")]


@pytest.fixture
def router(monkeypatch):
    """The reference router, freshly imported, with its module search path on mask_b200/ext."""
    for k, v in {"SPARSENE_SRBCRS_MODULE_PATH": EXT, "SPARSENE_SRBCRS_ALLOW_NON_SRC_FP32": "1",
                 "SPARSENE_DTC_MODULE_PATH": EXT, "SPARSENE_DTC_ALLOW_NON_SRC_FP32": "1",
                 "SPARSENE_ALLOW_CSR_FALLBACK": "0"}.items():
        monkeypatch.setenv(k, v)
    for k in ("SPARSENE_SRBCRS_VARIANT", "SPARSENE_SPMM_VARIANT", "SPARSENE_DTC_VARIANT", "SPARSENE_SPMM_BACKEND",
              "SPARSENE_SRBCRS_BALANCE", "SPARSENE_SRBCRS_TILE_B", "SPARSENE_DTC_TILE_B"):
        monkeypatch.delenv(k, raising=False)
    monkeypatch.syspath_prepend(GCN_DIR)
    for name in ("external_backend_spmm", "eva_gcn_sparsene", "SRBCRSSpMM", "DTCSpMM", "_common"):
        sys.modules.pop(name, None)
    mod = importlib.import_module("external_backend_spmm")
    mod.reset_backend_state()
    yield mod
    mod.reset_backend_state()
    for name in ("external_backend_spmm", "eva_gcn_sparsene", "SRBCRSSpMM", "DTCSpMM", "_common"):
        sys.modules.pop(name, None)


def _dev(m):
    import torch
    return (torch.from_numpy(m.rowptr).cuda(), torch.from_numpy(m.colind).cuda(), torch.from_numpy(m.values).cuda())


@pytest.mark.parametrize("variant", ["16x8", "16x8_strict_lb", "16x8_multi_binding"])
@pytest.mark.parametrize("N", [64, 30])
def test_router_srbcrs_spmm(router, oracle_mod, monkeypatch, variant, N):
    import torch
    monkeypatch.setenv("SPARSENE_SRBCRS_VARIANT", variant)
    m = cases.SMALL["rmat10"]()
    rp, ci, va = _dev(m)
    B = np.random.Generator(np.random.PCG64(61)).standard_normal((m.K, N), dtype=np.float32)
    Bd = torch.from_numpy(B).cuda()
    out = router.srbcrs_spmm(rp, ci, va, Bd, m.M, N, m.M)
    backend = router._ROUTER.get(router.BackendConfig(name="sr_bcrs", variant=variant))
    assert os.path.dirname(os.path.abspath(backend._module.__file__)) == EXT      # our module, not a fallback
    assert backend._preprocess_func.__name__ == {"16x8": "preprocess_gpu_16x8", "16x8_strict_lb": "preprocess_gpu_16x8_strict_lb",
                                                 "16x8_multi_binding": "preprocess_gpu_16x8_multi_binding"}[variant]
    assert out.shape == (m.M, N)
    ref = oracle_mod.spmm_f32(m.M, m.rowptr, m.colind, m.values, B)
    absp = oracle_mod.spmm_abs_f64(m.M, m.rowptr, m.colind, m.values, B)
    assert oracle_mod.check_tolerance(out.cpu().numpy(), ref, absp)[0] == 0
    # second call: the router's preprocess cache hits, same result; the balance entry point too
    out2 = router.srbcrs_spmm(rp, ci, va, Bd, m.M, N, m.M)
    assert torch.equal(out, out2) and len(backend._cache) == 1
    monkeypatch.setenv("SPARSENE_SRBCRS_BALANCE", "1")
    out3 = router.srbcrs_spmm(rp, ci, va, Bd, m.M, N, m.M)
    assert oracle_mod.check_tolerance(out3.cpu().numpy(), ref, absp)[0] == 0


def test_router_base_variant_fails_loudly(router, monkeypatch):
    """The router's default SR-BCRS variant is the 32x32 one, which this library does not build:
    with the CSR fallback off (its default) the caller gets a RuntimeError, not a silent detour."""
    import torch
    monkeypatch.setenv("SPARSENE_SRBCRS_VARIANT", "base")
    m = cases.SMALL["rmat10"]()
    rp, ci, va = _dev(m)
    with pytest.raises(RuntimeError):
        router.srbcrs_spmm(rp, ci, va, torch.zeros((m.K, 32), device="cuda"), m.M, 32, m.M)


@pytest.mark.parametrize("variant", ["base", "strict_lb", "multi_binding"])
def test_router_dtc_spmm(router, oracle_mod, monkeypatch, variant):
    """ME-TCF through the router: the reference's DTC preprocess takes no values (unit-weight graphs,
    examples/src_fp32/dtc/testbed/DTCSpMM_kernel.cu:450), so the product is pattern x dense."""
    import torch
    monkeypatch.setenv("SPARSENE_DTC_VARIANT", variant)
    m = cases.SMALL["rmat10"]()
    rp, ci, va = _dev(m)
    B = np.random.Generator(np.random.PCG64(62)).standard_normal((m.K, 48), dtype=np.float32)
    out = router.dtc_spmm(rp, ci, va, torch.from_numpy(B).cuda(), m.M, 48, m.M)
    backend = router._ROUTER.get(router.BackendConfig(name="dtc", variant=variant))
    assert os.path.dirname(os.path.abspath(backend._module.__file__)) == EXT
    ones = np.ones_like(m.values)
    ref = oracle_mod.spmm_f32(m.M, m.rowptr, m.colind, ones, B)
    absp = oracle_mod.spmm_abs_f64(m.M, m.rowptr, m.colind, ones, B)
    assert out.shape == (m.M, 48)
    assert oracle_mod.check_tolerance(out.cpu().numpy(), ref, absp)[0] == 0


def test_router_spmm_external_dispatch(router, oracle_mod, monkeypatch):
    import torch
    monkeypatch.setenv("SPARSENE_SPMM_BACKEND", "sr_bcrs")
    monkeypatch.setenv("SPARSENE_SRBCRS_VARIANT", "16x8")
    m = cases.SMALL["uniform512"]()
    rp, ci, va = _dev(m)
    B = np.random.Generator(np.random.PCG64(63)).standard_normal((m.K, 128), dtype=np.float32)
    out = router.spmm_external(rp.to(torch.int64), ci.to(torch.int64), va, torch.from_numpy(B).cuda(), m.M, 128, m.M)
    ref = oracle_mod.spmm_f32(m.M, m.rowptr, m.colind, m.values, B)
    absp = oracle_mod.spmm_abs_f64(m.M, m.rowptr, m.colind, m.values, B)
    assert oracle_mod.check_tolerance(out.cpu().numpy(), ref, absp)[0] == 0


def test_gcn_driver_forward_and_backward(router, monkeypatch):
    """The reference's GCN model and autograd function, one training step: forward uses A, backward
    A^T (a non-symmetric A, so the two differ), both through the router on this library; the same
    model on the driver's own torch backend (cuSPARSE CSR, FP32) is the comparison."""
    import scipy.sparse as sp
    import torch
    monkeypatch.setenv("SPARSENE_SRBCRS_VARIANT", "16x8")
    drv = importlib.import_module("eva_gcn_sparsene")
    m = cases.SMALL["uniform512"]()          # square, not symmetric
    A = sp.csr_matrix((m.values, m.colind, m.rowptr), shape=(m.M, m.K))
    At = A.T.tocsr()
    At.sort_indices()
    dev = torch.device("cuda")
    t = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a)).to(dev, dt)  # noqa: E731
    g = torch.Generator().manual_seed(5)
    data = drv.GraphData(name="uniform512", num_nodes=m.M, num_edges=m.nnz,
                         rowptr=t(m.rowptr, torch.int64), colind=t(m.colind, torch.int64), values=t(m.values, torch.float32),
                         rowptr_t=t(At.indptr, torch.int64), colind_t=t(At.indices, torch.int64), values_t=t(At.data, torch.float32),
                         edge_index=torch.zeros((2, 0), dtype=torch.int64, device=dev), framework_graph=None,
                         x=torch.randn((m.M, 32), generator=g).to(dev), y=torch.randint(0, 8, (m.M,), generator=g).to(dev))
    torch.manual_seed(11)
    model = drv.ReplaceableGCN(32, 16, 8, num_layers=3, dropout=0.0).to(dev)
    results = {}
    for which in ("external", "torch"):
        backend = drv.SpMMBackend.build(which, "external_backend_spmm", "srbcrs_spmm")
        model.zero_grad(set_to_none=True)
        out = model(data, backend)
        loss = torch.nn.functional.nll_loss(out, data.y)
        loss.backward()
        results[which] = (out.detach().clone(), [p.grad.detach().clone() for p in model.parameters()])
    assert router._ROUTER.get(router.BackendConfig(name="sr_bcrs", variant="16x8"))._cache, "the router never reached the extension"
    out_e, grads_e = results["external"]
    out_t, grads_t = results["torch"]
    assert torch.allclose(out_e, out_t, rtol=2e-2, atol=2e-2)
    for ge, gt in zip(grads_e, grads_t):
        assert float((ge - gt).abs().max()) <= 2e-2 * float(gt.abs().max()) + 1e-5
