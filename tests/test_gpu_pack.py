"""GPU parity: the device format builder against the CPU oracle and the golden fixtures,
bit for bit, through the C ABI."""
import numpy as np
import pytest

from tests import cases

pytestmark = pytest.mark.gpu
BITS = lambda a: np.ascontiguousarray(a).view(np.int32) if a.dtype == np.float32 else a


def _dev(m):
    import torch
    return (torch.from_numpy(m.rowptr).cuda(), torch.from_numpy(m.colind).cuda(), torch.from_numpy(m.values).cuda())


def _check_srbcrs(p, want, prefix=""):
    assert p.T == len(want[prefix + "val_sidx"]) // 8
    for k in ("val_soff", "val_sidx", "val_block_val"):
        assert np.array_equal(BITS(getattr(p, k).cpu().numpy()), BITS(want[prefix + k])), k


def _check_metcf(p, want, prefix=""):
    assert p.nnz_pad == len(want[prefix + "val_coo_idx"])
    for k in ("val_soff", "val_sidx", "val_coo_off", "val_coo_idx", "val_coo_val"):
        assert np.array_equal(BITS(getattr(p, k).cpu().numpy()), BITS(want[prefix + k])), k


def _check_mco(p, want, prefix=""):
    assert p.T == int(want[prefix + "val_soff"][-1])
    for k in ("val_soff", "val_sidx", "val_mco_off", "val_mco_val"):
        assert np.array_equal(BITS(getattr(p, k).cpu().numpy()), BITS(want[prefix + k])), k
    assert np.array_equal(p.val_mco_mask.cpu().numpy().view(np.uint64), want[prefix + "val_mco_mask"])


@pytest.mark.parametrize("name", cases.golden_names())
def test_pack_mco_matches_golden(name):
    """The bitmap leaf against arrays made by the reference bridge's own packer."""
    from mask_b200 import engine
    m, g = cases.load_golden(name)
    rp, ci, va = _dev(m)
    _check_mco(engine.pack_mco(rp, ci, va, m.M, m.K, skip_zero_values=True), g, "mco_")


@pytest.mark.parametrize("name", sorted(cases.SMALL))
def test_pack_mco_matches_oracle(oracle_mod, name):
    from mask_b200 import engine
    m = cases.SMALL[name]()
    rp, ci, va = _dev(m)
    _check_mco(engine.pack_mco(rp, ci, va, m.M, m.K), oracle_mod.pack_mco(m.M, m.rowptr, m.colind, m.values))
    # explicit zeros: kept by the BIT-TCF testbed packer, dropped by the bridge's
    vz = m.values.copy()
    vz[::3] = 0.0
    import torch
    vzd = torch.from_numpy(vz).cuda()
    for skip in (False, True):
        _check_mco(engine.pack_mco(rp, ci, vzd, m.M, m.K, skip_zero_values=skip),
                   oracle_mod.pack_mco(m.M, m.rowptr, m.colind, vz, skip_zero_values=skip))
    _check_mco(engine.pack_mco(rp, ci, None, m.M, m.K), oracle_mod.pack_mco(m.M, m.rowptr, m.colind, np.ones_like(m.values)))


@pytest.mark.parametrize("name", cases.golden_names())
def test_pack_matches_golden(name):
    from mask_b200 import engine
    m, g = cases.load_golden(name)
    rp, ci, va = _dev(m)
    _check_srbcrs(engine.pack_srbcrs(rp, ci, va, m.M, m.K), g, "sr_")
    _check_metcf(engine.pack_metcf(rp, ci, va, m.M, m.K), g, "me_")


@pytest.mark.parametrize("name", sorted(cases.SMALL))
def test_pack_matches_oracle(oracle_mod, name):
    from mask_b200 import engine
    m = cases.SMALL[name]()
    rp, ci, va = _dev(m)
    p = engine.pack_srbcrs(rp, ci, va, m.M, m.K, side_outputs=True)
    _check_srbcrs(p, oracle_mod.pack_srbcrs(m.M, m.rowptr, m.colind, m.values))
    bp, e2c, e2r = oracle_mod.edge_maps(m.M, m.rowptr, m.colind)
    assert np.array_equal(p.block_partition.cpu().numpy(), bp)
    assert np.array_equal(p.edge_to_col.cpu().numpy(), e2c)
    assert np.array_equal(p.edge_to_row.cpu().numpy(), e2r)
    _check_metcf(engine.pack_metcf(rp, ci, va, m.M, m.K), oracle_mod.pack_metcf(m.M, m.rowptr, m.colind, m.values))


def test_pack_metcf_unit_values(oracle_mod):
    """values=None stores 1.0 for every entry, as the reference extension packer does."""
    from mask_b200 import engine
    m = cases.SMALL["rmat10"]()
    rp, ci, _ = _dev(m)
    p = engine.pack_metcf(rp, ci, None, m.M, m.K)
    _check_metcf(p, oracle_mod.pack_metcf(m.M, m.rowptr, m.colind, np.ones_like(m.values)))


@pytest.mark.parametrize("workload,kw", [("rmat20_gcn", dict(scale=16)), ("stencil27_100", dict(grid=40)),
                                         ("rmat22_sym", dict(scale=15))])
def test_pack_medium_matches_oracle(oracle_mod, workload, kw):
    """Medium sizes (hub windows with tens of thousands of entries, scans spanning many chunks)."""
    from mask_b200 import engine, generators as G
    m, _ = G.make_workload(workload, **kw)
    rp, ci, va = _dev(m)
    _check_srbcrs(engine.pack_srbcrs(rp, ci, va, m.M, m.K), oracle_mod.pack_srbcrs(m.M, m.rowptr, m.colind, m.values))
    _check_metcf(engine.pack_metcf(rp, ci, va, m.M, m.K), oracle_mod.pack_metcf(m.M, m.rowptr, m.colind, m.values))


def test_pack_rejects_bad_input():
    import torch
    from mask_b200 import engine, _lib
    m = cases.SMALL["uniform512"]()
    rp, ci, va = _dev(m)
    bad = ci.clone()
    s = int(m.rowptr[5])
    bad[s], bad[s + 1] = ci[s + 1], ci[s]  # row 5 no longer ascending
    with pytest.raises(_lib.MaskError) as e:
        engine.pack_srbcrs(rp, bad, va, m.M, m.K)
    assert e.value.status == 3
    oob = ci.clone()
    oob[0] = m.K
    with pytest.raises(_lib.MaskError) as e:
        engine.pack_srbcrs(rp, oob, va, m.M, m.K)
    assert e.value.status == 6
    with pytest.raises(RuntimeError):
        engine.pack_srbcrs(rp, ci.to(torch.int64), va, m.M, m.K)
    with pytest.raises(RuntimeError):
        engine.pack_srbcrs(rp.cpu(), ci, va, m.M, m.K)
    # the context is still healthy
    assert engine.pack_srbcrs(rp, ci, va, m.M, m.K).T > 0


def test_plan_tables(oracle_mod):
    """Plans cover every tile exactly once, in order, and the strict_lb policy reproduces the
    reference tables (plus empty fragments for windows without tiles)."""
    from mask_b200 import engine
    for name in ("m33_empty_window", "hub_rows", "rmat10", "all_empty"):
        m = cases.SMALL[name]()
        rp, ci, va = _dev(m)
        p = engine.pack_srbcrs(rp, ci, va, m.M, m.K)
        soff = p.val_soff.cpu().numpy()
        W = (m.M + 15) // 16
        for policy, gt in (("auto", 0), ("auto", 4), ("row", 0), ("strict_lb", 8), ("multi_bind", 0)):
            plan = engine.Plan(p.val_soff, m.M, p.T, policy, gt)
            fo, fw, go = (x.numpy() for x in plan.export())
            info = plan.info()
            assert fo[0] == 0 and fo[-1] == p.T and np.all(np.diff(fo) >= 0)
            assert go[0] == 0 and go[-1] == info["fragments"] and np.all(np.diff(go) > 0)
            assert np.all(np.diff(fw) >= 0) and set(fw.tolist()) == set(range(W))  # every window is written
            for f in range(info["fragments"]):
                assert soff[fw[f]] <= fo[f] and fo[f + 1] <= soff[fw[f] + 1]
            if policy == "row":
                assert info["partial"] == 0 and info["groups"] == W
            if policy == "strict_lb":
                rbo, rb2w, _ = oracle_mod.strict_lb_plan(m.M, soff, 8)
                keep = np.diff(fo) > 0
                assert np.array_equal(fo[:-1][keep], rbo[:-1]) and np.array_equal(fw[keep], rb2w)


@pytest.mark.parametrize("kind", ["first_col_sort", "jaccard_greedy", "row_rcm"])
@pytest.mark.parametrize("name", ["rmat10", "hub_rows", "m33_empty_window", "stencil8"])
def test_reordered_pack_and_product(oracle_mod, name, kind):
    """Rows reordered like the Format-DSL bridge: the packed arrays equal the oracle's pack of the
    permuted CSR, and the product comes back in the original row order (row map in the epilogue)."""
    import torch
    from mask_b200 import engine, _lib
    m = cases.SMALL[name]()
    rp, ci, va = _dev(m)
    if kind == "row_rcm" and m.M != m.K:
        with pytest.raises(_lib.MaskError):
            engine.pack_srbcrs(rp, ci, va, m.M, m.K, reorder=kind)
        return
    p = engine.pack_srbcrs(rp, ci, va, m.M, m.K, reorder=kind)
    order = oracle_mod.reorder_rows(kind, m.M, m.K, m.rowptr, m.colind)
    assert np.array_equal(p.row_order.cpu().numpy(), order)
    prp, pci, pva = oracle_mod.permute_csr(m.M, m.rowptr, m.colind, m.values, order)
    _check_srbcrs(p, oracle_mod.pack_srbcrs(m.M, prp, pci, pva))
    for N, gt in ((512, 0), (96, 3)):   # tcgen05 kernel / mma.sync kernel with split windows
        B = np.random.Generator(np.random.PCG64(N)).standard_normal((m.K, N), dtype=np.float32)
        out = torch.full((m.M, N), float("nan"), device="cuda")
        engine.spmm(p, torch.from_numpy(B).cuda(), out=out, plan=p.new_plan("auto", gt))
        ref = oracle_mod.spmm_f32(m.M, m.rowptr, m.colind, m.values, B)
        absp = oracle_mod.spmm_abs_f64(m.M, m.rowptr, m.colind, m.values, B)
        bad, worst = oracle_mod.check_tolerance(out.cpu().numpy(), ref, absp)
        assert bad == 0, worst
    with pytest.raises(RuntimeError):
        engine.spmm(p, torch.zeros((m.K, 16), device="cuda"), plan=engine.Plan(p.val_soff, m.M, p.T))


def test_generators_gpu_passes_are_exact(monkeypatch):
    """The large R-MAT workloads do their integer passes (bit assembly, sort + deduplication, value
    hash) on the GPU when one is there; the matrix must be bit-identical to the host-only path."""
    from mask_b200 import generators as G
    got = {}
    for where, floor in (("gpu", 0), ("host", 1 << 62)):
        monkeypatch.setattr(G, "GPU_MIN_ITEMS", floor)
        got[where] = (G.rmat_symmetric_uniform(scale=13, samples_per_node=16, seed=401),
                      G.rmat_gcn_normalised(scale=13, samples_per_node=8, seed=201))
    for a, b in zip(got["gpu"], got["host"]):
        assert a.M == b.M and np.array_equal(a.rowptr, b.rowptr) and np.array_equal(a.colind, b.colind)
        assert np.array_equal(a.values.view(np.int32), b.values.view(np.int32))


@pytest.mark.parametrize("name", cases.golden_names() + ["rmat10", "hub_rows", "stencil8", "all_empty", "uniform512", "rmat12u",
                                                         "m33_empty_window", "wide_k"])
def test_device_reorders_match_golden_and_oracle(oracle_mod, name):
    """mask_reorder_rows (device kernels: radix sorts, one block per Jaccard bucket, level-synchronous
    Cuthill-McKee over all components) against the fixtures made by the reference bridge and against
    the oracle's sequential restatement: the permutations must be identical."""
    import torch
    from mask_b200 import _lib, engine
    L = _lib.lib()
    if name in cases.SMALL:
        m, g = cases.SMALL[name](), {}
    else:
        m, g = cases.load_golden(name)
    rp, ci, _ = _dev(m)
    for kind in ("first_col_sort", "jaccard_greedy", "row_rcm"):
        if kind == "row_rcm" and m.M != m.K:
            with pytest.raises(_lib.MaskError):
                engine.reorder_rows(rp, ci, m.M, m.K, kind)
            continue
        order = engine.reorder_rows(rp, ci, m.M, m.K, kind).cpu().numpy()
        assert np.array_equal(np.sort(order), np.arange(m.M)), kind          # a permutation
        assert np.array_equal(order, oracle_mod.reorder_rows(kind, m.M, m.K, m.rowptr, m.colind)), kind
        if "order_" + kind in g:
            assert np.array_equal(order, g["order_" + kind]), kind
    assert np.array_equal(engine.reorder_rows(rp, ci, m.M, m.K, "none").cpu().numpy(), np.arange(m.M))
    bad = torch.zeros(m.M, dtype=torch.int32, device="cuda")
    assert L.mask_reorder_rows(9, rp.data_ptr(), ci.data_ptr(), m.M, m.K, bad.data_ptr(), None) == 1


def test_device_reorders_on_a_power_law_graph(oracle_mod):
    """2^16 nodes, hub rows with thousands of entries, thousands of isolated nodes and small
    components: every order equals the sequential one."""
    from mask_b200 import engine, generators as G
    m, _ = G.make_workload("rmat20_gcn", scale=16)
    rp, ci, _ = _dev(m)
    for kind in ("first_col_sort", "jaccard_greedy", "row_rcm"):
        order = engine.reorder_rows(rp, ci, m.M, m.K, kind).cpu().numpy()
        assert np.array_equal(order, oracle_mod.reorder_rows(kind, m.M, m.K, m.rowptr, m.colind)), kind


def test_column_features_match_numpy():
    """mask_features_columns (device: histogram of gathered ids, radix sort, prefix sums) against the
    same quantities from NumPy on the packed ids."""
    import ctypes as C
    import torch
    from mask_b200 import _lib, engine
    L = _lib.lib()
    m = cases.SMALL["rmat12u"]()
    rp, ci, va = _dev(m)
    p = engine.pack_srbcrs(rp, ci, va, m.M, m.K)
    f = _lib.ColumnFeatures()
    N = 512
    _lib.check(L.mask_features_columns(p.val_soff.data_ptr(), p.val_sidx.data_ptr(), m.M, m.K, p.T, N, C.byref(f),
                                       C.c_void_p(torch.cuda.current_stream().cuda_stream)), "mask_features_columns")
    sidx = p.val_sidx.cpu().numpy().astype(np.int64)
    soff = p.val_soff.cpu().numpy().astype(np.int64)
    assert f.gathers == 8 * p.T == sidx.size
    counts = np.bincount(sidx, minlength=m.K)
    assert f.distinct_columns == int((counts > 0).sum())
    top = np.sort(counts)[::-1].cumsum()
    for i, width in enumerate((512, 256, 128)):
        rows = min(m.K, max(1, (f.l2_bytes // 2) // (min(N, width) * 4)))
        assert f.hub_columns[i] == rows
        assert abs(f.hub_share[i] - top[rows - 1] / sidx.size) < 1e-12
    win = np.repeat(np.arange(soff.size - 1), np.diff(soff))          # window of every tile
    diag = np.repeat(win, 8) * 16 * m.K // m.M
    d = np.abs(sidx - diag)
    bucket = np.where(d == 0, 0, np.floor(np.log2(np.maximum(d, 1))).astype(np.int64) + 1)
    hist = np.bincount(bucket, minlength=33).cumsum()
    for q, got in ((0.5, f.band_p50), (0.9, f.band_p90)):
        b = int(np.searchsorted(hist, q * sidx.size, side="left"))
        assert got == (0 if b == 0 else min(1 << b, m.K))
    assert f.local_rows == min(m.K, max(0, ((f.l2_bytes // 2) // (512 * 4) - 16) // 2))
    assert abs(f.local_share - float((d <= f.local_rows).mean())) < 1e-12


def test_plan_table_tells_a_stencil_from_a_power_law_graph():
    """The plan table is keyed on matrix features: a 27-point stencil keeps its gathers within a narrow
    band (4 slabs per sweep: tile values read once), a large power-law graph does not and gains from
    narrower rows of B (2 slabs).  Both plans must still multiply correctly."""
    import torch
    from mask_b200 import engine, generators as G
    st = G.stencil27(grid=40)
    pl, _ = G.make_workload("rmat20_gcn", scale=19)
    plans = {}
    for name, m in (("stencil", st), ("power_law", pl)):
        rp, ci, va = _dev(m)
        p = engine.pack_srbcrs(rp, ci, va, m.M, m.K)
        plan = p.new_plan("auto")
        f = plan.column_features()
        assert f is not None and f["gathers"] == 8 * p.T
        plans[name] = (f, engine.kernel_signature(p, 512, plan)[0])
        B = torch.randn((m.K, 512), device="cuda")
        out = engine.spmm(p, B, plan=plan)
        ref = torch.sparse.mm(torch.sparse_csr_tensor(rp.long(), ci.long(), va, size=(m.M, m.K)), B)
        assert plan.status() == 0
        assert float((out - ref).abs().max()) <= 2e-2 * float(ref.abs().max())
    fs, ks = plans["stencil"]
    fp, kp = plans["power_law"]
    assert fs["band_p90"] * 16 < fp["band_p90"] and fs["local_share"] >= 0.9 > fp["local_share"]   # local against scattered gathers
    assert fs["nslab_wide"] == 4 and "nslab=4" in ks
    assert fp["nslab_wide"] == 2 and "nslab=2" in kp
    assert fp["hub_share"][1] > fp["hub_share"][0] + 0.02
