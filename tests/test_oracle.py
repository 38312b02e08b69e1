"""CPU tests: the oracle against the golden fixtures (generated from the reference project's own
packers and planners), against the reference builds when they are present, and its own
consistency (packed formats decode back to the CSR product)."""
import numpy as np
import pytest

from tests import cases

BITS = lambda a: np.ascontiguousarray(a).view(np.int32) if a.dtype == np.float32 else a


@pytest.mark.parametrize("name", cases.golden_names())
def test_oracle_matches_golden(oracle_mod, name):
    m, g = cases.load_golden(name)
    sr = oracle_mod.pack_srbcrs(m.M, m.rowptr, m.colind, m.values)
    for k in ("val_soff", "val_sidx", "val_block_val"):
        assert np.array_equal(BITS(sr[k]), BITS(g["sr_" + k])), (name, k)
    me = oracle_mod.pack_metcf(m.M, m.rowptr, m.colind, m.values)
    for k in ("val_soff", "val_sidx", "val_coo_off", "val_coo_idx", "val_coo_val"):
        assert np.array_equal(BITS(me[k]), BITS(g["me_" + k])), (name, k)
    mc = oracle_mod.pack_mco(m.M, m.rowptr, m.colind, m.values, skip_zero_values=True)
    for k in ("val_soff", "val_sidx", "val_mco_off", "val_mco_mask", "val_mco_val"):
        assert np.array_equal(BITS(mc[k]), BITS(g["mco_" + k])), (name, k)
    for wl in (64, 8):
        rbo, rb2w, go = oracle_mod.strict_lb_plan(m.M, sr["val_soff"], wl)
        assert np.array_equal(rbo, g[f"slb{wl}_row_block_offset"])
        assert np.array_equal(rb2w, g[f"slb{wl}_row_block_to_window"])
        assert np.array_equal(go, g[f"slb{wl}_group_offset"])
    tw, ws, ts = oracle_mod.multi_bind_plan(m.M, sr["val_soff"])
    assert np.array_equal(tw, g["mb_task_window"])
    assert np.array_equal(ws, g["mb_window_split"])
    assert np.array_equal(ts, g["mb_task_soff"])


@pytest.mark.parametrize("name", sorted(cases.SMALL))
def test_oracle_matches_reference_build(oracle_mod, name):
    if not oracle_mod.ref_available():
        pytest.skip("oracle/_ref not built (needs a checkout of the reference project)")
    m = cases.SMALL[name]()
    sr = oracle_mod.pack_srbcrs(m.M, m.rowptr, m.colind, m.values)
    rr = oracle_mod.ref_pack_srbcrs(m.M, m.K, m.rowptr, m.colind, m.values)
    assert sr["T"] == rr["T"]
    for k in ("val_soff", "val_sidx", "val_block_val"):
        assert np.array_equal(BITS(sr[k]), BITS(rr[k])), (name, k)
    me = oracle_mod.pack_metcf(m.M, m.rowptr, m.colind, m.values)
    rm = oracle_mod.ref_pack_metcf(m.M, m.K, m.rowptr, m.colind, m.values)
    assert me["T"] == rm["T"] and me["nnz_pad"] == rm["nnz_pad"]
    for k in ("val_soff", "val_sidx", "val_coo_off", "val_coo_idx", "val_coo_val"):
        assert np.array_equal(BITS(me[k]), BITS(rm[k])), (name, k)
    mc = oracle_mod.pack_mco(m.M, m.rowptr, m.colind, m.values, skip_zero_values=True)
    rc = oracle_mod.ref_pack_mco(m.M, m.K, m.rowptr, m.colind, m.values)
    assert mc["T"] == rc["T"] and mc["nval"] == rc["nval"]
    for k in ("val_soff", "val_sidx", "val_mco_off", "val_mco_mask", "val_mco_val"):
        assert np.array_equal(BITS(mc[k]), BITS(rc[k])), (name, k)
    for wl in (64, 5):
        for a, b in zip(oracle_mod.strict_lb_plan(m.M, sr["val_soff"], wl),
                        oracle_mod.ref_strict_lb_plan(m.M, sr["val_soff"], wl)):
            assert np.array_equal(a, b)
    for a, b in zip(oracle_mod.multi_bind_plan(m.M, sr["val_soff"]), oracle_mod.ref_multi_bind_plan(m.M, sr["val_soff"])):
        assert np.array_equal(a, b)


@pytest.mark.parametrize("name", ["m17", "m33_empty_window", "hub_rows", "rmat10", "stencil8", "all_empty"])
def test_packed_formats_decode_to_csr_product(oracle_mod, name):
    """Both packed formats, evaluated tile by tile without operand rounding, give the CSR product
    up to FP32 summation order."""
    m = cases.SMALL[name]()
    rng = np.random.Generator(np.random.PCG64(3))
    B = rng.standard_normal((m.K, 24), dtype=np.float32)
    ref = oracle_mod.spmm_f32(m.M, m.rowptr, m.colind, m.values, B)
    absp = oracle_mod.spmm_abs_f64(m.M, m.rowptr, m.colind, m.values, B)
    sr = oracle_mod.pack_srbcrs(m.M, m.rowptr, m.colind, m.values)
    me = oracle_mod.pack_metcf(m.M, m.rowptr, m.colind, m.values)
    for got in (oracle_mod.spmm_from_srbcrs(m.M, sr, B, round_tf32=False),
                oracle_mod.spmm_from_metcf(m.M, me, B, round_tf32=False)):
        bad, worst = oracle_mod.check_tolerance(got, ref, absp, rtol=1e-6, atol=1e-7)
        assert bad == 0, worst
    # with TF32 operand rounding the result stays inside the product tolerance
    got = oracle_mod.spmm_from_srbcrs(m.M, sr, B, round_tf32=True)
    bad, worst = oracle_mod.check_tolerance(got, ref, absp)
    assert bad == 0 and worst < 0.6, worst


def test_spmm_matches_numpy(oracle_mod):
    m = cases.SMALL["uniform512"]()
    rng = np.random.Generator(np.random.PCG64(4))
    B = rng.standard_normal((m.K, 16), dtype=np.float32)
    dense = np.zeros((m.M, m.K), dtype=np.float64)
    rows = np.repeat(np.arange(m.M), np.diff(m.rowptr))
    dense[rows, m.colind] = m.values
    want = dense @ B.astype(np.float64)
    got = oracle_mod.spmm_f32(m.M, m.rowptr, m.colind, m.values, B)
    assert np.allclose(got, want, rtol=1e-5, atol=1e-5)
    one = oracle_mod.spmm_f32(m.M, m.rowptr, m.colind, m.values, B, threads=1)
    assert np.array_equal(one, got)  # threading does not change per-row arithmetic
    part = oracle_mod.spmm_f32(m.M, m.rowptr, m.colind, m.values, B, rows=(100, 200))
    assert np.array_equal(part[100:200], got[100:200]) and not part[:100].any()


def test_rna_tf32_and_swizzles(oracle_mod):
    L = oracle_mod.lib()
    assert L.oracle_rna_tf32(1.0) == 1.0
    x = np.float32(1.0 + 2.0 ** -11)  # exactly half way between two TF32 values: ties away
    assert L.oracle_rna_tf32(float(x)) == np.float32(1.0 + 2.0 ** -10)
    assert L.oracle_rna_tf32(float(-x)) == -np.float32(1.0 + 2.0 ** -10)
    assert sorted(L.oracle_sw223(i) for i in range(128)) == list(range(128))
    assert sorted(L.oracle_sw123(i) for i in range(128)) == list(range(128))
    assert L.oracle_sw223(40) == 40 ^ 4 and L.oracle_sw223(127) == 127 ^ 12 and L.oracle_sw123(33) == 33 ^ 4


def test_generators_contract():
    from mask_b200 import generators as G
    for name, kw in (("uniform4096", dict(n=256)), ("rmat20_gcn", dict(scale=9)), ("stencil27_100", dict(grid=6)),
                     ("rmat22_sym", dict(scale=9)), ("rmat21_gcn", dict(scale=9))):
        m, _ = G.make_workload(name, **kw)
        G.check_csr(m)
        m2, _ = G.make_workload(name, **kw)
        assert np.array_equal(m.colind, m2.colind) and np.array_equal(m.values, m2.values)
    s, _ = G.make_workload("rmat22_sym", scale=9)
    d = np.zeros((s.M, s.K), dtype=np.float32)
    d[np.repeat(np.arange(s.M), np.diff(s.rowptr)), s.colind] = s.values
    assert np.array_equal(d, d.T)
    st = G.stencil27(grid=4)
    assert st.nnz == (3 * 4 - 2) ** 3  # sum over the grid of the truncated neighbourhood sizes


@pytest.mark.parametrize("name", cases.golden_names())
def test_reorders_match_golden(oracle_mod, name):
    m, g = cases.load_golden(name)
    for kind in ("first_col_sort", "jaccard_greedy", "row_rcm"):
        if "order_" + kind not in g:
            continue
        assert np.array_equal(oracle_mod.reorder_rows(kind, m.M, m.K, m.rowptr, m.colind), g["order_" + kind]), kind


@pytest.mark.parametrize("name", sorted(cases.SMALL))
def test_reorders_match_reference_build(oracle_mod, name):
    if not oracle_mod.ref_available():
        pytest.skip("oracle/_ref not built (needs a checkout of the reference project)")
    m = cases.SMALL[name]()
    for kind in ("first_col_sort", "jaccard_greedy") + (("row_rcm",) if m.M == m.K else ()):
        a = oracle_mod.reorder_rows(kind, m.M, m.K, m.rowptr, m.colind)
        assert np.array_equal(a, oracle_mod.ref_reorder_rows(kind, m.M, m.K, m.rowptr, m.colind)), kind
        assert sorted(a.tolist()) == list(range(m.M))


def test_matrix_market_writer_round_trip(tmp_path):
    """The pattern file the reference's testbeds and bridge read: 1-based coordinates, row-major."""
    import scipy.io
    from mask_b200 import generators as G
    m = cases.SMALL["m33_empty_window"]()
    path = str(tmp_path / "m.mtx")
    G.write_matrix_market(m, path)
    a = scipy.io.mmread(path).tocsr()
    a.sort_indices()
    assert a.shape == (m.M, m.K) and a.nnz == m.nnz
    assert np.array_equal(a.indptr, m.rowptr) and np.array_equal(a.indices, m.colind)
