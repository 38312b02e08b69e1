"""GPU parity: the SpMM kernels against the host FP32 reference SpMM of the oracle, through the
C ABI.  Tolerance (stated by the task): |C - Cref|_ij <= 2e-3 * (|A|.|B|)_ij + 1e-6."""
import numpy as np
import pytest

from tests import cases

pytestmark = pytest.mark.gpu
RTOL, ATOL = 2e-3, 1e-6


def _dev(m):
    import torch
    return (torch.from_numpy(m.rowptr).cuda(), torch.from_numpy(m.colind).cuda(), torch.from_numpy(m.values).cuda())


def _dense(K, N, seed):
    rng = np.random.Generator(np.random.PCG64(seed))
    return rng.standard_normal((K, N), dtype=np.float32)


def _assert_close(oracle_mod, m, B, got, relu=False):
    ref = oracle_mod.spmm_f32(m.M, m.rowptr, m.colind, m.values, B)
    absp = oracle_mod.spmm_abs_f64(m.M, m.rowptr, m.colind, m.values, B)
    if relu:
        # max(x,0) is 1-Lipschitz, so the same bound holds after the activation
        ref = np.maximum(ref, 0)
    bad, worst = oracle_mod.check_tolerance(got, ref, absp, RTOL, ATOL)
    assert bad == 0, f"{bad} elements outside tolerance, worst ratio {worst}"
    return worst


@pytest.mark.parametrize("name", sorted(cases.SMALL))
@pytest.mark.parametrize("N", [64, 512])
def test_srbcrs_spmm_matches_oracle(oracle_mod, name, N):
    import torch
    from mask_b200 import engine
    m = cases.SMALL[name]()
    rp, ci, va = _dev(m)
    p = engine.pack_srbcrs(rp, ci, va, m.M, m.K)
    B = _dense(m.K, N, 17)
    out = torch.full((m.M, N), float("nan"), device="cuda")  # every element must be overwritten
    engine.spmm(p, torch.from_numpy(B).cuda(), out=out)
    _assert_close(oracle_mod, m, B, out.cpu().numpy())


@pytest.mark.parametrize("N", [4, 16, 36, 100, 128, 160, 256, 320, 1024])
def test_srbcrs_spmm_column_counts(oracle_mod, N):
    import torch
    from mask_b200 import engine
    m = cases.SMALL["three_four_tiles"]()
    rp, ci, va = _dev(m)
    p = engine.pack_srbcrs(rp, ci, va, m.M, m.K)
    B = _dense(m.K, N, N)
    out = torch.full((m.M, N), float("nan"), device="cuda")
    engine.spmm(p, torch.from_numpy(B).cuda(), out=out)
    _assert_close(oracle_mod, m, B, out.cpu().numpy())


@pytest.mark.parametrize("policy,gt", [("auto", 0), ("auto", 2), ("row", 0), ("strict_lb", 0), ("strict_lb", 3),
                                       ("multi_bind", 0), ("ref_auto", 0)])
@pytest.mark.parametrize("name", ["hub_rows", "rmat10", "m33_empty_window", "all_empty", "m17"])
def test_srbcrs_spmm_policies(oracle_mod, name, policy, gt):
    """Every task mapping (including windows split over several blocks and summed from scratch)
    gives the same product; split-window results are deterministic."""
    import torch
    from mask_b200 import engine
    m = cases.SMALL[name]()
    rp, ci, va = _dev(m)
    p = engine.pack_srbcrs(rp, ci, va, m.M, m.K)
    N = 96
    B = _dense(m.K, N, 5)
    Bd = torch.from_numpy(B).cuda()
    plan = engine.Plan(p.val_soff, m.M, p.T, policy, gt)
    out1 = torch.full((m.M, N), float("nan"), device="cuda")
    engine.spmm(p, Bd, out=out1, plan=plan)
    _assert_close(oracle_mod, m, B, out1.cpu().numpy())
    out2 = torch.full((m.M, N), float("nan"), device="cuda")
    engine.spmm(p, Bd, out=out2, plan=plan)
    assert torch.equal(out1, out2)


@pytest.mark.parametrize("use_async,nq,knob", [(0, 1, 0), (0, 2, 0), (0, 2, 4), (0, 4, 0), (0, 4, 3),
                                                (1, 1, 0), (1, 1, 4), (1, 2, 0), (1, 2, 3), (1, 2, 45), (1, 2, 5),
                                                (1, 2, 6), (1, 2, 8), (1, 4, 0), (1, 4, 3), (1, 4, 43), (1, 4, 5),
                                                (1, 4, 6), (1, 4, 8)])
@pytest.mark.parametrize("name,N", [("rmat12u", 512), ("hub_rows", 200), ("m33_empty_window", 64)])
def test_srbcrs_spmm_kernel_variants(oracle_mod, name, N, use_async, nq, knob):
    """Register-pipelined kernel (knob = occupancy target) and shared-memory ring kernel
    (knob = ring slots per warp), every column-slab width."""
    import torch
    from mask_b200 import engine
    m = cases.SMALL[name]()
    rp, ci, va = _dev(m)
    p = engine.pack_srbcrs(rp, ci, va, m.M, m.K)
    B = _dense(m.K, N, 9)
    try:
        engine.tune("sweep", 0)
        engine.tune("async", use_async)
        engine.tune("nq", nq)
        engine.tune("stages" if use_async else "min_blocks", knob)
        out = torch.full((m.M, N), float("nan"), device="cuda")
        engine.spmm(p, torch.from_numpy(B).cuda(), out=out, plan=engine.Plan(p.val_soff, m.M, p.T, "auto", 3))
    finally:
        engine.tune("sweep", 1)
        engine.tune("async", 1)
        engine.tune("nq", 0)
        engine.tune("stages", 0)
        engine.tune("min_blocks", 0)
    _assert_close(oracle_mod, m, B, out.cpu().numpy())


@pytest.mark.parametrize("name", ["m1", "m17", "m33_empty_window", "hub_rows", "rmat10", "stencil8", "all_empty",
                                  "one_tile_windows"])
@pytest.mark.parametrize("N", [32, 128, 256, 512])
def test_metcf_spmm_matches_oracle(oracle_mod, name, N):
    import torch
    from mask_b200 import engine
    m = cases.SMALL[name]()
    rp, ci, va = _dev(m)
    p = engine.pack_metcf(rp, ci, va, m.M, m.K)
    B = _dense(m.K, N, 23)
    out = torch.full((m.M, N), float("nan"), device="cuda")
    engine.spmm(p, torch.from_numpy(B).cuda(), out=out, policy="auto")
    _assert_close(oracle_mod, m, B, out.cpu().numpy())
    # a dense tile with more than 32 entries exercises the long-run path
    plan2 = engine.Plan(p.val_soff, m.M, p.T, "auto", 2)
    out2 = engine.spmm(p, torch.from_numpy(B).cuda(), plan=plan2)
    _assert_close(oracle_mod, m, B, out2.cpu().numpy())
    assert plan2.status() == 0
    try:  # and the mma.sync ME-TCF kernel
        engine.tune("sweep", 0)
        out3 = engine.spmm(p, torch.from_numpy(B).cuda(), plan=plan2)
    finally:
        engine.tune("sweep", 1)
    _assert_close(oracle_mod, m, B, out3.cpu().numpy())


@pytest.mark.parametrize("name", ["m1", "m17", "m33_empty_window", "hub_rows", "rmat10", "stencil8", "all_empty",
                                  "one_tile_windows", "uniform512"])
@pytest.mark.parametrize("N", [40, 128, 256, 512])
def test_mco_spmm_matches_oracle(oracle_mod, name, N):
    """MCO / BIT-TCF (bitmap leaf): tcgen05 kernel in its slab variants, the register-pipelined
    kernel, split windows, ReLU; and exactly the product the oracle
    computes from the same arrays with both operands rounded."""
    import torch
    from mask_b200 import engine
    m = cases.SMALL[name]()
    rp, ci, va = _dev(m)
    p = engine.pack_mco(rp, ci, va, m.M, m.K)
    B = _dense(m.K, N, 29)
    Bd = torch.from_numpy(B).cuda()
    out = torch.full((m.M, N), float("nan"), device="cuda")
    engine.spmm(p, Bd, out=out)
    _assert_close(oracle_mod, m, B, out.cpu().numpy())
    plan2 = engine.Plan(p.val_soff, m.M, p.T, "auto", 2)
    out2 = engine.spmm(p, Bd, plan=plan2, relu=True)
    _assert_close(oracle_mod, m, B, out2.cpu().numpy(), relu=True)
    assert plan2.status() == 0
    outs = []
    try:
        for sweep, nslab in ((0, 0), (2, 1), (2, 2)):   # warp-level kernels; tcgen05 with 1 and 2 slabs
            engine.tune("sweep", sweep)
            engine.tune("nslab", nslab)
            o = torch.full((m.M, N), float("nan"), device="cuda")
            engine.spmm(p, Bd, out=o, plan=plan2)
            outs.append(o)
    finally:
        engine.tune("sweep", 1)
        engine.tune("nslab", 0)
    for o in outs:
        _assert_close(oracle_mod, m, B, o.cpu().numpy())
    assert plan2.status() == 0


def test_relu_epilogue(oracle_mod):
    import torch
    from mask_b200 import engine
    m = cases.SMALL["hub_rows"]()
    rp, ci, va = _dev(m)
    p = engine.pack_srbcrs(rp, ci, va, m.M, m.K)
    B = _dense(m.K, 64, 2)
    for gt in (0, 2):  # direct stores and the split-window fix-up path
        out = engine.spmm(p, torch.from_numpy(B).cuda(), relu=True, plan=engine.Plan(p.val_soff, m.M, p.T, "auto", gt))
        assert float(out.min()) >= 0.0
        _assert_close(oracle_mod, m, B, out.cpu().numpy(), relu=True)


def test_linearity_and_golden_product(oracle_mod):
    """Size-independent properties: A(x+y) = Ax + Ay within tolerance; golden fixtures multiply
    to the oracle product."""
    import torch
    from mask_b200 import engine
    for name in cases.golden_names():
        m, g = cases.load_golden(name)
        rp, ci, va = _dev(m)
        p = engine.pack_srbcrs(rp, ci, va, m.M, m.K)
        B = _dense(m.K, 48, 31)
        out = engine.spmm(p, torch.from_numpy(B).cuda())
        _assert_close(oracle_mod, m, B, out.cpu().numpy())
    m = cases.SMALL["rmat12u"]()
    rp, ci, va = _dev(m)
    p = engine.pack_srbcrs(rp, ci, va, m.M, m.K)
    X, Y = torch.from_numpy(_dense(m.K, 128, 1)).cuda(), torch.from_numpy(_dense(m.K, 128, 2)).cuda()
    lhs = engine.spmm(p, X + Y).cpu().numpy()
    rhs = (engine.spmm(p, X) + engine.spmm(p, Y)).cpu().numpy()
    absp = oracle_mod.spmm_abs_f64(m.M, m.rowptr, m.colind, m.values, (X.abs() + Y.abs()).cpu().numpy())
    bad, worst = oracle_mod.check_tolerance(lhs, rhs, absp, 2 * RTOL, ATOL)
    assert bad == 0, worst


def test_spmm_argument_errors():
    import torch
    from mask_b200 import engine, _lib
    m = cases.SMALL["m17"]()
    rp, ci, va = _dev(m)
    p = engine.pack_srbcrs(rp, ci, va, m.M, m.K)
    with pytest.raises(RuntimeError):
        engine.spmm(p, torch.zeros((m.K + 1, 16), device="cuda"))
    with pytest.raises(RuntimeError):
        engine.spmm(p, torch.zeros((m.K, 16), device="cuda", dtype=torch.float64))
    with pytest.raises(_lib.MaskError):
        engine.spmm(p, torch.zeros((m.K, 18), device="cuda"))  # N % 4 != 0
    assert engine.spmm(p, torch.zeros((m.K, 0), device="cuda")).shape == (m.M, 0)


def test_session_host_buffers(oracle_mod):
    """The host-buffer seam: packed arrays, B and C all on the host."""
    import ctypes as C
    from mask_b200 import _lib
    L = _lib.lib()
    m = cases.SMALL["rmat10"]()
    sr = oracle_mod.pack_srbcrs(m.M, m.rowptr, m.colind, m.values)
    B = _dense(m.K, 64, 3)
    for make in ("packed", "csr"):
        h = C.c_void_p()
        if make == "packed":
            _lib.check(L.mask_session_create_srbcrs(m.M, m.K, sr["T"], sr["val_soff"].ctypes.data, sr["val_sidx"].ctypes.data,
                                                    sr["val_block_val"].ctypes.data, 0, C.byref(h)), "create")
        else:
            _lib.check(L.mask_session_create_csr(m.M, m.K, m.nnz, m.rowptr.ctypes.data, m.colind.ctypes.data,
                                                 m.values.ctypes.data, 0, C.byref(h)), "create")
        assert L.mask_session_tiles(h) == sr["T"]
        out = np.full((m.M, 64), np.nan, dtype=np.float32)
        ms = C.c_float()
        _lib.check(L.mask_session_spmm_host(h, B.ctypes.data, out.ctypes.data, 64, C.byref(ms)), "spmm_host")
        assert ms.value > 0
        _assert_close(oracle_mod, m, B, out)
        # wide products go through the column-chunk pipeline (upload / multiply / download overlapped);
        # with chunking switched off the same call gives the same product
        B2 = _dense(m.K, 512, 5)
        outs = []
        for chunk in (-1, 256, 0):
            _lib.check(L.mask_tune(b"session_chunk", chunk), "tune")
            o = np.full((m.M, 512), np.nan, dtype=np.float32)
            _lib.check(L.mask_session_spmm_host(h, B2.ctypes.data, o.ctypes.data, 512, C.byref(ms)), "spmm_host")
            assert ms.value > 0
            _assert_close(oracle_mod, m, B2, o)
            outs.append(o)
        _lib.check(L.mask_tune(b"session_chunk", -1), "tune")
        L.mask_session_destroy(h)


def test_medium_rmat_against_oracle(oracle_mod):
    """A 2^16-node power-law graph at N=512: thousands of groups, split hub windows."""
    import torch
    from mask_b200 import engine, generators as G
    m, bseed = G.make_workload("rmat20_gcn", scale=16)
    rp, ci, va = _dev(m)
    p = engine.pack_srbcrs(rp, ci, va, m.M, m.K)
    B = G.dense_normal(m.K, 512, bseed)
    out = engine.spmm(p, torch.from_numpy(B).cuda())
    assert p.plan("auto").info()["partial"] > 0
    _assert_close(oracle_mod, m, B, out.cpu().numpy())
    pm = engine.pack_metcf(rp, ci, va, m.M, m.K)
    out2 = engine.spmm(pm, torch.from_numpy(B).cuda())
    _assert_close(oracle_mod, m, B, out2.cpu().numpy())


@pytest.mark.parametrize("fmt", ["srbcrs", "metcf", "mco"])
def test_long_persistent_runs_every_encoding(oracle_mod, fmt):
    """A 2^18-node power-law graph: every resident block walks its rings some two thousand times per
    launch, for the 6-stage ring of SR-BCRS and the 5-stage ring of the compact encodings, at one and
    two slabs per sweep, several launches each.  Hand-over faults that need many ring revolutions to
    show (a waiter that misses a barrier phase) end in a bounded wait giving up, so the plan's status
    word is checked beside the sampled rows."""
    import torch
    from mask_b200 import engine, generators as G
    m, bseed = G.make_workload("rmat20_gcn", scale=18)
    rp, ci, va = _dev(m)
    p = {"srbcrs": engine.pack_srbcrs, "metcf": engine.pack_metcf, "mco": engine.pack_mco}[fmt](rp, ci, va, m.M, m.K)
    rng = np.random.Generator(np.random.PCG64(5))
    rows = np.unique(np.concatenate([rng.integers(0, m.M, size=2048), np.arange(0, 48), np.arange(m.M - 16, m.M)]))
    rows_d = torch.from_numpy(rows).cuda()
    for N in (512, 128):
        B = G.dense_normal(m.K, N, bseed + N)
        Bd = torch.from_numpy(B).cuda()
        ref, absp = oracle_mod.spmm_rows(m.rowptr, m.colind, m.values, B, rows)
        plan = p.new_plan("auto")
        out = torch.empty((m.M, N), device="cuda")
        for _ in range(4):
            out.fill_(float("nan"))
            engine.spmm(p, Bd, out=out, plan=plan)
            assert plan.status() == 0
            bad, worst = oracle_mod.check_tolerance(out[rows_d].cpu().numpy(), ref, absp, RTOL, ATOL)
            assert bad == 0, (N, worst)
        assert not bool(torch.isnan(out[:: 997]).any())


@pytest.mark.parametrize("name,N,gt", [("m1", 512, 0), ("m17", 512, 0), ("m33_empty_window", 512, 0), ("all_empty", 512, 0),
                                       ("hub_rows", 512, 3), ("hub_rows", 1024, 0), ("rmat12u", 512, 0),
                                       ("rmat12u", 512, 200), ("stencil8", 1024, 0), ("three_four_tiles", 512, 1),
                                       ("rmat12u", 128, 0), ("hub_rows", 256, 3), ("rmat10", 384, 0), ("m17", 768, 0),
                                       ("m33_empty_window", 128, 0), ("stencil8", 256, 0),
                                       ("rmat12u", 64, 0), ("hub_rows", 100, 3), ("three_four_tiles", 36, 2),
                                       ("rmat10", 4, 0), ("uniform512", 200, 5), ("one_tile_windows", 520, 0)])
@pytest.mark.parametrize("nslab", [0, 1, 2, 4])
def test_srbcrs_spmm_tcgen05_kernel(oracle_mod, name, N, gt, nslab):
    """The persistent tcgen05 / tensor-memory kernel with 1, 2 or 4 slabs of 128 columns per column
    block (0 = the plan's choice), any N % 4 == 0: same contract, its bounded waits must not have
    expired, and results are deterministic.  Operand B is truncated to TF32 by the tensor core (the
    tile values are rounded), which stays inside the product tolerance.  ME-TCF and MCO go through
    the same kernel family."""
    import torch
    from mask_b200 import engine
    m = cases.SMALL[name]()
    rp, ci, va = _dev(m)
    p = engine.pack_srbcrs(rp, ci, va, m.M, m.K)
    B = _dense(m.K, N, 41)
    Bd = torch.from_numpy(B).cuda()
    plan = engine.Plan(p.val_soff, m.M, p.T, "auto", gt)
    pm = engine.pack_metcf(rp, ci, va, m.M, m.K)
    pc = engine.pack_mco(rp, ci, va, m.M, m.K)
    try:
        engine.tune("sweep", 2)      # also for narrow N, where the library would pick the warp-level kernel
        engine.tune("nslab", nslab)
        out = torch.full((m.M, N), float("nan"), device="cuda")
        engine.spmm(p, Bd, out=out, plan=plan)
        out2 = torch.full((m.M, N), float("nan"), device="cuda")
        engine.spmm(p, Bd, out=out2, plan=plan, relu=True)
        out3 = torch.full((m.M, N), float("nan"), device="cuda")
        engine.spmm(pm, Bd, out=out3, plan=plan)
        out4 = torch.full((m.M, N), float("nan"), device="cuda")
        engine.spmm(pc, Bd, out=out4, plan=plan)
        # the TMA-fed kernel: a plan that holds the rounded tile values
        engine.tune("tma", 1)
        plan_t = p.new_plan("auto", gt, prepare=True)
        assert engine.kernel_signature(p, N, plan_t)[0].startswith("spmm_tma_kernel") or p.T == 0
        out5 = torch.full((m.M, N), float("nan"), device="cuda")
        engine.spmm(p, Bd, out=out5, plan=plan_t)
        out6 = torch.full((m.M, N), float("nan"), device="cuda")
        engine.spmm(p, Bd, out=out6, plan=plan_t, relu=True)
    finally:
        engine.tune("sweep", 1)
        engine.tune("nslab", 0)
        engine.tune("tma", 0)
    assert plan.status() == 0 and plan_t.status() == 0
    _assert_close(oracle_mod, m, B, out5.cpu().numpy())
    assert torch.equal(torch.relu(out5), out6)
    _assert_close(oracle_mod, m, B, out.cpu().numpy())
    _assert_close(oracle_mod, m, B, out3.cpu().numpy())
    _assert_close(oracle_mod, m, B, out4.cpu().numpy())
    assert torch.equal(torch.relu(out), out2)


@pytest.mark.parametrize("name,N,gt,umma,fmt,reorder", [
    ("rmat12u", 64, 0, 1, "srbcrs", "none"),       # narrow N: cp.async ring kernel (warp-level MMA)
    ("hub_rows", 64, 3, 1, "srbcrs", "none"),      # split windows: fix-up kernel writes the rows
    ("rmat12u", 512, 0, 1, "srbcrs", "none"),      # tcgen05 kernel, 4 slabs
    ("hub_rows", 128, 3, 1, "srbcrs", "none"),     # tcgen05 kernel + fix-up
    ("hub_rows", 64, 3, 2, "srbcrs", "none"),      # tcgen05 kernel forced at narrow N
    ("m17", 40, 0, 0, "metcf", "none"),            # register kernel, ragged last window
    ("m17", 40, 0, 1, "metcf", "none"),            # tcgen05 kernel, ME-TCF
    ("rmat10", 64, 0, 1, "srbcrs", "row_rcm"),     # rows scattered back through the row map
    ("rmat10", 256, 0, 1, "srbcrs", "row_rcm"),    # the same through the tcgen05 epilogue
])
def test_peer_outputs_receive_the_same_rows(oracle_mod, name, N, gt, umma, fmt, reorder):
    """mask_plan_set_peer_outputs: every extra output base gets exactly the rows C gets (here the
    'peers' are two more buffers on the same GPU; across GPUs they are peer-mapped addresses)."""
    import torch
    from mask_b200 import engine, _lib
    m = cases.SMALL[name]()
    rp, ci, va = _dev(m)
    if fmt == "metcf":
        p = engine.pack_metcf(rp, ci, va, m.M, m.K)
        plan = engine.Plan(p.val_soff, m.M, p.T, "auto", gt)
    else:
        p = engine.pack_srbcrs(rp, ci, va, m.M, m.K, reorder=reorder)
        plan = p.new_plan("auto", gt)
    B = _dense(m.K, N, 43)
    Bd = torch.from_numpy(B).cuda()
    out = torch.full((m.M, N), float("nan"), device="cuda")
    peers = [torch.full((m.M, N), float("nan"), device="cuda") for _ in range(2)]
    ptrs = torch.tensor([t.data_ptr() for t in peers], dtype=torch.int64, device="cuda")
    try:
        engine.tune("sweep", umma)
        plan.set_peer_outputs(ptrs)
        engine.spmm(p, Bd, out=out, plan=plan, relu=True)
        plan.set_peer_outputs(None)
        plain = torch.full((m.M, N), float("nan"), device="cuda")
        engine.spmm(p, Bd, out=plain, plan=plan, relu=True)
    finally:
        engine.tune("sweep", 1)
    assert plan.status() == 0
    assert torch.equal(out, plain)
    for t in peers:
        assert torch.equal(t, out)
    with pytest.raises(_lib.MaskError):
        plan.set_peer_outputs(torch.zeros(16, dtype=torch.int64, device="cuda"))


@pytest.mark.parametrize("name", ["m17", "m33_empty_window", "hub_rows", "rmat10", "stencil8", "uniform512"])
@pytest.mark.parametrize("N", [64, 200, 512])
def test_tf32x3_compensated_products(oracle_mod, name, N):
    """MASK_NUMERICS_TF32X3: hi*hi plus the two residual products per MMA.  What is left is the
    lo*lo term and the rounding of the residuals (about 2^-21 per product) plus FP32 summation
    order, so the result must sit within 2e-5 * (|A|.|B|) of the host FP32 product -- a hundred
    times tighter than the single-product contract -- also through ReLU and split windows."""
    import torch
    from mask_b200 import engine, _lib
    m = cases.SMALL[name]()
    rp, ci, va = _dev(m)
    p = engine.pack_srbcrs(rp, ci, va, m.M, m.K)
    B = _dense(m.K, N, 31)
    Bd = torch.from_numpy(B).cuda()
    ref = oracle_mod.spmm_f32(m.M, m.rowptr, m.colind, m.values, B)
    absp = oracle_mod.spmm_abs_f64(m.M, m.rowptr, m.colind, m.values, B)
    plan = engine.Plan(p.val_soff, m.M, p.T, "auto", 3)
    for relu in (False, True):
        out = torch.full((m.M, N), float("nan"), device="cuda")
        engine.spmm(p, Bd, out=out, plan=plan, relu=relu, tf32x3=True)
        want = np.maximum(ref, 0) if relu else ref
        bad, worst = oracle_mod.check_tolerance(out.cpu().numpy(), want, absp, 2e-5, 1e-6)
        assert bad == 0, f"{bad} elements outside the compensated tolerance, worst ratio {worst}"
    pm = engine.pack_metcf(rp, ci, va, m.M, m.K)
    with pytest.raises(_lib.MaskError):
        engine.spmm(pm, Bd, tf32x3=True)


@pytest.mark.parametrize("N", [512, 128])
def test_truncated_operand_worst_case(oracle_mod, N):
    """The tcgen05 path hands B to the tensor core as FP32 bits, which drops the low 13 mantissa bits
    (truncation) where the reference rounds to nearest.  Worst case for that: every B value has all
    13 dropped bits set, and A and B are positive so that no error cancels (GCN: normalised
    adjacency times post-ReLU features).  Per product the bound is 2^-10 (B) + 2^-11 (A, rounded) =
    1.46e-3 of |a||b|, inside the 2e-3 contract; measured here, together with the reference
    binaries' own gate 1e-3 + 1e-3 |ref| against an FP32 product."""
    import torch
    from mask_b200 import engine, generators as G
    m, _ = G.make_workload("rmat20_gcn", scale=12)       # positive, GCN-normalised values
    rp, ci, va = _dev(m)
    p = engine.pack_srbcrs(rp, ci, va, m.M, m.K)
    B = np.abs(_dense(m.K, N, 47)) + np.float32(0.25)
    B = (B.view(np.uint32) | np.uint32(0x1FFF)).view(np.float32)
    plan = p.plan("auto")
    out = engine.spmm(p, torch.from_numpy(B).cuda(), plan=plan).cpu().numpy()
    assert plan.status() == 0
    worst = _assert_close(oracle_mod, m, B, out)
    assert worst < 0.80, worst                            # 1.46e-3 / 2e-3 = 0.73 is the analytical ceiling
    ref = oracle_mod.spmm_f32(m.M, m.rowptr, m.colind, m.values, B)
    gate = np.abs(out - ref) / (1e-3 + 1e-3 * np.abs(ref))
    assert float(gate.max()) < 1.0, float(gate.max())     # the reference testbed's cuSPARSE gate


def test_product_with_more_than_2_31_elements(oracle_mod):
    """M * N = 2^31: output offsets need 64 bits.  A thin random matrix with 2^22 rows at N = 512;
    sampled rows from the whole range, including the last windows, against the CPU oracle."""
    import torch
    from mask_b200 import engine, generators as G
    M, K, N, per_row = 1 << 22, 1 << 16, 512, 3
    rng = np.random.Generator(np.random.PCG64(91))
    cols = np.sort(rng.integers(0, K // per_row, size=(M, per_row), dtype=np.int64) * per_row
                   + np.arange(per_row, dtype=np.int64)[None, :], axis=1)      # distinct within a row
    rowptr = (np.arange(M + 1, dtype=np.int64) * per_row).astype(np.int32)
    colind = cols.astype(np.int32).ravel()
    values = rng.uniform(-1, 1, size=colind.size).astype(np.float32)
    m = G.CSR(M, K, rowptr, colind, values)
    rp, ci, va = _dev(m)
    p = engine.pack_srbcrs(rp, ci, va, M, K)
    del rp, ci, va
    B = _dense(K, N, 53)
    Bd = torch.from_numpy(B).cuda()
    out = torch.full((M, N), float("nan"), device="cuda")
    assert out.numel() == 1 << 31
    plan = p.plan("auto")
    engine.spmm(p, Bd, out=out, plan=plan)
    assert plan.status() == 0
    rows = np.unique(np.concatenate([rng.integers(0, M, size=4096), np.arange(M - 64, M), np.arange(0, 32),
                                     np.arange((1 << 21) - 32, (1 << 21) + 32)]))   # around offset 2^30 elements = 2^32 bytes
    ref, absp = oracle_mod.spmm_rows(rowptr, colind, values, B, rows)
    got = out[torch.from_numpy(rows).cuda()].cpu().numpy()
    bad, worst = oracle_mod.check_tolerance(got, ref, absp, RTOL, ATOL)
    assert bad == 0, worst
    assert not bool(torch.isnan(out[-1]).any()) and not bool(torch.isnan(out[:: 1 << 12]).any())
