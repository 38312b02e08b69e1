"""GPU test of the entry point for callers that cannot allocate device memory
(mask_spmm_srbcrs_static_scratch): a server or plug-in host whose device heap is owned by its own
arena has no buffer to offer for the partial tiles of split windows, so the library keeps a fixed
one in its device image.  The result must equal what mask_spmm_srbcrs produces with a
caller-provided buffer, on two calls in a row (the second call finds the first call's leftovers in
the shared array), and oversized requests must be refused.  Collected last on purpose."""
import ctypes as C

import numpy as np
import pytest

from tests import cases

pytestmark = pytest.mark.gpu
RTOL, ATOL = 2e-3, 1e-6  # |C - Cref|_ij <= 2e-3 * (|A|.|B|)_ij + 1e-6


def _call_static(L, plan, p, B, out, relu=False):
    import torch
    return L.mask_spmm_srbcrs_static_scratch(plan._h, p.val_soff.data_ptr(), p.val_sidx.data_ptr(),
                                             p.val_block_val.data_ptr(), p.M, p.K, B.size(1), B.data_ptr(), B.size(1),
                                             out.data_ptr(), out.size(1), 1 if relu else 0,
                                             C.c_void_p(torch.cuda.current_stream().cuda_stream))


@pytest.mark.parametrize("name,N,group_tiles", [("hub_rows", 96, 3), ("rmat12u", 512, 16), ("m33_empty_window", 64, 0)])
def test_static_scratch_matches_caller_scratch(oracle_mod, name, N, group_tiles):
    import torch
    from mask_b200 import _lib, engine
    L = _lib.lib()
    m = cases.SMALL[name]()
    rp, ci, va = (torch.from_numpy(x).cuda() for x in (m.rowptr, m.colind, m.values))
    p = engine.pack_srbcrs(rp, ci, va, m.M, m.K)
    plan = engine.Plan(p.val_soff, m.M, p.T, "auto", group_tiles)
    if group_tiles:
        assert plan.info()["partial"] > 0  # the scratch path is really exercised
    assert plan.scratch_bytes(N) <= L.mask_static_scratch_capacity()
    rng = np.random.Generator(np.random.PCG64(77))
    Bh = rng.standard_normal((m.K, N), dtype=np.float32)
    B = torch.from_numpy(Bh).cuda()
    want = engine.spmm(p, B, plan=plan)  # existing entry point, caller-provided scratch
    ref = oracle_mod.spmm_f32(m.M, m.rowptr, m.colind, m.values, Bh)
    absp = oracle_mod.spmm_abs_f64(m.M, m.rowptr, m.colind, m.values, Bh)
    for call in range(2):  # the second call runs on top of the first call's partial tiles
        out = torch.full((m.M, N), float("nan"), device="cuda")
        _lib.check(_call_static(L, plan, p, B, out), "mask_spmm_srbcrs_static_scratch")
        torch.cuda.synchronize()
        bad, worst = oracle_mod.check_tolerance(out.cpu().numpy(), want.cpu().numpy(), absp, RTOL, ATOL)
        assert bad == 0, (call, worst)
        bad, worst = oracle_mod.check_tolerance(out.cpu().numpy(), ref, absp, RTOL, ATOL)
        assert bad == 0, (call, worst)
    # a different product in between must not disturb a later one (shared array, no stale reads)
    other = torch.full((m.M, N), float("nan"), device="cuda")
    _lib.check(_call_static(L, plan, p, B * 3.0, other, relu=True), "mask_spmm_srbcrs_static_scratch")
    out = torch.full((m.M, N), float("nan"), device="cuda")
    _lib.check(_call_static(L, plan, p, B, out), "mask_spmm_srbcrs_static_scratch")
    bad, worst = oracle_mod.check_tolerance(out.cpu().numpy(), want.cpu().numpy(), absp, RTOL, ATOL)
    assert bad == 0, worst


def _one_wide_window(K):
    """16 rows that together hold K distinct columns: one window of K / 8 tiles."""
    from mask_b200 import generators as G
    per_row = K // 16
    rowptr = (np.arange(17) * per_row).astype(np.int32)
    colind = np.arange(16 * per_row, dtype=np.int32)
    rng = np.random.Generator(np.random.PCG64(3))
    return G.CSR(16, K, rowptr, colind, rng.uniform(-1, 1, size=colind.size).astype(np.float32))


def test_static_scratch_allocates_nothing_and_fills_to_the_brim(oracle_mod):
    """The point of the entry point: a caller whose device heap is spoken for can use it.  After one
    warm-up call (which looks up the array's address) further calls leave the device's free memory
    and torch's allocator exactly as they were.  The plan here needs the whole array: 1024 partial
    tiles at N = 512 is the stated limit, and it must be accepted, not refused."""
    import torch
    from mask_b200 import _lib, engine
    L = _lib.lib()
    N = 512
    m = _one_wide_window(8192)   # 1024 tiles in one window; group_tiles = 1 cuts it into 1024 pieces
    rp, ci, va = (torch.from_numpy(x).cuda() for x in (m.rowptr, m.colind, m.values))
    p = engine.pack_srbcrs(rp, ci, va, m.M, m.K)
    plan = engine.Plan(p.val_soff, m.M, p.T, "auto", 1)
    assert plan.info()["partial"] == 1024 and plan.scratch_bytes(N) == L.mask_static_scratch_capacity()
    rng = np.random.Generator(np.random.PCG64(78))
    Bh = rng.standard_normal((m.K, N), dtype=np.float32)
    B = torch.from_numpy(Bh).cuda()
    out = torch.full((m.M, N), float("nan"), device="cuda")
    _lib.check(_call_static(L, plan, p, B, out), "warm-up call")
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    stats0 = (torch.cuda.memory_allocated(), torch.cuda.memory_reserved(), torch.cuda.memory_stats().get("num_alloc_retries", 0),
              torch.cuda.memory_stats().get("allocation.all.allocated", 0))
    for _ in range(5):
        _lib.check(_call_static(L, plan, p, B, out), "mask_spmm_srbcrs_static_scratch")
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    stats1 = (torch.cuda.memory_allocated(), torch.cuda.memory_reserved(), torch.cuda.memory_stats().get("num_alloc_retries", 0),
              torch.cuda.memory_stats().get("allocation.all.allocated", 0))
    assert free1 == free0, "the driver's free memory changed: something was allocated or freed"
    assert stats1 == stats0, "torch's allocator was used"
    ref = oracle_mod.spmm_f32(m.M, m.rowptr, m.colind, m.values, Bh)
    absp = oracle_mod.spmm_abs_f64(m.M, m.rowptr, m.colind, m.values, Bh)
    bad, worst = oracle_mod.check_tolerance(out.cpu().numpy(), ref, absp, RTOL, ATOL)
    assert bad == 0, worst
    # one more tile than the array holds is refused
    m2 = _one_wide_window(8192 + 16 * 8)
    rp, ci, va = (torch.from_numpy(x).cuda() for x in (m2.rowptr, m2.colind, m2.values))
    p2 = engine.pack_srbcrs(rp, ci, va, m2.M, m2.K)
    plan2 = engine.Plan(p2.val_soff, m2.M, p2.T, "auto", 1)
    assert plan2.info()["partial"] > 1024
    assert _call_static(L, plan2, p2, torch.zeros((m2.K, N), device="cuda"), out) == 4  # MASK_ERR_SCRATCH_TOO_SMALL


def test_static_scratch_refuses_oversized_plans():
    import torch
    from mask_b200 import _lib, engine, generators as G
    L = _lib.lib()
    m, bseed = G.make_workload("rmat20_gcn", scale=14)
    rp, ci, va = (torch.from_numpy(x).cuda() for x in (m.rowptr, m.colind, m.values))
    p = engine.pack_srbcrs(rp, ci, va, m.M, m.K)
    plan = engine.Plan(p.val_soff, m.M, p.T, "strict_lb", 4)  # thousands of windows cut at group boundaries
    N = 512
    assert plan.scratch_bytes(N) > L.mask_static_scratch_capacity()
    B = torch.zeros((m.K, N), device="cuda")
    out = torch.full((m.M, N), 7.0, device="cuda")
    assert _call_static(L, plan, p, B, out) == 4  # MASK_ERR_SCRATCH_TOO_SMALL
    assert b"built-in buffer" in L.mask_last_error()
    torch.cuda.synchronize()
    assert float(out.min()) == 7.0 and float(out.max()) == 7.0  # nothing was launched
