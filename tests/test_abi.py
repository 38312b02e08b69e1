"""CPU tests of the C ABI: the library loads, exports every symbol the header declares, and its
host-only entry points (task planners, argument validation) behave; no GPU work is issued."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from mask_b200 import _lib
from tests import cases

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    text = open(os.path.join(ROOT, "include", "mask_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mask_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    L = C.CDLL(_lib.LIB_PATH)
    names = header_functions()
    assert len(names) >= 20
    for n in names:
        assert hasattr(L, n), f"{n} is declared in include/mask_b200.h but not exported"
    assert set(names) == set(_lib.SIGNATURES), set(names) ^ set(_lib.SIGNATURES)


def test_version_and_status_strings():
    L = _lib.lib()
    assert L.mask_version() >= 100
    assert L.mask_status_string(0) == b"ok"
    assert b"ascending" in L.mask_status_string(3)


def _planner_strict(L, soff, M, wl):
    nf, ng = C.c_int64(), C.c_int64()
    assert L.mask_plan_strict_lb(soff.ctypes.data, M, wl, None, None, None, C.byref(nf), C.byref(ng)) == 0
    rbo = np.zeros(nf.value + 1, np.int32)
    rb2w = np.zeros(max(nf.value, 1), np.int32)
    go = np.zeros(ng.value + 1, np.int32)
    assert L.mask_plan_strict_lb(soff.ctypes.data, M, wl, rbo.ctypes.data, rb2w.ctypes.data, go.ctypes.data,
                                 C.byref(nf), C.byref(ng)) == 0
    return rbo, rb2w[:nf.value], go


def _planner_multi(L, soff, M):
    W = (M + 15) // 16
    nt = C.c_int64()
    assert L.mask_plan_multi_bind(soff.ctypes.data, M, None, None, None, C.byref(nt)) == 0
    tw = np.zeros(max(nt.value, 1), np.int32)
    ws = np.zeros(max(W, 1), np.int32)
    ts = np.zeros(nt.value + 1, np.int32)
    assert L.mask_plan_multi_bind(soff.ctypes.data, M, tw.ctypes.data, ws.ctypes.data, ts.ctypes.data, C.byref(nt)) == 0
    return tw[:nt.value], ws[:W], ts


@pytest.mark.parametrize("name", cases.golden_names())
def test_host_planners_match_golden(name):
    L = _lib.lib()
    m, g = cases.load_golden(name)
    soff = np.ascontiguousarray(g["sr_val_soff"])
    for wl in (64, 8):
        rbo, rb2w, go = _planner_strict(L, soff, m.M, wl)
        assert np.array_equal(rbo, g[f"slb{wl}_row_block_offset"])
        assert np.array_equal(rb2w, g[f"slb{wl}_row_block_to_window"])
        assert np.array_equal(go, g[f"slb{wl}_group_offset"])
    tw, ws, ts = _planner_multi(L, soff, m.M)
    assert np.array_equal(tw, g["mb_task_window"])
    assert np.array_equal(ws, g["mb_window_split"])
    assert np.array_equal(ts, g["mb_task_soff"])


@pytest.mark.parametrize("name", sorted(cases.SMALL))
def test_host_planners_match_oracle(oracle_mod, name):
    L = _lib.lib()
    m = cases.SMALL[name]()
    soff = oracle_mod.pack_srbcrs(m.M, m.rowptr, m.colind, m.values)["val_soff"]
    for wl in (64, 3):
        for a, b in zip(_planner_strict(L, soff, m.M, wl), oracle_mod.strict_lb_plan(m.M, soff, wl)):
            assert np.array_equal(a, b)
    for a, b in zip(_planner_multi(L, soff, m.M), oracle_mod.multi_bind_plan(m.M, soff)):
        assert np.array_equal(a, b)


def test_invalid_arguments_are_reported_not_raised():
    L = _lib.lib()
    nf, ng = C.c_int64(), C.c_int64()
    assert L.mask_plan_strict_lb(None, 16, 64, None, None, None, C.byref(nf), C.byref(ng)) == 1
    assert L.mask_last_error() != b""
    assert L.mask_pack_scratch_bytes(0, 10) == 0
    assert L.mask_pack_scratch_bytes(1000, 10000) >= 4 * 4 * 10000
    T = C.c_int64()
    assert L.mask_pack_analyze(None, None, 16, 16, 0, None, 0, None, C.byref(T), None) == 1
    assert L.mask_spmm_srbcrs(None, None, None, None, 16, 16, 64, None, 64, None, 64, None, 0, 0, None) == 1
    assert L.mask_tune(b"no_such_knob", 1) == 1
    assert L.mask_plan_scratch_bytes(None, 64) == 0
    h = C.c_void_p()
    assert L.mask_session_create_srbcrs(0, 4, 0, None, None, None, 0, C.byref(h)) == 1 and not h.value
    with pytest.raises(_lib.MaskError):
        _lib.check(1, "demo")


@pytest.mark.parametrize("name", cases.golden_names() + ["rmat10", "hub_rows", "stencil8", "all_empty"])
def test_host_reorders_match_golden_and_oracle(oracle_mod, name):
    """mask_reorder_rows against the fixtures made by the reference bridge and against the oracle."""
    L = _lib.lib()
    if name in cases.SMALL:
        m, g = cases.SMALL[name](), {}
    else:
        m, g = cases.load_golden(name)
    for kind in ("first_col_sort", "jaccard_greedy", "row_rcm"):
        order = np.zeros(m.M, np.int32)
        rc = L.mask_reorder_rows(_lib.REORDER[kind], m.rowptr.ctypes.data, m.colind.ctypes.data, m.M, m.K, order.ctypes.data)
        if kind == "row_rcm" and m.M != m.K:
            assert rc == 1
            continue
        assert rc == 0
        assert np.array_equal(order, oracle_mod.reorder_rows(kind, m.M, m.K, m.rowptr, m.colind)), kind
        if "order_" + kind in g:
            assert np.array_equal(order, g["order_" + kind]), kind
    ident = np.zeros(m.M, np.int32)
    assert L.mask_reorder_rows(0, m.rowptr.ctypes.data, m.colind.ctypes.data, m.M, m.K, ident.ctypes.data) == 0
    assert np.array_equal(ident, np.arange(m.M))
    assert L.mask_reorder_rows(9, m.rowptr.ctypes.data, m.colind.ctypes.data, m.M, m.K, ident.ctypes.data) == 1
