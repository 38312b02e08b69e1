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


def _write_checkpoint(L, path, M, packed):
    return L.mask_metcf_checkpoint_write(path.encode(), M, packed["T"], packed["nnz_pad"], packed["val_soff"].ctypes.data,
                                         packed["val_sidx"].ctypes.data, packed["val_coo_off"].ctypes.data,
                                         packed["val_coo_idx"].ctypes.data, packed["val_coo_val"].ctypes.data)


def _read_checkpoint(L, path, M, K):
    T, pad = C.c_int64(), C.c_int64()
    assert L.mask_metcf_checkpoint_header(path.encode(), C.byref(T), C.byref(pad)) == 0
    T, pad = T.value, pad.value
    W = (M + 15) // 16
    out = dict(val_soff=np.zeros(W + 1, np.int32), val_sidx=np.zeros(8 * T, np.int32), val_coo_off=np.zeros(2 * T + 1, np.int32),
               val_coo_idx=np.zeros(pad, np.int32), val_coo_val=np.zeros(pad, np.float32), T=T, nnz_pad=pad)
    rc = L.mask_metcf_checkpoint_read(path.encode(), M, K, T, pad, out["val_soff"].ctypes.data, out["val_sidx"].ctypes.data,
                                      out["val_coo_off"].ctypes.data, out["val_coo_idx"].ctypes.data,
                                      out["val_coo_val"].ctypes.data)
    return rc, out


@pytest.mark.parametrize("path,M,K,sp,want", [
    ("/data/sets/web-Google.mtx", 916428, 916428, 0.0, "web-Google_M916428_K916428_TBK8_RWM16_METCF.checkpoint"),
    ("cage.tar.mtx", 5, 7, 0.5, "cage.tar_M5_K7_TBK8_RWM16_METCF.checkpoint"),
    ("", 100, 200, 0.9995, "synthetic_M100_K200_TBK8_RWM16_sp0p9995_METCF.checkpoint"),
    ("", 100, 200, 0.5, "synthetic_M100_K200_TBK8_RWM16_sp0p5_METCF.checkpoint"),
    ("", 16, 16, 1.0, "synthetic_M16_K16_TBK8_RWM16_sp1_METCF.checkpoint"),
    ("", 16, 16, 0.99999, "synthetic_M16_K16_TBK8_RWM16_sp1_METCF.checkpoint"),
])
def test_metcf_checkpoint_name_follows_the_reference(oracle_mod, path, M, K, sp, want):
    """The cache file must be found by the reference binary too: same name from the same path,
    including the sparsity token it appends for matrices generated in memory."""
    L = _lib.lib()
    buf = C.create_string_buffer(256)
    assert L.mask_metcf_checkpoint_name_for(path.encode(), M, K, sp, buf, 256) == 0
    assert buf.value.decode() == want
    if oracle_mod.ref_available():
        assert oracle_mod.ref_metcf_checkpoint_stem(path, M, K, sp) == want
    assert L.mask_metcf_checkpoint_name_for(path.encode(), M, K, sp, buf, 8) == 1


@pytest.mark.parametrize("name", ["rmat10", "m17", "hub_rows"])
def test_metcf_checkpoint_file(oracle_mod, tmp_path, name):
    """Write / read round trip, validation on load, and byte compatibility with the reference's own
    storeCheckpoint / loadCheckpoint when the reference build is present."""
    L = _lib.lib()
    m = cases.SMALL[name]()
    packed = oracle_mod.pack_metcf(m.M, m.rowptr, m.colind, m.values)
    buf = C.create_string_buffer(256)
    assert L.mask_metcf_checkpoint_name(name.encode(), m.M, m.K, buf, 256) == 0
    fname = buf.value.decode()
    assert fname == f"{name}_M{m.M}_K{m.K}_TBK8_RWM16_METCF.checkpoint"
    mine = str(tmp_path / "mine" / fname)
    os.makedirs(os.path.dirname(mine))
    assert _write_checkpoint(L, mine, m.M, packed) == 0
    rc, back = _read_checkpoint(L, mine, m.M, m.K)
    assert rc == 0
    for k in ("val_soff", "val_sidx", "val_coo_off", "val_coo_idx", "val_coo_val"):
        assert np.array_equal(back[k].view(np.int32), packed[k].view(np.int32)), k
    # a column outside [0, K) or a truncated file is refused
    assert _read_checkpoint(L, mine, m.M, 1)[0] == 6
    with open(mine, "rb") as f:
        blob = f.read()
    short = str(tmp_path / "short.checkpoint")
    with open(short, "wb") as f:
        f.write(blob[:-8])
    T, pad = C.c_int64(), C.c_int64()
    assert L.mask_metcf_checkpoint_header(short.encode(), C.byref(T), C.byref(pad)) == 0
    assert _read_checkpoint(L, short, m.M, m.K)[0] == 1
    if oracle_mod.ref_available():
        ref_dir = str(tmp_path / "ref")
        os.makedirs(ref_dir)
        ref_path, _ = oracle_mod.ref_metcf_checkpoint_roundtrip(ref_dir, name, m.M, m.K, m.rowptr, m.colind, m.values)
        with open(ref_path, "rb") as f:
            assert f.read() == blob                     # same bytes as the reference writes
        loaded = oracle_mod.ref_metcf_load_checkpoint(os.path.dirname(mine), name, m.M, m.K)   # reference reads ours
        for k in ("val_soff", "val_sidx", "val_coo_off", "val_coo_idx", "val_coo_val"):
            assert np.array_equal(loaded[k].view(np.int32), packed[k].view(np.int32)), k


def test_features_and_ref_auto_rule(oracle_mod):
    L = _lib.lib()
    for name in ("rmat12u", "hub_rows", "stencil8", "all_empty", "m1"):
        m = cases.SMALL[name]()
        soff = oracle_mod.pack_srbcrs(m.M, m.rowptr, m.colind, m.values)["val_soff"]
        f = _lib.Features()
        assert L.mask_features_from_soff(soff.ctypes.data, m.M, m.nnz, C.byref(f)) == 0
        lens = np.sort(np.diff(soff))
        W = len(lens)
        rank = lambda q: int(lens[min(W - 1, int(np.ceil(W * q)) - 1)])
        assert (f.row_windows, f.tiles, f.nnz) == (W, int(soff[-1]), m.nnz)
        assert (f.tiles_p50, f.tiles_p95, f.tiles_p99, f.tiles_max) == (rank(0.5), rank(0.95), rank(0.99), int(lens[-1]))
        assert f.empty_windows == int((lens == 0).sum())
        assert abs(f.tiles_mean - (soff[-1] / W)) < 1e-12
        assert f.heavy_tail == int(lens[-1] > max(64, 4 * max(rank(0.95), 1)))
        if soff[-1]:
            assert abs(f.tile_fill - m.nnz / (128.0 * soff[-1])) < 1e-12
            assert abs(f.top5_window_share - lens[-5:].sum() / soff[-1]) < 1e-12
