"""CPU oracle for the SR-BCRS 16x8 / ME-TCF SpMM path -- TEST INFRASTRUCTURE ONLY.

ctypes front end of ``liboracle.so`` (built from ``oracle.c`` by ``oracle/Makefile``) and, when
present, of the reference project's own host packers built into ``oracle/_ref``.  Only the
test-suite, the smoke check and the CPU-baseline / reference legs of the benchmark import this
package; the product library never does.  Parity status: pinned against the reference builds
(see the header of ``oracle.c``).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

_i32p = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")
_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_f64p = np.ctypeslib.ndpointer(dtype=np.float64, flags="C_CONTIGUOUS")


def build(ref: bool = True) -> None:
    """Compiles liboracle.so (and oracle/_ref/*.so when the reference checkout is present)."""
    target = "all" if ref else "oracle"
    subprocess.run(["make", "-C", _HERE, target, "-j4"], check=True, stdout=subprocess.DEVNULL)


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            build(ref=False)
        L = C.CDLL(path)
        L.oracle_srbcrs_count.restype = C.c_int64
        L.oracle_srbcrs_count.argtypes = [C.c_int, _i32p, _i32p, _i32p]
        L.oracle_srbcrs_fill.restype = None
        L.oracle_srbcrs_fill.argtypes = [C.c_int, _i32p, _i32p, _f32p, _i32p, _i32p, _f32p]
        L.oracle_edge_maps.restype = None
        L.oracle_edge_maps.argtypes = [C.c_int, _i32p, _i32p, _i32p, _i32p, _i32p]
        L.oracle_metcf_count.restype = C.c_int64
        L.oracle_metcf_count.argtypes = [C.c_int, _i32p, _i32p, _i32p, C.POINTER(C.c_int64)]
        L.oracle_metcf_fill.restype = None
        L.oracle_metcf_fill.argtypes = [C.c_int, _i32p, _i32p, _f32p, _i32p, _i32p, _i32p, _i32p, _f32p, C.c_int64]
        L.oracle_strict_lb_plan.restype = C.c_int64
        L.oracle_strict_lb_plan.argtypes = [C.c_int, _i32p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                                            C.POINTER(C.c_int64)]
        L.oracle_multi_bind_plan.restype = C.c_int64
        L.oracle_multi_bind_plan.argtypes = [C.c_int, _i32p, C.c_void_p, C.c_void_p, C.c_void_p]
        L.oracle_spmm_f32.restype = None
        L.oracle_spmm_f32.argtypes = [C.c_int, C.c_int, C.c_int, _i32p, _i32p, _f32p, _f32p, C.c_int64, _f32p,
                                      C.c_int64, C.c_int]
        L.oracle_spmm_abs_f64.restype = None
        L.oracle_spmm_abs_f64.argtypes = [C.c_int, C.c_int, C.c_int, _i32p, _i32p, _f32p, _f32p, C.c_int64,
                                          _f64p, C.c_int64, C.c_int]
        L.oracle_spmm_from_srbcrs.restype = None
        L.oracle_spmm_from_srbcrs.argtypes = [C.c_int, C.c_int, _i32p, _i32p, _f32p, _f32p, C.c_int64, _f32p,
                                              C.c_int64, C.c_int]
        L.oracle_spmm_from_metcf.restype = None
        L.oracle_spmm_from_metcf.argtypes = [C.c_int, C.c_int, _i32p, _i32p, _i32p, _i32p, _f32p, _f32p,
                                             C.c_int64, _f32p, C.c_int64, C.c_int]
        L.oracle_check_tolerance.restype = C.c_int64
        L.oracle_check_tolerance.argtypes = [C.c_int64, C.c_int, _f32p, C.c_int64, _f32p, C.c_int64, _f64p,
                                             C.c_int64, C.c_double, C.c_double, C.POINTER(C.c_double)]
        L.oracle_reorder_first_col.restype = None
        L.oracle_reorder_first_col.argtypes = [C.c_int, C.c_int, _i32p, _i32p, _i32p]
        L.oracle_reorder_rcm.restype = C.c_int
        L.oracle_reorder_rcm.argtypes = [C.c_int, C.c_int, _i32p, _i32p, _i32p]
        L.oracle_reorder_jaccard.restype = None
        L.oracle_reorder_jaccard.argtypes = [C.c_int, C.c_int, _i32p, _i32p, _i32p]
        L.oracle_permute_csr.restype = None
        L.oracle_permute_csr.argtypes = [C.c_int, _i32p, _i32p, _f32p, _i32p, _i32p, _i32p, _f32p]
        L.oracle_max_threads.restype = C.c_int
        L.oracle_rna_tf32.restype = C.c_float
        L.oracle_rna_tf32.argtypes = [C.c_float]
        L.oracle_sw223.restype = C.c_int
        L.oracle_sw223.argtypes = [C.c_int]
        L.oracle_sw123.restype = C.c_int
        L.oracle_sw123.argtypes = [C.c_int]
        _LIB = L
    return _LIB


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


def pack_srbcrs(M, rowptr, colind, values):
    """-> dict(val_soff int32[W+1], val_sidx int32[8T], val_block_val f32[128T], T)."""
    L = lib()
    rowptr, colind, values = _c(rowptr, np.int32), _c(colind, np.int32), _c(values, np.float32)
    W = (M + 15) // 16
    soff = np.zeros(W + 1, dtype=np.int32)
    T = int(L.oracle_srbcrs_count(M, rowptr, colind, soff))
    sidx = np.zeros(8 * T, dtype=np.int32)
    blk = np.zeros(128 * T, dtype=np.float32)
    L.oracle_srbcrs_fill(M, rowptr, colind, values, soff, sidx, blk)
    return dict(val_soff=soff, val_sidx=sidx, val_block_val=blk, T=T)


def edge_maps(M, rowptr, colind):
    """-> (block_partition int32[W], edge_to_col int32[nnz], edge_to_row int32[nnz])."""
    L = lib()
    rowptr, colind = _c(rowptr, np.int32), _c(colind, np.int32)
    W = (M + 15) // 16
    bp = np.zeros(W, dtype=np.int32)
    e2c = np.zeros(colind.shape[0], dtype=np.int32)
    e2r = np.zeros(colind.shape[0], dtype=np.int32)
    L.oracle_edge_maps(M, rowptr, colind, bp, e2c, e2r)
    return bp, e2c, e2r


def pack_metcf(M, rowptr, colind, values):
    """-> dict(val_soff, val_sidx, val_coo_off int32[2T+1], val_coo_idx int32[nnz_pad],
    val_coo_val f32[nnz_pad], T, nnz_pad)."""
    L = lib()
    rowptr, colind, values = _c(rowptr, np.int32), _c(colind, np.int32), _c(values, np.float32)
    W = (M + 15) // 16
    soff = np.zeros(W + 1, dtype=np.int32)
    pad = C.c_int64(0)
    T = int(L.oracle_metcf_count(M, rowptr, colind, soff, C.byref(pad)))
    pad = int(pad.value)
    sidx = np.zeros(8 * T, dtype=np.int32)
    off = np.zeros(2 * T + 1, dtype=np.int32)
    idx = np.zeros(pad, dtype=np.int32)
    val = np.zeros(pad, dtype=np.float32)
    L.oracle_metcf_fill(M, rowptr, colind, values, soff, sidx, off, idx, val, pad)
    return dict(val_soff=soff, val_sidx=sidx, val_coo_off=off, val_coo_idx=idx, val_coo_val=val, T=T,
                nnz_pad=pad)


def pack_mco(M, rowptr, colind, values, skip_zero_values=False):
    """-> dict(val_soff, val_sidx, val_mco_off int32[T+1], val_mco_mask uint64[2T], val_mco_val f32[nval], T, nval)."""
    L = lib()
    rowptr, colind, values = _c(rowptr, np.int32), _c(colind, np.int32), _c(values, np.float32)
    W = (M + 15) // 16
    soff = np.zeros(W + 1, dtype=np.int32)
    T = int(L.oracle_srbcrs_count(M, rowptr, colind, soff))
    sidx = np.zeros(8 * T, dtype=np.int32)
    off = np.zeros(T + 1, dtype=np.int32)
    mask = np.zeros(2 * T, dtype=np.uint64)
    val = np.zeros(len(values) + 3 * T + 4, dtype=np.float32)
    L.oracle_mco_pack.restype = C.c_int64
    L.oracle_mco_pack.argtypes = [C.c_int] + [C.c_void_p] * 3 + [C.c_int] + [C.c_void_p] * 5
    nval = int(L.oracle_mco_pack(M, rowptr.ctypes.data, colind.ctypes.data, values.ctypes.data, int(skip_zero_values),
                                 soff.ctypes.data, sidx.ctypes.data, off.ctypes.data, mask.ctypes.data, val.ctypes.data))
    return dict(val_soff=soff, val_sidx=sidx, val_mco_off=off, val_mco_mask=mask, val_mco_val=val[:nval].copy(), T=T, nval=nval)


def spmm_from_mco(M, packed, B, round_tf32=False):
    L = lib()
    B = _c(B, np.float32)
    N = B.shape[1]
    out = np.empty((M, N), dtype=np.float32)
    L.oracle_spmm_from_mco.restype = None
    L.oracle_spmm_from_mco.argtypes = [C.c_int, C.c_int] + [C.c_void_p] * 6 + [C.c_int64, C.c_void_p, C.c_int64, C.c_int]
    a = {k: np.ascontiguousarray(packed[k]) for k in ("val_soff", "val_sidx", "val_mco_off", "val_mco_mask", "val_mco_val")}
    L.oracle_spmm_from_mco(M, N, a["val_soff"].ctypes.data, a["val_sidx"].ctypes.data, a["val_mco_off"].ctypes.data,
                           a["val_mco_mask"].ctypes.data, a["val_mco_val"].ctypes.data, B.ctypes.data, N, out.ctypes.data, N,
                           int(round_tf32))
    return out


def strict_lb_plan(M, val_soff, workload=64):
    """-> (row_block_offset int32[F+1], row_block_to_window int32[F], group_offset int32[G+1])."""
    L = lib()
    val_soff = _c(val_soff, np.int32)
    ng = C.c_int64(0)
    F = int(L.oracle_strict_lb_plan(M, val_soff, workload, None, None, None, C.byref(ng)))
    G = int(ng.value)
    rbo = np.zeros(F + 1, dtype=np.int32)
    rb2w = np.zeros(max(F, 1), dtype=np.int32)
    go = np.zeros(G + 1, dtype=np.int32)
    L.oracle_strict_lb_plan(M, val_soff, workload, rbo.ctypes.data, rb2w.ctypes.data, go.ctypes.data,
                            C.byref(ng))
    return rbo, rb2w[:F], go


def multi_bind_plan(M, val_soff):
    """-> (task_window int32[P], window_split int32[W], task_soff int32[P+1])."""
    L = lib()
    val_soff = _c(val_soff, np.int32)
    W = (M + 15) // 16
    P = int(L.oracle_multi_bind_plan(M, val_soff, None, None, None))
    tw = np.zeros(max(P, 1), dtype=np.int32)
    ws = np.zeros(max(W, 1), dtype=np.int32)
    ts = np.zeros(P + 1, dtype=np.int32)
    L.oracle_multi_bind_plan(M, val_soff, tw.ctypes.data, ws.ctypes.data, ts.ctypes.data)
    return tw[:P], ws[:W], ts


REORDER_KINDS = {"row_rcm": 1, "first_col_sort": 2, "jaccard_greedy": 3}


def reorder_rows(kind, M, K, rowptr, colind):
    """row_order[new_row] = original_row for one of the bridge's three reorders."""
    L = lib()
    rowptr, colind = _c(rowptr, np.int32), _c(colind, np.int32)
    order = np.zeros(M, dtype=np.int32)
    if kind == "first_col_sort":
        L.oracle_reorder_first_col(M, K, rowptr, colind, order)
    elif kind == "row_rcm":
        if L.oracle_reorder_rcm(M, K, rowptr, colind, order) != 0:
            raise ValueError("row_rcm needs a square matrix")
    elif kind == "jaccard_greedy":
        L.oracle_reorder_jaccard(M, K, rowptr, colind, order)
    else:
        raise ValueError(kind)
    return order


def permute_csr(M, rowptr, colind, values, order):
    L = lib()
    rowptr, colind, values = _c(rowptr, np.int32), _c(colind, np.int32), _c(values, np.float32)
    rp = np.zeros(M + 1, dtype=np.int32)
    ci = np.zeros_like(colind)
    va = np.zeros_like(values)
    L.oracle_permute_csr(M, rowptr, colind, values, _c(order, np.int32), rp, ci, va)
    return rp, ci, va


def ref_reorder_rows(kind, M, K, rowptr, colind):
    R = _ref("libref_bridge.so")
    R.ref_reorder_rows.restype = C.c_int
    R.ref_reorder_rows.argtypes = [C.c_int, C.c_int, C.c_int, _i32p, _i32p, _i32p]
    order = np.zeros(M, dtype=np.int32)
    rc = R.ref_reorder_rows(REORDER_KINDS[kind], M, K, _c(rowptr, np.int32), _c(colind, np.int32), order)
    if rc != 0:
        raise ValueError(f"reference reorder failed ({rc})")
    return order


def ref_pack_mco(M, K, rowptr, colind, values):
    """The Format-DSL bridge's own packer in its bitmap ("column_condensed") mode, built from the
    reference sources: dict like pack_mco(skip_zero_values=True); the bridge pads the value array
    to a multiple of 8 at the very end, which is cut off here."""
    R = _ref("libref_bridge_mco.so")
    R.ref_bridge_pack.restype = C.c_int
    R.ref_bridge_pack.argtypes = [C.c_int, C.c_int] + [C.c_void_p] * 10
    rowptr, colind, values = _c(rowptr, np.int32), _c(colind, np.int32), _c(values, np.float32)
    tiles, nv = C.c_int(0), C.c_longlong(0)
    args = (M, K, rowptr.ctypes.data, colind.ctypes.data, values.ctypes.data, C.addressof(tiles), C.addressof(nv))
    if R.ref_bridge_pack(*args, None, None, None, None, None) != 0:
        raise ValueError("reference bridge packer failed")
    T, n = tiles.value, nv.value
    W = (M + 15) // 16
    soff = np.zeros(W + 1, dtype=np.int32)
    sidx = np.zeros(8 * T, dtype=np.int32)
    off = np.zeros(T + 1, dtype=np.int32)
    mask = np.zeros(2 * T, dtype=np.uint64)
    val = np.zeros(max(n, 1), dtype=np.float32)
    if R.ref_bridge_pack(*args, soff.ctypes.data, sidx.ctypes.data, off.ctypes.data, mask.ctypes.data, val.ctypes.data) != 0:
        raise ValueError("reference bridge packer failed")
    nval = int(off[T])
    return dict(val_soff=soff, val_sidx=sidx, val_mco_off=off, val_mco_mask=mask, val_mco_val=val[:nval].copy(), T=T, nval=nval)


def max_threads() -> int:
    return int(lib().oracle_max_threads())


def spmm_f32(M, rowptr, colind, values, B, threads=None, rows=None):
    """Host FP32 reference SpMM (the reference project's cpu_spmm loops).  ``rows=(r0, r1)``
    restricts the computation to a row range (other rows of the result stay zero)."""
    L = lib()
    B = _c(B, np.float32)
    N = B.shape[1]
    Cm = np.zeros((M, N), dtype=np.float32)
    r0, r1 = rows if rows is not None else (0, M)
    L.oracle_spmm_f32(r0, r1, N, _c(rowptr, np.int32), _c(colind, np.int32), _c(values, np.float32), B, N, Cm, N,
                      threads or max_threads())
    return Cm


def spmm_abs_f64(M, rowptr, colind, values, B, rows=None):
    """(|A|.|B|) in FP64 -- the denominator of the tolerance."""
    L = lib()
    B = _c(B, np.float32)
    N = B.shape[1]
    Cm = np.zeros((M, N), dtype=np.float64)
    r0, r1 = rows if rows is not None else (0, M)
    L.oracle_spmm_abs_f64(r0, r1, N, _c(rowptr, np.int32), _c(colind, np.int32), _c(values, np.float32), B, N,
                          Cm, N, max_threads())
    return Cm


def spmm_rows(rowptr, colind, values, B, rows):
    """Reference product and |A|.|B| restricted to a list of rows: (C[rows], (|A|.|B|)[rows])."""
    rows = np.asarray(rows, dtype=np.int64)
    rp = np.asarray(rowptr).astype(np.int64)
    lens = rp[rows + 1] - rp[rows]
    ptr = np.zeros(rows.size + 1, dtype=np.int64)
    np.cumsum(lens, out=ptr[1:])
    idx = np.repeat(rp[rows] - ptr[:-1], lens) + np.arange(int(ptr[-1]), dtype=np.int64)
    cols, vals = np.ascontiguousarray(colind[idx]), np.ascontiguousarray(values[idx])
    ptr32 = ptr.astype(np.int32)
    return spmm_f32(rows.size, ptr32, cols, vals, B), spmm_abs_f64(rows.size, ptr32, cols, vals, B)


def spmm_from_srbcrs(M, packed, B, round_tf32=True):
    L = lib()
    B = _c(B, np.float32)
    N = B.shape[1]
    Cm = np.zeros((M, N), dtype=np.float32)
    L.oracle_spmm_from_srbcrs(M, N, packed["val_soff"], packed["val_sidx"], packed["val_block_val"], B, N, Cm, N,
                              int(round_tf32))
    return Cm


def spmm_from_metcf(M, packed, B, round_tf32=True):
    L = lib()
    B = _c(B, np.float32)
    N = B.shape[1]
    Cm = np.zeros((M, N), dtype=np.float32)
    L.oracle_spmm_from_metcf(M, N, packed["val_soff"], packed["val_sidx"], packed["val_coo_off"],
                             packed["val_coo_idx"], packed["val_coo_val"], B, N, Cm, N, int(round_tf32))
    return Cm


RTOL, ATOL = 2e-3, 1e-6  # |C - Cref|_ij <= 2e-3 * (|A|.|B|)_ij + 1e-6


def check_tolerance(got, ref, absprod, rtol=RTOL, atol=ATOL):
    """-> (number of violating elements, worst |got-ref| / (rtol*absprod + atol))."""
    L = lib()
    got, ref, absprod = _c(got, np.float32), _c(ref, np.float32), _c(absprod, np.float64)
    assert got.shape == ref.shape == absprod.shape and got.ndim == 2
    worst = C.c_double(0.0)
    bad = int(L.oracle_check_tolerance(got.shape[0], got.shape[1], got, got.shape[1], ref, ref.shape[1], absprod,
                                       absprod.shape[1], rtol, atol, C.byref(worst)))
    return bad, float(worst.value)


# ---- the reference project's own host code (oracle/_ref, built from the reference sources) ----

def ref_available() -> bool:
    return all(os.path.exists(os.path.join(_HERE, "_ref", n)) for n in
               ("libref_srbcrs.so", "libref_strict_lb.so", "libref_multi_bind.so", "libref_metcf.so",
                "libref_bridge.so", "libref_bridge_mco.so"))


def _ref(name):
    return C.CDLL(os.path.join(_HERE, "_ref", name))


def ref_pack_srbcrs(M, K, rowptr, colind, values):
    R = _ref("libref_srbcrs.so")
    rowptr, colind, values = _c(rowptr, np.int32).copy(), _c(colind, np.int32).copy(), _c(values, np.float32).copy()
    R.ref_srbcrs_pack.restype = C.c_int
    R.ref_srbcrs_pack.argtypes = [C.c_int, C.c_int, C.c_int, _i32p, _i32p, _f32p]
    T = int(R.ref_srbcrs_pack(M, K, colind.shape[0], rowptr, colind, values))
    W = (M + 15) // 16
    soff = np.zeros(W + 1, dtype=np.int32)
    sidx = np.zeros(8 * T, dtype=np.int32)
    blk = np.zeros(128 * T, dtype=np.float32)
    R.ref_srbcrs_fetch.restype = None
    R.ref_srbcrs_fetch.argtypes = [_i32p, _i32p, _f32p]
    R.ref_srbcrs_fetch(soff, sidx, blk)
    return dict(val_soff=soff, val_sidx=sidx, val_block_val=blk, T=T)


def ref_pack_metcf(M, K, rowptr, colind, values):
    R = _ref("libref_metcf.so")
    rowptr, colind, values = _c(rowptr, np.int32), _c(colind, np.int32), _c(values, np.float32)
    R.ref_metcf_pack.restype = C.c_int
    R.ref_metcf_pack.argtypes = [C.c_int, C.c_int, _i32p, _i32p, _f32p, C.POINTER(C.c_int)]
    pad = C.c_int(0)
    T = int(R.ref_metcf_pack(M, K, rowptr, colind, values, C.byref(pad)))
    pad = int(pad.value)
    W = (M + 15) // 16
    soff = np.zeros(W + 1, dtype=np.int32)
    sidx = np.zeros(8 * T, dtype=np.int32)
    off = np.zeros(2 * T + 1, dtype=np.int32)
    idx = np.zeros(pad, dtype=np.int32)
    val = np.zeros(pad, dtype=np.float32)
    R.ref_metcf_fetch.restype = None
    R.ref_metcf_fetch.argtypes = [_i32p, _i32p, _i32p, _i32p, _f32p]
    R.ref_metcf_fetch(soff, sidx, off, idx, val)
    return dict(val_soff=soff, val_sidx=sidx, val_coo_off=off, val_coo_idx=idx, val_coo_val=val, T=T,
                nnz_pad=pad)


def ref_metcf_checkpoint_roundtrip(cache_dir, matrix_name, M, K, rowptr, colind, values):
    """Packs with the reference, writes its checkpoint into cache_dir with the reference's own
    storeCheckpoint and returns the file path."""
    R = _ref("libref_metcf.so")
    os.environ["SPARSENE_MTX_CACHE_DIR"] = cache_dir
    os.environ.pop("SPARSENE_DISABLE_MTX_CACHE", None)
    packed = ref_pack_metcf(M, K, rowptr, colind, values)
    R.ref_metcf_store_checkpoint.restype = C.c_int
    R.ref_metcf_store_checkpoint.argtypes = [C.c_char_p, C.c_int, C.c_int]
    fake_path = f"/data/{matrix_name}.mtx".encode()
    if R.ref_metcf_store_checkpoint(fake_path, M, K) != 1:
        raise RuntimeError("reference storeCheckpoint failed")
    return os.path.join(cache_dir, f"{matrix_name}_M{M}_K{K}_TBK8_RWM16_METCF.checkpoint"), packed


def ref_metcf_checkpoint_stem(file_path: str, M: int, K: int, sparsity: float) -> str:
    """The reference's own buildCheckpointStem."""
    R = _ref("libref_metcf.so")
    R.ref_metcf_checkpoint_stem.restype = C.c_int
    R.ref_metcf_checkpoint_stem.argtypes = [C.c_char_p, C.c_int, C.c_int, C.c_float, C.c_char_p, C.c_int]
    buf = C.create_string_buffer(512)
    if R.ref_metcf_checkpoint_stem(file_path.encode(), M, K, sparsity, buf, 512) != 1:
        raise RuntimeError("name too long")
    return buf.value.decode()


def ref_metcf_load_checkpoint(cache_dir, matrix_name, M, K):
    """Loads <cache_dir>/<name>_..._METCF.checkpoint with the reference's own loadCheckpoint."""
    R = _ref("libref_metcf.so")
    os.environ["SPARSENE_MTX_CACHE_DIR"] = cache_dir
    R.ref_metcf_load_checkpoint.restype = C.c_int
    R.ref_metcf_load_checkpoint.argtypes = [C.c_char_p, C.c_int, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int)]
    T, pad = C.c_int(0), C.c_int(0)
    if R.ref_metcf_load_checkpoint(f"/data/{matrix_name}.mtx".encode(), M, K, C.byref(T), C.byref(pad)) != 1:
        raise RuntimeError("reference loadCheckpoint failed")
    T, pad = int(T.value), int(pad.value)
    W = (M + 15) // 16
    soff = np.zeros(W + 1, dtype=np.int32)
    sidx = np.zeros(8 * T, dtype=np.int32)
    off = np.zeros(2 * T + 1, dtype=np.int32)
    idx = np.zeros(pad, dtype=np.int32)
    val = np.zeros(pad, dtype=np.float32)
    R.ref_metcf_fetch.restype = None
    R.ref_metcf_fetch.argtypes = [_i32p, _i32p, _i32p, _i32p, _f32p]
    R.ref_metcf_fetch(soff, sidx, off, idx, val)
    return dict(val_soff=soff, val_sidx=sidx, val_coo_off=off, val_coo_idx=idx, val_coo_val=val, T=T, nnz_pad=pad)


def ref_strict_lb_plan(M, val_soff, workload=64):
    R = _ref("libref_strict_lb.so")
    val_soff = _c(val_soff, np.int32).copy()
    R.ref_strict_lb_plan.restype = C.c_int
    R.ref_strict_lb_plan.argtypes = [C.c_int, C.c_int, _i32p, C.c_int, C.POINTER(C.c_int)]
    ng = C.c_int(0)
    F = int(R.ref_strict_lb_plan(M, int(val_soff[-1]), val_soff, workload, C.byref(ng)))
    G = int(ng.value)
    rbo = np.zeros(F + 1, dtype=np.int32)
    rb2w = np.zeros(max(F, 1), dtype=np.int32)
    go = np.zeros(G + 1, dtype=np.int32)
    R.ref_strict_lb_fetch.restype = None
    R.ref_strict_lb_fetch.argtypes = [_i32p, _i32p, _i32p]
    R.ref_strict_lb_fetch(rbo, rb2w, go)
    return rbo, rb2w[:F], go


def ref_multi_bind_plan(M, val_soff):
    R = _ref("libref_multi_bind.so")
    val_soff = _c(val_soff, np.int32).copy()
    W = (M + 15) // 16
    R.ref_multi_bind_plan.restype = C.c_int
    R.ref_multi_bind_plan.argtypes = [C.c_int, C.c_int, _i32p]
    P = int(R.ref_multi_bind_plan(M, int(val_soff[-1]), val_soff))
    tw = np.zeros(max(P, 1), dtype=np.int32)
    ws = np.zeros(max(W, 1), dtype=np.int32)
    ts = np.zeros(P + 1, dtype=np.int32)
    R.ref_multi_bind_fetch.restype = None
    R.ref_multi_bind_fetch.argtypes = [_i32p, _i32p, _i32p]
    R.ref_multi_bind_fetch(tw, ws, ts)
    return tw[:P], ws[:W], ts


def ref_gpu_available() -> bool:
    return os.path.exists(os.path.join(_HERE, "_ref", "libref_gpu_srbcrs.so"))


def ref_gpu_srbcrs(M, N, K, packed, B, warmup=3, repeat=10):
    """Runs the reference project's own SR-BCRS 16x8 kernel (recompiled for sm_100a) on host
    arrays; returns (C, mean kernel ms)."""
    R = _ref("libref_gpu_srbcrs.so")
    R.ref_gpu_srbcrs_run.restype = C.c_float
    R.ref_gpu_srbcrs_run.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, _i32p, _i32p, _f32p, _f32p, _f32p, C.c_int,
                                     C.c_int]
    B = _c(B, np.float32)
    out = np.zeros((M, N), dtype=np.float32)
    ms = float(R.ref_gpu_srbcrs_run(M, N, K, int(packed["T"]), _c(packed["val_sidx"], np.int32),
                                    _c(packed["val_soff"], np.int32), B, _c(packed["val_block_val"], np.float32), out,
                                    warmup, repeat))
    if ms < 0:
        raise RuntimeError(f"reference GPU kernel failed (code {ms})")
    return out, ms
