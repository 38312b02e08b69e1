"""ctypes binding of ``libmask_b200.so`` (the C ABI declared in ``include/mask_b200.h``).

The library is the only compute path of this package: if it is missing the import fails loudly;
there is no CPU or PyTorch fallback.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "csrc", "libmask_b200.so")

vp, i32, i64, sz = C.c_void_p, C.c_int32, C.c_int64, C.c_size_t

# name -> (restype, argtypes); every symbol declared in include/mask_b200.h
SIGNATURES = {
    "mask_version": (C.c_int, []),
    "mask_status_string": (C.c_char_p, [C.c_int]),
    "mask_last_error": (C.c_char_p, []),
    "mask_pack_scratch_bytes": (sz, [i32, i64]),
    "mask_pack_analyze": (C.c_int, [vp, vp, i32, i32, i64, vp, sz, vp, C.POINTER(i64), vp]),
    "mask_srbcrs_fill": (C.c_int, [vp, vp, vp, i32, i64, vp, vp, i64, vp, vp, vp, vp, vp, vp]),
    "mask_metcf_offsets": (C.c_int, [vp, i32, i64, vp, vp, i64, vp, vp, C.POINTER(i64), vp]),
    "mask_metcf_fill": (C.c_int, [vp, vp, vp, i32, i64, vp, vp, i64, vp, vp, i64, vp, vp, vp, vp]),
    "mask_mco_offsets": (C.c_int, [vp, i32, i64, vp, vp, i64, C.c_int, vp, vp, C.POINTER(i64), vp]),
    "mask_mco_fill": (C.c_int, [vp, vp, i32, i64, vp, vp, i64, C.c_int, vp, vp, i64, vp, vp, vp]),
    "mask_reorder_rows": (C.c_int, [C.c_int, vp, vp, i32, i32, vp, vp]),
    "mask_csr_permute_rows": (C.c_int, [vp, vp, vp, i32, vp, vp, vp, vp, vp]),
    "mask_plan_set_row_map": (C.c_int, [vp, vp]),
    "mask_plan_set_peer_outputs": (C.c_int, [vp, vp, i32]),
    "mask_peer_alloc": (C.c_int, [C.c_size_t, C.POINTER(C.c_void_p), vp]),
    "mask_peer_open": (C.c_int, [vp, C.POINTER(C.c_void_p)]),
    "mask_peer_close": (C.c_int, [vp]),
    "mask_peer_free": (C.c_int, [vp]),
    "mask_features_from_soff": (C.c_int, [vp, i32, i64, vp]),
    "mask_metcf_checkpoint_name": (C.c_int, [C.c_char_p, i32, i32, C.c_char_p, sz]),
    "mask_metcf_checkpoint_name_for": (C.c_int, [C.c_char_p, i32, i32, C.c_float, C.c_char_p, sz]),
    "mask_metcf_checkpoint_write": (C.c_int, [C.c_char_p, i32, i64, i64, vp, vp, vp, vp, vp]),
    "mask_metcf_checkpoint_header": (C.c_int, [C.c_char_p, C.POINTER(i64), C.POINTER(i64)]),
    "mask_metcf_checkpoint_read": (C.c_int, [C.c_char_p, i32, i32, i64, i64, vp, vp, vp, vp, vp]),
    "mask_plan_strict_lb": (C.c_int, [vp, i32, i32, vp, vp, vp, C.POINTER(i64), C.POINTER(i64)]),
    "mask_plan_multi_bind": (C.c_int, [vp, i32, vp, vp, vp, C.POINTER(i64)]),
    "mask_plan_create": (C.c_int, [vp, i32, i64, C.c_int, i32, vp, C.POINTER(vp)]),
    "mask_plan_destroy": (None, [vp]),
    "mask_plan_scratch_bytes": (sz, [vp, i32]),
    "mask_plan_info": (C.c_int, [vp, C.POINTER(i64), C.POINTER(i64), C.POINTER(i64), C.POINTER(i32)]),
    "mask_plan_export": (C.c_int, [vp, vp, vp, vp]),
    "mask_features_columns": (C.c_int, [vp, vp, i32, i32, i64, i32, vp, vp]),
    "mask_plan_autotune": (C.c_int, [vp, vp, vp, i32, vp]),
    "mask_plan_column_features": (C.c_int, [vp, vp, C.POINTER(i32)]),
    "mask_plan_prepare_values": (C.c_int, [vp, vp, vp]),
    "mask_plan_status": (C.c_int, [vp, C.POINTER(i32), vp]),
    "mask_spmm_srbcrs": (C.c_int, [vp, vp, vp, vp, i32, i32, i32, vp, i64, vp, i64, vp, sz, C.c_int, vp]),
    "mask_spmm_metcf": (C.c_int, [vp, vp, vp, vp, vp, vp, i32, i32, i32, vp, i64, vp, i64, vp, sz, C.c_int, vp]),
    "mask_spmm_mco": (C.c_int, [vp, vp, vp, vp, vp, vp, i32, i32, i32, vp, i64, vp, i64, vp, sz, C.c_int, vp]),
    "mask_static_scratch_capacity": (sz, []),
    "mask_spmm_srbcrs_static_scratch": (C.c_int, [vp, vp, vp, vp, i32, i32, i32, vp, i64, vp, i64, C.c_int, vp]),
    "mask_tune": (C.c_int, [C.c_char_p, C.c_int]),
    "mask_spmm_kernel_name": (C.c_int, [vp, C.c_int, i32, C.c_int, C.c_char_p, sz]),
    "mask_kernel_revision": (C.c_int, []),
    "mask_copy_2d_async": (C.c_int, [vp, sz, vp, sz, sz, sz, C.c_int, vp]),
    "mask_session_create_srbcrs": (C.c_int, [i32, i32, i64, vp, vp, vp, C.c_int, C.POINTER(vp)]),
    "mask_session_create_csr": (C.c_int, [i32, i32, i64, vp, vp, vp, C.c_int, C.POINTER(vp)]),
    "mask_session_spmm_host": (C.c_int, [vp, vp, vp, i32, C.POINTER(C.c_float)]),
    "mask_session_tiles": (i64, [vp]),
    "mask_session_destroy": (None, [vp]),
}

REORDER = {"none": 0, "row_rcm": 1, "first_col_sort": 2, "jaccard_greedy": 3}
POLICY = {"auto": 0, "row": 1, "strict_lb": 2, "multi_bind": 3, "ref_auto": 4}


class Features(C.Structure):
    """mask_features"""
    _fields_ = [("row_windows", i32), ("empty_windows", i32), ("tiles", i64), ("nnz", i64), ("tiles_mean", C.c_double),
                ("tiles_p50", i32), ("tiles_p95", i32), ("tiles_p99", i32), ("tiles_max", i32),
                ("top5_window_share", C.c_double), ("tile_fill", C.c_double), ("heavy_tail", i32)]


class ColumnFeatures(C.Structure):
    """mask_column_features"""
    _fields_ = [("gathers", i64), ("distinct_columns", i32), ("band_p50", i32), ("band_p90", i32), ("hub_columns", i32 * 3),
                ("hub_share", C.c_double * 3), ("l2_bytes", i32), ("local_rows", i32), ("local_share", C.c_double)]

    def as_dict(self):
        return dict(gathers=int(self.gathers), distinct_columns=int(self.distinct_columns), band_p50=int(self.band_p50),
                    band_p90=int(self.band_p90), hub_columns=list(self.hub_columns), hub_share=[round(x, 4) for x in self.hub_share],
                    l2_bytes=int(self.l2_bytes), local_rows=int(self.local_rows), local_share=round(float(self.local_share), 4))


EPILOGUE_NONE, EPILOGUE_RELU = 0, 1
NUMERICS_TF32X3 = 0x100   # OR-able into the epilogue argument (SR-BCRS)

_lib = None


class MaskError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, status: int, where: str, detail: str):
        super().__init__(f"{where}: status {status} ({detail})")
        self.status = status


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `make -C mask_b200/csrc` "
                "(or `python -c 'import __graft_entry__ as g; g.build()'`). There is no fallback path.")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)  # AttributeError if the library does not export it
            fn.restype = res
            fn.argtypes = args
        _lib = L
        # development switch: MASK_B200_TUNE="knob=value,..." applies mask_tune() knobs at load time
        for item in filter(None, os.environ.get("MASK_B200_TUNE", "").split(",")):
            name, _, value = item.partition("=")
            if L.mask_tune(name.strip().encode(), int(value)) != 0:
                raise RuntimeError(f"MASK_B200_TUNE: unknown knob {name!r}")
    return _lib


def check(status: int, where: str) -> None:
    if status != 0:
        L = lib()
        detail = L.mask_last_error().decode() or L.mask_status_string(status).decode()
        raise MaskError(status, where, detail)
