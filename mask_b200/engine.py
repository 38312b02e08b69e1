"""Torch-tensor front end of the C ABI: device format builder, execution plans and SpMM.

PyTorch is used for device memory and streams only; every computation happens in
``libmask_b200.so``.  All tensors are CUDA tensors on the current device.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import torch

from . import _lib
from ._lib import check, lib


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _req(t, dtype, name):
    if not (isinstance(t, torch.Tensor) and t.is_cuda):
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    if t.dtype != dtype:
        raise RuntimeError(f"{name} must be {str(dtype).replace('torch.', '')}")


class Plan:
    """How tiles are dealt to thread blocks (``mask_plan``)."""

    def __init__(self, val_soff: torch.Tensor, M: int, T: int, policy: str = "auto", group_tiles: int = 0):
        _req(val_soff, torch.int32, "val_soff")
        h = C.c_void_p()
        check(lib().mask_plan_create(_ptr(val_soff), M, T, _lib.POLICY[policy], group_tiles, _stream(), C.byref(h)),
              "mask_plan_create")
        self._h = h
        self.policy = policy
        self.M, self.T = M, T
        self._scratch = None

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h and lib is not None:  # module globals may already be gone at interpreter exit
            try:
                lib().mask_plan_destroy(h)
            except Exception:
                pass

    def scratch_bytes(self, N: int) -> int:
        return int(lib().mask_plan_scratch_bytes(self._h, N))

    def info(self) -> dict:
        f, g, p, gt = C.c_int64(), C.c_int64(), C.c_int64(), C.c_int32()
        check(lib().mask_plan_info(self._h, C.byref(f), C.byref(g), C.byref(p), C.byref(gt)), "mask_plan_info")
        return dict(fragments=f.value, groups=g.value, partial=p.value, group_tiles=gt.value)

    def column_features(self) -> dict | None:
        """What mask_plan_autotune measured and chose (None if it has not run)."""
        f, ns = _lib.ColumnFeatures(), C.c_int32(0)
        if lib().mask_plan_column_features(self._h, C.byref(f), C.byref(ns)) != 0:
            return None
        d = f.as_dict()
        d["nslab_wide"] = int(ns.value)
        return d

    def status(self) -> int:
        """Device status word: non-zero if a kernel using this plan gave up on a bounded wait."""
        v = C.c_int32(0)
        check(lib().mask_plan_status(self._h, C.byref(v), _stream()), "mask_plan_status")
        return int(v.value)

    def set_peer_outputs(self, ptrs: torch.Tensor | None) -> None:
        """ptrs: int64 CUDA tensor of device addresses (bases of the peers' copies of C), or None."""
        if ptrs is None:
            check(lib().mask_plan_set_peer_outputs(self._h, None, 0), "mask_plan_set_peer_outputs")
            self._peer_ptrs = None
            return
        _req(ptrs, torch.int64, "ptrs")
        check(lib().mask_plan_set_peer_outputs(self._h, _ptr(ptrs), int(ptrs.numel())), "mask_plan_set_peer_outputs")
        self._peer_ptrs = ptrs  # keep the array alive as long as the plan uses it

    def export(self):
        """Host copies of (frag_offset[F+1], frag_window[F], group_offset[G+1])."""
        i = self.info()
        fo = torch.zeros(i["fragments"] + 1, dtype=torch.int32)
        fw = torch.zeros(max(i["fragments"], 1), dtype=torch.int32)
        go = torch.zeros(i["groups"] + 1, dtype=torch.int32)
        check(lib().mask_plan_export(self._h, _ptr(fo), _ptr(fw), _ptr(go)), "mask_plan_export")
        return fo, fw[: i["fragments"]], go

    def scratch(self, N: int, device) -> torch.Tensor | None:
        """Partial-tile buffer for the current stream: products on different streams may overlap on
        the GPU, so each stream gets its own buffer (products on one stream run in order and share it)."""
        need = self.scratch_bytes(N)
        if need == 0:
            return None
        if self._scratch is None:
            self._scratch = {}
        key = (torch.cuda.current_stream().cuda_stream, device)
        buf = self._scratch.get(key)
        if buf is None or buf.numel() < need:
            buf = self._scratch[key] = torch.empty(need, dtype=torch.uint8, device=device)
        return buf


@dataclass
class PackedSRBCRS:
    """SR-BCRS 16x8: val_soff int32[W+1], val_sidx int32[8T], val_block_val f32[128T]."""
    M: int
    K: int
    T: int
    nnz: int
    val_soff: torch.Tensor
    val_sidx: torch.Tensor
    val_block_val: torch.Tensor
    block_partition: torch.Tensor | None = None
    edge_to_col: torch.Tensor | None = None
    edge_to_row: torch.Tensor | None = None
    row_order: torch.Tensor | None = None   # set when the rows were reordered: packed row i = original row row_order[i]
    plans: dict = field(default_factory=dict)

    def plan(self, policy: str = "auto", group_tiles: int = 0) -> Plan:
        key = (policy, group_tiles)
        if key not in self.plans:
            self.plans[key] = self.new_plan(policy, group_tiles)
        return self.plans[key]

    def new_plan(self, policy: str = "auto", group_tiles: int = 0, prepare: bool = False, autotune: bool = True) -> Plan:
        """A plan for this matrix: tuned from the matrix's column features (``autotune``), carrying the
        row map when the rows were reordered and, on request, the rounded copy of the tile values that
        the TMA-fed kernel reads (``prepare``; as much device memory as val_block_val again)."""
        p = Plan(self.val_soff, self.M, self.T, policy, group_tiles)
        if autotune and self.T > 0:
            check(lib().mask_plan_autotune(p._h, _ptr(self.val_soff), _ptr(self.val_sidx), self.K, _stream()), "mask_plan_autotune")
        if prepare and isinstance(self, PackedSRBCRS) and self.T > 0:
            check(lib().mask_plan_prepare_values(p._h, _ptr(self.val_block_val), _stream()), "mask_plan_prepare_values")
        if self.row_order is not None:
            check(lib().mask_plan_set_row_map(p._h, _ptr(self.row_order)), "mask_plan_set_row_map")
            p._row_order = self.row_order  # keep the array alive as long as the plan
        return p


@dataclass
class PackedMETCF:
    """ME-TCF: val_soff, val_sidx (tail 0), val_coo_off int32[2T+1], val_coo_idx / val_coo_val [nnz_pad]."""
    M: int
    K: int
    T: int
    nnz: int
    nnz_pad: int
    val_soff: torch.Tensor
    val_sidx: torch.Tensor
    val_coo_off: torch.Tensor
    val_coo_idx: torch.Tensor
    val_coo_val: torch.Tensor
    row_order: torch.Tensor | None = None
    plans: dict = field(default_factory=dict)

    plan = PackedSRBCRS.plan
    new_plan = PackedSRBCRS.new_plan


@dataclass
class PackedMCO:
    """MCO / BIT-TCF: val_soff, val_sidx (tail = last real column), val_mco_off int32[T+1],
    val_mco_mask int64[2T] (bit Swizzle<1,2,3>(8r+c)), val_mco_val float32[nval]."""
    M: int
    K: int
    T: int
    nnz: int
    nval: int
    val_soff: torch.Tensor
    val_sidx: torch.Tensor
    val_mco_off: torch.Tensor
    val_mco_mask: torch.Tensor
    val_mco_val: torch.Tensor
    row_order: torch.Tensor | None = None
    plans: dict = field(default_factory=dict)

    plan = PackedSRBCRS.plan
    new_plan = PackedSRBCRS.new_plan


def _analyze(rowptr, colind, M, K):
    _req(rowptr, torch.int32, "rowptr")
    _req(colind, torch.int32, "colind")
    if M < 1:
        raise RuntimeError("num_nodes must be positive")
    if rowptr.numel() != M + 1:
        raise RuntimeError("rowptr must have num_nodes + 1 entries")
    L = lib()
    nnz = int(colind.numel())
    dev = rowptr.device
    W = (M + 15) // 16
    ws_bytes = int(L.mask_pack_scratch_bytes(M, nnz))
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    val_soff = torch.empty(W + 1, dtype=torch.int32, device=dev)
    T = C.c_int64(0)
    check(L.mask_pack_analyze(_ptr(rowptr), _ptr(colind), M, K, nnz, _ptr(ws), ws_bytes, _ptr(val_soff), C.byref(T),
                              _stream()), "mask_pack_analyze")
    return ws, val_soff, int(T.value), nnz


def reorder_rows(rowptr, colind, M: int, K: int, kind: str) -> torch.Tensor:
    """Row order of one of the Format-DSL bridge's reorders (``row_rcm``, ``first_col_sort``,
    ``jaccard_greedy``), computed on the device; returns order[new] = original as an int32 tensor
    on the CSR's device."""
    _req(rowptr, torch.int32, "rowptr")
    _req(colind, torch.int32, "colind")
    order = torch.empty(M, dtype=torch.int32, device=rowptr.device)
    check(lib().mask_reorder_rows(_lib.REORDER[kind], _ptr(rowptr), _ptr(colind), M, K, _ptr(order), _stream()), "mask_reorder_rows")
    return order


def permute_rows(rowptr, colind, values, M: int, order: torch.Tensor):
    """Device CSR whose row i is row order[i] of the input."""
    _req(order, torch.int32, "order")
    rp = torch.empty_like(rowptr)
    ci = torch.empty_like(colind)
    va = torch.empty_like(values)
    check(lib().mask_csr_permute_rows(_ptr(rowptr), _ptr(colind), _ptr(values), M, _ptr(order), _ptr(rp), _ptr(ci),
                                      _ptr(va), _stream()), "mask_csr_permute_rows")
    return rp, ci, va


def pack_srbcrs(rowptr, colind, values, M: int, K: int, side_outputs: bool = False, reorder: str = "none") -> PackedSRBCRS:
    """CSR (device, rows strictly ascending) -> SR-BCRS 16x8 on the device.  With ``reorder`` the
    rows are packed in that order and products still come back in the original row order."""
    _req(values, torch.float32, "values")
    if values.numel() != colind.numel():
        raise RuntimeError("values length must equal colind length")
    if reorder != "none":
        order = reorder_rows(rowptr, colind, M, K, reorder)
        packed = pack_srbcrs(*permute_rows(rowptr, colind, values, M, order), M, K, side_outputs)
        packed.row_order = order
        return packed
    ws, val_soff, T, nnz = _analyze(rowptr, colind, M, K)
    dev = rowptr.device
    val_sidx = torch.empty(8 * T, dtype=torch.int32, device=dev)
    val_block_val = torch.empty(128 * T, dtype=torch.float32, device=dev)
    bp = e2c = e2r = None
    if side_outputs:
        bp = torch.empty((M + 15) // 16, dtype=torch.int32, device=dev)
        e2c = torch.empty(nnz, dtype=torch.int32, device=dev)
        e2r = torch.empty(nnz, dtype=torch.int32, device=dev)
    check(lib().mask_srbcrs_fill(_ptr(rowptr), _ptr(colind), _ptr(values), M, nnz, _ptr(ws), _ptr(val_soff), T,
                                 _ptr(val_sidx), _ptr(val_block_val), _ptr(bp), _ptr(e2c), _ptr(e2r), _stream()),
          "mask_srbcrs_fill")
    return PackedSRBCRS(M, K, T, nnz, val_soff, val_sidx, val_block_val, bp, e2c, e2r)


def pack_metcf(rowptr, colind, values, M: int, K: int) -> PackedMETCF:
    """CSR (device) -> ME-TCF on the device.  ``values=None`` stores 1.0 for every entry."""
    if values is not None:
        _req(values, torch.float32, "values")
    ws, val_soff, T, nnz = _analyze(rowptr, colind, M, K)
    dev = rowptr.device
    L = lib()
    val_coo_off = torch.empty(2 * T + 1, dtype=torch.int32, device=dev)
    tile_rows = torch.empty(max(T, 1), dtype=torch.int64, device=dev)
    pad = C.c_int64(0)
    check(L.mask_metcf_offsets(_ptr(rowptr), M, nnz, _ptr(ws), _ptr(val_soff), T, _ptr(val_coo_off), _ptr(tile_rows),
                               C.byref(pad), _stream()), "mask_metcf_offsets")
    nnz_pad = int(pad.value)
    val_sidx = torch.empty(8 * T, dtype=torch.int32, device=dev)
    val_coo_idx = torch.empty(nnz_pad, dtype=torch.int32, device=dev)
    val_coo_val = torch.empty(nnz_pad, dtype=torch.float32, device=dev)
    check(L.mask_metcf_fill(_ptr(rowptr), _ptr(colind), _ptr(values), M, nnz, _ptr(ws), _ptr(val_soff), T,
                            _ptr(val_coo_off), _ptr(tile_rows), nnz_pad, _ptr(val_sidx), _ptr(val_coo_idx),
                            _ptr(val_coo_val), _stream()), "mask_metcf_fill")
    return PackedMETCF(M, K, T, nnz, nnz_pad, val_soff, val_sidx, val_coo_off, val_coo_idx, val_coo_val)


def pack_mco(rowptr, colind, values, M: int, K: int, skip_zero_values: bool = False) -> PackedMCO:
    """CSR (device) -> MCO / BIT-TCF on the device.  ``skip_zero_values`` follows the Format-DSL
    bridge (explicit zeros are dropped); the BIT-TCF testbed keeps them."""
    if values is not None:
        _req(values, torch.float32, "values")
    ws, val_soff, T, nnz = _analyze(rowptr, colind, M, K)
    dev = rowptr.device
    L = lib()
    val_mco_mask = torch.empty(2 * max(T, 1), dtype=torch.int64, device=dev)
    val_mco_off = torch.empty(T + 1, dtype=torch.int32, device=dev)
    nv = C.c_int64(0)
    check(L.mask_mco_offsets(_ptr(values), M, nnz, _ptr(ws), _ptr(val_soff), T, int(skip_zero_values), _ptr(val_mco_mask),
                             _ptr(val_mco_off), C.byref(nv), _stream()), "mask_mco_offsets")
    nval = int(nv.value)
    val_sidx = torch.empty(8 * T, dtype=torch.int32, device=dev)
    val_mco_val = torch.empty(max(nval, 4), dtype=torch.float32, device=dev)
    check(L.mask_mco_fill(_ptr(rowptr), _ptr(values), M, nnz, _ptr(ws), _ptr(val_soff), T, int(skip_zero_values),
                          _ptr(val_mco_mask), _ptr(val_mco_off), nval, _ptr(val_sidx), _ptr(val_mco_val), _stream()),
          "mask_mco_fill")
    return PackedMCO(M, K, T, nnz, nval, val_soff, val_sidx, val_mco_off, val_mco_mask[:2 * T], val_mco_val[:nval])


def spmm(packed, dense: torch.Tensor, out: torch.Tensor | None = None, policy: str = "auto", relu: bool = False,
         plan: Plan | None = None, tf32x3: bool = False) -> torch.Tensor:
    """out[M,N] = A @ dense[K,N] on the current stream.  ``out`` is fully overwritten.
    ``tf32x3`` (SR-BCRS): compensated products, FP32-level accuracy at about 1.7x the time."""
    _req(dense, torch.float32, "dense")
    if dense.dim() != 2:
        raise RuntimeError("dense must be 2-D")
    if dense.size(0) != packed.K:
        raise RuntimeError(f"dense has {dense.size(0)} rows, the matrix has {packed.K} columns")
    N = int(dense.size(1))
    if out is None:
        out = torch.empty((packed.M, N), dtype=torch.float32, device=dense.device)
    else:
        _req(out, torch.float32, "out")
        if tuple(out.shape) != (packed.M, N):
            raise RuntimeError("out has the wrong shape")
    if N == 0:
        return out
    plan = plan or packed.plan(policy)
    if packed.row_order is not None and getattr(plan, "_row_order", None) is not packed.row_order:
        raise RuntimeError("this matrix was packed from reordered rows: use packed.plan() / packed.new_plan()")
    scratch = plan.scratch(N, dense.device)
    sb = 0 if scratch is None else scratch.numel()
    epi = (_lib.EPILOGUE_RELU if relu else _lib.EPILOGUE_NONE) | (_lib.NUMERICS_TF32X3 if tf32x3 else 0)
    L = lib()
    if isinstance(packed, PackedMCO):
        check(L.mask_spmm_mco(plan._h, _ptr(packed.val_soff), _ptr(packed.val_sidx), _ptr(packed.val_mco_off),
                              _ptr(packed.val_mco_mask), _ptr(packed.val_mco_val), packed.M, packed.K, N, _ptr(dense),
                              N, _ptr(out), N, _ptr(scratch), sb, epi, _stream()), "mask_spmm_mco")
    elif isinstance(packed, PackedMETCF):
        check(L.mask_spmm_metcf(plan._h, _ptr(packed.val_soff), _ptr(packed.val_sidx), _ptr(packed.val_coo_off),
                                _ptr(packed.val_coo_idx), _ptr(packed.val_coo_val), packed.M, packed.K, N, _ptr(dense),
                                N, _ptr(out), N, _ptr(scratch), sb, epi, _stream()), "mask_spmm_metcf")
    else:
        check(L.mask_spmm_srbcrs(plan._h, _ptr(packed.val_soff), _ptr(packed.val_sidx), _ptr(packed.val_block_val),
                                 packed.M, packed.K, N, _ptr(dense), N, _ptr(out), N, _ptr(scratch), sb, epi,
                                 _stream()), "mask_spmm_srbcrs")
    return out


def kernel_signature(packed, N: int, plan: Plan, tf32x3: bool = False) -> tuple[str, int]:
    """(name of the kernel ``spmm`` launches for this matrix, plan and N; the library's kernel revision)."""
    fmt = 2 if isinstance(packed, PackedMCO) else (1 if isinstance(packed, PackedMETCF) else 0)
    buf = C.create_string_buffer(128)
    check(lib().mask_spmm_kernel_name(plan._h, fmt, N, _lib.NUMERICS_TF32X3 if tf32x3 else 0, buf, 128), "mask_spmm_kernel_name")
    return buf.value.decode(), int(lib().mask_kernel_revision())


def tune(name: str, value: int) -> None:
    check(lib().mask_tune(name.encode(), value), "mask_tune")
