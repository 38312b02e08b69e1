"""Caller-level SpMM callables with the signature the reference's GCN driver expects from an
external backend: ``fn(rowptr, colind, values, dense, num_rows, feat_dim, num_nodes_ori) -> Tensor``
(end2end/gcn/eva_gcn_sparsene.py:249-264; the reference's own provider is
end2end/gcn/external_backend_spmm.py:1441-1485, which can also be pointed at ``mask_b200/ext``).

Preprocessing (device packing + plan) is cached per CSR identity -- data pointers, shape and
variant, like the reference router (external_backend_spmm.py:805-841) -- so it is paid once per
graph.  Selection follows the reference's environment switches: ``SPARSENE_SPMM_BACKEND``
(``sr_bcrs`` | ``dtc``), ``SPARSENE_SRBCRS_VARIANT`` / ``SPARSENE_DTC_VARIANT``
(``16x8`` | ``base`` | ``strict_lb`` | ``multi_binding`` and the 16x8_* spellings).
There is no CSR fallback: failures raise.
"""
from __future__ import annotations

import os

import torch

from . import engine

_cache: dict = {}

_POLICY = {"base": "auto", "16x8": "auto", "strict_lb": "strict_lb", "16x8_strict_lb": "strict_lb",
           "multi_binding": "multi_bind", "multi_bind": "multi_bind", "16x8_multi_binding": "multi_bind"}


def reset_backend_state() -> None:
    """Drops every cached packed matrix (external_backend_spmm.py:1406-1414)."""
    _cache.clear()


def _pack_square_first(pack, rp, ci, va, num_rows):
    """Packs with K = num_rows (graph adjacency, no device round trip for the column count) and asks
    the device for the largest column only when the packer reports one beyond that."""
    from ._lib import MaskError
    try:
        return pack(rp, ci, va, num_rows, num_rows)
    except MaskError as e:
        if e.status != 6 or not ci.numel():   # MASK_ERR_COLUMN_RANGE
            raise
    return pack(rp, ci, va, num_rows, int(ci.max().item()) + 1)


def _prep(fmt, rowptr, colind, values, num_rows, variant):
    key = (fmt, variant, int(rowptr.data_ptr()), int(colind.data_ptr()), int(values.data_ptr()) if values is not None else 0,
           int(num_rows), int(colind.numel()))
    hit = _cache.get(key)
    if hit is None:
        rp = rowptr if rowptr.dtype == torch.int32 else rowptr.to(torch.int32)
        ci = colind if colind.dtype == torch.int32 else colind.to(torch.int32)
        va = None if values is None else (values if values.dtype == torch.float32 else values.to(torch.float32))
        rp, ci = rp.contiguous(), ci.contiguous()
        if fmt == "sr_bcrs":
            if va is None:   # pattern-only graph: unit weights
                va = torch.ones(ci.numel(), dtype=torch.float32, device=ci.device)
            packed = _pack_square_first(engine.pack_srbcrs, rp, ci, va.contiguous(), int(num_rows))
        else:
            packed = _pack_square_first(engine.pack_metcf, rp, ci, None if va is None else va.contiguous(), int(num_rows))
        hit = (packed, (rowptr, colind, values))  # keep the CSR alive: the key holds its addresses
        _cache[key] = hit
    return hit[0]


def _run(fmt, variant, rowptr, colind, values, dense, num_rows):
    policy = _POLICY.get(variant)
    if policy is None:
        raise RuntimeError(f"unknown {fmt} variant '{variant}'")
    packed = _prep(fmt, rowptr, colind, values, num_rows, variant)
    d = dense if (dense.dtype == torch.float32 and dense.is_contiguous()) else dense.to(torch.float32).contiguous()
    n = int(d.shape[1])
    if n % 4:  # the kernels take any multiple of 4; pad like the reference pads to its tile width
        d = torch.nn.functional.pad(d, (0, 4 - n % 4))
    if packed.K > d.shape[0]:
        raise RuntimeError(f"dense has {d.shape[0]} rows but the matrix references column {packed.K - 1}")
    if packed.K < d.shape[0]:
        d = d[: packed.K]
    out = engine.spmm(packed, d, policy=policy)
    return out if out.shape[1] == n else out[:, :n].contiguous()


def srbcrs_spmm(rowptr, colind, values, dense, num_rows, feat_dim, num_nodes_ori):
    variant = os.getenv("SPARSENE_SRBCRS_VARIANT", os.getenv("SPARSENE_SPMM_VARIANT", "16x8")).strip().lower() or "16x8"
    return _run("sr_bcrs", variant, rowptr, colind, values, dense, num_rows)


def dtc_spmm(rowptr, colind, values, dense, num_rows, feat_dim, num_nodes_ori):
    variant = os.getenv("SPARSENE_DTC_VARIANT", "base").strip().lower() or "base"
    return _run("dtc", variant, rowptr, colind, values, dense, num_rows)


def spmm_external(rowptr, colind, values, dense, num_rows, feat_dim, num_nodes_ori):
    name = os.getenv("SPARSENE_SPMM_BACKEND", "sr_bcrs").strip().lower()
    if name == "dtc":
        return dtc_spmm(rowptr, colind, values, dense, num_rows, feat_dim, num_nodes_ori)
    if name in ("sr_bcrs", "srbcrs"):
        return srbcrs_spmm(rowptr, colind, values, dense, num_rows, feat_dim, num_nodes_ori)
    raise RuntimeError(f"backend '{name}' is not provided by this library (sr_bcrs and dtc are)")
