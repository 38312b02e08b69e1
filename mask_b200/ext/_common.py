"""Shared plumbing of the extension-compatible modules: argument checks with the reference
extensions' error behaviour (RuntimeError, like TORCH_CHECK) and the module-level cache that keeps
the packed arrays alive between preprocess and run."""
from __future__ import annotations

import os
import sys
import threading

import torch

_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if _ROOT not in sys.path:  # the modules are imported by bare name from this directory
    sys.path.insert(0, _ROOT)

from mask_b200 import engine  # noqa: E402

_lock = threading.Lock()


def check_input(t, name, dtype=None):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise RuntimeError(f"{name} must be {str(dtype).replace('torch.', '')}")


class Cache:
    """Packed matrices keyed by the data pointer of the row_window_offset tensor handed back to the
    caller (examples/src_fp32/sr_bcrs/testbed/SRBCRSSpMM_kernel.cu:368-385, 408-421)."""

    def __init__(self):
        self._entries = {}

    def put(self, row_window_offset, packed, policy):
        with _lock:
            self._entries[int(row_window_offset.data_ptr())] = (packed, policy)

    def get(self, row_window_offset):
        with _lock:
            hit = self._entries.get(int(row_window_offset.data_ptr()))
        if hit is None:
            raise RuntimeError("preprocess cache miss: run preprocess_gpu first and keep its row_window_offset tensor")
        return hit

    def clear(self):
        with _lock:
            self._entries.clear()


def fill_side_outputs(packed_or_maps, block_partition, edge_to_col, edge_to_row):
    bp, e2c, e2r = packed_or_maps
    W = bp.numel()
    if block_partition.numel() >= W:
        block_partition[:W].copy_(bp)
    if edge_to_col.numel() >= e2c.numel():
        edge_to_col[: e2c.numel()].copy_(e2c)
    if edge_to_row.numel() >= e2r.numel():
        edge_to_row[: e2r.numel()].copy_(e2r)


def pack_without_sync(pack, rowptr, colind, num_nodes, *more):
    """Packs with K = num_nodes (a graph adjacency: the common case, no extra device round trip)
    and only when the packer reports a column beyond that asks the device for the largest one."""
    from mask_b200 import _lib
    try:
        return pack(rowptr, colind, *more, num_nodes, num_nodes)
    except _lib.MaskError as e:
        if e.status != 6 or not colind.numel():   # MASK_ERR_COLUMN_RANGE
            raise
    K = int(colind.max().item()) + 1
    return pack(rowptr, colind, *more, num_nodes, K)


def run(cache, dense, row_window_offset, num_nodes, policy_override=None):
    if not isinstance(dense, torch.Tensor) or not dense.is_cuda or dense.dtype != torch.float32:
        raise RuntimeError("dense must be a float32 CUDA tensor")
    check_input(row_window_offset, "row_window_offset")
    packed, policy = cache.get(row_window_offset)
    if dense.dim() != 2:
        raise RuntimeError("dense must be 2-D")
    # like the reference extension: any layout (made contiguous here) and any number of rows that
    # covers the matrix's columns (examples/src_fp32/sr_bcrs/testbed/SRBCRSSpMM_kernel.cu:404-406)
    if dense.size(0) < packed.K:
        raise RuntimeError(f"dense has {dense.size(0)} rows but the matrix references column {packed.K - 1}")
    dense = dense[: packed.K].contiguous()
    if int(num_nodes) != packed.M:
        raise RuntimeError(f"num_nodes mismatch: preprocess saw {packed.M}, run got {num_nodes}")
    if dense.size(1) == 0:
        return [torch.empty((packed.M, 0), dtype=torch.float32, device=dense.device)]
    if packed.T == 0:
        raise RuntimeError("matrix has no stored entries (CSR fallback disabled)")
    return [engine.spmm(packed, dense, policy=policy_override or policy)]
