"""Drop-in for the reference project's ``DTCSpMM`` torch extension (ME-TCF format;
examples/src_fp32/dtc/testbed/DTCSpMM.cpp:219-230, dtc_runtime_api.h:9-45): same function names,
argument order and tuple shapes, served by the B200 library.

Like the reference, ``preprocess_gpu`` takes no values and stores 1.0 for every entry
(DTCSpMM_kernel.cu:450); pass ``values=`` to carry real weights (an extension of the reference
signature).  The ``multi_binding`` and ``*_balance`` entry points are aliases of the base path in
the reference (DTCSpMM.cpp:64-87,117-134,185-217) and select task mappings here.
"""
from __future__ import annotations

import torch

from _common import Cache, check_input, engine, fill_side_outputs, pack_without_sync, run

_cache = Cache()


def _preprocess(colind, rowptr, num_nodes, blk_h, blk_w, block_partition, edge_to_col, edge_to_row, policy, values):
    for t, n, dt in ((colind, "colind", torch.int32), (rowptr, "rowptr", torch.int32),
                     (block_partition, "block_partition", None), (edge_to_col, "edge_to_col", None),
                     (edge_to_row, "edge_to_row", None)):
        check_input(t, n, dt)
    if values is not None:
        check_input(values, "values", torch.float32)
    if int(num_nodes) < 1:
        raise RuntimeError("num_nodes must be positive")
    if int(blk_h) != 16 or int(blk_w) != 8:
        raise RuntimeError(f"ME-TCF uses 16x8 tiles: got blk_h={blk_h} blk_w={blk_w}")
    num_nodes = int(num_nodes)
    packed = pack_without_sync(engine.pack_metcf, rowptr, colind, num_nodes, values)
    K = packed.K
    # side outputs come from the SR-BCRS fill of the same analysis (tiles per window, condensed
    # column and row of every entry)
    ones = values if values is not None else torch.ones(colind.numel(), dtype=torch.float32, device=colind.device)
    sr = engine.pack_srbcrs(rowptr, colind, ones, num_nodes, K, side_outputs=True)
    fill_side_outputs((sr.block_partition, sr.edge_to_col, sr.edge_to_row), block_partition, edge_to_col, edge_to_row)
    del sr
    _cache.put(packed.val_soff, packed, policy)
    # (row_window_offset, tcblock_rowid, tcblocktile_id, tcblock_offset, sparse_a_to_x_idx, T)
    return (packed.val_soff, torch.zeros(packed.T, dtype=torch.int32, device=rowptr.device), packed.val_sidx,
            packed.val_coo_off, packed.val_coo_idx, packed.T)


def preprocess_gpu(colind, rowptr, num_nodes, blk_h, blk_w, block_partition, edge_to_col, edge_to_row, values=None):
    return _preprocess(colind, rowptr, num_nodes, blk_h, blk_w, block_partition, edge_to_col, edge_to_row, "auto", values)


def preprocess_gpu_strict_lb(colind, rowptr, num_nodes, blk_h, blk_w, block_partition, edge_to_col, edge_to_row,
                             values=None):
    return _preprocess(colind, rowptr, num_nodes, blk_h, blk_w, block_partition, edge_to_col, edge_to_row, "strict_lb",
                       values)


def preprocess_gpu_multi_binding(colind, rowptr, num_nodes, blk_h, blk_w, block_partition, edge_to_col, edge_to_row,
                                 values=None):
    return _preprocess(colind, rowptr, num_nodes, blk_h, blk_w, block_partition, edge_to_col, edge_to_row, "multi_bind",
                       values)


def _run(dense, row_window_offset, tcblocktile_id, tcblock_offset, sparse_a_to_x_idx, num_nodes, policy=None):
    check_input(tcblocktile_id, "tcblocktile_id")
    check_input(tcblock_offset, "tcblock_offset")
    check_input(sparse_a_to_x_idx, "sparse_a_to_x_idx")
    return run(_cache, dense, row_window_offset, num_nodes, policy)


def run_DTCSpMM(dense, row_window_offset, tcblocktile_id, tcblock_offset, sparse_a_to_x_idx, num_nodes, num_edges, exeplan):
    return _run(dense, row_window_offset, tcblocktile_id, tcblock_offset, sparse_a_to_x_idx, num_nodes)


def run_DTCSpMM_strict_lb(dense, row_window_offset, tcblocktile_id, tcblock_offset, sparse_a_to_x_idx, num_nodes,
                          num_edges, exeplan):
    return _run(dense, row_window_offset, tcblocktile_id, tcblock_offset, sparse_a_to_x_idx, num_nodes, "strict_lb")


def run_DTCSpMM_multi_binding(dense, row_window_offset, tcblocktile_id, tcblock_offset, sparse_a_to_x_idx, num_nodes,
                              num_edges, exeplan):
    return _run(dense, row_window_offset, tcblocktile_id, tcblock_offset, sparse_a_to_x_idx, num_nodes, "multi_bind")


def run_DTCSpMM_balance(dense, row_window_offset, tcblocktile_id, tcblock_offset, sparse_a_to_x_idx, num_nodes, exeplan):
    return _run(dense, row_window_offset, tcblocktile_id, tcblock_offset, sparse_a_to_x_idx, num_nodes)


def run_DTCSpMM_strict_lb_balance(dense, row_window_offset, tcblocktile_id, tcblock_offset, sparse_a_to_x_idx, num_nodes,
                                  exeplan):
    return _run(dense, row_window_offset, tcblocktile_id, tcblock_offset, sparse_a_to_x_idx, num_nodes, "strict_lb")


def run_DTCSpMM_multi_binding_balance(dense, row_window_offset, tcblocktile_id, tcblock_offset, sparse_a_to_x_idx,
                                      num_nodes, exeplan):
    return _run(dense, row_window_offset, tcblocktile_id, tcblock_offset, sparse_a_to_x_idx, num_nodes, "multi_bind")


def DTCSpMM_gcn(dense, row_window_offset, tcblocktile_id, tcblock_offset, sparse_a_to_x_idx, num_nodes, num_edges):
    """Variant without the exeplan string that the reference router also accepts
    (end2end/gcn/external_backend_spmm.py:442-451)."""
    return _run(dense, row_window_offset, tcblocktile_id, tcblock_offset, sparse_a_to_x_idx, num_nodes)


def reset_cache():
    _cache.clear()
