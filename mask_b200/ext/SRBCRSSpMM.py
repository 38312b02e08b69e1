"""Drop-in for the reference project's ``SRBCRSSpMM`` torch extension
(examples/src_fp32/sr_bcrs/testbed/SRBCRSSpMM.cpp:194-204): same function names, argument order,
tuple shapes and error type, served by the B200 library.

Put this directory on the module search path of the reference's router
(``SPARSENE_SRBCRS_MODULE_PATH=<repo>/mask_b200/ext SPARSENE_SRBCRS_ALLOW_NON_SRC_FP32=1``,
end2end/gcn/external_backend_spmm.py:569-601) and select the 16x8 variant
(``SPARSENE_SRBCRS_VARIANT=16x8``).  Packing runs on the device; the tile-width switches
SRBCRS_TILE_B of the reference have no effect (any N that is a multiple of 4 is accepted).
"""
from __future__ import annotations

import torch

from _common import Cache, check_input, engine, fill_side_outputs, pack_without_sync, run

_cache = Cache()
_BASE_MSG = ("the 32x32 SR-BCRS variant is not built in this library: select the 16x8 variant "
             "(SPARSENE_SRBCRS_VARIANT=16x8, blk_h=16, blk_w=8)")


def _preprocess(colind, rowptr, values, num_nodes, blk_h, blk_w, block_partition, edge_to_col, edge_to_row, policy):
    for t, n, dt in ((colind, "colind", torch.int32), (rowptr, "rowptr", torch.int32), (values, "values", torch.float32),
                     (block_partition, "block_partition", None), (edge_to_col, "edge_to_col", None),
                     (edge_to_row, "edge_to_row", None)):
        check_input(t, n, dt)
    if int(num_nodes) < 1:
        raise RuntimeError("num_nodes must be positive")
    if int(blk_h) != 16:
        raise RuntimeError(f"blk_h mismatch for SR-BCRS variant: expected 16 got {blk_h}")
    if int(blk_w) != 8:
        raise RuntimeError(f"blk_w mismatch for SR-BCRS variant: expected 8 got {blk_w}")
    if values.numel() != colind.numel():
        raise RuntimeError("values length must equal colind length")
    num_nodes = int(num_nodes)
    packed = pack_without_sync(lambda rp, ci, va, M, K: engine.pack_srbcrs(rp, ci, va, M, K, side_outputs=True),
                               rowptr, colind, num_nodes, values)
    fill_side_outputs((packed.block_partition, packed.edge_to_col, packed.edge_to_row), block_partition, edge_to_col,
                      edge_to_row)
    dev = rowptr.device
    zeros1 = torch.zeros(1, dtype=torch.int32, device=dev)
    _cache.put(packed.val_soff, packed, policy)
    # (row_window_offset, tcblock_rowid, tcblocktile_id, tcblock_offset, sparse_a_to_x_idx, T)
    return (packed.val_soff, torch.zeros(packed.T, dtype=torch.int32, device=dev), packed.val_sidx, zeros1,
            torch.zeros(1, dtype=torch.int32, device=dev), packed.T)


def preprocess_gpu(*args, **kwargs):
    raise RuntimeError(_BASE_MSG)


def preprocess_gpu_16x8(colind, rowptr, values, num_nodes, blk_h, blk_w, block_partition, edge_to_col, edge_to_row):
    return _preprocess(colind, rowptr, values, num_nodes, blk_h, blk_w, block_partition, edge_to_col, edge_to_row, "auto")


def preprocess_gpu_16x8_strict_lb(colind, rowptr, values, num_nodes, blk_h, blk_w, block_partition, edge_to_col,
                                  edge_to_row):
    return _preprocess(colind, rowptr, values, num_nodes, blk_h, blk_w, block_partition, edge_to_col, edge_to_row,
                       "strict_lb")


def preprocess_gpu_16x8_multi_binding(colind, rowptr, values, num_nodes, blk_h, blk_w, block_partition, edge_to_col,
                                      edge_to_row):
    return _preprocess(colind, rowptr, values, num_nodes, blk_h, blk_w, block_partition, edge_to_col, edge_to_row,
                       "multi_bind")


def run_SRBCRS(*args, **kwargs):
    raise RuntimeError(_BASE_MSG)


run_SRBCRS_balance = run_SRBCRS


def _check_handles(tcblocktile_id, tcblock_offset, sparse_a_to_x_idx):
    check_input(tcblocktile_id, "tcblocktile_id")
    check_input(tcblock_offset, "tcblock_offset")
    check_input(sparse_a_to_x_idx, "sparse_a_to_x_idx")


def run_SRBCRS_16x8(dense, row_window_offset, tcblocktile_id, tcblock_offset, sparse_a_to_x_idx, num_nodes, num_edges,
                    exeplan):
    _check_handles(tcblocktile_id, tcblock_offset, sparse_a_to_x_idx)
    return run(_cache, dense, row_window_offset, num_nodes)


def run_SRBCRS_16x8_balance(dense, row_window_offset, tcblocktile_id, tcblock_offset, sparse_a_to_x_idx, num_nodes,
                            exeplan):
    _check_handles(tcblocktile_id, tcblock_offset, sparse_a_to_x_idx)
    return run(_cache, dense, row_window_offset, num_nodes)


def run_SRBCRS_16x8_strict_lb(dense, row_window_offset, tcblocktile_id, tcblock_offset, sparse_a_to_x_idx, num_nodes,
                              num_edges, exeplan):
    _check_handles(tcblocktile_id, tcblock_offset, sparse_a_to_x_idx)
    return run(_cache, dense, row_window_offset, num_nodes, "strict_lb")


def run_SRBCRS_16x8_multi_binding(dense, row_window_offset, tcblocktile_id, tcblock_offset, sparse_a_to_x_idx, num_nodes,
                                  num_edges, exeplan):
    _check_handles(tcblocktile_id, tcblock_offset, sparse_a_to_x_idx)
    return run(_cache, dense, row_window_offset, num_nodes, "multi_bind")


# The router's balance call (SPARSENE_SRBCRS_BALANCE=1) passes no num_edges and looks for these
# spellings first (end2end/gcn/external_backend_spmm.py:737-763); without them it would pick the
# eight-argument functions above and fail on the argument count.
def run_SRBCRS_16x8_strict_lb_balance(dense, row_window_offset, tcblocktile_id, tcblock_offset, sparse_a_to_x_idx, num_nodes,
                                      exeplan):
    _check_handles(tcblocktile_id, tcblock_offset, sparse_a_to_x_idx)
    return run(_cache, dense, row_window_offset, num_nodes, "strict_lb")


def run_SRBCRS_16x8_multi_binding_balance(dense, row_window_offset, tcblocktile_id, tcblock_offset, sparse_a_to_x_idx,
                                          num_nodes, exeplan):
    _check_handles(tcblocktile_id, tcblock_offset, sparse_a_to_x_idx)
    return run(_cache, dense, row_window_offset, num_nodes, "multi_bind")


def reset_cache():
    _cache.clear()
