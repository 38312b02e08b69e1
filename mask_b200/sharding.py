"""Row-panel partitioning of A for multi-GPU SpMM.

Output rows are independent, so with the dense operand replicated a product needs no exchange:
rank p multiplies rows [b_p, b_{p+1}) and keeps that panel of C.  Panels start on 16-row window
boundaries (so every rank packs whole windows and the concatenation of the per-rank formats'
windows is the single-GPU window sequence) and are cut where the running count of stored entries
crosses equal shares.  The reference project is single-GPU; this module is new.
"""
from __future__ import annotations

import numpy as np

WIN = 16


def balanced_panels(win_prefix: np.ndarray, M: int, parts: int) -> list[int]:
    """Boundaries b_0=0 <= b_1 <= ... <= b_parts=M, each a multiple of 16 (except M), cutting the
    per-window cost whose exclusive prefix sum is ``win_prefix`` (W+1 entries) into equal shares.
    With val_soff as the prefix the panels hold equal numbers of 16x8 tiles, which is what the
    SpMM kernel's time follows."""
    W = (M + WIN - 1) // WIN
    assert parts >= 1 and win_prefix.shape[0] == W + 1
    win_rows = np.minimum(np.arange(W + 1, dtype=np.int64) * WIN, M)
    win_nnz = np.asarray(win_prefix).astype(np.int64)
    nnz = int(win_nnz[W])
    bounds = [0]
    for p in range(1, parts):
        target = (nnz * p) // parts
        w = int(np.searchsorted(win_nnz, target, side="left"))
        # the boundary whose prefix is closest to the target
        if w > 0 and w <= W and abs(int(win_nnz[w - 1]) - target) < abs(int(win_nnz[min(w, W)]) - target):
            w -= 1
        w = min(max(w, bounds[-1] // WIN if bounds[-1] % WIN == 0 else W), W)
        bounds.append(int(win_rows[w]))
    bounds.append(M)
    for a, b in zip(bounds, bounds[1:]):
        assert a <= b
    return bounds


# A window costs its tiles plus a fixed part for the 16 rows of C it writes.  Fitted on the
# 2^20-node power-law graph at N = 512 over 8 GPUs with equal tile counts per rank: per-rank time
# 0.393 ms (8.7 k rows) ... 0.570 ms (392 k rows) = 1.58e-6 ms per tile + 4.6e-7 ms per row, i.e. one
# window of 16 rows weighs about as much as 4.7 tiles.
WINDOW_OVERHEAD_TILES = 5


def spmm_cost_prefix(val_soff: np.ndarray, window_overhead_tiles: int = WINDOW_OVERHEAD_TILES) -> np.ndarray:
    """Exclusive prefix of the per-window SpMM cost model (tiles + a fixed share per window)."""
    soff = np.asarray(val_soff).astype(np.int64)
    return soff + window_overhead_tiles * np.arange(soff.shape[0], dtype=np.int64)


def minimax_panels(win_prefix: np.ndarray, M: int, parts: int, row_cost: float) -> list[int]:
    """Boundaries on window boundaries that minimise the largest panel cost when a panel costs
    ``max(its share of win_prefix, row_cost * its rows)`` -- two resources used at the same time,
    e.g. the tiles a rank multiplies and the finished rows it stores into its peers' memory while
    it multiplies.  Found by bisection on the bound with a greedy feasibility walk (each panel is
    extended as far as the bound allows, which is optimal for contiguous panels)."""
    W = (M + WIN - 1) // WIN
    pref = np.asarray(win_prefix).astype(np.int64)
    assert parts >= 1 and pref.shape[0] == W + 1 and row_cost >= 0
    win_rows = np.minimum(np.arange(W + 1, dtype=np.int64) * WIN, M)

    def walk(bound: float):
        """Window indices of the boundaries under `bound`, or None when `parts` panels do not suffice."""
        cuts, w = [0], 0
        for _ in range(parts):
            if w == W:
                cuts.append(W)
                continue
            by_tiles = int(np.searchsorted(pref, pref[w] + bound, side="right")) - 1
            by_rows = int(np.searchsorted(win_rows, win_rows[w] + (bound / row_cost if row_cost > 0 else M), side="right")) - 1
            nxt = min(by_tiles, by_rows, W)
            if nxt <= w:
                return None   # a single window exceeds the bound
            cuts.append(nxt)
            w = nxt
        return cuts if w == W else None

    lo, hi = 0.0, float(max(int(pref[W]), row_cost * M, 1))
    best = walk(hi)
    assert best is not None
    for _ in range(48):
        mid = 0.5 * (lo + hi)
        got = walk(mid)
        if got is None:
            lo = mid
        else:
            hi, best = mid, got
        if hi - lo <= 1e-3 * hi:
            break
    return [int(win_rows[w]) for w in best]


def panel_costs(win_prefix: np.ndarray, M: int, bounds: list[int], row_cost: float) -> list[float]:
    """``max(share of win_prefix, row_cost * rows)`` of every panel of `bounds`."""
    pref = np.asarray(win_prefix).astype(np.int64)
    out = []
    for a, b in zip(bounds, bounds[1:]):
        wa, wb = a // WIN, (b + WIN - 1) // WIN
        out.append(max(float(pref[wb] - pref[wa]), row_cost * (b - a)))
    return out


# What storing one finished row of H into one peer costs, in tiles of SpMM work at the same width:
# a row of N floats over a link that moves ~700 GB/s of 128-byte stores, against ~1.7 ns per tile at
# N = 512 (both scale with N, so the ratio does not).
PEER_ROW_COST_TILES = 1.72


def rebalanced_panels(win_prefix: np.ndarray, M: int, bounds: list[int], seconds: list[float]) -> list[int]:
    """Re-cuts panels from measured times.  The cost model behind `win_prefix` cannot see what the
    memory system does with a panel (on a power-law graph the hub rows at the top gather rows of B
    with little reuse, the sparse rows at the bottom mostly gather hub columns that stay in L2), so
    after one timed product per rank the model's cost inside old panel r is scaled by
    seconds[r] / (model cost of panel r) and the scaled cost is cut into equal shares.  Every rank
    must pass the same `seconds` (all-gathered) to get the same boundaries."""
    W = (M + WIN - 1) // WIN
    pref = np.asarray(win_prefix).astype(np.float64)
    parts = len(bounds) - 1
    assert pref.shape[0] == W + 1 and len(seconds) == parts and bounds[0] == 0 and bounds[-1] == M
    wb = [min((b + WIN - 1) // WIN, W) for b in bounds]
    scaled = np.zeros(W + 1, dtype=np.float64)
    for r in range(parts):
        a, b = wb[r], wb[r + 1]
        if b <= a:
            continue
        seg = pref[a:b + 1] - pref[a]
        share = float(seg[-1])
        # a panel without model cost: spread its time over its windows
        seg = seg * (float(seconds[r]) / share) if share > 0 else np.linspace(0.0, float(seconds[r]), b - a + 1)
        scaled[a + 1:b + 1] = scaled[a] + seg[1:]
    total = float(scaled[W])
    if total <= 0:
        return list(bounds)
    as_int = np.round(scaled / total * float(1 << 40)).astype(np.int64)
    return balanced_panels(np.maximum.accumulate(as_int), M, parts)


def nnz_balanced_panels(rowptr: np.ndarray, M: int, parts: int) -> list[int]:
    """Panels holding equal numbers of stored entries."""
    assert rowptr.shape[0] == M + 1
    W = (M + WIN - 1) // WIN
    win_rows = np.minimum(np.arange(W + 1, dtype=np.int64) * WIN, M)
    return balanced_panels(rowptr[win_rows], M, parts)


def panel_of(bounds: list[int], rank: int) -> tuple[int, int]:
    return bounds[rank], bounds[rank + 1]
