"""Generates tests/golden/*.npz from the REFERENCE project's own host packers and planners.

Run in a container that holds a checkout of the reference project (its path in $MASK_REF):

    make -C oracle ref          # builds oracle/_ref/*.so from the reference sources
    python tests/golden/make_golden.py

Each fixture stores a small CSR matrix together with what the reference code produced for it:
SR-BCRS 16x8 arrays (convertToSRBCRS), ME-TCF arrays (buildMETCFMetadata), the strict_lb tables
for a group size of 64 and of 8 tiles, the multi_bind tables, and the row orders of the Format-DSL
bridge's reorders (first_col_sort, jaccard_greedy; row_rcm for square matrices).  The fixtures travel with the
repository; the reference checkout does not.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import oracle  # noqa: E402
from mask_b200 import generators as G  # noqa: E402


def ragged(seed, M, K, dens, empty_rows=(), heavy_row=None):
    """Random CSR with chosen empty rows and optionally one dense row."""
    rng = np.random.Generator(np.random.PCG64(seed))
    rows = []
    for r in range(M):
        if r in empty_rows:
            cols = np.zeros(0, dtype=np.int32)
        elif heavy_row is not None and r == heavy_row:
            cols = np.arange(K, dtype=np.int32)
        else:
            cols = np.flatnonzero(rng.random(K) < dens).astype(np.int32)
        rows.append(cols)
    rowptr = np.zeros(M + 1, dtype=np.int32)
    rowptr[1:] = np.cumsum([len(c) for c in rows])
    colind = np.concatenate(rows).astype(np.int32) if rowptr[-1] else np.zeros(0, dtype=np.int32)
    values = rng.uniform(-1, 1, size=colind.shape[0]).astype(np.float32)
    return G.CSR(M, K, rowptr, colind, values)


CASES = {
    "rmat8_gcn": lambda: G.rmat_gcn_normalised(scale=8, samples_per_node=8, seed=201),
    "uniform300": lambda: G.uniform_random(n=300, density=0.02, seed=101),
    "stencil5": lambda: G.stencil27(grid=5, seed=301),
    "ragged37": lambda: ragged(7, 37, 90, 0.08, empty_rows=set(range(16, 32)) | {3, 36}),
    "heavy50": lambda: ragged(8, 50, 700, 0.01, empty_rows={0}, heavy_row=20),
    "single_row": lambda: ragged(9, 1, 40, 0.3),
    "m17": lambda: ragged(10, 17, 64, 0.2),
}


def main():
    assert oracle.ref_available(), "build oracle/_ref first: make -C oracle ref"
    for name, make in CASES.items():
        m = make()
        G.check_csr(m)
        sr = oracle.ref_pack_srbcrs(m.M, m.K, m.rowptr, m.colind, m.values)
        me = oracle.ref_pack_metcf(m.M, m.K, m.rowptr, m.colind, m.values)
        out = dict(M=m.M, K=m.K, rowptr=m.rowptr, colind=m.colind, values=m.values,
                   sr_val_soff=sr["val_soff"], sr_val_sidx=sr["val_sidx"], sr_val_block_val=sr["val_block_val"],
                   me_val_soff=me["val_soff"], me_val_sidx=me["val_sidx"], me_val_coo_off=me["val_coo_off"],
                   me_val_coo_idx=me["val_coo_idx"], me_val_coo_val=me["val_coo_val"])
        mc = oracle.ref_pack_mco(m.M, m.K, m.rowptr, m.colind, m.values)
        out.update(mco_val_soff=mc["val_soff"], mco_val_sidx=mc["val_sidx"], mco_val_mco_off=mc["val_mco_off"],
                   mco_val_mco_mask=mc["val_mco_mask"], mco_val_mco_val=mc["val_mco_val"])
        for wl in (64, 8):
            rbo, rb2w, go = oracle.ref_strict_lb_plan(m.M, sr["val_soff"], wl)
            out[f"slb{wl}_row_block_offset"] = rbo
            out[f"slb{wl}_row_block_to_window"] = rb2w
            out[f"slb{wl}_group_offset"] = go
        for kind in ("first_col_sort", "jaccard_greedy") + (("row_rcm",) if m.M == m.K else ()):
            out["order_" + kind] = oracle.ref_reorder_rows(kind, m.M, m.K, m.rowptr, m.colind)
        tw, ws, ts = oracle.ref_multi_bind_plan(m.M, sr["val_soff"])
        out.update(mb_task_window=tw, mb_window_split=ws, mb_task_soff=ts)
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **out)
        print(f"{name}: M={m.M} K={m.K} nnz={m.nnz} T={sr['T']} nnz_pad={me['nnz_pad']} -> {os.path.getsize(path)} bytes")


if __name__ == "__main__":
    main()
