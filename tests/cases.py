"""Shared matrices for the parity tests (seeded, small enough for the CPU oracle)."""
import glob
import os

import numpy as np

from mask_b200 import generators as G

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def golden_names():
    return sorted(os.path.splitext(os.path.basename(p))[0] for p in glob.glob(os.path.join(GOLDEN_DIR, "*.npz")))


def load_golden(name):
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    d = {k: z[k] for k in z.files}
    csr = G.CSR(int(d["M"]), int(d["K"]), d["rowptr"], d["colind"], d["values"])
    return csr, d


def random_csr(seed, M, K, dens, empty_rows=(), heavy_rows=()):
    rng = np.random.Generator(np.random.PCG64(seed))
    rows = []
    for r in range(M):
        if r in empty_rows:
            cols = np.zeros(0, dtype=np.int32)
        elif r in heavy_rows:
            cols = np.flatnonzero(rng.random(K) < 0.7).astype(np.int32)
        else:
            cols = np.flatnonzero(rng.random(K) < dens).astype(np.int32)
        rows.append(cols)
    rowptr = np.zeros(M + 1, dtype=np.int32)
    rowptr[1:] = np.cumsum([len(c) for c in rows])
    colind = np.concatenate(rows).astype(np.int32) if rowptr[-1] else np.zeros(0, dtype=np.int32)
    values = rng.uniform(-1, 1, size=colind.shape[0]).astype(np.float32)
    return G.CSR(M, K, rowptr, colind, values)


# name -> builder; sizes the oracle finishes in well under a second each
SMALL = {
    "m1": lambda: random_csr(1, 1, 33, 0.3),
    "m15": lambda: random_csr(2, 15, 40, 0.2),
    "m16": lambda: random_csr(3, 16, 40, 0.2),
    "m17": lambda: random_csr(4, 17, 40, 0.2),
    "m33_empty_window": lambda: random_csr(5, 33, 100, 0.1, empty_rows=set(range(16, 32))),
    "all_empty": lambda: random_csr(6, 40, 50, 0.0, empty_rows=set(range(40))),
    "one_tile_windows": lambda: random_csr(7, 64, 8, 0.5),
    "three_four_tiles": lambda: random_csr(8, 96, 30, 0.12),
    "hub_rows": lambda: random_csr(9, 200, 3000, 0.002, heavy_rows={5, 77}),
    "uniform512": lambda: G.uniform_random(n=512, density=0.02, seed=11),
    "rmat10": lambda: G.rmat_gcn_normalised(scale=10, samples_per_node=8, seed=201),
    "rmat12u": lambda: G.rmat_symmetric_uniform(scale=12, samples_per_node=16, seed=401),
    "stencil8": lambda: G.stencil27(grid=8, seed=301),
    "wide_k": lambda: random_csr(12, 48, 100000, 0.0002),
}
