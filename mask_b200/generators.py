"""Seeded synthetic workloads with the shapes and value distributions of the five benchmark
configurations (uniform-random, R-MAT power-law graph, 27-point stencil, large R-MAT for the
row-sharded sweep, GCN adjacency).

The reference project evaluates on 26 SuiteSparse / GNN matrices that are not distributed with
it (``dataset/matrices.tar.gz`` is a git-LFS pointer); these generators stand in for them.  All
matrices come back as CSR with int32 indices, rows sorted strictly ascending (deduplicated),
float32 values -- the input contract of the packers.  Everything is NumPy on the host and fully
determined by the seed, so every rank of a multi-GPU run can rebuild the same matrix.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


@dataclass
class CSR:
    """Compressed sparse rows: ``rowptr`` int32[M+1], ``colind`` int32[nnz], ``values`` f32[nnz]."""

    M: int
    K: int
    rowptr: np.ndarray
    colind: np.ndarray
    values: np.ndarray

    @property
    def nnz(self) -> int:
        return int(self.colind.shape[0])

    def row_slice(self, r0: int, r1: int) -> "CSR":
        """Rows [r0, r1) as their own CSR (global column ids kept)."""
        s, e = int(self.rowptr[r0]), int(self.rowptr[r1])
        return CSR(r1 - r0, self.K, (self.rowptr[r0:r1 + 1] - s).astype(np.int32),
                   self.colind[s:e], self.values[s:e])


def _csr_from_sorted_keys(keys: np.ndarray, n: int, k: int) -> tuple[np.ndarray, np.ndarray]:
    rows = keys // k
    colind = (keys - rows * k).astype(np.int32)
    counts = np.bincount(rows, minlength=n)
    rowptr = np.zeros(n + 1, dtype=np.int64)
    np.cumsum(counts, out=rowptr[1:])
    assert rowptr[-1] < 2**31, "nnz must fit int32"
    return rowptr.astype(np.int32), colind


def _splitmix64(x: np.ndarray) -> np.ndarray:
    x = (x + np.uint64(0x9E3779B97F4A7C15)).astype(np.uint64)
    x = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    x = (x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return x ^ (x >> np.uint64(31))


def uniform_random(n: int = 4096, density: float = 0.005, seed: int = 101) -> CSR:
    """Bernoulli(density) pattern plus a unit diagonal; off-diagonal values U(-1,1)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    target = int(round(density * n * n))
    # sample with replacement then deduplicate: the count lands within a fraction of a percent
    keys = rng.integers(0, n * n, size=target, dtype=np.int64)
    diag = np.arange(n, dtype=np.int64) * (n + 1)
    keys = np.unique(np.concatenate([keys, diag]))
    rowptr, colind = _csr_from_sorted_keys(keys, n, n)
    values = rng.uniform(-1.0, 1.0, size=keys.shape[0]).astype(np.float32)
    rows = (keys // n).astype(np.int32)
    values[rows == colind] = 1.0
    return CSR(n, n, rowptr, colind, values)


def _rmat_edges(scale: int, n_samples: int, seed: int, a=0.57, b=0.19, c=0.19) -> tuple[np.ndarray, np.ndarray]:
    """R-MAT: one quadrant draw per bit, no noise.  Returns int64 (src, dst) samples."""
    rng = np.random.Generator(np.random.PCG64(seed))
    src = np.zeros(n_samples, dtype=np.int64)
    dst = np.zeros(n_samples, dtype=np.int64)
    ab, abc = np.float32(a + b), np.float32(a + b + c)
    for _ in range(scale):
        r = rng.random(n_samples, dtype=np.float32)
        row_bit = r >= ab
        col_bit = ((r >= np.float32(a)) & (r < ab)) | (r >= abc)
        src = (src << 1) | row_bit
        dst = (dst << 1) | col_bit
    return src, dst


def _symmetric_rmat_keys(scale: int, samples_per_node: int, seed: int, self_loops: bool) -> np.ndarray:
    n = 1 << scale
    src, dst = _rmat_edges(scale, samples_per_node * n, seed)
    parts = [src * n + dst, dst * n + src]
    if self_loops:
        parts.append(np.arange(n, dtype=np.int64) * (n + 1))
    return np.unique(np.concatenate(parts))


def rmat_gcn_normalised(scale: int = 20, samples_per_node: int = 8, seed: int = 201) -> CSR:
    """Symmetric R-MAT adjacency (a=.57,b=.19,c=.19,d=.05) with self-loops, deduplicated, values
    1/sqrt(deg_i * deg_j) where deg is the stored row length."""
    n = 1 << scale
    keys = _symmetric_rmat_keys(scale, samples_per_node, seed, self_loops=True)
    rowptr, colind = _csr_from_sorted_keys(keys, n, n)
    deg = np.diff(rowptr).astype(np.float64)
    rows = np.repeat(np.arange(n, dtype=np.int64), np.diff(rowptr))
    values = (1.0 / np.sqrt(deg[rows] * deg[colind])).astype(np.float32)
    return CSR(n, n, rowptr, colind, values)


def rmat_symmetric_uniform(scale: int = 22, samples_per_node: int = 16, seed: int = 401) -> CSR:
    """Symmetric R-MAT, values U(-1,1) drawn once per undirected edge (so A == A^T)."""
    n = 1 << scale
    keys = _symmetric_rmat_keys(scale, samples_per_node, seed, self_loops=False)
    rowptr, colind = _csr_from_sorted_keys(keys, n, n)
    rows = keys // n
    cols = keys - rows * n
    canon = (np.minimum(rows, cols) * n + np.maximum(rows, cols)).astype(np.uint64)
    h = _splitmix64(canon ^ np.uint64(seed))
    values = ((h >> np.uint64(40)).astype(np.float64) / float(1 << 24) * 2.0 - 1.0).astype(np.float32)
    return CSR(n, n, rowptr, colind, values)


def stencil27(grid: int = 100, seed: int = 301) -> CSR:
    """27-point stencil on a grid^3 lattice truncated at the boundary; off-diagonals U(0.5,1.5),
    diagonal 27."""
    g = grid
    n = g * g * g
    idx = np.arange(n, dtype=np.int64)
    z, y, x = idx // (g * g), (idx // g) % g, idx % g
    cols = np.empty((n, 27), dtype=np.int32)
    valid = np.empty((n, 27), dtype=bool)
    j = 0
    for dz in (-1, 0, 1):
        for dy in (-1, 0, 1):
            for dx in (-1, 0, 1):
                zz, yy, xx = z + dz, y + dy, x + dx
                ok = (zz >= 0) & (zz < g) & (yy >= 0) & (yy < g) & (xx >= 0) & (xx < g)
                cols[:, j] = (zz * g * g + yy * g + xx).astype(np.int32)
                valid[:, j] = ok
                j += 1
    counts = valid.sum(axis=1)
    rowptr = np.zeros(n + 1, dtype=np.int64)
    np.cumsum(counts, out=rowptr[1:])
    colind = cols[valid]
    rng = np.random.Generator(np.random.PCG64(seed))
    values = rng.uniform(0.5, 1.5, size=colind.shape[0]).astype(np.float32)
    rows = np.repeat(np.arange(n, dtype=np.int32), counts)
    values[rows == colind] = 27.0
    return CSR(n, n, rowptr.astype(np.int32), colind, values)


def dense_normal(rows: int, cols: int, seed: int) -> np.ndarray:
    """Dense operand B: float32 N(0,1), row-major."""
    rng = np.random.Generator(np.random.PCG64(seed))
    return rng.standard_normal((rows, cols), dtype=np.float32)


def glorot_uniform(fan_in: int, fan_out: int, seed: int) -> np.ndarray:
    rng = np.random.Generator(np.random.PCG64(seed))
    lim = float(np.sqrt(6.0 / (fan_in + fan_out)))
    return rng.uniform(-lim, lim, size=(fan_in, fan_out)).astype(np.float32)


WORKLOADS = {
    # name: (builder, full-size kwargs, dense-operand seed)
    "uniform4096": (uniform_random, dict(n=4096, density=0.005, seed=101), 102),
    "rmat20_gcn": (rmat_gcn_normalised, dict(scale=20, samples_per_node=8, seed=201), 202),
    "stencil27_100": (stencil27, dict(grid=100, seed=301), 302),
    "rmat22_sym": (rmat_symmetric_uniform, dict(scale=22, samples_per_node=16, seed=401), 402),
    "rmat21_gcn": (rmat_gcn_normalised, dict(scale=21, samples_per_node=10, seed=501), 502),
}


def make_workload(name: str, **overrides) -> tuple[CSR, int]:
    """Builds a named workload (optionally scaled down through keyword overrides such as
    ``scale=12`` or ``grid=20``); returns the matrix and the seed for its dense operand."""
    builder, kwargs, bseed = WORKLOADS[name]
    kw = dict(kwargs)
    kw.update(overrides)
    return builder(**kw), bseed


def check_csr(csr: CSR) -> None:
    """Asserts the packer input contract: monotone rowptr, in-range strictly ascending columns."""
    rp, ci = csr.rowptr.astype(np.int64), csr.colind
    assert rp[0] == 0 and rp[-1] == ci.shape[0] and np.all(np.diff(rp) >= 0)
    assert ci.size == 0 or (ci.min() >= 0 and ci.max() < csr.K)
    if ci.size > 1:
        asc = np.diff(ci.astype(np.int64)) > 0
        row_start = np.zeros(ci.shape[0], dtype=bool)
        row_start[rp[1:-1][rp[1:-1] < ci.shape[0]]] = True
        assert np.all(asc | row_start[1:]), "rows must be strictly ascending"


def write_matrix_market(csr: CSR, path: str) -> None:
    """Writes the sparsity pattern as a MatrixMarket ``coordinate pattern general`` file (1-based,
    row-major order): the input format of the reference's testbeds and of its Format-DSL host
    bridge, which assign their own deterministic values to the entries."""
    rows = np.repeat(np.arange(csr.M, dtype=np.int64), np.diff(csr.rowptr)) + 1
    cols = csr.colind.astype(np.int64) + 1
    with open(path, "w") as f:
        f.write("%%MatrixMarket matrix coordinate pattern general\n")
        f.write(f"{csr.M} {csr.K} {csr.nnz}\n")
        np.savetxt(f, np.stack([rows, cols], axis=1), fmt="%d")
