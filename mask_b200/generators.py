"""Seeded synthetic workloads with the shapes and value distributions of the five benchmark
configurations (uniform-random, R-MAT power-law graph, 27-point stencil, large R-MAT for the
row-sharded sweep, GCN adjacency).

The reference project evaluates on 26 SuiteSparse / GNN matrices that are not distributed with
it (``dataset/matrices.tar.gz`` is a git-LFS pointer); these generators stand in for them.  All
matrices come back as CSR with int32 indices, rows sorted strictly ascending (deduplicated),
float32 values -- the input contract of the packers.  Every random draw is NumPy on the host and
the result is fully determined by the seed, so every rank of a multi-GPU run gets the same matrix.
The heavy integer passes of the large R-MAT graphs (bit assembly, sort + deduplication, the value
hash) run on the GPU when one is visible -- they are exact, so the matrix is bit-identical either
way -- and ``make_workload_cached`` keeps finished matrices in a temporary directory so that the
ranks of one job, and the jobs that follow on the same machine, build each matrix once.
"""
from __future__ import annotations

import os
import tempfile
import time
from dataclasses import dataclass

import numpy as np


GPU_MIN_ITEMS = 1 << 22   # below this many samples / entries the host does everything


def _cuda(items: int = 1 << 62):
    """torch, if a CUDA device can take the exact integer passes of the big generators."""
    if items < GPU_MIN_ITEMS:
        return None
    try:
        import torch
        return torch if torch.cuda.is_available() else None
    except Exception:
        return None


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
    if k & (k - 1) == 0:
        sh = k.bit_length() - 1
        rows = keys >> sh
        colind = (keys & (k - 1)).astype(np.int32)
    else:
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


def _rmat_edges(scale: int, n_samples: int, seed: int, a=0.57, b=0.19, c=0.19):
    """R-MAT: one quadrant draw per bit, no noise.  Returns int64 (src, dst) samples (NumPy arrays,
    or CUDA tensors when a GPU does the bit assembly)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    ab, abc = np.float32(a + b), np.float32(a + b + c)
    torch = _cuda(n_samples)
    if torch is not None:
        src = torch.zeros(n_samples, dtype=torch.int64, device="cuda")
        dst = torch.zeros(n_samples, dtype=torch.int64, device="cuda")
        for _ in range(scale):
            r = torch.from_numpy(rng.random(n_samples, dtype=np.float32)).cuda()
            row_bit = r >= float(ab)
            col_bit = ((r >= float(np.float32(a))) & (r < float(ab))) | (r >= float(abc))
            src = (src << 1) | row_bit
            dst = (dst << 1) | col_bit
        return src, dst
    src = np.zeros(n_samples, dtype=np.int64)
    dst = np.zeros(n_samples, dtype=np.int64)
    for _ in range(scale):
        r = rng.random(n_samples, dtype=np.float32)
        row_bit = r >= ab
        col_bit = ((r >= np.float32(a)) & (r < ab)) | (r >= abc)
        src = (src << 1) | row_bit
        dst = (dst << 1) | col_bit
    return src, dst


def _symmetric_rmat_keys(scale: int, samples_per_node: int, seed: int, self_loops: bool) -> np.ndarray:
    """Sorted, deduplicated keys row * n + col of the symmetrised sample set."""
    n = 1 << scale
    src, dst = _rmat_edges(scale, samples_per_node * n, seed)
    if not isinstance(src, np.ndarray):   # CUDA tensors: sort + deduplicate there
        import torch
        parts = [src * n + dst, dst * n + src]
        del src, dst
        if self_loops:
            parts.append(torch.arange(n, dtype=torch.int64, device="cuda") * (n + 1))
        keys = torch.unique(torch.cat(parts))
        del parts
        out = keys.cpu().numpy()
        del keys
        torch.cuda.empty_cache()
        return out
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
    torch = _cuda(keys.shape[0])
    if torch is not None:   # the same 64-bit hash in two's-complement int64 (logical shifts by masking)
        k = torch.from_numpy(keys).cuda()
        rows = k >> scale
        cols = k & (n - 1)
        x = (torch.minimum(rows, cols) * n + torch.maximum(rows, cols)) ^ seed
        del k, rows, cols

        def i64(v):
            return v - (1 << 64) if v >= (1 << 63) else v

        x = x + i64(0x9E3779B97F4A7C15)
        x = (x ^ ((x >> 30) & ((1 << 34) - 1))) * i64(0xBF58476D1CE4E5B9)
        x = (x ^ ((x >> 27) & ((1 << 37) - 1))) * i64(0x94D049BB133111EB)
        x = x ^ ((x >> 31) & ((1 << 33) - 1))
        values = (((x >> 40) & ((1 << 24) - 1)).to(torch.float64) / float(1 << 24) * 2.0 - 1.0).to(torch.float32).cpu().numpy()
        del x
        torch.cuda.empty_cache()
        return CSR(n, n, rowptr, colind, values)
    rows = keys >> scale
    cols = keys & (n - 1)
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


def dense_normal_blocks(rows: int, cols: int, seed: int, threads: int, block_rows: int = 1 << 16) -> np.ndarray:
    """N(0,1) float32 like ``dense_normal`` but drawn by ``threads`` workers, every block of rows
    from its own PCG64 stream spawned from the seed (so the values differ from ``dense_normal``'s
    single stream).  For operands of several GiB where only the distribution matters."""
    from concurrent.futures import ThreadPoolExecutor
    out = np.empty((rows, cols), dtype=np.float32)
    starts = list(range(0, rows, block_rows))
    seqs = np.random.SeedSequence(seed).spawn(len(starts))

    def fill(i):
        r0 = starts[i]
        r1 = min(rows, r0 + block_rows)
        np.random.Generator(np.random.PCG64(seqs[i])).standard_normal((r1 - r0, cols), dtype=np.float32, out=out[r0:r1])

    with ThreadPoolExecutor(max_workers=max(1, threads)) as ex:
        list(ex.map(fill, range(len(starts))))
    return out


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


def make_workload_cached(name: str, cache_dir: str | None = None, wait_s: float = 900.0, **overrides) -> tuple[CSR, int]:
    """``make_workload`` through a file cache (``$MASK_B200_CACHE`` or a folder in the system's
    temporary directory): the first caller builds and saves the matrix, concurrent callers (the
    other ranks of a job) wait for the file, later callers load it."""
    builder, kwargs, bseed = WORKLOADS[name]
    kw = dict(kwargs)
    kw.update(overrides)
    root = cache_dir or os.environ.get("MASK_B200_CACHE") or os.path.join(tempfile.gettempdir(), "mask_b200_workloads")
    os.makedirs(root, exist_ok=True)
    tag = name + "".join(f"_{k}{v}" for k, v in sorted(kw.items())) + "_v1"
    path, lock = os.path.join(root, tag + ".npz"), os.path.join(root, tag + ".lock")

    def load():
        z = np.load(path)
        return CSR(int(z["M"]), int(z["K"]), z["rowptr"], z["colind"], z["values"]), bseed

    if os.path.exists(path):
        return load()
    try:
        fd = os.open(lock, os.O_CREAT | os.O_EXCL | os.O_WRONLY)
        os.close(fd)
        mine = True
    except FileExistsError:
        mine = False
    if not mine:   # somebody else is building it
        t0 = time.time()
        while time.time() - t0 < wait_s:
            if os.path.exists(path):
                return load()
            time.sleep(0.5)
        return builder(**kw), bseed   # a stale lock: build without the cache
    try:
        m = builder(**kw)
        tmp = path + f".{os.getpid()}.tmp.npz"
        np.savez(tmp, M=m.M, K=m.K, rowptr=m.rowptr, colind=m.colind, values=m.values)
        os.replace(tmp, path)
    finally:
        try:
            os.remove(lock)
        except OSError:
            pass
    return m, bseed


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
