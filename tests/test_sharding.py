"""Host-side logic of the multi-GPU path on CPU: panel/chunk partitioning, and the row-sharded
2-layer GCN forward run by two gloo ranks (the per-panel SpMM is the oracle's CPU product here;
on a GPU the same harness gets the device kernels)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mask_b200 import generators as G
from mask_b200.gcn import ShardedGCN2, chunk_bounds
from mask_b200.sharding import balanced_panels, nnz_balanced_panels


def test_minimax_panels_against_exhaustive_search():
    """Panels that minimise max(SpMM cost, rows stored into peers): optimal among all window-aligned
    cuts on small cases, and equal to the plain balance when rows cost nothing."""
    import itertools
    from mask_b200.sharding import minimax_panels, panel_costs
    rng = np.random.default_rng(7)
    for _ in range(120):
        M = int(rng.integers(1, 170))
        W = (M + 15) // 16
        t = rng.integers(0, 30, size=W)
        t[:max(1, W // 4)] *= 5                       # heavy windows first, as on a power-law graph
        pref = np.concatenate([[0], np.cumsum(t)]).astype(np.int64)
        parts, rc = int(rng.integers(1, 5)), float(rng.choice([0.0, 0.1, 1.0, 3.0]))
        b = minimax_panels(pref, M, parts, rc)
        assert b[0] == 0 and b[-1] == M and len(b) == parts + 1
        assert all(x % 16 == 0 for x in b[:-1] if x != M) and all(x <= y for x, y in zip(b, b[1:]))
        best = min(max(panel_costs(pref, M, [0] + [min(c * 16, M) for c in cuts] + [M], rc))
                   for cuts in itertools.combinations_with_replacement(range(W + 1), parts - 1))
        assert max(panel_costs(pref, M, b, rc)) <= best * 1.002 + 1e-9
    # rows dominate: equal row counts whatever the tiles
    pref = np.concatenate([[0], np.cumsum([100, 50, 20, 5, 1, 1, 1, 1])]).astype(np.int64)
    assert minimax_panels(pref, 128, 4, 100.0) == [0, 32, 64, 96, 128]


def test_rebalanced_panels_follow_measured_times():
    """Re-cutting from per-panel times: when the real cost per unit of model cost falls from the top
    of the matrix to the bottom, one round brings the slowest panel from 16 % to under 4 % above the
    mean; equal times leave the panels (nearly) where they are; idle panels are handled."""
    from mask_b200.sharding import rebalanced_panels
    rng = np.random.default_rng(3)
    W = 4000
    M = W * 16
    model = rng.integers(1, 40, size=W).astype(np.int64)
    model[:200] *= 20
    pref = np.concatenate([[0], np.cumsum(model)])
    true = np.concatenate([[0], np.cumsum(model * np.linspace(1.6, 0.8, W))])

    def times(b):
        return [float(true[y // 16] - true[x // 16]) for x, y in zip(b, b[1:])]

    b0 = balanced_panels(pref, M, 8)
    t0 = times(b0)
    assert max(t0) > 1.12 * (sum(t0) / 8)
    b1 = rebalanced_panels(pref, M, b0, t0)
    assert b1[0] == 0 and b1[-1] == M and all(x % 16 == 0 for x in b1) and all(x < y for x, y in zip(b1, b1[1:]))
    t1 = times(b1)
    assert max(t1) < 1.04 * (sum(t1) / 8)
    share = [int(pref[y // 16] - pref[x // 16]) for x, y in zip(b0, b0[1:])]
    same = rebalanced_panels(pref, M, b0, [float(x) for x in share])
    assert max(abs(x - y) for x, y in zip(same, b0)) <= 16
    # a panel with no rows and no time, ragged M
    assert rebalanced_panels(np.array([0, 4, 8, 12]), 40, [0, 0, 32, 40], [0.0, 2.0, 1.0])[-1] == 40


def test_panels_are_window_aligned_and_balanced():
    m = G.rmat_gcn_normalised(scale=12, samples_per_node=8, seed=201)
    for parts in (1, 2, 3, 4, 8):
        b = nnz_balanced_panels(m.rowptr, m.M, parts)
        assert b[0] == 0 and b[-1] == m.M and len(b) == parts + 1
        assert all(x % 16 == 0 for x in b[:-1]) and all(x <= y for x, y in zip(b, b[1:]))
        share = [int(m.rowptr[y] - m.rowptr[x]) for x, y in zip(b, b[1:])]
        assert max(share) - min(share) <= 2 * int(np.diff(m.rowptr).max()) * 16 + 1
    # ragged M, generic cost prefix, more parts than windows
    prefix = np.array([0, 5, 5, 9], dtype=np.int64)
    assert balanced_panels(prefix, 40, 2) in ([0, 16, 40], [0, 32, 40])
    b = balanced_panels(prefix, 40, 8)
    assert b[0] == 0 and b[-1] == 40 and all(x <= y for x, y in zip(b, b[1:]))
    assert chunk_bounds(prefix, 40, 16, 40, 2)[0] == 16 and chunk_bounds(prefix, 40, 16, 40, 2)[-1] == 40
    from mask_b200.sharding import spmm_cost_prefix
    assert spmm_cost_prefix(prefix, 5).tolist() == [0, 10, 15, 24]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _cpu_ops():
    import oracle

    def pack(csr):
        return csr

    def spmm(csr, dense, relu):
        out = torch.from_numpy(oracle.spmm_f32(csr.M, csr.rowptr, csr.colind, csr.values, dense.numpy(), threads=1))
        return torch.relu(out) if relu else out

    return pack, spmm


def _rank_main(rank, world, port, chunks, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m = G.rmat_gcn_normalised(scale=9, samples_per_node=6, seed=501)
        X = torch.from_numpy(G.dense_normal(m.K, 24, 502))
        W1 = torch.from_numpy(G.glorot_uniform(24, 16, 503))
        W2 = torch.from_numpy(G.glorot_uniform(16, 8, 504))
        pack, spmm = _cpu_ops()
        net = ShardedGCN2(m, rank, world, pack, spmm, chunks=chunks)
        out = net.forward(X, W1, W2)
        q.put((rank, net.bounds, out.numpy()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,chunks", [(2, 3), (3, 1)])
def test_sharded_gcn_forward_matches_single_process(world, chunks):
    import oracle
    m = G.rmat_gcn_normalised(scale=9, samples_per_node=6, seed=501)
    X = G.dense_normal(m.K, 24, 502)
    W1, W2 = G.glorot_uniform(24, 16, 503), G.glorot_uniform(16, 8, 504)
    h1 = np.maximum(oracle.spmm_f32(m.M, m.rowptr, m.colind, m.values, X @ W1, threads=1), 0)
    want = oracle.spmm_f32(m.M, m.rowptr, m.colind, m.values, h1 @ W2, threads=1)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, chunks, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    full = np.zeros_like(want)
    for rank, bounds, out in got:
        full[bounds[rank]:bounds[rank + 1]] = out
    assert np.allclose(full, want, rtol=1e-5, atol=1e-6)


class _SharedBuf:
    def __init__(self, copies, rank):
        self.copies, self.local = copies, copies[rank]


class _CpuFusedOps:
    """FusedGCN2's device pieces on CPU ranks: the ranks' copies of H1 are shared-memory tensors,
    and 'storing to the peers' is writing the panel's rows into every copy."""

    def __init__(self, rank, shared, delay):
        self.rank, self.shared, self.delay = rank, shared, delay   # shared[b][rank] = tensor [M, hidden]
        self.pack, self._spmm = _cpu_ops()

    def shared_h1(self, rows, cols):
        return [_SharedBuf(self.shared[b], self.rank) for b in range(2)]

    def spmm_to_all(self, csr, dense, buf, r0, r1):
        import time
        rows = self._spmm(csr, dense, True)
        for i, copy in enumerate(buf.copies):
            if self.delay and i != self.rank:
                time.sleep(self.delay)    # a slow link: the barrier, not luck, must cover it
            copy[r0:r1] = rows

    def spmm(self, csr, dense):
        return self._spmm(csr, dense.clone(), False)

    def close(self):
        pass


def _fused_rank_main(rank, world, port, shared, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from mask_b200.gcn import FusedGCN2
        from mask_b200.sharding import spmm_cost_prefix
        import oracle
        m = G.rmat_gcn_normalised(scale=9, samples_per_node=6, seed=501)
        X = torch.from_numpy(G.dense_normal(m.K, 24, 502))
        W1 = torch.from_numpy(G.glorot_uniform(24, 16, 503))
        W2 = torch.from_numpy(G.glorot_uniform(16, 8, 504))
        prefix = spmm_cost_prefix(oracle.pack_srbcrs(m.M, m.rowptr, m.colind, m.values)["val_soff"])
        net = FusedGCN2(m, rank, world, torch.device("cpu"), prefix, hidden=16,
                        ops=_CpuFusedOps(rank, shared, delay=0.05 if rank == 0 else 0.0))
        outs = [net.forward(X * s, W1, W2).numpy() for s in (1.0, -2.0, 1.0, 3.0)]
        q.put((rank, net.bounds, outs, net.bounds1))
        net.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_fused_gcn_protocol_on_cpu_ranks(world):
    """Panels, H1 double-buffering and barrier placement of FusedGCN2 with gloo ranks whose
    'peer stores' go to shared-memory copies; one rank's stores are slow.  Four forwards with
    different inputs reuse both buffers twice."""
    import oracle
    m = G.rmat_gcn_normalised(scale=9, samples_per_node=6, seed=501)
    X = G.dense_normal(m.K, 24, 502)
    W1, W2 = G.glorot_uniform(24, 16, 503), G.glorot_uniform(16, 8, 504)
    wants = []
    for s in (1.0, -2.0, 1.0, 3.0):
        h1 = np.maximum(oracle.spmm_f32(m.M, m.rowptr, m.colind, m.values, (X * s) @ W1, threads=1), 0)
        wants.append(oracle.spmm_f32(m.M, m.rowptr, m.colind, m.values, h1, threads=1) @ W2)
    shared = [[torch.full((m.M, 16), float("nan")).share_memory_() for _ in range(world)] for _ in range(2)]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_fused_rank_main, args=(r, world, port, shared, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = [q.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for i, want in enumerate(wants):
        full = np.zeros_like(want)
        for rank, bounds, outs, _ in got:
            full[bounds[rank]:bounds[rank + 1]] = outs[i]
        assert np.allclose(full, want, rtol=1e-4, atol=1e-5), i
    # the layer that also stores into the peers is cut differently from the one that only multiplies
    # (hub rows first: equal tiles are unequal rows), and every rank agrees on both partitions
    assert len({tuple(b1) for _, _, _, b1 in got}) == 1 and len({tuple(b) for _, b, _, _ in got}) == 1
    assert got[0][3] != got[0][1]


def _gpu_rank_main(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from mask_b200.gcn import device_ops, tile_prefix_on_device
        dev = torch.device("cuda", rank)
        m = G.rmat_gcn_normalised(scale=12, samples_per_node=8, seed=501)
        X = torch.from_numpy(G.dense_normal(m.K, 64, 502)).to(dev)
        W1 = torch.from_numpy(G.glorot_uniform(64, 64, 503)).to(dev)
        W2 = torch.from_numpy(G.glorot_uniform(64, 32, 504)).to(dev)
        pack, spmm = device_ops(dev)
        net = ShardedGCN2(m, rank, world, pack, spmm, win_prefix=tile_prefix_on_device(m, dev), chunks=3)
        out = net.forward(X, W1, W2)
        torch.cuda.synchronize()
        # the same forward with the exchange fused into the SpMM epilogue (peer stores); three
        # forwards so that both H1 buffers and the reuse of the first are exercised
        from mask_b200.gcn import FusedGCN2, cost_prefix_on_device
        fused = FusedGCN2(m, rank, world, dev, cost_prefix_on_device(m, dev), hidden=64)
        outs = [fused.forward(X * s, W1, W2) for s in (1.0, 2.0, 1.0)]
        torch.cuda.synchronize()
        assert torch.equal(outs[0], outs[2]) and not torch.equal(outs[0], outs[1])
        assert all(p.status() == 0 for p in fused.plans)
        q.put((rank, net.bounds, out.cpu().numpy(), fused.bounds, outs[2].cpu().numpy()))
        fused.close()
    finally:
        dist.destroy_process_group()


def _gcn_reference(m, X, W1, W2):
    import oracle
    h1 = np.maximum(oracle.spmm_f32(m.M, m.rowptr, m.colind, m.values, X @ W1), 0)
    return oracle.spmm_f32(m.M, m.rowptr, m.colind, m.values, h1 @ W2)


@pytest.mark.gpu
def test_gcn_forward_single_gpu():
    from mask_b200.gcn import device_ops, tile_prefix_on_device
    dev = torch.device("cuda", 0)
    m = G.rmat_gcn_normalised(scale=12, samples_per_node=8, seed=501)
    X, W1, W2 = G.dense_normal(m.K, 64, 502), G.glorot_uniform(64, 64, 503), G.glorot_uniform(64, 32, 504)
    pack, spmm = device_ops(dev)
    net = ShardedGCN2(m, 0, 1, pack, spmm, win_prefix=tile_prefix_on_device(m, dev), chunks=3)
    torch.backends.cuda.matmul.allow_tf32 = False
    out = net.forward(*(torch.from_numpy(a).to(dev) for a in (X, W1, W2))).cpu().numpy()
    want = _gcn_reference(m, X, W1, W2)
    # two chained TF32 products: compare at the scale of the result
    assert np.abs(out - want).max() <= 4e-3 * np.abs(want).max() + 1e-6


@pytest.mark.gpu
def test_gcn_forward_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    m = G.rmat_gcn_normalised(scale=12, samples_per_node=8, seed=501)
    X, W1, W2 = G.dense_normal(m.K, 64, 502), G.glorot_uniform(64, 64, 503), G.glorot_uniform(64, 32, 504)
    want = _gcn_reference(m, X, W1, W2)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_gpu_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = [q.get(timeout=300) for _ in range(2)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    full, full_fused = np.zeros_like(want), np.zeros_like(want)
    for rank, bounds, out, fbounds, fout in got:
        full[bounds[rank]:bounds[rank + 1]] = out
        full_fused[fbounds[rank]:fbounds[rank + 1]] = fout
    assert np.abs(full - want).max() <= 4e-3 * np.abs(want).max() + 1e-6
    assert np.abs(full_fused - want).max() <= 4e-3 * np.abs(want).max() + 1e-6


@pytest.mark.gpu
def test_fused_gcn_forward_single_gpu():
    """FusedGCN2 with one rank: library-allocated H1 buffers, reassociated layer 2."""
    from mask_b200.gcn import FusedGCN2, cost_prefix_on_device
    dev = torch.device("cuda", 0)
    m = G.rmat_gcn_normalised(scale=12, samples_per_node=8, seed=501)
    X, W1, W2 = G.dense_normal(m.K, 64, 502), G.glorot_uniform(64, 64, 503), G.glorot_uniform(64, 32, 504)
    net = FusedGCN2(m, 0, 1, dev, cost_prefix_on_device(m, dev), hidden=64)
    torch.backends.cuda.matmul.allow_tf32 = False
    args = [torch.from_numpy(a).to(dev) for a in (X, W1, W2)]
    out = net.forward(*args).cpu().numpy()
    out2 = net.forward(*args).cpu().numpy()
    net.close()
    want = _gcn_reference(m, X, W1, W2)
    assert np.abs(out - want).max() <= 4e-3 * np.abs(want).max() + 1e-6
    assert np.array_equal(out, out2)
