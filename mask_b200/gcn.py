"""Row-sharded 2-layer GCN forward: ``out = A·(ReLU(A·(X·W1))·W2)`` over P ranks.

The reference project is single-GPU (its GCN driver, end2end/gcn/eva_gcn_sparsene.py:316-343,
calls one SpMM per layer on one device); this module is the multi-GPU harness the benchmark
configurations ask for.  Rank p owns a contiguous panel of rows of A (whole 16-row windows,
balanced by tile count) packed with global column ids, and a replica of X, W1, W2.

Layer 1 needs no exchange: every rank computes ``X·W1`` (dense, replicated) and multiplies its
panel.  Layer 2 needs all rows of ``Z = ReLU(A·XW1)·W2``: each rank computes its rows of Z and the
panels are reassembled with collectives that write straight into the full Z.  To overlap the
exchange with compute, a panel is cut into chunks: as soon as chunk c of Z is computed its
collectives are enqueued on a side stream while chunk c+1 is being multiplied.  Remote data
always lands in this GPU's own memory first; the layer-2 gather then reads local memory only.

Panels have different row counts (equal tile counts), so the reassembly uses one broadcast per
(source rank, chunk) into that rank's row range of Z instead of an equal-size all-gather.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch
import torch.distributed as dist

from .sharding import PEER_ROW_COST_TILES, balanced_panels, minimax_panels, nnz_balanced_panels


@dataclass
class PanelChunk:
    r0: int          # global first row
    r1: int          # global end row
    packed: object   # what `pack` returned for rows [r0, r1)


def chunk_bounds(win_prefix: np.ndarray, M: int, r0: int, r1: int, chunks: int) -> list[int]:
    """Cuts rows [r0, r1) (r0 on a window boundary) into `chunks` pieces of equal cost, where
    `win_prefix` is the global exclusive prefix of per-window cost (W+1 entries)."""
    w0, w1 = r0 // 16, (r1 + 15) // 16
    local = np.asarray(win_prefix[w0:w1 + 1], dtype=np.int64) - int(win_prefix[w0])
    b = balanced_panels(local, r1 - r0, chunks)
    return [r0 + x for x in b]


class ShardedGCN2:
    """Holds one rank's packed panel chunks and runs the 2-layer forward.

    pack(csr_rows) -> packed and spmm(packed, dense, relu) -> Tensor are injected so that the
    host-side logic (partition, chunking, reassembly) can be exercised on CPU ranks; the product
    uses the device format builder and SpMM kernels (`device_ops`)."""

    def __init__(self, csr, rank: int, world: int, pack, spmm, win_prefix=None, chunks: int = 4, group=None):
        self.M, self.K = csr.M, csr.K
        self.rank, self.world, self.group = rank, world, group
        self.spmm = spmm
        if win_prefix is None:
            self.bounds = nnz_balanced_panels(csr.rowptr, csr.M, world)
            W = (csr.M + 15) // 16
            win_rows = np.minimum(np.arange(W + 1, dtype=np.int64) * 16, csr.M)
            win_prefix = csr.rowptr[win_rows]
        else:
            self.bounds = balanced_panels(np.asarray(win_prefix), csr.M, world)
        # every rank needs every rank's chunk boundaries (they are the broadcast row ranges)
        self.chunk_rows = [chunk_bounds(win_prefix, csr.M, self.bounds[p], self.bounds[p + 1], chunks)
                           for p in range(world)]
        mine = self.chunk_rows[rank]
        self.chunks = [PanelChunk(a, b, pack(csr.row_slice(a, b)) if b > a else None) for a, b in zip(mine, mine[1:])]
        self.n_chunks = chunks

    def _layer(self, dense, relu, then=None):
        """Multiplies this rank's chunks by `dense`; `then(c, rows)` runs right after chunk c."""
        outs = []
        for c, ch in enumerate(self.chunks):
            if ch.packed is None:
                rows = dense.new_zeros((0, dense.shape[1]))
            else:
                rows = self.spmm(ch.packed, dense, relu)
            outs.append(rows)
            if then is not None:
                then(c, rows)
        return outs

    def forward(self, X: torch.Tensor, W1: torch.Tensor, W2: torch.Tensor) -> torch.Tensor:
        """Returns this rank's rows [bounds[rank], bounds[rank+1]) of the output."""
        cuda = X.is_cuda
        XW1 = X @ W1
        Z = torch.empty((self.M, W2.shape[1]), dtype=X.dtype, device=X.device)
        side = torch.cuda.Stream() if cuda else None
        pending = []

        def exchange(c, h1_rows):
            ch = self.chunks[c]
            if ch.r1 > ch.r0:
                Z[ch.r0:ch.r1] = h1_rows @ W2
            if self.world == 1:
                return
            ev = torch.cuda.Event() if cuda else None
            if cuda:
                ev.record()
                side.wait_event(ev)
            ctx = torch.cuda.stream(side) if cuda else _null()
            with ctx:
                for src in range(self.world):
                    a, b = self.chunk_rows[src][c], self.chunk_rows[src][c + 1]
                    if b > a:
                        pending.append(dist.broadcast(Z[a:b], src=src, group=self.group, async_op=True))

        self._layer(XW1, True, exchange)
        for w in pending:
            w.wait()
        if cuda and side is not None:
            torch.cuda.current_stream().wait_stream(side)
        outs = self._layer(Z, False)
        return torch.cat(outs, dim=0) if outs else Z.new_zeros((0, Z.shape[1]))


class FusedGCN2:
    """The same forward with the exchange fused into the layer-1 SpMM: its epilogue stores every
    finished row of ``H1 = ReLU(A·XW1)`` into all ranks' copies of H1 (peer-mapped buffers, plain
    stores over NVLink) while the product is still running, so there is no collective on the data
    path, only a one-word all-reduce as the barrier between the layers.  Layer 2 is reassociated,
    ``out = (A·H1)·W2``, so that what the SpMM produces is what the peers need.

    The two layers are partitioned separately (``bounds1`` for layer 1, ``bounds`` for layer 2 and the
    rows a rank returns): layer 1 pays for the rows it stores into its peers as well as for its tiles.

    H1 is double-buffered: a rank that races ahead into the next forward writes the other buffer,
    and cannot get a second forward ahead because of the barrier, so no rank's layer-2 reads are
    overwritten.

    ``ops`` supplies the three device-specific pieces, so that the protocol (panels, buffer
    rotation, barrier placement) also runs on CPU ranks in the tests:
      ops.pack(csr_rows) -> packed
      ops.shared_h1(rows, cols) -> list of two objects with ``.local`` (this rank's full copy)
      ops.spmm_to_all(packed, dense, h1_buffer, r0, r1)   # ReLU(A_panel·dense) -> rows [r0,r1) of EVERY rank's copy
      ops.spmm(packed, dense) -> Tensor                    # plain product of the panel
      ops.close()
    """

    def __init__(self, csr, rank: int, world: int, device, win_prefix, hidden: int, group=None, ops=None,
                 peer_row_cost: float | None = None):
        self.M, self.K, self.rank, self.world, self.group = csr.M, csr.K, rank, world, group
        if csr.M != csr.K:
            raise RuntimeError("the GCN forward needs a square adjacency matrix")
        # Layer 2 only multiplies: its panels (the rows of the output a rank returns) are balanced by SpMM
        # cost.  Layer 1 also stores every finished row into world - 1 peers while it multiplies, and on a
        # power-law graph equal tile counts mean very unequal row counts (the hub rows come first): its
        # panels minimise the larger of the two costs.  A rank packs its rows once per distinct panel.
        self.bounds = balanced_panels(np.asarray(win_prefix), csr.M, world)
        if peer_row_cost is None:
            peer_row_cost = PEER_ROW_COST_TILES * (world - 1)
        self.bounds1 = (minimax_panels(np.asarray(win_prefix), csr.M, world, peer_row_cost)
                        if world > 1 and peer_row_cost > 0 else list(self.bounds))
        self.p0, self.p1 = self.bounds1[rank], self.bounds1[rank + 1]
        self.r0, self.r1 = self.bounds[rank], self.bounds[rank + 1]
        self.ops = ops if ops is not None else _FusedDeviceOps(device, rank, world, group)
        self.packed1 = self.ops.pack(csr.row_slice(self.p0, self.p1)) if self.p1 > self.p0 else None
        if (self.p0, self.p1) == (self.r0, self.r1):
            self.packed = self.packed1
        else:
            self.packed = self.ops.pack(csr.row_slice(self.r0, self.r1)) if self.r1 > self.r0 else None
        self.hidden = hidden
        self.h1 = self.ops.shared_h1(csr.M, hidden)
        self.flag = torch.zeros(1, dtype=torch.int32, device=device)
        self.step = 0

    @property
    def plans(self):
        return getattr(self.ops, "plans", [])

    def forward(self, X: torch.Tensor, W1: torch.Tensor, W2: torch.Tensor) -> torch.Tensor:
        """Returns this rank's rows [bounds[rank], bounds[rank+1]) of the output."""
        if W1.shape[1] != self.hidden:
            raise RuntimeError("W1 does not match the hidden width this object was built for")
        XW1 = X @ W1
        buf = self.h1[self.step & 1]
        self.step += 1
        if self.packed1 is not None:
            self.ops.spmm_to_all(self.packed1, XW1, buf, self.p0, self.p1)
        if self.world > 1:
            dist.all_reduce(self.flag, group=self.group)   # (stream-ordered) barrier: every panel of H1 has landed
        if self.packed is None:
            return X.new_zeros((0, W2.shape[1]))
        return self.ops.spmm(self.packed, buf.local) @ W2

    def close(self) -> None:
        self.ops.close()


class _FusedDeviceOps:
    """The product path of FusedGCN2: device format builder, one plan per H1 buffer with the peers'
    addresses attached (`mask_plan_set_peer_outputs`), buffers from `mask_peer_alloc`."""

    def __init__(self, device, rank, world, group):
        from . import engine
        self.engine, self.device, self.rank, self.world, self.group = engine, device, rank, world, group
        self.plans, self.buffers, self._by_buffer = [], [], {}

    def pack(self, csr):
        return device_ops(self.device)[0](csr)

    def shared_h1(self, rows, cols):
        from .peer import PeerBuffer
        self.buffers = [PeerBuffer((rows, cols), self.device, self.rank, self.world, self.group) for _ in range(2)]
        return self.buffers

    def spmm_to_all(self, packed, dense, buf, r0, r1):
        plan = self._by_buffer.get(id(buf))
        if plan is None:
            plan = packed.new_plan()
            if self.world > 1:
                plan.set_peer_outputs(buf.others(r0 * dense.shape[1] * 4))
            self._by_buffer[id(buf)] = plan
            self.plans.append(plan)
        self.engine.spmm(packed, dense, out=buf.local[r0:r1], relu=True, plan=plan)

    def spmm(self, packed, dense):
        return self.engine.spmm(packed, dense)

    def close(self):
        self.plans, self._by_buffer = [], {}
        for b in self.buffers:
            b.close()
        self.buffers = []


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


def device_ops(device):
    """pack / spmm for the product path: device format builder and SpMM kernels."""
    from . import engine

    def pack(csr):
        rp, ci, va = (torch.from_numpy(np.ascontiguousarray(x)).to(device) for x in (csr.rowptr, csr.colind, csr.values))
        return engine.pack_srbcrs(rp, ci, va, csr.M, csr.K)

    def spmm(packed, dense, relu):
        return engine.spmm(packed, dense, relu=relu)

    return pack, spmm


def tile_prefix_on_device(csr, device) -> np.ndarray:
    """val_soff of the whole matrix (tiles before each window), from the device format builder."""
    from . import engine
    rp = torch.from_numpy(csr.rowptr).to(device)
    ci = torch.from_numpy(csr.colind).to(device)
    _, val_soff, _, _ = engine._analyze(rp, ci, csr.M, csr.K)
    return val_soff.cpu().numpy()


def cost_prefix_on_device(csr, device) -> np.ndarray:
    """Per-window cost prefix (tiles plus a fixed share per window) for balancing panels and chunks."""
    from .sharding import spmm_cost_prefix
    return spmm_cost_prefix(tile_prefix_on_device(csr, device))
