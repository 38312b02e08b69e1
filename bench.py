#!/usr/bin/env python
"""SpMM benchmark: effective GFLOP/s (2*nnz*N/t) at N=512 on 1/2/4/8 B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

A step is one product C = A*B over the whole matrix.  The default workload is the largest
row-sharded configuration, the symmetric R-MAT graph with 2^22 nodes and average degree 32
(values U(-1,1)) packed as SR-BCRS 16x8, B 2^22 x 512 FP32 N(0,1); `--workload rmat20_gcn`,
`stencil27_100`, `uniform4096`, `rmat21_gcn` select the other configurations.  All inputs are
synthetic and seeded (the reference project's evaluation matrices are not distributed with it).
With N > 1 ranks (torchrun) the rows of A are cut into balanced panels on window boundaries, B is
replicated, every rank multiplies its panel and no collective is on the device-timed data path
(strong scaling: the total work is fixed).  Every rank checks seeded sample rows of its own
result (plus the rows of its heaviest windows) against the CPU oracle.

One JSON line is printed by rank 0:
  value      device-side throughput, inputs resident in HBM, CUDA events on the launch stream,
             max over ranks
  e2e        the same product with HOST buffers, copies inside the timed region: at 1 GPU through the
             host-buffer C-ABI call (pinned host B in, host C out); at N > 1 every rank uploads 1/N of B,
             the ranks all-gather it over NVLink chunk by chunk while earlier chunks multiply, and every
             rank downloads its panel of C
  roofline   algorithmic bytes per launch / measured kernel time, against the measured HBM peak
  cpu_baseline  the host FP32 reference SpMM (CPU port of the reference's cpu_spmm) timed on this
             box's cores on the same matrix (rank 0, N=1 only); also used to verify the GPU result
--impl reference times that CPU implementation alone, with all host threads.

Extra lines on request (each prints its own JSON line instead of the one above):
  --gcn [--gcn-fused]   row-sharded 2-layer GCN forward; fused = the layer-1 SpMM stores H1 into every
                        rank's copy through peer memory instead of NCCL broadcasts
  --bridge              the reference's Format-DSL bridge and ME-TCF testbed executables (built by
                        `make -C oracle bridge` where a checkout of the reference is present) with the
                        operator the reference emits and with the hand-written sm_100a operator includes
  --baselines           cuSPARSE CSR and the reference's own kernel recompiled for sm_100a, same inputs
Other switches: --format srbcrs|metcf|mco, --workload, --scale, --cols (= --n), --policy, kernel knobs.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "SpMM effective GFLOP/s (2*nnz*N/t) at N=512"
UNIT = "GFLOP/s"
FALLBACK_HBM_GBS = 6650.0


def log(*a):
    print(*a, file=sys.stderr, flush=True)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.002):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        self.period = period_s
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception as e:  # NVML missing: report clocks as unknown rather than fail the bench
            self.nv = None
            log(f"[bench] NVML unavailable: {e}")

    def _run(self):
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
            getattr(nv, "nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80): "hw_power_brake",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def build_workload(name: str, scale: int | None):
    from mask_b200 import generators as G
    kw = {}
    if scale is not None:
        kw = {"grid": scale} if name.startswith("stencil") else ({"n": scale} if name.startswith("uniform") else {"scale": scale})
    t0 = time.time()
    m, bseed = G.make_workload_cached(name, **kw)
    log(f"[bench] workload {name} {kw}: M={m.M} nnz={m.nnz} built in {time.time() - t0:.1f}s")
    return m, bseed


def panel_bounds(m, parts: int, dev) -> list[int]:
    """Row panel boundaries on 16-row window boundaries.  Panels are balanced by a cost model of
    the kernel -- 16x8 tiles plus a fixed share per window for the rows of C it writes (equal to
    balanced nnz up to tile fill and row count): every rank runs the cheap window analysis of the
    device format builder on the whole matrix to get tiles per window."""
    if parts == 1:
        return [0, m.M], None
    import torch
    from mask_b200 import engine
    from mask_b200.sharding import balanced_panels, spmm_cost_prefix
    rp = torch.from_numpy(m.rowptr).to(dev)
    ci = torch.from_numpy(m.colind).to(dev)
    _, val_soff, _, _ = engine._analyze(rp, ci, m.M, m.K)
    prefix = spmm_cost_prefix(val_soff.cpu().numpy())
    return balanced_panels(prefix, m.M, parts), prefix


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one launch of the dominant kernel, from
# one-pass ncu captures of exactly this workload on one GPU.  Each entry names the kernel and the
# library's kernel revision it was captured on; the bench reports it only while that still runs.
NCU_TRAFFIC = {
    ("rmat22_sym", None, 512, "srbcrs"): {"kernel": "spmm_sweep_kernel<nslab=2,srbcrs>", "revision": 4, "bytes": 149.007e9 + 10.976e9,
                                          "capture": "ncu 1-pass dram__bytes_read/write.sum, one launch of this workload at full size"},
    ("rmat20_gcn", None, 512, "srbcrs"): {"kernel": "spmm_sweep_kernel<nslab=2,srbcrs>", "revision": 4, "bytes": 14.803e9 + 2.376e9,
                                          "capture": "ncu 1-pass dram__bytes_read/write.sum, one launch of this workload at full size"},
    ("stencil27_100", None, 512, "srbcrs"): {"kernel": "spmm_sweep_kernel<nslab=4,srbcrs>", "revision": 4, "bytes": 5.808e9 + 2.035e9,
                                             "capture": "ncu 1-pass dram__bytes_read/write.sum, one launch of this workload at full size"},
}


def algorithmic_bytes(T: int, W: int, M: int, N: int, distinct_cols: int) -> int:
    """A values + column metadata + every touched row of B once + C written once."""
    return 4 * 128 * T + 4 * (8 * T + W + 1) + 4 * N * distinct_cols + 4 * M * N


def dense_operand(K: int, N: int, bseed: int, dev):
    """The dense operand on the device (plus the host copy when it was drawn there).  Up to 2 GiB
    it is NumPy's PCG64 N(0,1) like every other input; beyond that drawing it on the host would
    take longer than the whole benchmark, so it comes from the device's generator with the same
    seed (identical on every rank)."""
    import torch
    from mask_b200 import generators as G
    if int(K) * N * 4 <= (1 << 31):
        Bh = G.dense_normal(K, N, bseed)
        return torch.from_numpy(Bh).to(dev), Bh, f"N(0,1), NumPy PCG64 seed {bseed}"
    gen = torch.Generator(device=dev)
    gen.manual_seed(bseed)
    Bd = torch.randn((K, N), dtype=torch.float32, device=dev, generator=gen)
    return Bd, None, f"N(0,1), device generator seed {bseed}"


class VerifySample:
    """Rows of one rank's panel and their exact products from the CPU oracle: the whole panel for
    the configurations up to 2^20 rows on one GPU, else seeded random rows plus every row of the
    panel's heaviest windows (longest tile runs; taken heaviest first within a budget of stored
    entries so that the host work stays bounded).  Only the rows of B the sample touches are
    brought to the host."""

    def __init__(self, oracle, panel, val_soff, Bd, seed: int, n_random: int, n_heavy: int, full: bool = False,
                 heavy_entries: int = 1 << 25):
        import torch
        self.oracle = oracle
        rp = panel.rowptr.astype(np.int64)
        if full:
            rows = np.arange(panel.M, dtype=np.int64)
            self.how = f"all {panel.M} rows"
        else:
            rng = np.random.Generator(np.random.PCG64(seed))
            order = np.argsort(np.diff(val_soff), kind="stable")[::-1][:n_heavy]
            win_entries = rp[np.minimum((order + 1) * 16, panel.M)] - rp[np.minimum(order * 16, panel.M)]
            keep = max(min(8, order.size), int(np.searchsorted(np.cumsum(win_entries), heavy_entries, side="right")))
            heavy = order[:keep]
            rows = np.unique(np.concatenate([rng.integers(0, panel.M, size=min(n_random, panel.M)),
                                             (heavy[:, None] * 16 + np.arange(16)[None, :]).ravel()]))
            self.how = f"{min(n_random, panel.M)} seeded rows + all rows of the {heavy.size} heaviest windows"
        self.rows = rows[rows < panel.M].astype(np.int64)
        lens = rp[self.rows + 1] - rp[self.rows]
        sub_ptr = np.zeros(self.rows.size + 1, dtype=np.int64)
        np.cumsum(lens, out=sub_ptr[1:])
        idx = np.repeat(rp[self.rows] - sub_ptr[:-1], lens) + np.arange(int(sub_ptr[-1]), dtype=np.int64)
        cols = panel.colind[idx]
        vals = np.ascontiguousarray(panel.values[idx])
        ucols, inv = np.unique(cols, return_inverse=True)
        Bsub = Bd[torch.from_numpy(ucols.astype(np.int64)).to(Bd.device)].cpu().numpy()
        ptr32, inv32 = sub_ptr.astype(np.int32), inv.astype(np.int32)
        self.ref = oracle.spmm_f32(self.rows.size, ptr32, inv32, vals, Bsub)
        self.absp = oracle.spmm_abs_f64(self.rows.size, ptr32, inv32, vals, Bsub)

    def check(self, out_dev):
        import torch
        got = out_dev[torch.from_numpy(self.rows).to(out_dev.device)].cpu().numpy()
        return self.oracle.check_tolerance(got, self.ref, self.absp)

    def check_host(self, rows_host):
        return self.oracle.check_tolerance(np.ascontiguousarray(rows_host), self.ref, self.absp)


def packing_parity(oracle, panel, packed, max_entries: int = 1 << 24):
    """Byte comparison of the device-built SR-BCRS arrays with the CPU oracle's packing of the same rows: the
    whole panel, or its leading windows holding at most `max_entries` stored entries (windows are packed
    independently, so the leading windows of the panel's arrays are the arrays of the leading rows).
    Returns (mismatching arrays, windows compared, tiles compared)."""
    rows = panel.M
    if panel.nnz > max_entries:
        rows = max(16, int(np.searchsorted(panel.rowptr, max_entries, side="right") - 1) // 16 * 16)
    rp = np.ascontiguousarray(panel.rowptr[:rows + 1])
    n = int(rp[-1])
    want = oracle.pack_srbcrs(rows, rp, np.ascontiguousarray(panel.colind[:n]), np.ascontiguousarray(panel.values[:n]))
    W, T = (rows + 15) // 16, int(want["T"])
    got = {"val_soff": packed.val_soff[:W + 1], "val_sidx": packed.val_sidx[:8 * T], "val_block_val": packed.val_block_val[:128 * T]}
    bad = []
    for name, dev_arr in got.items():
        a = dev_arr.cpu().numpy()
        b = want[name]
        if a.shape != b.shape or not np.array_equal(a.view(np.uint32), b.view(np.uint32)):
            bad.append(name)
    return bad, W, T


def cpu_baseline(m, N, Bd, Bh):
    """The oracle's host FP32 SpMM (CPU port of the reference's cpu_spmm) with every host thread on
    a bounded sample: the leading rows of the matrix holding at most 2^26 stored entries."""
    import oracle
    threads = host_threads()
    Lo = oracle.lib()
    rows = m.M
    if m.nnz > (1 << 26):
        rows = max(16, int(np.searchsorted(m.rowptr, 1 << 26)) // 16 * 16)
    if Bh is None:
        Bh = Bd.cpu().numpy()
    nnz_s = int(m.rowptr[rows])
    Cs = np.zeros((rows, N), dtype=np.float32)
    t0 = time.perf_counter()
    Lo.oracle_spmm_f32(0, rows, N, m.rowptr, m.colind, m.values, Bh, N, Cs, N, threads)
    cpu_s = time.perf_counter() - t0
    what = "the whole workload once" if rows == m.M else f"rows [0,{rows}) of {m.M}"
    return {"value": 2.0 * nnz_s * N / cpu_s / 1e9, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"{what} ({nnz_s} of {m.nnz} stored entries, N={N}), {cpu_s:.2f} s"}


def e2e_single(args, m, packed, Bd, Bh, sample):
    """One GPU: the host-buffer C-ABI call, pinned host B in, host C out."""
    import torch
    from mask_b200 import _lib
    if args.format != "srbcrs":
        raise RuntimeError("the host-buffer session packs SR-BCRS")
    L = _lib.lib()
    N = args.n
    hB = (torch.from_numpy(Bh) if Bh is not None else Bd.cpu()).pin_memory()
    hC = torch.empty((m.M, N), dtype=torch.float32).pin_memory()
    sr_host = {k: getattr(packed, k).cpu().numpy() for k in ("val_soff", "val_sidx", "val_block_val")}
    sess = C.c_void_p()
    _lib.check(L.mask_session_create_srbcrs(m.M, m.K, packed.T, sr_host["val_soff"].ctypes.data,
                                            sr_host["val_sidx"].ctypes.data, sr_host["val_block_val"].ctypes.data,
                                            _lib.POLICY[args.policy], C.byref(sess)), "mask_session_create_srbcrs")
    del sr_host
    kms = C.c_float()
    for _ in range(2):
        _lib.check(L.mask_session_spmm_host(sess, hB.data_ptr(), hC.data_ptr(), N, C.byref(kms)), "spmm_host")
    t0 = time.perf_counter()
    for _ in range(args.e2e_steps):
        _lib.check(L.mask_session_spmm_host(sess, hB.data_ptr(), hC.data_ptr(), N, C.byref(kms)), "spmm_host")
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.e2e_steps
    L.mask_session_destroy(sess)
    e2e = {"value": 2.0 * m.nnz * N / (e2e_ms * 1e-3) / 1e9, "unit": UNIT,
           "h2d_bytes_per_step": int(m.K) * N * 4, "d2h_bytes_per_step": int(m.M) * N * 4,
           "ms_per_step": e2e_ms, "steps": args.e2e_steps,
           "api": "mask_session_spmm_host (C ABI, pinned host B in, host C out)"}
    host_rows = hC.numpy()[sample.rows] if sample is not None else None
    return e2e, host_rows


def e2e_sharded(args, m, panel, packed, plan, Bd, dev, rank, world, sample):
    """N ranks: rank p holds rows [pK/N, (p+1)K/N) of B and its panel of C in pinned host memory.  B
    is cut into 128-column chunks; for every chunk each rank uploads its share, the ranks all-gather
    the chunk over NVLink (NCCL) into their own full copy, multiply it and download their panel's
    columns -- four streams, so uploads, gathers, products and downloads of different chunks overlap
    and only 1/N of B crosses each rank's host link."""
    import torch
    import torch.distributed as dist
    from mask_b200 import _lib, engine
    L = _lib.lib()
    N, K = args.n, int(m.K)
    w = 128
    if N % w != 0 or K % world != 0:
        raise RuntimeError("the sharded end-to-end leg needs N % 128 == 0 and K divisible by the ranks")
    share = K // world
    chunks = N // w
    hB = Bd[rank * share:(rank + 1) * share].cpu().pin_memory()     # this rank's rows of B, row-major [share, N]
    hC = torch.empty((panel.M, N), dtype=torch.float32).pin_memory()
    part = [torch.empty((share, w), dtype=torch.float32, device=dev) for _ in range(chunks)]
    full = [torch.empty((K, w), dtype=torch.float32, device=dev) for _ in range(chunks)]
    outc = [torch.empty((panel.M, w), dtype=torch.float32, device=dev) for _ in range(chunks)]
    up, comm, comp, down = (torch.cuda.Stream(device=dev) for _ in range(4))
    H2D, D2H = 1, 2

    def copy2d(dst, dpitch, src, spitch, width, height, kind, stream):
        _lib.check(L.mask_copy_2d_async(dst, dpitch, src, spitch, width, height, kind, C.c_void_p(stream.cuda_stream)), "mask_copy_2d_async")

    def one():
        for c in range(chunks):
            c0 = c * w
            copy2d(part[c].data_ptr(), w * 4, hB.data_ptr() + c0 * 4, N * 4, w * 4, share, H2D, up)
            e_up = torch.cuda.Event()
            e_up.record(up)
            comm.wait_event(e_up)
            with torch.cuda.stream(comm):
                dist.all_gather_into_tensor(full[c], part[c])
                e_g = torch.cuda.Event()
                e_g.record(comm)
            comp.wait_event(e_g)
            with torch.cuda.stream(comp):
                engine.spmm(packed, full[c], out=outc[c], plan=plan)
                e_k = torch.cuda.Event()
                e_k.record(comp)
            down.wait_event(e_k)
            copy2d(hC.data_ptr() + c0 * 4, N * 4, outc[c].data_ptr(), w * 4, w * 4, panel.M, D2H, down)
        for st in (up, comm, comp, down):
            st.synchronize()

    for _ in range(2):
        one()
    dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(args.e2e_steps):
        one()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.e2e_steps
    te = torch.tensor([e2e_ms], dtype=torch.float64, device=dev)
    dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_ms = float(te.item())
    if plan.status() != 0:
        raise RuntimeError("a kernel gave up on a bounded wait in the end-to-end leg")
    e2e = {"value": 2.0 * m.nnz * N / (e2e_ms * 1e-3) / 1e9, "unit": UNIT,
           "h2d_bytes_per_step": share * N * 4, "d2h_bytes_per_step": int(panel.M) * N * 4,
           "ms_per_step": e2e_ms, "steps": args.e2e_steps,
           "api": "per rank: upload 1/N of B (pinned host) per 128-column chunk, NCCL all-gather into the rank's full copy, "
                  "engine.spmm per chunk, download of the panel's columns; bytes are per rank"}
    host_rows = hC.numpy()[sample.rows] if sample is not None else None
    return e2e, host_rows


def run_reference(args):
    """CPU arm: the host FP32 reference SpMM with every host thread, on the same workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    from mask_b200 import generators as G
    m, bseed = build_workload(args.workload, args.scale)
    N = args.n
    threads = host_threads()
    # beyond 2 GiB the operand is drawn by all threads at once (independent PCG64 streams per row
    # block); only the timing depends on it here
    B = G.dense_normal(m.K, N, bseed) if int(m.K) * N * 4 <= (1 << 31) else G.dense_normal_blocks(m.K, N, bseed, threads)
    L = oracle.lib()
    Cm = None

    def run(r0, r1):
        t0 = time.perf_counter()
        L.oracle_spmm_f32(r0, r1, N, m.rowptr, m.colind, m.values, B, N, Cm, N, threads)
        return time.perf_counter() - t0

    # size the per-step sample so the whole run stays within about two minutes
    probe_rows = min(m.M, max(16, m.M // 64))
    Cm = np.zeros((probe_rows, N), dtype=np.float32)
    tp = run(0, probe_rows)
    est_full = tp * m.nnz / max(1, int(m.rowptr[probe_rows]))
    budget = 120.0 / (args.steps + args.warmup)
    frac = min(1.0, budget / max(est_full, 1e-9))
    rows = m.M if frac >= 1.0 else max(16, int(m.M * frac) // 16 * 16)
    nnz_s = int(m.rowptr[rows])
    Cm = np.zeros((rows, N), dtype=np.float32)
    for _ in range(args.warmup):
        run(0, rows)
    t = 0.0
    for _ in range(args.steps):
        t += run(0, rows)
    ms = t / args.steps * 1e3
    val = 2.0 * nnz_s * N / (ms * 1e-3) / 1e9
    sample = f"rows [0,{rows}) of {m.M} ({nnz_s} of {m.nnz} stored entries) per step"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "M": m.M, "K": m.K, "nnz": m.nnz, "N": N},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }), flush=True)


def host_threads() -> int:
    """Threads for the CPU arm: every core this process may run on.  torchrun exports
    OMP_NUM_THREADS=1 for its workers, which must not shrink the CPU baseline to one core."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def run_gcn(args, m, bseed, dev, rank, world):
    """2-layer GCN forward out = A*(ReLU(A*(X*W1))*W2), features = hidden = classes = N, row-sharded
    with the panels of Z = ReLU(A*XW1)*W2 reassembled over NCCL between the layers."""
    import torch
    import torch.distributed as dist
    from mask_b200 import generators as G
    from mask_b200.gcn import ShardedGCN2, device_ops, tile_prefix_on_device
    N = args.n
    X = torch.from_numpy(G.dense_normal(m.K, N, bseed)).to(dev)
    W1 = torch.from_numpy(G.glorot_uniform(N, N, bseed + 1)).to(dev)
    W2 = torch.from_numpy(G.glorot_uniform(N, N, bseed + 2)).to(dev)
    pack, spmm = device_ops(dev)
    if args.gcn_fused:
        from mask_b200.gcn import FusedGCN2, cost_prefix_on_device
        net = FusedGCN2(m, rank, world, dev, cost_prefix_on_device(m, dev), hidden=N)
    else:
        net = ShardedGCN2(m, rank, world, pack, spmm, win_prefix=tile_prefix_on_device(m, dev), chunks=4)
    torch.backends.cuda.matmul.allow_tf32 = True
    for _ in range(args.warmup):
        net.forward(X, W1, W2)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        net.forward(X, W1, W2)
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / args.steps], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    if rank == 0:
        flops = 2 * (2.0 * m.nnz * N) + 2 * (2.0 * m.M * N * N)
        how = "exchange fused into the SpMM epilogue (peer stores)" if args.gcn_fused else "chunked NCCL broadcasts"
        print(json.dumps({"metric": "2-layer GCN forward (row-sharded), ms per forward", "exchange": how, "value": ms, "unit": "ms",
                          "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
                          "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "tf32",
                          "data": "synthetic", "spmm_gflops_effective": 2 * 2.0 * m.nnz * N / (ms * 1e-3) / 1e9,
                          "total_gflops_effective": flops / (ms * 1e-3) / 1e9,
                          "config": {"workload": args.workload, "M": m.M, "nnz": m.nnz, "features": N, "chunks": 1 if args.gcn_fused else 4,
                                     "panels": net.bounds, "panels_layer1": getattr(net, "bounds1", net.bounds)}}), flush=True)
    if args.gcn_fused:
        net.close()
    if world > 1:
        dist.destroy_process_group()


def run_bridge(args, m):
    """Same-box comparison at the reference's Format-DSL bridge seam: the reference's own bridge
    executable (its packer, its timing loop, its cuSPARSE check) built once with the operator its
    compiler emits and once with the hand-written sm_100a operator include; both are made by
    `make -C oracle bridge` where a checkout of the reference is present.  The bridge reads a
    MatrixMarket file, so the workload's pattern is written to a temporary one."""
    import subprocess
    import tempfile
    from mask_b200 import generators as G
    here = os.path.dirname(os.path.abspath(__file__))
    runs = [("reference_emitted_operator_tile64", "bridge_refgen_tn64"), ("sm100_operator_tile64", "bridge_sm100_tn64"),
            ("sm100_operator_tile128", "bridge_sm100_tn128"),
            ("reference_emitted_operator_tile64_fast_tf32", "bridge_refgen_fast_tn64"),
            ("sm100_operator_tile64_fast_tf32", "bridge_sm100_fast_tn64")]
    out = {}
    with tempfile.TemporaryDirectory() as tmp:
        mtx = os.path.join(tmp, "w.mtx")
        G.write_matrix_market(m, mtx)
        for label, exe in runs:
            path = os.path.join(here, "oracle", "_ref", exe)
            if not os.path.exists(path):
                out[label] = {"unavailable": "not built (needs a checkout of the reference)"}
                continue
            out[label] = {}
            for policy in ("row", "strict_lb"):
                js = os.path.join(tmp, "r.json")
                cmd = [path, "--filename", mtx, "--dataset", args.workload, "--result-json", js, "--n", str(args.n), "--warmup",
                       str(max(args.warmup, 3)), "--repeat", str(args.steps), "--execution-policy", policy]
                r = subprocess.run(cmd, capture_output=True, text=True)
                if r.returncode not in (0, 2) or not os.path.exists(js):
                    out[label][policy] = {"error": (r.stderr or r.stdout)[-200:]}
                    continue
                rep = json.load(open(js))
                ms = rep["timing"]["generated_ms"]
                out[label][policy] = {"ms": ms, "gflops": 2.0 * m.nnz * args.n / (ms * 1e-3) / 1e9,
                                      "cusparse_ms": rep["timing"]["cusparse_ms"], "passed": rep["correctness"]["passed"],
                                      "max_abs_error": rep["correctness"]["max_abs_error"], "tiles": rep["packed"]["tiles"]}
                os.remove(js)
        # the ME-TCF testbed with its generated-operator host program (prints mykernel_time / VERIFICATION)
        for label, exe in (("dtc_testbed_reference_operator_tile64", "dtc_generated_ref"), ("dtc_testbed_sm100_operator_tile64", "dtc_generated_sm100")):
            path = os.path.join(here, "oracle", "_ref", exe)
            if not os.path.exists(path):
                out[label] = {"unavailable": "not built (needs a checkout of the reference)"}
                continue
            r = subprocess.run([path, "-filename", mtx, "-N", str(args.n), "-warmup", str(max(args.warmup, 3)), "-repeat", str(args.steps)],
                               capture_output=True, text=True, env=dict(os.environ, SPARSENE_DISABLE_MTX_CACHE="1"))
            rec = {"exit_code": r.returncode}
            for line in r.stdout.splitlines():
                if line.startswith("mykernel_time:"):
                    rec["ms"] = float(line.split()[1])
                    rec["gflops"] = 2.0 * m.nnz * args.n / (rec["ms"] * 1e-3) / 1e9
                if line.startswith("cusparse_time:"):
                    rec["cusparse_ms"] = float(line.split()[1])
                if line.startswith("VERIFICATION"):
                    rec["verification"] = line[len("VERIFICATION "):]
            out[label] = rec
    print(json.dumps({"metric": "SpMM through the reference's Format-DSL bridge executable, kernel ms", "unit": "ms", "n_gpus": 1,
                      "config": {"workload": args.workload, "M": m.M, "nnz": m.nnz, "N": args.n}, "bridge": out}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="mask_b200", choices=["mask_b200", "reference"])
    ap.add_argument("--workload", default="rmat22_sym")
    ap.add_argument("--scale", type=int, default=None, help="shrink the workload (R-MAT scale / grid / n)")
    ap.add_argument("--n", "--cols", dest="n", type=int, default=512, help="columns of B (use --cols under torchrun, whose own parser claims --n)")
    ap.add_argument("--format", default="srbcrs", choices=["srbcrs", "metcf", "mco"])
    ap.add_argument("--policy", default="auto")
    ap.add_argument("--group-tiles", type=int, default=0)
    ap.add_argument("--session-chunk", type=int, default=-1, help="columns per chunk of the host-buffer pipeline (-1 automatic, 0 off)")
    ap.add_argument("--sweep", type=int, default=1, help="1 = tcgen05 kernel except where the warp-level one measures faster, 2 = always, 0 = warp-level kernels only")
    ap.add_argument("--nslab", type=int, default=0, help="tcgen05 kernel: 128-column slabs per sweep (0 = the plan table's choice)")
    ap.add_argument("--calibrate", type=int, default=2, help="multi-GPU: rounds of measured re-balancing of the row panels before the timed region (0 = cost model only)")
    ap.add_argument("--e2e-steps", type=int, default=3, help="0 skips the host-buffer leg")
    ap.add_argument("--nq", type=int, default=0, help="kernel variant: 32-column groups per warp (0 = default)")
    ap.add_argument("--min-blocks", type=int, default=0, help="kernel variant: occupancy target (0 = default)")
    ap.add_argument("--stages", type=int, default=0, help="kernel variant: ring slots per warp (0 = default)")
    ap.add_argument("--no-async", action="store_true", help="use the register-pipelined kernel")
    ap.add_argument("--bridge", action="store_true",
                    help="time the reference's Format-DSL bridge executable with its emitted operator and with the sm_100a one (extra line)")
    ap.add_argument("--gcn-fused", action="store_true", help="with --gcn: layer-1 SpMM stores H1 straight into every rank's copy")
    ap.add_argument("--gcn", action="store_true", help="time the row-sharded 2-layer GCN forward instead (extra line)")
    ap.add_argument("--baselines", action="store_true",
                    help="also time cuSPARSE (torch.sparse CSR) and the reference's own SR-BCRS kernel recompiled for sm_100a")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline / verification leg")
    ap.add_argument("--no-tf32-probe", action="store_true", help="skip the dense TF32 GEMM peak measurement")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl != "reference" else args.warmup
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist
    from mask_b200 import _lib, engine, generators as G

    # keep stdout to the one JSON line: NCCL's version banner (NCCL_DEBUG=VERSION) goes to stderr
    os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
    if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
        os.environ["NCCL_DEBUG"] = "WARN"
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    N = args.n
    engine.tune("nq", args.nq)
    engine.tune("min_blocks", args.min_blocks)
    engine.tune("stages", args.stages)
    engine.tune("sweep", args.sweep)
    engine.tune("nslab", args.nslab)
    engine.tune("session_chunk", args.session_chunk)
    engine.tune("async", 0 if args.no_async else 1)

    m, bseed = build_workload(args.workload, args.scale)
    dev = torch.device("cuda", local)
    if args.gcn:
        return run_gcn(args, m, bseed, dev, rank, world)
    if args.bridge:
        return run_bridge(args, m) if rank == 0 else None
    bounds, cost_prefix = panel_bounds(m, world, dev)
    Bd, Bh, b_source = dense_operand(m.K, N, bseed, dev)

    def prepare(bounds):
        """Packs this rank's panel and plans it."""
        r0, r1 = bounds[rank], bounds[rank + 1]
        panel = m.row_slice(r0, r1) if world > 1 else m
        rp, ci, va = (torch.from_numpy(np.ascontiguousarray(x)).to(dev) for x in (panel.rowptr, panel.colind, panel.values))
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        packed = {"srbcrs": engine.pack_srbcrs, "metcf": engine.pack_metcf, "mco": engine.pack_mco}[args.format](rp, ci, va, panel.M, panel.K)
        torch.cuda.synchronize()
        pack_ms = (time.perf_counter() - t0) * 1e3
        distinct = int(torch.unique(ci).numel()) if panel.nnz else 0
        del rp, va, ci
        plan = packed.new_plan(args.policy, args.group_tiles)
        out = torch.empty((panel.M, N), dtype=torch.float32, device=dev)
        return panel, packed, plan, out, pack_ms, distinct

    panel, packed, plan, out, pack_ms, distinct = prepare(bounds)
    # Measured balance: the cost model cannot see what L2 does with a panel, so the ranks time a few
    # products, share the times and re-cut the panels from them (at most --calibrate times, outside the
    # timed region; the matrix is packed again only on the ranks whose panel moved).
    calibration = []
    for _ in range(args.calibrate if world > 1 else 0):
        from mask_b200.sharding import rebalanced_panels
        for _ in range(2):
            engine.spmm(packed, Bd, out=out, plan=plan)
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.barrier()
        c0.record()
        for _ in range(3):
            engine.spmm(packed, Bd, out=out, plan=plan)
        c1.record()
        torch.cuda.synchronize()
        mine = torch.tensor([c0.elapsed_time(c1) / 3.0], dtype=torch.float64, device=dev)
        every = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(every, mine)
        times = [float(x.item()) for x in every]
        calibration.append([round(x, 4) for x in times])
        if max(times) <= 1.03 * (sum(times) / world):
            break
        new_bounds = rebalanced_panels(cost_prefix, m.M, bounds, times)
        moved = (new_bounds[rank], new_bounds[rank + 1]) != (bounds[rank], bounds[rank + 1])
        bounds = new_bounds
        if moved:
            del packed, plan, out
            torch.cuda.empty_cache()
            panel, packed, plan, out, pack_ms, distinct = prepare(bounds)
    r0, r1 = bounds[rank], bounds[rank + 1]
    info = plan.info()
    launches_per_step = 1 + (1 if info["partial"] > 0 else 0)
    log(f"[bench] rank {rank}: rows [{r0},{r1}) nnz={panel.nnz} T={packed.T} pack {pack_ms:.1f} ms plan {info}")

    def step():
        engine.spmm(packed, Bd, out=out, plan=plan)

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    with ClockSampler(local) as clocks:
        ev[0].record()
        for i in range(args.steps):
            step()
            ev[i + 1].record()
        torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    kernel_status = plan.status()
    if kernel_status != 0:
        raise RuntimeError("a kernel gave up on a bounded wait during the timed region; the result is invalid")
    total_ms = ev[0].elapsed_time(ev[-1])
    per_launch = [ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps)]
    t = torch.tensor([total_ms], dtype=torch.float64, device=dev)
    per_rank_ms = [total_ms / args.steps]
    if world > 1:
        every = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(every, t)
        per_rank_ms = [float(x.item()) / args.steps for x in every]
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = float(t.item()) / args.steps
    value = 2.0 * m.nnz * N / (ms_per_step * 1e-3) / 1e9

    # ---- verification: every rank checks sample rows of its own panel against the CPU oracle ----
    verified = None
    sample = None
    if not args.no_cpu:
        import oracle
        # whole C for the configurations up to 2^20 rows on one GPU; else 65 536 seeded rows and the 1024
        # heaviest windows over the job, every rank taking its share from its own panel
        sample = VerifySample(oracle, panel, packed.val_soff.cpu().numpy(), Bd, seed=7 + rank,
                              n_random=max(4096, 65536 // world), n_heavy=max(8, 1024 // world),
                              full=(world == 1 and panel.M <= (1 << 20)))
        bad, worst = sample.check(out)
        counts = torch.tensor([bad, sample.rows.size], dtype=torch.int64, device=dev)
        worst_t = torch.tensor([worst], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(counts, op=dist.ReduceOp.SUM)
            dist.all_reduce(worst_t, op=dist.ReduceOp.MAX)
        verified = {"rows_checked": int(counts[1].item()), "violations": int(counts[0].item()),
                    "worst_ratio": float(worst_t.item()), "ranks_checked": world,
                    "how": f"rank 0 of {world}: {sample.how} of its panel (every rank likewise), CPU oracle FP32 SpMM",
                    "tolerance": "|C-Cref| <= 2e-3*(|A|.|B|) + 1e-6"}
        if bad:
            log(f"[bench] rank {rank}: VERIFICATION FAILED: {bad} elements outside tolerance")
        if args.format == "srbcrs":   # the packed arrays themselves, byte for byte against the oracle's packing
            wrong, w_cmp, t_cmp = packing_parity(oracle, panel, packed)
            pk = torch.tensor([len(wrong), w_cmp, t_cmp], dtype=torch.int64, device=dev)
            if world > 1:
                dist.all_reduce(pk, op=dist.ReduceOp.SUM)
            verified["packing"] = {"mismatching_arrays": int(pk[0].item()), "windows_compared": int(pk[1].item()),
                                   "tiles_compared": int(pk[2].item()),
                                   "how": "val_soff, val_sidx, val_block_val of every rank's panel (leading windows up to 2^24 "
                                          "stored entries) byte for byte against the CPU oracle's packing"}
            if wrong:
                log(f"[bench] rank {rank}: PACKING MISMATCH in {wrong}")

    # ---- end to end with host buffers ----
    e2e = None
    try:
        if args.e2e_steps <= 0:
            raise RuntimeError("skipped (--e2e-steps 0)")
        if world == 1:
            e2e, host_rows = e2e_single(args, m, packed, Bd, Bh, sample)
        else:
            e2e, host_rows = e2e_sharded(args, m, panel, packed, plan, Bd, dev, rank, world, sample)
        if sample is not None and host_rows is not None:
            bad2, _ = sample.check_host(host_rows)
            bt = torch.tensor([bad2], dtype=torch.int64, device=dev)
            if world > 1:
                dist.all_reduce(bt, op=dist.ReduceOp.SUM)
            verified["e2e_violations"] = int(bt.item())
    except Exception as e:  # the headline device number must still be printed
        log(f"[bench] rank {rank}: e2e leg failed: {e!r}")
        e2e = None

    # ---- dense TF32 GEMM peak of this GPU (denominator of the tensor-core bound) ----
    tf32_tflops = None
    try:
        if args.no_tf32_probe:
            raise RuntimeError("skipped (--no-tf32-probe)")
        torch.backends.cuda.matmul.allow_tf32 = True
        ga = torch.randn(8192, 8192, device=dev)
        gb = torch.randn(8192, 8192, device=dev)
        best = 1e9
        for i in range(8):
            g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            g0.record()
            torch.matmul(ga, gb)
            g1.record()
            torch.cuda.synchronize()
            if i >= 2:
                best = min(best, g0.elapsed_time(g1))
        tf32_tflops = 2.0 * 8192 ** 3 / (best * 1e-3) / 1e12
        del ga, gb
    except Exception as e:
        log(f"[bench] TF32 peak measurement failed: {e}")

    # ---- roofline of the dominant kernel (rank-local) ----
    hbm_gbs, peak_src = measured_peaks()
    W = (panel.M + 15) // 16
    G_rows = int(packed.T) * 8  # upper bound of rows fetched without inter-window reuse (incl. padding)
    if args.format == "srbcrs":
        bytes_alg = algorithmic_bytes(packed.T, W, panel.M, N, distinct)
    elif args.format == "metcf":
        bytes_alg = 8 * packed.nnz_pad + 4 * (2 * packed.T + 1) + 4 * (8 * packed.T + W + 1) + 4 * N * distinct + 4 * panel.M * N
    else:  # MCO: 16 B of mask and one offset per tile, the compact values
        bytes_alg = 4 * packed.nval + 20 * packed.T + 4 + 4 * (8 * packed.T + W + 1) + 4 * N * distinct + 4 * panel.M * N
    kernel_ms = float(np.mean(per_launch))
    achieved = bytes_alg / (kernel_ms * 1e-3) / 1e9
    kernel_name, kernel_rev = engine.kernel_signature(packed, N, plan)
    traffic = None
    cap = NCU_TRAFFIC.get((args.workload, args.scale, N, args.format))
    if world == 1 and cap is not None and cap["kernel"] == kernel_name and cap["revision"] == kernel_rev:
        traffic = cap["bytes"]   # only while the library still runs the kernel revision that was captured
    roofline = {"bound": "hbm", "achieved": achieved, "peak": hbm_gbs, "unit": "GB/s", "frac": achieved / hbm_gbs,
                "traffic": traffic, "traffic_capture": cap["capture"] if traffic is not None else None,
                "peak_source": peak_src, "bytes_algorithmic": bytes_alg,
                "kernel_ms": kernel_ms, "kernel": kernel_name + (" (+ spmm_fixup_kernel)" if info["partial"] else ""),
                "kernel_revision": kernel_rev,
                "bytes_gather_no_reuse": bytes_alg - 4 * N * distinct + 4 * N * G_rows,
                "padded_tile_tflop": 256.0 * packed.T * N / 1e12,
                "tf32_dense_peak_tflops_measured": tf32_tflops,
                "tensor_bound_ms": (256.0 * packed.T * N / 1e12) / tf32_tflops * 1e3 if tf32_tflops else None,
                "hbm_bound_ms": bytes_alg / (hbm_gbs * 1e9) * 1e3}

    # ---- CPU baseline: the oracle's host SpMM on a bounded sample (rank 0, single GPU only) ----
    cpu = None
    if world == 1 and not args.no_cpu:
        cpu = cpu_baseline(m, N, Bd, Bh)

    # ---- same-box GPU baselines (rank 0, single GPU, on request) ----
    gpu_baselines = None
    if args.baselines and world == 1 and args.format == "srbcrs":
        gpu_baselines = {}
        if Bh is None:
            Bh = Bd.cpu().numpy()
        rp = torch.from_numpy(np.ascontiguousarray(panel.rowptr)).to(dev)
        va = torch.from_numpy(np.ascontiguousarray(panel.values)).to(dev)
        ci = torch.from_numpy(np.ascontiguousarray(panel.colind)).to(dev)
        try:
            A_t = torch.sparse_csr_tensor(rp.to(torch.int64), ci.to(torch.int64), va, size=(m.M, m.K))
            for _ in range(3):
                ref_out = torch.sparse.mm(A_t, Bd)
            torch.cuda.synchronize()
            c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            c0.record()
            for _ in range(10):
                ref_out = torch.sparse.mm(A_t, Bd)
            c1.record()
            torch.cuda.synchronize()
            cms = c0.elapsed_time(c1) / 10
            gpu_baselines["cusparse_csr_fp32"] = {"ms": cms, "gflops": 2.0 * m.nnz * N / (cms * 1e-3) / 1e9,
                                                  "how": "torch.sparse.mm (CSR, FP32) on the same inputs"}
            del A_t, ref_out
        except Exception as e:
            gpu_baselines["cusparse_csr_fp32"] = {"error": str(e)[:200]}
        try:
            import oracle
            if not oracle.ref_gpu_available():
                raise RuntimeError("oracle/_ref/libref_gpu_srbcrs.so not built")
            host_packed = {k: getattr(packed, k).cpu().numpy() for k in ("val_soff", "val_sidx", "val_block_val")}
            host_packed["T"] = packed.T
            rC, rms = oracle.ref_gpu_srbcrs(m.M, N, m.K, host_packed, Bh, warmup=3, repeat=10)
            agree = float(np.abs(rC[:4096] - out[:4096].cpu().numpy()).max())
            gpu_baselines["reference_srbcrs_16x8_kernel_sm100a"] = {
                "ms": rms, "gflops": 2.0 * m.nnz * N / (rms * 1e-3) / 1e9, "max_abs_diff_first_4096_rows": agree,
                "how": "sr_bcrs_spmm_kernel_tf32 of the reference (kernel.inc) recompiled for sm_100a, its own grid mapping"}
        except Exception as e:
            gpu_baselines["reference_srbcrs_16x8_kernel_sm100a"] = {"error": str(e)[:200]}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "tf32", "data": "synthetic",
            "config": {"workload": args.workload + (f" scale={args.scale}" if args.scale else ""), "M": m.M, "K": m.K,
                       "nnz": m.nnz, "N": N, "format": {"srbcrs": "SR-BCRS 16x8", "metcf": "ME-TCF", "mco": "MCO / BIT-TCF"}[args.format],
                       "B": b_source,
                       "tiles_rank0": packed.T, "policy": args.policy, "plan": info, "pack_ms_rank0": pack_ms,
                       "partition": "row panels on window boundaries balanced by tiles + 5 per window, B replicated" if world > 1 else "none",
                       "panel_rows": [bounds[i + 1] - bounds[i] for i in range(world)],
                       "per_rank_ms": [round(x, 4) for x in per_rank_ms],
                       "calibration_ms": calibration,
                       "l2": "no flush needed: B and C (M*N*4 bytes each) are far larger than the 126 MB L2" if 4 * m.M * N > (1 << 29)
                             else "inputs smaller than L2: the timed loop reuses them (L2-resident regime of this configuration)"},
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks.summary(), "verified": verified, "kernel_status": kernel_status, "gpu_baselines": gpu_baselines,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
