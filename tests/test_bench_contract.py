"""The JSON line bench.py prints: keys and types the measurement contract asks for.  The CPU arm
(--impl reference) runs anywhere; the GPU arm needs a B200."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BASE_KEYS = {"metric": str, "value": float, "unit": str, "n_gpus": int, "steps": int, "warmup": int, "ms_per_step": float,
             "higher_is_better": bool, "scaling": str, "dtype": str, "data": str, "config": dict}


def _run(*args):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1, "exactly one JSON line on stdout"
    return json.loads(lines[0])


def _check_base(d):
    for k, t in BASE_KEYS.items():
        assert k in d and isinstance(d[k], t), k
    assert "vs_baseline" in d and d["vs_baseline"] is None      # no published number for this exact metric
    assert "workload" in d["config"] and "model" not in d["config"]
    assert d["higher_is_better"] is True and d["value"] > 0 and d["ms_per_step"] > 0


def test_reference_arm_line():
    d = _run("--impl", "reference", "--scale", "12", "--steps", "2", "--warmup", "1")
    _check_base(d)
    assert d["impl"] == "reference" and d["dtype"] == "f32" and d["n_gpus"] == 1
    cb = d["cpu_baseline"]
    assert cb["kind"] in ("port", "reference") and cb["cores"] >= 1 and cb["sample"] and cb["value"] == d["value"]
    e = d["e2e"]
    assert e["value"] == d["value"] and e["unit"] == d["unit"] and e["h2d_bytes_per_step"] == 0 and e["d2h_bytes_per_step"] == 0
    assert d.get("gpu_launches", 0) == 0


@pytest.mark.gpu
def test_gpu_arm_line():
    d = _run("--scale", "14", "--steps", "3", "--warmup", "3", "--e2e-steps", "2")
    _check_base(d)
    assert d["n_gpus"] == 1 and d["steps"] == 3 and d["warmup"] == 3 and d["dtype"] == "tf32" and d["scaling"] in ("weak", "strong")
    rf = d["roofline"]
    assert rf["bound"] in ("hbm", "tensor") and rf["unit"] in ("GB/s", "TFLOP/s")
    assert abs(rf["frac"] - rf["achieved"] / rf["peak"]) < 1e-9 and "traffic" in rf
    cb = d["cpu_baseline"]
    assert cb["kind"] in ("port", "reference") and cb["cores"] >= 1 and cb["value"] > 0 and cb["sample"]
    e = d["e2e"]
    assert e["value"] > 0 and e["h2d_bytes_per_step"] > 0 and e["d2h_bytes_per_step"] > 0 and e["value"] != d["value"]
    assert d["gpu_launches"] >= d["steps"]
    ck = d["clocks"]
    assert ck["sm_mhz"] > 0 and ck["sm_max_mhz"] >= ck["sm_mhz"] and isinstance(ck["reasons"], list)
    assert d["kernel_status"] == 0 and d["verified"]["violations"] == 0


def test_verification_sampler_on_host_tensors():
    """bench.VerifySample with CPU tensors: the whole matrix, or seeded rows plus the heaviest windows within
    the entry budget; a single corrupted element of a sampled row is reported."""
    import numpy as np
    import torch
    sys.path.insert(0, ROOT)
    import bench
    import oracle
    from mask_b200 import generators as G
    m = G.rmat_gcn_normalised(scale=11, samples_per_node=8, seed=201)
    B = torch.from_numpy(G.dense_normal(m.K, 32, 5))
    soff = oracle.pack_srbcrs(m.M, m.rowptr, m.colind, m.values)["val_soff"]
    ref = torch.from_numpy(oracle.spmm_f32(m.M, m.rowptr, m.colind, m.values, B.numpy()))
    full = bench.VerifySample(oracle, m, soff, B, seed=7, n_random=100, n_heavy=4, full=True)
    assert full.rows.size == m.M and full.check(ref)[0] == 0
    part = bench.VerifySample(oracle, m, soff, B, seed=7, n_random=300, n_heavy=40, full=False, heavy_entries=4000)
    assert 300 * 0.8 < part.rows.size < m.M and "heaviest windows" in part.how
    heaviest = int(np.argmax(np.diff(soff)))
    assert set(range(heaviest * 16, heaviest * 16 + 16)) <= set(part.rows.tolist())   # the heaviest window is always in
    assert part.check(ref)[0] == 0
    bad = ref.clone()
    bad[int(part.rows[5]), 3] += 1.0
    assert part.check(bad)[0] == 1 and part.check_host(bad[torch.from_numpy(part.rows)].numpy())[0] == 1
