"""Host side of the `sm100` bridge target: the plan for the SR-BCRS mapping must be the reference's
own plan (tests/golden/bridge_plans.json, written by the reference's select_backend) up to the
target fields, and unsupported designs are refused the way the reference refuses them."""
import copy
import json
import os

import pytest

from mask_b200 import bridge

HERE = os.path.dirname(os.path.abspath(__file__))
GOLD = json.load(open(os.path.join(HERE, "golden", "bridge_plans.json")))


@pytest.mark.parametrize("key", sorted(GOLD))
def test_plan_matches_the_reference_plan(key):
    want = GOLD[key]["plan"]
    reorder, tile_n = key.split("/")
    reorder = None if reorder == "None" else reorder
    spec = bridge.sr_bcrs_spec(reorder)
    assert spec == GOLD[key]["spec"]
    got = bridge.select_backend(spec, tile_n=int(tile_n)).to_dict()
    for field in want:
        if field in ("target", "compute_capability", "notes"):
            continue
        assert got[field] == want[field], field
    assert got["target"] == "sm100" and got["compute_capability"] == 100
    assert list(got["notes"][:2]) == list(want["notes"][:2])


def test_refusals():
    spec = bridge.sr_bcrs_spec()
    with pytest.raises(ValueError):
        bridge.select_backend(spec, target="sm80")
    with pytest.raises(ValueError):
        bridge.select_backend(spec, tile_n=48)
    for mutate in (lambda s: s["atomic"].update(type="mco"), lambda s: s["params"].update(BLK_M=32),
                   lambda s: s["params"].pop("BLK_K"), lambda s: s["atomic"].update(layout="col_major"),
                   lambda s: s["levels"].pop(), lambda s: s["levels"][0]["axes"][1].update(type="df"),
                   lambda s: s["levels"][1]["axes"][0].update(reorder="row_rcm"),
                   lambda s: s["levels"][0]["axes"][0].update(reorder="hilbert")):
        bad = copy.deepcopy(spec)
        mutate(bad)
        with pytest.raises(ValueError):
            bridge.select_backend(bad)


def test_manifest_and_configure_command():
    plan = bridge.select_backend(bridge.sr_bcrs_spec("first_col_sort"), tile_n=128)
    man = bridge.generation_manifest(plan)
    assert os.path.isfile(man["operator_path"]) and man["backend_plan"]["tile_n"] == 128
    assert man["launch_contract"]["threads_per_block"] == 32
    cmd = bridge.cmake_configure_command(plan, "/ref/examples/src_fp32/acc/testbed", "/tmp/b")
    assert f"-DSPARSENE_GENERATED_OPERATOR={man['operator_path']}" in cmd
    for want in ("-DSPARSENE_TILE_N=128", "-DSPARSENE_ROW_REORDER=2", "-DSPARSENE_PACKING_MODE=2", "-DSPARSENE_BLK_K=8",
                 "-DSPARSENE_LOGICAL_BLK_M=16", "-DSPARSENE_PHYSICAL_BLK_M=16", "-DSPARSENE_CUSTOM_CUDA_ARCHITECTURES=100a"):
        assert want in cmd
