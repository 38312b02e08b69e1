"""Writes tests/golden/bridge_plans.json: the reference's own ``select_backend`` output for the
SR-BCRS 16x8 mapping (plain and with each row reorder), imported from a checkout of the reference
named by $MASK_REF.  tests/test_bridge_host.py compares mask_b200.bridge with it.

    python tests/golden/make_bridge_plan.py
"""
import json
import os
import sys

ref = os.environ["MASK_REF"]   # the checkout must be named: there is no default location
sys.path.insert(0, os.path.join(ref, "python"))
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from sparsene.op_gen.backend_registry import select_backend  # noqa: E402  (the reference)

from mask_b200 import bridge  # noqa: E402

out = {}
for reorder in (None, "row_rcm", "first_col_sort", "jaccard_greedy"):
    for tile_n in (64, 128):
        spec = bridge.sr_bcrs_spec(reorder)
        plan = select_backend(spec, target="sm80", tile_n=tile_n, max_tiles_per_execution_segment=32)
        out[f"{reorder}/{tile_n}"] = {"spec": spec, "plan": plan.to_dict()}
path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "bridge_plans.json")
json.dump(out, open(path, "w"), indent=1, sort_keys=True)
print(path, len(out))
