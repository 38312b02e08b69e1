"""Test infrastructure: runs the reference project's own Format -> CUDA compiler (imported from a
checkout named by $MASK_REF) on its built-in SR-BCRS 16x8 format and writes the
emitted operator include to oracle/_ref/gen/operators/sr_bcrs_16x8.inc.  That file is the
reference-generated kernel the DSL host bridge is built with for same-box comparisons; it is a
build product of the reference and is not kept in the history.

    python oracle/gen_ref_operator.py [tile_n]
"""
import os
import sys
from pathlib import Path

ref = Path(os.environ["MASK_REF"])   # the checkout must be named: there is no default location
sys.path.insert(0, str(ref / "python"))
sys.path.insert(0, str(ref / "python" / "test"))
here = Path(__file__).resolve().parent
out = here / "_ref" / "gen"
out.mkdir(parents=True, exist_ok=True)
os.chdir(out)

import run_builtin_backend_e2e as R  # noqa: E402  (the reference's own driver module)

tile_n = int(sys.argv[1]) if len(sys.argv) > 1 else 64
m = R.generate_candidate(out, tile_n=tile_n, max_tiles=32)
print(m["operator_path"], m["backend_plan"])
