"""The `sm100` target of the reference's Format-DSL bridge, host side.

The reference selects an executable backend for a Format-DSL mapping with
``select_backend(spec, target="sm80", tile_n=…)`` (python/sparsene/op_gen/backend_registry.py:77-303),
lowers the format to a CUDA operator include, and configures the bridge testbed
``examples/src_fp32/acc/testbed`` with that include (python/test/run_custom_format_e2e.py:56-118).
It rejects every target but sm80/a800 (backend_registry.py:223-224).  This module is what an
``sm100`` target adds: the same plan for the formats whose kernels exist here (column-condensed
dense tiles = SR-BCRS, with or without a row reorder, and its sparse-row variant), the path of the
hand-written operator include instead of a lowering step, and the same configure command.

Field names, values and error behaviour (``ValueError``) follow the reference so that its runners
can consume the plan unchanged; only ``target`` / ``compute_capability`` differ.
"""
from __future__ import annotations

import os
from dataclasses import asdict, dataclass
from typing import Any, Mapping

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
OPERATOR_INCLUDE = os.path.join(_ROOT, "include", "mask_b200_operator_sm100.inc")
REORDER_CODES = {None: 0, "row_rcm": 1, "first_col_sort": 2, "jaccard_greedy": 3}
PACKING_CODES = {"column_condensed_dense": 2, "sparse_row_column_condensed_dense": 4}


@dataclass(frozen=True)
class BackendPlan:
    backend: str
    codegen_format_name: str
    target: str
    compute_capability: int
    logical_blk_m: int
    logical_blk_k: int
    physical_blk_m: int
    physical_blk_k: int
    tile_n: int
    mma_m: int
    mma_n: int
    mma_k: int
    max_tiles_per_execution_segment: int
    packing_mode: str
    row_reorder: str | None
    notes: tuple[str, ...]
    logical_inner_blk_k: int | None = None

    def to_dict(self) -> dict[str, Any]:
        return asdict(self)


def sr_bcrs_spec(row_reorder: str | None = None) -> dict[str, Any]:
    """The Format-DSL mapping of SR-BCRS 16x8 (python/sparsene/formats/SR_BCRS.py:5-20)."""
    x_o = {"name": "X_o", "type": "df", "direction": "ROW", "length": "M"}
    if row_reorder:
        x_o["reorder"] = row_reorder
    return {
        "format_name": "SR_BCRS_16x8",
        "levels": [
            {"level": 1, "name": "row_window", "axes": [
                x_o,
                {"name": "Y_s", "type": "sv", "direction": "COL", "length": "K"},
                {"name": "X_i", "type": "df", "direction": "ROW", "length": "BLK_M"}]},
            {"level": 2, "name": "condensed_block", "axes": [
                {"name": "Y_so", "type": "df", "direction": "COL", "length": "K/BLK_K"},
                {"name": "Y_si", "type": "df", "direction": "COL", "length": "BLK_K"},
                {"name": "X_i", "type": "df", "direction": "ROW", "length": "BLK_M"}]},
        ],
        "atomic": {"type": "dense", "x_axis": "X_i", "y_axis": "Y_si", "layout": "row_major"},
        "params": {"BLK_M": 16, "BLK_K": 8},
    }


def _axes(level: Mapping[str, Any]) -> dict[str, Mapping[str, Any]]:
    return {str(a.get("name")): a for a in level.get("axes", [])}


def _expect(axes, name, types, direction):
    a = axes.get(name)
    if a is None:
        raise ValueError(f"sm100 tensor-core backend requires axis {name}")
    if a.get("type") not in types or a.get("direction") != direction:
        raise ValueError(f"axis {name} must be one of {sorted(types)}/{direction}, got {a.get('type')}/{a.get('direction')}")
    return a


def select_backend(spec: Mapping[str, Any], *, target: str = "sm100", tile_n: int = 64,
                   max_tiles_per_execution_segment: int = 32) -> BackendPlan:
    """The reference's selection rules for the dense-leaf column-condensed hierarchies, with the
    checks of the hand-written operator: BLK_M = 16, BLK_K = 8, tile_n 32 / 64 / 128."""
    if target not in {"sm100", "b200"}:
        raise ValueError(f"Unknown target {target!r}; available target: sm100/b200")
    levels = spec.get("levels", [])
    atomic = spec.get("atomic", {})
    params = spec.get("params", {})
    if atomic.get("type") != "dense":
        raise ValueError("No sm100 backend for this design: the hand-written operator takes a dense atomic leaf")
    if len(levels) == 2:
        outer, inner = _axes(levels[0]), _axes(levels[1])
        x_outer = _expect(outer, "X_o", {"df"}, "ROW")
        _expect(outer, "Y_s", {"sv"}, "COL")
        _expect(outer, "X_i", {"df"}, "ROW")
        _expect(inner, "Y_so", {"df", "dv"}, "COL")
        _expect(inner, "Y_si", {"df"}, "COL")
        _expect(inner, "X_i", {"df"}, "ROW")
        if atomic.get("x_axis") != "X_i" or atomic.get("y_axis") != "Y_si":
            raise ValueError("TCF leaf must map x_axis=X_i and y_axis=Y_si")
        packing_mode, backend = "column_condensed_dense", "sr_bcrs_dense_tensorcore_v1"
    elif len(levels) == 3:
        sparse_rows, outer, inner = _axes(levels[0]), _axes(levels[1]), _axes(levels[2])
        x_outer = _expect(sparse_rows, "X_s", {"sv"}, "ROW")
        _expect(sparse_rows, "Y", {"df"}, "COL")
        _expect(outer, "X_so", {"df"}, "ROW")
        _expect(outer, "Y_s", {"sv"}, "COL")
        _expect(outer, "X_si", {"df"}, "ROW")
        _expect(inner, "Y_so", {"df", "dv"}, "COL")
        _expect(inner, "Y_si", {"df"}, "COL")
        _expect(inner, "X_si", {"df"}, "ROW")
        if atomic.get("x_axis") != "X_si" or atomic.get("y_axis") != "Y_si":
            raise ValueError("sparse-row dense leaf must map x_axis=X_si and y_axis=Y_si")
        packing_mode, backend = "sparse_row_column_condensed_dense", "sparse_row_sr_bcrs_dense_tensorcore_v1"
    else:
        raise ValueError("No sm100 backend for this hierarchy: expected two-level column condensation or sparse-row SR-BCRS")
    if atomic.get("layout", "row_major") != "row_major":
        raise ValueError("tensor-core backends require a row-major atomic leaf")
    reorders = {a.get("reorder") for lv in levels for a in lv.get("axes", []) if a.get("reorder") is not None}
    if len(reorders) > 1 or not reorders.issubset({"row_rcm", "first_col_sort", "jaccard_greedy"}):
        raise ValueError(f"Unsupported reorder contract: {sorted(reorders)}")
    row_reorder = next(iter(reorders), None)
    if row_reorder and x_outer.get("reorder") != row_reorder:
        raise ValueError("row reorder must be attached to the outer sparse/dense row axis")
    if packing_mode == "sparse_row_column_condensed_dense" and row_reorder:
        raise ValueError("sparse-row physicalization does not yet compose with an additional row reorder")
    try:
        blk_m, blk_k = int(params["BLK_M"]), int(params["BLK_K"])
    except (KeyError, TypeError, ValueError) as exc:
        raise ValueError("Tensor-core backend requires concrete integer BLK_M and BLK_K") from exc
    if blk_m != 16 or blk_k != 8:
        raise ValueError(f"the sm100 operator implements BLK_M=16, BLK_K=8, got {blk_m}x{blk_k}")
    if tile_n not in (32, 64, 128):
        raise ValueError(f"the sm100 operator supports tile_n 32, 64 or 128, got {tile_n}")
    if max_tiles_per_execution_segment < 1:
        raise ValueError("max_tiles_per_execution_segment must be positive")
    notes = ["Format conversion, optional row reorder, and output inverse mapping are outside timing.",
             "All generated GPU work, including work on physically padded zeros, is inside timing.",
             "Hand-written sm_100a operator include; no lowering step."]
    return BackendPlan(backend=backend, codegen_format_name="SR_BCRS", target="sm100", compute_capability=100,
                       logical_blk_m=16, logical_blk_k=8, physical_blk_m=16, physical_blk_k=8, tile_n=tile_n,
                       mma_m=16, mma_n=8, mma_k=8, max_tiles_per_execution_segment=max_tiles_per_execution_segment,
                       packing_mode=packing_mode, row_reorder=row_reorder, notes=tuple(notes))


def generation_manifest(plan: BackendPlan, operator_path: str = OPERATOR_INCLUDE) -> dict[str, Any]:
    """What the reference's ``generate_candidate`` writes (python/test/run_builtin_backend_e2e.py:79-114),
    for the hand-written operator."""
    return {
        "schema_version": "sparsene.builtin_backend_generation.v1",
        "candidate": "sr_bcrs_16x8_sm100",
        "format_source": "python/sparsene/formats/SR_BCRS.py::SR_BCRS_FORMAT",
        "agent_independent": True,
        "backend_plan": plan.to_dict(),
        "operator_path": os.path.abspath(operator_path),
        "launch_contract": {"threads_per_block": 32, "warps_per_block": 1, "synchronization": "warp", "lowered_block_barriers": 0},
        "performance_contract": "sparsene.kernel_only_post_conversion.v1",
    }


def cmake_configure_command(plan: BackendPlan, testbed_dir: str, build_dir: str, operator_path: str = OPERATOR_INCLUDE,
                            fast_tf32: bool = False) -> list[str]:
    """The configure command of ``compile_one`` (python/test/run_custom_format_e2e.py:56-100) for this plan."""
    cmd = ["cmake", "-S", str(testbed_dir), "-B", str(build_dir), "-DCMAKE_BUILD_TYPE=Release",
           f"-DSPARSENE_GENERATED_OPERATOR={os.path.abspath(operator_path)}",
           f"-DSPARSENE_LOGICAL_BLK_M={plan.logical_blk_m}", f"-DSPARSENE_PHYSICAL_BLK_M={plan.physical_blk_m}",
           f"-DSPARSENE_BLK_K={plan.physical_blk_k}", f"-DSPARSENE_LOGICAL_BLK_K={plan.logical_blk_k}",
           f"-DSPARSENE_TILE_N={plan.tile_n}", f"-DSPARSENE_ROW_REORDER={REORDER_CODES[plan.row_reorder]}",
           f"-DSPARSENE_PACKING_MODE={PACKING_CODES[plan.packing_mode]}",
           f"-DSPARSENE_MAX_TILES_PER_SEGMENT={plan.max_tiles_per_execution_segment}",
           "-DSPARSENE_CUSTOM_CUDA_ARCHITECTURES=100a"]
    if fast_tf32:
        cmd.append("-DCMAKE_CUDA_FLAGS=-DSPARSENE_FAST_TF32")
    return cmd
