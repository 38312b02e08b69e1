// Build check for include/mask_b200_operator_sm100.inc without the reference tree: the include is
// compiled for sm_100a with the macro the bridge defines before it, and its three kernels are
// instantiated with stand-ins for the bridge's shape types (the operator reads none of them).
// The object is not linked into the library.
#define SPARSENE_TILE_N 64
#include "../../include/mask_b200_operator_sm100.inc"

namespace {
struct ShapeStandIn {};
}

template __global__ void generated_kernel<ShapeStandIn, ShapeStandIn, ShapeStandIn, ShapeStandIn>(float*, float*, int*, float*, int*,
                                                                                             int, int, int, int, int);
template __global__ void generated_task_mapped_kernel<ShapeStandIn, ShapeStandIn, ShapeStandIn, ShapeStandIn>(
    float*, float*, int*, float*, int*, const int*, const int*, const int*, const int*, const int*, int, int, int, int, int);
template __global__ void generated_bound_task_kernel<ShapeStandIn, ShapeStandIn, ShapeStandIn, ShapeStandIn>(
    float*, float*, int*, float*, int*, const int*, const int*, const int*, int, int, int, int, int);

static_assert(SPARSENE_GENERATED_REQUIRES_SINGLE_WARP == 1 && SPARSENE_GENERATED_THREADS_PER_BLOCK == 32, "bridge contract");
