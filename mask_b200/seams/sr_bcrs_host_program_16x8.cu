// Drop-in replacement for the reference testbed's host program
// examples/src_fp32/sr_bcrs/testbed/host_program_16x8.cu: it defines the function the testbed's
// main_16x8.cu declares (main_16x8.cu:32-44) -- host pointers to the packed SR-BCRS arrays and to
// B in, C (M x N, host) out, "mykernel_time: <ms> ms" on stdout -- on top of libmask_b200.so.
// Build the testbed with this file in place of host_program_16x8.cu and link -lmask_b200.
#include <cstdio>
#include <cstdlib>

#include "mask_b200.h"

template <int TILE_M, int TILE_N, int TILE_K>
void sr_bcrs_test_tf32(int M, int N, int K, int TCBlock_num, int* val_sidx, int* val_soff, float* B_val,
                       float* val_block_val, float* C, bool is_ncu_test, int warmup_time, int execute_time) {
    static_assert(TILE_M == 16 && TILE_K == 8, "the library implements the 16x8 tile");
    mask_session* s = nullptr;
    if (mask_session_create_srbcrs(M, K, TCBlock_num, val_soff, val_sidx, val_block_val, MASK_POLICY_AUTO, &s) != MASK_OK) {
        fprintf(stderr, "mask_b200: %s\n", mask_last_error());
        exit(-1);
    }
    const int runs = is_ncu_test ? 1 : warmup_time + execute_time;
    float ms = 0.f, total = 0.f;
    for (int i = 0; i < runs; i++) {   // every call uploads B, multiplies and downloads C; ms = the kernels alone
        if (mask_session_spmm_host(s, B_val, C, N, &ms) != MASK_OK) {
            fprintf(stderr, "mask_b200: %s\n", mask_last_error());
            exit(-1);
        }
        if (i >= warmup_time) total += ms;
    }
    if (!is_ncu_test && execute_time > 0) printf("mykernel_time: %f ms\n", total / execute_time);
    mask_session_destroy(s);
}

template void sr_bcrs_test_tf32<16, 64, 8>(int M, int N, int K, int TCBlock_num, int* val_sidx, int* val_soff, float* B_val,
                                           float* val_block_val, float* C, bool is_ncu_test, int warmup_time,
                                           int execute_time);
