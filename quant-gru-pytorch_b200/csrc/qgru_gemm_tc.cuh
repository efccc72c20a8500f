// qgru_gemm_tc.cuh - launch interface of the tcgen05 input-projection GEMM (qgru_gemm_tc.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "qgru_internal.h"

namespace qgru {

// Cached tensor maps of the two operands (opaque 128-byte CUtensorMap objects).
struct TcGemmState {
    bool valid = false;
    const void *x8 = nullptr, *w8 = nullptr;
    long long x_rows = 0, w_rows = 0;
    int Kpad = 0;
    int order = 0;   // tile order: 0 auto, 1 token-tile-major (W and x slabs stream), 2 W-stationary
    alignas(64) unsigned char map_w[128];
    alignas(64) unsigned char map_x[128];
};

// ih[n][m] = requant( sum_k w8[m][k] * x8[n][k] ) for n < N tokens, m < C channels, stored as
// ih_bytes-wide integers (1, 2 or 4).  With ps.enabled the value is further rescaled to the input
// scale of the channel's gate (the form the fused recurrence cell consumes).
// Both operands are [rows][Kpad] bytes with Kpad a multiple of 128 and rows ALLOCATED up to a
// multiple of 128 (x_rows_alloc, w_rows_alloc) so that no tile load leaves the allocation.
// x_row0: the launch works on tokens x_row0 .. x_row0 + N - 1 of x8 (a chunk of timesteps); ih then
// holds those N tokens from its first row on.
// Returns QGRU_ERR_UNSUPPORTED when the shapes do not meet that, QGRU_ERR_CUDA on failure.
int tc_gemm_launch(TcGemmState &st, const uint8_t *x8, long long x_rows_alloc, const int8_t *w8,
                   long long w_rows_alloc, void *ih, long long N, int C, int Kpad, bool x_unsigned,
                   int ih_bytes, LinearConsts lc, PreScale ps, bool fast, bool notie, int *abort_flag, int sms,
                   cudaStream_t stream, std::string *err, long long x_row0 = 0);

}  // namespace qgru
