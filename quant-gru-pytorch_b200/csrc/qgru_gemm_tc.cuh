// qgru_gemm_tc.cuh - input projection on the 5th-generation tensor cores (tcgen05, kind::i8).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "qgru_internal.h"

namespace qgru {

struct TcGemmState {
    bool valid = false;
};

int tc_gemm_launch(TcGemmState &st, int device, int sm_count, const uint8_t *x8, const int8_t *w8,
                   void *ih, long long N, int C, int Kpad, bool x_unsigned, int ih_bytes,
                   LinearConsts lc, cudaStream_t stream, std::string *err);

}  // namespace qgru
