#include "qgru_gemm_tc.cuh"
namespace qgru {
int tc_gemm_launch(TcGemmState &, int, int, const uint8_t *, const int8_t *, void *, long long, int,
                   int, bool, int, LinearConsts, cudaStream_t, std::string *err) {
    if (err) *err = "tcgen05 GEMM not built";
    return QGRU_ERR_UNSUPPORTED;
}
}  // namespace qgru
