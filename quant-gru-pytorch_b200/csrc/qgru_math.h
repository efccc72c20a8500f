// qgru_math.h - the integer arithmetic contract, shared by host set-up code and kernels.
//
// Every function states the reference definition it must agree with bit for bit
// (paths relative to the reference project's root).  POT2 mode is carried as a
// FixedPointScale with multiplier 1, which is what the reference's own quantize boundary
// does (toFixedScale, include/quantize_ops_helper.h:280-283) and gives
// rshift_round(x * 1, n) == rshift_round(x, n).
#pragma once
#include <stdint.h>

#include "qgru.h"

#if defined(__CUDACC__)
#define QG_HD __host__ __device__ __forceinline__
#else
#define QG_HD inline
#endif

namespace qgru {

// FixedPointScale / Pot2Rescale (include/quantize_param_types.h:37-46), widened to ints.
struct Rescale {
    int32_t mult;   // 1 in POT2 mode, else 32768..65535
    int32_t shift;  // > 0: rounding right shift; <= 0: left shift
};

// rshift_round(int64_t, int8_t): banker's rounding on the magnitude
// (include/quantize_ops_helper.h:183-206).  Branch-free form of the same definition:
// |x| + (half - 1) + (bit n of |x|) carries into bit n exactly when the remainder is above
// half, or equal to half with an odd quotient.
QG_HD int64_t rshift_round64(int64_t x, int n) {
    if (n <= 0) return (int64_t)((uint64_t)x << (-n));
    const int64_t sgn = x >> 63;
    const uint64_t a = (uint64_t)((x ^ sgn) - sgn);
    const uint64_t odd = (a >> n) & 1ull;
    const uint64_t q = (a + ((1ull << (n - 1)) - 1ull) + odd) >> n;
    return ((int64_t)q ^ sgn) - sgn;
}

// applyRescale(int64_t, FixedPointScale) (include/quantize_ops_helper.h:228-230).
QG_HD int64_t rescale64(int64_t x, Rescale r) { return rshift_round64(x * (int64_t)r.mult, r.shift); }

// The same for an operand known to fit in int32: one widening multiply.
QG_HD int64_t rescale32(int32_t x, Rescale r) {
    return rshift_round64((int64_t)x * (int64_t)r.mult, r.shift);
}

// Fast form for the common case 0 < shift < 32 and |x * mult| < 2^31 (checked on the host
// when a plan is built): all arithmetic in 32 bits.
QG_HD int32_t rescale_narrow(int32_t x, Rescale r) {
    const int32_t p = x * r.mult;
    const int32_t sgn = p >> 31;
    const uint32_t a = (uint32_t)((p ^ sgn) - sgn);
    const uint32_t odd = (a >> r.shift) & 1u;
    const uint32_t q = (a + ((1u << (r.shift - 1)) - 1u) + odd) >> r.shift;
    return ((int32_t)q ^ sgn) - sgn;
}

// QuantBitWidth::qmin / qmax (include/quantize_bitwidth_config.h:14-22).
QG_HD int32_t qmin_of(int bits, bool uns) {
    if (bits >= 32) return (int32_t)0x80000000;
    return uns ? 0 : -(1 << (bits - 1));
}
QG_HD int32_t qmax_of(int bits, bool uns) {
    if (bits >= 32) return 0x7FFFFFFF;
    return uns ? (int32_t)((1u << bits) - 1u) : (1 << (bits - 1)) - 1;
}
QG_HD int32_t clampi(int32_t v, int32_t lo, int32_t hi) { return v < lo ? lo : (v > hi ? hi : v); }

// piecewise_linear_raw on an already clamped input (include/quantize_ops_helper.h:560-589):
// first segment whose threshold exceeds q, else the last one.
QG_HD int32_t lut_raw(const qgru_lut &lut, int32_t q) {
    int seg = QGRU_LUT_SEGMENTS - 1;
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
    for (int i = QGRU_LUT_SEGMENTS - 2; i >= 0; --i)
        if (q < lut.seg[i].threshold) seg = i;
    const qgru_lut_segment s = lut.seg[seg];
    const int64_t bx = (int64_t)s.q_b * (int64_t)(q - lut.zp_x);
    const int n = (int)(int8_t)s.n_bx;
    const int32_t term = (n >= 0) ? (int32_t)rshift_round64(bx, n) : (int32_t)((uint64_t)bx << (-n));
    return (int32_t)((uint32_t)term + (uint32_t)s.term_c);
}

}  // namespace qgru
