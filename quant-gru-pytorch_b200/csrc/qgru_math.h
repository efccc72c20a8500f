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
    int32_t mult;    // 1 in POT2 mode, else 32768..65535
    int32_t shift;   // > 0: rounding right shift; <= 0: left shift
    // Shift-free form (set_fast_form; mq == 0 where it does not exist), see mul_round_hi:
    int32_t mq;      // mult << k, k chosen so that 2^30 <= mq < 2^31
    int32_t e;       // shift + k - 32, 0..31: the quotient is the high product word >> e
    int32_t add_hi;  // high and low word of 2^(31+e): one half in units of the quotient
    uint32_t add_lo;
    int32_t emask;   // 2^e - 1: the bits of the high word that belong to the remainder
    int32_t pad;
};

// A fused linear layer's requantization with its per-channel constant folded into the rounding
// addend: k = corr * mq + 2^(31+e), so that out = round(acc * mq + k) handles acc + corr in the
// one multiply-add (see lin_round).  mq == 0: the channel has no such form.
struct FastLin {
    int32_t mq, e, emask, k_hi;
    uint32_t k_lo;
    int32_t pad;
};

// rshift_round(int64_t, int8_t) (include/quantize_ops_helper.h:183-206): round half to even
// of x / 2^n, defined there on the magnitude with the sign restored.  Round-half-even is an
// odd function, so the same value comes out of floor arithmetic on the signed number: with
// f = floor(x / 2^n) and r = x - f*2^n, adding (2^(n-1) - 1) + (f & 1) carries into bit n
// exactly when r > half, or r == half and f is odd.  No abs / negate, and an arithmetic
// shift at the end.  n <= 0 is a left shift, as in the reference.
QG_HD int64_t rshift_round64(int64_t x, int n) {
    if (n <= 0) return (int64_t)((uint64_t)x << (-n));
    const int64_t odd = (x >> n) & 1;
    return (x + (((int64_t)1 << (n - 1)) - 1) + odd) >> n;
}

// applyRescale(int64_t, FixedPointScale) (include/quantize_ops_helper.h:228-230).
QG_HD int64_t rescale64(int64_t x, Rescale r) { return rshift_round64(x * (int64_t)r.mult, r.shift); }

// Fill the shift-free form (host, once per scale).  With k = 30 - floor(log2(mult)) the
// product x * (mult << k) of a 32-bit x stays below 2^62 and equals x * mult * 2^k, so
// x * mult / 2^shift == product / 2^(32 + e) with e = shift + k - 32.  The form exists for
// 0 <= e <= 31: shifts 17..48 of a 16-bit multiplier, 2..33 in POT2 mode (mult = 1).
QG_HD void set_fast_form(Rescale *r) {
    r->mq = 0;
    r->e = 0;
    r->add_hi = 0;
    r->add_lo = 0;
    r->emask = 0;
    r->pad = 0;
    if (r->mult <= 0 || r->mult > 65535) return;
    int lg = 0;
    while ((r->mult >> (lg + 1)) != 0) ++lg;
    const int k = 30 - lg, e = r->shift + k - 32;
    if (e < 0 || e > 31) return;
    const uint64_t add = (uint64_t)1 << (31 + e);
    r->mq = (int32_t)((uint32_t)r->mult << k);
    r->e = e;
    r->add_hi = (int32_t)(add >> 32);
    r->add_lo = (uint32_t)add;
    r->emask = (int32_t)(((uint32_t)1 << e) - 1u);
}

// Round-half-even of t / 2^(32+e), where t already holds the value plus one half (2^(31+e)):
// the arithmetic shift gives round-half-up; the value was an exact tie precisely when the low
// 32+e bits of t are all zero, and then the even neighbour is the result with its lowest bit
// cleared.  Equal to rshift_round64(value, 32 + e); a 32-bit shift by a uniform amount, one
// compare, one select.
QG_HD int32_t round_tie_even(int64_t t, int32_t e, int32_t emask) {
    const int32_t hi = (int32_t)(t >> 32);
    const uint32_t lo = (uint32_t)t;
    const int32_t q = hi >> e;
    return ((((uint32_t)hi & (uint32_t)emask) | lo) == 0u) ? (q & ~1) : q;
}

// Round-half-even of x * mult / 2^shift through the shift-free form.  Tie = false drops the
// tie rule (round half up): equal wherever no operand can produce an exact tie, which the host
// proves per scale with rescale_can_tie before it picks that form.
template <bool Tie = true>
QG_HD int32_t mul_round_hi(int32_t x, const Rescale &r) {
    const int64_t add = (int64_t)(((uint64_t)(uint32_t)r.add_hi << 32) | (uint64_t)r.add_lo);
    const int64_t t = (int64_t)x * (int64_t)r.mq + add;
    if (Tie) return round_tie_even(t, r.e, r.emask);
    return (int32_t)(t >> 32) >> r.e;
}

// Round-half-even of (acc + corr) * mult / 2^shift with corr folded into f's addend.
template <bool Tie = true>
QG_HD int32_t lin_round(int32_t acc, const FastLin &f) {
    const int64_t k = (int64_t)(((uint64_t)(uint32_t)f.k_hi << 32) | (uint64_t)f.k_lo);
    const int64_t t = (int64_t)acc * (int64_t)f.mq + k;
    if (Tie) return round_tie_even(t, f.e, f.emask);
    return (int32_t)(t >> 32) >> f.e;
}

// Can x * mult / 2^shift be an exact tie (remainder exactly one half) for some integer x in
// [lo, hi]?  x * mult = q * 2^shift + 2^(shift-1) needs x * mult to hold the factor 2 exactly
// shift - 1 times: with t = trailing zeros of mult, x must be an odd multiple of
// 2^(shift-1-t).  No such x in the interval: round-half-even and round-half-up agree on it.
QG_HD bool rescale_can_tie(int32_t mult, int32_t shift, int64_t lo, int64_t hi) {
    if (shift <= 0 || mult <= 0 || lo > hi) return false;   // left shift: no remainder
    int t = 0;
    while (((mult >> t) & 1) == 0) ++t;
    const int need = shift - 1 - t;
    if (need < 0) return false;          // x * mult is a multiple of 2^shift for every x
    if (need >= 62) return false;        // only x = 0 has that many factors of two, and 0 is no tie
    // multiples of 2^n in [lo, hi]: floor(hi / 2^n) - ceil(lo / 2^n) + 1
    const int64_t n1 = (hi >> need) - (-((-lo) >> need)) + 1;
    const int64_t n2 = (hi >> (need + 1)) - (-((-lo) >> (need + 1))) + 1;
    return n1 - n2 > 0;
}

// FastLin of a channel: the scale's shift-free form and its constant corr (|corr| < 2^31).
QG_HD FastLin make_fast_lin(const Rescale &r, int64_t corr) {
    FastLin f;
    f.mq = 0; f.e = 0; f.emask = 0; f.k_hi = 0; f.k_lo = 0; f.pad = 0;
    if (r.mq == 0 || corr >= 0x7fffffffll || corr <= -0x7fffffffll) return f;
    const int64_t add = (int64_t)(((uint64_t)(uint32_t)r.add_hi << 32) | (uint64_t)r.add_lo);
    const int64_t k = corr * (int64_t)r.mq + add;
    f.mq = r.mq;
    f.e = r.e;
    f.emask = r.emask;
    f.k_hi = (int32_t)(k >> 32);
    f.k_lo = (uint32_t)k;
    return f;
}

// applyRescale for an operand known to fit in int32.  Scales without the shift-free form
// fall back to the 64-bit shifts.
QG_HD int32_t rescale32(int32_t x, Rescale r) {
    if (r.mq != 0) return mul_round_hi(x, r);
    return (int32_t)rshift_round64((int64_t)x * (int64_t)r.mult, r.shift);
}

// Fast form for 0 < shift < 32 and |x * mult| < 2^30 (checked on the host when a plan is
// built): all arithmetic in 32 bits.
QG_HD int32_t rescale_narrow(int32_t x, Rescale r) {
    const int32_t p = x * r.mult;
    const int32_t odd = (p >> r.shift) & 1;
    return (p + ((1 << (r.shift - 1)) - 1) + odd) >> r.shift;
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
// max then min (two instructions on the device); equal to the usual clamp for lo <= hi
QG_HD int32_t clampi(int32_t v, int32_t lo, int32_t hi) {
    const int32_t t = v > lo ? v : lo;
    return t < hi ? t : hi;
}

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
