// qgru_host.cc - host-only part of the C ABI: scale encoding, LUT generation and the
// MinMax quant-parameter derivation.  No CUDA call is made from this file.
//
// These are the pieces of the reference that run on the host on every forward call of its
// Python binding (GRUQuantParamsPy::to_cpp regenerates the three LUTs,
// pytorch/lib/gru_interface_binding.cc:1229-1284) and at finalize_calibration.  They feed
// the bit-exact contract, so every float expression keeps the reference's operand order and
// precision (float unless the reference widens to double); build without fast-math and
// without FMA contraction.
#include <algorithm>
#include <cfloat>
#include <cmath>
#include <cstring>
#include <vector>

#include "qgru_internal.h"

namespace qgru {

// encodeMShift, include/quantize_ops_helper.h:245-264.
bool encode_mshift(float scale, Rescale *out) {
    if (!(scale > 0.0f)) return false;
    int e = 0;
    const double mant = std::frexp(static_cast<double>(scale), &e);
    uint32_t m = static_cast<uint32_t>(std::llround(mant * 65536.0));
    if (m == 65536u) {
        m = 32768u;
        e += 1;
    }
    if (m < 32768u) m = 32768u;
    const int shift = 16 - e;
    if (shift < -128 || shift > 127) return false;
    out->mult = static_cast<int32_t>(m);
    out->shift = shift;
    out->mq = 0;
    out->e = 0;
    out->add_hi = 0;
    out->add_lo = 0;
    out->emask = 0;
    out->pad = 0;
    return true;
}

// pot2Shift, include/quantize_ops_helper.h:272-275.
int pot2_shift(float scale) {
    if (!(scale > 0.0f)) return 0;
    return static_cast<int8_t>(std::lround(-std::log2(static_cast<double>(scale))));
}

// toFixedScale, include/quantize_ops_helper.h:280-283.
bool to_fixed_scale(float scale, bool pot2, Rescale *out) {
    if (pot2) {
        *out = Rescale{1, pot2_shift(scale), 0, 0, 0, 0, 0, 0};
        return true;
    }
    return encode_mshift(scale, out);
}

// decode_scale, include/quantize_ops_helper.h:94-100.
float decode_scale(Rescale r) {
    return static_cast<float>(static_cast<uint16_t>(r.mult)) * ldexpf(1.0f, -r.shift);
}

// makeRescale<R>, include/quantize_ops_helper.h:296-312.
bool make_rescale(float src, float dst, bool pot2, Rescale *out) {
    if (pot2) {
        *out = Rescale{1, static_cast<int8_t>(pot2_shift(src) - pot2_shift(dst)), 0, 0, 0, 0, 0, 0};
        return true;
    }
    return encode_mshift(src / dst, out);
}
// makeRescaleProduct<R>, include/quantize_ops_helper.h:315-331.
bool make_rescale_product(float a, float b, float dst, bool pot2, Rescale *out) {
    if (pot2) {
        *out = Rescale{1, static_cast<int8_t>(pot2_shift(a) + pot2_shift(b) - pot2_shift(dst)), 0, 0, 0, 0, 0, 0};
        return true;
    }
    return encode_mshift((a * b) / dst, out);
}
// makeRescaleToProduct<R>, include/quantize_ops_helper.h:334-350.
bool make_rescale_to_product(float src, float a, float b, bool pot2, Rescale *out) {
    if (pot2) {
        *out = Rescale{1, static_cast<int8_t>(pot2_shift(src) - (pot2_shift(a) + pot2_shift(b))), 0, 0, 0, 0, 0, 0};
        return true;
    }
    return encode_mshift(src / (a * b), out);
}

int32_t op_qmin(const qgru_op &o) { return qmin_of(o.bits, o.bits < 32 && o.is_unsigned); }
int32_t op_qmax(const qgru_op &o) { return qmax_of(o.bits, o.bits < 32 && o.is_unsigned); }

int32_t lut_eval(const qgru_lut &lut, int32_t q_x, const qgru_op &in_bw, const qgru_op &out_bw) {
    const int32_t q = clampi(q_x, op_qmin(in_bw), op_qmax(in_bw));
    return clampi(lut_raw(lut, q), op_qmin(out_bw), op_qmax(out_bw));
}

namespace {

// linear_fit, src/quantize_ops.cu:996-1017 (single precision sums, in sample order).
void least_squares(const float *x, const float *y, int n, float &b, float &c) {
    float sx = 0.0f, sy = 0.0f, sxy = 0.0f, sxx = 0.0f;
    for (int i = 0; i < n; ++i) {
        sx += x[i];
        sy += y[i];
        sxy += x[i] * y[i];
        sxx += x[i] * x[i];
    }
    const float denom = n * sxx - sx * sx;
    if (std::abs(denom) < 1e-9f) {
        b = 0.0f;
        c = sy / n;
        return;
    }
    b = (n * sxy - sx * sy) / denom;
    c = (sy - b * sx) / n;
}

// adaptive_segmentation_sigmoid, src/quantize_ops.cu:1022-1117: break points that put more
// segments near x = 0.  The weights always come from the sigmoid's slope, for tanh tables too.
std::vector<float> break_points(float lo, float hi, int segments) {
    constexpr int kSamples = 1000;
    constexpr float kCenterWeight = 5.0f, kCenterRange = 2.0f;
    std::vector<float> xs(kSamples), w(kSamples - 1), cum(kSamples - 1);
    for (int i = 0; i < kSamples; ++i) xs[i] = lo + (hi - lo) * static_cast<float>(i) / (kSamples - 1);
    for (int i = 0; i + 1 < kSamples; ++i) {
        const float x = xs[i], xn = xs[i + 1];
        const float y = 1.0f / (1.0f + std::exp(-x));
        const float yn = 1.0f / (1.0f + std::exp(-xn));
        const float slope = std::abs(yn - y) / (xn - x + 1e-9f);
        const float dist = std::abs(x);
        w[i] = dist < kCenterRange ? kCenterWeight * (1.0f - dist / kCenterRange) + 1.0f
                                   : 1.0f + slope * 0.5f;
    }
    float total = 0.0f;
    for (float v : w) total += v;
    for (float &v : w) v /= total;
    cum[0] = w[0];
    for (int i = 1; i + 1 < kSamples; ++i) cum[i] = cum[i - 1] + w[i];

    std::vector<float> pts;
    pts.push_back(lo);
    for (int i = 1; i < segments; ++i) {
        const float target = static_cast<float>(i) / segments;
        int idx = static_cast<int>(std::lower_bound(cum.begin(), cum.end(), target) - cum.begin());
        idx = std::min(idx, kSamples - 2);
        pts.push_back(xs[idx]);
    }
    pts.push_back(hi);
    std::sort(pts.begin(), pts.end());
    pts.erase(std::unique(pts.begin(), pts.end(),
                          [](float a, float b) { return std::abs(a - b) < 1e-9f; }),
              pts.end());
    while (static_cast<int>(pts.size()) < segments + 1) {
        float widest = 0.0f;
        size_t at = 0;
        for (size_t i = 0; i + 1 < pts.size(); ++i) {
            const float gap = pts[i + 1] - pts[i];
            if (gap > widest) {
                widest = gap;
                at = i;
            }
        }
        pts.insert(pts.begin() + at + 1, (pts[at] + pts[at + 1]) / 2.0f);
    }
    return pts;
}

// generate_sigmoid_lut / generate_tanh_lut, float-scale overloads
// (src/quantize_ops.cu:1148-1221, 1237-1307) with quantize_multiplier_signed (:1137-1146).
void build_lut(bool is_tanh, const qgru_op &in, const qgru_op &out, qgru_lut *lut) {
    const float sx = in.scale, sy = out.scale;
    const int32_t zx = in.zero_point, zy = out.zero_point;
    const float limit = is_tanh ? 4.0f : 8.0f;
    float x_lo = static_cast<float>(op_qmin(in) - zx) * sx;
    float x_hi = static_cast<float>(op_qmax(in) - zx) * sx;
    x_lo = std::max(x_lo, -limit);
    x_hi = std::min(x_hi, limit);
    std::memset(lut, 0, sizeof(*lut));
    lut->zp_x = zx;
    const std::vector<float> pts = break_points(x_lo, x_hi, QGRU_LUT_SEGMENTS);
    constexpr int kFit = 100;
    float xv[kFit], yv[kFit];
    for (int s = 0; s < QGRU_LUT_SEGMENTS; ++s) {
        const float a = pts[s], e = pts[s + 1];
        for (int j = 0; j < kFit; ++j) {
            const float x = a + (e - a) * static_cast<float>(j) / (kFit - 1);
            xv[j] = x;
            yv[j] = is_tanh ? std::tanh(x) : 1.0f / (1.0f + std::exp(-x));
        }
        float b, c;
        least_squares(xv, yv, kFit, b, c);
        const float slope = b * (sx / sy);
        int32_t q_b = 0;
        int8_t n = 0;
        if (!(std::abs(slope) < 1e-12f)) {
            const int32_t qmax = op_qmax(out);
            n = static_cast<int8_t>(std::floor(std::log2(static_cast<double>(qmax) / std::abs(slope))));
            int64_t q = static_cast<int64_t>(std::rint(static_cast<double>(slope) * std::ldexp(1.0, n)));
            q = std::max<int64_t>(-qmax, std::min<int64_t>(qmax, q));
            q_b = static_cast<int32_t>(q);
        }
        lut->seg[s].q_b = q_b;
        lut->seg[s].n_bx = n;
        lut->seg[s].term_c = static_cast<int32_t>(rintf(c / sy + static_cast<float>(zy)));
        const int32_t thr = static_cast<int32_t>(rintf(e / sx + zx));
        lut->seg[s].threshold = clampi(thr, op_qmin(in), op_qmax(in));
    }
}

// get_minimum_scale, include/histogram_collector.h:31-35.
float minimum_scale(int64_t steps) {
    return std::min(1.19209290e-07f, 0.01f / static_cast<float>(steps));
}

// calibrateContinuousScaleFromRange (include/pot_sqnr_calibrator.h:546-613) followed by
// encodeScaleResult(coverage_round = true) and storedScaleForMode (:451-524, :72-74).
bool calibrate_minmax(float mn, float mx, bool pot2, qgru_op *op) {
    const bool uns = op->bits < 32 && op->is_unsigned;
    const bool sym = op->symmetric != 0;
    const int32_t qlo = op_qmin(*op), qhi = op_qmax(*op);
    const int64_t steps = static_cast<int64_t>(qhi) - static_cast<int64_t>(qlo);
    if (steps <= 0) return false;
    const float tiny = minimum_scale(steps);
    const float lo0 = std::min(mn, 0.0f), hi0 = std::max(mx, 0.0f);
    const float grow = ((hi0 - lo0) / static_cast<float>(steps) < tiny) ? tiny : 0.0f;
    float lo = lo0, hi = hi0;
    if (sym) {
        if (uns) {
            hi = hi0 + static_cast<float>(steps) * grow;
            lo = 0.0f;
        } else {
            hi = hi0 + std::floor(static_cast<float>(steps) / 2.0f) * grow;
            lo = lo0 - std::ceil(static_cast<float>(steps) / 2.0f) * grow;
        }
    } else {
        hi = hi0 + static_cast<float>(steps) * grow;
    }
    float scale, range_min;
    if (sym && uns) {
        scale = std::max(std::max(hi, tiny) / static_cast<float>(qhi), tiny);
        range_min = 0.0f;
    } else if (sym) {
        const int64_t pos = steps / 2, neg = (steps + 1) / 2;
        const int extra = (steps == 3) ? 1 : 0;
        const float from_max = (pos + extra > 0) ? hi / static_cast<float>(pos + extra) : 0.0f;
        const float from_min = (neg > 0) ? -lo / static_cast<float>(neg) : 0.0f;
        scale = std::max(std::max(from_max, from_min), tiny);
        range_min = -static_cast<float>(neg) * scale;
    } else {
        const float range = std::max(hi - lo, tiny * static_cast<float>(steps));
        scale = std::max(range / static_cast<float>(steps), tiny);
        range_min = lo;
    }
    if (pot2) {
        const float nf = std::floor(std::log2(1.0f / scale));
        if (nf < -128.0f || nf > 127.0f) return false;
        const int8_t n = static_cast<int8_t>(nf);
        const float po2 = std::pow(2.0f, -static_cast<float>(n));
        if (sym) {
            op->zero_point = 0;
        } else {
            const float aligned = std::floor(range_min / po2) * po2;
            op->zero_point = static_cast<int32_t>(rintf(static_cast<float>(qlo) - aligned / po2));
        }
        op->scale = po2;
        return true;
    }
    Rescale fs;
    if (!encode_mshift(scale, &fs)) return false;
    const float effective = decode_scale(fs);
    op->zero_point = sym ? 0 : static_cast<int32_t>(rintf(static_cast<float>(qlo) - range_min / effective));
    op->scale = scale;
    return true;
}

bool calibrate_channels(qgru_op *op, int gran, bool pot2, int H, const float *mins,
                        const float *maxs, float *scales) {
    const int C = 3 * H;
    qgru_op t = *op;
    if (gran == QGRU_PER_TENSOR) {
        const float mn = *std::min_element(mins, mins + C), mx = *std::max_element(maxs, maxs + C);
        if (!calibrate_minmax(mn, mx, pot2, &t)) return false;
        std::fill(scales, scales + C, t.scale);
    } else if (gran == QGRU_PER_GATE) {
        for (int g = 0; g < 3; ++g) {
            float mn = FLT_MAX, mx = -FLT_MAX;
            for (int c = g * H; c < (g + 1) * H; ++c) {
                mn = std::min(mn, mins[c]);
                mx = std::max(mx, maxs[c]);
            }
            if (!calibrate_minmax(mn, mx, pot2, &t)) return false;
            std::fill(scales + g * H, scales + (g + 1) * H, t.scale);
        }
    } else {
        for (int c = 0; c < C; ++c) {
            if (!calibrate_minmax(mins[c], maxs[c], pot2, &t)) return false;
            scales[c] = t.scale;
        }
    }
    op->scale = scales[0];
    op->zero_point = 0;
    return true;
}


// ------------------------------------------------------------------ histogram calibration
// Histogram -> continuous scale (Percentile or SQNR) -> stored scale and zero point.  All
// single precision, operand order as in the reference: these results are compared exactly.

struct ContScale {
    float scale, min, max;
};

float hist_bin_width(const float min_val, const float max_val, int bins) {
    if (bins <= 0 || max_val <= min_val) return 1.0f;   // Histogram::bin_width, include/histogram_collector.h:76-79
    return (max_val - min_val) / bins;
}

// Histogram::getPercentileRange, include/histogram_collector.h:105-165.
void percentile_range(const float *counts, int bins, float min_val, float max_val, long long total,
                      float clip, float *pmin, float *pmax) {
    *pmin = min_val;
    *pmax = max_val;
    if (bins <= 0 || total <= 0 || clip <= 0.0f) return;
    std::vector<float> cum(bins);
    cum[0] = counts[0];
    for (int i = 1; i < bins; ++i) cum[i] = cum[i - 1] + counts[i];
    const float sum = cum[bins - 1];
    if (sum < 1e-6f) return;
    const float bw = hist_bin_width(min_val, max_val, bins);
    const float keep = 1.0f - clip;
    const float lo_thr = sum * clip, hi_thr = sum * keep;
    int lo_i = 0, hi_i = bins - 1;
    for (int i = 0; i < bins; ++i)
        if (cum[i] >= lo_thr) { lo_i = i; break; }
    for (int i = 0; i < bins; ++i)
        if (cum[i] >= hi_thr) { hi_i = i; break; }
    float a = min_val + lo_i * bw, b = min_val + hi_i * bw;
    if (b <= a) b = max_val;
    *pmin = a;
    *pmax = b;
}

// calibratePercentile, include/pot_sqnr_calibrator.h:99-186.
ContScale calibrate_percentile(const float *counts, int bins, float min_val, float max_val, long long total,
                               int64_t steps, bool sym, bool uns, float percentile) {
    const float tiny = minimum_scale(steps);
    const float clip = (100.0f - percentile) / 100.0f;
    float pmin, pmax;
    percentile_range(counts, bins, min_val, max_val, total, clip, &pmin, &pmax);
    pmin = std::min(pmin, 0.0f);
    pmax = std::max(pmax, 0.0f);
    pmin = std::max(-FLT_MAX, std::min(pmin, 0.0f));
    pmax = std::min(FLT_MAX, std::max(pmax, 0.0f));
    if ((pmax - pmin) / static_cast<float>(steps) < tiny) {
        if (sym && !uns) {
            pmin -= tiny * static_cast<float>((steps + 1) / 2);
            pmax += tiny * static_cast<float>(steps / 2);
        } else {
            pmax += tiny * static_cast<float>(steps);
        }
    }
    ContScale r;
    if (sym && uns) {
        const float data_max = std::max(pmax, tiny);
        r.scale = std::max(data_max / static_cast<float>(steps), tiny);
        r.min = 0.0f;
        r.max = r.scale * static_cast<float>(steps);
    } else if (sym) {
        const int64_t pos = steps / 2, neg = (steps + 1) / 2;
        const float from_max = pos > 0 ? pmax / static_cast<float>(pos) : FLT_MAX;
        const float from_min = neg > 0 ? -pmin / static_cast<float>(neg) : FLT_MAX;
        r.scale = std::max(from_max, from_min);
        r.min = -static_cast<float>(neg) * r.scale;
        r.max = static_cast<float>(pos) * r.scale;
    } else {
        r.scale = (pmax - pmin) / static_cast<float>(steps);
        r.min = pmin;
        r.max = pmax;
    }
    r.scale = std::max(r.scale, tiny);
    return r;
}

// sqnr_detail::estimateNoise, include/pot_sqnr_calibrator.h:210-238 (gamma = 3, p = 2).
float sqnr_noise(const float *counts, int bins, float min_val, float bw, float delta, float offset,
                 int64_t steps) {
    if (delta <= 0) return FLT_MAX;
    const float gamma = 3.0f, p = 2.0f;
    float noise = 0.0f;
    for (int i = 0; i < bins; ++i) {
        const float count = counts[i];
        if (count < 1e-6f) continue;
        const float x = min_val + (i + 0.5f) * bw;
        float q = rintf(x / delta - offset);
        const bool clipped = (q < 0) || (q > static_cast<float>(steps));
        q = std::max(0.0f, std::min(static_cast<float>(steps), q));
        const float x_recon = (q + offset) * delta;
        float err = std::pow(std::abs(x_recon - x), p);
        if (clipped) err *= gamma;
        noise += err * count;
    }
    return noise;
}

// calibrateSqnr with searchSymmetric / searchAsymmetric, include/pot_sqnr_calibrator.h:246-381
// (101 symmetric deltas; 17 deltas x min(steps + 2, 21) offsets otherwise).
bool calibrate_sqnr(const float *counts, int bins, float hmin, float hmax, int64_t steps, bool sym,
                    bool uns, ContScale *out) {
    const float tiny = minimum_scale(steps);
    const float bw = hist_bin_width(hmin, hmax, bins);
    const float min_val = std::min(hmin, 0.0f);
    float max_val = std::max(hmax, 0.0f);
    const float floor_max = min_val + tiny * static_cast<float>(steps);
    max_val = (max_val > floor_max) ? max_val : floor_max;
    float best_noise = FLT_MAX;
    ContScale best{0, 0, 0};
    if (sym) {
        float max_delta, offset;
        if (uns) {
            max_delta = max_val / static_cast<float>(steps);
            offset = 0.0f;
        } else {
            max_delta = 2.0f * std::max(max_val, -min_val) / static_cast<float>(steps);
            offset = -static_cast<float>((steps + 1) / 2);
        }
        max_delta = std::max(max_delta, tiny);
        const int cand = 101, div = cand - 1;
        for (int d = 1; d <= cand; ++d) {
            float delta = max_delta * d / div;
            delta = std::max(delta, tiny);
            const float noise = sqnr_noise(counts, bins, hmin, bw, delta, offset, steps);
            if (noise < best_noise) {
                best_noise = noise;
                best.scale = delta;
                best.min = offset * delta;
                best.max = best.min + steps * delta;
            }
        }
    } else {
        const float max_delta = (max_val - min_val) / static_cast<float>(steps);
        const float obs_off = rintf(min_val / max_delta);
        const float obs_min = max_delta * obs_off;
        const float obs_max = obs_min + max_delta * static_cast<float>(steps);
        const int n_off = std::min(static_cast<int>(steps + 2), 21);
        std::vector<float> offs(n_off);
        const float step = static_cast<float>(steps) / (n_off - 2);
        for (int o = 0; o < n_off - 1; ++o) offs[o] = rintf(-static_cast<float>(steps) + o * step);
        offs[n_off - 1] = obs_off;
        const int cand = 17;
        for (int d = 1; d <= cand; ++d) {
            float delta = max_delta * d / (cand - 1);
            delta = std::max(delta, tiny);
            for (int o = 0; o < n_off; ++o) {
                float t_min = delta * offs[o];
                float t_max = t_min + delta * static_cast<float>(steps);
                t_min = std::max(obs_min, t_min);
                t_max = std::min(obs_max, t_max);
                float cd = (t_max - t_min) / static_cast<float>(steps);
                cd = std::max(cd, tiny);
                const float co = rintf(t_min / cd);
                const float noise = sqnr_noise(counts, bins, hmin, bw, cd, co, steps);
                if (noise < best_noise) {
                    best_noise = noise;
                    best.scale = cd;
                    best.min = co * cd;
                    best.max = best.min + steps * cd;
                }
            }
        }
    }
    if (best_noise == FLT_MAX) return false;
    *out = best;
    return true;
}

// encodeScaleResult(coverage_round = false) + storedScaleForMode, include/pot_sqnr_calibrator.h:
// 72-74, 388-447, 451-524: POT2 rounds the scale to the nearest power of two; otherwise the
// zero point is computed against the decoded 16-bit-mantissa scale and the continuous scale is
// what is stored.
bool encode_histogram_scale(const ContScale &c, bool pot2, qgru_op *op) {
    const bool sym = op->symmetric != 0;
    const int32_t qlo = op_qmin(*op);
    if (!(c.scale > 0.0f)) return false;
    if (pot2) {
        const float nf = rintf(-std::log2(c.scale));
        if (nf < -128.0f || nf > 127.0f) return false;
        const int8_t n = static_cast<int8_t>(nf);
        const float po2 = std::pow(2.0f, -static_cast<float>(n));
        op->zero_point = sym ? 0 : static_cast<int32_t>(rintf(static_cast<float>(qlo) - c.min / po2));
        op->scale = po2;
        return true;
    }
    Rescale fs;
    if (!encode_mshift(c.scale, &fs)) return false;
    const float effective = decode_scale(fs);
    op->zero_point = sym ? 0 : static_cast<int32_t>(rintf(static_cast<float>(qlo) - c.min / effective));
    op->scale = c.scale;
    return true;
}

// calibrateContinuousScaleFromHistogram + encodeScaleResult for one histogram.
int calibrate_histogram(const float *counts, int bins, float min_val, float max_val, long long total,
                        bool pot2, bool use_percentile, float percentile, qgru_op *op) {
    if (!counts || bins <= 0 || total <= 0) return QGRU_ERR_NOT_READY;   // Histogram::is_valid
    const bool uns = op->bits < 32 && op->is_unsigned;
    const bool sym = op->symmetric != 0;
    const int64_t steps = static_cast<int64_t>(op_qmax(*op)) - static_cast<int64_t>(op_qmin(*op));
    if (steps <= 0) return QGRU_ERR_BAD_ARG;
    ContScale c;
    if (use_percentile) {
        c = calibrate_percentile(counts, bins, min_val, max_val, total, steps, sym, uns, percentile);
    } else if (!calibrate_sqnr(counts, bins, min_val, max_val, steps, sym, uns, &c)) {
        return QGRU_ERR_RANGE;
    }
    return encode_histogram_scale(c, pot2, op) ? QGRU_OK : QGRU_ERR_RANGE;
}

}  // namespace
}  // namespace qgru

namespace qgru {
int calibrate_histogram_op(const float *counts, int bins, float min_val, float max_val, long long total,
                           bool pot2, bool use_percentile, float percentile, qgru_op *op) {
    return calibrate_histogram(counts, bins, min_val, max_val, total, pot2, use_percentile, percentile, op);
}
}  // namespace qgru

using namespace qgru;

extern "C" {

int qgru_calibrate_from_histogram(const float *counts, int num_bins, float min_val, float max_val,
                                  int64_t total_count, int use_pot2, int use_percentile, float percentile,
                                  qgru_op *op) {
    if (!counts || !op || op->bits < 1 || op->bits > 32) return QGRU_ERR_BAD_ARG;
    return calibrate_histogram(counts, num_bins, min_val, max_val, total_count, use_pot2 != 0,
                               use_percentile != 0, percentile, op);
}

const char *qgru_status_string(int status) {
    switch (status) {
        case QGRU_OK: return "ok";
        case QGRU_ERR_BAD_ARG: return "bad argument";
        case QGRU_ERR_CUDA: return "CUDA error";
        case QGRU_ERR_TIMEOUT: return "device-side wait timed out";
        case QGRU_ERR_UNSUPPORTED: return "unsupported configuration";
        case QGRU_ERR_NOT_READY: return "parameters or weights not set";
        case QGRU_ERR_NOMEM: return "out of memory";
        case QGRU_ERR_RANGE: return "scale cannot be encoded";
        default: return "unknown status";
    }
}

const char *qgru_version(void) { return "qgru-b200 0.1"; }

int qgru_encode_mshift(float scale, uint16_t *multiplier, int8_t *shift) {
    if (!multiplier || !shift) return QGRU_ERR_BAD_ARG;
    Rescale r;
    if (!encode_mshift(scale, &r)) return QGRU_ERR_RANGE;
    *multiplier = static_cast<uint16_t>(r.mult);
    *shift = static_cast<int8_t>(r.shift);
    return QGRU_OK;
}

int qgru_decode_effective_scale(float scale, int use_pot2, float *effective) {
    if (!effective) return QGRU_ERR_BAD_ARG;
    if (!(scale > 0.0f)) return QGRU_ERR_BAD_ARG;
    Rescale r;
    if (!to_fixed_scale(scale, use_pot2 != 0, &r)) return QGRU_ERR_RANGE;
    *effective = decode_scale(r);
    return QGRU_OK;
}

int64_t qgru_rshift_round(int64_t x, int n) { return rshift_round64(x, n); }

int32_t qgru_apply_rescale(int32_t x, uint16_t multiplier, int shift) {
    Rescale r{(int32_t)multiplier, shift, 0, 0, 0, 0, 0, 0};
    set_fast_form(&r);
    return rescale32(x, r);
}

int qgru_rescale_can_tie(uint16_t multiplier, int shift, int64_t lo, int64_t hi) {
    return rescale_can_tie((int32_t)multiplier, shift, lo, hi) ? 1 : 0;
}

int32_t qgru_apply_rescale_half_up(int32_t x, uint16_t multiplier, int shift) {
    Rescale r{(int32_t)multiplier, shift, 0, 0, 0, 0, 0, 0};
    set_fast_form(&r);
    if (r.mq == 0) return rescale32(x, r);
    return mul_round_hi<false>(x, r);
}

int32_t qgru_lut_eval(const qgru_lut *lut, int32_t q_x, const qgru_op *in_bw,
                      const qgru_op *out_bw) {
    return lut_eval(*lut, q_x, *in_bw, *out_bw);
}

int qgru_generate_luts(qgru_params *p) {
    if (!p) return QGRU_ERR_BAD_ARG;
    static const int in_op[3] = {QGRU_OP_UPDATE_IN, QGRU_OP_RESET_IN, QGRU_OP_NEW_IN};
    static const int out_op[3] = {QGRU_OP_UPDATE_OUT, QGRU_OP_RESET_OUT, QGRU_OP_NEW_OUT};
    for (int g = 0; g < 3; ++g) {
        if (!(p->op[in_op[g]].scale > 0.0f) || !(p->op[out_op[g]].scale > 0.0f)) return QGRU_ERR_RANGE;
        build_lut(g == QGRU_LUT_NEW, p->op[in_op[g]], p->op[out_op[g]], &p->lut[g]);
    }
    return QGRU_OK;
}

void qgru_ranges_reset(qgru_ranges *r, int hidden) {
    if (!r) return;
    r->hidden = hidden;
    for (int i = 0; i < QGRU_NUM_OPS; ++i) {
        r->min_v[i] = FLT_MAX;
        r->max_v[i] = -FLT_MAX;
    }
    float *mins[4] = {r->min_W, r->min_R, r->min_bw, r->min_br};
    float *maxs[4] = {r->max_W, r->max_R, r->max_bw, r->max_br};
    for (int k = 0; k < 4; ++k) {
        if (mins[k]) std::fill(mins[k], mins[k] + 3 * hidden, FLT_MAX);
        if (maxs[k]) std::fill(maxs[k], maxs[k] + 3 * hidden, -FLT_MAX);
    }
}

int qgru_calc_params_from_ranges(const qgru_ranges *r, qgru_params *p, float *scale_W,
                                 float *scale_R, float *scale_bw, float *scale_br) {
    if (!r || !p || !scale_W || !scale_R || !scale_bw || !scale_br || r->hidden <= 0)
        return QGRU_ERR_BAD_ARG;
    if (!r->min_W || !r->max_W || !r->min_R || !r->max_R || !r->min_bw || !r->max_bw ||
        !r->min_br || !r->max_br)
        return QGRU_ERR_BAD_ARG;
    // ensureSymmetricWeightBiasConfig, src/gru_interface.cc:26-32
    if (!p->op[QGRU_OP_W].symmetric || !p->op[QGRU_OP_R].symmetric ||
        !p->op[QGRU_OP_BW].symmetric || !p->op[QGRU_OP_BR].symmetric)
        return QGRU_ERR_UNSUPPORTED;
    const bool pot2 = p->use_pot2 != 0;
    const int H = r->hidden;
    p->hidden = H;
    static const int scalar_ops[] = {QGRU_OP_X, QGRU_OP_H, QGRU_OP_IH_LINEAR, QGRU_OP_HH_LINEAR,
                                     QGRU_OP_UPDATE_IN, QGRU_OP_RESET_IN, QGRU_OP_NEW_IN,
                                     QGRU_OP_MUL_RESET_HIDDEN, QGRU_OP_MUL_NEW_CONTRIB,
                                     QGRU_OP_MUL_OLD_CONTRIB};
    for (int k : scalar_ops)
        if (!calibrate_minmax(r->min_v[k], r->max_v[k], pot2, &p->op[k])) return QGRU_ERR_RANGE;
    // activation outputs are widened to a range of at least 0.5 around their centre
    // (ensureMinRange, include/calibration_utils.h:27-45; src/gru_interface.cc:130-145)
    for (int k : {QGRU_OP_UPDATE_OUT, QGRU_OP_RESET_OUT, QGRU_OP_NEW_OUT}) {
        float mn = r->min_v[k], mx = r->max_v[k];
        if (mx - mn < 0.5f) {
            const float c = (mn + mx) / 2.0f;
            mn = c - 0.5f / 2.0f;
            mx = c + 0.5f / 2.0f;
        }
        if (!calibrate_minmax(mn, mx, pot2, &p->op[k])) return QGRU_ERR_RANGE;
    }
    if (!calibrate_channels(&p->op[QGRU_OP_W], p->granularity[0], pot2, H, r->min_W, r->max_W, scale_W) ||
        !calibrate_channels(&p->op[QGRU_OP_R], p->granularity[1], pot2, H, r->min_R, r->max_R, scale_R) ||
        !calibrate_channels(&p->op[QGRU_OP_BW], p->granularity[2], pot2, H, r->min_bw, r->max_bw, scale_bw) ||
        !calibrate_channels(&p->op[QGRU_OP_BR], p->granularity[3], pot2, H, r->min_br, r->max_br, scale_br))
        return QGRU_ERR_RANGE;
    return qgru_generate_luts(p);
}

}  // extern "C"
