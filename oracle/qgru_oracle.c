/*
 * qgru_oracle.c - TEST INFRASTRUCTURE, not product code.
 *
 * A plain-C restatement of the CPU integer path of CX9898/quant-gru-pytorch, used only as
 * the checker in tests/, in the smoke test and as the "port" CPU baseline of the benchmark.
 * The product library never links, loads or calls anything in this file.
 *
 * Parity of this restatement is PINNED: tests/test_oracle_vs_ref.py compares every function
 * here with the unmodified reference sources compiled into oracle/_ref/ (see Makefile), and
 * tests/golden/ holds input/output vectors generated from those reference sources.
 *
 * Each function cites the reference lines it restates (paths relative to the reference root).
 * Compile with -ffp-contract=off -fno-fast-math: the float expressions below must be
 * evaluated operation by operation in IEEE single/double precision like the reference's.
 */
#include <float.h>
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "qgru.h"

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ primitives */

/* include/quantize_ops_helper.h:183-206 (int64 overload; the one the datapath uses). */
ORC_API int64_t orc_rshift_round(int64_t x, int n) {
    if (n <= 0) return (int64_t)((uint64_t)x << (-n));
    const int neg = x < 0;
    const int64_t a = neg ? -x : x;
    const int64_t half = (int64_t)1 << (n - 1);
    const int64_t mask = ((int64_t)1 << n) - 1;
    const int64_t q = a >> n;
    const int64_t r = a & mask;
    int64_t res;
    if (r > half) res = q + 1;
    else if (r < half) res = q;
    else res = (q & 1) ? q + 1 : q;
    return neg ? -res : res;
}

/* One execution-time rescale: FixedPointScale or Pot2Rescale
 * (include/quantize_param_types.h:37-46). */
typedef struct orc_rescale {
    uint16_t mult;
    int8_t shift;
    uint8_t pot2;
} orc_rescale;

/* include/quantize_ops_helper.h:224-230. */
static int64_t apply_rescale(int64_t x, orc_rescale r) {
    if (r.pot2) return orc_rshift_round(x, r.shift);
    return orc_rshift_round(x * (int64_t)r.mult, r.shift);
}

/* include/quantize_ops_helper.h:245-264.  Returns 0 on success, 1 where the reference throws. */
ORC_API int orc_encode_mshift(float scale, uint16_t *mult, int8_t *shift) {
    if (!(scale > 0.0f)) return 1;
    int e = 0;
    double mant = frexp((double)scale, &e);
    uint32_t m = (uint32_t)llround(mant * 65536.0);
    if (m == 65536u) { m = 32768u; e += 1; }
    if (m < 32768u) m = 32768u;
    const int s = 16 - e;
    if (s < -128 || s > 127) return 1;
    *mult = (uint16_t)m;
    *shift = (int8_t)s;
    return 0;
}

/* include/quantize_ops_helper.h:272-275. */
static int8_t pot2_shift(float scale) {
    if (!(scale > 0.0f)) return 0;
    return (int8_t)lround(-log2((double)scale));
}

/* toFixedScale, include/quantize_ops_helper.h:280-283. */
static int to_fixed_scale(float scale, int use_pot2, uint16_t *m, int8_t *s) {
    if (use_pot2) { *m = 1; *s = pot2_shift(scale); return 0; }
    return orc_encode_mshift(scale, m, s);
}

/* decode_scale, include/quantize_ops_helper.h:94-100. */
static float decode_scale(uint16_t m, int8_t s) { return (float)m * ldexpf(1.0f, -(int)s); }

/* makeRescale / makeRescaleProduct / makeRescaleToProduct,
 * include/quantize_ops_helper.h:296-350. */
static int make_rescale(float src, float dst, int pot2, orc_rescale *r) {
    r->pot2 = (uint8_t)pot2;
    if (pot2) { r->mult = 1; r->shift = (int8_t)(pot2_shift(src) - pot2_shift(dst)); return 0; }
    return orc_encode_mshift(src / dst, &r->mult, &r->shift);
}
static int make_rescale_product(float a, float b, float dst, int pot2, orc_rescale *r) {
    r->pot2 = (uint8_t)pot2;
    if (pot2) {
        r->mult = 1;
        r->shift = (int8_t)(pot2_shift(a) + pot2_shift(b) - pot2_shift(dst));
        return 0;
    }
    return orc_encode_mshift((a * b) / dst, &r->mult, &r->shift);
}
static int make_rescale_to_product(float src, float a, float b, int pot2, orc_rescale *r) {
    r->pot2 = (uint8_t)pot2;
    if (pot2) {
        r->mult = 1;
        r->shift = (int8_t)(pot2_shift(src) - (pot2_shift(a) + pot2_shift(b)));
        return 0;
    }
    return orc_encode_mshift(src / (a * b), &r->mult, &r->shift);
}

/* QuantBitWidth::qmin/qmax, include/quantize_bitwidth_config.h:14-22. */
static int32_t qmin_of(int bits, int uns) {
    if (bits >= 32) return INT32_MIN;
    return uns ? 0 : -(1 << (bits - 1));
}
static int32_t qmax_of(int bits, int uns) {
    if (bits >= 32) return INT32_MAX;
    return uns ? (int32_t)((1u << bits) - 1u) : (1 << (bits - 1)) - 1;
}
static int eff_unsigned(const qgru_op *o) { return o->bits >= 32 ? 0 : o->is_unsigned; }

/* clamp_by_bitwidth, include/quantize_ops_helper.h:365-376. */
static int32_t clamp_bw(int32_t v, const qgru_op *o) {
    const int32_t lo = qmin_of(o->bits, eff_unsigned(o)), hi = qmax_of(o->bits, eff_unsigned(o));
    return v < lo ? lo : (v > hi ? hi : v);
}

/* clamp_by_bitwidth<Training>: *keep = 1 iff v was inside the range (the flag the backward pass
 * multiplies gradients with), include/quantize_ops_helper.h:365-376.  keep may be NULL. */
static int32_t clamp_keep(int32_t v, const qgru_op *o, uint8_t *keep) {
    const int32_t c = clamp_bw(v, o);
    if (keep) *keep = (uint8_t)(c == v);
    return c;
}

/* quantize(float, FixedPointScale, zp, bw), include/quantize_ops_helper.h:528-533. */
static int32_t quantize_fs(float x, uint16_t m, int8_t s, int32_t zp, const qgru_op *o) {
    float q = rintf(x / decode_scale(m, s)) + (float)zp;
    return clamp_bw((int32_t)q, o);
}

/* dequantize(q, FixedPointScale, zp), include/quantize_ops_helper.h:504-508. */
static float dequantize_fs(int32_t q, uint16_t m, int8_t s, int32_t zp) {
    return (float)(q - zp) * decode_scale(m, s);
}

/* ------------------------------------------------------------------------- LUT */

/* piecewise_linear, include/quantize_ops_helper.h:560-606. */
static int32_t lut_eval_keep(const qgru_lut *lut, int32_t q_x, const qgru_op *in_bw,
                             const qgru_op *out_bw, uint8_t *keep_in, uint8_t *keep_out);
ORC_API int32_t orc_lut_eval(const qgru_lut *lut, int32_t q_x, const qgru_op *in_bw,
                             const qgru_op *out_bw) {
    return lut_eval_keep(lut, q_x, in_bw, out_bw, NULL, NULL);
}
/* The training branch keeps the two clamp flags (gate input, gate output),
 * include/quantize_ops_helper.h:760-783. */
static int32_t lut_eval_keep(const qgru_lut *lut, int32_t q_x, const qgru_op *in_bw,
                             const qgru_op *out_bw, uint8_t *keep_in, uint8_t *keep_out) {
    const int32_t q = clamp_keep(q_x, in_bw, keep_in);
    int seg = QGRU_LUT_SEGMENTS - 1;
    for (int i = 0; i < QGRU_LUT_SEGMENTS; ++i)
        if (q < lut->seg[i].threshold) { seg = i; break; }
    const qgru_lut_segment *s = &lut->seg[seg];
    const int32_t x_off = q - lut->zp_x;
    const int64_t bx = (int64_t)s->q_b * (int64_t)x_off;
    const int n = (int8_t)s->n_bx;
    const int32_t term = (n >= 0) ? (int32_t)orc_rshift_round(bx, n)
                                  : (int32_t)((uint64_t)bx << (-n));
    return clamp_keep((int32_t)((uint32_t)term + (uint32_t)s->term_c), out_bw, keep_out);
}

/* linear_fit, src/quantize_ops.cu:996-1017. */
static void linear_fit(const float *x, const float *y, int n, float *b, float *c) {
    float sx = 0.0f, sy = 0.0f, sxy = 0.0f, sx2 = 0.0f;
    for (int i = 0; i < n; ++i) {
        sx += x[i];
        sy += y[i];
        sxy += x[i] * y[i];
        sx2 += x[i] * x[i];
    }
    float denom = n * sx2 - sx * sx;
    if (fabsf(denom) < 1e-9f) { *b = 0.0f; *c = sy / n; return; }
    *b = (n * sxy - sx * sy) / denom;
    *c = (sy - *b * sx) / n;
}

static int cmp_float(const void *a, const void *b) {
    const float x = *(const float *)a, y = *(const float *)b;
    return (x > y) - (x < y);
}

/* adaptive_segmentation_sigmoid, src/quantize_ops.cu:1022-1117.  `points` receives
 * num_segments+1 values; returns the number of points produced. */
static int adaptive_segmentation(float x_min, float x_max, int num_segments, float *points) {
    const float centerWeight = 5.0f, centerRange = 2.0f;
    enum { NS = 1000 };
    static __thread float xs[NS], w[NS - 1], cw[NS - 1];
    for (int i = 0; i < NS; ++i) xs[i] = x_min + (x_max - x_min) * (float)i / (NS - 1);
    for (int i = 0; i < NS - 1; ++i) {
        const float x = xs[i], xn = xs[i + 1];
        const float y = 1.0f / (1.0f + expf(-x));
        const float yn = 1.0f / (1.0f + expf(-xn));
        const float slope = fabsf(yn - y) / (xn - x + 1e-9f);
        const float d = fabsf(x);
        if (d < centerRange) w[i] = centerWeight * (1.0f - d / centerRange) + 1.0f;
        else w[i] = 1.0f + slope * 0.5f;
    }
    float sum = 0.0f;
    for (int i = 0; i < NS - 1; ++i) sum += w[i];
    for (int i = 0; i < NS - 1; ++i) w[i] /= sum;
    cw[0] = w[0];
    for (int i = 1; i < NS - 1; ++i) cw[i] = cw[i - 1] + w[i];

    int np = 0;
    float pts[64];
    pts[np++] = x_min;
    for (int i = 1; i < num_segments; ++i) {
        const float target = (float)i / num_segments;
        int lo = 0, hi = NS - 1; /* std::lower_bound over cw[0..NS-2] */
        while (lo < hi) {
            const int mid = (lo + hi) / 2;
            if (cw[mid] < target) lo = mid + 1; else hi = mid;
        }
        int idx = lo;
        if (idx >= NS - 1) idx = NS - 2;
        pts[np++] = xs[idx];
    }
    pts[np++] = x_max;
    qsort(pts, (size_t)np, sizeof(float), cmp_float);
    /* std::unique with |a-b| < 1e-9 */
    int m = 0;
    for (int i = 0; i < np; ++i) {
        if (m == 0 || !(fabsf(pts[m - 1] - pts[i]) < 1e-9f)) pts[m++] = pts[i];
    }
    np = m;
    while (np < num_segments + 1) {
        float max_gap = 0.0f;
        int gi = 0;
        for (int i = 0; i + 1 < np; ++i) {
            const float gap = pts[i + 1] - pts[i];
            if (gap > max_gap) { max_gap = gap; gi = i; }
        }
        const float nw = (pts[gi] + pts[gi + 1]) / 2.0f;
        for (int i = np; i > gi + 1; --i) pts[i] = pts[i - 1];
        pts[gi + 1] = nw;
        ++np;
    }
    memcpy(points, pts, sizeof(float) * (size_t)np);
    return np;
}

/* quantize_multiplier_signed, src/quantize_ops.cu:1137-1146. */
static void quantize_multiplier_signed(float value, const qgru_op *out_bw, int32_t *q_out,
                                       int8_t *n_out) {
    if (fabsf(value) < 1e-12f) { *q_out = 0; *n_out = 0; return; }
    const int32_t max_q = qmax_of(out_bw->bits, eff_unsigned(out_bw));
    const int8_t n = (int8_t)floor(log2((double)max_q / fabsf(value)));
    int64_t q = (int64_t)rint((double)value * ldexp(1.0, n));
    if (q > max_q) q = max_q;
    if (q < -(int64_t)max_q) q = -(int64_t)max_q;
    *q_out = (int32_t)q;
    *n_out = n;
}

/* generate_sigmoid_lut / generate_tanh_lut (float-scale overloads),
 * src/quantize_ops.cu:1148-1221 and 1237-1307. */
static void generate_lut(int is_tanh, float scale_x, int32_t zp_x, float scale_y, int32_t zp_y,
                         const qgru_op *in_bw, const qgru_op *out_bw, qgru_lut *lut) {
    const int32_t qmn = qmin_of(in_bw->bits, eff_unsigned(in_bw));
    const int32_t qmx = qmax_of(in_bw->bits, eff_unsigned(in_bw));
    float x_min = (float)(qmn - zp_x) * scale_x;
    float x_max = (float)(qmx - zp_x) * scale_x;
    const float R = is_tanh ? 4.0f : 8.0f;
    x_min = fmaxf(x_min, -R);
    x_max = fminf(x_max, R);
    memset(lut, 0, sizeof(*lut));
    lut->zp_x = zp_x;
    float pts[64];
    adaptive_segmentation(x_min, x_max, QGRU_LUT_SEGMENTS, pts);
    for (int i = 0; i < QGRU_LUT_SEGMENTS; ++i) {
        const float xs = pts[i], xe = pts[i + 1];
        float xv[100], yv[100];
        for (int j = 0; j < 100; ++j) {
            const float x = xs + (xe - xs) * (float)j / 99;
            xv[j] = x;
            yv[j] = is_tanh ? tanhf(x) : 1.0f / (1.0f + expf(-x));
        }
        float b, c;
        linear_fit(xv, yv, 100, &b, &c);
        const float m_real = b * (scale_x / scale_y);
        int32_t q_b;
        int8_t n;
        quantize_multiplier_signed(m_real, out_bw, &q_b, &n);
        const int32_t term_c = (int32_t)rintf(c / scale_y + (float)zp_y);
        /* `coeff.x_end / scale_x + zp_x`: float + int32 -> float */
        int32_t thr = (int32_t)rintf(xe / scale_x + (float)zp_x);
        thr = clamp_bw(thr, in_bw);
        lut->seg[i].q_b = q_b;
        lut->seg[i].n_bx = n;
        lut->seg[i].term_c = term_c;
        lut->seg[i].threshold = thr;
    }
}

/* generate_piecewise_linear_lut_to_params, src/quantize_ops.cu:21-52. */
ORC_API int orc_generate_luts(qgru_params *p) {
    generate_lut(0, p->op[QGRU_OP_UPDATE_IN].scale, p->op[QGRU_OP_UPDATE_IN].zero_point,
                 p->op[QGRU_OP_UPDATE_OUT].scale, p->op[QGRU_OP_UPDATE_OUT].zero_point,
                 &p->op[QGRU_OP_UPDATE_IN], &p->op[QGRU_OP_UPDATE_OUT], &p->lut[QGRU_LUT_UPDATE]);
    generate_lut(0, p->op[QGRU_OP_RESET_IN].scale, p->op[QGRU_OP_RESET_IN].zero_point,
                 p->op[QGRU_OP_RESET_OUT].scale, p->op[QGRU_OP_RESET_OUT].zero_point,
                 &p->op[QGRU_OP_RESET_IN], &p->op[QGRU_OP_RESET_OUT], &p->lut[QGRU_LUT_RESET]);
    generate_lut(1, p->op[QGRU_OP_NEW_IN].scale, p->op[QGRU_OP_NEW_IN].zero_point,
                 p->op[QGRU_OP_NEW_OUT].scale, p->op[QGRU_OP_NEW_OUT].zero_point,
                 &p->op[QGRU_OP_NEW_IN], &p->op[QGRU_OP_NEW_OUT], &p->lut[QGRU_LUT_NEW]);
    return 0;
}

/* --------------------------------------------------- params from MinMax ranges */

/* get_minimum_scale, include/histogram_collector.h:31-35. */
static float minimum_scale(int64_t num_steps) {
    const float eps = 1.19209290e-07f;
    const float v = 0.01f / (float)num_steps;
    return eps < v ? eps : v;
}

/* calibrateContinuousScaleFromRange, include/pot_sqnr_calibrator.h:546-613. */
static int continuous_from_range(float mn, float mx, const qgru_op *o, int symmetric,
                                 float *scale_out, float *min_out) {
    const int uns = eff_unsigned(o);
    const int32_t qmn = qmin_of(o->bits, uns), qmx = qmax_of(o->bits, uns);
    const int64_t num_steps = (int64_t)qmx - (int64_t)qmn;
    if (num_steps <= 0) return 1;
    const float ms = minimum_scale(num_steps);
    const float min0 = fminf(mn, 0.0f), max0 = fmaxf(mx, 0.0f);
    const float diff = (max0 - min0) / (float)num_steps;
    const float adj = (diff < ms) ? ms : 0.0f;
    float umin = min0, umax = max0;
    if (symmetric) {
        if (uns) { umax = max0 + (float)num_steps * adj; umin = 0.0f; }
        else {
            umax = max0 + floorf((float)num_steps / 2.0f) * adj;
            umin = min0 - ceilf((float)num_steps / 2.0f) * adj;
        }
    } else {
        umax = max0 + (float)num_steps * adj;
    }
    float scale, amin;
    if (symmetric) {
        if (uns) {
            const float dmax = fmaxf(umax, ms);
            scale = fmaxf(dmax / (float)qmx, ms);
            amin = 0.0f;
        } else {
            const int64_t pos = num_steps / 2, neg = (num_steps + 1) / 2;
            const int add = (num_steps == 3) ? 1 : 0;
            const float dmax = (pos + add > 0) ? umax / (float)(pos + add) : 0.0f;
            const float dmin = (neg > 0) ? -umin / (float)neg : 0.0f;
            scale = fmaxf(fmaxf(dmax, dmin), ms);
            amin = -(float)neg * scale;
        }
    } else {
        const float range = fmaxf(umax - umin, ms * (float)num_steps);
        scale = fmaxf(range / (float)num_steps, ms);
        amin = umin;
    }
    *scale_out = scale;
    *min_out = amin;
    return 0;
}

/* encodeScaleResult(coverage_round=true) + storedScaleForMode,
 * include/pot_sqnr_calibrator.h:451-524 and 72-74. */
static int encode_scale(float cscale, float cmin, const qgru_op *o, int symmetric, int pot2,
                        int coverage_round, float *stored_scale, int32_t *zp) {
    const int64_t qmn = qmin_of(o->bits, eff_unsigned(o));
    if (pot2) {
        float nf;
        if (coverage_round) nf = floorf(log2f(1.0f / cscale));
        else nf = rintf(-log2f(cscale));
        if (nf < -128.0f || nf > 127.0f) return 1;
        const int8_t n = (int8_t)nf;
        const float po2 = powf(2.0f, -(float)n);
        if (symmetric) *zp = 0;
        else if (coverage_round) {
            const float amin = floorf(cmin / po2) * po2;
            *zp = (int32_t)rintf((float)qmn - amin / po2);
        } else {
            *zp = (int32_t)rintf((float)qmn - cmin / po2);
        }
        *stored_scale = po2;
        return 0;
    }
    uint16_t m;
    int8_t s;
    if (orc_encode_mshift(cscale, &m, &s)) return 1;
    const float eff = (float)m * ldexpf(1.0f, -(int)s);
    *zp = symmetric ? 0 : (int32_t)rintf((float)qmn - cmin / eff);
    *stored_scale = cscale;
    return 0;
}

static int calibrate_scalar(float mn, float mx, qgru_op *o, int pot2) {
    float cs, cmin;
    if (continuous_from_range(mn, mx, o, o->symmetric, &cs, &cmin)) return 1;
    return encode_scale(cs, cmin, o, o->symmetric, pot2, 1, &o->scale, &o->zero_point);
}

/* ensureMinRange, include/calibration_utils.h:27-45. */
static void ensure_min_range(float *mn, float *mx, float thr) {
    const float range = *mx - *mn;
    if (range < thr) {
        const float c = (*mn + *mx) / 2.0f;
        *mn = c - thr / 2.0f;
        *mx = c + thr / 2.0f;
    }
}

static int calibrate_channels(qgru_op *o, int gran, int pot2, int H, const float *mins,
                              const float *maxs, float *scales) {
    const int C = 3 * H;
    qgru_op tmp = *o;
    if (gran == QGRU_PER_TENSOR) {
        float mn = mins[0], mx = maxs[0];
        for (int c = 1; c < C; ++c) { if (mins[c] < mn) mn = mins[c]; if (maxs[c] > mx) mx = maxs[c]; }
        if (calibrate_scalar(mn, mx, &tmp, pot2)) return 1;
        for (int c = 0; c < C; ++c) scales[c] = tmp.scale;
    } else if (gran == QGRU_PER_GATE) {
        for (int g = 0; g < 3; ++g) {
            float mn = FLT_MAX, mx = -FLT_MAX;
            for (int c = g * H; c < (g + 1) * H; ++c) { mn = fminf(mn, mins[c]); mx = fmaxf(mx, maxs[c]); }
            if (calibrate_scalar(mn, mx, &tmp, pot2)) return 1;
            for (int c = g * H; c < (g + 1) * H; ++c) scales[c] = tmp.scale;
        }
    } else {
        for (int c = 0; c < C; ++c) {
            if (calibrate_scalar(mins[c], maxs[c], &tmp, pot2)) return 1;
            scales[c] = tmp.scale;
        }
    }
    o->scale = scales[0];
    o->zero_point = 0;
    return 0;
}

/* calculateGRUQuantitativeParameters, src/gru_interface.cc:51-158. */
ORC_API int orc_calc_params_from_ranges(const qgru_ranges *r, qgru_params *p, float *sW,
                                        float *sR, float *sbw, float *sbr) {
    if (!p->op[QGRU_OP_W].symmetric || !p->op[QGRU_OP_R].symmetric ||
        !p->op[QGRU_OP_BW].symmetric || !p->op[QGRU_OP_BR].symmetric)
        return 1; /* ensureSymmetricWeightBiasConfig, src/gru_interface.cc:26-32 */
    const int pot2 = p->use_pot2 != 0;
    const int H = r->hidden;
    p->hidden = H;
    static const int plain[] = {QGRU_OP_X, QGRU_OP_H, QGRU_OP_IH_LINEAR, QGRU_OP_HH_LINEAR,
                                QGRU_OP_UPDATE_IN, QGRU_OP_RESET_IN, QGRU_OP_NEW_IN,
                                QGRU_OP_MUL_RESET_HIDDEN, QGRU_OP_MUL_NEW_CONTRIB,
                                QGRU_OP_MUL_OLD_CONTRIB};
    for (size_t i = 0; i < sizeof(plain) / sizeof(plain[0]); ++i) {
        const int k = plain[i];
        if (calibrate_scalar(r->min_v[k], r->max_v[k], &p->op[k], pot2)) return 1;
    }
    static const int acts[] = {QGRU_OP_UPDATE_OUT, QGRU_OP_RESET_OUT, QGRU_OP_NEW_OUT};
    for (int i = 0; i < 3; ++i) {
        const int k = acts[i];
        float mn = r->min_v[k], mx = r->max_v[k];
        ensure_min_range(&mn, &mx, 0.5f);
        if (calibrate_scalar(mn, mx, &p->op[k], pot2)) return 1;
    }
    if (calibrate_channels(&p->op[QGRU_OP_W], p->granularity[0], pot2, H, r->min_W, r->max_W, sW)) return 1;
    if (calibrate_channels(&p->op[QGRU_OP_R], p->granularity[1], pot2, H, r->min_R, r->max_R, sR)) return 1;
    if (calibrate_channels(&p->op[QGRU_OP_BW], p->granularity[2], pot2, H, r->min_bw, r->max_bw, sbw)) return 1;
    if (calibrate_channels(&p->op[QGRU_OP_BR], p->granularity[3], pot2, H, r->min_br, r->max_br, sbr)) return 1;
    return orc_generate_luts(p);
}

/* ------------------------------------------------------- quantize boundaries */

/* quantitativeWeightCPU, src/gru_interface.cc:341-373. */
ORC_API int orc_quantize_weights(int I, int H, const float *W, const float *R, const float *bw,
                                 const float *br, const qgru_params *p, const float *sW,
                                 const float *sR, const float *sbw, const float *sbr,
                                 int32_t *W_q, int32_t *R_q, int32_t *bw_q, int32_t *br_q) {
    const int C = 3 * H;
    const int pot2 = p->use_pot2 != 0;
    for (int m = 0; m < C; ++m) {
        uint16_t mu;
        int8_t sh;
        if (to_fixed_scale(sW[m], pot2, &mu, &sh)) return 1;
        for (int k = 0; k < I; ++k)
            W_q[(size_t)k * C + m] = quantize_fs(W[(size_t)k * C + m], mu, sh, 0, &p->op[QGRU_OP_W]);
        if (to_fixed_scale(sR[m], pot2, &mu, &sh)) return 1;
        for (int k = 0; k < H; ++k)
            R_q[(size_t)k * C + m] = quantize_fs(R[(size_t)k * C + m], mu, sh, 0, &p->op[QGRU_OP_R]);
        if (to_fixed_scale(sbw[m], pot2, &mu, &sh)) return 1;
        bw_q[m] = quantize_fs(bw[m], mu, sh, 0, &p->op[QGRU_OP_BW]);
        if (to_fixed_scale(sbr[m], pot2, &mu, &sh)) return 1;
        br_q[m] = quantize_fs(br[m], mu, sh, 0, &p->op[QGRU_OP_BR]);
    }
    return 0;
}

/* x / h0 quantize, src/gru_interface.cc:806-824. */
ORC_API int orc_quantize(const float *x, int32_t *out, size_t n, const qgru_params *p, int op) {
    uint16_t m;
    int8_t s;
    if (to_fixed_scale(p->op[op].scale, p->use_pot2 != 0, &m, &s)) return 1;
    for (size_t i = 0; i < n; ++i) out[i] = quantize_fs(x[i], m, s, p->op[op].zero_point, &p->op[op]);
    return 0;
}

/* h dequantize, src/gru_interface.cc:838-840. */
ORC_API int orc_dequantize(const int32_t *q, float *out, size_t n, const qgru_params *p, int op) {
    uint16_t m;
    int8_t s;
    if (to_fixed_scale(p->op[op].scale, p->use_pot2 != 0, &m, &s)) return 1;
    for (size_t i = 0; i < n; ++i) out[i] = dequantize_fs(q[i], m, s, p->op[op].zero_point);
    return 0;
}

/* ------------------------------------------------------------ integer forward */

typedef struct orc_derived {
    /* fillLinearParamsCPU, src/gru_forward_cpu_quant.cc:221-243 */
    orc_rescale *gemm_x, *bias_w, *gemm_h, *bias_r; /* [3H] */
    /* fillGateParamsCPU, src/gru_forward_cpu_quant.cc:246-285 */
    orc_rescale ih_to_z, hh_to_z, ih_to_r, hh_to_r, ih_to_n, rh_to_n, n_to_h, uh_to_h;
    int32_t one_q;
} orc_derived;

static int derive(const qgru_params *p, const float *sW, const float *sR, const float *sbw,
                  const float *sbr, orc_derived *d) {
    const int C = 3 * p->hidden, pot2 = p->use_pot2 != 0;
    const float s_x = p->op[QGRU_OP_X].scale, s_h = p->op[QGRU_OP_H].scale;
    const float s_ih = p->op[QGRU_OP_IH_LINEAR].scale, s_hh = p->op[QGRU_OP_HH_LINEAR].scale;
    d->gemm_x = (orc_rescale *)malloc(sizeof(orc_rescale) * 4 * (size_t)C);
    if (!d->gemm_x) return 1;
    d->bias_w = d->gemm_x + C;
    d->gemm_h = d->bias_w + C;
    d->bias_r = d->gemm_h + C;
    int bad = 0;
    for (int c = 0; c < C; ++c) {
        bad |= make_rescale_product(sW[c], s_x, s_ih, pot2, &d->gemm_x[c]);
        bad |= make_rescale_to_product(sbw[c], sW[c], s_x, pot2, &d->bias_w[c]);
        bad |= make_rescale_product(sR[c], s_h, s_hh, pot2, &d->gemm_h[c]);
        bad |= make_rescale_to_product(sbr[c], sR[c], s_h, pot2, &d->bias_r[c]);
    }
    bad |= make_rescale(s_ih, p->op[QGRU_OP_UPDATE_IN].scale, pot2, &d->ih_to_z);
    bad |= make_rescale(s_hh, p->op[QGRU_OP_UPDATE_IN].scale, pot2, &d->hh_to_z);
    bad |= make_rescale(s_ih, p->op[QGRU_OP_RESET_IN].scale, pot2, &d->ih_to_r);
    bad |= make_rescale(s_hh, p->op[QGRU_OP_RESET_IN].scale, pot2, &d->hh_to_r);
    bad |= make_rescale(s_ih, p->op[QGRU_OP_NEW_IN].scale, pot2, &d->ih_to_n);
    bad |= make_rescale_product(p->op[QGRU_OP_RESET_OUT].scale, s_hh, p->op[QGRU_OP_NEW_IN].scale,
                                pot2, &d->rh_to_n);
    d->one_q = (int32_t)rintf(1.0f / p->op[QGRU_OP_UPDATE_OUT].scale) +
               p->op[QGRU_OP_UPDATE_OUT].zero_point;
    bad |= make_rescale(p->op[QGRU_OP_NEW_OUT].scale, s_h, pot2, &d->n_to_h);
    bad |= make_rescale_product(p->op[QGRU_OP_UPDATE_OUT].scale, s_h, s_h, pot2, &d->uh_to_h);
    if (bad) { free(d->gemm_x); d->gemm_x = NULL; }
    return bad;
}

/* computeUpdateGate / computeResetGate (inference branch),
 * include/quantize_ops_helper.h:749-821 and 832-901. */
static int32_t sigmoid_gate(int32_t ih, int32_t hh, const qgru_params *p, orc_rescale r_ih,
                            orc_rescale r_hh, int op_in, int op_out, int lut, uint8_t *keep) {
    const int64_t ih_d = (int64_t)ih - p->op[QGRU_OP_IH_LINEAR].zero_point;
    const int64_t hh_d = (int64_t)hh - p->op[QGRU_OP_HH_LINEAR].zero_point;
    const int32_t a = (int32_t)apply_rescale(ih_d, r_ih);
    const int32_t b = (int32_t)apply_rescale(hh_d, r_hh);
    const int32_t in = (int32_t)((uint32_t)a + (uint32_t)b + (uint32_t)p->op[op_in].zero_point);
    return lut_eval_keep(&p->lut[lut], in, &p->op[op_in], &p->op[op_out], keep, keep ? keep + 1 : NULL);
}

/* computeNewGate, include/quantize_ops_helper.h:917-997. */
static int32_t new_gate(int32_t ih, int32_t hh, int32_t r, const qgru_params *p,
                        const orc_derived *d, uint8_t *keep) {
    const int64_t r_d = (int64_t)r - p->op[QGRU_OP_RESET_OUT].zero_point;
    const int64_t hh_d = (int64_t)hh - p->op[QGRU_OP_HH_LINEAR].zero_point;
    const int32_t rh = (int32_t)apply_rescale(r_d * hh_d, d->rh_to_n);
    const int32_t a = (int32_t)apply_rescale((int64_t)ih - p->op[QGRU_OP_IH_LINEAR].zero_point, d->ih_to_n);
    const int32_t in = (int32_t)((uint32_t)a + (uint32_t)rh + (uint32_t)p->op[QGRU_OP_NEW_IN].zero_point);
    return lut_eval_keep(&p->lut[QGRU_LUT_NEW], in, &p->op[QGRU_OP_NEW_IN], &p->op[QGRU_OP_NEW_OUT], keep,
                         keep ? keep + 1 : NULL);
}

/* computeHiddenState, include/quantize_ops_helper.h:1008-1084. */
static int32_t hidden_state(int32_t u, int32_t n, int32_t h_old, const qgru_params *p,
                            const orc_derived *d, uint8_t *keep) {
    const int32_t zp_h = p->op[QGRU_OP_H].zero_point;
    const int32_t zp_u = p->op[QGRU_OP_UPDATE_OUT].zero_point;
    const int64_t n_d = (int64_t)n - p->op[QGRU_OP_NEW_OUT].zero_point;
    const int32_t n_al = (int32_t)((uint32_t)(int32_t)apply_rescale(n_d, d->n_to_h) + (uint32_t)zp_h);
    const int64_t u_d = (int64_t)u - zp_u;
    const int64_t h_d = (int64_t)h_old - zp_h;
    const int64_t old_c = u_d * h_d;
    const int64_t one_minus_u = (int64_t)d->one_q - u;
    const int64_t omu_d = one_minus_u - zp_u;
    const int64_t n_ald = (int64_t)n_al - zp_h;
    const int64_t new_c = omu_d * n_ald;
    const int32_t h_new = (int32_t)((uint32_t)(int32_t)apply_rescale(old_c + new_c, d->uh_to_h) + (uint32_t)zp_h);
    return clamp_keep(h_new, &p->op[QGRU_OP_H], keep);
}

/* ComputeLinearX / ComputeLinearH with PrecomputeWeightSums,
 * src/gru_forward_cpu_quant.cc:76-168.  Wt is [K][C] (haste layout), in is [N][K]. */
static void linear(int N, int K, int C, const int32_t *Wt, const int32_t *in, const int32_t *bias,
                   int32_t zp_in, const orc_rescale *r_gemm, const orc_rescale *r_bias,
                   const qgru_op *out_op, int32_t *out, uint8_t *keep) {
    int64_t *wsum = (int64_t *)malloc(sizeof(int64_t) * (size_t)C);
    int64_t *acc = (int64_t *)malloc(sizeof(int64_t) * (size_t)C);
    for (int m = 0; m < C; ++m) {
        int64_t s = 0;
        for (int k = 0; k < K; ++k) s += Wt[(size_t)k * C + m];
        wsum[m] = s * zp_in;
    }
    for (int n = 0; n < N; ++n) {
        for (int m = 0; m < C; ++m) acc[m] = 0;
        for (int k = 0; k < K; ++k) {
            const int64_t xv = in[(size_t)n * K + k];
            const int32_t *wr = Wt + (size_t)k * C;
            for (int m = 0; m < C; ++m) acc[m] += (int64_t)wr[m] * xv;
        }
        for (int m = 0; m < C; ++m) {
            const int64_t g = acc[m] - wsum[m];
            const int64_t b = apply_rescale((int64_t)bias[m], r_bias[m]);
            const int64_t v = apply_rescale(g + b, r_gemm[m]);
            const int32_t res = (int32_t)((uint32_t)(int32_t)v + (uint32_t)out_op->zero_point);
            out[(size_t)n * C + m] = clamp_keep(res, out_op, keep ? keep + (size_t)n * C + m : NULL);
        }
    }
    free(wsum);
    free(acc);
}

/* ForwardPassQuantCPU::RunImpl + the h_q[0] initialisation of quantGRUForwardCPU,
 * src/gru_forward_cpu_quant.cc:302-325 and src/gru_interface.cc:815-824. */
static int forward_i32_impl(int T, int B, int I, int H, const int32_t *W, const int32_t *R,
                            const int32_t *bw, const int32_t *br, const int32_t *x_q,
                            const int32_t *h0_q, const qgru_params *p, const float *sW,
                            const float *sR, const float *sbw, const float *sbr, int32_t *h_q,
                            int32_t *v_q, uint8_t *const *masks);

ORC_API int orc_forward_i32(int T, int B, int I, int H, const int32_t *W, const int32_t *R,
                            const int32_t *bw, const int32_t *br, const int32_t *x_q,
                            const int32_t *h0_q, const qgru_params *p, const float *sW,
                            const float *sR, const float *sbw, const float *sbr, int32_t *h_q) {
    return forward_i32_impl(T, B, I, H, W, R, bw, br, x_q, h0_q, p, sW, sR, sbw, sbr, h_q, NULL, NULL);
}

/* Training-mode forward: also v_q [T,B,4H] = (update, reset, new gate outputs, R*h + br row of
 * the new gate), src/gru_forward_cpu_quant.cc:199-205. */
ORC_API int orc_forward_i32_v(int T, int B, int I, int H, const int32_t *W, const int32_t *R,
                              const int32_t *bw, const int32_t *br, const int32_t *x_q,
                              const int32_t *h0_q, const qgru_params *p, const float *sW,
                              const float *sR, const float *sbw, const float *sbr, int32_t *h_q,
                              int32_t *v_q) {
    return forward_i32_impl(T, B, I, H, W, R, bw, br, x_q, h0_q, p, sW, sR, sbw, sbr, h_q, v_q, NULL);
}

/* Training-mode forward with the five clamp masks of quantGRUForwardInt32
 * (include/gru_interface.h:380-402; written by src/gru_forward_gpu_quant.cu:168-178 and
 * :318-348): masks[0] W*x+bw [T*B,3H], masks[1] R*h+br [T*B,3H], masks[2] gate inputs
 * [T*B,3H], masks[3] gate outputs [T*B,3H], masks[4] h [T*B,H]; 1 = the value was not clamped.
 * Any of the five may be NULL. */
ORC_API int orc_forward_i32_train(int T, int B, int I, int H, const int32_t *W, const int32_t *R,
                                  const int32_t *bw, const int32_t *br, const int32_t *x_q,
                                  const int32_t *h0_q, const qgru_params *p, const float *sW,
                                  const float *sR, const float *sbw, const float *sbr, int32_t *h_q,
                                  int32_t *v_q, uint8_t *const *masks) {
    return forward_i32_impl(T, B, I, H, W, R, bw, br, x_q, h0_q, p, sW, sR, sbw, sbr, h_q, v_q, masks);
}

static int forward_i32_impl(int T, int B, int I, int H, const int32_t *W, const int32_t *R,
                            const int32_t *bw, const int32_t *br, const int32_t *x_q,
                            const int32_t *h0_q, const qgru_params *p, const float *sW,
                            const float *sR, const float *sbw, const float *sbr, int32_t *h_q,
                            int32_t *v_q, uint8_t *const *masks) {
    if (p->hidden != H) return 1;
    uint8_t *m_ih = masks ? masks[0] : NULL, *m_hh = masks ? masks[1] : NULL;
    uint8_t *m_gi = masks ? masks[2] : NULL, *m_go = masks ? masks[3] : NULL;
    uint8_t *m_h = masks ? masks[4] : NULL;
    orc_derived d;
    if (derive(p, sW, sR, sbw, sbr, &d)) return 1;
    const int C = 3 * H;
    const size_t NH = (size_t)B * H;
    int32_t *ih = (int32_t *)malloc(sizeof(int32_t) * (size_t)T * B * C);
    int32_t *hh = (int32_t *)malloc(sizeof(int32_t) * (size_t)B * C);
    if (!ih || !hh) { free(ih); free(hh); free(d.gemm_x); return 1; }
    for (size_t i = 0; i < NH; ++i) h_q[i] = h0_q ? h0_q[i] : p->op[QGRU_OP_H].zero_point;
    linear(T * B, I, C, W, x_q, bw, p->op[QGRU_OP_X].zero_point, d.gemm_x, d.bias_w,
           &p->op[QGRU_OP_IH_LINEAR], ih, m_ih);
    for (int t = 0; t < T; ++t) {
        const int32_t *h_in = h_q + (size_t)t * NH;
        int32_t *h_out = h_q + (size_t)(t + 1) * NH;
        const int32_t *iht = ih + (size_t)t * B * C;
        linear(B, H, C, R, h_in, br, p->op[QGRU_OP_H].zero_point, d.gemm_h, d.bias_r,
               &p->op[QGRU_OP_HH_LINEAR], hh, m_hh ? m_hh + (size_t)t * B * C : NULL);
        for (int b = 0; b < B; ++b) {
            for (int j = 0; j < H; ++j) {
                const size_t w = (size_t)b * C + j;
                uint8_t ku[2], kr[2], kn[2], kh;
                const int32_t u = sigmoid_gate(iht[w], hh[w], p, d.ih_to_z, d.hh_to_z,
                                               QGRU_OP_UPDATE_IN, QGRU_OP_UPDATE_OUT, QGRU_LUT_UPDATE, ku);
                const int32_t r = sigmoid_gate(iht[w + H], hh[w + H], p, d.ih_to_r, d.hh_to_r,
                                               QGRU_OP_RESET_IN, QGRU_OP_RESET_OUT, QGRU_LUT_RESET, kr);
                const int32_t n = new_gate(iht[w + 2 * H], hh[w + 2 * H], r, p, &d, kn);
                h_out[(size_t)b * H + j] = hidden_state(u, n, h_in[(size_t)b * H + j], p, &d, &kh);
                const size_t mw = (size_t)t * B * C + w;
                if (m_gi) { m_gi[mw] = ku[0]; m_gi[mw + H] = kr[0]; m_gi[mw + 2 * H] = kn[0]; }
                if (m_go) { m_go[mw] = ku[1]; m_go[mw + H] = kr[1]; m_go[mw + 2 * H] = kn[1]; }
                if (m_h) m_h[((size_t)t * B + b) * H + j] = kh;
                if (v_q) {
                    int32_t *vb = v_q + ((size_t)t * B + b) * 4 * H + j;
                    vb[0] = u;
                    vb[H] = r;
                    vb[2 * H] = n;
                    vb[3 * H] = hh[w + 2 * H];
                }
            }
        }
    }
    free(ih);
    free(hh);
    free(d.gemm_x);
    return 0;
}

/* Batch-sliced, multi-threaded driver of orc_forward_i32 (rows of a batch are independent);
 * the all-cores "port" CPU baseline. */
typedef struct mt_job {
    int T, B, I, H, b0, b1;
    const int32_t *W, *R, *bw, *br, *x_q, *h0_q;
    const qgru_params *p;
    const float *sW, *sR, *sbw, *sbr;
    int32_t *h_q;
    int rc;
} mt_job;

static void *mt_worker(void *arg) {
    mt_job *j = (mt_job *)arg;
    const int Bs = j->b1 - j->b0;
    if (Bs <= 0) { j->rc = 0; return NULL; }
    int32_t *xs = (int32_t *)malloc(sizeof(int32_t) * (size_t)j->T * Bs * j->I);
    int32_t *hs = (int32_t *)malloc(sizeof(int32_t) * (size_t)(j->T + 1) * Bs * j->H);
    if (!xs || !hs) { free(xs); free(hs); j->rc = 1; return NULL; }
    for (int t = 0; t < j->T; ++t)
        memcpy(xs + (size_t)t * Bs * j->I, j->x_q + ((size_t)t * j->B + j->b0) * j->I,
               sizeof(int32_t) * (size_t)Bs * j->I);
    j->rc = orc_forward_i32(j->T, Bs, j->I, j->H, j->W, j->R, j->bw, j->br, xs,
                            j->h0_q ? j->h0_q + (size_t)j->b0 * j->H : NULL, j->p, j->sW, j->sR,
                            j->sbw, j->sbr, hs);
    for (int t = 0; t <= j->T; ++t)
        memcpy(j->h_q + ((size_t)t * j->B + j->b0) * j->H, hs + (size_t)t * Bs * j->H,
               sizeof(int32_t) * (size_t)Bs * j->H);
    free(xs);
    free(hs);
    return NULL;
}

ORC_API int orc_forward_i32_mt(int T, int B, int I, int H, const int32_t *W, const int32_t *R,
                               const int32_t *bw, const int32_t *br, const int32_t *x_q,
                               const int32_t *h0_q, const qgru_params *p, const float *sW,
                               const float *sR, const float *sbw, const float *sbr, int32_t *h_q,
                               int nthreads) {
    if (nthreads < 1) nthreads = 1;
    if (nthreads > B) nthreads = B;
    if (nthreads > 256) nthreads = 256;
    mt_job jobs[256];
    pthread_t th[256];
    for (int w = 0; w < nthreads; ++w) {
        mt_job *j = &jobs[w];
        j->T = T; j->B = B; j->I = I; j->H = H;
        j->b0 = (int)((int64_t)B * w / nthreads);
        j->b1 = (int)((int64_t)B * (w + 1) / nthreads);
        j->W = W; j->R = R; j->bw = bw; j->br = br; j->x_q = x_q; j->h0_q = h0_q;
        j->p = p; j->sW = sW; j->sR = sR; j->sbw = sbw; j->sbr = sbr; j->h_q = h_q; j->rc = 0;
        pthread_create(&th[w], NULL, mt_worker, j);
    }
    int rc = 0;
    for (int w = 0; w < nthreads; ++w) { pthread_join(th[w], NULL); rc |= jobs[w].rc; }
    return rc;
}

/* quantGRUForwardCPU, int32-weights overload, src/gru_interface.cc:796-867 (v == NULL). */
ORC_API int orc_forward_f32(int T, int B, int I, int H, const int32_t *W, const int32_t *R,
                            const int32_t *bw, const int32_t *br, const float *x, const float *h0,
                            const qgru_params *p, const float *sW, const float *sR,
                            const float *sbw, const float *sbr, float *h) {
    const size_t nx = (size_t)T * B * I, nh = (size_t)(T + 1) * B * H, NH = (size_t)B * H;
    int32_t *xq = (int32_t *)malloc(sizeof(int32_t) * nx);
    int32_t *hq = (int32_t *)malloc(sizeof(int32_t) * nh);
    int32_t *h0q = h0 ? (int32_t *)malloc(sizeof(int32_t) * NH) : NULL;
    int rc = orc_quantize(x, xq, nx, p, QGRU_OP_X);
    if (!rc && h0) rc = orc_quantize(h0, h0q, NH, p, QGRU_OP_H);
    if (!rc) rc = orc_forward_i32(T, B, I, H, W, R, bw, br, xq, h0q, p, sW, sR, sbw, sbr, hq);
    if (!rc) rc = orc_dequantize(hq, h, nh, p, QGRU_OP_H);
    free(xq);
    free(hq);
    free(h0q);
    return rc;
}

/* -------------------------------------------------- float forward + MinMax fold */

static void fold(float v, float *mn, float *mx) {
    if (isfinite(v)) { if (v < *mn) *mn = v; if (v > *mx) *mx = v; }
}

/* The fp32 GRU of src/gru_forward_gpu.cu:23-125 (inference; zoneout off) with the range
 * folding of updateGRUQuantizationRangesGPU (src/calibration_gpu.cu:1847-1953).  The
 * reference's GEMMs are cuBLAS SGEMMs whose summation order is unspecified; here dot
 * products are accumulated in double and rounded once, the most accurate fp32 answer, so
 * that any correct fp32 implementation lies within a few ulp.  `ranges` may be NULL (plain
 * float forward), `v` may be NULL; h is [(T+1),B,H]. */
ORC_API int orc_forward_float(int T, int B, int I, int H, const float *W, const float *R,
                              const float *bw, const float *br, const float *x, const float *h0,
                              float *h, float *v, qgru_ranges *ranges) {
    const int C = 3 * H;
    const size_t NH = (size_t)B * H;
    float *wx = (float *)malloc(sizeof(float) * (size_t)C);
    float *rh = (float *)malloc(sizeof(float) * (size_t)C);
    double *acc = (double *)malloc(sizeof(double) * (size_t)C);
    if (!wx || !rh || !acc) { free(wx); free(rh); free(acc); return 1; }
    for (size_t i = 0; i < NH; ++i) h[i] = h0 ? h0[i] : 0.0f;
    qgru_ranges *g = ranges;
    if (g) {
        for (size_t i = 0; i < (size_t)T * B * I; ++i) fold(x[i], &g->min_v[QGRU_OP_X], &g->max_v[QGRU_OP_X]);
        for (int c = 0; c < C; ++c) {
            for (int k = 0; k < I; ++k) fold(W[(size_t)k * C + c], &g->min_W[c], &g->max_W[c]);
            for (int k = 0; k < H; ++k) fold(R[(size_t)k * C + c], &g->min_R[c], &g->max_R[c]);
            fold(bw[c], &g->min_bw[c], &g->max_bw[c]);
            fold(br[c], &g->min_br[c], &g->max_br[c]);
        }
    }
    for (int t = 0; t < T; ++t) {
        const float *hin = h + (size_t)t * NH;
        float *hout = h + (size_t)(t + 1) * NH;
        for (int b = 0; b < B; ++b) {
            const float *xr = x + ((size_t)t * B + b) * I;
            for (int c = 0; c < C; ++c) acc[c] = 0.0;
            for (int k = 0; k < I; ++k) {
                const double xv = xr[k];
                const float *wr = W + (size_t)k * C;
                for (int c = 0; c < C; ++c) acc[c] += (double)wr[c] * xv;
            }
            for (int c = 0; c < C; ++c) wx[c] = (float)acc[c];
            for (int c = 0; c < C; ++c) acc[c] = 0.0;
            for (int k = 0; k < H; ++k) {
                const double hv = hin[(size_t)b * H + k];
                const float *rr = R + (size_t)k * C;
                for (int c = 0; c < C; ++c) acc[c] += (double)rr[c] * hv;
            }
            for (int c = 0; c < C; ++c) rh[c] = (float)acc[c];
            for (int j = 0; j < H; ++j) {
                const float wz = wx[j] + bw[j], rz = rh[j] + br[j];
                const float z_pre = wz + rz;
                const float z = 1.0f / (1.0f + expf(-z_pre));
                const float wr_ = wx[H + j] + bw[H + j], rr_ = rh[H + j] + br[H + j];
                const float r_pre = wr_ + rr_;
                const float r = 1.0f / (1.0f + expf(-r_pre));
                const float wg = wx[2 * H + j] + bw[2 * H + j], rg = rh[2 * H + j] + br[2 * H + j];
                const float g_pre = wg + r * rg;
                const float gg = tanhf(g_pre);
                const float h_old = hin[(size_t)b * H + j];
                const float old_c = z * h_old;
                const float new_c = (1.0f - z) * gg;
                const float hn = old_c + new_c;
                hout[(size_t)b * H + j] = hn;
                if (v) {
                    float *vb = v + ((size_t)t * B + b) * 4 * H + j;
                    vb[0] = z; vb[H] = r; vb[2 * H] = gg; vb[3 * H] = rg;
                }
                if (g) {
                    fold(hn, &g->min_v[QGRU_OP_H], &g->max_v[QGRU_OP_H]);
                    fold(wz, &g->min_v[QGRU_OP_IH_LINEAR], &g->max_v[QGRU_OP_IH_LINEAR]);
                    fold(wr_, &g->min_v[QGRU_OP_IH_LINEAR], &g->max_v[QGRU_OP_IH_LINEAR]);
                    fold(wg, &g->min_v[QGRU_OP_IH_LINEAR], &g->max_v[QGRU_OP_IH_LINEAR]);
                    fold(rz, &g->min_v[QGRU_OP_HH_LINEAR], &g->max_v[QGRU_OP_HH_LINEAR]);
                    fold(rr_, &g->min_v[QGRU_OP_HH_LINEAR], &g->max_v[QGRU_OP_HH_LINEAR]);
                    fold(rg, &g->min_v[QGRU_OP_HH_LINEAR], &g->max_v[QGRU_OP_HH_LINEAR]);
                    fold(z_pre, &g->min_v[QGRU_OP_UPDATE_IN], &g->max_v[QGRU_OP_UPDATE_IN]);
                    fold(r_pre, &g->min_v[QGRU_OP_RESET_IN], &g->max_v[QGRU_OP_RESET_IN]);
                    fold(g_pre, &g->min_v[QGRU_OP_NEW_IN], &g->max_v[QGRU_OP_NEW_IN]);
                    fold(z, &g->min_v[QGRU_OP_UPDATE_OUT], &g->max_v[QGRU_OP_UPDATE_OUT]);
                    fold(r, &g->min_v[QGRU_OP_RESET_OUT], &g->max_v[QGRU_OP_RESET_OUT]);
                    fold(gg, &g->min_v[QGRU_OP_NEW_OUT], &g->max_v[QGRU_OP_NEW_OUT]);
                    fold(r * rg, &g->min_v[QGRU_OP_MUL_RESET_HIDDEN], &g->max_v[QGRU_OP_MUL_RESET_HIDDEN]);
                    fold(new_c, &g->min_v[QGRU_OP_MUL_NEW_CONTRIB], &g->max_v[QGRU_OP_MUL_NEW_CONTRIB]);
                    fold(old_c, &g->min_v[QGRU_OP_MUL_OLD_CONTRIB], &g->max_v[QGRU_OP_MUL_OLD_CONTRIB]);
                }
            }
        }
    }
    free(wx);
    free(rh);
    free(acc);
    return 0;
}

/* ------------------------------------------------------- histogram calibration */

/* Histogram::bin_width, include/histogram_collector.h:76-79. */
static float hist_bw(float mn, float mx, int bins) {
    if (bins <= 0 || mx <= mn) return 1.0f;
    return (mx - mn) / bins;
}

/* Histogram::getPercentileRange, include/histogram_collector.h:105-165: cumulative sum in
 * single precision, first bins whose cumulative count reaches total*clip and total*(1-clip),
 * left bin edges. */
static void percentile_range(const float *counts, int bins, float mn, float mx, int64_t total,
                             float clip, float *pmin, float *pmax) {
    *pmin = mn;
    *pmax = mx;
    if (bins <= 0 || total <= 0 || clip <= 0.0f) return;
    float *cum = (float *)malloc(sizeof(float) * (size_t)bins);
    cum[0] = counts[0];
    for (int i = 1; i < bins; ++i) cum[i] = cum[i - 1] + counts[i];
    const float sum = cum[bins - 1];
    if (sum >= 1e-6f) {
        const float bw = hist_bw(mn, mx, bins);
        const float keep = 1.0f - clip;
        const float t_lo = sum * clip, t_hi = sum * keep;
        int i_lo = 0, i_hi = bins - 1;
        for (int i = 0; i < bins; ++i) if (cum[i] >= t_lo) { i_lo = i; break; }
        for (int i = 0; i < bins; ++i) if (cum[i] >= t_hi) { i_hi = i; break; }
        float a = mn + i_lo * bw, b = mn + i_hi * bw;
        if (b <= a) b = mx;
        *pmin = a;
        *pmax = b;
    }
    free(cum);
}

/* calibratePercentile, include/pot_sqnr_calibrator.h:99-186. */
static void continuous_percentile(const float *counts, int bins, float mn, float mx, int64_t total,
                                  int64_t steps, int sym, int uns, float percentile,
                                  float *scale_out, float *min_out) {
    const float ms = minimum_scale(steps);
    const float clip = (100.0f - percentile) / 100.0f;
    float pmin, pmax;
    percentile_range(counts, bins, mn, mx, total, clip, &pmin, &pmax);
    pmin = fminf(pmin, 0.0f);
    pmax = fmaxf(pmax, 0.0f);
    pmin = fmaxf(-FLT_MAX, fminf(pmin, 0.0f));
    pmax = fminf(FLT_MAX, fmaxf(pmax, 0.0f));
    if ((pmax - pmin) / (float)steps < ms) {
        if (sym && !uns) {
            pmin -= ms * (float)((steps + 1) / 2);
            pmax += ms * (float)(steps / 2);
        } else {
            pmax += ms * (float)steps;
        }
    }
    float scale, rmin;
    if (sym && uns) {
        const float dmax = fmaxf(pmax, ms);
        scale = fmaxf(dmax / (float)steps, ms);
        rmin = 0.0f;
    } else if (sym) {
        const int64_t pos = steps / 2, neg = (steps + 1) / 2;
        const float d_max = pos > 0 ? pmax / (float)pos : FLT_MAX;
        const float d_min = neg > 0 ? -pmin / (float)neg : FLT_MAX;
        scale = fmaxf(d_max, d_min);
        rmin = -(float)neg * scale;
    } else {
        scale = (pmax - pmin) / (float)steps;
        rmin = pmin;
    }
    *scale_out = fmaxf(scale, ms);
    *min_out = rmin;
}

/* sqnr_detail::estimateNoise, include/pot_sqnr_calibrator.h:210-238, gamma 3, p 2. */
static float sqnr_noise(const float *counts, int bins, float hmin, float bw, float delta,
                        float offset, int64_t steps) {
    if (delta <= 0) return FLT_MAX;
    float total = 0.0f;
    for (int i = 0; i < bins; ++i) {
        const float cnt = counts[i];
        if (cnt < 1e-6f) continue;
        const float x = hmin + (i + 0.5f) * bw;
        float q = rintf(x / delta - offset);
        const int clipped = (q < 0) || (q > (float)steps);
        q = fmaxf(0.0f, fminf((float)steps, q));
        const float xr = (q + offset) * delta;
        float err = powf(fabsf(xr - x), 2.0f);
        if (clipped) err *= 3.0f;
        total += err * cnt;
    }
    return total;
}

/* calibrateSqnr / searchSymmetric / searchAsymmetric, include/pot_sqnr_calibrator.h:246-381. */
static int continuous_sqnr(const float *counts, int bins, float hmin, float hmax, int64_t steps,
                           int sym, int uns, float *scale_out, float *min_out) {
    const float ms = minimum_scale(steps);
    const float bw = hist_bw(hmin, hmax, bins);
    const float vmin = fminf(hmin, 0.0f);
    float vmax = fmaxf(hmax, 0.0f);
    const float lim = vmin + ms * (float)steps;
    vmax = (vmax > lim) ? vmax : lim;
    float best = FLT_MAX, best_scale = 0.0f, best_min = 0.0f;
    if (sym) {
        float max_delta, offset;
        if (uns) { max_delta = vmax / (float)steps; offset = 0.0f; }
        else { max_delta = 2.0f * fmaxf(vmax, -vmin) / (float)steps; offset = -(float)((steps + 1) / 2); }
        max_delta = fmaxf(max_delta, ms);
        for (int d = 1; d <= 101; ++d) {
            float delta = max_delta * d / 100;
            delta = fmaxf(delta, ms);
            const float noise = sqnr_noise(counts, bins, hmin, bw, delta, offset, steps);
            if (noise < best) { best = noise; best_scale = delta; best_min = offset * delta; }
        }
    } else {
        const float max_delta = (vmax - vmin) / (float)steps;
        const float o_obs = rintf(vmin / max_delta);
        const float obs_min = max_delta * o_obs;
        const float obs_max = obs_min + max_delta * (float)steps;
        int n_off = (int)(steps + 2);
        if (n_off > 21) n_off = 21;
        float offs[21];
        const float step = (float)steps / (n_off - 2);
        for (int o = 0; o < n_off - 1; ++o) offs[o] = rintf(-(float)steps + o * step);
        offs[n_off - 1] = o_obs;
        for (int d = 1; d <= 17; ++d) {
            float delta = max_delta * d / 16;
            delta = fmaxf(delta, ms);
            for (int o = 0; o < n_off; ++o) {
                float tmin = delta * offs[o];
                float tmax = tmin + delta * (float)steps;
                tmin = fmaxf(obs_min, tmin);
                tmax = fminf(obs_max, tmax);
                float cd = (tmax - tmin) / (float)steps;
                cd = fmaxf(cd, ms);
                const float co = rintf(tmin / cd);
                const float noise = sqnr_noise(counts, bins, hmin, bw, cd, co, steps);
                if (noise < best) { best = noise; best_scale = cd; best_min = co * cd; }
            }
        }
    }
    if (best == FLT_MAX) return 1;
    *scale_out = best_scale;
    *min_out = best_min;
    return 0;
}

/* histCalibrate of calculateGRUQuantitativeParametersFromHistograms, src/gru_interface.cc:
 * 1092-1100: continuous scale from the histogram, then encodeScaleResult(coverage_round =
 * false) and storedScaleForMode. */
ORC_API int orc_calibrate_from_histogram(const float *counts, int bins, float min_val, float max_val,
                                         int64_t total, int use_pot2, int use_percentile,
                                         float percentile, qgru_op *op) {
    if (bins <= 0 || total <= 0) return 1;
    const int uns = eff_unsigned(op);
    const int64_t steps = (int64_t)qmax_of(op->bits, uns) - (int64_t)qmin_of(op->bits, uns);
    if (steps <= 0) return 1;
    float cs, cmin;
    if (use_percentile)
        continuous_percentile(counts, bins, min_val, max_val, total, steps, op->symmetric, uns, percentile, &cs, &cmin);
    else if (continuous_sqnr(counts, bins, min_val, max_val, steps, op->symmetric, uns, &cs, &cmin))
        return 1;
    return encode_scale(cs, cmin, op, op->symmetric, use_pot2, 0, &op->scale, &op->zero_point);
}

/* One histogram collector with the rules of GPUHistogramCollector::collect
 * (src/calibration_gpu.cu:820-876) and the arithmetic of its kernels (histogram_kernel_shared
 * :66-104, redistribute_histogram_kernel :116-158, build_histogram :499-522,
 * redistribute_histogram :524-540), evaluated one operation at a time except for the two
 * multiply-adds of the redistribution kernel, which nvcc fuses when it compiles the reference. */
typedef struct orc_hist {
    int bins;
    float *counts;
    float min_val, max_val;
    int64_t total;
    int valid;
    float limit_min, limit_max;
} orc_hist;

ORC_API orc_hist *orc_hist_new(int bins) {
    orc_hist *h = (orc_hist *)calloc(1, sizeof(orc_hist));
    h->bins = bins;
    h->counts = (float *)calloc((size_t)bins, sizeof(float));
    h->min_val = FLT_MAX;
    h->max_val = -FLT_MAX;
    return h;
}
ORC_API void orc_hist_free(orc_hist *h) {
    if (!h) return;
    free(h->counts);
    free(h);
}

static void hist_add(float *counts, int bins, const float *data, size_t n, float mn, float mx) {
    float bw = (mx - mn) / bins;
    if (bw < 1e-9f) bw = 1e-9f;
    const float inv = 1.0f / bw;
    for (size_t i = 0; i < n; ++i) {
        const float v = data[i];
        if (!isfinite(v)) continue;
        int b;
        if (v < mn) b = 0;
        else if (v > mx) b = bins - 1;
        else {
            b = (int)((v - mn) * inv);
            if (b > bins - 1) b = bins - 1;
        }
        counts[b] += 1.0f;
    }
}

static void hist_redistribute(const float *src, float smin, float sbw, float *dst, float dmin,
                              float dbw, int bins) {
    const float inv = 1.0f / dbw;
    for (int i = 0; i < bins; ++i) {
        const float cnt = src[i];
        if (cnt <= 0) continue;
        const float start = fmaf((float)i, sbw, smin);      /* as nvcc contracts the kernel's a + i * w */
        int d = (int)((start - dmin) * inv);
        if (d > bins - 1) d = bins - 1;
        const float end = fmaf(dbw, (float)(d + 1), dmin);
        const float split = rintf(((end - start) / sbw) * cnt);
        const float first = fminf(split, cnt);
        dst[d] += first;
        const float rest = cnt - first;
        if (rest > 0) {
            int o = (int)((start + dbw - dmin) * inv);
            if (o > bins - 1) o = bins - 1;
            dst[o] += rest;
        }
    }
}

ORC_API int orc_hist_collect(orc_hist *h, const float *data, size_t n) {
    if (n == 0) return 0;
    float dmin = FLT_MAX, dmax = -FLT_MAX;
    for (size_t i = 0; i < n; ++i)
        if (isfinite(data[i])) { dmin = fminf(dmin, data[i]); dmax = fmaxf(dmax, data[i]); }
    if (dmin > dmax) dmin = dmax = 0.0f;
    if (dmin == dmax) { dmin -= 0.5f; dmax += 0.5f; }
    const float eps = 1.19209290e-07f, v = 0.01f / (float)h->bins;
    const float tiny_range = (eps < v ? eps : v) * h->bins;
    float range = dmax - dmin;
    if (range < tiny_range || isnan(range) || isinf(range)) {
        dmin = fminf(dmin, 0.0f);
        dmax = fmaxf(dmax, 0.0f);
        range = tiny_range;
        dmax = dmin + tiny_range;
    }
    if (!h->valid) {
        memset(h->counts, 0, sizeof(float) * (size_t)h->bins);
        h->min_val = dmin;
        h->max_val = dmax;
        hist_add(h->counts, h->bins, data, n, dmin, dmax);
        h->total = (int64_t)n;
        h->valid = 1;
        h->limit_min = dmin - range * INFINITY / 2.0f;
        h->limit_max = dmax + range * INFINITY / 2.0f;
        return 0;
    }
    const float nmin = fmaxf(h->limit_min, fminf(dmin, h->min_val));
    const float nmax = fminf(h->limit_max, fmaxf(dmax, h->max_val));
    if (nmin == h->min_val && nmax == h->max_val) {
        hist_add(h->counts, h->bins, data, n, h->min_val, h->max_val);
    } else {
        float *fresh = (float *)calloc((size_t)h->bins, sizeof(float));
        const float sbw_check = hist_bw(h->min_val, h->max_val, h->bins);
        if (fabsf(sbw_check) >= (eps < v ? eps : v) && !isnan(sbw_check) && !isinf(sbw_check)) {
            const float sbw = (h->max_val - h->min_val) / h->bins;
            float dbw = (nmax - nmin) / h->bins;
            if (dbw < 1e-9f) dbw = 1e-9f;
            hist_redistribute(h->counts, h->min_val, sbw, fresh, nmin, dbw, h->bins);
        }
        hist_add(fresh, h->bins, data, n, nmin, nmax);
        free(h->counts);
        h->counts = fresh;
        h->min_val = nmin;
        h->max_val = nmax;
    }
    h->total += (int64_t)n;
    return 0;
}

ORC_API int orc_hist_get(const orc_hist *h, float *counts, float *min_val, float *max_val, int64_t *total) {
    if (counts) memcpy(counts, h->counts, sizeof(float) * (size_t)h->bins);
    *min_val = h->min_val;
    *max_val = h->max_val;
    *total = h->valid ? h->total : 0;
    return 0;
}

/* ------------------------------------------- float-storage quantized forward (inference) */

static float fs_clampf(float v, const qgru_op *o) {
    const float lo = (float)qmin_of(o->bits, eff_unsigned(o)), hi = (float)qmax_of(o->bits, eff_unsigned(o));
    return fmaxf(lo, fminf(v, hi));   /* clamp_f, include/quantize_ops_helper.h:416-431 */
}
/* quantize_f(src, FixedPointScale, zp, bw), include/quantize_ops_helper.h:514-519: the zero
 * point is added BEFORE the rounding, unlike quantize() of the integer path. */
static float fs_quantize(float x, float scale, int32_t zp, const qgru_op *o) {
    return fs_clampf(rintf(x / scale + (float)zp), o);
}
/* biasRescaleInline, src/gru_forward_gpu_quant_fp.cu:117-142. */
static float fs_linear(float gemm, float wsum_zp, float bias, float inv_bias, float inv_gemm,
                       const qgru_op *out) {
    const float val = gemm - wsum_zp;
    const float bias_term = rintf(bias * inv_bias);
    const float combined = val + bias_term;
    return fs_clampf(rintf(combined * inv_gemm) + (float)out->zero_point, out);
}
/* real_sigmoid_f / real_tanh_f, include/quantize_ops_helper.h:687-720. */
static float fs_act(float q_x, const qgru_op *in, const qgru_op *out, int is_tanh) {
    const float x = (q_x - (float)in->zero_point) * in->scale;
    const float y = is_tanh ? tanhf(x) : 1.0f / (1.0f + expf(-x));
    return fs_clampf(rintf(y / out->scale + (float)out->zero_point), out);
}

/* quantGRUForwardFP, inference mode (src/gru_interface.cc:894-995; ForwardPassQuantFP and
 * PointwiseOperationsFP, src/gru_forward_gpu_quant_fp.cu:572-770, 821-1003, 1177-1232): quantized
 * values held as floats, float requantization, real sigmoid / tanh.  W..br are the quantized
 * weights (the values quantizeGRUWeights produces are those of the integer path).  The
 * reference's two products are fp32 SGEMMs over integer-valued operands; they are evaluated here
 * as exact integer sums converted to float, which is what an fp32 sum gives below 2^24.  expf
 * and tanhf are the host's, the reference's are CUDA's: a gate output can differ by one step
 * where the two libraries round a value across a .5 boundary.
 * h [(T+1),B,H] dequantized; x_q_out [T,B,I] (quantized x as floats) may be NULL. */
ORC_API int orc_forward_fstorage(int T, int B, int I, int H, const int32_t *W, const int32_t *R,
                                 const int32_t *bw, const int32_t *br, const float *x, const float *h0,
                                 const qgru_params *p, const float *sW, const float *sR,
                                 const float *sbw, const float *sbr, float *h, float *x_q_out) {
    if (p->hidden != H) return 1;
    const int C = 3 * H, pot2 = p->use_pot2 != 0;
    const size_t NH = (size_t)B * H;
    const qgru_op *ox = &p->op[QGRU_OP_X], *oh = &p->op[QGRU_OP_H];
    const qgru_op *oih = &p->op[QGRU_OP_IH_LINEAR], *ohh = &p->op[QGRU_OP_HH_LINEAR];
    const qgru_op *ozi = &p->op[QGRU_OP_UPDATE_IN], *ozo = &p->op[QGRU_OP_UPDATE_OUT];
    const qgru_op *ori = &p->op[QGRU_OP_RESET_IN], *oro = &p->op[QGRU_OP_RESET_OUT];
    const qgru_op *oni = &p->op[QGRU_OP_NEW_IN], *ono = &p->op[QGRU_OP_NEW_OUT];
    uint16_t m;
    int8_t s;
    if (to_fixed_scale(ox->scale, pot2, &m, &s)) return 1;
    const float x_scale = decode_scale(m, s);
    if (to_fixed_scale(oh->scale, pot2, &m, &s)) return 1;
    const float h_scale = decode_scale(m, s);
    /* setRescaleParam, src/gru_forward_gpu_quant_fp.cu:821-1003: ratios of the stored scales */
    const float ih_to_z = oih->scale / ozi->scale, hh_to_z = ohh->scale / ozi->scale;
    const float ih_to_r = oih->scale / ori->scale, hh_to_r = ohh->scale / ori->scale;
    const float ih_to_n = oih->scale / oni->scale;
    const float rh_to_n = (oro->scale * ohh->scale) / oni->scale;
    const float one_q = rintf(1.0f / ozo->scale) + (float)ozo->zero_point;
    const float uh_to_h = (ozo->scale * oh->scale) / oh->scale;
    const float n_to_h = ono->scale / oh->scale;
    const float zp_x = (float)ox->zero_point, zp_h = (float)oh->zero_point;
    const float zp_ih = (float)oih->zero_point, zp_hh = (float)ohh->zero_point;

    float *cst = (float *)malloc(sizeof(float) * 6 * (size_t)C);
    float *xq = (float *)malloc(sizeof(float) * (size_t)T * B * I);
    float *hq = (float *)malloc(sizeof(float) * 2 * NH);
    float *ih = (float *)malloc(sizeof(float) * (size_t)C), *hh = (float *)malloc(sizeof(float) * (size_t)C);
    int64_t *acc = (int64_t *)malloc(sizeof(int64_t) * (size_t)C);
    if (!cst || !xq || !hq || !ih || !hh || !acc) { free(cst); free(xq); free(hq); free(ih); free(hh); free(acc); return 1; }
    float *inv_gx = cst, *inv_bw = cst + C, *inv_gh = cst + 2 * C, *inv_br = cst + 3 * C;
    float *wsx = cst + 4 * C, *wsh = cst + 5 * C;
    for (int c = 0; c < C; ++c) {
        const float s_wx = sW[c] * ox->scale, s_rh = sR[c] * oh->scale;
        inv_gx[c] = s_wx / oih->scale;
        inv_bw[c] = sbw[c] / s_wx;
        inv_gh[c] = s_rh / ohh->scale;
        inv_br[c] = sbr[c] / s_rh;
        /* computeWeightSumKernel, :442-458: float sum of the column, times the zero point */
        float sum = 0.0f;
        for (int k = 0; k < I; ++k) sum += (float)W[(size_t)k * C + c];
        wsx[c] = ox->zero_point != 0 ? sum * zp_x : 0.0f;
        sum = 0.0f;
        for (int k = 0; k < H; ++k) sum += (float)R[(size_t)k * C + c];
        wsh[c] = oh->zero_point != 0 ? sum * zp_h : 0.0f;
    }
    for (size_t i = 0; i < (size_t)T * B * I; ++i) {
        xq[i] = fs_quantize(x[i], x_scale, ox->zero_point, ox);
        if (x_q_out) x_q_out[i] = xq[i];
    }
    float *cur = hq, *nxt = hq + NH;
    for (size_t i = 0; i < NH; ++i) {
        cur[i] = h0 ? fs_quantize(h0[i], h_scale, oh->zero_point, oh) : zp_h;
        h[i] = (cur[i] - zp_h) * h_scale;
    }
    for (int t = 0; t < T; ++t) {
        for (int b = 0; b < B; ++b) {
            const float *xr = xq + ((size_t)t * B + b) * I, *hr = cur + (size_t)b * H;
            for (int c = 0; c < C; ++c) acc[c] = 0;
            for (int k = 0; k < I; ++k) {
                const int64_t xv = (int64_t)xr[k];
                const int32_t *wr = W + (size_t)k * C;
                for (int c = 0; c < C; ++c) acc[c] += (int64_t)wr[c] * xv;
            }
            for (int c = 0; c < C; ++c)
                ih[c] = fs_linear((float)acc[c], wsx[c], (float)bw[c], inv_bw[c], inv_gx[c], oih);
            for (int c = 0; c < C; ++c) acc[c] = 0;
            for (int k = 0; k < H; ++k) {
                const int64_t hv = (int64_t)hr[k];
                const int32_t *rr = R + (size_t)k * C;
                for (int c = 0; c < C; ++c) acc[c] += (int64_t)rr[c] * hv;
            }
            for (int c = 0; c < C; ++c)
                hh[c] = fs_linear((float)acc[c], wsh[c], (float)br[c], inv_br[c], inv_gh[c], ohh);
            for (int j = 0; j < H; ++j) {
                /* computeUpdateGateFP / computeResetGateFP, :153-239 */
                float a = rintf((ih[j] - zp_ih) * ih_to_z), c2 = rintf((hh[j] - zp_hh) * hh_to_z);
                const float u = fs_act(fs_clampf(a + c2 + (float)ozi->zero_point, ozi), ozi, ozo, 0);
                a = rintf((ih[j + H] - zp_ih) * ih_to_r);
                c2 = rintf((hh[j + H] - zp_hh) * hh_to_r);
                const float r = fs_act(fs_clampf(a + c2 + (float)ori->zero_point, ori), ori, oro, 0);
                /* computeNewGateFP, :241-290 */
                const float rh = rintf(((r - (float)oro->zero_point) * (hh[j + 2 * H] - zp_hh)) * rh_to_n);
                a = rintf((ih[j + 2 * H] - zp_ih) * ih_to_n);
                const float n = fs_act(fs_clampf(a + rh + (float)oni->zero_point, oni), oni, ono, 1);
                /* computeHiddenStateFP, :302-372 */
                const float n_h = rintf((n - (float)ono->zero_point) * n_to_h) + zp_h;
                const float old_c = (u - (float)ozo->zero_point) * (hr[j] - zp_h);
                const float new_c = ((one_q - u) - (float)ozo->zero_point) * (n_h - zp_h);
                const float hn = fs_clampf(rintf((old_c + new_c) * uh_to_h) + zp_h, oh);
                nxt[(size_t)b * H + j] = hn;
                h[(size_t)(t + 1) * NH + (size_t)b * H + j] = (hn - zp_h) * h_scale;
            }
        }
        float *tmp = cur; cur = nxt; nxt = tmp;
    }
    free(cst); free(xq); free(hq); free(ih); free(hh); free(acc);
    return 0;
}
