// qgru_internal.h - declarations shared by the host set-up code and the CUDA translation
// units of libqgru_b200.  Nothing here is part of the public ABI (include/qgru.h).
#pragma once
#include <stdint.h>

#include <string>

#include "qgru.h"
#include "qgru_math.h"

namespace qgru {

// ---- host helpers implemented in qgru_host.cc
bool encode_mshift(float scale, Rescale *out);
int pot2_shift(float scale);
bool to_fixed_scale(float scale, bool pot2, Rescale *out);
float decode_scale(Rescale r);
bool make_rescale(float src, float dst, bool pot2, Rescale *out);
bool make_rescale_product(float a, float b, float dst, bool pot2, Rescale *out);
bool make_rescale_to_product(float src, float a, float b, bool pot2, Rescale *out);
// one histogram -> op->scale / op->zero_point by Percentile or SQNR (qgru_host.cc)
int calibrate_histogram_op(const float *counts, int bins, float min_val, float max_val, long long total,
                           bool pot2, bool use_percentile, float percentile, qgru_op *op);
int32_t op_qmin(const qgru_op &o);
int32_t op_qmax(const qgru_op &o);
int32_t lut_eval(const qgru_lut &lut, int32_t q_x, const qgru_op &in_bw, const qgru_op &out_bw);

// ---- device-visible constants of the gate datapath: the scalar part of
// GateQuantParamsT<R> (include/quantize_param_types.h:148-193), derived once per
// set_params instead of being passed by value (968 bytes) on every launch.
enum { ACT_Z = 0, ACT_R = 1, ACT_N = 2 };

struct GateConsts {
    int32_t zp_ih, zp_hh, zp_h;
    int32_t zp_in[3], zp_out[3];          // gate input / output zero points (z, r, n)
    int32_t one_q;                        // round(1/s_z) + zp_z
    Rescale ih_to[3];                     // weight_ih_linear -> gate input (z, r, n)
    Rescale hh_to[2];                     // weight_hh_linear -> gate input (z, r)
    Rescale rh_to_n;                      // (r - zp)(hh_n - zp) -> new gate input
    Rescale n_to_h;                       // new gate output -> h
    Rescale uh_to_h;                      // s_z * s_h -> h
    int32_t in_lo[3], in_hi[3], out_lo[3], out_hi[3];
    int32_t h_lo, h_hi, ih_lo, ih_hi, hh_lo, hh_hi;
    int32_t table_size[3];                // > 0: direct table over the clamped input range
    int32_t table_off[3];                 // offset of that table in the table array (ints)
    int32_t narrow;                       // 1: every gate rescale fits the 32-bit fast form
    float h_scale;                        // decode_scale(toFixedScale(h)) for the float output
    // "fused" form of the cell used by the tensor-core recurrence when every gate input and
    // the R*h+br output are narrow enough to tabulate (see build_fused_tables in qgru_api.cu)
    int32_t fused_ok;
    int32_t k1;                           // one_q - 2*zp_z : (1 - z) numerator minus z_d
    int32_t ft_off[5];                    // offsets of TZ, TR, TN, THZ, THR in the fused table block
    int32_t ih_pre_bytes;                 // storage width (2 or 4) of the pre-rescaled W*x+bw values
    int32_t ft_ih_off, ft_ih_n;           // table of the GEMM-side pre-rescale in the same block (n per gate, 0: none)
    // Index arithmetic of the five fused-cell lookups with the zero points, the clamp and the
    // table offset folded: entry = table[min(max(v + fi_c[k], fi_lo[k]), fi_hi[k])], k = TZ, TR,
    // TN (v = gate input before its clamp) or THZ, THR (v = requantized R*h row before its zero
    // point).  hn_clo/hn_chi clamp the new gate's R*h row in the same zero-point-free domain.
    int32_t fi_c[5], fi_lo[5], fi_hi[5];
    int32_t hn_clo, hn_chi;
    int32_t cell_notie;                   // 1: neither rescale of the fused cell can meet an exact tie (rescale_can_tie)
    qgru_lut lut[3];
};

// What the input-projection GEMM applies after the requantization when the recurrence runs the
// fused cell: out = rescale(ih - zp_ih -> gate input scale of the channel's gate) + zp_in[gate].
struct PreScale {
    int32_t enabled, H, zp_ih;
    Rescale to[3];
    int32_t zp_in[3];
    // optional table of that function over the clamped W*x+bw range (gate-major, n entries per
    // gate, index = value - lo); null when the range is too wide to tabulate
    const int32_t *table;
    int32_t table_n, lo;
};

// GateQuantParamsFP + the scalar part of LinearRescaleParamsFP
// (ForwardPassQuantFP::setRescaleParam, src/gru_forward_gpu_quant_fp.cu:821-1003).
struct FsConsts {
    float zp_x, zp_h, zp_ih, zp_hh;
    float zp_in[3], zp_out[3];      // gate inputs / outputs: z, r, n
    float s_in[3], s_out[3];
    float ih_to[3];                 // weight_ih_linear -> gate input
    float hh_to[2];                 // weight_hh_linear -> z, r input
    float rh_to_n;                  // (r * hh_n) -> new gate input
    float n_to_h, uh_to_h, one_q;
    float ih_lo, ih_hi, hh_lo, hh_hi, h_lo, h_hi;
    float in_lo[3], in_hi[3], out_lo[3], out_hi[3];
    float h_scale;                  // decoded scale of h, for the dequantized output
    int h_bits;                     // 8: signed state bytes, 9: unsigned
    // Gate outputs tabulated over the clamped gate input (built on the device by the very code
    // that evaluates a gate directly): entry tab_off[g] + (input - in_lo[g]) of a float table the
    // kernel holds in shared memory.  tab_on = 0: evaluate sigmoid / tanh per cell.
    int tab_on;
    int tab_off[3];
};

// Per output channel constants of one fused linear layer:
//   out = clamp( int32( rescale( acc + corr[m], rs[m] ) ) + zp_out )
// with corr[m] = rescale(bias_q[m], bias_rs[m]) - zp_in * sum_k W_q[k][m]
// (src/gru_forward_cpu_quant.cc:92-99,125-138).
struct LinearConsts {
    const int64_t *corr;  // [3H] device
    const Rescale *rs;    // [3H] device
    const FastLin *fl;    // [3H] device: rs and corr in the folded shift-free form (mq == 0: none)
    int32_t zp_out, lo, hi;
    int32_t fits32;       // 1: acc + corr fits int32 for every channel (one widening multiply)
    // float-storage forward: [3][fs_C] floats (offset, bias term, scale ratio per channel); when
    // set, the epilogue is the reference's float requantization instead of the integer one
    const float *fs = nullptr;
    int32_t fs_C = 0;
};

}  // namespace qgru
