// qgru_device.cuh - __device__ building blocks shared by every kernel file: dp4a wrappers,
// the gate datapath and the fused-linear epilogue.  Only inline device functions live here,
// so any translation unit may include it.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "qgru_internal.h"

namespace qgru {

// ------------------------------------------------------------------ small helpers

__device__ __forceinline__ int dp4a_ss(int a, int b, int c) { return __dp4a(a, b, c); }
// a: four signed bytes, b: four unsigned bytes
__device__ __forceinline__ int dp4a_su(int a, unsigned b, int c) {
    int d;
    asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
template <bool BUnsigned>
__device__ __forceinline__ int dp4a_w(int w, unsigned act, int c) {
    if constexpr (BUnsigned) return dp4a_su(w, act, c);
    else return dp4a_ss(w, (int)act, c);
}

__device__ __forceinline__ unsigned ld_acquire(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Predicated global load of one W*x+bw value, widened to 32 bits by the load itself; 0 where `ok`
// is false.  One instruction with no dependent select behind it, so a warp that prefetches its
// operands keeps issuing while they are in flight.
__device__ __forceinline__ int32_t ld_ih_pred(const int8_t *p, bool ok) {
    int32_t v;
    asm volatile("{\n.reg .pred q;\nsetp.ne.b32 q, %2, 0;\nmov.b32 %0, 0;\n@q ld.global.s8 %0, [%1];\n}"
                 : "=r"(v) : "l"(p), "r"((int)ok));
    return v;
}
__device__ __forceinline__ int32_t ld_ih_pred(const int16_t *p, bool ok) {
    int32_t v;
    asm volatile("{\n.reg .pred q;\nsetp.ne.b32 q, %2, 0;\nmov.b32 %0, 0;\n@q ld.global.s16 %0, [%1];\n}"
                 : "=r"(v) : "l"(p), "r"((int)ok));
    return v;
}
__device__ __forceinline__ int32_t ld_ih_pred(const int32_t *p, bool ok) {
    int32_t v;
    asm volatile("{\n.reg .pred q;\nsetp.ne.b32 q, %2, 0;\nmov.b32 %0, 0;\n@q ld.global.s32 %0, [%1];\n}"
                 : "=r"(v) : "l"(p), "r"((int)ok));
    return v;
}

// ------------------------------------------------------------ gate datapath (a4-a8)

// piecewise_linear with its two clamps (include/quantize_ops_helper.h:600-606).  Where the
// gate input is narrow enough the host tabulated the function over the whole clamped input
// range; the table holds exactly the values the segment evaluation produces.
__device__ __forceinline__ int32_t activation(const GateConsts &gc, const int32_t *tables,
                                              int which, int32_t pre) {
    const int32_t q = clampi(pre, gc.in_lo[which], gc.in_hi[which]);
    if (gc.table_size[which] > 0) return tables[gc.table_off[which] + (q - gc.in_lo[which])];
    return clampi(lut_raw(gc.lut[which], q), gc.out_lo[which], gc.out_hi[which]);
}

template <bool Narrow>
__device__ __forceinline__ int32_t rescale_diff(int32_t v, int32_t zp, Rescale r) {
    if constexpr (Narrow) return rescale_narrow(v - zp, r);
    else return (int32_t)rescale64((int64_t)v - (int64_t)zp, r);
}

// computeUpdateGate / computeResetGate / computeNewGate / computeHiddenState, inference
// branch (include/quantize_ops_helper.h:749-1084).  ih_* and hh_* are the clamped outputs of
// the two fused linear layers; h_old is the quantized previous state.
// gates: optional [3] out, the quantized update, reset and new gate outputs (the reference's
// training buffer v, src/gru_forward_gpu_quant.cu:318-330).
template <bool Narrow>
__device__ __forceinline__ int32_t gru_cell(const GateConsts &gc, const int32_t *tables,
                                            int32_t ih_z, int32_t ih_r, int32_t ih_n,
                                            int32_t hh_z, int32_t hh_r, int32_t hh_n,
                                            int32_t h_old, int32_t *gates = nullptr) {
    const int32_t z_pre = rescale_diff<Narrow>(ih_z, gc.zp_ih, gc.ih_to[ACT_Z]) +
                          rescale_diff<Narrow>(hh_z, gc.zp_hh, gc.hh_to[ACT_Z]) + gc.zp_in[ACT_Z];
    const int32_t z = activation(gc, tables, ACT_Z, z_pre);
    const int32_t r_pre = rescale_diff<Narrow>(ih_r, gc.zp_ih, gc.ih_to[ACT_R]) +
                          rescale_diff<Narrow>(hh_r, gc.zp_hh, gc.hh_to[ACT_R]) + gc.zp_in[ACT_R];
    const int32_t r = activation(gc, tables, ACT_R, r_pre);

    const int64_t r_hh = ((int64_t)r - gc.zp_out[ACT_R]) * ((int64_t)hh_n - gc.zp_hh);
    const int32_t n_pre = rescale_diff<Narrow>(ih_n, gc.zp_ih, gc.ih_to[ACT_N]) +
                          (int32_t)rescale64(r_hh, gc.rh_to_n) + gc.zp_in[ACT_N];
    const int32_t n = activation(gc, tables, ACT_N, n_pre);

    const int32_t n_h = rescale_diff<Narrow>(n, gc.zp_out[ACT_N], gc.n_to_h) + gc.zp_h;
    const int64_t z_d = (int64_t)z - gc.zp_out[ACT_Z];
    const int64_t old_c = z_d * ((int64_t)h_old - gc.zp_h);
    const int64_t one_minus = ((int64_t)gc.one_q - z) - gc.zp_out[ACT_Z];
    const int64_t new_c = one_minus * ((int64_t)n_h - gc.zp_h);
    const int32_t h_new = (int32_t)rescale64(old_c + new_c, gc.uh_to_h) + gc.zp_h;
    if (gates) {
        gates[0] = z;
        gates[1] = r;
        gates[2] = n;
    }
    return clampi(h_new, gc.h_lo, gc.h_hi);
}

// piecewise_linear in the training branch (include/quantize_ops_helper.h:760-783): always the
// segment evaluation, and the two clamp flags (1 = inside the range) are kept.
__device__ __forceinline__ int32_t activation_keep(const GateConsts &gc, int which, int32_t pre,
                                                   uint8_t &keep_in, uint8_t &keep_out) {
    const int32_t q = clampi(pre, gc.in_lo[which], gc.in_hi[which]);
    keep_in = q == pre;
    const int32_t raw = lut_raw(gc.lut[which], q);
    const int32_t out = clampi(raw, gc.out_lo[which], gc.out_hi[which]);
    keep_out = out == raw;
    return out;
}

// gru_cell in training mode: the gate outputs and the seven clamp flags of one cell
// (src/gru_forward_gpu_quant.cu:296-348).  keep[0..2] gate inputs z, r, n; keep[3..5] gate
// outputs; keep[6] the new state.
__device__ __forceinline__ int32_t gru_cell_train(const GateConsts &gc, int32_t ih_z, int32_t ih_r,
                                                  int32_t ih_n, int32_t hh_z, int32_t hh_r, int32_t hh_n,
                                                  int32_t h_old, int32_t *gates, uint8_t *keep) {
    const int32_t z_pre = rescale_diff<false>(ih_z, gc.zp_ih, gc.ih_to[ACT_Z]) +
                          rescale_diff<false>(hh_z, gc.zp_hh, gc.hh_to[ACT_Z]) + gc.zp_in[ACT_Z];
    const int32_t z = activation_keep(gc, ACT_Z, z_pre, keep[0], keep[3]);
    const int32_t r_pre = rescale_diff<false>(ih_r, gc.zp_ih, gc.ih_to[ACT_R]) +
                          rescale_diff<false>(hh_r, gc.zp_hh, gc.hh_to[ACT_R]) + gc.zp_in[ACT_R];
    const int32_t r = activation_keep(gc, ACT_R, r_pre, keep[1], keep[4]);
    const int64_t r_hh = ((int64_t)r - gc.zp_out[ACT_R]) * ((int64_t)hh_n - gc.zp_hh);
    const int32_t n_pre = rescale_diff<false>(ih_n, gc.zp_ih, gc.ih_to[ACT_N]) +
                          (int32_t)rescale64(r_hh, gc.rh_to_n) + gc.zp_in[ACT_N];
    const int32_t n = activation_keep(gc, ACT_N, n_pre, keep[2], keep[5]);
    const int32_t n_h = rescale_diff<false>(n, gc.zp_out[ACT_N], gc.n_to_h) + gc.zp_h;
    const int64_t z_d = (int64_t)z - gc.zp_out[ACT_Z];
    const int64_t old_c = z_d * ((int64_t)h_old - gc.zp_h);
    const int64_t one_minus = ((int64_t)gc.one_q - z) - gc.zp_out[ACT_Z];
    const int64_t new_c = one_minus * ((int64_t)n_h - gc.zp_h);
    const int32_t h_new = (int32_t)rescale64(old_c + new_c, gc.uh_to_h) + gc.zp_h;
    gates[0] = z;
    gates[1] = r;
    gates[2] = n;
    const int32_t h_c = clampi(h_new, gc.h_lo, gc.h_hi);
    keep[6] = h_c == h_new;
    return h_c;
}

// The same cell with everything that depends on one narrow operand tabulated on the host:
//   a_*   W*x+bw already rescaled to the gate's input scale, zp_in included (GEMM epilogue)
//   THZ/THR[hh - hh_lo]      = rescale(hh - zp_hh -> z / r input scale)
//   TZ/TR[clamp(pre) - lo]   = sigmoid LUT output minus its zero point
//   TN[clamp(pre) - lo]      = rescale(tanh LUT output - zp_n -> h scale)
// Each table entry is produced by the very functions above, so the result is identical; the
// host checks that the two products below fit 32 bits before enabling this form.
__device__ __forceinline__ int32_t gru_cell_fused(const GateConsts &gc, const int32_t *ft, int32_t a_z,
                                                  int32_t a_r, int32_t a_n, int32_t hh_z, int32_t hh_r,
                                                  int32_t hh_n, int32_t h_old) {
    const int32_t z_pre = a_z + ft[gc.ft_off[3] + (hh_z - gc.hh_lo)];
    const int32_t z_d = ft[gc.ft_off[0] + (clampi(z_pre, gc.in_lo[ACT_Z], gc.in_hi[ACT_Z]) - gc.in_lo[ACT_Z])];
    const int32_t r_pre = a_r + ft[gc.ft_off[4] + (hh_r - gc.hh_lo)];
    const int32_t r_d = ft[gc.ft_off[1] + (clampi(r_pre, gc.in_lo[ACT_R], gc.in_hi[ACT_R]) - gc.in_lo[ACT_R])];
    const int32_t n_pre = a_n + (int32_t)rescale32(r_d * (hh_n - gc.zp_hh), gc.rh_to_n);
    const int32_t n_d = ft[gc.ft_off[2] + (clampi(n_pre, gc.in_lo[ACT_N], gc.in_hi[ACT_N]) - gc.in_lo[ACT_N])];
    const int32_t comb = z_d * (h_old - gc.zp_h) + (gc.k1 - z_d) * n_d;
    return clampi((int32_t)rescale32(comb, gc.uh_to_h) + gc.zp_h, gc.h_lo, gc.h_hi);
}

// 32-bit load from a shared-memory window address: table lookups stay on the shared-memory
// path with 32-bit address arithmetic.
__device__ __forceinline__ int32_t lds_i32(uint32_t addr) {
    int32_t v;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
// Sign- or zero-extend a state byte held in the low bits of x: bits = 8 for int8 storage, 9 for
// uint8 (bit 8 is zero, so the value stays non-negative).
__device__ __forceinline__ int32_t state_byte(uint32_t x, uint32_t bits) {
    int32_t d;
    asm("bfe.s32 %0, %1, 0, %2;" : "=r"(d) : "r"(x), "r"(bits));
    return d;
}

// gru_cell_fused for scales that all have the shift-free form (Rescale::mq != 0, checked on the
// host): no branch anywhere, so the compiler can interleave the dependency chains of several
// cells, which is what hides the table-lookup latency at four warps per scheduler.  Zero
// points, clamps and table offsets are folded into one add and one max/min pair per lookup
// (GateConsts::fi_*).  In three pieces, so that a kernel can start on the update and reset
// gates while the tensor core still works on the rows of the new gate.  `tab` is the
// shared-window address of the fused table block, `q` a requantized R*h row before its zero
// point (lin_round).
__device__ __forceinline__ int32_t ft_lookup(const GateConsts &gc, uint32_t tab, int k, int32_t v) {
    const int32_t idx = min(max(v + gc.fi_c[k], gc.fi_lo[k]), gc.fi_hi[k]);
    return lds_i32(tab + 4u * (uint32_t)idx);
}
//   which = ACT_Z / ACT_R: sigmoid LUT output minus its zero point
__device__ __forceinline__ int32_t fused_gate_fast(const GateConsts &gc, uint32_t tab, int which, int32_t a_pre,
                                                   int32_t q) {
    return ft_lookup(gc, tab, which, a_pre + ft_lookup(gc, tab, 3 + which, q));
}
template <bool Tie = true>
__device__ __forceinline__ int32_t fused_finish_fast(const GateConsts &gc, uint32_t tab, int32_t a_n, int32_t q_n,
                                                     int32_t z_d, int32_t r_d, int32_t h_old) {
    const int32_t hh_nd = min(max(q_n, gc.hn_clo), gc.hn_chi);        // R*h row of the new gate minus zp
    const int32_t n_d = ft_lookup(gc, tab, ACT_N, a_n + mul_round_hi<Tie>(r_d * hh_nd, gc.rh_to_n));
    const int32_t comb = z_d * (h_old - gc.zp_h) + (gc.k1 - z_d) * n_d;
    return min(max(mul_round_hi<Tie>(comb, gc.uh_to_h) + gc.zp_h, gc.h_lo), gc.h_hi);
}

// Epilogue of a fused linear layer (src/gru_forward_cpu_quant.cc:130-138).
__device__ __forceinline__ int32_t linear_epilogue(int64_t acc, int64_t corr, Rescale rs,
                                                   int32_t zp_out, int32_t lo, int32_t hi,
                                                   uint8_t *keep = nullptr) {
    const int32_t v = (int32_t)rescale64(acc + corr, rs) + zp_out;
    const int32_t c = clampi(v, lo, hi);
    if (keep) *keep = c == v;
    return c;
}
// The same when acc + corr is known to fit int32 (LinearConsts::fits32).
__device__ __forceinline__ int32_t linear_epilogue32(int32_t acc, int32_t corr, Rescale rs,
                                                     int32_t zp_out, int32_t lo, int32_t hi) {
    const int32_t v = (int32_t)rescale32(acc + corr, rs) + zp_out;
    return clampi(v, lo, hi);
}

// ---- float-storage forward (the reference's quantGRUForwardFP): float requantization
__device__ __forceinline__ float fs_clamp(float v, float lo, float hi) { return fmaxf(lo, fminf(v, hi)); }

// biasRescaleInline (src/gru_forward_gpu_quant_fp.cu:117-142).  acc is the exact integer
// sum_k W*x; off = float(sum_k W) * zp_in as computeWeightSumKernel leaves it (:442-458, one
// rounded product); bias_term = round(bias * inv_bias).  Sub, add and multiply are kept as
// separate roundings, as in the reference's compiled kernel (none of them is an a*b+c there).
__device__ __forceinline__ float fs_linear(int acc, float off, float bias_term, float inv_gemm,
                                           float zp_out, float lo, float hi) {
    const float val = __fsub_rn((float)acc, off);
    const float combined = __fadd_rn(val, bias_term);
    return fs_clamp(rintf(__fmul_rn(combined, inv_gemm)) + zp_out, lo, hi);
}
__device__ __forceinline__ float fs_offset(int wsum, float zp_in) { return __fmul_rn((float)wsum, zp_in); }
__device__ __forceinline__ float fs_bias_term(int bias_q, float inv_bias) {
    return rintf(__fmul_rn((float)bias_q, inv_bias));
}

__device__ __forceinline__ float fs_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }

// The gate and state arithmetic of PointwiseOperationsFP (src/gru_forward_gpu_quant_fp.cu:714-770)
// in two pieces, so that a kernel may compute the update and the reset gate on different threads.
// ih / hh are the requantized, clamped linear outputs, h_old the quantized previous state.
// The activation half of a gate: real_sigmoid_f / real_tanh_f (include/quantize_ops_helper.h:
// 687-720) on a clamped gate input; g = 0 update, 1 reset (sigmoid), 2 new (tanh).
__device__ __forceinline__ float fs_activation(const FsConsts &fc, int g, float in) {
    const float x = (in - fc.zp_in[g]) * fc.s_in[g];
    const float y = g == 2 ? tanhf(x) : fs_sigmoid(x);
    return fs_clamp(rintf(y / fc.s_out[g] + fc.zp_out[g]), fc.out_lo[g], fc.out_hi[g]);
}
// The same through the table (tab: shared-window address of the float table), or directly.
__device__ __forceinline__ float fs_activation_tab(const FsConsts &fc, uint32_t tab, int g, float in) {
    if (fc.tab_on) return __int_as_float(lds_i32(tab + 4u * (uint32_t)(fc.tab_off[g] + (int)(in - fc.in_lo[g]))));
    return fs_activation(fc, g, in);
}
// computeUpdateGateFP / computeResetGateFP (:153-239); g = 0 update, 1 reset
__device__ __forceinline__ float fs_gate_input(const FsConsts &fc, int g, float ih, float hh) {
    const float a = rintf((ih - fc.zp_ih) * fc.ih_to[g]);
    const float c = rintf((hh - fc.zp_hh) * fc.hh_to[g]);
    return fs_clamp(a + c + fc.zp_in[g], fc.in_lo[g], fc.in_hi[g]);
}
__device__ __forceinline__ float fs_sigmoid_gate(const FsConsts &fc, int g, float ih, float hh) {
    return fs_activation(fc, g, fs_gate_input(fc, g, ih, hh));
}
// computeNewGateFP (:241-290) and computeHiddenStateFP (:302-372): returns the new quantized state
__device__ __forceinline__ float fs_new_gate_input(const FsConsts &fc, float r, float ih_n, float hh_n) {
    const float rh = rintf(((r - fc.zp_out[1]) * (hh_n - fc.zp_hh)) * fc.rh_to_n);
    const float a_n = rintf((ih_n - fc.zp_ih) * fc.ih_to[2]);
    return fs_clamp(a_n + rh + fc.zp_in[2], fc.in_lo[2], fc.in_hi[2]);
}
__device__ __forceinline__ float fs_state(const FsConsts &fc, float u, float n, float h_old) {
    const float n_h = rintf((n - fc.zp_out[2]) * fc.n_to_h) + fc.zp_h;
    const float old_c = (u - fc.zp_out[0]) * (h_old - fc.zp_h);
    const float new_c = ((fc.one_q - u) - fc.zp_out[0]) * (n_h - fc.zp_h);
    return fs_clamp(rintf((old_c + new_c) * fc.uh_to_h) + fc.zp_h, fc.h_lo, fc.h_hi);
}
__device__ __forceinline__ float fs_finish(const FsConsts &fc, float u, float r, float ih_n, float hh_n,
                                           float h_old) {
    return fs_state(fc, u, fs_activation(fc, 2, fs_new_gate_input(fc, r, ih_n, hh_n)), h_old);
}
// The gates through the table where it exists (tab_on), else evaluated.
__device__ __forceinline__ float fs_sigmoid_gate_tab(const FsConsts &fc, uint32_t tab, int g, float ih, float hh) {
    return fs_activation_tab(fc, tab, g, fs_gate_input(fc, g, ih, hh));
}
__device__ __forceinline__ float fs_finish_tab(const FsConsts &fc, uint32_t tab, float u, float r, float ih_n,
                                               float hh_n, float h_old) {
    return fs_state(fc, u, fs_activation_tab(fc, tab, 2, fs_new_gate_input(fc, r, ih_n, hh_n)), h_old);
}
__device__ __forceinline__ float fs_cell(const FsConsts &fc, const float ih[3], const float hh[3],
                                         float h_old) {
    const float u = fs_sigmoid_gate(fc, 0, ih[0], hh[0]);
    const float r = fs_sigmoid_gate(fc, 1, ih[1], hh[1]);
    return fs_finish(fc, u, r, ih[2], hh[2], h_old);
}

// linear_epilogue32 for a scale with the shift-free form.
template <bool Tie = true>
__device__ __forceinline__ int32_t linear_epilogue_fast(int32_t acc, const FastLin &f, int32_t zp_out,
                                                        int32_t lo, int32_t hi) {
    return clampi(lin_round<Tie>(acc, f) + zp_out, lo, hi);
}

}  // namespace qgru
