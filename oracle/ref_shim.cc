// ref_shim.cc - TEST INFRASTRUCTURE, not product code.
//
// A thin extern "C" driver around the UNMODIFIED reference sources (compiled where they
// lie by oracle/Makefile into oracle/_ref/).  It lets the tests, the golden-vector
// generator and the CPU-baseline leg of the benchmark call the reference's own CPU
// integer path through ctypes, using the POD types of include/qgru.h as the exchange
// format.  Only host functions of the reference are reached: the CPU forward
// (src/gru_forward_cpu_quant.cc), quantitativeWeightCPU / quantGRUForwardCPU /
// calculateGRUQuantitativeParameters (src/gru_interface.cc) and the LUT generator
// (src/quantize_ops.cu:21-52).  No CUDA call is made by anything reached from the ref_*
// functions.  The ref_gpu_* functions at the end of the file are the exception: they run the
// reference's own GPU paths (integer forward, float forward, float-storage forward, MinMax and
// histogram calibration) on the current CUDA device, with host buffers in and out, so that
// the GPU tests can hold the product against the reference itself on the same machine.
#include <array>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

#include <cublas_v2.h>
#include <cuda_runtime.h>

#include "calibration_gpu.cuh"
#include "gru_interface.h"
#include "gru_quant_cpu.h"
#include "pot_sqnr_calibrator.h"
#include "quantize_ops_helper.h"

#include "qgru.h"
#include "ref_pod.h"

namespace {

thread_local std::string g_err;

using refpod::bwOf;
using refpod::fillConfig;
using refpod::fromPod;
using refpod::lutFromPod;
using refpod::qpOf;

void lutToPod(const SigmoidLUT &in, qgru_lut &out) {
    std::memset(&out, 0, sizeof(out));
    for (int i = 0; i < NUM_SEGMENTS; ++i) {
        out.seg[i].q_b = in.segments[i].q_b;
        out.seg[i].n_bx = in.segments[i].n_BX_total;
        out.seg[i].term_c = in.segments[i].term_c_precomputed;
        out.seg[i].threshold = in.segments[i].threshold;
    }
    out.zp_x = in.zp_x;
}

void scalarToPod(const QuantParam &q, qgru_op &o) {
    o.scale = q.scale;
    o.zero_point = q.zero_point;
}

void toPod(const GRUQuantParams &q, qgru_params &p, float *sW, float *sR, float *sbw, float *sbr) {
    p.hidden = q.hidden_;
    scalarToPod(q.x_, p.op[QGRU_OP_X]);
    scalarToPod(q.h_, p.op[QGRU_OP_H]);
    scalarToPod(q.W_.tensor(), p.op[QGRU_OP_W]);
    scalarToPod(q.R_.tensor(), p.op[QGRU_OP_R]);
    scalarToPod(q.bw_.tensor(), p.op[QGRU_OP_BW]);
    scalarToPod(q.br_.tensor(), p.op[QGRU_OP_BR]);
    scalarToPod(q.weight_ih_linear_, p.op[QGRU_OP_IH_LINEAR]);
    scalarToPod(q.weight_hh_linear_, p.op[QGRU_OP_HH_LINEAR]);
    scalarToPod(q.update_gate_input_, p.op[QGRU_OP_UPDATE_IN]);
    scalarToPod(q.update_gate_output_, p.op[QGRU_OP_UPDATE_OUT]);
    scalarToPod(q.reset_gate_input_, p.op[QGRU_OP_RESET_IN]);
    scalarToPod(q.reset_gate_output_, p.op[QGRU_OP_RESET_OUT]);
    scalarToPod(q.new_gate_input_, p.op[QGRU_OP_NEW_IN]);
    scalarToPod(q.new_gate_output_, p.op[QGRU_OP_NEW_OUT]);
    scalarToPod(q.mul_reset_hidden_, p.op[QGRU_OP_MUL_RESET_HIDDEN]);
    scalarToPod(q.mul_new_contribution_, p.op[QGRU_OP_MUL_NEW_CONTRIB]);
    scalarToPod(q.mul_old_contribution_, p.op[QGRU_OP_MUL_OLD_CONTRIB]);
    for (int c = 0; c < q.hidden_ * 3; ++c) {
        if (sW) sW[c] = q.W_.channel(c).scale;
        if (sR) sR[c] = q.R_.channel(c).scale;
        if (sbw) sbw[c] = q.bw_.channel(c).scale;
        if (sbr) sbr[c] = q.br_.channel(c).scale;
    }
    lutToPod(q.sigmoid_update_gate_lut_, p.lut[QGRU_LUT_UPDATE]);
    lutToPod(q.sigmoid_reset_gate_lut_, p.lut[QGRU_LUT_RESET]);
    lutToPod(q.tanh_new_gate_lut_, p.lut[QGRU_LUT_NEW]);
}

template <class F>
int guarded(F &&f) {
    try {
        f();
        return 0;
    } catch (const std::exception &e) {
        g_err = e.what();
        return 1;
    } catch (...) {
        g_err = "unknown exception";
        return 1;
    }
}

// The reference's integer core with int32 inputs and outputs: what quantGRUForwardCPU
// (src/gru_interface.cc:796-835) does between quantising x and dequantising h.
void forwardI32(int T, int B, int I, int H, const int32_t *W, const int32_t *R, const int32_t *bw,
                const int32_t *br, const int32_t *x_q, const int32_t *h0_q,
                const GRUQuantParams &q, int32_t *h_q) {
    const int NH = B * H;
    for (int i = 0; i < NH; ++i) h_q[i] = h0_q ? h0_q[i] : q.h_.zero_point;
    cpu::ForwardPassQuantCPU fwd(false, B, I, H);
    fwd.setRescaleParam(q);
    fwd.Run(T, W, R, bw, br, x_q, h_q, nullptr, 0.0f, nullptr);
}

}  // namespace

extern "C" {

const char *ref_last_error() { return g_err.c_str(); }

int ref_encode_mshift(float scale, uint16_t *m, int8_t *s) {
    return guarded([&] {
        FixedPointScale f = encodeMShift(scale);
        *m = f.multiplier;
        *s = f.shift;
    });
}

int64_t ref_rshift_round(int64_t x, int n) { return rshift_round(x, static_cast<int8_t>(n)); }

int32_t ref_lut_eval(const qgru_lut *lut, int32_t q_x, const qgru_op *in_bw, const qgru_op *out_bw) {
    SigmoidLUT l;
    lutFromPod(*lut, l);
    return piecewise_linear(q_x, l, bwOf(*in_bw), bwOf(*out_bw));
}

int ref_generate_luts(qgru_params *p) {
    return guarded([&] {
        std::vector<float> ones(p->hidden * 3, 1.0f);
        GRUQuantParams q = fromPod(*p, ones.data(), ones.data(), ones.data(), ones.data());
        generate_piecewise_linear_lut_to_params(q);
        lutToPod(q.sigmoid_update_gate_lut_, p->lut[QGRU_LUT_UPDATE]);
        lutToPod(q.sigmoid_reset_gate_lut_, p->lut[QGRU_LUT_RESET]);
        lutToPod(q.tanh_new_gate_lut_, p->lut[QGRU_LUT_NEW]);
    });
}

int ref_calc_params_from_ranges(const qgru_ranges *r, qgru_params *p, float *sW, float *sR,
                                float *sbw, float *sbr) {
    return guarded([&] {
        OperatorQuantConfig cfg;
        fillConfig(*p, cfg);
        GRUQuantizationRanges g(r->hidden);
        const int C = r->hidden * 3;
        g.min_x_ = r->min_v[QGRU_OP_X]; g.max_x_ = r->max_v[QGRU_OP_X];
        g.min_h_ = r->min_v[QGRU_OP_H]; g.max_h_ = r->max_v[QGRU_OP_H];
        g.min_Wx_ = r->min_v[QGRU_OP_IH_LINEAR]; g.max_Wx_ = r->max_v[QGRU_OP_IH_LINEAR];
        g.min_Rh_ = r->min_v[QGRU_OP_HH_LINEAR]; g.max_Rh_ = r->max_v[QGRU_OP_HH_LINEAR];
        g.min_update_gate_input_ = r->min_v[QGRU_OP_UPDATE_IN]; g.max_update_gate_input_ = r->max_v[QGRU_OP_UPDATE_IN];
        g.min_update_gate_output_ = r->min_v[QGRU_OP_UPDATE_OUT]; g.max_update_gate_output_ = r->max_v[QGRU_OP_UPDATE_OUT];
        g.min_reset_gate_input_ = r->min_v[QGRU_OP_RESET_IN]; g.max_reset_gate_input_ = r->max_v[QGRU_OP_RESET_IN];
        g.min_reset_gate_output_ = r->min_v[QGRU_OP_RESET_OUT]; g.max_reset_gate_output_ = r->max_v[QGRU_OP_RESET_OUT];
        g.min_new_gate_input_ = r->min_v[QGRU_OP_NEW_IN]; g.max_new_gate_input_ = r->max_v[QGRU_OP_NEW_IN];
        g.min_new_gate_output_ = r->min_v[QGRU_OP_NEW_OUT]; g.max_new_gate_output_ = r->max_v[QGRU_OP_NEW_OUT];
        g.min_mul_reset_hidden_ = r->min_v[QGRU_OP_MUL_RESET_HIDDEN]; g.max_mul_reset_hidden_ = r->max_v[QGRU_OP_MUL_RESET_HIDDEN];
        g.min_mul_new_contribution_ = r->min_v[QGRU_OP_MUL_NEW_CONTRIB]; g.max_mul_new_contribution_ = r->max_v[QGRU_OP_MUL_NEW_CONTRIB];
        g.min_mul_old_contribution_ = r->min_v[QGRU_OP_MUL_OLD_CONTRIB]; g.max_mul_old_contribution_ = r->max_v[QGRU_OP_MUL_OLD_CONTRIB];
        g.min_W_.assign(r->min_W, r->min_W + C); g.max_W_.assign(r->max_W, r->max_W + C);
        g.min_R_.assign(r->min_R, r->min_R + C); g.max_R_.assign(r->max_R, r->max_R + C);
        g.min_bw_.assign(r->min_bw, r->min_bw + C); g.max_bw_.assign(r->max_bw, r->max_bw + C);
        g.min_br_.assign(r->min_br, r->min_br + C); g.max_br_.assign(r->max_br, r->max_br + C);
        GRUQuantParams q = calculateGRUQuantitativeParameters(g, cfg);
        toPod(q, *p, sW, sR, sbw, sbr);
    });
}

int ref_quantize_weights(int I, int H, const float *W, const float *R, const float *bw,
                         const float *br, const qgru_params *p, const float *sW, const float *sR,
                         const float *sbw, const float *sbr, int32_t *W_q, int32_t *R_q,
                         int32_t *bw_q, int32_t *br_q) {
    return guarded([&] {
        GRUQuantParams q = fromPod(*p, sW, sR, sbw, sbr);
        quantitativeWeightCPU(I, H, W, R, bw, br, q, W_q, R_q, bw_q, br_q);
    });
}

// quantize() of one activation tensor with operator `op` of p (src/gru_interface.cc:806-809).
int ref_quantize(const float *x, int32_t *out, size_t n, const qgru_params *p, int op) {
    return guarded([&] {
        const QuantParam qp = qpOf(p->op[op]);
        const FixedPointScale fs = toFixedScale(qp, p->use_pot2 != 0);
        const QuantBitWidth bw = bwOf(p->op[op]);
        for (size_t i = 0; i < n; ++i) out[i] = quantize(x[i], fs, qp.zero_point, bw);
    });
}

int ref_dequantize(const int32_t *q_in, float *out, size_t n, const qgru_params *p, int op) {
    return guarded([&] {
        const QuantParam qp = qpOf(p->op[op]);
        const FixedPointScale fs = toFixedScale(qp, p->use_pot2 != 0);
        for (size_t i = 0; i < n; ++i) out[i] = dequantize(q_in[i], fs, qp.zero_point);
    });
}

int ref_forward_i32(int T, int B, int I, int H, const int32_t *W, const int32_t *R,
                    const int32_t *bw, const int32_t *br, const int32_t *x_q, const int32_t *h0_q,
                    const qgru_params *p, const float *sW, const float *sR, const float *sbw,
                    const float *sbr, int32_t *h_q) {
    return guarded([&] {
        GRUQuantParams q = fromPod(*p, sW, sR, sbw, sbr);
        forwardI32(T, B, I, H, W, R, bw, br, x_q, h0_q, q, h_q);
    });
}

// Same result as ref_forward_i32, computed on `nthreads` host threads by cutting the batch
// into independent slices (rows of a batch never interact in a GRU).  Used as the
// all-cores CPU baseline; the reference itself is single threaded.
// Training-mode forward of the CPU path: also returns v_q [T,B,4H] = (update, reset, new gate
// outputs, R*h + br row of the new gate), src/gru_forward_cpu_quant.cc:199-205.
int ref_forward_i32_v(int T, int B, int I, int H, const int32_t *W, const int32_t *R,
                      const int32_t *bw, const int32_t *br, const int32_t *x_q, const int32_t *h0_q,
                      const qgru_params *p, const float *sW, const float *sR, const float *sbw,
                      const float *sbr, int32_t *h_q, int32_t *v_q) {
    return guarded([&] {
        GRUQuantParams q = fromPod(*p, sW, sR, sbw, sbr);
        const int NH = B * H;
        for (int i = 0; i < NH; ++i) h_q[i] = h0_q ? h0_q[i] : q.h_.zero_point;
        cpu::ForwardPassQuantCPU fwd(true, B, I, H);
        fwd.setRescaleParam(q);
        fwd.Run(T, W, R, bw, br, x_q, h_q, v_q, 0.0f, nullptr);
    });
}

int ref_forward_i32_mt(int T, int B, int I, int H, const int32_t *W, const int32_t *R,
                       const int32_t *bw, const int32_t *br, const int32_t *x_q,
                       const int32_t *h0_q, const qgru_params *p, const float *sW,
                       const float *sR, const float *sbw, const float *sbr, int32_t *h_q,
                       int nthreads) {
    return guarded([&] {
        GRUQuantParams q = fromPod(*p, sW, sR, sbw, sbr);
        if (nthreads < 1) nthreads = 1;
        if (nthreads > B) nthreads = B;
        std::vector<std::thread> th;
        std::vector<std::string> errs(nthreads);
        for (int w = 0; w < nthreads; ++w) {
            th.emplace_back([&, w] {
                try {
                    const int b0 = static_cast<int>(static_cast<int64_t>(B) * w / nthreads);
                    const int b1 = static_cast<int>(static_cast<int64_t>(B) * (w + 1) / nthreads);
                    const int Bs = b1 - b0;
                    if (Bs <= 0) return;
                    std::vector<int32_t> xs(static_cast<size_t>(T) * Bs * I);
                    std::vector<int32_t> hs(static_cast<size_t>(T + 1) * Bs * H);
                    std::vector<int32_t> h0s;
                    for (int t = 0; t < T; ++t)
                        std::memcpy(&xs[static_cast<size_t>(t) * Bs * I],
                                    &x_q[(static_cast<size_t>(t) * B + b0) * I],
                                    sizeof(int32_t) * Bs * I);
                    if (h0_q) h0s.assign(h0_q + static_cast<size_t>(b0) * H, h0_q + static_cast<size_t>(b1) * H);
                    forwardI32(T, Bs, I, H, W, R, bw, br, xs.data(), h0_q ? h0s.data() : nullptr, q,
                               hs.data());
                    for (int t = 0; t <= T; ++t)
                        std::memcpy(&h_q[(static_cast<size_t>(t) * B + b0) * H],
                                    &hs[static_cast<size_t>(t) * Bs * H], sizeof(int32_t) * Bs * H);
                } catch (const std::exception &e) {
                    errs[w] = e.what();
                }
            });
        }
        for (auto &t : th) t.join();
        for (auto &e : errs)
            if (!e.empty()) throw std::runtime_error(e);
    });
}

// quantGRUForwardCPU, int32-weights overload (src/gru_interface.cc:796-867): float x in,
// float h out.
int ref_forward_f32(int T, int B, int I, int H, const int32_t *W, const int32_t *R,
                    const int32_t *bw, const int32_t *br, const float *x, const float *h0,
                    const qgru_params *p, const float *sW, const float *sR, const float *sbw,
                    const float *sbr, float *h) {
    return guarded([&] {
        GRUQuantParams q = fromPod(*p, sW, sR, sbw, sbr);
        quantGRUForwardCPU(false, T, B, I, H, W, R, bw, br, x, h0, q, h, nullptr);
    });
}


// ---- histogram calibration: the reference's host code (header-only), run as it is

// calibrateContinuousScaleFromHistogram + encodeScaleResult + storedScaleForMode
// (include/pot_sqnr_calibrator.h), the body of histCalibrate in
// calculateGRUQuantitativeParametersFromHistograms (src/gru_interface.cc:1092-1100).
int ref_calibrate_from_histogram(const float *counts, int bins, float min_val, float max_val,
                                 int64_t total, int use_pot2, int use_percentile, float percentile,
                                 qgru_op *op) {
    return guarded([&] {
        Histogram h(bins);
        h.counts.assign(counts, counts + bins);
        h.min_val = min_val;
        h.max_val = max_val;
        h.total_count = total;
        const QuantBitWidth bw = bwOf(*op);
        const bool sym = op->symmetric != 0;
        ContinuousScaleResult c = calibrateContinuousScaleFromHistogram(h, bw, sym, use_percentile != 0, percentile);
        EncodedScaleResult e = encodeScaleResult(c.scale, c.min, bw, sym, use_pot2 != 0);
        op->scale = storedScaleForMode(e, use_pot2 != 0);
        op->zero_point = e.zero_point;
    });
}

// the reference's CPU HistogramCollector (include/histogram_collector.h), one object per handle
void *ref_hist_new(int bins) { return new HistogramCollector(bins); }
void ref_hist_free(void *h) { delete static_cast<HistogramCollector *>(h); }
int ref_hist_collect(void *h, const float *data, size_t n) {
    return guarded([&] { static_cast<HistogramCollector *>(h)->collect(data, n); });
}
int ref_hist_get(void *h, float *counts, float *min_val, float *max_val, int64_t *total) {
    return guarded([&] {
        const Histogram &g = static_cast<HistogramCollector *>(h)->histogram();
        if (counts) std::memcpy(counts, g.counts.data(), sizeof(float) * g.counts.size());
        *min_val = g.min_val;
        *max_val = g.max_val;
        *total = g.total_count;
    });
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// The reference's GPU paths, host buffers in and out.  Test infrastructure for machines with a
// CUDA device; every function returns 1 (message in ref_last_error) when a CUDA call fails.
namespace {

void cudaOk(cudaError_t e, const char *what) {
    if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

template <class T>
struct DevBuf {
    T *p = nullptr;
    size_t n = 0;
    DevBuf() = default;
    explicit DevBuf(size_t count) : n(count) {
        if (n) cudaOk(cudaMalloc(&p, n * sizeof(T)), "cudaMalloc");
    }
    DevBuf(const T *host, size_t count) : DevBuf(host ? count : 0) {
        if (n) cudaOk(cudaMemcpy(p, host, n * sizeof(T), cudaMemcpyHostToDevice), "copy in");
    }
    DevBuf(const DevBuf &) = delete;
    DevBuf &operator=(const DevBuf &) = delete;
    ~DevBuf() {
        if (p) cudaFree(p);
    }
    void zero() {
        if (n) cudaOk(cudaMemset(p, 0, n * sizeof(T)), "cudaMemset");
    }
    void toHost(T *host) const {
        if (host && n) cudaOk(cudaMemcpy(host, p, n * sizeof(T), cudaMemcpyDeviceToHost), "copy out");
    }
};

cublasHandle_t &blasHandle() {
    static cublasHandle_t h = nullptr;
    if (!h) init_gru_cublas(h);
    return h;
}

void rangesFromPod(const qgru_ranges &r, GRUQuantizationRanges &g) {
    const int C = r.hidden * 3;
    g.min_x_ = r.min_v[QGRU_OP_X]; g.max_x_ = r.max_v[QGRU_OP_X];
    g.min_h_ = r.min_v[QGRU_OP_H]; g.max_h_ = r.max_v[QGRU_OP_H];
    g.min_Wx_ = r.min_v[QGRU_OP_IH_LINEAR]; g.max_Wx_ = r.max_v[QGRU_OP_IH_LINEAR];
    g.min_Rh_ = r.min_v[QGRU_OP_HH_LINEAR]; g.max_Rh_ = r.max_v[QGRU_OP_HH_LINEAR];
    g.min_update_gate_input_ = r.min_v[QGRU_OP_UPDATE_IN]; g.max_update_gate_input_ = r.max_v[QGRU_OP_UPDATE_IN];
    g.min_update_gate_output_ = r.min_v[QGRU_OP_UPDATE_OUT]; g.max_update_gate_output_ = r.max_v[QGRU_OP_UPDATE_OUT];
    g.min_reset_gate_input_ = r.min_v[QGRU_OP_RESET_IN]; g.max_reset_gate_input_ = r.max_v[QGRU_OP_RESET_IN];
    g.min_reset_gate_output_ = r.min_v[QGRU_OP_RESET_OUT]; g.max_reset_gate_output_ = r.max_v[QGRU_OP_RESET_OUT];
    g.min_new_gate_input_ = r.min_v[QGRU_OP_NEW_IN]; g.max_new_gate_input_ = r.max_v[QGRU_OP_NEW_IN];
    g.min_new_gate_output_ = r.min_v[QGRU_OP_NEW_OUT]; g.max_new_gate_output_ = r.max_v[QGRU_OP_NEW_OUT];
    g.min_mul_reset_hidden_ = r.min_v[QGRU_OP_MUL_RESET_HIDDEN]; g.max_mul_reset_hidden_ = r.max_v[QGRU_OP_MUL_RESET_HIDDEN];
    g.min_mul_new_contribution_ = r.min_v[QGRU_OP_MUL_NEW_CONTRIB]; g.max_mul_new_contribution_ = r.max_v[QGRU_OP_MUL_NEW_CONTRIB];
    g.min_mul_old_contribution_ = r.min_v[QGRU_OP_MUL_OLD_CONTRIB]; g.max_mul_old_contribution_ = r.max_v[QGRU_OP_MUL_OLD_CONTRIB];
    g.min_W_.assign(r.min_W, r.min_W + C); g.max_W_.assign(r.max_W, r.max_W + C);
    g.min_R_.assign(r.min_R, r.min_R + C); g.max_R_.assign(r.max_R, r.max_R + C);
    g.min_bw_.assign(r.min_bw, r.min_bw + C); g.max_bw_.assign(r.max_bw, r.max_bw + C);
    g.min_br_.assign(r.min_br, r.min_br + C); g.max_br_.assign(r.max_br, r.max_br + C);
}

void rangesToPod(const GRUQuantizationRanges &g, qgru_ranges &r) {
    const size_t C = size_t(r.hidden) * 3;
    r.min_v[QGRU_OP_X] = g.min_x_; r.max_v[QGRU_OP_X] = g.max_x_;
    r.min_v[QGRU_OP_H] = g.min_h_; r.max_v[QGRU_OP_H] = g.max_h_;
    r.min_v[QGRU_OP_IH_LINEAR] = g.min_Wx_; r.max_v[QGRU_OP_IH_LINEAR] = g.max_Wx_;
    r.min_v[QGRU_OP_HH_LINEAR] = g.min_Rh_; r.max_v[QGRU_OP_HH_LINEAR] = g.max_Rh_;
    r.min_v[QGRU_OP_UPDATE_IN] = g.min_update_gate_input_; r.max_v[QGRU_OP_UPDATE_IN] = g.max_update_gate_input_;
    r.min_v[QGRU_OP_UPDATE_OUT] = g.min_update_gate_output_; r.max_v[QGRU_OP_UPDATE_OUT] = g.max_update_gate_output_;
    r.min_v[QGRU_OP_RESET_IN] = g.min_reset_gate_input_; r.max_v[QGRU_OP_RESET_IN] = g.max_reset_gate_input_;
    r.min_v[QGRU_OP_RESET_OUT] = g.min_reset_gate_output_; r.max_v[QGRU_OP_RESET_OUT] = g.max_reset_gate_output_;
    r.min_v[QGRU_OP_NEW_IN] = g.min_new_gate_input_; r.max_v[QGRU_OP_NEW_IN] = g.max_new_gate_input_;
    r.min_v[QGRU_OP_NEW_OUT] = g.min_new_gate_output_; r.max_v[QGRU_OP_NEW_OUT] = g.max_new_gate_output_;
    r.min_v[QGRU_OP_MUL_RESET_HIDDEN] = g.min_mul_reset_hidden_; r.max_v[QGRU_OP_MUL_RESET_HIDDEN] = g.max_mul_reset_hidden_;
    r.min_v[QGRU_OP_MUL_NEW_CONTRIB] = g.min_mul_new_contribution_; r.max_v[QGRU_OP_MUL_NEW_CONTRIB] = g.max_mul_new_contribution_;
    r.min_v[QGRU_OP_MUL_OLD_CONTRIB] = g.min_mul_old_contribution_; r.max_v[QGRU_OP_MUL_OLD_CONTRIB] = g.max_mul_old_contribution_;
    auto put = [&](float *dst, const std::vector<float> &src) {
        if (dst && src.size() == C) std::memcpy(dst, src.data(), C * sizeof(float));
    };
    put(r.min_W, g.min_W_); put(r.max_W, g.max_W_);
    put(r.min_R, g.min_R_); put(r.max_R, g.max_R_);
    put(r.min_bw, g.min_bw_); put(r.max_bw, g.max_bw_);
    put(r.min_br, g.min_br_); put(r.max_br, g.max_br_);
}

// the collector that include/qgru.h's histogram index names, in the CPU copy of a collector set
const HistogramCollector *histByIndex(const GRUHistogramCollectors &c, int index) {
    const int C3 = c.hidden_ * 3;
    switch (index) {
        case QGRU_OP_X: return &c.x_hist;
        case QGRU_OP_H: return &c.h_hist;
        case QGRU_OP_W: return &c.W_tensor_hist;
        case QGRU_OP_R: return &c.R_tensor_hist;
        case QGRU_OP_BW: return &c.bw_tensor_hist;
        case QGRU_OP_BR: return &c.br_tensor_hist;
        case QGRU_OP_IH_LINEAR: return &c.Wx_hist;
        case QGRU_OP_HH_LINEAR: return &c.Rh_hist;
        case QGRU_OP_UPDATE_IN: return &c.update_gate_input_hist;
        case QGRU_OP_UPDATE_OUT: return &c.update_gate_output_hist;
        case QGRU_OP_RESET_IN: return &c.reset_gate_input_hist;
        case QGRU_OP_RESET_OUT: return &c.reset_gate_output_hist;
        case QGRU_OP_NEW_IN: return &c.new_gate_input_hist;
        case QGRU_OP_NEW_OUT: return &c.new_gate_output_hist;
        case QGRU_OP_MUL_RESET_HIDDEN: return &c.mul_reset_hidden_hist;
        case QGRU_OP_MUL_NEW_CONTRIB: return &c.mul_new_contribution_hist;
        case QGRU_OP_MUL_OLD_CONTRIB: return &c.mul_old_contribution_hist;
        default: break;
    }
    if (index >= QGRU_HIST_GATE0 && index < QGRU_HIST_CHANNEL0) {
        const int k = (index - QGRU_HIST_GATE0) / 3, g = (index - QGRU_HIST_GATE0) % 3;
        const std::array<HistogramCollector, 3> *a[4] = {&c.W_gate_hist, &c.R_gate_hist, &c.bw_gate_hist,
                                                         &c.br_gate_hist};
        return &(*a[k])[g];
    }
    if (index >= QGRU_HIST_CHANNEL0 && index < QGRU_HIST_CHANNEL0 + 4 * C3) {
        const int k = (index - QGRU_HIST_CHANNEL0) / C3, ch = (index - QGRU_HIST_CHANNEL0) % C3;
        const std::vector<HistogramCollector> *a[4] = {&c.W_hist, &c.R_hist, &c.bw_hist, &c.br_hist};
        return &(*a[k])[ch];
    }
    throw std::invalid_argument("histogram index out of range");
}

struct GpuHistSet {
    GRUGPUHistogramCollectors gpu;
    GRUHistogramCollectors cpu;   // refreshed by ref_gpu_histset_sync
    explicit GpuHistSet(int hidden, int bins) : gpu(hidden, bins) {}
};

}  // namespace

extern "C" {

int ref_gpu_device_count() {
    int n = 0;
    return cudaGetDeviceCount(&n) == cudaSuccess ? n : 0;
}

// quantGRUForwardInt32 (src/gru_interface.cc:551): the reference's GPU integer core.
// masks[5] = weight_ih_linear, weight_hh_linear, gate_input, gate_output, h (each may be null
// HERE; in training mode the reference's own kernels write the two linear masks without a null
// check, src/gru_forward_gpu_quant.cu:168-178, so all five device buffers are always handed
// to it in that mode and only the requested ones are copied back).
int ref_gpu_forward_i32(int training, int T, int B, int I, int H, const int32_t *W, const int32_t *R,
                        const int32_t *bw, const int32_t *br, const int32_t *x_q, const int32_t *h0_q,
                        const qgru_params *p, const float *sW, const float *sR, const float *sbw,
                        const float *sbr, int32_t *h_q, int32_t *v_q, uint8_t *const *masks) {
    return guarded([&] {
        GRUQuantParams q = fromPod(*p, sW, sR, sbw, sbr);
        const size_t C3 = size_t(H) * 3, TB = size_t(T) * B;
        DevBuf<int32_t> dW(W, size_t(I) * C3), dR(R, size_t(H) * C3), dbw(bw, C3), dbr(br, C3),
            dx(x_q, TB * I), dh0(h0_q, size_t(B) * H), dh((TB + B) * H), dv((v_q || training) ? TB * H * 4 : 0);
        const size_t msz[5] = {TB * C3, TB * C3, TB * C3, TB * C3, TB * H};
        std::unique_ptr<DevBuf<uint8_t>> dm[5];
        uint8_t *mp[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};
        for (int k = 0; k < 5; ++k)
            if (training) {
                dm[k].reset(new DevBuf<uint8_t>(msz[k]));
                dm[k]->zero();
                mp[k] = dm[k]->p;
            }
        dh.zero();
        quantGRUForwardInt32(training != 0, T, B, I, H, dW.p, dR.p, dbw.p, dbr.p, dx.p, dh0.p, q,
                             blasHandle(), dh.p, dv.p, mp[0], mp[1], mp[2], mp[3], mp[4]);
        cudaOk(cudaDeviceSynchronize(), "quantGRUForwardInt32");
        dh.toHost(h_q);
        dv.toHost(v_q);
        for (int k = 0; k < 5; ++k)
            if (dm[k] && masks && masks[k]) dm[k]->toHost(masks[k]);
    });
}

// Device time of `iters` calls of quantGRUForwardInt32 (inference) with the inputs already
// resident on the device, after `warmup` untimed calls: milliseconds per call, CUDA events on
// the default stream around the calls (the reference synchronises the device inside each call).
int ref_gpu_time_forward_i32(int T, int B, int I, int H, const int32_t *W, const int32_t *R,
                             const int32_t *bw, const int32_t *br, const int32_t *x_q,
                             const qgru_params *p, const float *sW, const float *sR, const float *sbw,
                             const float *sbr, int warmup, int iters, float *ms_per_call) {
    return guarded([&] {
        GRUQuantParams q = fromPod(*p, sW, sR, sbw, sbr);
        const size_t C3 = size_t(H) * 3, TB = size_t(T) * B;
        DevBuf<int32_t> dW(W, size_t(I) * C3), dR(R, size_t(H) * C3), dbw(bw, C3), dbr(br, C3),
            dx(x_q, TB * I), dh((TB + B) * H);
        cudaEvent_t e0, e1;
        cudaOk(cudaEventCreate(&e0), "cudaEventCreate");
        cudaOk(cudaEventCreate(&e1), "cudaEventCreate");
        for (int i = 0; i < warmup + iters; ++i) {
            if (i == warmup) cudaOk(cudaEventRecord(e0, 0), "cudaEventRecord");
            quantGRUForwardInt32(false, T, B, I, H, dW.p, dR.p, dbw.p, dbr.p, dx.p, nullptr, q,
                                 blasHandle(), dh.p, nullptr);
        }
        cudaOk(cudaEventRecord(e1, 0), "cudaEventRecord");
        cudaOk(cudaEventSynchronize(e1), "cudaEventSynchronize");
        float ms = 0.f;
        cudaOk(cudaEventElapsedTime(&ms, e0, e1), "cudaEventElapsedTime");
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
        *ms_per_call = ms / (float)iters;
    });
}

// The same for quantGRUForwardFP (inference): float inputs resident, ms per call.
int ref_gpu_time_forward_fstorage(int T, int B, int I, int H, const float *W, const float *R,
                                  const float *bw, const float *br, const float *x,
                                  const qgru_params *p, const float *sW, const float *sR,
                                  const float *sbw, const float *sbr, int warmup, int iters,
                                  float *ms_per_call) {
    return guarded([&] {
        GRUQuantParams q = fromPod(*p, sW, sR, sbw, sbr);
        const size_t C3 = size_t(H) * 3, TB = size_t(T) * B;
        DevBuf<float> dW(W, size_t(I) * C3), dR(R, size_t(H) * C3), dbw(bw, C3), dbr(br, C3),
            dx(x, TB * I), dh((TB + B) * H);
        DevBuf<float> qW(size_t(I) * C3), qR(size_t(H) * C3), qbw(C3), qbr(C3), qx(TB * I);
        cudaEvent_t e0, e1;
        cudaOk(cudaEventCreate(&e0), "cudaEventCreate");
        cudaOk(cudaEventCreate(&e1), "cudaEventCreate");
        for (int i = 0; i < warmup + iters; ++i) {
            if (i == warmup) cudaOk(cudaEventRecord(e0, 0), "cudaEventRecord");
            quantGRUForwardFP(false, T, B, I, H, dW.p, dR.p, dbw.p, dbr.p, dx.p, nullptr, q, blasHandle(),
                              dh.p, nullptr, qW.p, qR.p, qbw.p, qbr.p, qx.p, nullptr, nullptr, nullptr,
                              nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr);
        }
        cudaOk(cudaEventRecord(e1, 0), "cudaEventRecord");
        cudaOk(cudaEventSynchronize(e1), "cudaEventSynchronize");
        float ms = 0.f;
        cudaOk(cudaEventElapsedTime(&ms, e0, e1), "cudaEventElapsedTime");
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
        *ms_per_call = ms / (float)iters;
    });
}

// hasteGRUBackward (src/gru_interface.cc:215) or, with use_masks, quantGRUBackward (:246) with
// all eleven masks (masks[11] in the order of qgru_bwd_masks; each must then be non-null).
// W_t [3H,I], R_t [3H,H], x_t [I,T*B]; dW..dbr are returned from zero, dh from zero.
int ref_gpu_backward(int T, int B, int I, int H, const float *W_t, const float *R_t, const float *bw,
                     const float *br, const float *x_t, const float *dh_new, const float *h,
                     const float *v, int use_masks, const uint8_t *const *masks, float *dx, float *dW,
                     float *dR, float *dbw, float *dbr, float *dh) {
    return guarded([&] {
        const size_t C3 = size_t(H) * 3, TB = size_t(T) * B;
        DevBuf<float> dWt(W_t, C3 * I), dRt(R_t, C3 * H), dbw_in(bw, C3), dbr_in(br, C3), dxt(x_t, TB * I),
            ddh_new(dh_new, (TB + B) * H), dh_all(h, (TB + B) * H), dv(v, TB * H * 4);
        DevBuf<float> o_dx(TB * I), o_dW(size_t(I) * C3), o_dR(size_t(H) * C3), o_dbw(C3), o_dbr(C3),
            o_dh(size_t(B) * H);
        o_dx.zero(); o_dW.zero(); o_dR.zero(); o_dbw.zero(); o_dbr.zero(); o_dh.zero();
        if (!use_masks) {
            hasteGRUBackward(T, B, I, H, dWt.p, dRt.p, dbw_in.p, dbr_in.p, dxt.p, ddh_new.p, dh_all.p, dv.p,
                             blasHandle(), o_dx.p, o_dW.p, o_dR.p, o_dbw.p, o_dbr.p, o_dh.p);
        } else {
            const size_t msz[11] = {TB * I, size_t(B) * H, size_t(I) * C3, size_t(H) * C3, C3, C3,
                                    TB * C3, TB * C3, TB * C3, TB * C3, TB * H};
            std::unique_ptr<DevBuf<uint8_t>> dm[11];
            for (int k = 0; k < 11; ++k) {
                if (!masks || !masks[k]) throw std::invalid_argument("ref_gpu_backward: all masks are required");
                dm[k].reset(new DevBuf<uint8_t>(masks[k], msz[k]));
            }
            quantGRUBackward(T, B, I, H, dWt.p, dRt.p, dbw_in.p, dbr_in.p, dxt.p, ddh_new.p, dh_all.p, dv.p,
                             blasHandle(), o_dx.p, o_dW.p, o_dR.p, o_dbw.p, o_dbr.p, o_dh.p, nullptr,
                             dm[0]->p, dm[1]->p, dm[2]->p, dm[3]->p, dm[4]->p, dm[5]->p, dm[6]->p, dm[7]->p,
                             dm[8]->p, dm[9]->p, dm[10]->p);
        }
        cudaOk(cudaDeviceSynchronize(), "backward");
        o_dx.toHost(dx); o_dW.toHost(dW); o_dR.toHost(dR); o_dbw.toHost(dbw); o_dbr.toHost(dbr); o_dh.toHost(dh);
    });
}

// hasteGRUForward (src/gru_interface.cc:173): the reference's fp32 GRU on the GPU.
int ref_gpu_forward_float(int T, int B, int I, int H, const float *W, const float *R, const float *bw,
                          const float *br, const float *x, const float *h0, float *h, float *v) {
    return guarded([&] {
        const size_t C3 = size_t(H) * 3, TB = size_t(T) * B;
        DevBuf<float> dW(W, size_t(I) * C3), dR(R, size_t(H) * C3), dbw(bw, C3), dbr(br, C3),
            dx(x, TB * I), dh0(h0, size_t(B) * H), dh((TB + B) * H), dv(TB * H * 4);
        dh.zero();
        hasteGRUForward(v != nullptr, T, B, I, H, dW.p, dR.p, dbw.p, dbr.p, dx.p, dh0.p, blasHandle(),
                        dh.p, dv.p);
        cudaOk(cudaDeviceSynchronize(), "hasteGRUForward");
        dh.toHost(h);
        dv.toHost(v);
    });
}

// quantGRUForwardFP (src/gru_interface.cc:894), inference mode: the float-storage quantized
// forward.  Returns h (dequantized) and, where asked, the quantized x and weights as floats.
int ref_gpu_forward_fstorage(int T, int B, int I, int H, const float *W, const float *R,
                             const float *bw, const float *br, const float *x, const float *h0,
                             const qgru_params *p, const float *sW, const float *sR, const float *sbw,
                             const float *sbr, float *h, float *x_q_out, float *W_q_out,
                             float *R_q_out, float *bw_q_out, float *br_q_out) {
    return guarded([&] {
        GRUQuantParams q = fromPod(*p, sW, sR, sbw, sbr);
        const size_t C3 = size_t(H) * 3, TB = size_t(T) * B;
        DevBuf<float> dW(W, size_t(I) * C3), dR(R, size_t(H) * C3), dbw(bw, C3), dbr(br, C3),
            dx(x, TB * I), dh0(h0, size_t(B) * H), dh((TB + B) * H);
        DevBuf<float> qW(size_t(I) * C3), qR(size_t(H) * C3), qbw(C3), qbr(C3), qx(TB * I);
        dh.zero();
        quantGRUForwardFP(false, T, B, I, H, dW.p, dR.p, dbw.p, dbr.p, dx.p, dh0.p, q, blasHandle(),
                          dh.p, nullptr, qW.p, qR.p, qbw.p, qbr.p, qx.p, nullptr, nullptr, nullptr,
                          nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr);
        cudaOk(cudaDeviceSynchronize(), "quantGRUForwardFP");
        dh.toHost(h);
        qx.toHost(x_q_out);
        qW.toHost(W_q_out);
        qR.toHost(R_q_out);
        qbw.toHost(bw_q_out);
        qbr.toHost(br_q_out);
    });
}

// quantGRUForwardFP with is_training = true: h, v (both dequantized) and the eleven masks
// (order of qgru_train_masks; all eleven host arrays required, h0 must be given: the kernels of
// this mode write their masks without a null check, src/gru_forward_gpu_quant_fp.cu:702-712).
int ref_gpu_forward_fstorage_train(int T, int B, int I, int H, const float *W, const float *R,
                                   const float *bw, const float *br, const float *x, const float *h0,
                                   const qgru_params *p, const float *sW, const float *sR,
                                   const float *sbw, const float *sbr, float *h, float *v,
                                   uint8_t *const *masks) {
    return guarded([&] {
        if (!h0 || !masks) throw std::invalid_argument("ref_gpu_forward_fstorage_train: h0 and masks are required");
        GRUQuantParams q = fromPod(*p, sW, sR, sbw, sbr);
        const size_t C3 = size_t(H) * 3, TB = size_t(T) * B;
        DevBuf<float> dW(W, size_t(I) * C3), dR(R, size_t(H) * C3), dbw(bw, C3), dbr(br, C3),
            dx(x, TB * I), dh0(h0, size_t(B) * H), dh((TB + B) * H), dv(TB * H * 4);
        DevBuf<float> qW(size_t(I) * C3), qR(size_t(H) * C3), qbw(C3), qbr(C3), qx(TB * I);
        const size_t msz[11] = {TB * I, size_t(B) * H, size_t(I) * C3, size_t(H) * C3, C3, C3,
                                TB * C3, TB * C3, TB * C3, TB * C3, TB * H};
        std::unique_ptr<DevBuf<uint8_t>> dm[11];
        for (int k = 0; k < 11; ++k) {
            if (!masks[k]) throw std::invalid_argument("ref_gpu_forward_fstorage_train: all masks are required");
            dm[k].reset(new DevBuf<uint8_t>(msz[k]));
            dm[k]->zero();
        }
        dh.zero();
        quantGRUForwardFP(true, T, B, I, H, dW.p, dR.p, dbw.p, dbr.p, dx.p, dh0.p, q, blasHandle(), dh.p,
                          dv.p, qW.p, qR.p, qbw.p, qbr.p, qx.p, dm[0]->p, dm[1]->p, dm[2]->p, dm[3]->p,
                          dm[4]->p, dm[5]->p, dm[6]->p, dm[7]->p, dm[8]->p, dm[9]->p, dm[10]->p);
        cudaOk(cudaDeviceSynchronize(), "quantGRUForwardFP");
        dh.toHost(h);
        dv.toHost(v);
        for (int k = 0; k < 11; ++k) dm[k]->toHost(masks[k]);
    });
}

// quantGRUForwardInt with is_training = true (src/gru_interface.cc:610): h, v (dequantized) and
// the eleven masks; same conventions as ref_gpu_forward_fstorage_train.
int ref_gpu_forward_int_train(int T, int B, int I, int H, const float *W, const float *R, const float *bw,
                              const float *br, const float *x, const float *h0, const qgru_params *p,
                              const float *sW, const float *sR, const float *sbw, const float *sbr,
                              float *h, float *v, uint8_t *const *masks) {
    return guarded([&] {
        if (!h0 || !masks) throw std::invalid_argument("ref_gpu_forward_int_train: h0 and masks are required");
        GRUQuantParams q = fromPod(*p, sW, sR, sbw, sbr);
        const size_t C3 = size_t(H) * 3, TB = size_t(T) * B;
        DevBuf<float> dW(W, size_t(I) * C3), dR(R, size_t(H) * C3), dbw(bw, C3), dbr(br, C3),
            dx(x, TB * I), dh0(h0, size_t(B) * H), dh((TB + B) * H), dv(TB * H * 4);
        const size_t msz[11] = {TB * I, size_t(B) * H, size_t(I) * C3, size_t(H) * C3, C3, C3,
                                TB * C3, TB * C3, TB * C3, TB * C3, TB * H};
        std::unique_ptr<DevBuf<uint8_t>> dm[11];
        for (int k = 0; k < 11; ++k) {
            if (!masks[k]) throw std::invalid_argument("ref_gpu_forward_int_train: all masks are required");
            dm[k].reset(new DevBuf<uint8_t>(msz[k]));
            dm[k]->zero();
        }
        dh.zero();
        quantGRUForwardInt(true, T, B, I, H, dW.p, dR.p, dbw.p, dbr.p, dx.p, dh0.p, q, blasHandle(), dh.p, dv.p,
                           dm[0]->p, dm[1]->p, dm[2]->p, dm[3]->p, dm[4]->p, dm[5]->p, dm[6]->p, dm[7]->p,
                           dm[8]->p, dm[9]->p, dm[10]->p, nullptr, nullptr, nullptr, nullptr, nullptr);
        cudaOk(cudaDeviceSynchronize(), "quantGRUForwardInt");
        dh.toHost(h);
        dv.toHost(v);
        for (int k = 0; k < 11; ++k) dm[k]->toHost(masks[k]);
    });
}

// forwardWithCalibrationGPU (src/gru_interface.cc:1283), MinMax: folds one batch into `r`.
int ref_gpu_calibrate_minmax(int T, int B, int I, int H, const float *W, const float *R,
                             const float *bw, const float *br, const float *x, qgru_ranges *r,
                             float *h) {
    return guarded([&] {
        const size_t C3 = size_t(H) * 3, TB = size_t(T) * B;
        GRUQuantizationRanges g(H);
        rangesFromPod(*r, g);
        DevBuf<float> dW(W, size_t(I) * C3), dR(R, size_t(H) * C3), dbw(bw, C3), dbr(br, C3),
            dx(x, TB * I), dh((TB + B) * H), dv(TB * H * 4);
        dh.zero();
        forwardWithCalibrationGPU(false, T, B, I, H, dW.p, dR.p, dbw.p, dbr.p, dx.p, nullptr,
                                  blasHandle(), CalibrationMethod::MINMAX, &g, nullptr,
                                  OperatorQuantConfig(), dh.p, dv.p);
        cudaOk(cudaDeviceSynchronize(), "forwardWithCalibrationGPU");
        rangesToPod(g, *r);
        dh.toHost(h);
    });
}

// One GPUHistogramCollector (src/calibration_gpu.cu:820-1039) fed from host arrays.
void *ref_gpu_hist_new(int bins) {
    void *out = nullptr;
    guarded([&] { out = new GPUHistogramCollector(bins); });
    return out;
}
void ref_gpu_hist_free(void *h) { delete static_cast<GPUHistogramCollector *>(h); }
int ref_gpu_hist_collect(void *h, const float *data, size_t n) {
    return guarded([&] {
        DevBuf<float> d(data, n);
        static_cast<GPUHistogramCollector *>(h)->collect(d.p, n);
        cudaOk(cudaDeviceSynchronize(), "GPUHistogramCollector::collect");
    });
}
int ref_gpu_hist_get(void *h, float *counts, float *min_val, float *max_val, int64_t *total) {
    return guarded([&] {
        const GPUHistogram &g = static_cast<GPUHistogramCollector *>(h)->histogram();
        if (counts && g.num_bins > 0) {
            std::vector<float> c = g.to_host();
            std::memcpy(counts, c.data(), sizeof(float) * c.size());
        }
        *min_val = g.min_val;
        *max_val = g.max_val;
        *total = g.total_count;
    });
}

// The whole collector set of one GRU (GRUGPUHistogramCollectors) through the calibration forward
// (collectAllHistogramsGPU, src/histogram_calibration_utils.cu:18-123).
void *ref_gpu_histset_new(int hidden, int bins) {
    void *out = nullptr;
    guarded([&] { out = new GpuHistSet(hidden, bins); });
    return out;
}
void ref_gpu_histset_free(void *s) { delete static_cast<GpuHistSet *>(s); }
int ref_gpu_histset_calibrate(void *s, int T, int B, int I, int H, const float *W, const float *R,
                              const float *bw, const float *br, const float *x,
                              const qgru_params *p, int use_percentile) {
    return guarded([&] {
        const size_t C3 = size_t(H) * 3, TB = size_t(T) * B;
        OperatorQuantConfig cfg;
        fillConfig(*p, cfg);
        DevBuf<float> dW(W, size_t(I) * C3), dR(R, size_t(H) * C3), dbw(bw, C3), dbr(br, C3),
            dx(x, TB * I), dh((TB + B) * H), dv(TB * H * 4);
        dh.zero();
        forwardWithCalibrationGPU(false, T, B, I, H, dW.p, dR.p, dbw.p, dbr.p, dx.p, nullptr,
                                  blasHandle(),
                                  use_percentile ? CalibrationMethod::PERCENTILE : CalibrationMethod::SQNR,
                                  nullptr, &static_cast<GpuHistSet *>(s)->gpu, cfg, dh.p, dv.p);
        cudaOk(cudaDeviceSynchronize(), "forwardWithCalibrationGPU");
    });
}
int ref_gpu_histset_sync(void *s) {
    return guarded([&] {
        auto *hs = static_cast<GpuHistSet *>(s);
        hs->cpu = convertGPUHistogramsToCPU(hs->gpu);
    });
}
// valid = 0 when that collector never received data (counts untouched)
int ref_gpu_histset_get(void *s, int index, float *counts, float *min_val, float *max_val,
                        int64_t *total, int *valid) {
    return guarded([&] {
        const HistogramCollector *c = histByIndex(static_cast<GpuHistSet *>(s)->cpu, index);
        *valid = c->is_valid() ? 1 : 0;
        const Histogram &g = c->histogram();
        if (counts && *valid) std::memcpy(counts, g.counts.data(), sizeof(float) * g.counts.size());
        *min_val = g.min_val;
        *max_val = g.max_val;
        *total = g.total_count;
    });
}
// calculateGRUQuantitativeParametersFromHistograms on the synced CPU copy
int ref_gpu_histset_params(void *s, qgru_params *p, int use_percentile, float percentile, float *sW,
                           float *sR, float *sbw, float *sbr) {
    return guarded([&] {
        OperatorQuantConfig cfg;
        fillConfig(*p, cfg);
        GRUQuantParams q = calculateGRUQuantitativeParametersFromHistograms(
            static_cast<GpuHistSet *>(s)->cpu, cfg, use_percentile != 0, percentile);
        toPod(q, *p, sW, sR, sbw, sbr);
    });
}

}  // extern "C"
