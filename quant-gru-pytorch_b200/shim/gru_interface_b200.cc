// gru_interface_b200.cc - the reference-side binding of libqgru_b200.so.
//
// This file is compiled AGAINST THE REFERENCE'S HEADERS (include/gru_interface.h,
// include/quantize_param_types.h of CX9898/quant-gru-pytorch) and defines the three integer
// forward entry points with exactly the reference's signatures:
//
//   quantGRUForwardInt32   include/gru_interface.h:389   (src/gru_interface.cc:551)
//   quantGRUForwardInt     include/gru_interface.h:266   (src/gru_interface.cc:610)
//   quantGRUForwardIntIO   include/gru_interface.h:305   (src/gru_interface.cc:736)
//
// Each marshals GRUQuantParams into the POD types of include/qgru.h, calls the C ABI on the
// current CUDA device and turns a status code back into the exception the reference throws.  A
// maintainer of the reference drops it in place of those three function bodies (the other
// functions of src/gru_interface.cc stay) and links libqgru_b200.so.
//
// Built into a library of its own, the definitions sit in namespace QGRU_SHIM_NAMESPACE when
// that macro is set, so that a test can link them beside the reference's own definitions of
// the same names and hold one against the other.
#include <cuda_runtime.h>

#include <map>
#include <mutex>
#include <stdexcept>
#include <string>
#include <tuple>
#include <vector>

#include "gru_interface.h"          // the reference's
#include "quantize_param_types.h"   // the reference's

#include "qgru.h"

namespace {

struct Marshalled {
    qgru_params pod{};
    std::vector<float> scale[4];   // W, R, bw, br: one scale per output channel
};

void put(qgru_op &o, const QuantParam &q, const QuantBitWidth &bw, bool symmetric) {
    o.scale = q.scale;
    o.zero_point = q.zero_point;
    o.bits = bw.bits_;
    o.is_unsigned = bw.is_unsigned_ ? 1 : 0;
    o.symmetric = symmetric ? 1 : 0;
    o.reserved = 0;
}

void put_lut(qgru_lut &out, const SigmoidLUT &in) {
    for (int i = 0; i < QGRU_LUT_SEGMENTS; ++i) {
        out.seg[i].q_b = in.segments[i].q_b;
        out.seg[i].n_bx = in.segments[i].n_BX_total;
        out.seg[i].term_c = in.segments[i].term_c_precomputed;
        out.seg[i].threshold = in.segments[i].threshold;
    }
    out.zp_x = in.zp_x;
    out.reserved[0] = out.reserved[1] = out.reserved[2] = 0;
}

// GRUQuantParams (include/quantize_param_types.h:96-146) -> qgru_params + four scale arrays.
// The per-channel arrays are the reference's "only authority" for weight scales whatever the
// granularity (per-tensor / per-gate values are already broadcast into them,
// src/gru_interface.cc:83-103).
Marshalled marshal(const GRUQuantParams &q, int hidden) {
    if (q.hidden_ != hidden) throw std::invalid_argument("GRUQuantParams.hidden_ does not match hidden_size");
    Marshalled m;
    const OperatorQuantConfig &c = q.bitwidth_config_;
    m.pod.hidden = hidden;
    m.pod.use_pot2 = c.usePOT2_ ? 1 : 0;
    put(m.pod.op[QGRU_OP_X], q.x_, c.x_, c.x_symmetric_);
    put(m.pod.op[QGRU_OP_H], q.h_, c.h_, c.h_symmetric_);
    const ChannelQuantParam *ch[4] = {&q.W_, &q.R_, &q.bw_, &q.br_};
    const QuantBitWidth *chbw[4] = {&c.W_, &c.R_, &c.bw_, &c.br_};
    const bool chsym[4] = {c.W_symmetric_, c.R_symmetric_, c.bw_symmetric_, c.br_symmetric_};
    const int chop[4] = {QGRU_OP_W, QGRU_OP_R, QGRU_OP_BW, QGRU_OP_BR};
    for (int k = 0; k < 4; ++k) {
        if ((int)ch[k]->size() != 3 * hidden) throw std::invalid_argument("per-channel scale array is not 3 * hidden long");
        put(m.pod.op[chop[k]], ch[k]->tensor(), *chbw[k], chsym[k]);
        m.pod.op[chop[k]].zero_point = 0;
        m.pod.granularity[k] = (int)ch[k]->granularity;
        m.scale[k].resize(3 * hidden);
        for (int i = 0; i < 3 * hidden; ++i) m.scale[k][i] = ch[k]->channel(i).scale;
    }
    put(m.pod.op[QGRU_OP_IH_LINEAR], q.weight_ih_linear_, c.weight_ih_linear_, c.weight_ih_linear_symmetric_);
    put(m.pod.op[QGRU_OP_HH_LINEAR], q.weight_hh_linear_, c.weight_hh_linear_, c.weight_hh_linear_symmetric_);
    put(m.pod.op[QGRU_OP_UPDATE_IN], q.update_gate_input_, c.update_gate_input_, c.update_gate_input_symmetric_);
    put(m.pod.op[QGRU_OP_UPDATE_OUT], q.update_gate_output_, c.update_gate_output_, c.update_gate_output_symmetric_);
    put(m.pod.op[QGRU_OP_RESET_IN], q.reset_gate_input_, c.reset_gate_input_, c.reset_gate_input_symmetric_);
    put(m.pod.op[QGRU_OP_RESET_OUT], q.reset_gate_output_, c.reset_gate_output_, c.reset_gate_output_symmetric_);
    put(m.pod.op[QGRU_OP_NEW_IN], q.new_gate_input_, c.new_gate_input_, c.new_gate_input_symmetric_);
    put(m.pod.op[QGRU_OP_NEW_OUT], q.new_gate_output_, c.new_gate_output_, c.new_gate_output_symmetric_);
    put(m.pod.op[QGRU_OP_MUL_RESET_HIDDEN], q.mul_reset_hidden_, c.mul_reset_hidden_, c.mul_reset_hidden_symmetric_);
    put(m.pod.op[QGRU_OP_MUL_NEW_CONTRIB], q.mul_new_contribution_, c.mul_new_contribution_,
        c.mul_new_contribution_symmetric_);
    put(m.pod.op[QGRU_OP_MUL_OLD_CONTRIB], q.mul_old_contribution_, c.mul_old_contribution_,
        c.mul_old_contribution_symmetric_);
    put_lut(m.pod.lut[QGRU_LUT_UPDATE], q.sigmoid_update_gate_lut_);
    put_lut(m.pod.lut[QGRU_LUT_RESET], q.sigmoid_reset_gate_lut_);
    put_lut(m.pod.lut[QGRU_LUT_NEW], q.tanh_new_gate_lut_);
    return m;
}

// One library handle per (device, input size, hidden size), created on first use and kept for
// the life of the process: the reference's entry points are stateless, the library's packed
// weights and workspace live in the handle.  The reference's binding is not thread-safe (one
// global cuBLAS handle); this cache takes a lock per call, which keeps that contract.
std::mutex g_mu;
std::map<std::tuple<int, int, int>, qgru_handle *> g_handles;

qgru_handle *handle_for(int I, int H) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) throw std::runtime_error("cudaGetDevice failed");
    const auto key = std::make_tuple(dev, I, H);
    auto it = g_handles.find(key);
    if (it != g_handles.end()) return it->second;
    qgru_handle *h = nullptr;
    const int st = qgru_create(&h, dev, I, H);
    if (st != QGRU_OK) throw std::runtime_error(std::string("qgru_create: ") + qgru_status_string(st));
    g_handles[key] = h;
    return h;
}

// Status -> the exception types the reference throws: std::invalid_argument for argument
// problems (ensureSymmetricWeightBiasConfig, src/gru_interface.cc:26-32), std::runtime_error for
// everything found after the device synchronisation (:594-602).
void check(qgru_handle *h, int st, const char *what) {
    if (st == QGRU_OK) return;
    const std::string msg = std::string(what) + ": " + qgru_status_string(st) + " (" + qgru_last_error(h) + ")";
    if (st == QGRU_ERR_BAD_ARG || st == QGRU_ERR_UNSUPPORTED || st == QGRU_ERR_RANGE) throw std::invalid_argument(msg);
    throw std::runtime_error(msg);
}

void set_params(qgru_handle *h, const GRUQuantParams &qp, int H) {
    const Marshalled m = marshal(qp, H);
    check(h, qgru_set_params(h, &m.pod, m.scale[0].data(), m.scale[1].data(), m.scale[2].data(), m.scale[3].data()),
          "qgru_set_params");
}

}  // namespace

#ifdef QGRU_SHIM_NAMESPACE
namespace QGRU_SHIM_NAMESPACE {
#endif

void quantGRUForwardInt32(bool is_training, int time_steps, int batch_size, int input_size, int hidden_size,
                          const int32_t *W_q, const int32_t *R_q, const int32_t *bw_q, const int32_t *br_q,
                          const int32_t *x_q, const int32_t *h0_q, const GRUQuantParams &quant_params,
                          const cublasHandle_t &, int32_t *h_q, int32_t *v_q, uint8_t *weight_ih_linear_mask,
                          uint8_t *weight_hh_linear_mask, uint8_t *gate_input_mask, uint8_t *gate_output_mask,
                          uint8_t *h_mask) {
    std::lock_guard<std::mutex> lock(g_mu);
    qgru_handle *h = handle_for(input_size, hidden_size);
    set_params(h, quant_params, hidden_size);
    check(h, qgru_set_weights_i32(h, W_q, R_q, bw_q, br_q, nullptr), "qgru_set_weights_i32");
    if (is_training && v_q) {   // the gate buffer and the five clamp masks (null members are skipped)
        const qgru_masks mk = {weight_ih_linear_mask, weight_hh_linear_mask, gate_input_mask, gate_output_mask, h_mask};
        check(h, qgru_forward_i32_train(h, time_steps, batch_size, x_q, h0_q, h_q, v_q, &mk, 0, nullptr),
              "qgru_forward_i32_train");
    } else {
        check(h, qgru_forward_i32(h, time_steps, batch_size, x_q, h0_q, h_q, 0, nullptr), "qgru_forward_i32");
    }
    check(h, qgru_synchronize(h, nullptr), "qgru_synchronize");   // the reference synchronises and throws here too
}

void quantGRUForwardInt(bool is_training, const int time_steps, const int batch_size, const int input_size,
                        const int hidden_size, const float *W, const float *R, const float *bw, const float *br,
                        const float *x, const float *h0, const GRUQuantParams &quant_parms, const cublasHandle_t &,
                        float *h_out, float *v, uint8_t *x_mask, uint8_t *h0_mask, uint8_t *W_mask, uint8_t *R_mask,
                        uint8_t *bw_mask, uint8_t *br_mask, uint8_t *weight_ih_linear_mask,
                        uint8_t *weight_hh_linear_mask, uint8_t *gate_input_mask, uint8_t *gate_output_mask,
                        uint8_t *h_mask, int32_t *W_q_out, int32_t *R_q_out, int32_t *bw_q_out, int32_t *br_q_out,
                        int32_t *x_q_out) {
    std::lock_guard<std::mutex> lock(g_mu);
    qgru_handle *h = handle_for(input_size, hidden_size);
    set_params(h, quant_parms, hidden_size);
    check(h, qgru_set_weights_f32(h, W, R, bw, br, nullptr), "qgru_set_weights_f32");
    if (is_training && v) {
        const qgru_train_masks mk = {x_mask, h0_mask, W_mask, R_mask, bw_mask, br_mask, weight_ih_linear_mask,
                                     weight_hh_linear_mask, gate_input_mask, gate_output_mask, h_mask};
        check(h, qgru_forward_f32_train(h, time_steps, batch_size, W, R, bw, br, x, h0, h_out, v, x_q_out, &mk, 0,
                                        nullptr), "qgru_forward_f32_train");
    } else {
        check(h, qgru_forward_f32(h, time_steps, batch_size, x, h0, h_out, x_q_out, 0, nullptr), "qgru_forward_f32");
    }
    if (W_q_out || R_q_out || bw_q_out || br_q_out)
        check(h, qgru_get_weights_i32(h, W_q_out, R_q_out, bw_q_out, br_q_out, nullptr), "qgru_get_weights_i32");
    check(h, qgru_synchronize(h, nullptr), "qgru_synchronize");
}

void quantGRUForwardIntIO(bool is_training, const int time_steps, const int batch_size, const int input_size,
                          const int hidden_size, const float *W, const float *R, const float *bw, const float *br,
                          const int32_t *x_q, const int32_t *h0_q, const GRUQuantParams &quant_parms,
                          const cublasHandle_t &, int32_t *h_q, int32_t *v_q, uint8_t *, uint8_t *, uint8_t *,
                          uint8_t *, uint8_t *weight_ih_linear_mask, uint8_t *weight_hh_linear_mask,
                          uint8_t *gate_input_mask, uint8_t *gate_output_mask, uint8_t *h_mask) {
    // the four weight masks are not produced on this path: the integer-in / integer-out entry is
    // the inference entry of QuantGRU.forward_quantized (pytorch/quant_gru.py:2318), which passes none
    std::lock_guard<std::mutex> lock(g_mu);
    qgru_handle *h = handle_for(input_size, hidden_size);
    set_params(h, quant_parms, hidden_size);
    check(h, qgru_set_weights_f32(h, W, R, bw, br, nullptr), "qgru_set_weights_f32");
    if (is_training && v_q) {
        const qgru_masks mk = {weight_ih_linear_mask, weight_hh_linear_mask, gate_input_mask, gate_output_mask, h_mask};
        check(h, qgru_forward_i32_train(h, time_steps, batch_size, x_q, h0_q, h_q, v_q, &mk, 0, nullptr),
              "qgru_forward_i32_train");
    } else {
        check(h, qgru_forward_i32(h, time_steps, batch_size, x_q, h0_q, h_q, 0, nullptr), "qgru_forward_i32");
    }
    check(h, qgru_synchronize(h, nullptr), "qgru_synchronize");
}

#ifdef QGRU_SHIM_NAMESPACE
}  // namespace QGRU_SHIM_NAMESPACE
#endif
