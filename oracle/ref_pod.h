// ref_pod.h - TEST INFRASTRUCTURE: the POD types of include/qgru.h -> the reference's
// GRUQuantParams (include/quantize_param_types.h of the reference), shared by the two test
// drivers that are compiled against the reference's headers (ref_shim.cc, shim_driver.cc).
#pragma once
#include <cstring>

#include "quantize_param_types.h"
#include "quantize_lut_types.h"

#include "qgru.h"

namespace refpod {

inline QuantBitWidth bwOf(const qgru_op &o) { return QuantBitWidth(o.bits, o.is_unsigned != 0); }

inline void fillConfig(const qgru_params &p, OperatorQuantConfig &c) {
    c.x_ = bwOf(p.op[QGRU_OP_X]);
    c.h_ = bwOf(p.op[QGRU_OP_H]);
    c.W_ = bwOf(p.op[QGRU_OP_W]);
    c.R_ = bwOf(p.op[QGRU_OP_R]);
    c.bw_ = bwOf(p.op[QGRU_OP_BW]);
    c.br_ = bwOf(p.op[QGRU_OP_BR]);
    c.weight_ih_linear_ = bwOf(p.op[QGRU_OP_IH_LINEAR]);
    c.weight_hh_linear_ = bwOf(p.op[QGRU_OP_HH_LINEAR]);
    c.update_gate_input_ = bwOf(p.op[QGRU_OP_UPDATE_IN]);
    c.update_gate_output_ = bwOf(p.op[QGRU_OP_UPDATE_OUT]);
    c.reset_gate_input_ = bwOf(p.op[QGRU_OP_RESET_IN]);
    c.reset_gate_output_ = bwOf(p.op[QGRU_OP_RESET_OUT]);
    c.new_gate_input_ = bwOf(p.op[QGRU_OP_NEW_IN]);
    c.new_gate_output_ = bwOf(p.op[QGRU_OP_NEW_OUT]);
    c.mul_reset_hidden_ = bwOf(p.op[QGRU_OP_MUL_RESET_HIDDEN]);
    c.mul_new_contribution_ = bwOf(p.op[QGRU_OP_MUL_NEW_CONTRIB]);
    c.mul_old_contribution_ = bwOf(p.op[QGRU_OP_MUL_OLD_CONTRIB]);
    c.x_symmetric_ = p.op[QGRU_OP_X].symmetric;
    c.h_symmetric_ = p.op[QGRU_OP_H].symmetric;
    c.W_symmetric_ = p.op[QGRU_OP_W].symmetric;
    c.R_symmetric_ = p.op[QGRU_OP_R].symmetric;
    c.bw_symmetric_ = p.op[QGRU_OP_BW].symmetric;
    c.br_symmetric_ = p.op[QGRU_OP_BR].symmetric;
    c.weight_ih_linear_symmetric_ = p.op[QGRU_OP_IH_LINEAR].symmetric;
    c.weight_hh_linear_symmetric_ = p.op[QGRU_OP_HH_LINEAR].symmetric;
    c.update_gate_input_symmetric_ = p.op[QGRU_OP_UPDATE_IN].symmetric;
    c.update_gate_output_symmetric_ = p.op[QGRU_OP_UPDATE_OUT].symmetric;
    c.reset_gate_input_symmetric_ = p.op[QGRU_OP_RESET_IN].symmetric;
    c.reset_gate_output_symmetric_ = p.op[QGRU_OP_RESET_OUT].symmetric;
    c.new_gate_input_symmetric_ = p.op[QGRU_OP_NEW_IN].symmetric;
    c.new_gate_output_symmetric_ = p.op[QGRU_OP_NEW_OUT].symmetric;
    c.mul_reset_hidden_symmetric_ = p.op[QGRU_OP_MUL_RESET_HIDDEN].symmetric;
    c.mul_new_contribution_symmetric_ = p.op[QGRU_OP_MUL_NEW_CONTRIB].symmetric;
    c.mul_old_contribution_symmetric_ = p.op[QGRU_OP_MUL_OLD_CONTRIB].symmetric;
    using G = OperatorQuantConfig::QuantizationGranularity;
    c.W_granularity_ = static_cast<G>(p.granularity[0]);
    c.R_granularity_ = static_cast<G>(p.granularity[1]);
    c.bw_granularity_ = static_cast<G>(p.granularity[2]);
    c.br_granularity_ = static_cast<G>(p.granularity[3]);
    c.usePOT2_ = p.use_pot2 != 0;
}

inline QuantParam qpOf(const qgru_op &o) { return QuantParam{o.scale, o.zero_point}; }

inline void lutFromPod(const qgru_lut &in, SigmoidLUT &out) {
    std::memset(&out, 0, sizeof(out));
    for (int i = 0; i < NUM_SEGMENTS; ++i) {
        out.segments[i].q_b = in.seg[i].q_b;
        out.segments[i].n_BX_total = static_cast<int8_t>(in.seg[i].n_bx);
        out.segments[i].term_c_precomputed = in.seg[i].term_c;
        out.segments[i].threshold = in.seg[i].threshold;
    }
    out.zp_x = in.zp_x;
}

inline void channelFromPod(ChannelQuantParam &c, int hidden, int gran, const float *scales) {
    c.granularity = static_cast<OperatorQuantConfig::QuantizationGranularity>(gran);
    c.hidden = hidden;
    c.resize(hidden * 3);
    for (int i = 0; i < hidden * 3; ++i) c.channel(i) = QuantParam{scales[i], 0};
}

inline GRUQuantParams fromPod(const qgru_params &p, const float *sW, const float *sR, const float *sbw,
                       const float *sbr) {
    GRUQuantParams q;
    fillConfig(p, q.bitwidth_config_);
    q.hidden_ = p.hidden;
    q.x_ = qpOf(p.op[QGRU_OP_X]);
    q.h_ = qpOf(p.op[QGRU_OP_H]);
    channelFromPod(q.W_, p.hidden, p.granularity[0], sW);
    channelFromPod(q.R_, p.hidden, p.granularity[1], sR);
    channelFromPod(q.bw_, p.hidden, p.granularity[2], sbw);
    channelFromPod(q.br_, p.hidden, p.granularity[3], sbr);
    q.weight_ih_linear_ = qpOf(p.op[QGRU_OP_IH_LINEAR]);
    q.weight_hh_linear_ = qpOf(p.op[QGRU_OP_HH_LINEAR]);
    q.update_gate_input_ = qpOf(p.op[QGRU_OP_UPDATE_IN]);
    q.update_gate_output_ = qpOf(p.op[QGRU_OP_UPDATE_OUT]);
    q.reset_gate_input_ = qpOf(p.op[QGRU_OP_RESET_IN]);
    q.reset_gate_output_ = qpOf(p.op[QGRU_OP_RESET_OUT]);
    q.new_gate_input_ = qpOf(p.op[QGRU_OP_NEW_IN]);
    q.new_gate_output_ = qpOf(p.op[QGRU_OP_NEW_OUT]);
    q.mul_reset_hidden_ = qpOf(p.op[QGRU_OP_MUL_RESET_HIDDEN]);
    q.mul_new_contribution_ = qpOf(p.op[QGRU_OP_MUL_NEW_CONTRIB]);
    q.mul_old_contribution_ = qpOf(p.op[QGRU_OP_MUL_OLD_CONTRIB]);
    lutFromPod(p.lut[QGRU_LUT_UPDATE], q.sigmoid_update_gate_lut_);
    lutFromPod(p.lut[QGRU_LUT_RESET], q.sigmoid_reset_gate_lut_);
    lutFromPod(p.lut[QGRU_LUT_NEW], q.tanh_new_gate_lut_);
    return q;
}

}  // namespace refpod
