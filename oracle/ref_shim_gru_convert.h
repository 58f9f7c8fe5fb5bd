// TEST INFRASTRUCTURE - not part of the shipped library.
//
// Conversions between the flat C structs of include/rxmet_b200.h and the reference's C++ parameter
// types, shared by the two adapters around the reference's sources (ref_shim_gru.cc: its CPU build,
// ref_shim_gru_cuda.cu: its CUDA build).  Nothing of the reference is copied here.
#pragma once

#include "gru_host.h"          // reference: GRUQuantParams, generate_piecewise_linear_lut_to_params
#include "rxmet_b200.h"

namespace refshim {

inline QuantBitWidth bwOf(const rxmet_gru_quant_config &c, int op) {
    return QuantBitWidth(c.bits[op], c.is_unsigned[op] != 0);
}

inline OperatorQuantConfig toRefConfig(const rxmet_gru_quant_config &c) {
    OperatorQuantConfig r;
    QuantBitWidth *bw[RXMET_GRU_NUM_OPS] = {
        &r.x_, &r.h_, &r.W_, &r.R_, &r.bw_, &r.br_, &r.weight_ih_linear_, &r.weight_hh_linear_,
        &r.update_gate_input_, &r.update_gate_output_, &r.reset_gate_input_, &r.reset_gate_output_,
        &r.new_gate_input_, &r.new_gate_output_, &r.mul_reset_hidden_,
        &r.mul_old_contribution_, &r.mul_new_contribution_};
    bool *sym[RXMET_GRU_NUM_OPS] = {
        &r.x_symmetric_, &r.h_symmetric_, &r.W_symmetric_, &r.R_symmetric_, &r.bw_symmetric_,
        &r.br_symmetric_, &r.weight_ih_linear_symmetric_, &r.weight_hh_linear_symmetric_,
        &r.update_gate_input_symmetric_, &r.update_gate_output_symmetric_,
        &r.reset_gate_input_symmetric_, &r.reset_gate_output_symmetric_,
        &r.new_gate_input_symmetric_, &r.new_gate_output_symmetric_,
        &r.mul_reset_hidden_symmetric_, &r.mul_old_contribution_symmetric_,
        &r.mul_new_contribution_symmetric_};
    for (int i = 0; i < RXMET_GRU_NUM_OPS; ++i) {
        *bw[i] = bwOf(c, i);
        *sym[i] = c.symmetric[i] != 0;
    }
    r.W_granularity_ = static_cast<OperatorQuantConfig::QuantizationGranularity>(c.W_granularity);
    r.R_granularity_ = static_cast<OperatorQuantConfig::QuantizationGranularity>(c.R_granularity);
    r.bw_granularity_ = static_cast<OperatorQuantConfig::QuantizationGranularity>(c.bw_granularity);
    r.br_granularity_ = static_cast<OperatorQuantConfig::QuantizationGranularity>(c.br_granularity);
    r.usePOT2_ = c.use_pot2 != 0;
    r.pot_scale_method_ = static_cast<PotScaleMethod>(c.pot_scale_method);
    r.pot_scale_tolerance_ = c.pot_scale_tolerance;
    return r;
}

// Same reconstruction the reference's Python binding performs in
// GRUQuantParamsPy::to_cpp (gru_interface_binding.cc:1261-1316).
inline GRUQuantParams toRefParams(const rxmet_gru_quant_params &p) {
    GRUQuantParams r;
    r.hidden_ = p.hidden;
    r.bitwidth_config_ = toRefConfig(p.config);
    auto qp = [&](int op) { return QuantParam{p.scale[op], p.zero_point[op]}; };
    r.x_ = qp(RXMET_GRU_X);
    r.h_ = qp(RXMET_GRU_H);
    r.weight_ih_linear_ = qp(RXMET_GRU_WEIGHT_IH_LINEAR);
    r.weight_hh_linear_ = qp(RXMET_GRU_WEIGHT_HH_LINEAR);
    r.update_gate_input_ = qp(RXMET_GRU_UPDATE_GATE_INPUT);
    r.update_gate_output_ = qp(RXMET_GRU_UPDATE_GATE_OUTPUT);
    r.reset_gate_input_ = qp(RXMET_GRU_RESET_GATE_INPUT);
    r.reset_gate_output_ = qp(RXMET_GRU_RESET_GATE_OUTPUT);
    r.new_gate_input_ = qp(RXMET_GRU_NEW_GATE_INPUT);
    r.new_gate_output_ = qp(RXMET_GRU_NEW_GATE_OUTPUT);
    r.mul_reset_hidden_ = qp(RXMET_GRU_MUL_RESET_HIDDEN);
    r.mul_old_contribution_ = qp(RXMET_GRU_MUL_OLD_CONTRIBUTION);
    r.mul_new_contribution_ = qp(RXMET_GRU_MUL_NEW_CONTRIBUTION);
    auto fill = [&](ChannelQuantParam &out, int gran, const float *scales) {
        out.hidden = p.hidden;
        out.resize(3 * p.hidden);
        out.granularity = static_cast<OperatorQuantConfig::QuantizationGranularity>(gran);
        for (int c = 0; c < 3 * p.hidden; ++c) out.channel(c) = QuantParam{scales[c], 0};
    };
    fill(r.W_, p.config.W_granularity, p.scale_W);
    fill(r.R_, p.config.R_granularity, p.scale_R);
    fill(r.bw_, p.config.bw_granularity, p.scale_bw);
    fill(r.br_, p.config.br_granularity, p.scale_br);
    generate_piecewise_linear_lut_to_params(r);
    return r;
}

}  // namespace refshim
