// extern "C" surface of the QuantLSTM part (declared in include/rxmet_b200_lstm.h).  Validates
// arguments, turns exceptions into status codes and hands over to the kernel launchers.
#include <cuda_runtime.h>

#include <cstring>

#include "common.h"
#include "lstm_kernels.h"
#include "lstm_params.h"
#include "rxmet_b200_lstm.h"

using namespace rxmet;

namespace {

#define RXMET_PTR(p) RXMET_REQUIRE((p) != nullptr, #p " must not be null")

void checkDims(int T, int B, int I, int H) {
    RXMET_REQUIRE(T > 0 && B > 0 && I > 0 && H > 0, "LSTM dimensions must be positive (T=%d B=%d I=%d H=%d)", T, B, I, H);
    RXMET_REQUIRE(static_cast<long long>(T) * B * 4LL * H < (1LL << 40), "LSTM problem too large");
}

void checkPairs(const float *bias_ih, const float *bias_hh, const float *h0, const float *c0) {
    RXMET_REQUIRE((bias_ih == nullptr) == (bias_hh == nullptr), "bias_ih and bias_hh are given together or not at all");
    RXMET_REQUIRE((h0 == nullptr) == (c0 == nullptr), "h0 and c0 are given together or not at all");
}

void runFloat(int T, int B, int I, int H, const float *weight_ih, const float *weight_hh, const float *bias_ih,
              const float *bias_hh, const float *x, const float *h0, const float *c0, float *output, float *final_hidden,
              float *final_cell, const rxmet_lstm_trace *trace, float *stats, void *ws, size_t wsBytes, void *stream) {
    checkDims(T, B, I, H);
    checkPairs(bias_ih, bias_hh, h0, c0);
    RXMET_PTR(weight_ih); RXMET_PTR(weight_hh); RXMET_PTR(x); RXMET_PTR(output); RXMET_PTR(final_hidden); RXMET_PTR(final_cell);
    lstm::ForwardFloatCall call{};
    call.T = T; call.B = B; call.I = I; call.H = H;
    call.weightIh = weight_ih; call.weightHh = weight_hh; call.biasIh = bias_ih; call.biasHh = bias_hh;
    call.x = x; call.h0 = h0; call.c0 = c0;
    call.output = output; call.finalHidden = final_hidden; call.finalCell = final_cell;
    call.trace = trace; call.stats = stats;
    lstm::forwardFloat(call, ws, wsBytes, static_cast<cudaStream_t>(stream));
}

lstm::Dequant gridOfPoint(const rxmet_lstm_quant_params &p, int op) {
    return {p.scale[op], static_cast<float>(p.zero_point[op])};
}

}  // namespace

extern "C" {

int rxmet_lstm_default_config(rxmet_lstm_quant_config *config) {
    return guarded([&] {
        RXMET_PTR(config);
        lstm::defaultConfig(config);
    });
}

int rxmet_lstm_ranges_reset(rxmet_lstm_ranges *ranges, int hidden_size) {
    return guarded([&] {
        RXMET_PTR(ranges);
        RXMET_REQUIRE(hidden_size > 0, "hidden_size must be positive");
        lstm::rangesReset(ranges, hidden_size);
    });
}

int rxmet_lstm_params_from_ranges(const rxmet_lstm_quant_config *config, const rxmet_lstm_ranges *ranges, int input_size,
                                  int hidden_size, int bias_enabled, float *weight_ih_scale, float *weight_hh_scale,
                                  float *bias_ih_scale, float *bias_hh_scale, rxmet_lstm_quant_params *params) {
    return guarded([&] {
        RXMET_PTR(config); RXMET_PTR(ranges); RXMET_PTR(params); RXMET_PTR(weight_ih_scale); RXMET_PTR(weight_hh_scale);
        RXMET_REQUIRE(!bias_enabled || (bias_ih_scale && bias_hh_scale), "bias scale arrays missing");
        lstm::paramsFromRanges(*config, *ranges, input_size, hidden_size, bias_enabled != 0, weight_ih_scale,
                               weight_hh_scale, bias_ih_scale, bias_hh_scale, params);
    });
}

int rxmet_lstm_derive_execution(const rxmet_lstm_quant_params *params, int require_exact_accumulation,
                                rxmet_lstm_execution *execution) {
    return guarded([&] {
        RXMET_PTR(params); RXMET_PTR(execution);
        lstm::deriveExecution(*params, require_exact_accumulation != 0, execution);
    });
}

size_t rxmet_lstm_workspace_bytes(int op, int T, int B, int I, int H) {
    if (T <= 0 || B <= 0 || I <= 0 || H <= 0) return 0;
    switch (op) {
        case 0: return lstm::forwardFloatWorkspaceBytes(T, B, I, H);
        case 1: return lstm::forwardQuantWorkspaceBytes(T, B, I, H);
        case 2: return lstm::backwardWorkspaceBytes(T, B, I, H);
        case 3: return lstm::histCalibrationWorkspaceBytes(T, B, I, H);
        default: return 0;
    }
}

int rxmet_lstm_forward_float(int T, int B, int I, int H, const float *weight_ih, const float *weight_hh,
                             const float *bias_ih, const float *bias_hh, const float *x, const float *h0, const float *c0,
                             float *output, float *final_hidden, float *final_cell, const rxmet_lstm_trace *trace,
                             void *workspace, size_t workspace_bytes, void *stream) {
    return guarded([&] {
        runFloat(T, B, I, H, weight_ih, weight_hh, bias_ih, bias_hh, x, h0, c0, output, final_hidden, final_cell, trace,
                 nullptr, workspace, workspace_bytes, stream);
    });
}

size_t rxmet_lstm_stats_floats(int H) { return H > 0 ? lstm::statsFloats(H) : 0; }

int rxmet_lstm_forward_calibrate_stats(int T, int B, int I, int H, const float *weight_ih, const float *weight_hh,
                                       const float *bias_ih, const float *bias_hh, const float *x, const float *h0,
                                       const float *c0, float *output, float *final_hidden, float *final_cell,
                                       float *stats_dev, void *workspace, size_t workspace_bytes, void *stream) {
    return guarded([&] {
        RXMET_PTR(stats_dev);
        runFloat(T, B, I, H, weight_ih, weight_hh, bias_ih, bias_hh, x, h0, c0, output, final_hidden, final_cell, nullptr,
                 stats_dev, workspace, workspace_bytes, stream);
    });
}

int rxmet_lstm_ranges_fold_stats(rxmet_lstm_ranges *ranges, const float *stats_host, int H, int bias_enabled) {
    return guarded([&] {
        RXMET_PTR(ranges); RXMET_PTR(stats_host);
        RXMET_REQUIRE(H > 0, "hidden size must be positive");
        for (int s = 0; s < (bias_enabled ? 4 : 2); ++s)
            RXMET_REQUIRE(ranges->channel_min[s] && ranges->channel_max[s], "per-channel range arrays missing");
        lstm::foldStats(ranges, stats_host, H, bias_enabled != 0);
    });
}

int rxmet_lstm_forward_quantized(int T, int B, int I, int H, const float *weight_ih, const float *weight_hh,
                                 const float *bias_ih, const float *bias_hh, const float *x, const float *h0,
                                 const float *c0, const rxmet_lstm_quant_params *params, int require_exact_accumulation,
                                 float *output, float *final_hidden, float *final_cell,
                                 const rxmet_lstm_trace *checkpoints, const rxmet_lstm_masters *masters, void *workspace,
                                 size_t workspace_bytes, void *stream) {
    return guarded([&] {
        checkDims(T, B, I, H);
        checkPairs(bias_ih, bias_hh, h0, c0);
        RXMET_PTR(params); RXMET_PTR(weight_ih); RXMET_PTR(weight_hh); RXMET_PTR(x); RXMET_PTR(output);
        RXMET_PTR(final_hidden); RXMET_PTR(final_cell);
        RXMET_REQUIRE(params->input_size == I && params->hidden_size == H,
                      "quantization parameters were made for input_size=%d hidden_size=%d, call has I=%d H=%d",
                      params->input_size, params->hidden_size, I, H);
        RXMET_REQUIRE((params->bias_enabled != 0) == (bias_ih != nullptr), "quantization parameters and call disagree on bias");
        const auto exec = lstm::deriveExec(*params, require_exact_accumulation != 0);
        lstm::ForwardQuantCall call{};
        call.T = T; call.B = B; call.I = I; call.H = H;
        call.weightIh = weight_ih; call.weightHh = weight_hh; call.biasIh = bias_ih; call.biasHh = bias_hh;
        call.x = x; call.h0 = h0; call.c0 = c0;
        call.output = output; call.finalHidden = final_hidden; call.finalCell = final_cell;
        call.checkpoints = checkpoints; call.masters = masters;
        lstm::forwardQuant(call, *exec, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
    });
}

int rxmet_lstm_backward_float(int T, int B, int I, int H, const float *weight_ih, const float *weight_hh, const float *x,
                              const float *h0, const float *c0, const float *gate_outputs, const float *cell_states,
                              const float *cell_tanh_outputs, const float *hidden_outputs, const float *grad_output,
                              const float *grad_final_hidden, const float *grad_final_cell,
                              const rxmet_lstm_backward_masks *masks, const rxmet_lstm_gradients *gradients,
                              void *workspace, size_t workspace_bytes, void *stream) {
    return guarded([&] {
        checkDims(T, B, I, H);
        RXMET_PTR(weight_ih); RXMET_PTR(weight_hh); RXMET_PTR(x); RXMET_PTR(gate_outputs); RXMET_PTR(cell_states);
        RXMET_PTR(cell_tanh_outputs); RXMET_PTR(hidden_outputs); RXMET_PTR(grad_output); RXMET_PTR(grad_final_hidden);
        RXMET_PTR(grad_final_cell); RXMET_PTR(gradients);
        RXMET_PTR(gradients->input); RXMET_PTR(gradients->weight_ih); RXMET_PTR(gradients->weight_hh);
        RXMET_PTR(gradients->initial_hidden); RXMET_PTR(gradients->initial_cell);
        RXMET_REQUIRE((h0 == nullptr) == (c0 == nullptr), "h0 and c0 are given together or not at all");
        lstm::BackwardCall call{};
        call.T = T; call.B = B; call.I = I; call.H = H;
        call.weightIh = weight_ih; call.weightHh = weight_hh; call.x = x; call.h0 = h0; call.c0 = c0;
        call.gateOutputs = gate_outputs; call.cellStates = cell_states; call.cellTanhOutputs = cell_tanh_outputs;
        call.hiddenOutputs = hidden_outputs; call.gradOutput = grad_output; call.gradFinalHidden = grad_final_hidden;
        call.gradFinalCell = grad_final_cell; call.masks = masks; call.grads = *gradients;
        lstm::backward(call, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
    });
}

int rxmet_lstm_backward_qat(int T, int B, int I, int H, const rxmet_lstm_quant_params *params, const float *q_weight_ih,
                            const float *q_weight_hh, const float *q_x, const float *q_h0, const float *q_c0,
                            const float *q_gate_outputs, const float *q_cell_states, const float *q_cell_tanh_outputs,
                            const float *q_hidden_outputs, const float *grad_output, const float *grad_final_hidden,
                            const float *grad_final_cell, const rxmet_lstm_backward_masks *masks,
                            const rxmet_lstm_gradients *gradients, void *workspace, size_t workspace_bytes, void *stream) {
    return guarded([&] {
        checkDims(T, B, I, H);
        RXMET_PTR(params); RXMET_PTR(q_weight_ih); RXMET_PTR(q_weight_hh); RXMET_PTR(q_x); RXMET_PTR(q_h0); RXMET_PTR(q_c0);
        RXMET_PTR(q_gate_outputs); RXMET_PTR(q_cell_states); RXMET_PTR(q_cell_tanh_outputs); RXMET_PTR(q_hidden_outputs);
        RXMET_PTR(grad_output); RXMET_PTR(grad_final_hidden); RXMET_PTR(grad_final_cell); RXMET_PTR(gradients);
        RXMET_PTR(gradients->input); RXMET_PTR(gradients->weight_ih); RXMET_PTR(gradients->weight_hh);
        RXMET_PTR(gradients->initial_hidden); RXMET_PTR(gradients->initial_cell);
        RXMET_REQUIRE(params->input_size == I && params->hidden_size == H, "quantization parameters do not match the call");
        RXMET_PTR(params->weight_ih_scale); RXMET_PTR(params->weight_hh_scale);
        lstm::BackwardCall call{};
        call.T = T; call.B = B; call.I = I; call.H = H;
        call.weightIh = q_weight_ih; call.weightHh = q_weight_hh; call.x = q_x; call.h0 = q_h0; call.c0 = q_c0;
        call.gateOutputs = q_gate_outputs; call.cellStates = q_cell_states; call.cellTanhOutputs = q_cell_tanh_outputs;
        call.hiddenOutputs = q_hidden_outputs; call.gradOutput = grad_output; call.gradFinalHidden = grad_final_hidden;
        call.gradFinalCell = grad_final_cell; call.masks = masks; call.grads = *gradients;
        call.quantized = true;
        call.dqX = gridOfPoint(*params, RXMET_LSTM_INPUT);
        call.dqH = gridOfPoint(*params, RXMET_LSTM_OUTPUT);
        call.dqC = gridOfPoint(*params, RXMET_LSTM_CELL_STATE);
        for (int g = 0; g < 4; ++g) call.dqGate[g] = gridOfPoint(*params, RXMET_LSTM_INPUT_GATE_OUTPUT + g);
        call.dqTanh = gridOfPoint(*params, RXMET_LSTM_CELL_TANH_OUTPUT);
        call.weightIhScale = params->weight_ih_scale;
        call.weightHhScale = params->weight_hh_scale;
        call.codesFitTensorPath = params->config.bitwidth[RXMET_LSTM_INPUT] <= 8 && params->config.bitwidth[RXMET_LSTM_OUTPUT] <= 8;
        call.codesFitTwoTerms = params->config.bitwidth[RXMET_LSTM_INPUT] <= 16 && params->config.bitwidth[RXMET_LSTM_OUTPUT] <= 16;
        call.weightCodesFitBf16 = params->config.bitwidth[RXMET_LSTM_WEIGHT_HH] <= 8;
        call.weightIhCodesFitBf16 = params->config.bitwidth[RXMET_LSTM_WEIGHT_IH] <= 8;
        lstm::backward(call, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
    });
}

}  // extern "C"
