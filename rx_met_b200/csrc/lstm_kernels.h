// Launchers of the QuantLSTM kernels (declarations shared by the C ABI layer).
#pragma once

#include <cuda_runtime.h>

#include "lstm_params.h"

namespace rxmet {
namespace lstm {

struct ForwardFloatCall {
    int T, B, I, H;
    const float *weightIh, *weightHh, *biasIh, *biasHh, *x, *h0, *c0;
    float *output, *finalHidden, *finalCell;
    const rxmet_lstm_trace *trace;  // optional
    float *stats;                   // optional packed min/max statistics (device)
};
size_t forwardFloatWorkspaceBytes(int T, int B, int I, int H);
void forwardFloat(const ForwardFloatCall &call, void *workspace, size_t workspaceBytes, cudaStream_t stream);

// Histogram calibration: float forward of one batch that updates ranges and histogram collectors.
size_t histCalibrationWorkspaceBytes(int T, int B, int I, int H);
void forwardCalibrateHist(const ForwardFloatCall &call, const rxmet_lstm_quant_config &config, rxmet_lstm_ranges *ranges,
                          rxmet_lstm_histograms *hists, void *workspace, size_t workspaceBytes, cudaStream_t stream,
                          const rxmet_exchange *exchange);
void paramsFromHistograms(const rxmet_lstm_quant_config &config, const rxmet_lstm_ranges &observed,
                          const rxmet_lstm_histograms &hists, int method, float percentile, int inputSize, int hidden,
                          bool bias, float *wIhScale, float *wHhScale, float *bIhScale, float *bHhScale,
                          rxmet_lstm_quant_params *out);

struct ForwardQuantCall {
    int T, B, I, H;
    const float *weightIh, *weightHh, *biasIh, *biasHh, *x, *h0, *c0;
    float *output, *finalHidden, *finalCell;
    const rxmet_lstm_trace *checkpoints;  // optional
    const rxmet_lstm_masters *masters;    // optional
};
size_t forwardQuantWorkspaceBytes(int T, int B, int I, int H);
// Picks the byte-code kernels (every grid <= 8 bits, accumulators below 2^24, I and H <= 128) or the
// wide kernels below.
void forwardQuant(const ForwardQuantCall &call, const Exec &exec, void *workspace, size_t workspaceBytes,
                  cudaStream_t stream);

// Activation grids up to 16 bits, weight grids up to 8 bits, H <= 512, I <= 256 (lstm_forward_wide.cu).
bool forwardQuantWideTakes(const Exec &exec, int I, int H, const char **why);
size_t forwardQuantWideWorkspaceBytes(int T, int B, int I, int H);
void forwardQuantWide(const ForwardQuantCall &call, const Exec &exec, void *workspace, size_t workspaceBytes,
                      cudaStream_t stream);
// c0 [B,H] (null = real zeros) -> centred cell codes, optional q-carrier copy and clamp mask.
void quantizeCellCodes(const float *c0, int B, int H, const ScalarExec &scalar, float *centred, float *carrier,
                       uint8_t *mask, cudaStream_t stream);

// How a saved tensor is turned into real values while it is loaded: real = (value - zeroPoint) * scale.
// The float backward uses {1, 0}; the QAT backward passes the grid of each saved q-carrier tensor.
struct Dequant {
    float scale = 1.0f;
    float zeroPoint = 0.0f;
};

struct BackwardCall {
    int T, B, I, H;
    const float *weightIh, *weightHh, *x, *h0, *c0;
    const float *gateOutputs, *cellStates, *cellTanhOutputs, *hiddenOutputs;
    const float *gradOutput, *gradFinalHidden, *gradFinalCell;
    const rxmet_lstm_backward_masks *masks;  // optional
    rxmet_lstm_gradients grads;
    // QAT: grids of the saved tensors and per-channel weight scales (host, 4H each); null = float
    bool quantized = false;
    Dequant dqX, dqH, dqC, dqGate[4], dqTanh;
    const float *weightIhScale = nullptr, *weightHhScale = nullptr;
    bool codesFitTensorPath = false;  // x and hidden grids span at most 256 codes around their zero points
    bool codesFitTwoTerms = false;    // x and hidden grids of at most 16 bits: a code is two exact bf16 terms
    bool weightCodesFitBf16 = false;  // weight_hh grid of at most 8 bits: codes are exact in bf16
    bool weightIhCodesFitBf16 = false;  // the same for weight_ih
};
size_t backwardWorkspaceBytes(int T, int B, int I, int H);
void backward(const BackwardCall &call, void *workspace, size_t workspaceBytes, cudaStream_t stream);

}  // namespace lstm
}  // namespace rxmet
