// Host-side parameter logic of the QuantLSTM path: calibration ranges -> scales and
// zero points, scales -> executable rescale encodings, and the per-launch parameter
// blocks (scalar struct, per-channel array, activation tables) the kernels consume.
#pragma once

#include <cstdint>
#include <memory>
#include <mutex>
#include <utility>
#include <vector>

#include "rxmet_b200_lstm.h"

namespace rxmet {
namespace lstm {

constexpr int kOps = RXMET_LSTM_NUM_OPS;

struct Grid {
    int32_t lo, hi;
};
Grid gridOf(const rxmet_lstm_quant_config &cfg, int op);

void defaultConfig(rxmet_lstm_quant_config *cfg);
void rangesReset(rxmet_lstm_ranges *ranges, int hidden);
void paramsFromRanges(const rxmet_lstm_quant_config &cfg, const rxmet_lstm_ranges &ranges, int inputSize, int hidden,
                      bool bias, float *wIhScale, float *wHhScale, float *bIhScale, float *bHhScale,
                      rxmet_lstm_quant_params *out);
// Fills `out` (per-channel arrays only where non-null) and returns whether every accumulator is
// provably exact in float; throws when requireExact is set and it is not.
void deriveExecution(const rxmet_lstm_quant_params &params, bool requireExact, rxmet_lstm_execution *out);
void foldStats(rxmet_lstm_ranges *ranges, const float *stats, int hidden, bool bias);

// Scale and zero point that cover [lo, hi] on a grid (calibrateMinMax of the reference, no
// power-of-two snapping); used by the histogram range search to score candidate ranges.
struct MinMaxParam {
    float scale;
    int32_t zeroPoint;
};
MinMaxParam minMaxParam(float lo, float hi, int bits, bool isUnsigned, bool symmetric);
Grid gridOfBits(int bits, bool isUnsigned);
size_t statsFloats(int hidden);

// A rescale in the form the kernels apply it: rint(v * mult * pow2), both factors floats.
struct DevRescale {
    float mult;  // (float)M, or 1 for a pure shift
    float pow2;  // 2^-shift
};

// Scalar parameters, passed to kernels by value.
struct ScalarExec {
    int32_t zp[kOps];
    float zpF[kOps];  // the same zero points as floats: kernels add them straight from the argument bank
    int32_t lo[kOps];
    int32_t hi[kOps];
    float scale[kOps];
    DevRescale ihToGate[4], hhToGate[4];
    DevRescale productToOutput;
    float forgetRatio, inputRatio;          // Q31 multiplier * 2^-31 as a float
    double forgetMantissa, inputMantissa;   // used instead when the ratio does not fit Q31
    int32_t forgetExponent, inputExponent;
    int32_t forgetUsesFp, inputUsesFp;
    int32_t xShift, hShift;  // codes are stored as (code - shift) so that they fit a signed byte
    int32_t biasEnabled;
};

// Per-channel parameters, one float block of kChannelFields arrays of 4H entries.
enum ChannelField {
    kWIhScale = 0, kWHhScale, kBIhScale, kBHhScale,
    kIhBiasMult, kIhBiasPow2, kHhBiasMult, kHhBiasPow2,
    kIhOutMult, kIhOutPow2, kHhOutMult, kHhOutPow2,
    kChannelFields
};

// Activation tables for grids of at most 8 bits: entry = ((output code - output zero point) << 1) | clamped,
// indexed by (input code - input grid minimum).  Order: input, forget, cell, output gate, tanh(cell).
constexpr int kTableSize = 256;
constexpr int kTables = 5;

// Activation tables for grids of 9 to 16 bits (the five tables back to back, table t has
// 2^bits(input grid of t) entries in the same entry format).  They are too large for shared memory and
// live in device memory, uploaded once per parameter set and device.
struct WideTables {
    std::vector<int32_t> entries;
    int offset[kTables] = {};
};

struct Exec {
    int hidden = 0;
    ScalarExec scalar{};
    std::vector<float> channel;            // kChannelFields * 4H
    std::vector<int32_t> tables;           // kTables * kTableSize; empty when a table input is wider than 8 bits
    WideTables wide;                       // filled instead when every table input has at most 16 bits
    bool exactAccumulators = false;        // every integer accumulator stays below 2^24
    bool weightsFitBytes = false;          // weight_ih and weight_hh grids of at most 8 bits
    int activationPlanes = 1;              // byte planes that hold an input / hidden code: 1 (<= 8 bit) or 2 (<= 16 bit); 0 = wider
    // Device copy of wide.entries on the current device (cudaMalloc on first use, freed with the Exec).
    const int32_t *wideTablesOnDevice() const;
    mutable std::mutex deviceLock;
    mutable std::vector<std::pair<int, std::shared_ptr<int32_t>>> deviceTables;  // (device ordinal, buffer)
};

// Cached on the content of `params`: callers pass the same encodings on every step.
std::shared_ptr<const Exec> deriveExec(const rxmet_lstm_quant_params &params, bool requireExact);

}  // namespace lstm
}  // namespace rxmet
