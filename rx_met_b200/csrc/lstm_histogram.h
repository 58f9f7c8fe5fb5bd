// Host side of the QuantLSTM histogram calibration: collector merge by re-binning, percentile and
// SQNR range selection, and the plan -> bin -> merge split that lets the binning run on the device.
#pragma once

#include <cstdint>
#include <utility>
#include <vector>

#include "rxmet_b200_lstm.h"

namespace rxmet {
namespace lstm {
namespace hist {

// Range a batch with the given finite extremes is binned over (degenerate ranges are padded).
std::pair<float, float> batchRange(float lo, float hi);
// Bin of a value in [lo, hi] split into `bins` (double arithmetic, as the device kernel does).
int binIndex(float value, float lo, float hi, int bins);
// Merges a batch histogram (counts over [lo, hi], `finite` finite samples) into a collector.
void mergeBatch(rxmet_lstm_histogram *h, const double *counts, float lo, float hi, uint64_t finite);
void collectHost(rxmet_lstm_histogram *h, const float *data, uint64_t rows, uint64_t cols, uint64_t rowStride);
void merge(rxmet_lstm_histogram *h, const rxmet_lstm_histogram &other);
std::pair<float, float> selectRange(const rxmet_lstm_histogram &h, int bits, bool isUnsigned, bool symmetric, int method,
                                    float percentile);

}  // namespace hist
}  // namespace lstm
}  // namespace rxmet
