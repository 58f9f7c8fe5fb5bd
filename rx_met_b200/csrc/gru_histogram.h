// Host side of the histogram calibration of the QuantGRU path: the collector arithmetic (range
// growth, redistribution of counts), the percentile and SQNR range searches, and the split of
// "collect" into plan -> bin -> commit so that the binning itself can run on the device.
#pragma once

#include <cstddef>
#include <cstdint>

#include "rxmet_b200.h"

namespace rxmet {
namespace hist {

// What a batch with the given finite extremes does to a collector, decided before any element is
// binned: the range [lo, hi] and the reciprocal bin width the batch is binned with, and the range
// the collector has afterwards.
struct Plan {
    enum Mode { kFirst, kSameRange, kExtended } mode = kFirst;
    float lo = 0, hi = 0, invBinWidth = 0;  // binning of the new data
    float newMin = 0, newMax = 0;           // range of the collector after the batch
    float dataMin = 0, dataMax = 0;
    float limitMin = 0, limitMax = 0;       // growth limits fixed by the first batch
};

void reset(rxmet_histogram *h);
Plan plan(const rxmet_histogram &h, float dataMin, float dataMax);
// Bins `rows` x `cols` host floats (row stride in floats) into counts[num_bins] (zeroed by the caller).
void binHost(const float *data, uint64_t rows, uint64_t cols, uint64_t rowStride, const Plan &p, int bins,
             uint32_t *counts);
void commit(rxmet_histogram *h, const Plan &p, const uint32_t *counts, uint64_t elements);
void collectHost(rxmet_histogram *h, const float *data, uint64_t rows, uint64_t cols, uint64_t rowStride);
void merge(rxmet_histogram *h, const rxmet_histogram &other);

struct Continuous {
    float scale, lo, hi;
};
Continuous calibrate(const rxmet_histogram &h, int32_t qlo, int32_t qhi, bool isUnsigned, bool symmetric,
                     bool usePercentile, float percentile);

}  // namespace hist
}  // namespace rxmet
