// Host side of the QuantLSTM histogram calibration.  Compiled by g++ without FMA contraction.
//
// Follows operators/quant-lstm/src/quantization/histogram.cc: a batch is binned over its own finite
// range (bin index in double), collectors merge by dropping every source bin's mass at the
// destination bin that holds the source bin's centre, the percentile range cuts half of the clipped
// mass from each side, and the SQNR search scores 101 symmetric or 17 x 21 asymmetric candidate
// ranges by the squared reconstruction error of the bin centres under min/max calibration.
#include "lstm_histogram.h"

#include <algorithm>
#include <cmath>
#include <limits>

#include "common.h"
#include "lstm_params.h"

namespace rxmet {
namespace lstm {
namespace hist {
namespace {

bool isEmpty(const rxmet_lstm_histogram &h) { return h.total_count == 0 || h.num_bins <= 0; }

float widthOf(const rxmet_lstm_histogram &h) {
    if (isEmpty(h) || !(h.minimum < h.maximum)) fail(RXMET_ERR_INVALID_ARGUMENT, "an empty or degenerate histogram has no bin width");
    return (h.maximum - h.minimum) / static_cast<float>(h.num_bins);
}

float centreOf(const rxmet_lstm_histogram &h, int index) { return h.minimum + (static_cast<float>(index) + 0.5f) * widthOf(h); }

struct Plain {  // a histogram by value, for the merge arithmetic
    float lo, hi;
    const double *counts;
    int bins;
    uint64_t total;
    float centre(int index) const { return lo + (static_cast<float>(index) + 0.5f) * ((hi - lo) / static_cast<float>(bins)); }
};

void addRebinned(const Plain &src, float lo, float hi, std::vector<double> *dst) {
    for (int i = 0; i < src.bins; ++i) {
        const double count = src.counts[i];
        if (count == 0.0) continue;
        (*dst)[binIndex(src.centre(i), lo, hi, src.bins)] += count;
    }
}

void mergePlain(rxmet_lstm_histogram *h, const Plain &other) {
    if (other.total == 0) return;
    RXMET_REQUIRE(other.bins == h->num_bins && other.lo < other.hi, "histogram to merge has a different layout");
    if (isEmpty(*h)) {
        std::copy(other.counts, other.counts + other.bins, h->counts);
        h->minimum = other.lo;
        h->maximum = other.hi;
        h->total_count = other.total;
        return;
    }
    const float lo = std::min(h->minimum, other.lo), hi = std::max(h->maximum, other.hi);
    std::vector<double> merged(h->num_bins, 0.0);
    addRebinned(Plain{h->minimum, h->maximum, h->counts, h->num_bins, h->total_count}, lo, hi, &merged);
    addRebinned(other, lo, hi, &merged);
    std::copy(merged.begin(), merged.end(), h->counts);
    h->minimum = lo;
    h->maximum = hi;
    h->total_count += other.total;
}

double noiseOf(const rxmet_lstm_histogram &h, float lo, float hi, int bits, bool isUnsigned, bool symmetric) {
    const MinMaxParam p = minMaxParam(lo, hi, bits, isUnsigned, symmetric);
    const Grid g = gridOfBits(bits, isUnsigned);
    double noise = 0.0;
    for (int i = 0; i < h.num_bins; ++i) {
        const double count = h.counts[i];
        if (count == 0.0) continue;
        const float value = centreOf(h, i);
        const double translated = std::nearbyint(static_cast<double>(value) / p.scale) + static_cast<double>(p.zeroPoint);
        const int32_t q = translated <= g.lo ? g.lo : (translated >= g.hi ? g.hi : static_cast<int32_t>(translated));
        const float back = static_cast<float>(static_cast<double>(static_cast<int64_t>(q) - p.zeroPoint) * static_cast<double>(p.scale));
        const double diff = static_cast<double>(back) - value;
        noise += diff * diff * count;
    }
    return noise;
}

std::pair<float, float> percentileRange(const rxmet_lstm_histogram &h, float percentile) {
    if (!std::isfinite(percentile) || percentile <= 0.0f || percentile > 100.0f)
        fail(RXMET_ERR_INVALID_ARGUMENT, "percentile must be in (0, 100]");
    if (percentile == 100.0f) return {h.minimum, h.maximum};
    const double clipped = (100.0 - static_cast<double>(percentile)) / 200.0;
    const double lowTarget = static_cast<double>(h.total_count) * clipped;
    const double highTarget = static_cast<double>(h.total_count) * (1.0 - clipped);
    double cumulative = 0.0;
    int low = 0, high = h.num_bins - 1;
    bool lowFound = false;
    for (int i = 0; i < h.num_bins; ++i) {
        cumulative += h.counts[i];
        if (!lowFound && cumulative >= lowTarget) {
            low = i;
            lowFound = true;
        }
        if (cumulative >= highTarget) {
            high = i;
            break;
        }
    }
    const float width = widthOf(h);
    const float lo = h.minimum + static_cast<float>(low) * width;
    const float hi = h.minimum + static_cast<float>(high + 1) * width;
    return lo < hi ? std::pair<float, float>{lo, hi} : std::pair<float, float>{h.minimum, h.maximum};
}

}  // namespace

std::pair<float, float> batchRange(float lo, float hi) {
    if (lo < hi) return {lo, hi};
    const float pad = std::max(std::abs(lo) * std::numeric_limits<float>::epsilon(), 1.0e-6f);
    return {lo - pad, hi + pad};
}

int binIndex(float value, float lo, float hi, int bins) {
    if (value <= lo) return 0;
    if (value >= hi) return bins - 1;
    const double normalized = (static_cast<double>(value) - lo) / (static_cast<double>(hi) - lo);
    return std::min(static_cast<int>(static_cast<size_t>(normalized * static_cast<double>(bins))), bins - 1);
}

void mergeBatch(rxmet_lstm_histogram *h, const double *counts, float lo, float hi, uint64_t finite) {
    mergePlain(h, Plain{lo, hi, counts, h->num_bins, finite});
}

void collectHost(rxmet_lstm_histogram *h, const float *data, uint64_t rows, uint64_t cols, uint64_t rowStride) {
    RXMET_REQUIRE(h->counts != nullptr && h->num_bins >= 2, "histogram needs a counts array and at least 2 bins");
    float lo = std::numeric_limits<float>::infinity(), hi = -lo;
    uint64_t finite = 0;
    for (uint64_t r = 0; r < rows; ++r)
        for (uint64_t c = 0; c < cols; ++c) {
            const float v = data[r * rowStride + c];
            if (std::isfinite(v)) {
                lo = std::min(lo, v);
                hi = std::max(hi, v);
                ++finite;
            }
        }
    if (finite == 0) return;
    const auto range = batchRange(lo, hi);
    std::vector<double> counts(h->num_bins, 0.0);
    for (uint64_t r = 0; r < rows; ++r)
        for (uint64_t c = 0; c < cols; ++c) {
            const float v = data[r * rowStride + c];
            if (std::isfinite(v)) ++counts[binIndex(v, range.first, range.second, h->num_bins)];
        }
    mergeBatch(h, counts.data(), range.first, range.second, finite);
}

void merge(rxmet_lstm_histogram *h, const rxmet_lstm_histogram &other) {
    if (isEmpty(other)) return;
    mergePlain(h, Plain{other.minimum, other.maximum, other.counts, other.num_bins, other.total_count});
}

std::pair<float, float> selectRange(const rxmet_lstm_histogram &h, int bits, bool isUnsigned, bool symmetric, int method,
                                    float percentile) {
    if (isEmpty(h)) fail(RXMET_ERR_INVALID_ARGUMENT, "an empty histogram cannot be calibrated");
    if (method == 1) return percentileRange(h, percentile);
    RXMET_REQUIRE(method == 0, "histogram calibration method must be 0 (sqnr) or 1 (percentile)");
    constexpr int kSymmetric = 101, kWidths = 17, kOffsets = 21;
    std::pair<float, float> best{h.minimum, h.maximum};
    double bestNoise = noiseOf(h, best.first, best.second, bits, isUnsigned, symmetric);
    if (symmetric) {
        const float extentAll = isUnsigned ? std::max(0.0f, h.maximum) : std::max(std::abs(h.minimum), std::abs(h.maximum));
        for (int k = 1; k <= kSymmetric; ++k) {
            const float extent = extentAll * static_cast<float>(k) / static_cast<float>(kSymmetric);
            const std::pair<float, float> range = isUnsigned ? std::pair<float, float>{0.0f, extent}
                                                              : std::pair<float, float>{-extent, extent};
            const double noise = noiseOf(h, range.first, range.second, bits, isUnsigned, symmetric);
            if (noise < bestNoise) {
                bestNoise = noise;
                best = range;
            }
        }
        return best;
    }
    const float spanAll = h.maximum - h.minimum;
    for (int w = 1; w <= kWidths; ++w) {
        const float span = spanAll * static_cast<float>(w) / static_cast<float>(kWidths);
        const float slack = spanAll - span;
        for (int o = 0; o < kOffsets; ++o) {
            const float fraction = static_cast<float>(o) / static_cast<float>(kOffsets - 1);
            const float lo = h.minimum + slack * fraction;
            const float hi = lo + span;
            const double noise = noiseOf(h, lo, hi, bits, isUnsigned, symmetric);
            if (noise < bestNoise) {
                bestNoise = noise;
                best = {lo, hi};
            }
        }
    }
    return best;
}

}  // namespace hist
}  // namespace lstm
}  // namespace rxmet
