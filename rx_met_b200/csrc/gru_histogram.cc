// Host side of the QuantGRU histogram calibration.  Compiled by g++ without FMA contraction: the
// float roundings here decide bin indices, redistributed counts and the chosen scales.
//
// Follows operators/quant-gru/include/histogram_collector.h (collector: first batch fixes the range,
// later batches extend it and split every old bin over at most two new ones, counts are floats) and
// operators/quant-gru/include/pot_sqnr_calibrator.h (percentile range; SQNR search over 101
// symmetric or 17 x 21 asymmetric candidates with clipping noise weighted by gamma = 3).
#include "gru_histogram.h"

#include <algorithm>
#include <cmath>
#include <limits>
#include <vector>

#include "common.h"

namespace rxmet {
namespace hist {
namespace {

constexpr float kFloatMax = std::numeric_limits<float>::max();
constexpr float kFloatLowest = std::numeric_limits<float>::lowest();

float minimumScale(int64_t steps) { return std::min(1.19209290e-07f, 0.01f / static_cast<float>(steps)); }

bool valid(const rxmet_histogram &h) { return h.num_bins > 0 && h.total_count > 0; }

float binWidth(const rxmet_histogram &h) {
    if (h.num_bins <= 0 || h.max_val <= h.min_val) return 1.0f;
    return (h.max_val - h.min_val) / h.num_bins;
}

bool unusableWidth(float w, int bins) { return std::abs(w) < minimumScale(bins) || std::isnan(w) || std::isinf(w); }

// Spreads the counts of `src` over `dst` bins of width dstWidth starting at newMin: a source bin
// lands in the destination bin that holds its left edge, the part beyond that bin's right edge
// (rounded to a whole count) goes to the bin one destination width further.
void redistribute(const float *counts, int bins, float srcMin, float srcWidth, float newMin, float dstWidth, float *dst) {
    if (unusableWidth(srcWidth, bins)) return;
    for (int i = 0; i < bins; ++i) {
        const float count = counts[i];
        if (count <= 0) continue;
        const float start = srcMin + i * srcWidth;
        int first = static_cast<int>((start - newMin) / dstWidth);
        first = std::min(first, bins - 1);
        const float firstEnd = newMin + dstWidth * (first + 1);
        const float share = std::min(rintf(((firstEnd - start) / srcWidth) * count), count);
        dst[first] += share;
        const float rest = count - share;
        if (rest > 0) {
            int second = static_cast<int>((start + dstWidth - newMin) / dstWidth);
            second = std::min(second, bins - 1);
            dst[second] += rest;
        }
    }
}

}  // namespace

void reset(rxmet_histogram *h) {
    RXMET_REQUIRE(h->counts != nullptr && h->num_bins > 0, "histogram needs a counts array and a bin count");
    std::fill(h->counts, h->counts + h->num_bins, 0.0f);
    h->min_val = kFloatMax;
    h->max_val = kFloatLowest;
    h->observed_min = kFloatMax;
    h->observed_max = kFloatLowest;
    h->total_count = 0;
    h->range_limit_set = 0;
    h->range_limit_min = h->range_limit_max = 0.0f;
}

Plan plan(const rxmet_histogram &h, float dataMin, float dataMax) {
    Plan p;
    if (dataMin > dataMax) dataMin = dataMax = 0.0f;  // nothing finite in the batch
    p.dataMin = dataMin;
    p.dataMax = dataMax;
    const int bins = h.num_bins;
    const float growth = std::numeric_limits<float>::infinity();
    if (!valid(h)) {
        p.mode = Plan::kFirst;
        const float minimumRange = minimumScale(bins) * bins;
        float span = dataMax - dataMin;
        float limitLo = dataMin, limitHi = dataMax;
        if (span < minimumRange || std::isnan(span) || std::isinf(span)) {
            limitLo = std::min(dataMin, 0.0f);
            limitHi = std::max(dataMax, 0.0f);
            span = minimumRange;
        }
        p.newMin = dataMin;
        p.newMax = dataMax;
        if (dataMin == dataMax) {  // a constant batch is binned over a unit-wide window around it
            p.lo = dataMin - 0.5f;
            p.hi = dataMax + 0.5f;
            p.invBinWidth = 1.0f / ((p.hi - p.lo) / bins);
        } else {
            p.lo = dataMin;
            p.hi = dataMax;
            p.invBinWidth = 1.0f / ((dataMax - dataMin) / bins);
        }
        p.limitMin = limitLo - span * growth / 2.0f;
        p.limitMax = limitHi + span * growth / 2.0f;
        return p;
    }
    float lo, hi;
    if (h.range_limit_set) {
        lo = std::max(h.range_limit_min, std::min(dataMin, h.min_val));
        hi = std::min(h.range_limit_max, std::max(dataMax, h.max_val));
    } else {
        lo = std::min(dataMin, h.min_val);
        hi = std::max(dataMax, h.max_val);
    }
    p.newMin = lo;
    p.newMax = hi;
    p.lo = lo;
    p.hi = hi;
    if (lo == h.min_val && hi == h.max_val) {
        p.mode = Plan::kSameRange;
        p.invBinWidth = 1.0f / binWidth(h);
    } else {
        p.mode = Plan::kExtended;
        p.invBinWidth = 1.0f / ((hi - lo) / bins);
    }
    return p;
}

void binHost(const float *data, uint64_t rows, uint64_t cols, uint64_t rowStride, const Plan &p, int bins,
             uint32_t *counts) {
    for (uint64_t r = 0; r < rows; ++r)
        for (uint64_t c = 0; c < cols; ++c) {
            const float v = data[r * rowStride + c];
            if (!std::isfinite(v)) continue;
            if (v < p.lo) {
                ++counts[0];
            } else if (v > p.hi) {
                ++counts[bins - 1];
            } else {
                const int idx = static_cast<int>((v - p.lo) * p.invBinWidth);
                ++counts[std::min(idx, bins - 1)];
            }
        }
}

void commit(rxmet_histogram *h, const Plan &p, const uint32_t *counts, uint64_t elements) {
    const int bins = h->num_bins;
    if (p.mode == Plan::kFirst) {
        reset(h);
        h->min_val = p.newMin;
        h->max_val = p.newMax;
        h->range_limit_min = p.limitMin;
        h->range_limit_max = p.limitMax;
        h->range_limit_set = 1;
    } else if (p.mode == Plan::kExtended) {
        std::vector<float> fresh(bins, 0.0f);
        redistribute(h->counts, bins, h->min_val, binWidth(*h), p.newMin, (p.newMax - p.newMin) / bins, fresh.data());
        std::copy(fresh.begin(), fresh.end(), h->counts);
        h->min_val = p.newMin;
        h->max_val = p.newMax;
    }
    // The reference adds 1.0f per element; a block add is the same value while counts stay below 2^24.
    for (int i = 0; i < bins; ++i)
        if (counts[i]) h->counts[i] += static_cast<float>(counts[i]);
    h->total_count += static_cast<int64_t>(elements);
    h->observed_min = std::min(h->observed_min, p.dataMin);
    h->observed_max = std::max(h->observed_max, p.dataMax);
}

void collectHost(rxmet_histogram *h, const float *data, uint64_t rows, uint64_t cols, uint64_t rowStride) {
    RXMET_REQUIRE(h->counts != nullptr && h->num_bins > 0, "histogram needs a counts array and a bin count");
    if (rows * cols == 0) return;
    float lo = kFloatMax, hi = kFloatLowest;
    for (uint64_t r = 0; r < rows; ++r)
        for (uint64_t c = 0; c < cols; ++c) {
            const float v = data[r * rowStride + c];
            if (std::isfinite(v)) {
                lo = std::min(lo, v);
                hi = std::max(hi, v);
            }
        }
    const Plan p = plan(*h, lo, hi);
    std::vector<uint32_t> counts(h->num_bins, 0u);
    binHost(data, rows, cols, rowStride, p, h->num_bins, counts.data());
    commit(h, p, counts.data(), rows * cols);
}

void merge(rxmet_histogram *h, const rxmet_histogram &other) {
    if (!valid(other)) return;
    RXMET_REQUIRE(h->num_bins == other.num_bins, "histograms with different bin counts cannot be merged");
    const int bins = h->num_bins;
    if (!valid(*h)) {
        std::copy(other.counts, other.counts + bins, h->counts);
        h->min_val = other.min_val;
        h->max_val = other.max_val;
        h->observed_min = other.observed_min;
        h->observed_max = other.observed_max;
        h->total_count = other.total_count;
        float span = other.max_val - other.min_val;
        const float minimumRange = minimumScale(bins) * bins;
        if (span < minimumRange) span = minimumRange;
        const float growth = std::numeric_limits<float>::infinity();
        h->range_limit_min = other.min_val - span * growth / 2.0f;
        h->range_limit_max = other.max_val + span * growth / 2.0f;
        h->range_limit_set = 1;
        return;
    }
    h->observed_min = std::min(h->observed_min, other.observed_min);
    h->observed_max = std::max(h->observed_max, other.observed_max);
    float lo, hi;
    if (h->range_limit_set) {
        lo = std::max(h->range_limit_min, std::min(other.min_val, h->min_val));
        hi = std::min(h->range_limit_max, std::max(other.max_val, h->max_val));
    } else {
        lo = std::min(other.min_val, h->min_val);
        hi = std::max(other.max_val, h->max_val);
    }
    if (lo == h->min_val && hi == h->max_val) {
        for (int i = 0; i < bins; ++i) h->counts[i] += other.counts[i];
    } else {
        std::vector<float> fresh(bins, 0.0f);
        const float width = (hi - lo) / bins;
        redistribute(h->counts, bins, h->min_val, binWidth(*h), lo, width, fresh.data());
        redistribute(other.counts, bins, other.min_val, binWidth(other), lo, width, fresh.data());
        std::copy(fresh.begin(), fresh.end(), h->counts);
        h->min_val = lo;
        h->max_val = hi;
    }
    h->total_count += other.total_count;
}

// ---- range searches ---------------------------------------------------------------

namespace {

std::pair<float, float> percentileRange(const rxmet_histogram &h, float clip) {
    if (!valid(h) || clip <= 0.0f) return {h.min_val, h.max_val};
    const int bins = h.num_bins;
    std::vector<float> cumulative(bins);
    cumulative[0] = h.counts[0];
    for (int i = 1; i < bins; ++i) cumulative[i] = cumulative[i - 1] + h.counts[i];
    const float total = cumulative[bins - 1];
    if (total < 1e-6f) return {h.min_val, h.max_val};
    const float width = binWidth(h);
    const float keep = 1.0f - clip;
    const float lowMass = total * clip, highMass = total * keep;
    int lowIndex = 0, highIndex = bins - 1;
    for (int i = 0; i < bins; ++i)
        if (cumulative[i] >= lowMass) { lowIndex = i; break; }
    for (int i = 0; i < bins; ++i)
        if (cumulative[i] >= highMass) { highIndex = i; break; }
    const float lo = h.min_val + lowIndex * width;
    float hi = h.min_val + highIndex * width;
    if (hi <= lo) hi = h.max_val;
    return {lo, hi};
}

Continuous fromPercentile(const rxmet_histogram &h, int64_t steps, bool symmetric, bool isUnsigned, float percentile) {
    const float floorScale = minimumScale(steps);
    const float clip = (100.0f - percentile) / 100.0f;
    auto [lo, hi] = percentileRange(h, clip);
    lo = std::max(kFloatLowest, std::min(std::min(lo, 0.0f), 0.0f));
    hi = std::min(kFloatMax, std::max(std::max(hi, 0.0f), 0.0f));
    const float n = static_cast<float>(steps);
    if ((hi - lo) / n < floorScale) {
        if (symmetric && !isUnsigned) {
            lo -= floorScale * static_cast<float>((steps + 1) / 2);
            hi += floorScale * static_cast<float>(steps / 2);
        } else {
            hi += floorScale * n;
        }
    }
    Continuous out{};
    if (symmetric && isUnsigned) {
        out.scale = std::max(std::max(hi, floorScale) / n, floorScale);
        out.lo = 0.0f;
        out.hi = out.scale * n;
    } else if (symmetric) {
        const int64_t pos = steps / 2, neg = (steps + 1) / 2;
        const float fromTop = pos > 0 ? hi / static_cast<float>(pos) : kFloatMax;
        const float fromBottom = neg > 0 ? -lo / static_cast<float>(neg) : kFloatMax;
        out.scale = std::max(fromTop, fromBottom);
        out.lo = -static_cast<float>(neg) * out.scale;
        out.hi = static_cast<float>(pos) * out.scale;
    } else {
        out.scale = (hi - lo) / n;
        out.lo = lo;
        out.hi = hi;
    }
    out.scale = std::max(out.scale, floorScale);
    return out;
}

// Expected reconstruction error of the histogram for a grid of `steps` steps of width delta whose
// code 0 sits at offset * delta; errors of clipped bins count gamma times.
float noiseOf(const rxmet_histogram &h, float delta, float offset, int64_t steps, float gamma, float p) {
    if (delta <= 0) return kFloatMax;
    const float width = binWidth(h);
    const float top = static_cast<float>(steps);
    float total = 0.0f;
    for (int i = 0; i < h.num_bins; ++i) {
        const float count = h.counts[i];
        if (count < 1e-6f) continue;
        const float x = h.min_val + (i + 0.5f) * width;
        float q = rintf(x / delta - offset);
        const bool clipped = q < 0 || q > top;
        q = std::max(0.0f, std::min(top, q));
        const float back = (q + offset) * delta;
        float error = std::pow(std::abs(back - x), p);
        if (clipped && gamma != 1.0f) error *= gamma;
        total += error * count;
    }
    return total;
}

struct Best {
    float scale = 0, lo = 0, hi = 0, noise = kFloatMax;
};

Continuous searchSymmetric(const rxmet_histogram &h, float lo, float hi, int64_t steps, bool isUnsigned) {
    constexpr int kCandidates = 101;
    const float floorScale = minimumScale(steps);
    const float n = static_cast<float>(steps);
    float widest, offset;
    if (isUnsigned) {
        widest = hi / n;
        offset = 0.0f;
    } else {
        widest = 2.0f * std::max(hi, -lo) / n;
        offset = -static_cast<float>((steps + 1) / 2);
    }
    widest = std::max(widest, floorScale);
    Best best;
    for (int d = 1; d <= kCandidates; ++d) {
        const float delta = std::max(widest * d / (kCandidates - 1), floorScale);
        const float noise = noiseOf(h, delta, offset, steps, 3.0f, 2.0f);
        if (noise < best.noise) {
            best.noise = noise;
            best.scale = delta;
            best.lo = offset * delta;
            best.hi = best.lo + steps * delta;
        }
    }
    if (best.noise == kFloatMax) fail(RXMET_ERR_INVALID_ARGUMENT, "calibrateSqnr: searchSymmetric failed to find valid scale");
    return {best.scale, best.lo, best.hi};
}

Continuous searchAsymmetric(const rxmet_histogram &h, float lo, float hi, int64_t steps) {
    constexpr int kDeltas = 17, kOffsets = 21;
    const float n = static_cast<float>(steps);
    const float widest = (hi - lo) / n;
    const float observedOffset = rintf(lo / widest);
    const float observedMin = widest * observedOffset;
    const float observedMax = observedMin + widest * n;
    const float floorScale = minimumScale(steps);
    const int offsetsCount = std::min(static_cast<int>(steps + 2), kOffsets);
    std::vector<float> offsets(offsetsCount);
    const float offsetStep = n / (offsetsCount - 2);
    for (int o = 0; o < offsetsCount - 1; ++o) offsets[o] = rintf(-n + o * offsetStep);
    offsets[offsetsCount - 1] = observedOffset;
    Best best;
    for (int d = 1; d <= kDeltas; ++d) {
        const float delta = std::max(widest * d / (kDeltas - 1), floorScale);
        for (int o = 0; o < offsetsCount; ++o) {
            float testMin = delta * offsets[o];
            float testMax = testMin + delta * n;
            testMin = std::max(observedMin, testMin);
            testMax = std::min(observedMax, testMax);
            const float clampedDelta = std::max((testMax - testMin) / n, floorScale);
            const float clampedOffset = rintf(testMin / clampedDelta);
            const float noise = noiseOf(h, clampedDelta, clampedOffset, steps, 3.0f, 2.0f);
            if (noise < best.noise) {
                best.noise = noise;
                best.scale = clampedDelta;
                best.lo = clampedOffset * clampedDelta;
                best.hi = best.lo + steps * clampedDelta;
            }
        }
    }
    if (best.noise == kFloatMax) fail(RXMET_ERR_INVALID_ARGUMENT, "calibrateSqnr: searchAsymmetric failed to find valid scale");
    return {best.scale, best.lo, best.hi};
}

}  // namespace

Continuous calibrate(const rxmet_histogram &h, int32_t qlo, int32_t qhi, bool isUnsigned, bool symmetric,
                     bool usePercentile, float percentile) {
    if (!valid(h)) fail(RXMET_ERR_INVALID_ARGUMENT, "Histogram is invalid in calibrateContinuousScaleFromHistogram");
    const int64_t steps = static_cast<int64_t>(qhi) - static_cast<int64_t>(qlo);
    RXMET_REQUIRE(steps > 0, "quantization grid has no steps");
    if (usePercentile) return fromPercentile(h, steps, symmetric, isUnsigned, percentile);
    const float floorScale = minimumScale(steps);
    const float lo = std::min(h.min_val, 0.0f);
    float hi = std::max(h.max_val, 0.0f);
    const float leastTop = lo + floorScale * static_cast<float>(steps);
    hi = hi > leastTop ? hi : leastTop;
    return symmetric ? searchSymmetric(h, lo, hi, steps, isUnsigned) : searchAsymmetric(h, lo, hi, steps);
}

}  // namespace hist
}  // namespace rxmet
