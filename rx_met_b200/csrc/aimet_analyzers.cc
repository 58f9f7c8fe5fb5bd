// Host side of the AIMET histogram analyzers: the running PDF statistics, the TF-enhanced
// (quantization + saturation cost search) and the percentile encodings.  Compiled by g++ without
// FMA contraction; the element type of the analyzers is float, so the expressions that the
// reference evaluates in its element type are evaluated in float here.
//
// Follows native/common/src/math_functions.cpp:226-316 (InitializePdf, UpdatePdf) and :433-467
// (findOriginalRange), native/common/src/TfEnhancedEncodingAnalyzer.cpp:86-411 and
// native/common/src/PercentileEncodingAnalyzer.cpp:86-203.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <limits>
#include <utility>
#include <vector>

#include "common.h"
#include "rxmet_b200.h"

using namespace rxmet;

namespace {

constexpr float kGamma = 3.0f;      // weight of the saturation cost
constexpr double kMinRange = 0.01;

int pdfSize() { return rxmet_aimet_pdf_size(); }

void requirePdf(const rxmet_aimet_pdf *pdf) {
    RXMET_REQUIRE(pdf != nullptr && pdf->x_left != nullptr && pdf->pdf != nullptr, "pdf and its two arrays must not be null");
}

// math_functions.cpp:226-269: the range of the first batch, tripled around its centre, cut into
// buckets whose left edges are multiples of the bucket size.
void initialize(rxmet_aimet_pdf *pdf, float lo, float hi, bool signedValues) {
    const int n = pdfSize();
    if (lo == hi) hi = std::max(hi, lo + 0.01f);
    const float centre = (hi + lo) / 2;
    lo = std::max(0.99f * std::numeric_limits<float>::lowest(), centre - 3 * (centre - lo));
    hi = std::min(0.99f * std::numeric_limits<float>::max(), centre + 3 * (hi - centre));
    double bucket;
    if (signedValues) bucket = (static_cast<double>(hi) - static_cast<double>(lo)) / n;
    else bucket = std::max(std::abs(hi), std::abs(lo)) / n;
    for (int i = 0; i < n; ++i) {
        pdf->x_left[i] = signedValues ? std::floor(lo / bucket + i) * bucket : i * bucket;
        pdf->pdf[i] = 0.0;
    }
    pdf->iterations = 0;
    pdf->initialized = 1;
}

// math_functions.cpp:433-467, element type float.
std::pair<float, float> observedRange(const rxmet_aimet_pdf *pdf) {
    const int n = pdfSize();
    float lo = static_cast<float>(pdf->x_left[0]), hi = static_cast<float>(pdf->x_left[n - 1]);
    for (int i = 0; i < n; ++i)
        if (pdf->pdf[i] > 0) {
            lo = static_cast<float>(pdf->x_left[i]);
            break;
        }
    for (int i = n - 1; i > 0; --i)
        if (pdf->pdf[i] > 0) {
            hi = static_cast<float>(pdf->x_left[i]);
            break;
        }
    lo = std::min(lo, 0.0f);
    hi = std::max(hi, 0.0f);
    hi = std::max(hi, lo + static_cast<float>(kMinRange));
    return {lo, hi};
}

// The encoding both analyzers return before any non-zero batch was seen.
rxmet_aimet_encoding coldEncoding(const rxmet_aimet_pdf *pdf, int bw, float steps) {
    rxmet_aimet_encoding e{};
    if (!pdf->updated) return e;  // nothing was offered: the all-zero encoding marks failure
    e.min = -1;
    e.max = 1;
    e.delta = (e.max - e.min) / static_cast<int>(steps);
    e.offset = std::floor(e.min / e.delta);
    e.min = e.offset * e.delta;
    e.max = e.min + static_cast<int>(steps) * e.delta;
    e.bw = bw;
    return e;
}

struct Candidate {
    float delta;
    int offset;
};

// TfEnhancedEncodingAnalyzer.cpp:150-175
bool clampToObserved(float observedMin, float observedMax, float steps, float &delta, int &offset) {
    float lo = std::max(delta * offset, std::numeric_limits<float>::lowest());
    float hi = std::min(delta * (offset + steps), std::numeric_limits<float>::max());
    if (lo < observedMin && hi > observedMax) return false;
    lo = std::max(observedMin, lo);
    hi = std::min(observedMax, hi);
    if (lo == hi) return false;
    delta = static_cast<float>((static_cast<double>(hi) - lo) / steps);
    offset = static_cast<int>(std::round(lo / delta));
    return true;
}

// TfEnhancedEncodingAnalyzer.cpp:177-218: 17 deltas x 21 offsets, clamped to the observed range,
// plus the observed range itself.
std::vector<Candidate> asymmetricCandidates(float observedMin, float observedMax, float steps) {
    std::vector<Candidate> out;
    const float observedDelta = static_cast<float>((static_cast<double>(observedMax) - static_cast<double>(observedMin)) / steps);
    const int observedOffset = static_cast<int>(std::round(observedMin / observedDelta));
    observedMin = std::max(observedDelta * observedOffset, std::numeric_limits<float>::lowest());
    observedMax = std::min(observedDelta * (observedOffset + steps), std::numeric_limits<float>::max());
    const float deltaMax = observedDelta;
    for (float f = static_cast<float>(1.0 / 16); f <= 1 + 1.0 / 16; f = static_cast<float>(f + 1.0 / 16)) {
        for (int i = 0; i <= 20; ++i) {
            float delta = f * deltaMax;
            int offset = static_cast<int>(-steps + steps / 20.0 * i);
            if (!clampToObserved(observedMin, observedMax, steps, delta, offset)) continue;
            out.push_back({delta, offset});
        }
    }
    out.push_back({observedDelta, observedOffset});
    return out;
}

// TfEnhancedEncodingAnalyzer.cpp:220-257: 101 deltas on the symmetric (or, for non-negative
// data in unsigned-symmetric mode, the unsigned) grid.
std::vector<Candidate> symmetricCandidates(float lo, float hi, float steps, bool unsignedSymmetric) {
    std::vector<Candidate> out;
    float deltaMax;
    int offset;
    if (lo == 0.0f && unsignedSymmetric) {
        deltaMax = hi / steps;
        offset = 0;
    } else {
        const float absoluteMax = std::max(std::abs(hi), std::abs(lo));
        deltaMax = static_cast<float>(absoluteMax / (steps / 2.0));
        offset = static_cast<int>(std::floor(-steps / 2));
    }
    for (float f = static_cast<float>(1.0 / 100); f <= 1 + 1.0 / 100; f = static_cast<float>(f + 1.0 / 100))
        out.push_back({f * deltaMax, offset});
    return out;
}

// TfEnhancedEncodingAnalyzer.cpp:299-363: squared error of the bucket centres, saturated parts
// weighted by kGamma.
double quantAndSatCost(const rxmet_aimet_pdf *pdf, const std::vector<float> &centres, int bw, float delta, int offset) {
    const int n = pdfSize();
    const float lo = delta * offset;
    const float stepSize = static_cast<float>(std::pow(2, bw) - 1);
    const float hi = delta * (offset + stepSize);
    const float start = static_cast<float>(pdf->x_left[0]);
    const double step = pdf->x_left[1] - pdf->x_left[0];
    int loIndex = static_cast<int>(std::floor((lo - start) / step));
    loIndex = std::min(std::max(0, loIndex), n - 1);
    int hiIndex = static_cast<int>(std::floor((hi - start) / step));
    hiIndex = std::min(std::max(0, hiIndex), n - 1);

    double bottom = 0;
    const float loCentre = centres[loIndex];
    for (int i = 0; i < loIndex; ++i) {
        const double mid = centres[i];
        bottom += pdf->pdf[i] * std::pow(mid - loCentre, 2);
    }
    double top = 0;
    const float hiCentre = centres[hiIndex];
    for (int i = hiIndex; i < n; ++i) {
        const double mid = centres[i];
        top += pdf->pdf[i] * std::pow(mid - hiCentre, 2);
    }
    double inside = 0;
    const float inverse = 1 / delta;
    for (int i = loIndex; i < hiIndex; ++i) {
        const float value = centres[i];
        const float dequantized = std::floor(value * inverse + 0.5f) * delta;
        inside += pdf->pdf[i] * std::pow(value - dequantized, 2);
    }
    const double cost = kGamma * (bottom + top) + inside;
    return std::min(cost, std::numeric_limits<double>::max());
}

}  // namespace

extern "C" {

int rxmet_aimet_pdf_reset(rxmet_aimet_pdf *pdf) {
    return guarded([&] {
        requirePdf(pdf);
        std::memset(pdf->x_left, 0, sizeof(double) * pdfSize());
        std::memset(pdf->pdf, 0, sizeof(double) * pdfSize());
        pdf->initialized = pdf->iterations = pdf->updated = 0;
    });
}

int rxmet_aimet_pdf_plan(rxmet_aimet_pdf *pdf, float batch_min, float batch_max, int signed_values, double *bucket_size,
                         int *pdf_offset, int *skip) {
    return guarded([&] {
        requirePdf(pdf);
        RXMET_REQUIRE(bucket_size && pdf_offset && skip, "outputs must not be null");
        pdf->updated = 1;
        *skip = 0;
        if (!pdf->initialized) {
            if (batch_min == 0 && batch_max == 0) {  // an all-zero batch cannot define the range
                *skip = 1;
                return;
            }
            initialize(pdf, batch_min, batch_max, signed_values != 0);
        }
        *bucket_size = pdf->x_left[1] - pdf->x_left[0];
        const double lo = signed_values ? pdf->x_left[0] : 0;
        *pdf_offset = static_cast<int>(std::round(lo / *bucket_size));
    });
}

int rxmet_aimet_pdf_commit(rxmet_aimet_pdf *pdf, const uint32_t *histogram, uint64_t count) {
    return guarded([&] {
        requirePdf(pdf);
        RXMET_REQUIRE(histogram != nullptr && pdf->initialized, "commit needs a planned pdf and a histogram");
        for (int i = 0; i < pdfSize(); ++i) {
            const double prob = static_cast<double>(histogram[i]) / static_cast<double>(count);
            pdf->pdf[i] = (pdf->pdf[i] * pdf->iterations + prob) / (pdf->iterations + 1);
        }
        pdf->iterations++;
    });
}

int rxmet_aimet_pdf_update_host(rxmet_aimet_pdf *pdf, const float *data, uint64_t count, int signed_values) {
    return guarded([&] {
        requirePdf(pdf);
        RXMET_REQUIRE(data != nullptr && count > 0, "data must not be empty");
        // extremes as the reference's CPU loops take them (std::min / std::max from +-DBL_MAX)
        float lo = static_cast<float>(std::numeric_limits<double>::max()), hi = static_cast<float>(-std::numeric_limits<double>::max());
        for (uint64_t i = 0; i < count; ++i) {
            lo = std::min(lo, data[i]);
            hi = std::max(hi, data[i]);
        }
        double bucket = 0;
        int offset = 0, skip = 0;
        if (rxmet_aimet_pdf_plan(pdf, lo, hi, signed_values, &bucket, &offset, &skip) != 0) fail(RXMET_ERR_INVALID_ARGUMENT, "%s", std::string(rxmet_last_error()).c_str());
        if (skip) return;
        std::vector<uint32_t> histogram(pdfSize(), 0u);
        const float inverse = static_cast<float>(1 / bucket);
        for (uint64_t i = 0; i < count; ++i) {
            const int index = static_cast<int>(std::floor(data[i] * inverse) - offset);
            if (index >= 0 && index < pdfSize()) histogram[index] += 1;
        }
        if (rxmet_aimet_pdf_commit(pdf, histogram.data(), count) != 0) fail(RXMET_ERR_INVALID_ARGUMENT, "%s", std::string(rxmet_last_error()).c_str());
    });
}

int rxmet_aimet_tf_enhanced_encoding(const rxmet_aimet_pdf *pdf, int bw, int symmetric, int strict_symmetric,
                                     int unsigned_symmetric, rxmet_aimet_encoding *encoding) {
    return guarded([&] {
        requirePdf(pdf);
        RXMET_REQUIRE(encoding != nullptr && bw >= 1 && bw <= 32, "encoding must not be null, bit width in [1, 32]");
        float steps = static_cast<float>(std::pow(2, bw) - 1);
        if (!pdf->initialized) {
            *encoding = coldEncoding(pdf, bw, steps);
            return;
        }
        const auto range = observedRange(pdf);
        std::vector<Candidate> candidates;
        if (symmetric) {
            if (strict_symmetric) steps -= 1;
            candidates = symmetricCandidates(range.first, range.second, steps, unsigned_symmetric != 0);
        } else {
            candidates = asymmetricCandidates(range.first, range.second, steps);
        }
        const int n = pdfSize();
        const double half = (pdf->x_left[1] - pdf->x_left[0]) / 2;
        std::vector<float> centres(n);
        for (int i = 0; i < n; ++i) centres[i] = static_cast<float>(static_cast<float>(pdf->x_left[i]) + half);
        float bestDelta = -1;
        int bestOffset = -1;
        double bestCost = std::numeric_limits<double>::max();
        for (const Candidate &c : candidates) {
            const double cost = quantAndSatCost(pdf, centres, bw, c.delta, c.offset);
            if (cost < bestCost) {
                bestCost = cost;
                bestDelta = c.delta;
                bestOffset = c.offset;
            }
        }
        rxmet_aimet_encoding e{};
        e.delta = bestDelta;
        e.offset = bestOffset;
        e.bw = bw;
        e.min = std::max(bestDelta * bestOffset, std::numeric_limits<float>::lowest());
        e.max = std::min(bestDelta * (bestOffset + steps), std::numeric_limits<float>::max());
        *encoding = e;
    });
}

int rxmet_aimet_percentile_encoding(const rxmet_aimet_pdf *pdf, int bw, int symmetric, int strict_symmetric,
                                    int unsigned_symmetric, float percentile, rxmet_aimet_encoding *encoding) {
    return guarded([&] {
        requirePdf(pdf);
        RXMET_REQUIRE(encoding != nullptr && bw >= 1 && bw <= 32, "encoding must not be null, bit width in [1, 32]");
        float steps = static_cast<float>(std::pow(2, bw) - 1);
        if (symmetric && strict_symmetric) steps -= 1;
        if (!pdf->initialized) {
            *encoding = coldEncoding(pdf, bw, steps);
            return;
        }
        const int n = pdfSize();
        const auto range = observedRange(pdf);
        float lo = range.first, hi = range.second;
        if (percentile != 100.0f) {
            const float width = static_cast<float>(pdf->x_left[1] - pdf->x_left[0]);
            lo = static_cast<float>(pdf->x_left[0]);
            hi = static_cast<float>(pdf->x_left[n - 1] + width);
            std::vector<double> cdf(pdf->pdf, pdf->pdf + n);
            for (int i = 1; i < n; ++i) cdf[i] += cdf[i - 1];
            const float left = 1 - percentile / 100;
            for (int i = 0; i < n; ++i)
                if (cdf[i] >= left) {
                    lo = static_cast<float>(pdf->x_left[i]);
                    break;
                }
            const float right = percentile / 100;
            for (int i = n - 1; i >= 0; --i)
                if (cdf[i] < right && pdf->x_left[i] < range.second) {  // never beyond the observed maximum
                    hi = static_cast<float>(pdf->x_left[i] + width);
                    break;
                }
            if (lo == hi) hi += width;
        }
        lo = std::min(lo, 0.0f);
        hi = std::max(hi, 0.0f);
        if (rxmet_aimet_compute_encoding(bw, lo, hi, symmetric, strict_symmetric, unsigned_symmetric, encoding) != 0)
            fail(RXMET_ERR_INVALID_ARGUMENT, "%s", std::string(rxmet_last_error()).c_str());
    });
}

}  // extern "C"
