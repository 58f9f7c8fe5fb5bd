// Host side of the AIMET native part: encodings from ranges and from min/max statistics.
// Compiled by g++ without FMA contraction.
//
// Follows native/common/src/quantization_utils.cpp:59-117 (getComputedEncodings) and
// native/common/src/MinMaxEncodingAnalyzer.cpp:80-107 (computeEncoding).
#include <algorithm>
#include <cmath>
#include <limits>

#include "common.h"
#include "rxmet_b200.h"

using namespace rxmet;

namespace {

rxmet_aimet_encoding encodingOf(int bw, double lo, double hi, bool symmetric, bool strict, bool unsignedSymmetric) {
    RXMET_REQUIRE(bw >= 1 && bw <= 32, "bit width must be in [1, 32]");
    RXMET_REQUIRE(!(symmetric && strict && unsignedSymmetric), "strict and unsigned symmetric modes are exclusive");
    rxmet_aimet_encoding e{};
    double steps = std::pow(2, bw) - 1;
    if (symmetric && strict) steps -= 1;
    e.bw = bw;
    const double floatLowest = std::numeric_limits<float>::lowest() * 0.99;
    const double floatMax = std::numeric_limits<float>::max() * 0.99;
    lo = std::clamp(lo, floatLowest, 0.0);
    hi = std::clamp(hi, 0.0, floatMax);
    unsignedSymmetric = unsignedSymmetric && lo >= 0.0;
    if (symmetric && !unsignedSymmetric) {
        const unsigned positive = static_cast<unsigned>(std::floor(steps / 2));
        const unsigned negative = static_cast<unsigned>(steps - positive);
        const unsigned extra = steps == 3 ? 1u : 0u;  // strict 2-bit grid: use every bin
        e.delta = std::max(hi / (positive + extra), -lo / negative);
        e.offset = -static_cast<double>(negative);
    } else {
        e.delta = (hi - lo) / steps;
        e.offset = std::clamp(std::round(lo / e.delta), -steps, 0.0);
    }
    if (e.offset < 0) e.delta = std::min(e.delta, floatLowest / e.offset);
    if (e.offset + steps > 0) e.delta = std::min(e.delta, floatMax / (e.offset + steps));
    e.min = e.delta * e.offset;
    e.max = e.delta * (e.offset + steps);
    return e;
}

}  // namespace

extern "C" {

int rxmet_aimet_compute_encoding(int bw, double range_min, double range_max, int symmetric, int strict_symmetric,
                                 int unsigned_symmetric, rxmet_aimet_encoding *encoding) {
    return guarded([&] {
        RXMET_REQUIRE(encoding != nullptr, "encoding must not be null");
        *encoding = encodingOf(bw, range_min, range_max, symmetric != 0, strict_symmetric != 0, unsigned_symmetric != 0);
    });
}

int rxmet_aimet_minmax_encoding(int bw, int dtype, double stats_min, double stats_max, int symmetric, int strict_symmetric,
                                int unsigned_symmetric, rxmet_aimet_encoding *encoding) {
    return guarded([&] {
        RXMET_REQUIRE(encoding != nullptr, "encoding must not be null");
        const double lo = std::min(0.0, stats_min);
        double hi = std::max(0.0, stats_max);
        RXMET_REQUIRE(dtype == 0 || dtype == 1, "dtype must be 0 (float) or 1 (double)");
        const double minRange = dtype == 0 ? static_cast<double>(0.01f) : 0.01;
        hi = std::max(hi, lo + minRange);
        *encoding = encodingOf(bw, lo, hi, symmetric != 0, strict_symmetric != 0, unsigned_symmetric != 0);
    });
}

}  // extern "C"
