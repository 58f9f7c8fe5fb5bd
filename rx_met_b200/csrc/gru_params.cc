// Host-side parameter derivation for the QuantGRU kernels.  All float
// arithmetic here must round exactly as the reference's host code does, since
// the multipliers, zero points and table entries decide the integer codes the
// kernels produce; this file is therefore compiled without FMA contraction and
// without fast-math.  Citations are <file under operators/quant-gru/>:<line>.
#include "gru_params.h"
#include "gru_histogram.h"

#include <algorithm>
#include <array>
#include <cfloat>
#include <cmath>
#include <cstring>
#include <limits>
#include <list>
#include <mutex>
#include <string>
#include <utility>

#include "common.h"

namespace rxmet {
namespace gru {
namespace {

struct Width {
    int bits;
    bool isUnsigned;
    // include/quantize_bitwidth_config.h:16-24
    int32_t lo() const {
        if (bits >= 32) return std::numeric_limits<int32_t>::min();
        return isUnsigned ? 0 : -(1 << (bits - 1));
    }
    int32_t hi() const {
        if (bits >= 32) return std::numeric_limits<int32_t>::max();
        return isUnsigned ? static_cast<int32_t>((1u << bits) - 1u) : (1 << (bits - 1)) - 1;
    }
};

Width widthOf(const rxmet_gru_quant_config &cfg, int op) {
    const int bits = cfg.bits[op];
    RXMET_REQUIRE(bits >= 1 && bits <= 32, "bit-width of quantization point %d is %d, expected 1..32", op, bits);
    return Width{bits, bits >= 32 ? false : cfg.is_unsigned[op] != 0};
}

// include/scale_encoding.h:87-106
Rescale encodeMShift(float scale) {
    RXMET_REQUIRE(scale > 0.0f, "scale must be > 0 to encode as M*2^-shift");
    int exponent = 0;
    const double mantissa = std::frexp(static_cast<double>(scale), &exponent);
    auto m = static_cast<uint32_t>(std::llround(mantissa * 65536.0));
    if (m == 65536u) {
        m = 32768u;
        exponent += 1;
    }
    m = std::max(m, 32768u);
    const int shift = 16 - exponent;
    RXMET_REQUIRE(shift >= -128 && shift <= 127, "M*2^-shift encoding: shift %d does not fit int8", shift);
    return Rescale{static_cast<int32_t>(m), shift};
}

// include/scale_encoding.h:114-117
int pot2Shift(float scale) {
    if (!(scale > 0.0f)) return 0;
    return static_cast<int8_t>(std::lround(-std::log2(static_cast<double>(scale))));
}

// Strategy object for the two rescale modes (include/scale_encoding.h:122-192).
class ScaleMode {
   public:
    explicit ScaleMode(bool pot2) : pot2_(pot2) {}

    float effective(float scale) const {
        if (pot2_) return std::ldexp(1.0f, -pot2Shift(scale));
        const Rescale r = encodeMShift(scale);
        return static_cast<float>(r.mult) * std::ldexp(1.0f, -r.shift);
    }
    Rescale ratio(float src, float dst) const {
        if (pot2_) return Rescale{1, static_cast<int8_t>(pot2Shift(src) - pot2Shift(dst))};
        return encodeMShift(src / dst);
    }
    Rescale productTo(float a, float b, float dst) const {
        if (pot2_) return Rescale{1, static_cast<int8_t>(pot2Shift(a) + pot2Shift(b) - pot2Shift(dst))};
        return encodeMShift((a * b) / dst);
    }
    Rescale toProduct(float src, float a, float b) const {
        if (pot2_) return Rescale{1, static_cast<int8_t>(pot2Shift(src) - (pot2Shift(a) + pot2Shift(b)))};
        return encodeMShift(src / (a * b));
    }

   private:
    bool pot2_;
};

// ---- ranges -> encodings -------------------------------------------------

// include/histogram_collector.h:34-38
float minimumScale(int64_t steps) { return std::min(1.19209290e-07f, 0.01f / static_cast<float>(steps)); }

struct Continuous {
    float scale, lo, hi;
};

// include/pot_sqnr_calibrator.h:372-439
Continuous continuousFromRange(float lo, float hi, Width w, bool symmetric) {
    const int32_t qlo = w.lo(), qhi = w.hi();
    const int64_t steps = static_cast<int64_t>(qhi) - static_cast<int64_t>(qlo);
    RXMET_REQUIRE(steps > 0, "quantization grid has no steps");
    const float floorScale = minimumScale(steps);
    const float nSteps = static_cast<float>(steps);
    const float lo0 = std::min(lo, 0.0f);
    const float hi0 = std::max(hi, 0.0f);
    const float widen = ((hi0 - lo0) / nSteps < floorScale) ? floorScale : 0.0f;

    Continuous out{};
    if (symmetric && w.isUnsigned) {
        const float top = hi0 + nSteps * widen;
        out.scale = std::max(std::max(top, floorScale) / static_cast<float>(qhi), floorScale);
        out.lo = 0.0f;
        out.hi = out.scale * static_cast<float>(qhi);
    } else if (symmetric) {
        const float top = hi0 + std::floor(nSteps / 2.0f) * widen;
        const float bottom = lo0 - std::ceil(nSteps / 2.0f) * widen;
        const int64_t pos = steps / 2, neg = (steps + 1) / 2;
        const int64_t extra = (steps == 3) ? 1 : 0;
        const float fromTop = (pos + extra > 0) ? top / static_cast<float>(pos + extra) : 0.0f;
        const float fromBottom = (neg > 0) ? -bottom / static_cast<float>(neg) : 0.0f;
        out.scale = std::max(std::max(fromTop, fromBottom), floorScale);
        out.lo = -static_cast<float>(neg) * out.scale;
        out.hi = static_cast<float>(pos) * out.scale;
    } else {
        const float top = hi0 + nSteps * widen;
        const float span = std::max(top - lo0, floorScale * nSteps);
        out.scale = std::max(span / nSteps, floorScale);
        out.lo = lo0;
        out.hi = lo0 + out.scale * nSteps;
    }
    return out;
}

// include/pot_scale_encode.h:63-103
bool nearPowerOfTwo(float value, float tolerance) {
    if (!(value > 0.0f)) return false;
    const float nearest = std::pow(2.0f, std::round(std::log2(value)));
    return std::abs(value - nearest) / nearest < tolerance;
}

std::pair<float, int> scaleToPowerOfTwo(float scale, int method, float lo, float hi, float tolerance) {
    RXMET_REQUIRE(scale > 0.0f, "scale must be > 0 to round to a power of two");
    const float n = -std::log2(scale);
    float chosen;
    switch (method) {
        case RXMET_POT_ROUND: chosen = std::round(n); break;
        case RXMET_POT_FLOOR: chosen = std::floor(n); break;
        default: chosen = nearPowerOfTwo(std::abs(hi - lo), tolerance) ? std::round(n) : std::floor(n);
    }
    RXMET_REQUIRE(chosen >= -128.0f && chosen <= 127.0f, "power-of-two exponent does not fit int8");
    const auto n8 = static_cast<int8_t>(chosen);
    return {std::pow(2.0f, -static_cast<float>(n8)), n8};
}

struct Encoding {
    float scale;  // value to store: continuous (affine mode) or 2^-n
    int32_t zeroPoint;
};

// include/gru_calibration_helpers.h:16-27 -> include/scale_encoding.h:207-320
Encoding encodeContinuous(const Continuous &c, Width w, bool symmetric, const rxmet_gru_quant_config &cfg) {
    const float qlo = static_cast<float>(w.lo());
    if (cfg.use_pot2) {
        const auto [po2, n] = scaleToPowerOfTwo(c.scale, cfg.pot_scale_method, c.lo, c.hi, cfg.pot_scale_tolerance);
        (void)n;
        int32_t zp = 0;
        if (!symmetric) {
            const float anchor = (cfg.pot_scale_method == RXMET_POT_FLOOR) ? std::floor(c.lo / po2) * po2 : c.lo;
            zp = static_cast<int32_t>(std::rint(qlo - anchor / po2));
        }
        return {po2, zp};
    }
    const Rescale ms = encodeMShift(c.scale);
    const float effective = static_cast<float>(ms.mult) * std::ldexp(1.0f, -ms.shift);
    const int32_t zp = symmetric ? 0 : static_cast<int32_t>(std::rint(qlo - c.lo / effective));
    return {c.scale, zp};
}

Encoding encodeRange(float lo, float hi, Width w, bool symmetric, const rxmet_gru_quant_config &cfg) {
    return encodeContinuous(continuousFromRange(lo, hi, w, symmetric), w, symmetric, cfg);
}

// Calls f(begin, end) for each scale group of a 3*hidden channel array.
template <class F>
void forEachGroup(int hidden, int granularity, F &&f) {
    const int channels = 3 * hidden;
    const int group = granularity == RXMET_PER_TENSOR ? channels : (granularity == RXMET_PER_GATE ? hidden : 1);
    for (int begin = 0; begin < channels; begin += group) f(begin, begin + group);
}

}  // namespace

// src/gru_host.cc:13-125
void paramsFromRanges(const rxmet_gru_ranges &r, const rxmet_gru_quant_config &cfg, rxmet_gru_quant_params *out) {
    RXMET_REQUIRE(out != nullptr && r.hidden > 0, "params_from_ranges: bad arguments");
    RXMET_REQUIRE(cfg.symmetric[RXMET_GRU_W] && cfg.symmetric[RXMET_GRU_R] && cfg.symmetric[RXMET_GRU_BW] &&
                      cfg.symmetric[RXMET_GRU_BR],
                  "W/R/bw/br must remain symmetric (zp=0)");
    RXMET_REQUIRE(out->scale_W && out->scale_R && out->scale_bw && out->scale_br,
                  "params_from_ranges: per-channel scale arrays are not set");
    out->hidden = r.hidden;
    out->config = cfg;
    std::fill(std::begin(out->scale), std::end(out->scale), 0.0f);
    std::fill(std::begin(out->zero_point), std::end(out->zero_point), 0);

    for (int op = 0; op < kOps; ++op) {
        if (op == RXMET_GRU_W || op == RXMET_GRU_R || op == RXMET_GRU_BW || op == RXMET_GRU_BR) continue;
        float lo = r.min[op], hi = r.max[op];
        const bool gateOutput = op == RXMET_GRU_UPDATE_GATE_OUTPUT || op == RXMET_GRU_RESET_GATE_OUTPUT ||
                                op == RXMET_GRU_NEW_GATE_OUTPUT;
        if (gateOutput && hi - lo < 0.5f) {  // include/calibration_utils.h:26-43, threshold src/gru_host.cc:95
            const float center = (lo + hi) / 2.0f;
            lo = center - 0.5f / 2.0f;
            hi = center + 0.5f / 2.0f;
        }
        const Encoding e = encodeRange(lo, hi, widthOf(cfg, op), cfg.symmetric[op] != 0, cfg);
        out->scale[op] = e.scale;
        out->zero_point[op] = e.zeroPoint;
    }

    auto weights = [&](float *dst, int granularity, int op, const float *mins, const float *maxs) {
        RXMET_REQUIRE(mins && maxs, "params_from_ranges: per-channel ranges are not set");
        forEachGroup(r.hidden, granularity, [&](int begin, int end) {
            const float lo = *std::min_element(mins + begin, mins + end);
            const float hi = *std::max_element(maxs + begin, maxs + end);
            const Encoding e = encodeRange(lo, hi, widthOf(cfg, op), cfg.symmetric[op] != 0, cfg);
            std::fill(dst + begin, dst + end, e.scale);
        });
    };
    weights(out->scale_W, cfg.W_granularity, RXMET_GRU_W, r.min_W, r.max_W);
    weights(out->scale_R, cfg.R_granularity, RXMET_GRU_R, r.min_R, r.max_R);

    // include/gru_calibration_helpers.h:33-62 : twice the observed extent.
    auto biases = [&](float *dst, int granularity, int op, const float *mins, const float *maxs) {
        RXMET_REQUIRE(mins && maxs, "params_from_ranges: per-channel ranges are not set");
        const Width w = widthOf(cfg, op);
        forEachGroup(r.hidden, granularity, [&](int begin, int end) {
            double extent = 0.0;
            for (int c = begin; c < end; ++c) {
                RXMET_REQUIRE(std::isfinite(mins[c]) && std::isfinite(maxs[c]) && mins[c] <= maxs[c],
                              "Bias calibration requires finite observations");
                extent = std::max(extent, std::max(std::abs(static_cast<double>(mins[c])),
                                                   std::abs(static_cast<double>(maxs[c]))));
            }
            double scale = std::max(2.0 * extent, 0.01) / w.hi();
            if (cfg.use_pot2) scale = std::exp2(std::ceil(std::log2(scale)));
            if (!std::isfinite(scale) || scale > std::numeric_limits<float>::max())
                fail(RXMET_ERR_INVALID_ARGUMENT, "Bias headroom scale exceeds float32 range");
            std::fill(dst + begin, dst + end, static_cast<float>(scale));
        });
    };
    biases(out->scale_bw, cfg.bw_granularity, RXMET_GRU_BW, r.min_bw, r.max_bw);
    biases(out->scale_br, cfg.br_granularity, RXMET_GRU_BR, r.min_br, r.max_br);
}

// src/gru_host.cc:254-335
void paramsFromHistograms(const rxmet_gru_histograms &hs, const rxmet_gru_quant_config &cfg, bool usePercentile,
                          float percentile, rxmet_gru_quant_params *out) {
    RXMET_REQUIRE(out != nullptr && hs.hidden > 0, "params_from_histograms: bad arguments");
    RXMET_REQUIRE(cfg.symmetric[RXMET_GRU_W] && cfg.symmetric[RXMET_GRU_R] && cfg.symmetric[RXMET_GRU_BW] &&
                      cfg.symmetric[RXMET_GRU_BR],
                  "W/R/bw/br must remain symmetric (zp=0)");
    RXMET_REQUIRE(out->scale_W && out->scale_R && out->scale_bw && out->scale_br,
                  "params_from_histograms: per-channel scale arrays are not set");
    out->hidden = hs.hidden;
    out->config = cfg;
    std::fill(std::begin(out->scale), std::end(out->scale), 0.0f);
    std::fill(std::begin(out->zero_point), std::end(out->zero_point), 0);
    auto fromHistogram = [&](const rxmet_histogram &h, int op, const char *name) {
        if (!(h.num_bins > 0 && h.total_count > 0)) fail(RXMET_ERR_INVALID_ARGUMENT, "%s is invalid.", name);
        const Width w = widthOf(cfg, op);
        const hist::Continuous c = hist::calibrate(h, w.lo(), w.hi(), w.isUnsigned, cfg.symmetric[op] != 0, usePercentile, percentile);
        return encodeContinuous(Continuous{c.scale, c.lo, c.hi}, w, cfg.symmetric[op] != 0, cfg);
    };
    static const char *kNames[kOps] = {"scale_x", "scale_h", "W", "R", "bw", "br", "scale_weight_ih_linear",
                                       "scale_weight_hh_linear", "scale_update_gate_input", "scale_update_gate_output",
                                       "scale_reset_gate_input", "scale_reset_gate_output", "scale_new_gate_input",
                                       "scale_new_gate_output", "scale_mul_reset_hidden", "scale_mul_old_contribution",
                                       "scale_mul_new_contribution"};
    for (int op = 0; op < kOps; ++op) {
        if (op == RXMET_GRU_W || op == RXMET_GRU_R || op == RXMET_GRU_BW || op == RXMET_GRU_BR) continue;
        const Encoding e = fromHistogram(hs.point[op], op, kNames[op]);
        out->scale[op] = e.scale;
        out->zero_point[op] = e.zeroPoint;
    }
    auto weights = [&](float *dst, int granularity, int op, int slot) {
        const int hidden = hs.hidden, channels = 3 * hidden;
        if (granularity == RXMET_PER_TENSOR) {
            std::fill(dst, dst + channels, fromHistogram(hs.point[op], op, kNames[op]).scale);
        } else if (granularity == RXMET_PER_GATE) {
            for (int g = 0; g < 3; ++g)
                std::fill(dst + g * hidden, dst + (g + 1) * hidden, fromHistogram(hs.gate[slot][g], op, kNames[op]).scale);
        } else {
            RXMET_REQUIRE(hs.channel[slot] != nullptr, "per-channel collectors are not set");
            for (int c = 0; c < channels; ++c) dst[c] = fromHistogram(hs.channel[slot][c], op, kNames[op]).scale;
        }
    };
    weights(out->scale_W, cfg.W_granularity, RXMET_GRU_W, 0);
    weights(out->scale_R, cfg.R_granularity, RXMET_GRU_R, 1);
    // biases: twice the observed extent of each group (include/gru_calibration_helpers.h:33-62)
    auto biases = [&](float *dst, int granularity, int op, int slot) {
        RXMET_REQUIRE(hs.channel[slot] != nullptr, "per-channel collectors are not set");
        const Width w = widthOf(cfg, op);
        forEachGroup(hs.hidden, granularity, [&](int begin, int end) {
            double extent = 0.0;
            for (int c = begin; c < end; ++c) {
                const float lo = hs.channel[slot][c].observed_min, hi = hs.channel[slot][c].observed_max;
                RXMET_REQUIRE(std::isfinite(lo) && std::isfinite(hi) && lo <= hi, "Bias calibration requires finite observations");
                extent = std::max(extent, std::max(std::abs(static_cast<double>(lo)), std::abs(static_cast<double>(hi))));
            }
            double scale = std::max(2.0 * extent, 0.01) / w.hi();
            if (cfg.use_pot2) scale = std::exp2(std::ceil(std::log2(scale)));
            if (!std::isfinite(scale) || scale > std::numeric_limits<float>::max())
                fail(RXMET_ERR_INVALID_ARGUMENT, "Bias headroom scale exceeds float32 range");
            std::fill(dst + begin, dst + end, static_cast<float>(scale));
        });
    };
    biases(out->scale_bw, cfg.bw_granularity, RXMET_GRU_BW, 2);
    biases(out->scale_br, cfg.br_granularity, RXMET_GRU_BR, 3);
}

namespace {

// ---- activation tables (src/quantize_lut.cc) ------------------------------

using Knots = std::array<float, kSegments + 1>;

// src/quantize_lut.cc:79-174 : knots follow the cumulative weight of 999
// intervals; intervals with |x| < 2 weigh up to 6x, the rest 1 + slope/2.
Knots chooseKnots(float lo, float hi) {
    constexpr int samples = 1000;
    std::vector<float> xs(samples), cumulative(samples - 1);
    for (int i = 0; i < samples; ++i) xs[i] = lo + (hi - lo) * static_cast<float>(i) / (samples - 1);
    auto sigmoid = [](float x) { return 1.0f / (1.0f + std::exp(-x)); };
    for (int i = 0; i + 1 < samples; ++i) {
        const float slope = std::abs(sigmoid(xs[i + 1]) - sigmoid(xs[i])) / (xs[i + 1] - xs[i] + 1e-9f);
        const float distance = std::abs(xs[i]);
        cumulative[i] = distance < 2.0f ? 5.0f * (1.0f - distance / 2.0f) + 1.0f : 1.0f + slope * 0.5f;
    }
    float total = 0.0f;
    for (float w : cumulative) total += w;
    float running = 0.0f;
    for (int i = 0; i + 1 < samples; ++i) {
        const float normalized = cumulative[i] / total;
        running = (i == 0) ? normalized : running + normalized;
        cumulative[i] = running;
    }

    std::vector<float> knots;
    knots.reserve(kSegments + 1);
    knots.push_back(lo);
    for (int s = 1; s < kSegments; ++s) {
        const float target = static_cast<float>(s) / kSegments;
        auto at = static_cast<int>(std::lower_bound(cumulative.begin(), cumulative.end(), target) - cumulative.begin());
        knots.push_back(xs[std::min(at, samples - 2)]);
    }
    knots.push_back(hi);
    std::sort(knots.begin(), knots.end());
    knots.erase(std::unique(knots.begin(), knots.end(), [](float a, float b) { return std::abs(a - b) < 1e-9f; }),
                knots.end());
    while (static_cast<int>(knots.size()) < kSegments + 1) {  // split the widest interval
        size_t widest = 0;
        float width = 0.0f;
        for (size_t i = 0; i + 1 < knots.size(); ++i) {
            if (knots[i + 1] - knots[i] > width) {
                width = knots[i + 1] - knots[i];
                widest = i;
            }
        }
        knots.insert(knots.begin() + widest + 1, (knots[widest] + knots[widest + 1]) / 2.0f);
    }
    Knots out{};
    std::copy_n(knots.begin(), kSegments + 1, out.begin());
    return out;
}

struct Line {
    float slope, intercept;
};

// src/quantize_lut.cc:53-76 and the 100-sample loops at :238-249 / :326-337.
template <class Fn>
Line fitSegment(float begin, float end, Fn &&fn) {
    constexpr int n = 100;
    float sx = 0.0f, sy = 0.0f, sxy = 0.0f, sxx = 0.0f;
    for (int j = 0; j < n; ++j) {
        const float x = begin + (end - begin) * static_cast<float>(j) / (n - 1);
        const float y = fn(x);
        sx += x;
        sy += y;
        sxy += x * y;
        sxx += x * x;
    }
    const float denom = n * sxx - sx * sx;
    if (std::abs(denom) < 1e-9f) return {0.0f, sy / n};
    const float slope = (n * sxy - sx * sy) / denom;
    return {slope, (sy - slope * sx) / n};
}

enum class Activation { Sigmoid, Tanh };

// src/quantize_lut.cc:190-364
Lut makeLut(Activation kind, float scaleIn, int32_t zpIn, float scaleOut, int32_t zpOut, Width in, Width outW) {
    const float limit = kind == Activation::Tanh ? 4.0f : 8.0f;
    const float lo = std::max(static_cast<float>(in.lo() - zpIn) * scaleIn, -limit);
    const float hi = std::min(static_cast<float>(in.hi() - zpIn) * scaleIn, limit);
    const Knots knots = chooseKnots(lo, hi);
    Lut lut{};
    lut.zp_x = zpIn;
    const int32_t qmax = outW.hi();
    for (int s = 0; s < kSegments; ++s) {
        const Line line = kind == Activation::Tanh
                              ? fitSegment(knots[s], knots[s + 1], [](float x) { return std::tanh(x); })
                              : fitSegment(knots[s], knots[s + 1], [](float x) { return 1.0f / (1.0f + std::exp(-x)); });
        const float gain = line.slope * (scaleIn / scaleOut);
        int32_t qb = 0;
        int nbx = 0;
        if (!(std::abs(gain) < 1e-12f)) {
            nbx = static_cast<int8_t>(std::floor(std::log2(static_cast<double>(qmax) / std::abs(gain))));
            const auto q = static_cast<int64_t>(std::rint(static_cast<double>(gain) * std::ldexp(1.0, nbx)));
            qb = static_cast<int32_t>(std::clamp<int64_t>(q, -static_cast<int64_t>(qmax), qmax));
        }
        lut.q_b[s] = qb;
        lut.n_bx[s] = nbx;
        lut.term_c[s] = static_cast<int32_t>(std::rint(line.intercept / scaleOut + static_cast<float>(zpOut)));
        const auto threshold = static_cast<int32_t>(std::rint(knots[s + 1] / scaleIn + zpIn));
        lut.threshold[s] = std::clamp(threshold, in.lo(), in.hi());
    }
    return lut;
}

struct Luts {
    Lut update, reset, fresh;
};

// src/quantize_lut.cc:17-48 : the tables come from the stored scales.
Luts makeLuts(const rxmet_gru_quant_params &p) {
    auto one = [&](Activation kind, int in, int out) {
        return makeLut(kind, p.scale[in], p.zero_point[in], p.scale[out], p.zero_point[out], widthOf(p.config, in),
                       widthOf(p.config, out));
    };
    return {one(Activation::Sigmoid, RXMET_GRU_UPDATE_GATE_INPUT, RXMET_GRU_UPDATE_GATE_OUTPUT),
            one(Activation::Sigmoid, RXMET_GRU_RESET_GATE_INPUT, RXMET_GRU_RESET_GATE_OUTPUT),
            one(Activation::Tanh, RXMET_GRU_NEW_GATE_INPUT, RXMET_GRU_NEW_GATE_OUTPUT)};
}

CodeClass classOf(Width w) {
    const int signedBits = w.bits + (w.isUnsigned ? 1 : 0);
    return signedBits <= 8 ? CodeClass::I8 : (signedBits <= 16 ? CodeClass::I16 : CodeClass::I32);
}
CodeClass wider(CodeClass a, CodeClass b) { return static_cast<int>(a) > static_cast<int>(b) ? a : b; }

std::string cacheKey(const rxmet_gru_quant_params &p) {
    std::string key;
    auto put = [&](const void *data, size_t bytes) { key.append(static_cast<const char *>(data), bytes); };
    const size_t channels = 3 * static_cast<size_t>(p.hidden);
    put(&p.hidden, sizeof(p.hidden));
    put(p.scale, sizeof(p.scale));
    put(p.zero_point, sizeof(p.zero_point));
    put(p.config.bits, sizeof(p.config.bits));
    put(p.config.is_unsigned, sizeof(p.config.is_unsigned));
    put(&p.config.use_pot2, sizeof(p.config.use_pot2));
    put(p.scale_W, channels * sizeof(float));
    put(p.scale_R, channels * sizeof(float));
    put(p.scale_bw, channels * sizeof(float));
    put(p.scale_br, channels * sizeof(float));
    return key;
}

// src/gru_forward_cpu_quant.cc:220-297 (fillLinearParamsCPU / fillGateParamsCPU)
std::shared_ptr<const Exec> buildExec(const rxmet_gru_quant_params &p) {
    auto exec = std::make_shared<Exec>();
    const int hidden = p.hidden, channels = 3 * hidden;
    const ScaleMode mode(p.config.use_pot2 != 0);
    exec->hidden = hidden;
    GateExec &g = exec->gate;
    for (int op = 0; op < kOps; ++op) {
        const Width w = widthOf(p.config, op);
        g.zp[op] = p.zero_point[op];
        g.qlo[op] = w.lo();
        g.qhi[op] = w.hi();
        g.eff[op] = 0.0f;
        const bool perChannel = op == RXMET_GRU_W || op == RXMET_GRU_R || op == RXMET_GRU_BW || op == RXMET_GRU_BR;
        if (!perChannel) {
            RXMET_REQUIRE(p.scale[op] > 0.0f, "scale of quantization point %d must be > 0", op);
            g.eff[op] = mode.effective(p.scale[op]);
        }
    }
    const float *s = p.scale;
    g.ih_to_update = mode.ratio(s[RXMET_GRU_WEIGHT_IH_LINEAR], s[RXMET_GRU_UPDATE_GATE_INPUT]);
    g.hh_to_update = mode.ratio(s[RXMET_GRU_WEIGHT_HH_LINEAR], s[RXMET_GRU_UPDATE_GATE_INPUT]);
    g.ih_to_reset = mode.ratio(s[RXMET_GRU_WEIGHT_IH_LINEAR], s[RXMET_GRU_RESET_GATE_INPUT]);
    g.hh_to_reset = mode.ratio(s[RXMET_GRU_WEIGHT_HH_LINEAR], s[RXMET_GRU_RESET_GATE_INPUT]);
    g.ih_to_new = mode.ratio(s[RXMET_GRU_WEIGHT_IH_LINEAR], s[RXMET_GRU_NEW_GATE_INPUT]);
    g.rh_to_new = mode.productTo(s[RXMET_GRU_RESET_GATE_OUTPUT], s[RXMET_GRU_WEIGHT_HH_LINEAR], s[RXMET_GRU_NEW_GATE_INPUT]);
    g.new_to_h = mode.ratio(s[RXMET_GRU_NEW_GATE_OUTPUT], s[RXMET_GRU_H]);
    g.update_old_to_h = mode.productTo(s[RXMET_GRU_UPDATE_GATE_OUTPUT], s[RXMET_GRU_H], s[RXMET_GRU_H]);
    g.quant_one = static_cast<int32_t>(std::rint(1.0f / s[RXMET_GRU_UPDATE_GATE_OUTPUT])) +
                  p.zero_point[RXMET_GRU_UPDATE_GATE_OUTPUT];
    const Luts luts = makeLuts(p);
    g.lut_update = luts.update;
    g.lut_reset = luts.reset;
    g.lut_new = luts.fresh;

    ChannelExec &c = exec->chan;
    c.eff_W.resize(channels); c.eff_R.resize(channels); c.eff_bw.resize(channels); c.eff_br.resize(channels);
    c.gemm_x.resize(channels); c.bias_x.resize(channels); c.gemm_h.resize(channels); c.bias_h.resize(channels);
    RXMET_REQUIRE(p.scale_W && p.scale_R && p.scale_bw && p.scale_br, "per-channel scale arrays are not set");
    for (int ch = 0; ch < channels; ++ch) {
        c.eff_W[ch] = mode.effective(p.scale_W[ch]);
        c.eff_R[ch] = mode.effective(p.scale_R[ch]);
        c.eff_bw[ch] = mode.effective(p.scale_bw[ch]);
        c.eff_br[ch] = mode.effective(p.scale_br[ch]);
        c.gemm_x[ch] = mode.productTo(p.scale_W[ch], s[RXMET_GRU_X], s[RXMET_GRU_WEIGHT_IH_LINEAR]);
        c.bias_x[ch] = mode.toProduct(p.scale_bw[ch], p.scale_W[ch], s[RXMET_GRU_X]);
        c.gemm_h[ch] = mode.productTo(p.scale_R[ch], s[RXMET_GRU_H], s[RXMET_GRU_WEIGHT_HH_LINEAR]);
        c.bias_h[ch] = mode.toProduct(p.scale_br[ch], p.scale_R[ch], s[RXMET_GRU_H]);
    }
    exec->weightClass = wider(classOf(widthOf(p.config, RXMET_GRU_W)), classOf(widthOf(p.config, RXMET_GRU_R)));
    exec->actClass = wider(classOf(widthOf(p.config, RXMET_GRU_X)), classOf(widthOf(p.config, RXMET_GRU_H)));
    exec->linearClass = wider(CodeClass::I16, wider(classOf(widthOf(p.config, RXMET_GRU_WEIGHT_IH_LINEAR)),
                                                    classOf(widthOf(p.config, RXMET_GRU_WEIGHT_HH_LINEAR))));
    return exec;
}

}  // namespace

void buildLuts(const rxmet_gru_quant_params &p, rxmet_lut_segment out[3][16]) {
    const Luts luts = makeLuts(p);
    const Lut *all[3] = {&luts.update, &luts.reset, &luts.fresh};
    for (int t = 0; t < 3; ++t)
        for (int s = 0; s < kSegments; ++s)
            out[t][s] = rxmet_lut_segment{all[t]->q_b[s], all[t]->n_bx[s], all[t]->term_c[s], all[t]->threshold[s]};
}

float decodeEffectiveScale(float scale, bool usePot2) {
    RXMET_REQUIRE(scale > 0.0f, "scale must be > 0");
    return ScaleMode(usePot2).effective(scale);
}

std::shared_ptr<const Exec> deriveExec(const rxmet_gru_quant_params &p) {
    RXMET_REQUIRE(p.hidden > 0, "quant params: hidden must be > 0");
    static std::mutex mutex;
    static std::list<std::pair<std::string, std::shared_ptr<const Exec>>> cache;  // most recent first
    const std::string key = cacheKey(p);
    {
        std::lock_guard<std::mutex> lock(mutex);
        for (auto it = cache.begin(); it != cache.end(); ++it) {
            if (it->first == key) {
                cache.splice(cache.begin(), cache, it);
                return cache.front().second;
            }
        }
    }
    std::shared_ptr<const Exec> exec = buildExec(p);
    std::lock_guard<std::mutex> lock(mutex);
    cache.emplace_front(key, exec);
    if (cache.size() > 16) cache.pop_back();
    return exec;
}

// Every ratio is ONE float division of float scales (products of two scales are rounded to float first), as the
// reference computes them on the host; this file is compiled without FMA contraction.
FpCarrierParams deriveFpCarrier(const rxmet_gru_quant_params &p) {
    FpCarrierParams out;
    FpCarrierScalars &s = out.s;
    for (int op = 0; op < kOps; ++op) {
        s.zp[op] = static_cast<float>(p.zero_point[op]);
        const int bits = p.config.bits[op];
        const int64_t qmin = p.config.is_unsigned[op] ? 0 : -(int64_t{1} << (bits - 1));
        const int64_t qmax = p.config.is_unsigned[op] ? (int64_t{1} << bits) - 1 : (int64_t{1} << (bits - 1)) - 1;
        float lo = static_cast<float>(qmin), hi = static_cast<float>(qmax);
        if (static_cast<double>(lo) < static_cast<double>(qmin)) lo = std::nextafterf(lo, INFINITY);
        if (static_cast<double>(hi) > static_cast<double>(qmax)) hi = std::nextafterf(hi, -INFINITY);
        s.lo[op] = lo;
        s.hi[op] = hi;
    }
    auto ratio = [](float src, float dst) { return src / dst; };
    const float *sc = p.scale;
    s.ihToUpdate = ratio(sc[RXMET_GRU_WEIGHT_IH_LINEAR], sc[RXMET_GRU_UPDATE_GATE_INPUT]);
    s.hhToUpdate = ratio(sc[RXMET_GRU_WEIGHT_HH_LINEAR], sc[RXMET_GRU_UPDATE_GATE_INPUT]);
    s.ihToReset = ratio(sc[RXMET_GRU_WEIGHT_IH_LINEAR], sc[RXMET_GRU_RESET_GATE_INPUT]);
    s.hhToReset = ratio(sc[RXMET_GRU_WEIGHT_HH_LINEAR], sc[RXMET_GRU_RESET_GATE_INPUT]);
    s.ihToNew = ratio(sc[RXMET_GRU_WEIGHT_IH_LINEAR], sc[RXMET_GRU_NEW_GATE_INPUT]);
    {
        const float product = sc[RXMET_GRU_RESET_GATE_OUTPUT] * sc[RXMET_GRU_WEIGHT_HH_LINEAR];
        s.rhToNew = ratio(product, sc[RXMET_GRU_NEW_GATE_INPUT]);
    }
    s.quantOne = rintf(1.0f / sc[RXMET_GRU_UPDATE_GATE_OUTPUT]) + static_cast<float>(p.zero_point[RXMET_GRU_UPDATE_GATE_OUTPUT]);
    {
        const float product = sc[RXMET_GRU_UPDATE_GATE_OUTPUT] * sc[RXMET_GRU_H];
        s.updateOldToH = ratio(product, sc[RXMET_GRU_H]);
    }
    s.newToH = ratio(sc[RXMET_GRU_NEW_GATE_OUTPUT], sc[RXMET_GRU_H]);
    const size_t C = 3 * static_cast<size_t>(p.hidden);
    out.channel.resize(4 * C);
    for (size_t c = 0; c < C; ++c) {
        const float wx = p.scale_W[c] * sc[RXMET_GRU_X];
        out.channel[c] = ratio(wx, sc[RXMET_GRU_WEIGHT_IH_LINEAR]);
        out.channel[C + c] = ratio(p.scale_bw[c], wx);
        const float rh = p.scale_R[c] * sc[RXMET_GRU_H];
        out.channel[2 * C + c] = ratio(rh, sc[RXMET_GRU_WEIGHT_HH_LINEAR]);
        out.channel[3 * C + c] = ratio(p.scale_br[c], rh);
    }
    return out;
}

}  // namespace gru
}  // namespace rxmet
