// Host-side parameter logic of the QuantLSTM path.  Compiled by g++ without FMA contraction:
// the float roundings here decide integer codes.
//
// Follows operators/quant-lstm/src/quantization/scale_encoding.cc (ranges -> scale / zero point,
// M+shift and power-of-two encodings), src/lstm/quant_params.cc (finalisation per granularity) and
// src/lstm/lstm_execution_params.cc (execution encodings and the float-exactness classes).
#include "lstm_params.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <limits>
#include <map>
#include <mutex>
#include <string>

#include "common.h"

namespace rxmet {
namespace lstm {
namespace {

bool isParameter(int op) { return op >= RXMET_LSTM_WEIGHT_IH && op <= RXMET_LSTM_BIAS_HH; }
bool isBias(int op) { return op == RXMET_LSTM_BIAS_IH || op == RXMET_LSTM_BIAS_HH; }

void checkConfig(const rxmet_lstm_quant_config &cfg) {
    RXMET_REQUIRE(cfg.scale_mode == RXMET_LSTM_SCALE_AFFINE || cfg.scale_mode == RXMET_LSTM_SCALE_POT2,
                  "scale_mode must be affine or pot2");
    for (int op = 0; op < kOps; ++op) {
        const int bits = cfg.bitwidth[op];
        RXMET_REQUIRE(bits >= 1 && bits <= 32, "operator bitwidth must be in [1, 32]");
        RXMET_REQUIRE(!(cfg.is_unsigned[op] && bits == 32), "UINT32 exceeds the int32 quantization metadata range");
        RXMET_REQUIRE(!(!cfg.is_unsigned[op] && cfg.is_symmetric[op] && bits == 1),
                      "signed symmetric INT1 has qmax=0 and is unsupported");
        RXMET_REQUIRE(cfg.granularity[op] <= RXMET_LSTM_PER_CHANNEL, "bad granularity");
        RXMET_REQUIRE(isParameter(op) || cfg.granularity[op] == RXMET_LSTM_PER_TENSOR,
                      "activation points are per tensor");
        RXMET_REQUIRE(!isParameter(op) || (cfg.is_symmetric[op] && !cfg.is_unsigned[op]),
                      "weights and biases are signed symmetric");
    }
}

double roundEven(double v) { return std::nearbyint(v); }

// ---- range -> scale / zero point ---------------------------------------------

struct Calibrated {
    float scale = 0.0f;
    int32_t zeroPoint = 0;
    float coveredMin = 0.0f, coveredMax = 0.0f;
};

int32_t zeroPointFor(float lower, float scale, Grid g) {
    const double candidate = static_cast<double>(g.lo) - static_cast<double>(lower) / scale;
    if (candidate <= g.lo) return g.lo;
    if (candidate >= g.hi) return g.hi;
    return static_cast<int32_t>(std::clamp<double>(roundEven(candidate), g.lo, g.hi));
}

float floorScale(Grid g) {
    const double steps = static_cast<double>(g.hi) - g.lo;
    return static_cast<float>(std::min(std::ldexp(1.0, -23), 0.01 / steps));
}

float finiteScale(double v) {
    const float s = static_cast<float>(v);
    if (!std::isfinite(s) || s <= 0.0f) fail(RXMET_ERR_INVALID_ARGUMENT, "calibrated scale is not a finite positive float");
    return s;
}

Calibrated fromMinMax(float lo, float hi, bool isUnsigned, bool symmetric, Grid g) {
    if (!std::isfinite(lo) || !std::isfinite(hi) || lo > hi)
        fail(RXMET_ERR_INVALID_ARGUMENT, "calibration range must be finite with minimum <= maximum");
    const double steps = static_cast<double>(g.hi) - g.lo;
    const float smallest = floorScale(g);
    const bool signedSym = symmetric && !isUnsigned;
    double wanted;
    if (signedSym) wanted = std::max(std::fabs(static_cast<double>(lo)), std::fabs(static_cast<double>(hi))) / g.hi;
    else if (symmetric) wanted = static_cast<double>(std::max(hi, 0.0f)) / g.hi;
    else wanted = (static_cast<double>(std::max(hi, 0.0f)) - std::min(lo, 0.0f)) / steps;
    Calibrated c;
    c.scale = wanted < static_cast<double>(smallest) ? smallest : finiteScale(wanted);
    if (signedSym) {
        const float extent = static_cast<float>(g.hi) * c.scale;
        c.coveredMin = -extent;
        c.coveredMax = extent;
    } else if (symmetric) {
        c.coveredMin = 0.0f;
        c.coveredMax = static_cast<float>(g.hi) * c.scale;
    } else {
        c.coveredMin = std::min(lo, 0.0f);
        c.coveredMax = c.coveredMin + static_cast<float>(steps) * c.scale;
    }
    c.zeroPoint = symmetric ? 0 : zeroPointFor(c.coveredMin, c.scale, g);
    return c;
}

void snapToPowerOfTwo(Calibrated *c, bool symmetric, Grid g) {
    const double span = std::fabs(static_cast<double>(c->coveredMax) - static_cast<double>(c->coveredMin));
    if (!std::isfinite(span) || span <= 0.0) fail(RXMET_ERR_INVALID_ARGUMENT, "pot2 needs a finite positive range");
    const double nearestPower = std::ldexp(1.0, static_cast<int>(roundEven(std::log2(span))));
    const bool nearPower = std::fabs(span - nearestPower) / nearestPower < 0.02;
    const double e = -std::log2(static_cast<double>(c->scale));
    const double chosen = nearPower ? roundEven(e) : std::floor(e);
    if (!std::isfinite(chosen) || chosen < -128 || chosen > 127) fail(RXMET_ERR_INVALID_ARGUMENT, "pot2 exponent exceeds int8");
    c->scale = finiteScale(std::ldexp(1.0, -static_cast<int>(chosen)));
    c->zeroPoint = symmetric ? 0 : zeroPointFor(c->coveredMin, c->scale, g);
}

Calibrated calibratePoint(const rxmet_lstm_quant_config &cfg, int op, float lo, float hi) {
    const Grid g = gridOf(cfg, op);
    Calibrated c = fromMinMax(lo, hi, cfg.is_unsigned[op] != 0, cfg.is_symmetric[op] != 0, g);
    if (cfg.scale_mode == RXMET_LSTM_SCALE_POT2) snapToPowerOfTwo(&c, cfg.is_symmetric[op] != 0, g);
    if (isBias(op)) {
        // biases keep a factor-two headroom (quant_params.cc:37-51)
        const double extent = std::max(std::fabs(static_cast<double>(lo)), std::fabs(static_cast<double>(hi)));
        double s = std::max(2.0 * extent, 0.01) / g.hi;
        if (cfg.scale_mode == RXMET_LSTM_SCALE_POT2) s = std::exp2(std::ceil(std::log2(s)));
        c.scale = finiteScale(s);
    }
    return c;
}

// ---- scale -> rescale encodings -------------------------------------------------

rxmet_lstm_rescale mShift(double ratio) {
    if (!std::isfinite(ratio) || ratio <= 0.0) fail(RXMET_ERR_INVALID_ARGUMENT, "rescale ratio must be finite and positive");
    int exponent = 0;
    const double mantissa = std::frexp(ratio, &exponent);
    long long m = static_cast<long long>(roundEven(mantissa * 65536.0));
    if (m == 65536) {
        m = 32768;
        ++exponent;
    }
    const int shift = 16 - exponent;
    if (shift < -128 || shift > 127) fail(RXMET_ERR_INVALID_ARGUMENT, "M+shift shift exceeds int8");
    return {1, static_cast<int32_t>(m), shift};
}

int exactExponent(float scale) {
    int e = 0;
    if (!(scale > 0.0f) || !std::isfinite(scale) || std::frexp(scale, &e) != 0.5f)
        fail(RXMET_ERR_INVALID_ARGUMENT, "pot2 rescale needs exact power-of-two scales");
    return e;
}

rxmet_lstm_rescale between(int mode, float from, float to) {
    if (mode == RXMET_LSTM_SCALE_AFFINE) return mShift(static_cast<double>(from) / to);
    const int shift = exactExponent(to) - exactExponent(from);
    if (shift < -128 || shift > 127) fail(RXMET_ERR_INVALID_ARGUMENT, "pot2 rescale shift exceeds int8");
    return {0, 1, shift};
}

float scaleProduct(float a, float b) {
    const float r = static_cast<float>(static_cast<double>(a) * b);
    if (!std::isfinite(r) || r <= 0.0f) fail(RXMET_ERR_INVALID_ARGUMENT, "product of scales is not a finite positive float");
    return r;
}

rxmet_lstm_cell_scale cellRatio(double ratio) {
    if (!std::isfinite(ratio) || ratio <= 0.0) fail(RXMET_ERR_INVALID_ARGUMENT, "cell ratio must be finite and positive");
    rxmet_lstm_cell_scale s{};
    const double q31 = std::ldexp(ratio, 31);
    if (std::isfinite(q31) && q31 > 0.5 && q31 < static_cast<double>(std::numeric_limits<int64_t>::max())) {
        s.multiplier = static_cast<int64_t>(roundEven(q31));
        return s;
    }
    int e = 0;
    s.fp_mantissa = std::frexp(ratio, &e);
    s.fp_exponent = e;
    s.uses_fp_scale = 1;
    return s;
}

// ---- float exactness bookkeeping --------------------------------------------------

uint64_t absOf(int64_t v) { return v < 0 ? uint64_t{0} - static_cast<uint64_t>(v) : static_cast<uint64_t>(v); }

uint64_t largestCentered(Grid g, int32_t zp) {
    return std::max(absOf(static_cast<int64_t>(g.lo) - zp), absOf(static_cast<int64_t>(g.hi) - zp));
}
uint64_t largestRaw(Grid g) { return std::max(absOf(g.lo), absOf(g.hi)); }

struct Bounds {
    long double widest = 0;     // largest intermediate magnitude
    long double precision = 0;  // largest value * odd part of a multiplier
    long double through(long double source, const rxmet_lstm_rescale &r) {
        unsigned m = r.is_m_shift ? static_cast<unsigned>(r.multiplier) : 1u;
        const long double scaled = source * m;
        while (m != 0 && (m & 1u) == 0) m >>= 1;
        precision = std::max(precision, source * m);
        const long double result = std::ceil(std::ldexp(scaled, -r.shift));
        widest = std::max({widest, scaled, result});
        return result;
    }
};

constexpr long double kExactLimit = 16777216.0L;  // 2^24
bool exactClass(long double accumulator, long double precision) { return accumulator < kExactLimit && precision < kExactLimit; }

struct LinearSide {
    int inOp, wOp, bOp, outOp;
    uint64_t reduction;
    const float *wScale, *bScale;
    rxmet_lstm_rescale *biasToAcc, *accToOut;
};

// Returns {all channels in the reference's "exact integer range" class, integer accumulator < 2^24}.
std::pair<bool, bool> deriveLinear(const rxmet_lstm_quant_params &p, const LinearSide &s, std::vector<rxmet_lstm_rescale> *b2a,
                                   std::vector<rxmet_lstm_rescale> *a2o) {
    const auto &cfg = p.config;
    const Grid gin = gridOf(cfg, s.inOp), gw = gridOf(cfg, s.wOp), gb = gridOf(cfg, s.bOp);
    bool allExact = true, accExact = true;
    const int channels = 4 * p.hidden_size;
    RXMET_REQUIRE(s.wScale != nullptr && (!p.bias_enabled || s.bScale != nullptr), "per-channel scale arrays missing");
    for (int ch = 0; ch < channels; ++ch) {
        const float accScale = scaleProduct(p.scale[s.inOp], s.wScale[ch]);
        const rxmet_lstm_rescale out = between(cfg.scale_mode, accScale, p.scale[s.outOp]);
        (*a2o)[ch] = out;
        long double bound = static_cast<long double>(s.reduction) * largestCentered(gin, p.zero_point[s.inOp]) * largestCentered(gw, 0);
        const long double weightSum = static_cast<long double>(s.reduction) * largestRaw(gw);
        const long double rawGemm = weightSum * largestRaw(gin);
        const long double zpCorrection = weightSum * absOf(p.zero_point[s.inOp]);
        Bounds track;
        track.widest = std::max(bound, rawGemm + zpCorrection);
        if (p.bias_enabled) {
            const rxmet_lstm_rescale b = between(cfg.scale_mode, s.bScale[ch], accScale);
            (*b2a)[ch] = b;
            bound += track.through(static_cast<long double>(largestCentered(gb, 0)), b);
        }
        const long double outBound = track.through(bound, out);
        const long double accumulator = std::max({bound, rawGemm, zpCorrection, outBound + absOf(p.zero_point[s.outOp])});
        allExact = allExact && exactClass(accumulator, track.precision);
        accExact = accExact && std::max({bound, rawGemm + zpCorrection}) < kExactLimit;
    }
    return {allExact, accExact};
}

struct Derived {
    rxmet_lstm_execution scalar{};
    std::vector<rxmet_lstm_rescale> ihB2a, ihA2o, hhB2a, hhA2o;
    bool referenceExact = false;  // the reference's ExactIntegerRange class everywhere
    bool accumulatorsExact = false;
};

Derived derive(const rxmet_lstm_quant_params &p, bool requireExact) {
    const auto &cfg = p.config;
    checkConfig(cfg);
    RXMET_REQUIRE(p.input_size > 0 && p.hidden_size > 0, "input_size and hidden_size must be positive");
    for (int op = 0; op < kOps; ++op) {
        if (isParameter(op)) continue;
        const Grid g = gridOf(cfg, op);
        RXMET_REQUIRE(std::isfinite(p.scale[op]) && p.scale[op] > 0.0f, "scale of point %d must be finite and positive", op);
        RXMET_REQUIRE(p.zero_point[op] >= g.lo && p.zero_point[op] <= g.hi, "zero point of point %d outside its grid", op);
        RXMET_REQUIRE(!cfg.is_symmetric[op] || p.zero_point[op] == 0, "symmetric point %d needs zero point 0", op);
    }
    Derived d;
    const size_t channels = 4 * static_cast<size_t>(p.hidden_size);
    d.ihB2a.assign(channels, {0, 1, 0});
    d.ihA2o = d.hhB2a = d.hhA2o = d.ihB2a;
    const LinearSide ih{RXMET_LSTM_INPUT, RXMET_LSTM_WEIGHT_IH, RXMET_LSTM_BIAS_IH, RXMET_LSTM_WEIGHT_IH_LINEAR,
                        static_cast<uint64_t>(p.input_size), p.weight_ih_scale, p.bias_ih_scale, nullptr, nullptr};
    const LinearSide hh{RXMET_LSTM_OUTPUT, RXMET_LSTM_WEIGHT_HH, RXMET_LSTM_BIAS_HH, RXMET_LSTM_WEIGHT_HH_LINEAR,
                        static_cast<uint64_t>(p.hidden_size), p.weight_hh_scale, p.bias_hh_scale, nullptr, nullptr};
    const auto a = deriveLinear(p, ih, &d.ihB2a, &d.ihA2o);
    const auto b = deriveLinear(p, hh, &d.hhB2a, &d.hhA2o);
    bool exact = a.first && b.first;
    d.accumulatorsExact = a.second && b.second;

    const int ihLin = RXMET_LSTM_WEIGHT_IH_LINEAR, hhLin = RXMET_LSTM_WEIGHT_HH_LINEAR;
    for (int g = 0; g < 4; ++g) {
        const int gi = RXMET_LSTM_INPUT_GATE_INPUT + g;
        d.scalar.ih_to_gate[g] = between(cfg.scale_mode, p.scale[ihLin], p.scale[gi]);
        d.scalar.hh_to_gate[g] = between(cfg.scale_mode, p.scale[hhLin], p.scale[gi]);
        Bounds track;
        const long double l = track.through(static_cast<long double>(largestCentered(gridOf(cfg, ihLin), p.zero_point[ihLin])),
                                            d.scalar.ih_to_gate[g]);
        const long double r = track.through(static_cast<long double>(largestCentered(gridOf(cfg, hhLin), p.zero_point[hhLin])),
                                            d.scalar.hh_to_gate[g]);
        exact = exact && exactClass(l + r + absOf(p.zero_point[gi]), track.precision);
    }
    const int fo = RXMET_LSTM_FORGET_GATE_OUTPUT, io = RXMET_LSTM_INPUT_GATE_OUTPUT, go = RXMET_LSTM_CELL_GATE_OUTPUT;
    const int oo = RXMET_LSTM_OUTPUT_GATE_OUTPUT, cs = RXMET_LSTM_CELL_STATE, ct = RXMET_LSTM_CELL_TANH_OUTPUT;
    d.scalar.forget_scale = cellRatio(static_cast<double>(p.scale[fo]) * p.scale[cs] / p.scale[cs]);
    d.scalar.input_scale = cellRatio(static_cast<double>(p.scale[io]) * p.scale[go] / p.scale[cs]);
    {
        auto ratioOf = [](const rxmet_lstm_cell_scale &s) {
            return s.uses_fp_scale ? std::ldexp(static_cast<long double>(s.fp_mantissa), s.fp_exponent)
                                   : std::ldexp(static_cast<long double>(s.multiplier), -31);
        };
        const uint64_t lhs = std::max(largestCentered(gridOf(cfg, fo), p.zero_point[fo]), largestCentered(gridOf(cfg, io), p.zero_point[io]));
        const uint64_t rhs = std::max(largestCentered(gridOf(cfg, cs), p.zero_point[cs]), largestCentered(gridOf(cfg, go), p.zero_point[go]));
        const long double product = static_cast<long double>(lhs) * rhs;
        const long double summed = std::ceil(product * (ratioOf(d.scalar.forget_scale) + ratioOf(d.scalar.input_scale))) + absOf(p.zero_point[cs]);
        exact = exact && exactClass(std::max(product, summed), 0);
    }
    d.scalar.product_to_output = between(cfg.scale_mode, scaleProduct(p.scale[oo], p.scale[ct]), p.scale[RXMET_LSTM_OUTPUT]);
    {
        const long double product = static_cast<long double>(largestCentered(gridOf(cfg, oo), p.zero_point[oo])) *
                                    largestCentered(gridOf(cfg, ct), p.zero_point[ct]);
        Bounds track;
        track.widest = product;
        const long double rescaled = track.through(product, d.scalar.product_to_output);
        exact = exact && exactClass(std::max(product, rescaled + absOf(p.zero_point[RXMET_LSTM_OUTPUT])), track.precision);
    }
    d.referenceExact = exact;
    d.scalar.exact_accumulation = exact ? 1 : 0;
    if (requireExact && !exact)
        fail(RXMET_ERR_INVALID_ARGUMENT, "require_exact_accumulation rejects a configuration with float precision risk");
    return d;
}

// ---- activation tables (host libm, the same functions the reference's CPU path calls) -----------

float sigmoidReal(float v) {
    if (v >= 0.0f) {
        const float e = std::exp(-v);
        return 1.0f / (1.0f + e);
    }
    const float e = std::exp(v);
    return e / (1.0f + e);
}

void buildTable(const rxmet_lstm_quant_params &p, int inOp, int outOp, bool isTanh, int32_t *table) {
    const Grid gi = gridOf(p.config, inOp), g = gridOf(p.config, outOp);
    for (int64_t q = gi.lo; q <= gi.hi; ++q) {
        const float real = static_cast<float>((static_cast<double>(q) - p.zero_point[inOp]) * static_cast<double>(p.scale[inOp]));
        const float act = isTanh ? std::tanh(real) : sigmoidReal(real);
        const double t = roundEven(static_cast<double>(act) / static_cast<double>(p.scale[outOp])) + p.zero_point[outOp];
        const bool clamped = t < g.lo || t > g.hi;
        const int32_t code = static_cast<int32_t>(t <= g.lo ? g.lo : (t >= g.hi ? g.hi : t));
        table[q - gi.lo] = ((code - p.zero_point[outOp]) * 2) | (clamped ? 1 : 0);
    }
}

DevRescale device(const rxmet_lstm_rescale &r) {
    return {r.is_m_shift ? static_cast<float>(r.multiplier) : 1.0f, std::ldexp(1.0f, -r.shift)};
}

}  // namespace

Grid gridOfBits(int bits, bool isUnsigned) {
    if (isUnsigned) return {0, static_cast<int32_t>((uint64_t{1} << bits) - 1u)};
    const int32_t hi = static_cast<int32_t>((uint64_t{1} << (bits - 1)) - 1u);
    return {-hi - 1, hi};
}

Grid gridOf(const rxmet_lstm_quant_config &cfg, int op) { return gridOfBits(cfg.bitwidth[op], cfg.is_unsigned[op] != 0); }

MinMaxParam minMaxParam(float lo, float hi, int bits, bool isUnsigned, bool symmetric) {
    const Calibrated c = fromMinMax(lo, hi, isUnsigned, symmetric, gridOfBits(bits, isUnsigned));
    return {c.scale, c.zeroPoint};
}

void defaultConfig(rxmet_lstm_quant_config *cfg) {
    std::memset(cfg, 0, sizeof(*cfg));
    cfg->scale_mode = RXMET_LSTM_SCALE_AFFINE;
    for (int op = 0; op < kOps; ++op) {
        cfg->bitwidth[op] = 8;
        cfg->is_symmetric[op] = 1;
        cfg->is_unsigned[op] = (op == RXMET_LSTM_INPUT_GATE_OUTPUT || op == RXMET_LSTM_FORGET_GATE_OUTPUT ||
                                op == RXMET_LSTM_OUTPUT_GATE_OUTPUT);
        cfg->granularity[op] = isParameter(op) ? RXMET_LSTM_PER_CHANNEL : RXMET_LSTM_PER_TENSOR;
    }
}

void rangesReset(rxmet_lstm_ranges *r, int hidden) {
    const float inf = std::numeric_limits<float>::infinity();
    for (int op = 0; op < kOps; ++op) { r->minimum[op] = inf; r->maximum[op] = -inf; }
    for (int k = 0; k < 3; ++k) { r->contribution_min[k] = inf; r->contribution_max[k] = -inf; }
    for (int s = 0; s < 4; ++s)
        for (int ch = 0; ch < 4 * hidden; ++ch) {
            if (r->channel_min[s]) r->channel_min[s][ch] = inf;
            if (r->channel_max[s]) r->channel_max[s][ch] = -inf;
        }
}

void paramsFromRanges(const rxmet_lstm_quant_config &cfg, const rxmet_lstm_ranges &ranges, int inputSize, int hidden,
                      bool bias, float *wIhScale, float *wHhScale, float *bIhScale, float *bHhScale,
                      rxmet_lstm_quant_params *out) {
    checkConfig(cfg);
    RXMET_REQUIRE(inputSize > 0 && hidden > 0, "input_size and hidden_size must be positive");
    float *dst[4] = {wIhScale, wHhScale, bIhScale, bHhScale};
    std::memset(out, 0, sizeof(*out));
    out->config = cfg;
    out->input_size = inputSize;
    out->hidden_size = hidden;
    out->bias_enabled = bias ? 1 : 0;
    const int channels = 4 * hidden;
    for (int op = 0; op < kOps; ++op) {
        if (!bias && isBias(op)) continue;
        if (!isParameter(op)) {
            const Calibrated c = calibratePoint(cfg, op, ranges.minimum[op], ranges.maximum[op]);
            out->scale[op] = c.scale;
            out->zero_point[op] = c.zeroPoint;
            continue;
        }
        const int slot = op - RXMET_LSTM_WEIGHT_IH;
        RXMET_REQUIRE(dst[slot] && ranges.channel_min[slot] && ranges.channel_max[slot], "per-channel arrays missing");
        const int span = cfg.granularity[op] == RXMET_LSTM_PER_TENSOR ? channels
                         : (cfg.granularity[op] == RXMET_LSTM_PER_GATE ? hidden : 1);
        for (int first = 0; first < channels; first += span) {
            float lo = std::numeric_limits<float>::infinity(), hi = -lo;
            for (int ch = first; ch < first + span; ++ch) {
                lo = std::min(lo, ranges.channel_min[slot][ch]);
                hi = std::max(hi, ranges.channel_max[slot][ch]);
            }
            const Calibrated c = calibratePoint(cfg, op, lo, hi);
            std::fill(dst[slot] + first, dst[slot] + first + span, c.scale);
        }
    }
    out->weight_ih_scale = wIhScale;
    out->weight_hh_scale = wHhScale;
    out->bias_ih_scale = bias ? bIhScale : nullptr;
    out->bias_hh_scale = bias ? bHhScale : nullptr;
}

void deriveExecution(const rxmet_lstm_quant_params &params, bool requireExact, rxmet_lstm_execution *out) {
    const Derived d = derive(params, requireExact);
    rxmet_lstm_rescale *keep[4] = {out->ih_bias_to_accumulator, out->ih_accumulator_to_output, out->hh_bias_to_accumulator,
                                   out->hh_accumulator_to_output};
    *out = d.scalar;
    out->ih_bias_to_accumulator = keep[0];
    out->ih_accumulator_to_output = keep[1];
    out->hh_bias_to_accumulator = keep[2];
    out->hh_accumulator_to_output = keep[3];
    const std::vector<rxmet_lstm_rescale> *src[4] = {&d.ihB2a, &d.ihA2o, &d.hhB2a, &d.hhA2o};
    for (int k = 0; k < 4; ++k) {
        if (!keep[k]) continue;
        if ((k == 0 || k == 2) && !params.bias_enabled) continue;
        std::copy(src[k]->begin(), src[k]->end(), keep[k]);
    }
}

size_t statsFloats(int hidden) { return 2 * (static_cast<size_t>(kOps) + 3 + 16 * static_cast<size_t>(hidden)); }

void foldStats(rxmet_lstm_ranges *r, const float *stats, int hidden, bool bias) {
    const size_t half = statsFloats(hidden) / 2;
    const float *mins = stats, *maxs = stats + half;
    auto usable = [](float lo, float hi) { return std::isfinite(lo) && std::isfinite(hi) && lo <= hi; };
    for (int op = 0; op < kOps; ++op) {
        if (isParameter(op) || !usable(mins[op], maxs[op])) continue;
        r->minimum[op] = std::min(r->minimum[op], mins[op]);
        r->maximum[op] = std::max(r->maximum[op], maxs[op]);
    }
    for (int k = 0; k < 3; ++k) {
        if (!usable(mins[kOps + k], maxs[kOps + k])) continue;
        r->contribution_min[k] = std::min(r->contribution_min[k], mins[kOps + k]);
        r->contribution_max[k] = std::max(r->contribution_max[k], maxs[kOps + k]);
    }
    const int channels = 4 * hidden;
    for (int s = 0; s < (bias ? 4 : 2); ++s)
        for (int ch = 0; ch < channels; ++ch) {
            const size_t i = kOps + 3 + static_cast<size_t>(s) * channels + ch;
            if (!usable(mins[i], maxs[i])) continue;
            r->channel_min[s][ch] = std::min(r->channel_min[s][ch], mins[i]);
            r->channel_max[s][ch] = std::max(r->channel_max[s][ch], maxs[i]);
        }
}

std::shared_ptr<const Exec> deriveExec(const rxmet_lstm_quant_params &p, bool requireExact) {
    static std::mutex mutex;
    static std::map<std::string, std::shared_ptr<const Exec>> cache;
    const size_t channels = 4 * static_cast<size_t>(std::max(p.hidden_size, 0));
    std::string key(reinterpret_cast<const char *>(&p), offsetof(rxmet_lstm_quant_params, weight_ih_scale));
    RXMET_REQUIRE(p.weight_ih_scale && p.weight_hh_scale, "weight scale arrays missing");
    RXMET_REQUIRE(!p.bias_enabled || (p.bias_ih_scale && p.bias_hh_scale), "bias scale arrays missing");
    const float *arrays[4] = {p.weight_ih_scale, p.weight_hh_scale, p.bias_enabled ? p.bias_ih_scale : nullptr,
                              p.bias_enabled ? p.bias_hh_scale : nullptr};
    for (const float *a : arrays)
        if (a) key.append(reinterpret_cast<const char *>(a), channels * sizeof(float));
    key.push_back(requireExact ? 1 : 0);
    {
        std::lock_guard<std::mutex> lock(mutex);
        auto it = cache.find(key);
        if (it != cache.end()) return it->second;
    }
    const Derived d = derive(p, requireExact);
    auto e = std::make_shared<Exec>();
    e->hidden = p.hidden_size;
    e->exactAccumulators = d.accumulatorsExact;
    ScalarExec &s = e->scalar;
    for (int op = 0; op < kOps; ++op) {
        const Grid g = gridOf(p.config, op);
        s.zp[op] = isParameter(op) ? 0 : p.zero_point[op];
        s.zpF[op] = static_cast<float>(s.zp[op]);
        s.lo[op] = g.lo;
        s.hi[op] = g.hi;
        s.scale[op] = isParameter(op) ? 0.0f : p.scale[op];
    }
    for (int g = 0; g < 4; ++g) {
        s.ihToGate[g] = device(d.scalar.ih_to_gate[g]);
        s.hhToGate[g] = device(d.scalar.hh_to_gate[g]);
    }
    s.productToOutput = device(d.scalar.product_to_output);
    s.forgetRatio = std::ldexp(static_cast<float>(d.scalar.forget_scale.multiplier), -31);
    s.inputRatio = std::ldexp(static_cast<float>(d.scalar.input_scale.multiplier), -31);
    s.forgetMantissa = d.scalar.forget_scale.fp_mantissa;
    s.inputMantissa = d.scalar.input_scale.fp_mantissa;
    s.forgetExponent = d.scalar.forget_scale.fp_exponent;
    s.inputExponent = d.scalar.input_scale.fp_exponent;
    s.forgetUsesFp = d.scalar.forget_scale.uses_fp_scale;
    s.inputUsesFp = d.scalar.input_scale.uses_fp_scale;
    // a grid that starts at 0 is stored shifted by half its width so that it fits a signed byte
    s.xShift = s.lo[RXMET_LSTM_INPUT] >= 0 ? (s.hi[RXMET_LSTM_INPUT] + 1) / 2 : 0;
    s.hShift = s.lo[RXMET_LSTM_OUTPUT] >= 0 ? (s.hi[RXMET_LSTM_OUTPUT] + 1) / 2 : 0;
    s.biasEnabled = p.bias_enabled;
    e->channel.assign(static_cast<size_t>(kChannelFields) * channels, 0.0f);
    auto field = [&](int f) { return e->channel.data() + static_cast<size_t>(f) * channels; };
    for (size_t ch = 0; ch < channels; ++ch) {
        field(kWIhScale)[ch] = p.weight_ih_scale[ch];
        field(kWHhScale)[ch] = p.weight_hh_scale[ch];
        field(kBIhScale)[ch] = p.bias_enabled ? p.bias_ih_scale[ch] : 1.0f;
        field(kBHhScale)[ch] = p.bias_enabled ? p.bias_hh_scale[ch] : 1.0f;
        const DevRescale ib = device(d.ihB2a[ch]), hb = device(d.hhB2a[ch]);
        const DevRescale io = device(d.ihA2o[ch]), ho = device(d.hhA2o[ch]);
        field(kIhBiasMult)[ch] = ib.mult; field(kIhBiasPow2)[ch] = ib.pow2;
        field(kHhBiasMult)[ch] = hb.mult; field(kHhBiasPow2)[ch] = hb.pow2;
        field(kIhOutMult)[ch] = io.mult;  field(kIhOutPow2)[ch] = io.pow2;
        field(kHhOutMult)[ch] = ho.mult;  field(kHhOutPow2)[ch] = ho.pow2;
    }
    bool tablesFit = true;
    const int tableIn[kTables] = {RXMET_LSTM_INPUT_GATE_INPUT, RXMET_LSTM_FORGET_GATE_INPUT, RXMET_LSTM_CELL_GATE_INPUT,
                                  RXMET_LSTM_OUTPUT_GATE_INPUT, RXMET_LSTM_CELL_STATE};
    const int tableOut[kTables] = {RXMET_LSTM_INPUT_GATE_OUTPUT, RXMET_LSTM_FORGET_GATE_OUTPUT, RXMET_LSTM_CELL_GATE_OUTPUT,
                                   RXMET_LSTM_OUTPUT_GATE_OUTPUT, RXMET_LSTM_CELL_TANH_OUTPUT};
    for (int t = 0; t < kTables; ++t) tablesFit = tablesFit && p.config.bitwidth[tableIn[t]] <= 8;
    if (tablesFit) {
        e->tables.assign(static_cast<size_t>(kTables) * kTableSize, 0);
        for (int t = 0; t < kTables; ++t)
            buildTable(p, tableIn[t], tableOut[t], t == 2 || t == 4, e->tables.data() + static_cast<size_t>(t) * kTableSize);
    }
    bool wideFit = true;
    for (int t = 0; t < kTables; ++t)
        wideFit = wideFit && p.config.bitwidth[tableIn[t]] <= 16 && p.config.bitwidth[tableOut[t]] <= 24;
    if (wideFit) {
        size_t total = 0;
        for (int t = 0; t < kTables; ++t) {
            e->wide.offset[t] = static_cast<int>(total);
            total += size_t{1} << p.config.bitwidth[tableIn[t]];
        }
        e->wide.entries.assign(total, 0);
        for (int t = 0; t < kTables; ++t)
            buildTable(p, tableIn[t], tableOut[t], t == 2 || t == 4, e->wide.entries.data() + e->wide.offset[t]);
    }
    e->weightsFitBytes = p.config.bitwidth[RXMET_LSTM_WEIGHT_IH] <= 8 && p.config.bitwidth[RXMET_LSTM_WEIGHT_HH] <= 8;
    const int actBits = std::max(p.config.bitwidth[RXMET_LSTM_INPUT], p.config.bitwidth[RXMET_LSTM_OUTPUT]);
    e->activationPlanes = actBits <= 8 ? 1 : (actBits <= 16 ? 2 : 0);
    std::lock_guard<std::mutex> lock(mutex);
    if (cache.size() > 64) cache.clear();
    cache[key] = e;
    return e;
}

const int32_t *Exec::wideTablesOnDevice() const {
    int device = 0;
    RXMET_CUDA(cudaGetDevice(&device));
    std::lock_guard<std::mutex> lock(deviceLock);
    for (const auto &entry : deviceTables)
        if (entry.first == device) return entry.second.get();
    RXMET_REQUIRE(!wide.entries.empty(), "activation tables of this parameter set were not built");
    int32_t *buffer = nullptr;
    const size_t bytes = wide.entries.size() * sizeof(int32_t);
    RXMET_CUDA(cudaMalloc(reinterpret_cast<void **>(&buffer), bytes));
    std::shared_ptr<int32_t> owner(buffer, [](int32_t *ptr) { cudaFree(ptr); });
    // synchronous on purpose: the entries are pageable host memory and the buffer is shared by every stream
    RXMET_CUDA(cudaMemcpy(buffer, wide.entries.data(), bytes, cudaMemcpyHostToDevice));
    deviceTables.emplace_back(device, owner);
    return buffer;
}

}  // namespace lstm
}  // namespace rxmet
