/*
 * TEST INFRASTRUCTURE - CPU restatement of the QuantLSTM host-side parameter
 * logic of rx-met.  Used only by tests, the smoke check and the CPU legs of
 * the benchmark as the checker; never linked into the shipped library.
 *
 * Pinned against the reference's own CPU sources compiled into
 * oracle/_ref/liblstm_ref.so (tests/test_lstm_cpu.py) and against the golden
 * JSON cases of operators/quant-lstm/tests/golden/spec.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#include "lstm_oracle.h"

void orc_lstm_type_range(const rxmet_lstm_quant_config *c, int op, int32_t *lo, int32_t *hi) {
    /* operators/quant-lstm/include/quantization/bit_width.h:38-46 */
    const int bits = c->bitwidth[op];
    if (c->is_unsigned[op]) {
        *lo = 0;
        *hi = (int32_t)((1ull << bits) - 1u);
    } else {
        *hi = (int32_t)((1ull << (bits - 1)) - 1u);
        *lo = -*hi - 1;
    }
}

static int is_parameter(int op) { return op >= RXMET_LSTM_WEIGHT_IH && op <= RXMET_LSTM_BIAS_HH; }
static int is_bias(int op) { return op == RXMET_LSTM_BIAS_IH || op == RXMET_LSTM_BIAS_HH; }

/* ---- calibration: range -> (scale, zero point) ---------------------------- */

static float minimum_scale(int32_t lo, int32_t hi) {
    /* operators/quant-lstm/src/quantization/scale_encoding.cc:31-38 */
    const double steps = (double)hi - lo;
    const double a = ldexp(1.0, -23), b = 0.01 / steps;
    return (float)(a < b ? a : b);
}

static int32_t compute_zero_point(float lower, float scale, int32_t lo, int32_t hi) {
    /* scale_encoding.cc:10-22 */
    const double candidate = (double)lo - (double)lower / scale;
    if (candidate <= (double)lo) return lo;
    if (candidate >= (double)hi) return hi;
    const double r = rint(candidate);
    return (int32_t)(r < lo ? lo : (r > hi ? hi : r));
}

typedef struct {
    float scale;
    int32_t zero_point;
    float adjusted_min, adjusted_max;
} calibrated;

static calibrated calibrate_minmax(float rmin, float rmax, int is_unsigned, int is_symmetric, int32_t lo, int32_t hi) {
    /* scale_encoding.cc:39-91 */
    const double steps = (double)hi - lo;
    const float min_scale = minimum_scale(lo, hi);
    float amin = rmin, amax = rmax;
    double candidate;
    if (is_symmetric && !is_unsigned) {
        const double a = fabs((double)rmin), b = fabs((double)rmax);
        candidate = (a > b ? a : b) / hi;
    } else if (is_symmetric) {
        amin = 0.0f;
        amax = rmax > 0.0f ? rmax : 0.0f;
        candidate = (double)amax / hi;
    } else {
        amin = rmin < 0.0f ? rmin : 0.0f;
        amax = rmax > 0.0f ? rmax : 0.0f;
        candidate = ((double)amax - amin) / steps;
    }
    const int fallback = candidate < (double)min_scale;
    const float scale = fallback ? min_scale : (float)candidate;
    if (is_symmetric && !is_unsigned) {
        const float extent = (float)hi * scale;
        amin = -extent;
        amax = extent;
    } else if (is_symmetric) {
        amin = 0.0f;
        amax = (float)hi * scale;
    } else {
        amin = rmin < 0.0f ? rmin : 0.0f;
        amax = amin + (float)steps * scale;
    }
    calibrated out;
    out.scale = scale;
    out.zero_point = is_symmetric ? 0 : compute_zero_point(amin, scale, lo, hi);
    out.adjusted_min = amin;
    out.adjusted_max = amax;
    return out;
}

static void to_pot2_cover_range(calibrated *c, int is_symmetric, int32_t lo, int32_t hi) {
    /* scale_encoding.cc:143-185 */
    const double rmin = c->adjusted_min, rmax = c->adjusted_max;
    const double real_range = fabs(rmax - rmin);
    const double range_log2 = log2(real_range);
    const int nearest = (int)rint(range_log2);
    const double nearest_power = ldexp(1.0, nearest);
    const int near_power = fabs(real_range - nearest_power) / nearest_power < 0.02;
    const double exponent_value = -log2((double)c->scale);
    const double selected = near_power ? rint(exponent_value) : floor(exponent_value);
    const int exponent = (int)(int8_t)selected;
    c->scale = (float)ldexp(1.0, -exponent);
    c->zero_point = is_symmetric ? 0 : compute_zero_point(c->adjusted_min, c->scale, lo, hi);
}

static calibrated calibrate_group(float rmin, float rmax, const rxmet_lstm_quant_config *cfg, int op) {
    /* operators/quant-lstm/src/lstm/quant_params.cc:27-53 */
    int32_t lo, hi;
    orc_lstm_type_range(cfg, op, &lo, &hi);
    calibrated c = calibrate_minmax(rmin, rmax, cfg->is_unsigned[op], cfg->is_symmetric[op], lo, hi);
    if (cfg->scale_mode == RXMET_LSTM_SCALE_POT2) to_pot2_cover_range(&c, cfg->is_symmetric[op], lo, hi);
    if (is_bias(op)) {
        const double a = fabs((double)rmin), b = fabs((double)rmax);
        const double extent = a > b ? a : b;
        double scale = (2.0 * extent > 0.01 ? 2.0 * extent : 0.01) / hi;
        if (cfg->scale_mode == RXMET_LSTM_SCALE_POT2) scale = exp2(ceil(log2(scale)));
        c.scale = (float)scale;
    }
    return c;
}

int orc_lstm_params_from_ranges(const rxmet_lstm_quant_config *config, const rxmet_lstm_ranges *ranges, int I, int H,
                                int bias, float *w_ih_scale, float *w_hh_scale, float *b_ih_scale, float *b_hh_scale,
                                rxmet_lstm_quant_params *params) {
    /* quant_params.cc:222-287 */
    float *dst[4] = {w_ih_scale, w_hh_scale, b_ih_scale, b_hh_scale};
    memset(params, 0, sizeof(*params));
    params->config = *config;
    params->input_size = I;
    params->hidden_size = H;
    params->bias_enabled = bias;
    for (int op = 0; op < RXMET_LSTM_NUM_OPS; ++op) {
        if (!bias && is_bias(op)) continue;
        if (!is_parameter(op)) {
            const calibrated c = calibrate_group(ranges->minimum[op], ranges->maximum[op], config, op);
            params->scale[op] = c.scale;
            params->zero_point[op] = c.zero_point;
            continue;
        }
        const int slot = op - RXMET_LSTM_WEIGHT_IH;
        const int gran = config->granularity[op];
        const int group_size = gran == RXMET_LSTM_PER_TENSOR ? 4 * H : (gran == RXMET_LSTM_PER_GATE ? H : 1);
        for (int start = 0; start < 4 * H; start += group_size) {
            float lo = INFINITY, hi = -INFINITY;
            for (int ch = start; ch < start + group_size; ++ch) {
                if (ranges->channel_min[slot][ch] < lo) lo = ranges->channel_min[slot][ch];
                if (ranges->channel_max[slot][ch] > hi) hi = ranges->channel_max[slot][ch];
            }
            const calibrated c = calibrate_group(lo, hi, config, op);
            for (int ch = start; ch < start + group_size; ++ch) dst[slot][ch] = c.scale;
        }
    }
    params->weight_ih_scale = w_ih_scale;
    params->weight_hh_scale = w_hh_scale;
    params->bias_ih_scale = bias ? b_ih_scale : NULL;
    params->bias_hh_scale = bias ? b_hh_scale : NULL;
    return 0;
}

/* ---- execution encodings --------------------------------------------------- */

static rxmet_lstm_rescale encode_m_shift(double ratio) {
    /* scale_encoding.cc:92-113 */
    int exponent = 0;
    const double mantissa = frexp(ratio, &exponent);
    int64_t multiplier = (int64_t)rint(mantissa * 65536.0);
    if (multiplier == 65536) {
        multiplier = 32768;
        ++exponent;
    }
    rxmet_lstm_rescale r = {1, (int32_t)multiplier, 16 - exponent};
    return r;
}

static rxmet_lstm_rescale encode_pot2(float source, float destination) {
    /* scale_encoding.cc:117-142 */
    int es = 0, ed = 0;
    frexpf(source, &es);
    frexpf(destination, &ed);
    rxmet_lstm_rescale r = {0, 1, ed - es};
    return r;
}

static rxmet_lstm_rescale encode(int mode, float source, float destination) {
    /* operators/quant-lstm/src/lstm/lstm_execution_params.cc:67-80 */
    return mode == RXMET_LSTM_SCALE_AFFINE ? encode_m_shift((double)source / destination)
                                           : encode_pot2(source, destination);
}

static float product_scale(float a, float b) { return (float)((double)a * b); }

static rxmet_lstm_cell_scale encode_cell_scale(double ratio) {
    /* lstm_execution_params.cc:49-66 */
    rxmet_lstm_cell_scale s;
    memset(&s, 0, sizeof(s));
    const double scaled = ldexp(ratio, 31);
    if (isfinite(scaled) && scaled > 0.5 && scaled < 9223372036854775807.0) {
        s.multiplier = (int64_t)rint(scaled);
        return s;
    }
    int exponent = 0;
    s.fp_mantissa = frexp(ratio, &exponent);
    s.fp_exponent = exponent;
    s.uses_fp_scale = 1;
    return s;
}

static uint64_t magnitude(int64_t v) { return v < 0 ? (uint64_t)0 - (uint64_t)v : (uint64_t)v; }

static uint64_t centered_max(const rxmet_lstm_quant_config *c, int op, int32_t zp) {
    int32_t lo, hi;
    orc_lstm_type_range(c, op, &lo, &hi);
    const uint64_t a = magnitude((int64_t)lo - zp), b = magnitude((int64_t)hi - zp);
    return a > b ? a : b;
}

static uint64_t uncentered_max(const rxmet_lstm_quant_config *c, int op) {
    int32_t lo, hi;
    orc_lstm_type_range(c, op, &lo, &hi);
    const uint64_t a = magnitude(lo), b = magnitude(hi);
    return a > b ? a : b;
}

static long double rescale_bound(long double source, rxmet_lstm_rescale r, long double *maximum,
                                 long double *precision_maximum) {
    /* lstm_execution_params.cc:98-112 */
    unsigned int m = r.is_m_shift ? (unsigned int)r.multiplier : 1u;
    const long double intermediate = source * m;
    while ((m & 1u) == 0u && m != 0) m >>= 1u;
    if (source * m > *precision_maximum) *precision_maximum = source * m;
    const long double result = ceill(ldexpl(intermediate, -r.shift));
    if (intermediate > *maximum) *maximum = intermediate;
    if (result > *maximum) *maximum = result;
    return result;
}

static int classify_exact(long double accumulator_maximum, long double precision_maximum) {
    /* operators/quant-lstm/src/quantization/numeric_safety.cc:253-264 */
    return accumulator_maximum < 16777216.0L && precision_maximum < 16777216.0L;
}

static int derive_linear(const rxmet_lstm_quant_params *p, int in_op, int w_op, int b_op, int out_op,
                         uint64_t reduction, const float *w_scale, const float *b_scale, rxmet_lstm_rescale *bias_to_acc,
                         rxmet_lstm_rescale *acc_to_out) {
    /* lstm_execution_params.cc:119-187 */
    const rxmet_lstm_quant_config *c = &p->config;
    int all_exact = 1;
    for (int ch = 0; ch < 4 * p->hidden_size; ++ch) {
        const float acc_scale = product_scale(p->scale[in_op], w_scale[ch]);
        const rxmet_lstm_rescale out = encode(c->scale_mode, acc_scale, p->scale[out_op]);
        if (acc_to_out) acc_to_out[ch] = out;
        const uint64_t lhs = centered_max(c, in_op, p->zero_point[in_op]);
        const uint64_t rhs = centered_max(c, w_op, 0);
        long double bound = (long double)reduction * lhs * rhs;
        const long double weight_sum_bound = (long double)reduction * uncentered_max(c, w_op);
        const long double raw_gemm_bound = weight_sum_bound * uncentered_max(c, in_op);
        const long double zp_correction_bound = weight_sum_bound * magnitude(p->zero_point[in_op]);
        long double maximum = bound > raw_gemm_bound + zp_correction_bound ? bound : raw_gemm_bound + zp_correction_bound;
        long double precision_maximum = 0;
        if (p->bias_enabled) {
            const rxmet_lstm_rescale b = encode(c->scale_mode, b_scale[ch], acc_scale);
            if (bias_to_acc) bias_to_acc[ch] = b;
            bound += rescale_bound((long double)centered_max(c, b_op, 0), b, &maximum, &precision_maximum);
        }
        const long double output_bound = rescale_bound(bound, out, &maximum, &precision_maximum);
        long double acc_max = bound;
        if (raw_gemm_bound > acc_max) acc_max = raw_gemm_bound;
        if (zp_correction_bound > acc_max) acc_max = zp_correction_bound;
        const long double with_zp = output_bound + magnitude(p->zero_point[out_op]);
        if (with_zp > acc_max) acc_max = with_zp;
        all_exact = all_exact && classify_exact(acc_max, precision_maximum);
    }
    return all_exact;
}

int orc_lstm_derive_execution(const rxmet_lstm_quant_params *p, int exact, rxmet_lstm_execution *out) {
    /* lstm_execution_params.cc:188-326 */
    (void)exact;
    const rxmet_lstm_quant_config *c = &p->config;
    int all_exact = 1;
    all_exact &= derive_linear(p, RXMET_LSTM_INPUT, RXMET_LSTM_WEIGHT_IH, RXMET_LSTM_BIAS_IH, RXMET_LSTM_WEIGHT_IH_LINEAR,
                               (uint64_t)p->input_size, p->weight_ih_scale, p->bias_ih_scale, out->ih_bias_to_accumulator,
                               out->ih_accumulator_to_output);
    all_exact &= derive_linear(p, RXMET_LSTM_OUTPUT, RXMET_LSTM_WEIGHT_HH, RXMET_LSTM_BIAS_HH, RXMET_LSTM_WEIGHT_HH_LINEAR,
                               (uint64_t)p->hidden_size, p->weight_hh_scale, p->bias_hh_scale, out->hh_bias_to_accumulator,
                               out->hh_accumulator_to_output);
    for (int g = 0; g < 4; ++g) {
        const int gi = RXMET_LSTM_INPUT_GATE_INPUT + g;
        out->ih_to_gate[g] = encode(c->scale_mode, p->scale[RXMET_LSTM_WEIGHT_IH_LINEAR], p->scale[gi]);
        out->hh_to_gate[g] = encode(c->scale_mode, p->scale[RXMET_LSTM_WEIGHT_HH_LINEAR], p->scale[gi]);
        long double maximum = 0, precision_maximum = 0;
        const long double lhs = rescale_bound((long double)centered_max(c, RXMET_LSTM_WEIGHT_IH_LINEAR,
                                                                        p->zero_point[RXMET_LSTM_WEIGHT_IH_LINEAR]),
                                              out->ih_to_gate[g], &maximum, &precision_maximum);
        const long double rhs = rescale_bound((long double)centered_max(c, RXMET_LSTM_WEIGHT_HH_LINEAR,
                                                                        p->zero_point[RXMET_LSTM_WEIGHT_HH_LINEAR]),
                                              out->hh_to_gate[g], &maximum, &precision_maximum);
        all_exact &= classify_exact(lhs + rhs + magnitude(p->zero_point[gi]), precision_maximum);
    }
    const int fo = RXMET_LSTM_FORGET_GATE_OUTPUT, io = RXMET_LSTM_INPUT_GATE_OUTPUT, co = RXMET_LSTM_CELL_GATE_OUTPUT;
    const int oo = RXMET_LSTM_OUTPUT_GATE_OUTPUT, cs = RXMET_LSTM_CELL_STATE, ct = RXMET_LSTM_CELL_TANH_OUTPUT;
    out->forget_scale = encode_cell_scale((double)p->scale[fo] * p->scale[cs] / p->scale[cs]);
    out->input_scale = encode_cell_scale((double)p->scale[io] * p->scale[co] / p->scale[cs]);
    {
        const uint64_t a = centered_max(c, fo, p->zero_point[fo]), b = centered_max(c, io, p->zero_point[io]);
        const uint64_t d = centered_max(c, cs, p->zero_point[cs]), e = centered_max(c, co, p->zero_point[co]);
        const long double product = (long double)(a > b ? a : b) * (d > e ? d : e);
        const long double rf = out->forget_scale.uses_fp_scale
                                   ? ldexpl((long double)out->forget_scale.fp_mantissa, out->forget_scale.fp_exponent)
                                   : ldexpl((long double)out->forget_scale.multiplier, -31);
        const long double ri = out->input_scale.uses_fp_scale
                                   ? ldexpl((long double)out->input_scale.fp_mantissa, out->input_scale.fp_exponent)
                                   : ldexpl((long double)out->input_scale.multiplier, -31);
        const long double other = ceill(product * (rf + ri)) + magnitude(p->zero_point[cs]);
        all_exact &= classify_exact(product > other ? product : other, 0);
    }
    out->product_to_output =
        encode(c->scale_mode, product_scale(p->scale[oo], p->scale[ct]), p->scale[RXMET_LSTM_OUTPUT]);
    {
        const long double product =
            (long double)centered_max(c, oo, p->zero_point[oo]) * centered_max(c, ct, p->zero_point[ct]);
        long double maximum = product, precision_maximum = 0;
        const long double rescaled = rescale_bound(product, out->product_to_output, &maximum, &precision_maximum);
        const long double other = rescaled + magnitude(p->zero_point[RXMET_LSTM_OUTPUT]);
        all_exact &= classify_exact(product > other ? product : other, precision_maximum);
    }
    out->exact_accumulation = all_exact;
    return 0;
}
