// TEST INFRASTRUCTURE - not part of the shipped library.
//
// C entry points over the reference's own QuantLSTM CPU sources (compiled where
// they lie in the reference checkout by oracle/Makefile, target `ref`).  The
// flat structs of include/rxmet_b200_lstm.h are used as the interchange format;
// every function converts them into the reference's own types and calls the
// reference's functions, nothing is re-implemented here.
#include <cstring>
#include <exception>
#include <string>
#include <vector>

#include "lstm/backward_float_cpu.h"
#include "lstm/calibration.h"
#include "lstm/forward_cpu.h"
#include "lstm/forward_float.h"
#include "lstm/lstm_execution_params.h"
#include "lstm/quant_config.h"
#include "lstm/quant_params.h"
#include "quantization/float_carrier_ops.h"
#include "quantization/histogram.h"
#include "quantization/real_activation.h"
#include "quantization/scale_encoding.h"
#include "rxmet_b200_lstm.h"

namespace ql = quant_lstm;
namespace qq = quant_lstm::quantization;

namespace {

thread_local std::string g_error;

template <class F>
int guarded(F &&f) {
    try {
        f();
        return 0;
    } catch (const std::exception &e) {
        g_error = e.what();
        return -1;
    }
}

ql::LstmOperatorQuantConfig toConfig(const rxmet_lstm_quant_config &c) {
    ql::LstmOperatorQuantConfig out;
    out.scale_mode = c.scale_mode == RXMET_LSTM_SCALE_POT2 ? qq::ScaleMode::Pot2 : qq::ScaleMode::Affine;
    for (int i = 0; i < RXMET_LSTM_NUM_OPS; ++i) {
        out.operators[i].type.bitwidth = static_cast<std::uint8_t>(c.bitwidth[i]);
        out.operators[i].type.is_unsigned = c.is_unsigned[i] != 0;
        out.operators[i].type.is_symmetric = c.is_symmetric[i] != 0;
        out.operators[i].granularity = static_cast<ql::QuantGranularity>(c.granularity[i]);
    }
    return out;
}

const float *channelScales(const rxmet_lstm_quant_params &p, int op) {
    switch (op) {
        case RXMET_LSTM_WEIGHT_IH: return p.weight_ih_scale;
        case RXMET_LSTM_WEIGHT_HH: return p.weight_hh_scale;
        case RXMET_LSTM_BIAS_IH: return p.bias_ih_scale;
        default: return p.bias_hh_scale;
    }
}

ql::LstmQuantParams toParams(const rxmet_lstm_quant_params &p, const ql::LstmOperatorQuantConfig &config) {
    ql::LstmQuantParams out;
    out.hidden_size = p.hidden_size;
    out.bias_enabled = p.bias_enabled != 0;
    const std::size_t channels = 4 * static_cast<std::size_t>(p.hidden_size);
    for (int i = 0; i < RXMET_LSTM_NUM_OPS; ++i) {
        const auto id = static_cast<ql::QuantOperator>(i);
        auto &dst = out.operators[i];
        dst.source_granularity = config.operators[i].granularity;
        if (!out.bias_enabled && ql::isBiasOperator(id)) continue;
        if (ql::isParameterOperator(id)) {
            const float *s = channelScales(p, i);
            for (std::size_t ch = 0; ch < channels; ++ch) dst.values.push_back({s[ch], 0});
        } else {
            dst.values.push_back({p.scale[i], p.zero_point[i]});
        }
        dst.group_diagnostics.resize(ql::quantizationGroupCount(id, dst.source_granularity, p.hidden_size));
    }
    return out;
}

rxmet_lstm_rescale flat(const ql::ExecutionRescale &r) {
    if (r.kind == ql::ExecutionRescaleKind::MShift) return {1, r.m_shift.multiplier, r.m_shift.shift};
    return {0, 1, r.pot2.shift};
}

rxmet_lstm_cell_scale flat(const ql::Q31Scale &s) {
    return {s.multiplier, s.fp_mantissa, s.fp_exponent, s.uses_fp_scale ? 1 : 0};
}

qq::HistogramCollector toCollector(const rxmet_lstm_histogram &s) {
    qq::HistogramCollector c(static_cast<std::size_t>(s.num_bins));
    if (s.total_count != 0) {
        qq::Histogram h;
        h.minimum = s.minimum;
        h.maximum = s.maximum;
        h.counts.assign(s.counts, s.counts + s.num_bins);
        h.total_count = s.total_count;
        c.merge(h);  // an empty collector takes the histogram over unchanged
    }
    return c;
}

void fromHistogram(const qq::Histogram &h, rxmet_lstm_histogram *s) {
    if (h.empty()) return;
    std::copy(h.counts.begin(), h.counts.end(), s->counts);
    s->minimum = h.minimum;
    s->maximum = h.maximum;
    s->total_count = h.total_count;
}

}  // namespace

extern "C" {

int ref_lstm_histogram_collect_host(rxmet_lstm_histogram *hist, const float *data, uint64_t count) {
    return guarded([&] {
        qq::HistogramCollector c = toCollector(*hist);
        c.collect(data, count);
        fromHistogram(c.histogram(), hist);
    });
}

int ref_lstm_histogram_merge(rxmet_lstm_histogram *hist, const rxmet_lstm_histogram *other) {
    return guarded([&] {
        qq::HistogramCollector c = toCollector(*hist);
        c.merge(toCollector(*other).histogram());
        fromHistogram(c.histogram(), hist);
    });
}

int ref_lstm_histogram_range(const rxmet_lstm_histogram *hist, int bits, int is_unsigned, int is_symmetric, int method,
                             float percentile, float *lo, float *hi) {
    return guarded([&] {
        const qq::HistogramCollector c = toCollector(*hist);
        qq::HistogramCalibrationOptions options;
        options.percentile = percentile;
        const qq::QuantizationType type{static_cast<std::uint8_t>(bits), is_unsigned != 0, is_symmetric != 0};
        const auto r = qq::calibrateHistogramRange(c.histogram(), type,
                                                   method == 1 ? qq::HistogramCalibrationMethod::Percentile
                                                               : qq::HistogramCalibrationMethod::Sqnr,
                                                   options);
        *lo = r.first;
        *hi = r.second;
    });
}

// Calibration session with method 1 = sqnr or 2 = percentile over `batches` equally shaped batches;
// returns the session's histogram collectors and the parameters it finalizes.
int ref_lstm_calibrate_hist(const rxmet_lstm_quant_config *config, int method, float percentile, int batches, int T,
                            int B, int I, int H, const float *w_ih, const float *w_hh, const float *b_ih,
                            const float *b_hh, const float *x_all, const float *h0, const float *c0,
                            rxmet_lstm_histograms *hists, float *w_ih_scale, float *w_hh_scale, float *b_ih_scale,
                            float *b_hh_scale, rxmet_lstm_quant_params *params) {
    return guarded([&] {
        const auto cfg = toConfig(*config);
        const bool bias = b_ih != nullptr;
        qq::HistogramCalibrationOptions options;
        options.percentile = percentile;
        ql::LstmCalibrationSession session(cfg, I, H, bias,
                                           method == 2 ? ql::CalibrationMethod::Percentile : ql::CalibrationMethod::Sqnr,
                                           options, static_cast<std::size_t>(hists->num_bins));
        const std::size_t per_batch = static_cast<std::size_t>(T) * B * I;
        for (int n = 0; n < batches; ++n)
            session.collect({T, B, I, H}, {w_ih, w_hh, b_ih, b_hh}, x_all + n * per_batch, h0, c0);
        const auto &fin = session.finalize(false);
        const auto &all = session.collector().histograms();
        for (int i = 0; i < RXMET_LSTM_NUM_OPS; ++i) {
            const auto id = static_cast<ql::QuantOperator>(i);
            const auto &groups = all[i];
            if (groups.empty()) continue;
            if (!ql::isParameterOperator(id)) {
                fromHistogram(groups[0].histogram(), &hists->point[i]);
                continue;
            }
            const int slot = i - RXMET_LSTM_WEIGHT_IH;
            const auto gran = cfg.operators[i].granularity;
            for (std::size_t g = 0; g < groups.size(); ++g) {
                rxmet_lstm_histogram *dst = gran == ql::QuantGranularity::PerTensor ? &hists->point[i]
                                            : (gran == ql::QuantGranularity::PerGate ? &hists->gate[slot][g] : &hists->channel[slot][g]);
                fromHistogram(groups[g].histogram(), dst);
            }
        }
        std::memset(params, 0, sizeof(*params));
        params->config = *config;
        params->input_size = I;
        params->hidden_size = H;
        params->bias_enabled = bias;
        float *dst[4] = {w_ih_scale, w_hh_scale, b_ih_scale, b_hh_scale};
        for (int i = 0; i < RXMET_LSTM_NUM_OPS; ++i) {
            const auto id = static_cast<ql::QuantOperator>(i);
            const auto &values = fin.quant_params.operators[i].values;
            if (values.empty()) continue;
            if (ql::isParameterOperator(id)) {
                for (int ch = 0; ch < 4 * H; ++ch) dst[i - RXMET_LSTM_WEIGHT_IH][ch] = values[ch].scale;
            } else {
                params->scale[i] = values[0].scale;
                params->zero_point[i] = values[0].zero_point;
            }
        }
        params->weight_ih_scale = w_ih_scale;
        params->weight_hh_scale = w_hh_scale;
        params->bias_ih_scale = bias ? b_ih_scale : nullptr;
        params->bias_hh_scale = bias ? b_hh_scale : nullptr;
    });
}

const char *ref_lstm_last_error() { return g_error.c_str(); }

int ref_lstm_forward_float(int T, int B, int I, int H, const float *w_ih, const float *w_hh, const float *b_ih,
                           const float *b_hh, const float *x, const float *h0, const float *c0, float *out, float *hn,
                           float *cn, float *ih_lin, float *hh_lin, float *gate_in, float *gate_out, float *cell,
                           float *cell_tanh, float *hidden) {
    return guarded([&] {
        ql::LstmFloatReferenceTrace trace;
        ql::lstmForwardFloatCpu({T, B, I, H}, {w_ih, w_hh, b_ih, b_hh}, x, h0, c0, out, hn, cn, &trace);
        auto put = [](float *dst, const std::vector<float> &src) {
            if (dst) std::memcpy(dst, src.data(), src.size() * sizeof(float));
        };
        put(ih_lin, trace.weight_input_hidden_linear);
        put(hh_lin, trace.weight_hidden_hidden_linear);
        put(gate_in, trace.gate_inputs);
        put(gate_out, trace.gate_outputs);
        put(cell, trace.cell_states);
        put(cell_tanh, trace.cell_tanh_outputs);
        put(hidden, trace.hidden_outputs);
    });
}

int ref_lstm_backward_float(int T, int B, int I, int H, const float *w_ih, const float *w_hh, const float *x,
                            const float *h0, const float *c0, const float *gate_out, const float *cell,
                            const float *cell_tanh, const float *hidden, const float *g_out, const float *g_hn,
                            const float *g_cn, float *dx, float *dw_ih, float *dw_hh, float *db_ih, float *db_hh,
                            float *dh0, float *dc0) {
    return guarded([&] {
        ql::lstmBackwardFloatCpu({T, B, I, H}, {w_ih, w_hh, nullptr, nullptr}, x, h0, c0,
                                 {gate_out, cell, cell_tanh, hidden}, g_out, g_hn, g_cn,
                                 {dx, dw_ih, dw_hh, db_ih, db_hh, dh0, dc0});
    });
}

// quantizeFp of `n` values; channel = index / row_width when scales has more than one entry.
int ref_lstm_quantize(const float *src, long long n, long long row_width, const float *scales, int zero_point,
                      int bitwidth, int is_unsigned, int is_symmetric, float *dst) {
    return guarded([&] {
        qq::QuantizationType type{static_cast<std::uint8_t>(bitwidth), is_unsigned != 0, is_symmetric != 0};
        for (long long i = 0; i < n; ++i) {
            const qq::QuantParam param{scales[row_width > 0 ? i / row_width : 0], zero_point};
            dst[i] = qq::quantizeFp(src[i], param, type);
        }
    });
}

int ref_lstm_real_activation(const float *src, long long n, float in_scale, int in_zp, int in_bits, int in_unsigned,
                             float out_scale, int out_zp, int out_bits, int out_unsigned, int is_tanh, float *dst) {
    return guarded([&] {
        qq::QuantizationType in_type{static_cast<std::uint8_t>(in_bits), in_unsigned != 0, false};
        qq::QuantizationType out_type{static_cast<std::uint8_t>(out_bits), out_unsigned != 0, false};
        for (long long i = 0; i < n; ++i)
            dst[i] = qq::realActivation(src[i], {in_scale, in_zp}, in_type, {out_scale, out_zp}, out_type,
                                        is_tanh ? qq::RealActivationKind::Tanh : qq::RealActivationKind::Sigmoid);
    });
}

int ref_lstm_params_from_ranges(const rxmet_lstm_quant_config *config, const rxmet_lstm_ranges *ranges, int I, int H,
                                int bias, float *w_ih_scale, float *w_hh_scale, float *b_ih_scale, float *b_hh_scale,
                                rxmet_lstm_quant_params *params) {
    return guarded([&] {
        const auto cfg = toConfig(*config);
        ql::LstmQuantizationRanges r;
        r.reset(cfg, H, bias != 0);
        for (int i = 0; i < RXMET_LSTM_NUM_OPS; ++i) {
            const auto id = static_cast<ql::QuantOperator>(i);
            auto &groups = r.operators[i];
            if (groups.empty()) continue;
            if (!ql::isParameterOperator(id)) {
                groups[0].minimum = ranges->minimum[i];
                groups[0].maximum = ranges->maximum[i];
                groups[0].sample_count = 1;
                continue;
            }
            const int slot = i - RXMET_LSTM_WEIGHT_IH;
            for (int ch = 0; ch < 4 * H; ++ch) {
                ql::CalibrationRange one;
                one.minimum = ranges->channel_min[slot][ch];
                one.maximum = ranges->channel_max[slot][ch];
                one.sample_count = 1;
                groups[ql::quantizationGroupIndex(id, cfg.operators[i].granularity, ch, H)].merge(one);
            }
        }
        const auto fin = ql::finalizeQuantParams(cfg, r, H, bias != 0);
        std::memset(params, 0, sizeof(*params));
        params->config = *config;
        params->input_size = I;
        params->hidden_size = H;
        params->bias_enabled = bias;
        float *dst[4] = {w_ih_scale, w_hh_scale, b_ih_scale, b_hh_scale};
        for (int i = 0; i < RXMET_LSTM_NUM_OPS; ++i) {
            const auto id = static_cast<ql::QuantOperator>(i);
            const auto &values = fin.operators[i].values;
            if (values.empty()) continue;
            if (ql::isParameterOperator(id)) {
                for (int ch = 0; ch < 4 * H; ++ch) dst[i - RXMET_LSTM_WEIGHT_IH][ch] = values[ch].scale;
            } else {
                params->scale[i] = values[0].scale;
                params->zero_point[i] = values[0].zero_point;
            }
        }
        params->weight_ih_scale = w_ih_scale;
        params->weight_hh_scale = w_hh_scale;
        params->bias_ih_scale = bias ? b_ih_scale : nullptr;
        params->bias_hh_scale = bias ? b_hh_scale : nullptr;
    });
}

int ref_lstm_derive_execution(const rxmet_lstm_quant_params *params, int exact, rxmet_lstm_execution *out) {
    return guarded([&] {
        const auto cfg = toConfig(params->config);
        const auto qp = toParams(*params, cfg);
        const auto e = ql::deriveLstmExecutionParams(cfg, qp, params->input_size, exact != 0);
        for (int g = 0; g < 4; ++g) {
            out->ih_to_gate[g] = flat(e.gates[g].input_hidden_to_gate);
            out->hh_to_gate[g] = flat(e.gates[g].hidden_hidden_to_gate);
        }
        out->forget_scale = flat(e.cell.forget_scale);
        out->input_scale = flat(e.cell.input_scale);
        out->product_to_output = flat(e.hidden.product_to_output);
        bool all_exact = true;
        auto scan = [&](const qq::NumericSafetyReport &r) {
            all_exact = all_exact && r.fp32_accumulation == qq::Fp32AccumulationClass::ExactIntegerRange;
        };
        for (const auto &r : e.diagnostics.input_hidden_linear) scan(r);
        for (const auto &r : e.diagnostics.hidden_hidden_linear) scan(r);
        for (const auto &r : e.diagnostics.gates) scan(r);
        scan(e.diagnostics.cell);
        scan(e.diagnostics.hidden);
        out->exact_accumulation = all_exact ? 1 : 0;
        const std::size_t channels = 4 * static_cast<std::size_t>(params->hidden_size);
        for (std::size_t ch = 0; ch < channels; ++ch) {
            if (out->ih_accumulator_to_output)
                out->ih_accumulator_to_output[ch] = flat(e.input_hidden_linear.accumulator_to_output[ch]);
            if (out->hh_accumulator_to_output)
                out->hh_accumulator_to_output[ch] = flat(e.hidden_hidden_linear.accumulator_to_output[ch]);
            if (params->bias_enabled && out->ih_bias_to_accumulator)
                out->ih_bias_to_accumulator[ch] = flat(e.input_hidden_linear.bias_to_accumulator[ch]);
            if (params->bias_enabled && out->hh_bias_to_accumulator)
                out->hh_bias_to_accumulator[ch] = flat(e.hidden_hidden_linear.bias_to_accumulator[ch]);
        }
    });
}

// q-carrier forward of the reference's CPU core on already quantized inputs.
int ref_lstm_forward_quantized(const rxmet_lstm_quant_params *params, int exact, int T, int B, const float *q_w_ih,
                               const float *q_w_hh, const float *q_b_ih, const float *q_b_hh, const float *q_x,
                               const float *q_h0, const float *q_c0, float *out, float *hn, float *cn, float *ih_lin,
                               float *hh_lin, float *gate_in, float *gate_out, float *cell, float *cell_tanh,
                               float *hidden) {
    return guarded([&] {
        const auto cfg = toConfig(params->config);
        const auto qp = toParams(*params, cfg);
        const auto e = ql::deriveLstmExecutionParams(cfg, qp, params->input_size, exact != 0);
        ql::LstmFpReferenceTrace trace;
        ql::lstmForwardQuantizedFpCpuReference({T, B, params->input_size, params->hidden_size},
                                               {q_w_ih, q_w_hh, q_b_ih, q_b_hh}, q_x, q_h0, q_c0, cfg, qp, e, out, hn,
                                               cn, &trace);
        auto put = [](float *dst, const std::vector<float> &src) {
            if (dst) std::memcpy(dst, src.data(), src.size() * sizeof(float));
        };
        put(ih_lin, trace.weight_ih_linear);
        put(hh_lin, trace.weight_hh_linear);
        put(gate_in, trace.gate_inputs);
        put(gate_out, trace.gate_outputs);
        put(cell, trace.cell_states);
        put(cell_tanh, trace.cell_tanh_outputs);
        put(hidden, trace.hidden_outputs);
    });
}

// The reference's exact integer forward (lstmForwardInt32CpuReference, operators/quant-lstm/src/lstm/
// forward_int32_cpu.cc:73) on the same q-carrier inputs: codes cross the shim as floats (they are
// integers below 2^24) and are converted to int32 here and back.
int ref_lstm_forward_int32(const rxmet_lstm_quant_params *params, int T, int B, const float *q_w_ih, const float *q_w_hh,
                           const float *q_b_ih, const float *q_b_hh, const float *q_x, const float *q_h0,
                           const float *q_c0, float *out, float *hn, float *cn, float *ih_lin, float *hh_lin,
                           float *gate_in, float *gate_out, float *cell, float *cell_tanh, float *hidden) {
    return guarded([&] {
        const auto cfg = toConfig(params->config);
        const auto qp = toParams(*params, cfg);
        const auto e = ql::deriveLstmExecutionParams(cfg, qp, params->input_size, false);
        const std::size_t I = params->input_size, H = params->hidden_size, C = 4 * H;
        auto ints = [](const float *src, std::size_t n) {
            std::vector<std::int32_t> v(src ? n : 0);
            for (std::size_t i = 0; i < v.size(); ++i) v[i] = static_cast<std::int32_t>(src[i]);
            return v;
        };
        const auto wih = ints(q_w_ih, C * I), whh = ints(q_w_hh, C * H), bih = ints(q_b_ih, C), bhh = ints(q_b_hh, C);
        const auto x = ints(q_x, static_cast<std::size_t>(T) * B * I), h0 = ints(q_h0, B * H), c0 = ints(q_c0, B * H);
        std::vector<std::int32_t> o(static_cast<std::size_t>(T) * B * H), h(B * H), c(B * H);
        ql::LstmInt32ReferenceTrace trace;
        ql::lstmForwardInt32CpuReference({T, B, params->input_size, params->hidden_size},
                                         {wih.data(), whh.data(), q_b_ih ? bih.data() : nullptr, q_b_hh ? bhh.data() : nullptr},
                                         x.data(), q_h0 ? h0.data() : nullptr, q_c0 ? c0.data() : nullptr, cfg, qp, e, o.data(),
                                         h.data(), c.data(), &trace);
        auto put = [](float *dst, const std::vector<std::int32_t> &src) {
            if (dst) for (std::size_t i = 0; i < src.size(); ++i) dst[i] = static_cast<float>(src[i]);
        };
        put(out, o); put(hn, h); put(cn, c);
        put(ih_lin, trace.weight_ih_linear); put(hh_lin, trace.weight_hh_linear);
        put(gate_in, trace.gate_inputs); put(gate_out, trace.gate_outputs);
        put(cell, trace.cell_states); put(cell_tanh, trace.cell_tanh_outputs); put(hidden, trace.hidden_outputs);
    });
}

// MinMax calibration session over `batches` equally shaped batches; returns the ranges it observed
// and the parameters it finalizes.
int ref_lstm_calibrate_minmax(const rxmet_lstm_quant_config *config, int batches, int T, int B, int I, int H,
                              const float *w_ih, const float *w_hh, const float *b_ih, const float *b_hh,
                              const float *x_all, const float *h0, const float *c0, rxmet_lstm_ranges *ranges,
                              float *w_ih_scale, float *w_hh_scale, float *b_ih_scale, float *b_hh_scale,
                              rxmet_lstm_quant_params *params) {
    return guarded([&] {
        const auto cfg = toConfig(*config);
        const bool bias = b_ih != nullptr;
        ql::LstmCalibrationSession session(cfg, I, H, bias);
        const std::size_t per_batch = static_cast<std::size_t>(T) * B * I;
        for (int n = 0; n < batches; ++n)
            session.collect({T, B, I, H}, {w_ih, w_hh, b_ih, b_hh}, x_all + n * per_batch, h0, c0);
        const auto &fin = session.finalize(false);
        const auto &observed = session.collector().ranges();
        for (int i = 0; i < RXMET_LSTM_NUM_OPS; ++i) {
            const auto id = static_cast<ql::QuantOperator>(i);
            const auto &groups = observed.operators[i];
            if (groups.empty()) continue;
            if (!ql::isParameterOperator(id)) {
                ranges->minimum[i] = groups[0].minimum;
                ranges->maximum[i] = groups[0].maximum;
            } else {
                for (int ch = 0; ch < 4 * H; ++ch) {
                    const auto &g = groups[ql::quantizationGroupIndex(id, cfg.operators[i].granularity, ch, H)];
                    ranges->channel_min[i - RXMET_LSTM_WEIGHT_IH][ch] = g.minimum;
                    ranges->channel_max[i - RXMET_LSTM_WEIGHT_IH][ch] = g.maximum;
                }
            }
        }
        const auto &contrib = session.collector().contributions();
        const ql::CalibrationRange *c3[3] = {&contrib.forget_times_old_cell, &contrib.input_times_cell,
                                             &contrib.output_times_cell_tanh};
        for (int k = 0; k < 3; ++k) {
            ranges->contribution_min[k] = c3[k]->minimum;
            ranges->contribution_max[k] = c3[k]->maximum;
        }
        std::memset(params, 0, sizeof(*params));
        params->config = *config;
        params->input_size = I;
        params->hidden_size = H;
        params->bias_enabled = bias;
        float *dst[4] = {w_ih_scale, w_hh_scale, b_ih_scale, b_hh_scale};
        for (int i = 0; i < RXMET_LSTM_NUM_OPS; ++i) {
            const auto id = static_cast<ql::QuantOperator>(i);
            const auto &values = fin.quant_params.operators[i].values;
            if (values.empty()) continue;
            if (ql::isParameterOperator(id)) {
                for (int ch = 0; ch < 4 * H; ++ch) dst[i - RXMET_LSTM_WEIGHT_IH][ch] = values[ch].scale;
            } else {
                params->scale[i] = values[0].scale;
                params->zero_point[i] = values[0].zero_point;
            }
        }
        params->weight_ih_scale = w_ih_scale;
        params->weight_hh_scale = w_hh_scale;
        params->bias_ih_scale = bias ? b_ih_scale : nullptr;
        params->bias_hh_scale = bias ? b_hh_scale : nullptr;
    });
}

}  // extern "C"
