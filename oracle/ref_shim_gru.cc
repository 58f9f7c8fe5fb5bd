// TEST INFRASTRUCTURE - not part of the shipped library.
//
// Thin extern "C" adapter around the reference's own CPU implementation of the
// QuantGRU path.  It is compiled together with the reference's unmodified
// sources (gru_host.cc, gru_forward_cpu.cc, gru_forward_cpu_quant.cc,
// quantize_lut.cc of operators/quant-gru/src) where they lie, by the Makefile
// beside this file, into oracle/_ref/libgru_ref.so.  Nothing of the reference
// is copied here: this file only converts between the flat C structs of
// include/rxmet_b200.h and the reference's C++ types and calls the
// reference's functions.  Tests use the result to pin the C restatement in
// gru_oracle.c and to generate golden fixtures.
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include "gru_host.h"          // reference: calculateGRUQuantitativeParameters, forwardWithCalibrationCPU, ...
#include "gru_quant_cpu.h"     // reference: cpu::ForwardPassQuantCPU
#include "scale_encoding.h"    // reference: toFixedScale, encodeMShift
#include "histogram_collector.h"   // reference: HistogramCollector, GRUHistogramCollectors
#include "pot_sqnr_calibrator.h"   // reference: calibrateContinuousScaleFromHistogram
#include "rxmet_b200.h"
#include "ref_shim_gru_convert.h"

namespace {

using refshim::bwOf;
using refshim::toRefConfig;
using refshim::toRefParams;

thread_local std::string g_error;

GRUQuantizationRanges toRefRanges(const rxmet_gru_ranges &s) {
    GRUQuantizationRanges r(s.hidden);
    float *mn[RXMET_GRU_NUM_OPS] = {};
    float *mx[RXMET_GRU_NUM_OPS] = {};
    mn[RXMET_GRU_X] = &r.min_x_; mx[RXMET_GRU_X] = &r.max_x_;
    mn[RXMET_GRU_H] = &r.min_h_; mx[RXMET_GRU_H] = &r.max_h_;
    mn[RXMET_GRU_WEIGHT_IH_LINEAR] = &r.min_Wx_; mx[RXMET_GRU_WEIGHT_IH_LINEAR] = &r.max_Wx_;
    mn[RXMET_GRU_WEIGHT_HH_LINEAR] = &r.min_Rh_; mx[RXMET_GRU_WEIGHT_HH_LINEAR] = &r.max_Rh_;
    mn[RXMET_GRU_UPDATE_GATE_INPUT] = &r.min_update_gate_input_; mx[RXMET_GRU_UPDATE_GATE_INPUT] = &r.max_update_gate_input_;
    mn[RXMET_GRU_UPDATE_GATE_OUTPUT] = &r.min_update_gate_output_; mx[RXMET_GRU_UPDATE_GATE_OUTPUT] = &r.max_update_gate_output_;
    mn[RXMET_GRU_RESET_GATE_INPUT] = &r.min_reset_gate_input_; mx[RXMET_GRU_RESET_GATE_INPUT] = &r.max_reset_gate_input_;
    mn[RXMET_GRU_RESET_GATE_OUTPUT] = &r.min_reset_gate_output_; mx[RXMET_GRU_RESET_GATE_OUTPUT] = &r.max_reset_gate_output_;
    mn[RXMET_GRU_NEW_GATE_INPUT] = &r.min_new_gate_input_; mx[RXMET_GRU_NEW_GATE_INPUT] = &r.max_new_gate_input_;
    mn[RXMET_GRU_NEW_GATE_OUTPUT] = &r.min_new_gate_output_; mx[RXMET_GRU_NEW_GATE_OUTPUT] = &r.max_new_gate_output_;
    mn[RXMET_GRU_MUL_RESET_HIDDEN] = &r.min_mul_reset_hidden_; mx[RXMET_GRU_MUL_RESET_HIDDEN] = &r.max_mul_reset_hidden_;
    mn[RXMET_GRU_MUL_OLD_CONTRIBUTION] = &r.min_mul_old_contribution_; mx[RXMET_GRU_MUL_OLD_CONTRIBUTION] = &r.max_mul_old_contribution_;
    mn[RXMET_GRU_MUL_NEW_CONTRIBUTION] = &r.min_mul_new_contribution_; mx[RXMET_GRU_MUL_NEW_CONTRIBUTION] = &r.max_mul_new_contribution_;
    for (int i = 0; i < RXMET_GRU_NUM_OPS; ++i) {
        if (mn[i]) { *mn[i] = s.min[i]; *mx[i] = s.max[i]; }
    }
    const int c3 = 3 * s.hidden;
    r.min_W_.assign(s.min_W, s.min_W + c3); r.max_W_.assign(s.max_W, s.max_W + c3);
    r.min_R_.assign(s.min_R, s.min_R + c3); r.max_R_.assign(s.max_R, s.max_R + c3);
    r.min_bw_.assign(s.min_bw, s.min_bw + c3); r.max_bw_.assign(s.max_bw, s.max_bw + c3);
    r.min_br_.assign(s.min_br, s.min_br + c3); r.max_br_.assign(s.max_br, s.max_br + c3);
    return r;
}

void fromRefRanges(const GRUQuantizationRanges &r, rxmet_gru_ranges *s) {
    s->min[RXMET_GRU_X] = r.min_x_; s->max[RXMET_GRU_X] = r.max_x_;
    s->min[RXMET_GRU_H] = r.min_h_; s->max[RXMET_GRU_H] = r.max_h_;
    s->min[RXMET_GRU_WEIGHT_IH_LINEAR] = r.min_Wx_; s->max[RXMET_GRU_WEIGHT_IH_LINEAR] = r.max_Wx_;
    s->min[RXMET_GRU_WEIGHT_HH_LINEAR] = r.min_Rh_; s->max[RXMET_GRU_WEIGHT_HH_LINEAR] = r.max_Rh_;
    s->min[RXMET_GRU_UPDATE_GATE_INPUT] = r.min_update_gate_input_; s->max[RXMET_GRU_UPDATE_GATE_INPUT] = r.max_update_gate_input_;
    s->min[RXMET_GRU_UPDATE_GATE_OUTPUT] = r.min_update_gate_output_; s->max[RXMET_GRU_UPDATE_GATE_OUTPUT] = r.max_update_gate_output_;
    s->min[RXMET_GRU_RESET_GATE_INPUT] = r.min_reset_gate_input_; s->max[RXMET_GRU_RESET_GATE_INPUT] = r.max_reset_gate_input_;
    s->min[RXMET_GRU_RESET_GATE_OUTPUT] = r.min_reset_gate_output_; s->max[RXMET_GRU_RESET_GATE_OUTPUT] = r.max_reset_gate_output_;
    s->min[RXMET_GRU_NEW_GATE_INPUT] = r.min_new_gate_input_; s->max[RXMET_GRU_NEW_GATE_INPUT] = r.max_new_gate_input_;
    s->min[RXMET_GRU_NEW_GATE_OUTPUT] = r.min_new_gate_output_; s->max[RXMET_GRU_NEW_GATE_OUTPUT] = r.max_new_gate_output_;
    s->min[RXMET_GRU_MUL_RESET_HIDDEN] = r.min_mul_reset_hidden_; s->max[RXMET_GRU_MUL_RESET_HIDDEN] = r.max_mul_reset_hidden_;
    s->min[RXMET_GRU_MUL_OLD_CONTRIBUTION] = r.min_mul_old_contribution_; s->max[RXMET_GRU_MUL_OLD_CONTRIBUTION] = r.max_mul_old_contribution_;
    s->min[RXMET_GRU_MUL_NEW_CONTRIBUTION] = r.min_mul_new_contribution_; s->max[RXMET_GRU_MUL_NEW_CONTRIBUTION] = r.max_mul_new_contribution_;
    const size_t n = sizeof(float) * 3 * r.hidden_;
    std::memcpy(s->min_W, r.min_W_.data(), n); std::memcpy(s->max_W, r.max_W_.data(), n);
    std::memcpy(s->min_R, r.min_R_.data(), n); std::memcpy(s->max_R, r.max_R_.data(), n);
    std::memcpy(s->min_bw, r.min_bw_.data(), n); std::memcpy(s->max_bw, r.max_bw_.data(), n);
    std::memcpy(s->min_br, r.min_br_.data(), n); std::memcpy(s->max_br, r.max_br_.data(), n);
}

void fromRefParams(const GRUQuantParams &r, rxmet_gru_quant_params *p) {
    p->hidden = r.hidden_;
    auto put = [&](int op, const QuantParam &q) { p->scale[op] = q.scale; p->zero_point[op] = q.zero_point; };
    for (int i = 0; i < RXMET_GRU_NUM_OPS; ++i) { p->scale[i] = 0.0f; p->zero_point[i] = 0; }
    put(RXMET_GRU_X, r.x_);
    put(RXMET_GRU_H, r.h_);
    put(RXMET_GRU_WEIGHT_IH_LINEAR, r.weight_ih_linear_);
    put(RXMET_GRU_WEIGHT_HH_LINEAR, r.weight_hh_linear_);
    put(RXMET_GRU_UPDATE_GATE_INPUT, r.update_gate_input_);
    put(RXMET_GRU_UPDATE_GATE_OUTPUT, r.update_gate_output_);
    put(RXMET_GRU_RESET_GATE_INPUT, r.reset_gate_input_);
    put(RXMET_GRU_RESET_GATE_OUTPUT, r.reset_gate_output_);
    put(RXMET_GRU_NEW_GATE_INPUT, r.new_gate_input_);
    put(RXMET_GRU_NEW_GATE_OUTPUT, r.new_gate_output_);
    put(RXMET_GRU_MUL_RESET_HIDDEN, r.mul_reset_hidden_);
    put(RXMET_GRU_MUL_OLD_CONTRIBUTION, r.mul_old_contribution_);
    put(RXMET_GRU_MUL_NEW_CONTRIBUTION, r.mul_new_contribution_);
    for (int c = 0; c < 3 * r.hidden_; ++c) {
        p->scale_W[c] = r.W_.channel(c).scale;
        p->scale_R[c] = r.R_.channel(c).scale;
        p->scale_bw[c] = r.bw_.channel(c).scale;
        p->scale_br[c] = r.br_.channel(c).scale;
    }
}

// Collector <-> flat struct.  The growth limits of a reference collector are private; with the
// reference's infinite growth limit they never constrain anything, so a collector rebuilt from its
// histogram alone behaves identically.
HistogramCollector toRefCollector(const rxmet_histogram &s) {
    HistogramCollector c(s.num_bins);
    if (s.num_bins > 0 && s.total_count > 0) {
        Histogram &h = c.histogram();
        h.counts.assign(s.counts, s.counts + s.num_bins);
        h.min_val = s.min_val;
        h.max_val = s.max_val;
        h.observed_min = s.observed_min;
        h.observed_max = s.observed_max;
        h.num_bins = s.num_bins;
        h.total_count = s.total_count;
    }
    return c;
}

void fromRefCollector(const HistogramCollector &c, rxmet_histogram *s) {
    const Histogram &h = c.histogram();
    if (!c.is_valid()) return;
    std::copy(h.counts.begin(), h.counts.end(), s->counts);
    s->min_val = h.min_val;
    s->max_val = h.max_val;
    s->observed_min = h.observed_min;
    s->observed_max = h.observed_max;
    s->total_count = h.total_count;
}

HistogramCollector *pointCollector(GRUHistogramCollectors &g, int op) {
    switch (op) {
        case RXMET_GRU_X: return &g.x_hist;
        case RXMET_GRU_H: return &g.h_hist;
        case RXMET_GRU_W: return &g.W_tensor_hist;
        case RXMET_GRU_R: return &g.R_tensor_hist;
        case RXMET_GRU_BW: return &g.bw_tensor_hist;
        case RXMET_GRU_BR: return &g.br_tensor_hist;
        case RXMET_GRU_WEIGHT_IH_LINEAR: return &g.Wx_hist;
        case RXMET_GRU_WEIGHT_HH_LINEAR: return &g.Rh_hist;
        case RXMET_GRU_UPDATE_GATE_INPUT: return &g.update_gate_input_hist;
        case RXMET_GRU_UPDATE_GATE_OUTPUT: return &g.update_gate_output_hist;
        case RXMET_GRU_RESET_GATE_INPUT: return &g.reset_gate_input_hist;
        case RXMET_GRU_RESET_GATE_OUTPUT: return &g.reset_gate_output_hist;
        case RXMET_GRU_NEW_GATE_INPUT: return &g.new_gate_input_hist;
        case RXMET_GRU_NEW_GATE_OUTPUT: return &g.new_gate_output_hist;
        case RXMET_GRU_MUL_RESET_HIDDEN: return &g.mul_reset_hidden_hist;
        case RXMET_GRU_MUL_OLD_CONTRIBUTION: return &g.mul_old_contribution_hist;
        default: return &g.mul_new_contribution_hist;
    }
}

std::vector<HistogramCollector> *channelCollectors(GRUHistogramCollectors &g, int slot) {
    return slot == 0 ? &g.W_hist : (slot == 1 ? &g.R_hist : (slot == 2 ? &g.bw_hist : &g.br_hist));
}
std::array<HistogramCollector, 3> *gateCollectors(GRUHistogramCollectors &g, int slot) {
    return slot == 0 ? &g.W_gate_hist : (slot == 1 ? &g.R_gate_hist : (slot == 2 ? &g.bw_gate_hist : &g.br_gate_hist));
}

GRUHistogramCollectors toRefHists(const rxmet_gru_histograms &s) {
    GRUHistogramCollectors g(s.hidden, s.num_bins);
    for (int op = 0; op < RXMET_GRU_NUM_OPS; ++op) *pointCollector(g, op) = toRefCollector(s.point[op]);
    for (int slot = 0; slot < 4; ++slot) {
        for (int c = 0; c < 3 * s.hidden; ++c) (*channelCollectors(g, slot))[c] = toRefCollector(s.channel[slot][c]);
        for (int k = 0; k < 3; ++k) (*gateCollectors(g, slot))[k] = toRefCollector(s.gate[slot][k]);
    }
    return g;
}

void fromRefHists(GRUHistogramCollectors &g, rxmet_gru_histograms *s) {
    for (int op = 0; op < RXMET_GRU_NUM_OPS; ++op) fromRefCollector(*pointCollector(g, op), &s->point[op]);
    for (int slot = 0; slot < 4; ++slot) {
        for (int c = 0; c < 3 * s->hidden; ++c) fromRefCollector((*channelCollectors(g, slot))[c], &s->channel[slot][c]);
        for (int k = 0; k < 3; ++k) fromRefCollector((*gateCollectors(g, slot))[k], &s->gate[slot][k]);
    }
}

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

}  // namespace

extern "C" {

const char *ref_last_error(void) { return g_error.c_str(); }

int ref_gru_params_from_ranges(const rxmet_gru_ranges *ranges, const rxmet_gru_quant_config *cfg,
                               rxmet_gru_quant_params *out) {
    return guarded([&] {
        const GRUQuantParams p = calculateGRUQuantitativeParameters(toRefRanges(*ranges), toRefConfig(*cfg));
        out->config = *cfg;
        fromRefParams(p, out);
    });
}

int ref_gru_build_luts(const rxmet_gru_quant_params *params, rxmet_lut_segment out[3][16]) {
    return guarded([&] {
        const GRUQuantParams p = toRefParams(*params);
        const SigmoidLUT *luts[3] = {&p.sigmoid_update_gate_lut_, &p.sigmoid_reset_gate_lut_, &p.tanh_new_gate_lut_};
        for (int l = 0; l < 3; ++l)
            for (int s = 0; s < NUM_SEGMENTS; ++s) {
                out[l][s].q_b = luts[l]->segments[s].q_b;
                out[l][s].n_bx_total = luts[l]->segments[s].n_BX_total;
                out[l][s].term_c = luts[l]->segments[s].term_c_precomputed;
                out[l][s].threshold = luts[l]->segments[s].threshold;
            }
    });
}

int ref_gru_decode_effective_scale(float scale, int use_pot2, float *out) {
    return guarded([&] { *out = decode_scale(toFixedScale(QuantParam{scale, 0}, use_pot2 != 0)); });
}

// Weight / bias codes exactly as quantitativeWeightCPU produces them.
int ref_gru_quantize_weights(int I, int H, const float *W, const float *R, const float *bw, const float *br,
                             const rxmet_gru_quant_params *params,
                             int32_t *W_q, int32_t *R_q, int32_t *bw_q, int32_t *br_q) {
    return guarded([&] { quantitativeWeightCPU(I, H, W, R, bw, br, toRefParams(*params), W_q, R_q, bw_q, br_q); });
}

// Full quantized forward on the reference's CPU integer core.  Mirrors the
// steps of quantGRUForwardCPU (gru_host.cc:161-252) but also hands back the
// integer codes: x_q [T,B,I], h_q [T+1,B,H], v_q [T,B,4H]; h / v receive the
// dequantized values the reference returns (either may be NULL).
int ref_gru_forward_quant(int T, int B, int I, int H,
                          const float *W, const float *R, const float *bw, const float *br,
                          const float *x, const float *h0, const rxmet_gru_quant_params *params,
                          int32_t *x_q, int32_t *h_q, int32_t *v_q, float *h, float *v) {
    return guarded([&] {
        const GRUQuantParams p = toRefParams(*params);
        const auto &cfg = p.bitwidth_config_;
        const bool pot = cfg.usePOT2_;
        const int H3 = 3 * H;
        std::vector<int32_t> W_q(static_cast<size_t>(I) * H3), R_q(static_cast<size_t>(H) * H3), bw_q(H3), br_q(H3);
        quantitativeWeightCPU(I, H, W, R, bw, br, p, W_q.data(), R_q.data(), bw_q.data(), br_q.data());
        const size_t nx = static_cast<size_t>(T) * B * I;
        const FixedPointScale fx = toFixedScale(p.x_, pot), fh = toFixedScale(p.h_, pot);
        for (size_t i = 0; i < nx; ++i) x_q[i] = quantize(x[i], fx, p.x_.zero_point, cfg.x_);
        for (int i = 0; i < B * H; ++i)
            h_q[i] = h0 ? quantize(h0[i], fh, p.h_.zero_point, cfg.h_) : p.h_.zero_point;
        cpu::ForwardPassQuantCPU fwd(true, B, I, H);
        fwd.setRescaleParam(p);
        fwd.Run(T, W_q.data(), R_q.data(), bw_q.data(), br_q.data(), x_q, h_q, v_q, 0.0f, nullptr);
        if (h || v) {
            std::vector<float> hh(static_cast<size_t>(T + 1) * B * H), vv(static_cast<size_t>(T) * B * H * 4);
            quantGRUForwardCPU(true, T, B, I, H, W_q.data(), R_q.data(), bw_q.data(), br_q.data(), x, h0, p,
                               hh.data(), vv.data());
            if (h) std::memcpy(h, hh.data(), hh.size() * sizeof(float));
            if (v) std::memcpy(v, vv.data(), vv.size() * sizeof(float));
        }
    });
}

// Float forward + min/max observation: forwardWithCalibrationCPU with MINMAX.
int ref_gru_forward_calibrate_minmax(int T, int B, int I, int H,
                                     const float *W, const float *R, const float *bw, const float *br,
                                     const float *x, const float *h0, const rxmet_gru_quant_config *cfg,
                                     rxmet_gru_ranges *ranges, float *h, float *v) {
    return guarded([&] {
        GRUQuantizationRanges r = toRefRanges(*ranges);
        forwardWithCalibrationCPU(T, B, I, H, W, R, bw, br, x, h0, CalibrationMethod::MINMAX, &r, nullptr,
                                  toRefConfig(*cfg), h, v);
        fromRefRanges(r, ranges);
    });
}

// ---- histogram calibration ------------------------------------------------------

int ref_histogram_collect_host(rxmet_histogram *hist, const float *data, uint64_t count) {
    return guarded([&] {
        HistogramCollector c = toRefCollector(*hist);
        c.collect(data, count);
        fromRefCollector(c, hist);
    });
}

int ref_histogram_merge(rxmet_histogram *hist, const rxmet_histogram *other) {
    return guarded([&] {
        HistogramCollector c = toRefCollector(*hist);
        c.merge(toRefCollector(*other).histogram());
        fromRefCollector(c, hist);
    });
}

int ref_histogram_calibrate(const rxmet_histogram *hist, int bits, int is_unsigned, int symmetric, int use_percentile,
                            float percentile, float *scale, float *range_min, float *range_max) {
    return guarded([&] {
        const HistogramCollector c = toRefCollector(*hist);
        const ContinuousScaleResult r = calibrateContinuousScaleFromHistogram(
            c.histogram(), QuantBitWidth(static_cast<int8_t>(bits), is_unsigned != 0), symmetric != 0, use_percentile != 0,
            percentile);
        *scale = r.scale;
        *range_min = r.min;
        *range_max = r.max;
    });
}

// Float forward + histogram observation: forwardWithCalibrationCPU with SQNR (the collectors are
// fed the same way for PERCENTILE).
int ref_gru_forward_calibrate_hist(int T, int B, int I, int H, const float *W, const float *R, const float *bw,
                                   const float *br, const float *x, const float *h0, const rxmet_gru_quant_config *cfg,
                                   rxmet_gru_histograms *hists, float *h, float *v) {
    return guarded([&] {
        GRUHistogramCollectors g = toRefHists(*hists);
        forwardWithCalibrationCPU(T, B, I, H, W, R, bw, br, x, h0, CalibrationMethod::SQNR, nullptr, &g,
                                  toRefConfig(*cfg), h, v);
        fromRefHists(g, hists);
    });
}

int ref_gru_params_from_histograms(const rxmet_gru_histograms *hists, const rxmet_gru_quant_config *cfg,
                                   int use_percentile, float percentile, rxmet_gru_quant_params *out) {
    return guarded([&] {
        GRUHistogramCollectors g = toRefHists(*hists);
        const GRUQuantParams p = calculateGRUQuantitativeParametersFromHistograms(g, toRefConfig(*cfg), use_percentile != 0,
                                                                                 percentile);
        fromRefParams(p, out);
    });
}

// Scalar primitives, for known-answer tests of rounding behaviour.
int64_t ref_rshift_round_i64(int64_t x, int n) { return rshift_round(x, static_cast<int8_t>(n)); }
int32_t ref_quantize(float v, float scale, int32_t zp, int bits, int is_unsigned) {
    return quantize<false>(v, scale, zp, QuantBitWidth(static_cast<int8_t>(bits), is_unsigned != 0));
}
void ref_encode_mshift(float scale, int32_t *multiplier, int32_t *shift) {
    const FixedPointScale f = encodeMShift(scale);
    *multiplier = f.multiplier;
    *shift = f.shift;
}

}  // extern "C"
