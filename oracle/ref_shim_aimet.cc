// TEST INFRASTRUCTURE - not part of the shipped library.
//
// extern "C" adapter around the reference's own CPU implementation of the AIMET native
// quantize-dequantize, min/max and histogram functions (native/common/src/trim_functions.cpp,
// math_functions.cpp, tensor_utils.cpp), compiled where they lie by the Makefile beside this file
// into oracle/_ref/libaimet_ref.so.  Nothing of the reference is copied; this file only calls it.
#include <cmath>
#include <cstdint>
#include <string>
#include <tuple>
#include <vector>

#include "DlQuantization/Quantization.hpp"
#include "math_functions.hpp"
#include "trim_functions.hpp"
#include "quantization_utils.hpp"
#include "MinMaxEncodingAnalyzer.h"
#include "TfEncodingAnalyzer.h"
#include "PercentileEncodingAnalyzer.h"
#include "TfEnhancedEncodingAnalyzer.h"

using namespace DlQuantization;

namespace {
TfEncoding enc(double mn, double mx, double delta, double offset, int bw) {
    TfEncoding e;
    e.min = mn; e.max = mx; e.delta = delta; e.offset = offset; e.bw = bw;
    return e;
}
}  // namespace

extern "C" {

int ref_aimet_qdq_f32(const float *in, uint64_t n, double mn, double mx, double delta, float *out) {
    try { quantizeDequantize(in, n, enc(mn, mx, delta, 0, 8), out, COMP_MODE_CPU, ROUND_NEAREST, nullptr); return 0; }
    catch (...) { return -1; }
}
int ref_aimet_qdq_f64(const double *in, uint64_t n, double mn, double mx, double delta, double *out) {
    try { quantizeDequantize(in, n, enc(mn, mx, delta, 0, 8), out, COMP_MODE_CPU, ROUND_NEAREST, nullptr); return 0; }
    catch (...) { return -1; }
}
int ref_aimet_qdq_per_channel_f32(const float *in, int channels, int n, int perChannel, float *out, float *mn,
                                  float *mx, float *delta, float *offset) {
    try {
        quantizeDequantizePerChannel(in, channels, n, perChannel, out, mn, mx, delta, offset, COMP_MODE_CPU,
                                     ROUND_NEAREST, nullptr);
        return 0;
    } catch (...) { return -1; }
}
int ref_aimet_qdq_broadcast_f32(const float *in, float *out, int nEnc, const double *mn, const double *mx,
                                const double *delta, int nd, const int64_t *shape, const int64_t *encShape) {
    try {
        Encodings e(nEnc);
        for (int i = 0; i < nEnc; ++i) e[i] = enc(mn[i], mx[i], delta[i], 0, 8);
        quantizeDequantizeBroadcast(in, out, e, TensorDims(shape, shape + nd), TensorDims(encShape, encShape + nd),
                                    COMP_MODE_CPU, nullptr);
        return 0;
    } catch (...) { return -1; }
}
int ref_aimet_to_fxp_f32(const float *in, uint64_t n, double mn, double mx, double delta, double offset, int bw,
                         int shiftToSigned, float *out) {
    try { quantizeToFxp(in, n, enc(mn, mx, delta, offset, bw), out, COMP_MODE_CPU, ROUND_NEAREST, shiftToSigned != 0); return 0; }
    catch (...) { return -1; }
}
int ref_aimet_minmax_f32(const float *in, uint64_t n, uint64_t block, float *mins, float *maxs) {
    try {
        auto r = GetMinMax(in, n, block, COMP_MODE_CPU, nullptr, nullptr);
        const auto &a = std::get<0>(r); const auto &b = std::get<1>(r);
        for (size_t i = 0; i < a.size(); ++i) { mins[i] = a[i]; maxs[i] = b[i]; }
        return 0;
    } catch (...) { return -1; }
}
// The reference exports the bucket counting only through UpdatePdf; with a PDF whose bucket edges
// are preset to (pdfOffset + i) * bucket and no earlier iteration, pdf[i] = count[i] / n exactly.
int ref_aimet_histogram_f32(const float *in, uint64_t n, uint32_t *hist, double bucket, int pdfOffset, int isSigned) {
    try {
        PDF pdf;
        pdf.xLeft.resize(PDF_SIZE);
        for (int i = 0; i < PDF_SIZE; ++i) pdf.xLeft[i] = (static_cast<double>(pdfOffset) + i) * bucket;
        pdf.pdf.assign(PDF_SIZE, 0.0);
        pdf.iterations = 0;
        UpdatePdf(in, n, COMP_MODE_CPU, isSigned != 0, pdf, nullptr);
        for (int i = 0; i < PDF_SIZE; ++i) hist[i] = static_cast<uint32_t>(std::llround(pdf.pdf[i] * static_cast<double>(n)));
        return 0;
    } catch (...) { return -1; }
}
int ref_aimet_pdf_size(void) { return PDF_SIZE; }

// out: {min, max, delta, offset, bw}
int ref_aimet_compute_encoding(int bw, double mn, double mx, int symmetric, int strict, int unsignedSymmetric, double *out) {
    try {
        const TfEncoding e = getComputedEncodings(static_cast<uint8_t>(bw), mn, mx, symmetric != 0, strict != 0, unsignedSymmetric != 0);
        out[0] = e.min; out[1] = e.max; out[2] = e.delta; out[3] = e.offset; out[4] = e.bw;
        return 0;
    } catch (...) { return -1; }
}

// MinMaxEncodingAnalyzer<float> fed the given statistics through updateStats on two one-element tensors.
int ref_aimet_minmax_encoding(int bw, float statsMin, float statsMax, int symmetric, int strict, int unsignedSymmetric,
                              double *out) {
    try {
        MinMaxEncodingAnalyzer<float> analyzer(TensorDims{1});
        const float values[2] = {statsMin, statsMax};
        analyzer.updateStats(values, TensorDims{2}, COMP_MODE_CPU, nullptr, nullptr);
        const Encodings all = analyzer.computeEncoding(static_cast<uint8_t>(bw), symmetric != 0, strict != 0, unsignedSymmetric != 0);
        const TfEncoding &e = all[0];
        out[0] = e.min; out[1] = e.max; out[2] = e.delta; out[3] = e.offset; out[4] = e.bw;
        return 0;
    } catch (...) { return -1; }
}

// TfEncodingAnalyzer<float> (running min / max that start at zero): the batches go through updateStats in CPU mode.
int ref_aimet_tf_encoding(const float *data, const uint64_t *sizes, int batches, int bw, int symmetric, int strict,
                          int unsignedSymmetric, double *out) {
    try {
        TfEncodingAnalyzer<float> analyzer;
        for (int b = 0; b < batches; ++b) { analyzer.updateStats(data, sizes[b], COMP_MODE_CPU); data += sizes[b]; }
        const TfEncoding e = analyzer.computeEncoding(static_cast<uint8_t>(bw), symmetric != 0, strict != 0, unsignedSymmetric != 0);
        out[0] = e.min; out[1] = e.max; out[2] = e.delta; out[3] = e.offset; out[4] = e.bw;
        return 0;
    } catch (...) { return -1; }
}

// Histogram analyzers: the batches (concatenated in `data`, `sizes[i]` values each) go through
// updateStats in CPU mode, then computeEncoding.  kind 0 = TF-enhanced, 1 = percentile.
// out: {min, max, delta, offset, bw}; pdfOut (optional): xLeft[PDF_SIZE] then pdf[PDF_SIZE].
int ref_aimet_histogram_encoding(int kind, const float *data, const uint64_t *sizes, int batches, int bw, int symmetric,
                                 int strict, int unsignedSymmetric, float percentile, double *out, double *pdfOut) {
    try {
        TfEncoding e{};
        std::vector<std::tuple<double, double>> hist;
        if (kind == 0) {
            TfEnhancedEncodingAnalyzer<float> analyzer;
            for (int b = 0; b < batches; ++b) { analyzer.updateStats(data, sizes[b], COMP_MODE_CPU); data += sizes[b]; }
            e = analyzer.computeEncoding(static_cast<uint8_t>(bw), symmetric != 0, strict != 0, unsignedSymmetric != 0);
            hist = analyzer.getStatsHistogram();
        } else {
            PercentileEncodingAnalyzer<float> analyzer;
            analyzer.setPercentileValue(percentile);
            for (int b = 0; b < batches; ++b) { analyzer.updateStats(data, sizes[b], COMP_MODE_CPU); data += sizes[b]; }
            e = analyzer.computeEncoding(static_cast<uint8_t>(bw), symmetric != 0, strict != 0, unsignedSymmetric != 0);
            hist = analyzer.getStatsHistogram();
        }
        out[0] = e.min; out[1] = e.max; out[2] = e.delta; out[3] = e.offset; out[4] = e.bw;
        if (pdfOut) {
            for (size_t i = 0; i < hist.size() && i < static_cast<size_t>(PDF_SIZE); ++i) {
                pdfOut[i] = std::get<0>(hist[i]);
                pdfOut[PDF_SIZE + i] = std::get<1>(hist[i]);
            }
            if (hist.empty()) for (int i = 0; i < 2 * PDF_SIZE; ++i) pdfOut[i] = 0.0;
        }
        return static_cast<int>(hist.size());
    } catch (...) { return -1; }
}

}  // extern "C"
