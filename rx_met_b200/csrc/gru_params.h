// Host-side derivation of everything the QuantGRU kernels execute with:
// encodings from calibration ranges, M*2^-shift / power-of-two rescales, the
// 16-segment activation tables and the per-channel linear-stage parameters.
// The results are plain structs that kernels take by value or as device arrays.
#pragma once

#include <cstdint>
#include <memory>
#include <mutex>
#include <vector>

#include "rxmet_b200.h"

namespace rxmet {
namespace gru {

constexpr int kOps = RXMET_GRU_NUM_OPS;
constexpr int kSegments = 16;

// round_half_even((x * mult) >> shift); shift <= 0 is a left shift.
struct Rescale {
    int32_t mult;
    int32_t shift;
};

// One activation table in structure-of-arrays form (friendlier to a warp-wide
// segment search than the reference's array of structs).
struct Lut {
    int32_t threshold[kSegments];
    int32_t q_b[kSegments];
    int32_t n_bx[kSegments];
    int32_t term_c[kSegments];
    int32_t zp_x;
};

// Scalar execution parameters of one direction; passed to kernels by value.
struct GateExec {
    int32_t zp[kOps];
    int32_t qlo[kOps];
    int32_t qhi[kOps];
    float eff[kOps];  // scale the quantize/dequantize boundary uses (decoded M*2^-shift or 2^-n)
    Rescale ih_to_update, hh_to_update;
    Rescale ih_to_reset, hh_to_reset;
    Rescale ih_to_new, rh_to_new;
    Rescale new_to_h, update_old_to_h;
    int32_t quant_one;  // the constant 1 on the update-gate output grid
    Lut lut_update, lut_reset, lut_new;
};

// Per-channel (3*hidden) parameters of the two linear stages, uploaded as one
// block: eight arrays of 3*hidden 32-bit words each.
struct ChannelExec {
    std::vector<float> eff_W, eff_R, eff_bw, eff_br;
    std::vector<Rescale> gemm_x, bias_x, gemm_h, bias_h;
};

// Storage class of a code tensor: the narrowest signed integer that holds the
// whole grid of a quantization point.
enum class CodeClass : int { I8 = 0, I16 = 1, I32 = 2 };

struct Exec {
    int hidden = 0;
    GateExec gate{};
    ChannelExec chan;
    CodeClass weightClass = CodeClass::I8;  // W and R codes
    CodeClass actClass = CodeClass::I8;     // x and h codes
    CodeClass linearClass = CodeClass::I16; // ih / hh linear codes
    // Page-locked host copy of the per-channel block (four float arrays, four Rescale arrays) in
    // the layout the kernels read, filled on first use: uploads from it are plain asynchronous
    // copies, while pageable sources make the runtime stage every call.
    mutable std::once_flag pinnedOnce;
    mutable std::shared_ptr<int32_t> pinnedChannels;
};

// Encodings from ranges (reference: operators/quant-gru/src/gru_host.cc:13-125).
void paramsFromRanges(const rxmet_gru_ranges &ranges, const rxmet_gru_quant_config &cfg,
                      rxmet_gru_quant_params *out);

// Encodings from histogram collectors, SQNR search or percentile clipping
// (reference: operators/quant-gru/src/gru_host.cc:254-335).
void paramsFromHistograms(const rxmet_gru_histograms &hists, const rxmet_gru_quant_config &cfg, bool usePercentile,
                          float percentile, rxmet_gru_quant_params *out);

// The three tables in the public segment layout
// (reference: operators/quant-gru/src/quantize_lut.cc:17-48).
void buildLuts(const rxmet_gru_quant_params &params, rxmet_lut_segment out[3][16]);

float decodeEffectiveScale(float scale, bool usePot2);

// Full execution parameters for a parameter set.  Results are cached on the
// content of `params`, because callers hand over the same encodings on every
// step and the table generation costs tens of microseconds.
std::shared_ptr<const Exec> deriveExec(const rxmet_gru_quant_params &params);

// Parameters of the FP32 carrier (floats holding integer codes, rescales = rint(x * ratio) with ratio = source
// scale / destination scale as one float division; reference: ForwardPassQuantFP::setRescaleParam,
// operators/quant-gru/src/gru_forward_gpu_quant_fp.cu:853-1044).  Scalars travel to kernels by value, the four
// per-channel arrays (3 * hidden floats each) are uploaded per call.
struct FpCarrierScalars {
    float zp[kOps];
    float lo[kOps], hi[kOps];            // clamp bounds of every point (clamp_f, quantize_ops_helper.h:334-354)
    float ihToUpdate, hhToUpdate, ihToReset, hhToReset, ihToNew, rhToNew, newToH, updateOldToH;
    float quantOne;                      // rint(1 / scale_update_gate_output) + its zero point
};
struct FpCarrierParams {
    FpCarrierScalars s{};
    std::vector<float> channel;          // [4][3 hidden]: gemm_x -> ih linear, bw -> gemm_x, gemm_h -> hh linear, br -> gemm_h
};
FpCarrierParams deriveFpCarrier(const rxmet_gru_quant_params &params);

}  // namespace gru
}  // namespace rxmet
