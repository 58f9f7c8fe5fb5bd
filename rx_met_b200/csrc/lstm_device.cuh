// Device-side scalar arithmetic of the QuantLSTM q-carrier, shared by the forward kernels.
// Every function keeps the float roundings of the reference literally (no contraction, one rounding
// per reference operation), because those roundings decide integer codes.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

#include "lstm_params.h"

namespace rxmet {
namespace lstm {
namespace dev {

// rint((v * M) * 2^-shift) with the product rounded once in float
// (applyRescaleCore, operators/quant-lstm/include/quantization/float_carrier_ops.h:77-92).
__device__ __forceinline__ float rescaleF(float v, DevRescale r) {
    return rintf(__fmul_rn(__fmul_rn(v, r.mult), r.pow2));
}

// value -> clamp(rint(value / scale) + zp): division and rounding in double as the reference does
// (quantizeFp, float_carrier_ops.h:49-59).
__device__ __forceinline__ int32_t quantizeCode(float v, float scale, int32_t zp, int32_t lo, int32_t hi, uint8_t &clamped) {
    const double t = rint(static_cast<double>(v) / static_cast<double>(scale)) + static_cast<double>(zp);
    clamped = (t < static_cast<double>(lo)) || (t > static_cast<double>(hi));
    return t <= static_cast<double>(lo) ? lo : (t >= static_cast<double>(hi) ? hi : static_cast<int32_t>(t));
}

// accumulator (already a float) -> centred linear code (code - zero point) and its clamp flag
// (linearValue, operators/quant-lstm/src/lstm/forward_quantized_fp_cpu.cc:17-45).
__device__ __forceinline__ float linearCentredF(float total, DevRescale out, float cLo, float cHi, uint8_t &clamped) {
    const float r = rescaleF(total, out);
    clamped = (r < cLo) || (r > cHi);
    return fminf(fmaxf(r, cLo), cHi);
}

// Cell-update ratio (scaleCellProductFpCore, operators/quant-lstm/include/lstm/quantized_cell_fp.h:72-80).
// The double-precision form (ratios that do not fit Q31) sits behind a call, so that the common
// single multiply is not accompanied by a speculative evaluation of it.
static __device__ __noinline__ float scaleCellWide(float product, double mantissa, int exponent) {
    return static_cast<float>(ldexp(static_cast<double>(product) * mantissa, exponent));
}
__device__ __forceinline__ float scaleCell(float product, float ratio, double mantissa, int exponent, int usesFp) {
    if (usesFp) return scaleCellWide(product, mantissa, exponent);
    return __fmul_rn(product, ratio);
}

// Four signed bytes times four unsigned bytes, accumulated.
__device__ __forceinline__ int32_t dotSignedUnsigned(uint32_t signedBytes, uint32_t unsignedBytes, int32_t acc) {
    int32_t d;
    asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(signedBytes), "r"(unsignedBytes), "r"(acc));
    return d;
}

}  // namespace dev
}  // namespace lstm
}  // namespace rxmet
