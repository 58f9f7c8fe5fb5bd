/*
 * TEST INFRASTRUCTURE - not part of the shipped library.
 *
 * Plain-C restatement of the AIMET native quantize-dequantize, fixed-point quantize, min/max
 * and PDF-histogram functions of the reference's CPU path (native/common/src).  Checked bit for
 * bit against the reference's own CPU sources compiled into oracle/_ref/libaimet_ref.so and
 * against the known-answer cases of tests/integration/test_native_qdq_alignment.py (ties to
 * even, float32 reciprocal, NaN preserved, infinities saturate).
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#define ORC_PDF_SIZE (512 * 3) /* native/common/src/math_functions.hpp:80 */

/* native/common/src/quantize_dequantize.hpp:36-46 : clamp in the real domain, multiply by the
 * ROUNDED reciprocal of the scale, round half to even, multiply back. */
static float qdq_f32(float v, float mn, float mx, float scale) {
    if (v != v) return v;
    const float clipped = fmaxf(fminf(v, mx), mn);
    const float scaled = clipped * (1.0f / scale);
    return nearbyintf(scaled) * scale;
}
static double qdq_f64(double v, double mn, double mx, double scale) {
    if (v != v) return v;
    const double clipped = fmax(fmin(v, mx), mn);
    return nearbyint(clipped * (1.0 / scale)) * scale;
}

/* native/common/src/trim_functions.cpp:186-194 */
void orc_aimet_qdq_f32(const float *in, uint64_t n, double mn, double mx, double delta, float *out) {
    for (uint64_t i = 0; i < n; ++i) out[i] = qdq_f32(in[i], (float)mn, (float)mx, (float)delta);
}
void orc_aimet_qdq_f64(const double *in, uint64_t n, double mn, double mx, double delta, double *out) {
    for (uint64_t i = 0; i < n; ++i) out[i] = qdq_f64(in[i], mn, mx, delta);
}

/* native/common/src/trim_functions.cpp:671-682 */
void orc_aimet_qdq_per_channel_f32(const float *in, int channels, int64_t n, int64_t per_channel, float *out,
                                   const float *mn, const float *mx, const float *delta) {
    for (int64_t i = 0; i < n; ++i) {
        const int c = (int)((i / per_channel) % channels);
        out[i] = qdq_f32(in[i], mn[c], mx[c], delta[c]);
    }
}

/* native/common/src/trim_functions.cpp:645-668 : strides of the broadcast shapes, encoding
 * stride 0 along broadcast dimensions. */
void orc_aimet_qdq_broadcast_f32(const float *in, float *out, int64_t n, int nd, const int64_t *in_strides,
                                 const int64_t *enc_strides, const float *mn, const float *mx, const float *delta) {
    for (int64_t i = 0; i < n; ++i) {
        int64_t e = 0, rem = i;
        for (int d = 0; d < nd; ++d) {
            const int64_t idx = rem / in_strides[d];
            rem -= idx * in_strides[d];
            e += enc_strides[d] * idx;
        }
        out[i] = qdq_f32(in[i], mn[e], mx[e], delta[e]);
    }
}

/* native/common/src/trim_functions.cpp:143-167,214-230 : saturate, scale, subtract the offset,
 * round half AWAY from zero, optional shift to the signed range. */
void orc_aimet_to_fxp_f32(const float *in, uint64_t n, double mn, double mx, double delta, double offset, int bw,
                          int shift_to_signed, float *out) {
    const unsigned int shift = shift_to_signed ? (unsigned int)pow(2, bw - 1) : 0u;
    for (uint64_t i = 0; i < n; ++i) {
        float v = fmaxf(fminf(in[i], (float)mx), (float)mn);
        v = v / (float)delta - (float)offset;
        v = roundf(v);
        out[i] = v - (float)shift;
    }
}

/* native/common/src/math_functions.cpp:120-133,355-375 : NaN never wins a comparison. */
void orc_aimet_minmax_f32(const float *in, uint64_t n, uint64_t block, float *mins, float *maxs) {
    const uint64_t blocks = n / block;
    for (uint64_t b = 0; b < blocks; ++b) {
        float lo = (float)1.79769313486231570815e+308, hi = -lo; /* float(DBL_MAX) = +inf */
        for (uint64_t i = 0; i < block; ++i) {
            const float v = in[b * block + i];
            lo = (v < lo) ? v : lo;
            hi = (hi < v) ? v : hi;
        }
        mins[b] = lo;
        maxs[b] = hi;
    }
}

/* native/common/src/math_functions.cpp:395-412 */
void orc_aimet_histogram_f32(const float *in, uint64_t n, uint32_t *hist, double bucket, int pdf_offset) {
    const float inv = (float)(1 / bucket);
    memset(hist, 0, sizeof(uint32_t) * ORC_PDF_SIZE);
    for (uint64_t i = 0; i < n; ++i) {
        const float slot = floorf(in[i] * inv) - (float)pdf_offset;
        if (slot >= 0.0f && slot < (float)ORC_PDF_SIZE) hist[(int)slot] += 1;
    }
}
