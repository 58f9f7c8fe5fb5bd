/*
 * TEST INFRASTRUCTURE - not part of the shipped library.
 *
 * Plain-C CPU restatement of the reference's QuantGRU path (encodings from
 * ranges, activation tables, integer-carrier forward with clamp masks, float
 * calibration forward with min/max observation, QAT backward).  Only tests,
 * the smoke check and the CPU-baseline leg of the benchmark may load it; the
 * shipped library never does.
 *
 * Parity pin: every function here is checked bit-for-bit (codes, encodings,
 * tables, ranges) against the reference's own CPU sources compiled into
 * oracle/_ref/libgru_ref.so and against the golden fixtures generated from
 * that build (tests/golden).  The backward has no CPU implementation in the
 * reference; it restates the CUDA kernel's arithmetic and is pinned by the
 * gradient identities the reference's own tests use.
 */
#ifndef RXMET_GRU_ORACLE_H_
#define RXMET_GRU_ORACLE_H_

#include <stdint.h>

#include "rxmet_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Integer rescale: round_half_even((x * multiplier) >> shift); a power-of-two
 * rescale has multiplier 1.  shift <= 0 means a left shift. */
typedef struct orc_rescale {
    int64_t multiplier;
    int32_t shift;
} orc_rescale;

typedef struct orc_bitwidth {
    int32_t bits;
    int32_t is_unsigned;
} orc_bitwidth;

typedef struct orc_lut {
    rxmet_lut_segment seg[16];
    int32_t zp_x;
} orc_lut;

/* Everything the integer core needs, derived once from the public params. */
typedef struct orc_gru_exec {
    int32_t hidden;
    orc_bitwidth bw[RXMET_GRU_NUM_OPS];
    int32_t zp[RXMET_GRU_NUM_OPS];
    float eff_scale[RXMET_GRU_NUM_OPS]; /* decoded M*2^-shift (or 2^-n) per scalar point */
    orc_rescale ih_to_update, hh_to_update, ih_to_reset, hh_to_reset, ih_to_new, rh_to_new;
    orc_rescale new_to_h, update_old_to_h;
    int32_t quant_one;
    orc_lut lut_update, lut_reset, lut_new;
    /* per channel, 3*hidden each (malloc'd) */
    float *eff_W, *eff_R, *eff_bw, *eff_br;
    orc_rescale *gemm_x, *bias_x, *gemm_h, *bias_h;
} orc_gru_exec;

/* primitives */
int64_t orc_rshift_round(int64_t x, int n);
int32_t orc_qmin(orc_bitwidth b);
int32_t orc_qmax(orc_bitwidth b);
int32_t orc_quantize(float v, float scale, int32_t zp, orc_bitwidth b, uint8_t *keep);
int orc_encode_mshift(float scale, int32_t *multiplier, int32_t *shift);

/* encodings / tables */
int orc_gru_params_from_ranges(const rxmet_gru_ranges *ranges, const rxmet_gru_quant_config *cfg,
                               rxmet_gru_quant_params *out);
int orc_gru_build_luts(const rxmet_gru_quant_params *params, rxmet_lut_segment out[3][16]);
int orc_gru_decode_effective_scale(float scale, int use_pot2, float *out);
int orc_gru_exec_init(orc_gru_exec *e, const rxmet_gru_quant_params *params);
void orc_gru_exec_free(orc_gru_exec *e);

/* forward paths (all host memory) */
int orc_gru_forward_quant(int is_training, int T, int B, int I, int H,
                          const float *W, const float *R, const float *bw, const float *br,
                          const float *x, const float *h0, const rxmet_gru_quant_params *params,
                          float *h, float *v,
                          int32_t *W_q, int32_t *R_q, int32_t *bw_q, int32_t *br_q,
                          int32_t *x_q, int32_t *h_q, int32_t *v_q,
                          const rxmet_gru_masks *masks);
int orc_gru_forward_fp(int T, int B, int I, int H,
                       const float *W, const float *R, const float *bw, const float *br,
                       const float *x, const float *h0, float *h, float *v);
int orc_gru_forward_calibrate_minmax(int T, int B, int I, int H,
                                     const float *W, const float *R, const float *bw, const float *br,
                                     const float *x, const float *h0,
                                     rxmet_gru_ranges *ranges, float *h, float *v);

/* backward (host memory).  codes are the int32 codes saved by the forward. */
int orc_gru_backward_quant(int T, int B, int I, int H,
                           const int32_t *W_q, const int32_t *R_q, const int32_t *bw_q,
                           const int32_t *br_q, const int32_t *x_q,
                           const float *dh_new, const float *h, const float *v,
                           const rxmet_gru_quant_params *params, const rxmet_gru_masks *masks,
                           float *dx, float *dW, float *dR, float *dbw, float *dbr, float *dh0);
int orc_gru_backward_fp(int T, int B, int I, int H,
                        const float *W, const float *R, const float *bw, const float *br,
                        const float *x, const float *dh_new, const float *h, const float *v,
                        float *dx, float *dW, float *dR, float *dbw, float *dbr, float *dh0);

#ifdef __cplusplus
}
#endif
#endif
