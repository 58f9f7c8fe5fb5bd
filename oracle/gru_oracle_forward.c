/*
 * TEST INFRASTRUCTURE - not part of the shipped library (see gru_oracle.h).
 *
 * Forward paths of the reference's QuantGRU restated in plain C: the integer
 * carrier (codes, clamp masks, dequantized outputs), the float forward and the
 * float calibration forward with min/max observation.  Citations are
 * <file under operators/quant-gru/>:<line>.
 */
#include <float.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "gru_oracle.h"

int64_t orc_apply_rescale(int64_t x, orc_rescale r);

/* include/quantize_ops_helper.h:267-278 : clamp; keep = 1 when not clamped. */
static int32_t clamp_bw(int32_t v, orc_bitwidth b, uint8_t *keep) {
    const int32_t lo = orc_qmin(b), hi = orc_qmax(b);
    if (keep) *keep = (v < lo || v > hi) ? 0 : 1;
    return v < lo ? lo : (v > hi ? hi : v);
}

/* include/quantize_ops_helper.h:503-532 : segment search with '<' and the
 * linear piece, no saturation. */
static int32_t lut_raw(int32_t q_x, const orc_lut *lut) {
    int s = 15;
    for (int i = 0; i < 16; ++i) {
        if (q_x < lut->seg[i].threshold) { s = i; break; }
    }
    const rxmet_lut_segment *p = &lut->seg[s];
    const int32_t off = q_x - lut->zp_x;
    const int64_t bx = (int64_t)p->q_b * (int64_t)off;
    const int32_t term = (p->n_bx_total >= 0) ? (int32_t)orc_rshift_round(bx, p->n_bx_total)
                                              : (int32_t)(bx << (-p->n_bx_total));
    return term + p->term_c;
}

/* include/quantize_ops_helper.h:683-838 : update and reset gates share one
 * form; the input clamp mask and the output clamp mask are separate. */
static int32_t sigmoid_gate(int32_t ih, int32_t hh, const orc_gru_exec *e, orc_rescale r_ih,
                            orc_rescale r_hh, int op_in, int op_out, const orc_lut *lut,
                            uint8_t *keep_in, uint8_t *keep_out) {
    const int64_t ih_d = (int64_t)ih - e->zp[RXMET_GRU_WEIGHT_IH_LINEAR];
    const int64_t hh_d = (int64_t)hh - e->zp[RXMET_GRU_WEIGHT_HH_LINEAR];
    const int32_t a = (int32_t)orc_apply_rescale(ih_d, r_ih);
    const int32_t b = (int32_t)orc_apply_rescale(hh_d, r_hh);
    const int32_t pre = a + b + e->zp[op_in];
    const int32_t pre_c = clamp_bw(pre, e->bw[op_in], keep_in);
    return clamp_bw(lut_raw(pre_c, lut), e->bw[op_out], keep_out);
}

/* include/quantize_ops_helper.h:854-936 */
static int32_t new_gate(int32_t ih, int32_t hh, int32_t r, const orc_gru_exec *e,
                        uint8_t *keep_in, uint8_t *keep_out) {
    const int64_t r_d = (int64_t)r - e->zp[RXMET_GRU_RESET_GATE_OUTPUT];
    const int64_t hh_d = (int64_t)hh - e->zp[RXMET_GRU_WEIGHT_HH_LINEAR];
    const int32_t rh = (int32_t)orc_apply_rescale(r_d * hh_d, e->rh_to_new);
    const int32_t a = (int32_t)orc_apply_rescale((int64_t)ih - e->zp[RXMET_GRU_WEIGHT_IH_LINEAR], e->ih_to_new);
    const int32_t pre = a + rh + e->zp[RXMET_GRU_NEW_GATE_INPUT];
    const int32_t pre_c = clamp_bw(pre, e->bw[RXMET_GRU_NEW_GATE_INPUT], keep_in);
    return clamp_bw(lut_raw(pre_c, &e->lut_new), e->bw[RXMET_GRU_NEW_GATE_OUTPUT], keep_out);
}

/* include/quantize_ops_helper.h:947-1023 */
static int32_t hidden_state(int32_t u, int32_t n, int32_t h_old, const orc_gru_exec *e, uint8_t *keep) {
    const int32_t zp_h = e->zp[RXMET_GRU_H];
    const int64_t n_d = (int64_t)n - e->zp[RXMET_GRU_NEW_GATE_OUTPUT];
    const int32_t n_al = (int32_t)orc_apply_rescale(n_d, e->new_to_h) + zp_h;
    const int64_t u_d = (int64_t)u - e->zp[RXMET_GRU_UPDATE_GATE_OUTPUT];
    const int64_t h_d = (int64_t)h_old - zp_h;
    const int64_t old_c = u_d * h_d;
    const int64_t one_minus_u = (int64_t)e->quant_one - u;
    const int64_t new_c = one_minus_u * ((int64_t)n_al - zp_h);
    const int32_t h_new = (int32_t)orc_apply_rescale(old_c + new_c, e->update_old_to_h) + zp_h;
    return clamp_bw(h_new, e->bw[RXMET_GRU_H], keep);
}

/* src/gru_forward_cpu_quant.cc:113-168 and src/gru_forward_gpu_quant.cu:109-180 :
 * out[n,m] = clamp(rescale(acc - sumW*zp + rescale(bias)) + zp_out). */
static void linear_stage(int N, int K, int C, const int32_t *Wq, const int32_t *in, const int32_t *bias,
                         int32_t zp_in, const orc_rescale *r_gemm, const orc_rescale *r_bias,
                         int32_t zp_out, orc_bitwidth bw_out, int32_t *out, uint8_t *mask) {
    int64_t *wsum = (int64_t *)malloc(sizeof(int64_t) * C);
    int64_t *bsh = (int64_t *)malloc(sizeof(int64_t) * C);
    for (int m = 0; m < C; ++m) {
        int64_t s = 0;
        for (int k = 0; k < K; ++k) s += Wq[(size_t)k * C + m];
        wsum[m] = s * zp_in;
        bsh[m] = orc_apply_rescale((int64_t)bias[m], r_bias[m]);
    }
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n) {
        int64_t acc[8];
        for (int m0 = 0; m0 < C; m0 += 8) {
            const int mw = C - m0 < 8 ? C - m0 : 8;
            for (int j = 0; j < mw; ++j) acc[j] = 0;
            for (int k = 0; k < K; ++k) {
                const int64_t a = in[(size_t)n * K + k];
                const int32_t *w = Wq + (size_t)k * C + m0;
                for (int j = 0; j < mw; ++j) acc[j] += (int64_t)w[j] * a;
            }
            for (int j = 0; j < mw; ++j) {
                const int m = m0 + j;
                const int64_t g = acc[j] - wsum[m];
                const int64_t res = orc_apply_rescale(g + bsh[m], r_gemm[m]);
                const int32_t q = (int32_t)res + zp_out;
                out[(size_t)n * C + m] = clamp_bw(q, bw_out, mask ? &mask[(size_t)n * C + m] : NULL);
            }
        }
    }
    free(wsum);
    free(bsh);
}

#define ORC_ALLOC(ptr, type, count, owned)                   \
    do {                                                     \
        if (!(ptr)) {                                        \
            (owned) = (type *)malloc(sizeof(type) * (count)); \
            (ptr) = (owned);                                 \
        }                                                    \
    } while (0)

/* src/gru_interface.cc:430-556 (quantGRUForwardInt), src/gru_host.cc:127-231 and
 * src/gru_forward_cpu_quant.cc:170-216,313-335. */
int orc_gru_forward_quant(int is_training, int T, int B, int I, int H,
                          const float *W, const float *R, const float *bw, const float *br,
                          const float *x, const float *h0, const rxmet_gru_quant_params *params,
                          float *h, float *v,
                          int32_t *W_q, int32_t *R_q, int32_t *bw_q, int32_t *br_q,
                          int32_t *x_q, int32_t *h_q, int32_t *v_q,
                          const rxmet_gru_masks *masks) {
    if (T <= 0 || B <= 0 || I <= 0 || H <= 0 || params->hidden != H) return -1;
    orc_gru_exec e;
    if (orc_gru_exec_init(&e, params)) return -1;
    const int C = 3 * H;
    const size_t NB = (size_t)T * B;
    rxmet_gru_masks none;
    memset(&none, 0, sizeof(none));
    const rxmet_gru_masks *mk = (is_training && masks) ? masks : &none;

    int32_t *oW = NULL, *oR = NULL, *obw = NULL, *obr = NULL, *ox = NULL, *oh = NULL, *ov = NULL;
    ORC_ALLOC(W_q, int32_t, (size_t)I * C, oW);
    ORC_ALLOC(R_q, int32_t, (size_t)H * C, oR);
    ORC_ALLOC(bw_q, int32_t, C, obw);
    ORC_ALLOC(br_q, int32_t, C, obr);
    ORC_ALLOC(x_q, int32_t, NB * I, ox);
    ORC_ALLOC(h_q, int32_t, (NB + B) * H, oh);
    ORC_ALLOC(v_q, int32_t, NB * H * 4, ov);
    int32_t *ih = (int32_t *)malloc(sizeof(int32_t) * NB * C);
    int32_t *hh = (int32_t *)malloc(sizeof(int32_t) * (size_t)B * C);

    /* weights and biases: per-channel symmetric, zero point 0 */
    for (int k = 0; k < I; ++k)
        for (int m = 0; m < C; ++m) {
            const size_t i = (size_t)k * C + m;
            W_q[i] = orc_quantize(W[i], e.eff_W[m], 0, e.bw[RXMET_GRU_W], mk->W ? &mk->W[i] : NULL);
        }
    for (int k = 0; k < H; ++k)
        for (int m = 0; m < C; ++m) {
            const size_t i = (size_t)k * C + m;
            R_q[i] = orc_quantize(R[i], e.eff_R[m], 0, e.bw[RXMET_GRU_R], mk->R ? &mk->R[i] : NULL);
        }
    for (int m = 0; m < C; ++m) {
        bw_q[m] = orc_quantize(bw[m], e.eff_bw[m], 0, e.bw[RXMET_GRU_BW], mk->bw ? &mk->bw[m] : NULL);
        br_q[m] = orc_quantize(br[m], e.eff_br[m], 0, e.bw[RXMET_GRU_BR], mk->br ? &mk->br[m] : NULL);
    }
    for (size_t i = 0; i < NB * I; ++i)
        x_q[i] = orc_quantize(x[i], e.eff_scale[RXMET_GRU_X], e.zp[RXMET_GRU_X], e.bw[RXMET_GRU_X],
                              mk->x ? &mk->x[i] : NULL);
    for (int i = 0; i < B * H; ++i)
        h_q[i] = h0 ? orc_quantize(h0[i], e.eff_scale[RXMET_GRU_H], e.zp[RXMET_GRU_H], e.bw[RXMET_GRU_H],
                                   mk->h0 ? &mk->h0[i] : NULL)
                    : e.zp[RXMET_GRU_H];

    linear_stage((int)NB, I, C, W_q, x_q, bw_q, e.zp[RXMET_GRU_X], e.gemm_x, e.bias_x,
                 e.zp[RXMET_GRU_WEIGHT_IH_LINEAR], e.bw[RXMET_GRU_WEIGHT_IH_LINEAR], ih, mk->weight_ih_linear);

    for (int t = 0; t < T; ++t) {
        const int32_t *h_old = h_q + (size_t)t * B * H;
        int32_t *h_new = h_q + (size_t)(t + 1) * B * H;
        const size_t off3 = (size_t)t * B * C;
        linear_stage(B, H, C, R_q, h_old, br_q, e.zp[RXMET_GRU_H], e.gemm_h, e.bias_h,
                     e.zp[RXMET_GRU_WEIGHT_HH_LINEAR], e.bw[RXMET_GRU_WEIGHT_HH_LINEAR], hh,
                     mk->weight_hh_linear ? mk->weight_hh_linear + off3 : NULL);
        for (int b = 0; b < B; ++b)
            for (int j = 0; j < H; ++j) {
                const size_t li = (size_t)b * C + j;
                const size_t gi = off3 + li;
                uint8_t ki[3], ko[3], kh;
                const int32_t z = sigmoid_gate(ih[gi], hh[li], &e, e.ih_to_update, e.hh_to_update,
                                               RXMET_GRU_UPDATE_GATE_INPUT, RXMET_GRU_UPDATE_GATE_OUTPUT,
                                               &e.lut_update, &ki[0], &ko[0]);
                const int32_t r = sigmoid_gate(ih[gi + H], hh[li + H], &e, e.ih_to_reset, e.hh_to_reset,
                                               RXMET_GRU_RESET_GATE_INPUT, RXMET_GRU_RESET_GATE_OUTPUT,
                                               &e.lut_reset, &ki[1], &ko[1]);
                const int32_t n = new_gate(ih[gi + 2 * H], hh[li + 2 * H], r, &e, &ki[2], &ko[2]);
                const size_t vi = ((size_t)t * B + b) * 4 * H + j;
                v_q[vi] = z;
                v_q[vi + H] = r;
                v_q[vi + 2 * H] = n;
                v_q[vi + 3 * H] = hh[li + 2 * H];
                h_new[(size_t)b * H + j] = hidden_state(z, n, h_old[(size_t)b * H + j], &e, &kh);
                for (int g = 0; g < 3; ++g) {
                    if (mk->gate_input) mk->gate_input[gi + (size_t)g * H] = ki[g];
                    if (mk->gate_output) mk->gate_output[gi + (size_t)g * H] = ko[g];
                }
                if (mk->h) mk->h[((size_t)t * B + b) * H + j] = kh;
            }
    }

    /* dequantize with the effective scales: x = (q - zp) * (M * 2^-shift)
     * (include/quantize_ops_helper.h:450-454, src/gru_host.cc:202-229). */
    if (h)
        for (size_t i = 0; i < (NB + B) * H; ++i)
            h[i] = (float)(h_q[i] - e.zp[RXMET_GRU_H]) * e.eff_scale[RXMET_GRU_H];
    if (v) {
        static const int vop[4] = {RXMET_GRU_UPDATE_GATE_OUTPUT, RXMET_GRU_RESET_GATE_OUTPUT,
                                   RXMET_GRU_NEW_GATE_OUTPUT, RXMET_GRU_WEIGHT_HH_LINEAR};
        for (size_t n = 0; n < NB; ++n)
            for (int g = 0; g < 4; ++g)
                for (int j = 0; j < H; ++j) {
                    const size_t i = n * 4 * H + (size_t)g * H + j;
                    v[i] = (float)(v_q[i] - e.zp[vop[g]]) * e.eff_scale[vop[g]];
                }
    }
    free(ih); free(hh);
    free(oW); free(oR); free(obw); free(obr); free(ox); free(oh); free(ov);
    orc_gru_exec_free(&e);
    return 0;
}

/* include/inline_ops.h:29-31 : on the host the unqualified exp() of the
 * reference resolves to the double overload, so the quotient is formed in
 * double and rounded to float once. */
static float sigmoid_f(float x) { return (float)(1.0 / (1.0 + exp((double)(-x)))); }

typedef struct fp_trace {
    float *wx, *rh, *z_pre, *r_pre, *n_pre, *z, *r, *n, *rh_mul, *new_c, *old_c;
} fp_trace;

/* src/gru_forward_cpu.cc:58-121 : sequential float sums in k order, bias added
 * after the sum. */
static void forward_float(int T, int B, int I, int H, const float *W, const float *R, const float *bw,
                          const float *br, const float *x, const float *h0, float *h, float *v,
                          fp_trace *tr) {
    const int C = 3 * H, nh = B * H;
    if (h0) memcpy(h, h0, sizeof(float) * nh);
    else memset(h, 0, sizeof(float) * nh);
    float *wx_row = (float *)malloc(sizeof(float) * C), *rh_row = (float *)malloc(sizeof(float) * C);
    for (int t = 0; t < T; ++t)
        for (int b = 0; b < B; ++b) {
            const size_t lin = ((size_t)t * B + b) * C;
            for (int c = 0; c < C; ++c) {
                float si = 0.0f, sh = 0.0f;
                for (int k = 0; k < I; ++k) si += x[((size_t)t * B + b) * I + k] * W[(size_t)k * C + c];
                for (int k = 0; k < H; ++k) sh += h[(size_t)t * nh + (size_t)b * H + k] * R[(size_t)k * C + c];
                wx_row[c] = si + bw[c];
                rh_row[c] = sh + br[c];
                if (tr) { tr->wx[lin + c] = wx_row[c]; tr->rh[lin + c] = rh_row[c]; }
            }
            for (int c = 0; c < H; ++c) {
                const size_t idx = (size_t)t * nh + (size_t)b * H + c;
                const float zp = wx_row[c] + rh_row[c];
                const float rp = wx_row[H + c] + rh_row[H + c];
                const float z = sigmoid_f(zp), r = sigmoid_f(rp);
                const float rec = rh_row[2 * H + c];
                const float rm = r * rec;
                const float np = wx_row[2 * H + c] + rm;
                const float n = tanhf(np);
                const float oc = z * h[idx];
                const float nc = (1.0f - z) * n;
                h[idx + nh] = oc + nc;
                if (tr) {
                    tr->z_pre[idx] = zp; tr->r_pre[idx] = rp; tr->n_pre[idx] = np;
                    tr->z[idx] = z; tr->r[idx] = r; tr->n[idx] = n;
                    tr->rh_mul[idx] = rm; tr->new_c[idx] = nc; tr->old_c[idx] = oc;
                }
                if (v) {
                    const size_t base = ((size_t)t * B + b) * H * 4 + c;
                    v[base] = z; v[base + H] = r; v[base + 2 * H] = n; v[base + 3 * H] = rec;
                }
            }
        }
    free(wx_row); free(rh_row);
}

int orc_gru_forward_fp(int T, int B, int I, int H, const float *W, const float *R, const float *bw,
                       const float *br, const float *x, const float *h0, float *h, float *v) {
    if (T <= 0 || B <= 0 || I <= 0 || H <= 0) return -1;
    forward_float(T, B, I, H, W, R, bw, br, x, h0, h, v, NULL);
    return 0;
}

/* src/gru_forward_cpu.cc:11-26 : finite values only; an all-non-finite block
 * observes 0. */
static void observe(const float *d, size_t n, float *mn, float *mx) {
    float lo = FLT_MAX, hi = -FLT_MAX;
    for (size_t i = 0; i < n; ++i)
        if (isfinite(d[i])) {
            if (d[i] < lo) lo = d[i];
            if (d[i] > hi) hi = d[i];
        }
    if (lo > hi) lo = hi = 0.0f;
    if (lo < *mn) *mn = lo;
    if (hi > *mx) *mx = hi;
}

/* src/gru_forward_cpu.cc:28-55 (per-channel part) */
static void observe_param(const float *vals, int rows, int H, float *mn, float *mx) {
    const int C = 3 * H;
    float *col = (float *)malloc(sizeof(float) * rows);
    for (int c = 0; c < C; ++c) {
        for (int k = 0; k < rows; ++k) col[k] = vals[(size_t)k * C + c];
        observe(col, (size_t)rows, &mn[c], &mx[c]);
    }
    free(col);
}

/* src/gru_forward_cpu.cc:58-151 with CalibrationMethod::MINMAX */
int orc_gru_forward_calibrate_minmax(int T, int B, int I, int H, const float *W, const float *R,
                                     const float *bw, const float *br, const float *x, const float *h0,
                                     rxmet_gru_ranges *rg, float *h, float *v) {
    if (T <= 0 || B <= 0 || I <= 0 || H <= 0 || rg->hidden != H) return -1;
    const size_t cnt = (size_t)T * B * H;
    fp_trace tr;
    float *buf = (float *)malloc(sizeof(float) * cnt * 15);
    tr.wx = buf; tr.rh = buf + 3 * cnt;
    float *p = buf + 6 * cnt;
    tr.z_pre = p; tr.r_pre = p + cnt; tr.n_pre = p + 2 * cnt; tr.z = p + 3 * cnt; tr.r = p + 4 * cnt;
    tr.n = p + 5 * cnt; tr.rh_mul = p + 6 * cnt; tr.new_c = p + 7 * cnt; tr.old_c = p + 8 * cnt;
    forward_float(T, B, I, H, W, R, bw, br, x, h0, h, v, &tr);
#define OBS(data, count, op) observe(data, count, &rg->min[op], &rg->max[op])
    OBS(x, (size_t)T * B * I, RXMET_GRU_X);
    OBS(h + (size_t)B * H, cnt, RXMET_GRU_H); /* h[0] is not sampled */
    OBS(tr.wx, 3 * cnt, RXMET_GRU_WEIGHT_IH_LINEAR);
    OBS(tr.rh, 3 * cnt, RXMET_GRU_WEIGHT_HH_LINEAR);
    OBS(tr.z_pre, cnt, RXMET_GRU_UPDATE_GATE_INPUT);
    OBS(tr.r_pre, cnt, RXMET_GRU_RESET_GATE_INPUT);
    OBS(tr.n_pre, cnt, RXMET_GRU_NEW_GATE_INPUT);
    OBS(tr.z, cnt, RXMET_GRU_UPDATE_GATE_OUTPUT);
    OBS(tr.r, cnt, RXMET_GRU_RESET_GATE_OUTPUT);
    OBS(tr.n, cnt, RXMET_GRU_NEW_GATE_OUTPUT);
    OBS(tr.rh_mul, cnt, RXMET_GRU_MUL_RESET_HIDDEN);
    OBS(tr.new_c, cnt, RXMET_GRU_MUL_NEW_CONTRIBUTION);
    OBS(tr.old_c, cnt, RXMET_GRU_MUL_OLD_CONTRIBUTION);
#undef OBS
    observe_param(W, I, H, rg->min_W, rg->max_W);
    observe_param(R, H, H, rg->min_R, rg->max_R);
    observe_param(bw, 1, H, rg->min_bw, rg->max_bw);
    observe_param(br, 1, H, rg->min_br, rg->max_br);
    free(buf);
    return 0;
}
