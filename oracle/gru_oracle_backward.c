/*
 * TEST INFRASTRUCTURE - not part of the shipped library (see gru_oracle.h).
 *
 * QAT / float backward of the reference's GRU restated in plain C.  The
 * reference has this path only as CUDA (operators/quant-gru/src/
 * gru_backward_gpu_quant.cu); the pointwise arithmetic below follows that
 * kernel in fp32, the three contractions (dh += R dq, dx = W dp, dW/dR) are
 * accumulated in double so that the checker is at least as accurate as any
 * fp32 summation order.
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "gru_oracle.h"

static float mk(const uint8_t *m, size_t i) { return m ? (float)m[i] : 1.0f; }

/* gru_backward_gpu_quant.cu:93-266 (pointwise) and :380-493 (time loop and the
 * whole-sequence GEMMs).  W [I,3H], R [H,3H], x [T,B,I] are real-valued. */
static int backward_core(int T, int B, int I, int H, const float *W, const float *R, const float *x,
                         const float *dh_new, const float *h, const float *v,
                         const rxmet_gru_masks *masks,
                         float *dx, float *dW, float *dR, float *dbw, float *dbr, float *dh0) {
    const int C = 3 * H;
    const size_t NB = (size_t)T * B;
    rxmet_gru_masks none;
    memset(&none, 0, sizeof(none));
    const rxmet_gru_masks *m = masks ? masks : &none;
    float *dp = (float *)malloc(sizeof(float) * NB * C);
    float *dq = (float *)malloc(sizeof(float) * NB * C);
    float *dh = (float *)calloc((size_t)B * H, sizeof(float));
    double *dbw_acc = (double *)calloc(C, sizeof(double));
    double *dbr_acc = (double *)calloc(C, sizeof(double));
    double *tmp = (double *)malloc(sizeof(double) * (size_t)B * H);

    for (int t = T - 1; t >= 0; --t) {
        float *dp_t = dp + (size_t)t * B * C, *dq_t = dq + (size_t)t * B * C;
        for (int b = 0; b < B; ++b)
            for (int j = 0; j < H; ++j) {
                const size_t bi = (size_t)b * H + j;
                const size_t hi = (size_t)t * B * H + bi;
                const size_t vi = ((size_t)t * B + b) * 4 * H + j;
                const size_t gi = ((size_t)t * B + b) * C + j;
                const size_t li = (size_t)b * C + j;
                float dh_total = dh_new[(size_t)(t + 1) * B * H + bi] + dh[bi];
                dh_total *= mk(m->h, hi);
                const float z = v[vi], r = v[vi + H], g = v[vi + 2 * H], q_g = v[vi + 3 * H];
                dh[bi] = z * dh_total;
                const float dg = (1.0f - z) * dh_total;
                const float dz = (h[hi] - g) * dh_total;
                float dp_g = (1.0f - g * g) * dg;
                dp_g *= mk(m->gate_output, gi + 2 * H);
                dp_g *= mk(m->gate_input, gi + 2 * H);
                const float dq_g = dp_g * r;
                const float dr = dp_g * q_g;
                const float dp_r = (r * (1.0f - r)) * dr;
                const float dp_z = (z * (1.0f - z)) * dz;
                float fpz = dp_z, fpr = dp_r, fpg = dp_g, fqz = dp_z, fqr = dp_r, fqg = dq_g;
                const float zo = mk(m->gate_output, gi), ro = mk(m->gate_output, gi + H);
                fpz *= zo; fqz *= zo; fpr *= ro; fqr *= ro;
                const float zi = mk(m->gate_input, gi), ri = mk(m->gate_input, gi + H);
                fpz *= zi; fqz *= zi; fpr *= ri; fqr *= ri;
                fqz *= mk(m->weight_hh_linear, gi);
                fqr *= mk(m->weight_hh_linear, gi + H);
                fqg *= mk(m->weight_hh_linear, gi + 2 * H);
                fpz *= mk(m->weight_ih_linear, gi);
                fpr *= mk(m->weight_ih_linear, gi + H);
                fpg *= mk(m->weight_ih_linear, gi + 2 * H);
                dp_t[li] = fpz; dp_t[li + H] = fpr; dp_t[li + 2 * H] = fpg;
                dq_t[li] = fqz; dq_t[li + H] = fqr; dq_t[li + 2 * H] = fqg;
                dbw_acc[j] += (double)(fpz * mk(m->bw, j));
                dbw_acc[j + H] += (double)(fpr * mk(m->bw, j + H));
                dbw_acc[j + 2 * H] += (double)(fpg * mk(m->bw, j + 2 * H));
                dbr_acc[j] += (double)(fqz * mk(m->br, j));
                dbr_acc[j + H] += (double)(fqr * mk(m->br, j + H));
                dbr_acc[j + 2 * H] += (double)(fqg * mk(m->br, j + 2 * H));
            }
        /* dh[b,k] += sum_j R[k,j] * dq[b,j] */
        for (int b = 0; b < B; ++b)
            for (int k = 0; k < H; ++k) {
                double s = 0.0;
                const float *rk = R + (size_t)k * C, *dqb = dq_t + (size_t)b * C;
                for (int j = 0; j < C; ++j) s += (double)rk[j] * (double)dqb[j];
                tmp[(size_t)b * H + k] = s;
            }
        for (size_t i = 0; i < (size_t)B * H; ++i) dh[i] = (float)((double)dh[i] + tmp[i]);
    }

    /* dx[n,i] = sum_j W[i,j] dp[n,j], then the input clamp mask */
#pragma omp parallel for schedule(static)
    for (long n = 0; n < (long)NB; ++n)
        for (int i = 0; i < I; ++i) {
            double s = 0.0;
            const float *wi = W + (size_t)i * C, *dpn = dp + (size_t)n * C;
            for (int j = 0; j < C; ++j) s += (double)wi[j] * (double)dpn[j];
            dx[(size_t)n * I + i] = (float)s * mk(m->x, (size_t)n * I + i);
        }
    /* dR[k,j] = sum_n h[n,k] dq[n,j] with h[n] the state entering step n */
#pragma omp parallel for schedule(static)
    for (int k = 0; k < H; ++k)
        for (int j = 0; j < C; ++j) {
            double s = 0.0;
            for (size_t n = 0; n < NB; ++n) s += (double)h[n * H + k] * (double)dq[n * C + j];
            dR[(size_t)k * C + j] = (float)s * mk(m->R, (size_t)k * C + j);
        }
#pragma omp parallel for schedule(static)
    for (int i = 0; i < I; ++i)
        for (int j = 0; j < C; ++j) {
            double s = 0.0;
            for (size_t n = 0; n < NB; ++n) s += (double)x[n * I + i] * (double)dp[n * C + j];
            dW[(size_t)i * C + j] = (float)s * mk(m->W, (size_t)i * C + j);
        }
    for (int c = 0; c < C; ++c) { dbw[c] = (float)dbw_acc[c]; dbr[c] = (float)dbr_acc[c]; }
    for (size_t i = 0; i < (size_t)B * H; ++i) dh0[i] = dh[i] * mk(m->h0, i);
    free(dp); free(dq); free(dh); free(dbw_acc); free(dbr_acc); free(tmp);
    return 0;
}

/* operators/quant-gru/pytorch/lib/gru_interface_binding.cc:842-870 : saved codes
 * are dequantized with the effective (M*2^-shift) scales before the backward. */
int orc_gru_backward_quant(int T, int B, int I, int H,
                           const int32_t *W_q, const int32_t *R_q, const int32_t *bw_q,
                           const int32_t *br_q, const int32_t *x_q,
                           const float *dh_new, const float *h, const float *v,
                           const rxmet_gru_quant_params *params, const rxmet_gru_masks *masks,
                           float *dx, float *dW, float *dR, float *dbw, float *dbr, float *dh0) {
    (void)bw_q; (void)br_q;
    if (T <= 0 || B <= 0 || I <= 0 || H <= 0 || params->hidden != H) return -1;
    orc_gru_exec e;
    if (orc_gru_exec_init(&e, params)) return -1;
    const int C = 3 * H;
    const size_t NB = (size_t)T * B;
    float *W = (float *)malloc(sizeof(float) * (size_t)I * C);
    float *R = (float *)malloc(sizeof(float) * (size_t)H * C);
    float *x = (float *)malloc(sizeof(float) * NB * I);
    for (int k = 0; k < I; ++k)
        for (int c = 0; c < C; ++c) W[(size_t)k * C + c] = (float)W_q[(size_t)k * C + c] * e.eff_W[c];
    for (int k = 0; k < H; ++k)
        for (int c = 0; c < C; ++c) R[(size_t)k * C + c] = (float)R_q[(size_t)k * C + c] * e.eff_R[c];
    for (size_t i = 0; i < NB * I; ++i)
        x[i] = ((float)x_q[i] - (float)e.zp[RXMET_GRU_X]) * e.eff_scale[RXMET_GRU_X];
    const int rc = backward_core(T, B, I, H, W, R, x, dh_new, h, v, masks, dx, dW, dR, dbw, dbr, dh0);
    free(W); free(R); free(x);
    orc_gru_exec_free(&e);
    return rc;
}

int orc_gru_backward_fp(int T, int B, int I, int H,
                        const float *W, const float *R, const float *bw, const float *br,
                        const float *x, const float *dh_new, const float *h, const float *v,
                        float *dx, float *dW, float *dR, float *dbw, float *dbr, float *dh0) {
    (void)bw; (void)br;
    if (T <= 0 || B <= 0 || I <= 0 || H <= 0) return -1;
    return backward_core(T, B, I, H, W, R, x, dh_new, h, v, NULL, dx, dW, dR, dbw, dbr, dh0);
}
