/*
 * TEST INFRASTRUCTURE - CPU restatement of the float LSTM forward, the float
 * backward through time (with the optional clamp masks of the QAT path) and the
 * min/max calibration collector of rx-met's QuantLSTM.  Checker only.
 *
 * Pinned against the reference's CPU sources compiled into
 * oracle/_ref/liblstm_ref.so (tests/test_lstm_cpu.py).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "lstm_oracle.h"

static float sigmoid_f(float v) {
    /* operators/quant-lstm/src/lstm/forward_float_cpu.cc:21-28 */
    if (v >= 0.0f) {
        const float e = expf(-v);
        return 1.0f / (1.0f + e);
    }
    const float e = expf(v);
    return e / (1.0f + e);
}

int orc_lstm_forward_float(int T, int B, int I, int H, const float *w_ih, const float *w_hh, const float *b_ih,
                           const float *b_hh, const float *x, const float *h0, const float *c0, float *out, float *hn,
                           float *cn, float *ih_lin, float *hh_lin, float *gate_in, float *gate_out, float *cell,
                           float *cell_tanh, float *hidden) {
    /* forward_float_cpu.cc:49-154 */
    const int C = 4 * H;
    const size_t BH = (size_t)B * H;
    for (size_t i = 0; i < BH; ++i) {
        hn[i] = h0 ? h0[i] : 0.0f;
        cn[i] = c0 ? c0[i] : 0.0f;
    }
    for (int t = 0; t < T; ++t) {
#pragma omp parallel for schedule(static)
        for (int b = 0; b < B; ++b) {
            float gates[4 * 1024];
            float *g = C <= 4096 ? gates : malloc(sizeof(float) * C);
            const float *xr = x + ((size_t)t * B + b) * I;
            float *hr = hn + (size_t)b * H, *cr = cn + (size_t)b * H;
            const size_t go = ((size_t)t * B + b) * C, so = ((size_t)t * B + b) * H;
            for (int ch = 0; ch < C; ++ch) {
                float a = b_ih ? b_ih[ch] : 0.0f, r = b_hh ? b_hh[ch] : 0.0f;
                for (int k = 0; k < I; ++k) a += w_ih[(size_t)ch * I + k] * xr[k];
                for (int k = 0; k < H; ++k) r += w_hh[(size_t)ch * H + k] * hr[k];
                g[ch] = a + r;
                if (ih_lin) ih_lin[go + ch] = a;
                if (hh_lin) hh_lin[go + ch] = r;
                if (gate_in) gate_in[go + ch] = g[ch];
            }
            for (int j = 0; j < H; ++j) {
                const float ig = sigmoid_f(g[j]), fg = sigmoid_f(g[H + j]), cg = tanhf(g[2 * H + j]);
                const float og = sigmoid_f(g[3 * H + j]);
                const float next_cell = fg * cr[j] + ig * cg;
                const float ct = tanhf(next_cell);
                const float next_hidden = og * ct;
                cr[j] = next_cell;
                if (gate_out) {
                    gate_out[go + j] = ig; gate_out[go + H + j] = fg;
                    gate_out[go + 2 * H + j] = cg; gate_out[go + 3 * H + j] = og;
                }
                if (cell) cell[so + j] = next_cell;
                if (cell_tanh) cell_tanh[so + j] = ct;
                if (hidden) hidden[so + j] = next_hidden;
                out[so + j] = next_hidden;
            }
            /* the new hidden row replaces the old one only after every channel of this row used it */
            for (int j = 0; j < H; ++j) hr[j] = out[so + j];
            if (g != gates) free(g);
        }
    }
    return 0;
}

static float keep(const uint8_t *mask, size_t i) { return mask == NULL || mask[i] == 0 ? 1.0f : 0.0f; }

int orc_lstm_backward_float_masked(int T, int B, int I, int H, const float *w_ih, const float *w_hh, const float *x,
                                   const float *h0, const float *c0, const float *gate_out, const float *cell,
                                   const float *cell_tanh, const float *hidden, const float *g_out, const float *g_hn,
                                   const float *g_cn, const rxmet_lstm_backward_masks *m, float *dx, float *dw_ih,
                                   float *dw_hh, float *db_ih, float *db_hh, float *dh0, float *dc0) {
    /* operators/quant-lstm/src/lstm/backward_float_cpu.cc:48-151; masks as in
     * operators/quant-lstm/src/lstm/backward_float_cuda.cu:50-104,306-324 */
    const int C = 4 * H;
    const size_t BH = (size_t)B * H, BC = (size_t)B * C;
    memset(dx, 0, sizeof(float) * T * B * I);
    memset(dw_ih, 0, sizeof(float) * C * I);
    memset(dw_hh, 0, sizeof(float) * C * H);
    memset(db_ih, 0, sizeof(float) * C);
    memset(db_hh, 0, sizeof(float) * C);
    float *gh = malloc(BH * sizeof(float)), *gc = malloc(BH * sizeof(float)), *gh_next = malloc(BH * sizeof(float));
    float *gi = malloc(BC * sizeof(float)), *gr = malloc(BC * sizeof(float));
    memcpy(gh, g_hn, BH * sizeof(float));
    memcpy(gc, g_cn, BH * sizeof(float));
    for (int t = T - 1; t >= 0; --t) {
        const size_t so = (size_t)t * BH, go = (size_t)t * BC;
        const float *c_prev = t == 0 ? c0 : cell + so - BH;
        const float *h_prev = t == 0 ? h0 : hidden + so - BH;
        for (int b = 0; b < B; ++b)
            for (int j = 0; j < H; ++j) {
                const size_t s = (size_t)b * H + j, gb = (size_t)b * C + j;
                const float ig = gate_out[go + gb], fg = gate_out[go + gb + H], cg = gate_out[go + gb + 2 * H];
                const float og = gate_out[go + gb + 3 * H], ct = cell_tanh[so + s];
                const float dh = (gh[s] + g_out[so + s]) * keep(m ? m->hidden_outputs : NULL, so + s);
                const float g_og = dh * ct;
                const float g_ct = dh * og * keep(m ? m->cell_tanh_outputs : NULL, so + s);
                const float dc = gc[s] + g_ct * (1.0f - ct * ct);
                const float mdc = dc * keep(m ? m->cell_states : NULL, so + s);
                const float g_fg = mdc * (c_prev ? c_prev[s] : 0.0f);
                const float g_ig = mdc * cg, g_cg = mdc * ig;
                const uint8_t *mo = m ? m->gate_outputs : NULL;
                const float o4[4] = {g_ig * keep(mo, go + gb), g_fg * keep(mo, go + gb + H),
                                     g_cg * keep(mo, go + gb + 2 * H), g_og * keep(mo, go + gb + 3 * H)};
                const float i4[4] = {o4[0] * ig * (1.0f - ig), o4[1] * fg * (1.0f - fg), o4[2] * (1.0f - cg * cg),
                                     o4[3] * og * (1.0f - og)};
                for (int g = 0; g < 4; ++g) {
                    const size_t gidx = gb + (size_t)g * H;
                    const float grad = i4[g] * keep(m ? m->gate_inputs : NULL, go + gidx);
                    gi[gidx] = grad * keep(m ? m->weight_ih_linear : NULL, go + gidx);
                    gr[gidx] = grad * keep(m ? m->weight_hh_linear : NULL, go + gidx);
                }
                gc[s] = mdc * fg;
            }
        memset(gh_next, 0, BH * sizeof(float));
        for (int b = 0; b < B; ++b) {
            const float *xr = x + ((size_t)t * B + b) * I;
            float *dxr = dx + ((size_t)t * B + b) * I;
            for (int ch = 0; ch < C; ++ch) {
                const float a = gi[(size_t)b * C + ch], r = gr[(size_t)b * C + ch];
                db_ih[ch] += a;
                db_hh[ch] += r;
                for (int k = 0; k < I; ++k) {
                    dxr[k] += a * w_ih[(size_t)ch * I + k];
                    dw_ih[(size_t)ch * I + k] += a * xr[k];
                }
                for (int k = 0; k < H; ++k) {
                    gh_next[(size_t)b * H + k] += r * w_hh[(size_t)ch * H + k];
                    dw_hh[(size_t)ch * H + k] += r * (h_prev ? h_prev[(size_t)b * H + k] : 0.0f);
                }
            }
        }
        float *tmp = gh; gh = gh_next; gh_next = tmp;
    }
    memcpy(dh0, gh, BH * sizeof(float));
    memcpy(dc0, gc, BH * sizeof(float));
    if (m) {
        struct { float *g; const uint8_t *k; size_t n; } post[7] = {
            {dx, m->input, (size_t)T * B * I}, {dw_ih, m->weight_ih, (size_t)C * I}, {dw_hh, m->weight_hh, (size_t)C * H},
            {db_ih, m->bias_ih, (size_t)C},    {db_hh, m->bias_hh, (size_t)C},        {dh0, m->initial_hidden, BH},
            {dc0, m->initial_cell, BH}};
        for (int q = 0; q < 7; ++q)
            if (post[q].k)
                for (size_t i = 0; i < post[q].n; ++i)
                    if (post[q].k[i]) post[q].g[i] = 0.0f;
    }
    free(gh); free(gc); free(gh_next); free(gi); free(gr);
    return 0;
}

int orc_lstm_backward_float(int T, int B, int I, int H, const float *w_ih, const float *w_hh, const float *x,
                            const float *h0, const float *c0, const float *gate_out, const float *cell,
                            const float *cell_tanh, const float *hidden, const float *g_out, const float *g_hn,
                            const float *g_cn, float *dx, float *dw_ih, float *dw_hh, float *db_ih, float *db_hh,
                            float *dh0, float *dc0) {
    return orc_lstm_backward_float_masked(T, B, I, H, w_ih, w_hh, x, h0, c0, gate_out, cell, cell_tanh, hidden, g_out,
                                          g_hn, g_cn, NULL, dx, dw_ih, dw_hh, db_ih, db_hh, dh0, dc0);
}

/* ---- min/max calibration ------------------------------------------------------ */

static void observe(float *lo, float *hi, const float *v, size_t n) {
    for (size_t i = 0; i < n; ++i) {
        if (v[i] < *lo) *lo = v[i];
        if (v[i] > *hi) *hi = v[i];
    }
}

static void observe_gate(float *lo, float *hi, const float *v, size_t rows, int H, int gate) {
    for (size_t r = 0; r < rows; ++r) observe(lo, hi, v + r * 4 * H + (size_t)gate * H, (size_t)H);
}

int orc_lstm_calibrate_minmax(const rxmet_lstm_quant_config *config, int batches, int T, int B, int I, int H,
                              const float *w_ih, const float *w_hh, const float *b_ih, const float *b_hh,
                              const float *x_all, const float *h0, const float *c0, rxmet_lstm_ranges *r,
                              float *w_ih_scale, float *w_hh_scale, float *b_ih_scale, float *b_hh_scale,
                              rxmet_lstm_quant_params *params) {
    /* operators/quant-lstm/src/lstm/calibration.cc:128-232 */
    const int C = 4 * H;
    const size_t rows = (size_t)T * B, BH = (size_t)B * H;
    for (int op = 0; op < RXMET_LSTM_NUM_OPS; ++op) { r->minimum[op] = INFINITY; r->maximum[op] = -INFINITY; }
    for (int k = 0; k < 3; ++k) { r->contribution_min[k] = INFINITY; r->contribution_max[k] = -INFINITY; }
    for (int s = 0; s < 4; ++s)
        for (int ch = 0; ch < C; ++ch) { r->channel_min[s][ch] = INFINITY; r->channel_max[s][ch] = -INFINITY; }
    float *out = malloc(rows * H * sizeof(float)), *hn = malloc(BH * sizeof(float)), *cn = malloc(BH * sizeof(float));
    float *ih = malloc(rows * C * sizeof(float)), *hh = malloc(rows * C * sizeof(float));
    float *gi = malloc(rows * C * sizeof(float)), *go = malloc(rows * C * sizeof(float));
    float *cs = malloc(rows * H * sizeof(float)), *ct = malloc(rows * H * sizeof(float));
    float *hs = malloc(rows * H * sizeof(float));
    const float zero = 0.0f;
    for (int n = 0; n < batches; ++n) {
        const float *x = x_all + (size_t)n * rows * I;
        orc_lstm_forward_float(T, B, I, H, w_ih, w_hh, b_ih, b_hh, x, h0, c0, out, hn, cn, ih, hh, gi, go, cs, ct, hs);
#define OBS(op, v, n) observe(&r->minimum[op], &r->maximum[op], v, n)
        OBS(RXMET_LSTM_INPUT, x, rows * I);
        if (h0) { OBS(RXMET_LSTM_OUTPUT, h0, BH); OBS(RXMET_LSTM_CELL_STATE, c0, BH); }
        else { OBS(RXMET_LSTM_OUTPUT, &zero, 1); OBS(RXMET_LSTM_CELL_STATE, &zero, 1); }
        OBS(RXMET_LSTM_OUTPUT, hs, rows * H);
        OBS(RXMET_LSTM_CELL_STATE, cs, rows * H);
        OBS(RXMET_LSTM_WEIGHT_IH_LINEAR, ih, rows * C);
        OBS(RXMET_LSTM_WEIGHT_HH_LINEAR, hh, rows * C);
        OBS(RXMET_LSTM_CELL_TANH_OUTPUT, ct, rows * H);
#undef OBS
        for (int g = 0; g < 4; ++g) {
            observe_gate(&r->minimum[RXMET_LSTM_INPUT_GATE_INPUT + g], &r->maximum[RXMET_LSTM_INPUT_GATE_INPUT + g], gi, rows, H, g);
            observe_gate(&r->minimum[RXMET_LSTM_INPUT_GATE_OUTPUT + g], &r->maximum[RXMET_LSTM_INPUT_GATE_OUTPUT + g], go, rows, H, g);
        }
        for (int ch = 0; ch < C; ++ch) {
            observe(&r->channel_min[0][ch], &r->channel_max[0][ch], w_ih + (size_t)ch * I, (size_t)I);
            observe(&r->channel_min[1][ch], &r->channel_max[1][ch], w_hh + (size_t)ch * H, (size_t)H);
            if (b_ih) {
                observe(&r->channel_min[2][ch], &r->channel_max[2][ch], b_ih + ch, 1);
                observe(&r->channel_min[3][ch], &r->channel_max[3][ch], b_hh + ch, 1);
            }
        }
        for (int t = 0; t < T; ++t)
            for (int b = 0; b < B; ++b)
                for (int j = 0; j < H; ++j) {
                    const size_t s = ((size_t)t * B + b) * H + j, gb = ((size_t)t * B + b) * C + j;
                    const float c_prev = t == 0 ? (c0 ? c0[(size_t)b * H + j] : 0.0f) : cs[s - BH];
                    const float v3[3] = {go[gb + H] * c_prev, go[gb] * go[gb + 2 * H], go[gb + 3 * H] * ct[s]};
                    for (int k = 0; k < 3; ++k) observe(&r->contribution_min[k], &r->contribution_max[k], &v3[k], 1);
                }
    }
    free(out); free(hn); free(cn); free(ih); free(hh); free(gi); free(go); free(cs); free(ct); free(hs);
    /* per-channel observations of coarser granularities are folded inside params_from_ranges */
    return orc_lstm_params_from_ranges(config, r, I, H, b_ih != NULL, w_ih_scale, w_hh_scale, b_ih_scale, b_hh_scale,
                                       params);
}
