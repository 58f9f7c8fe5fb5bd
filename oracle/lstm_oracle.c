/*
 * TEST INFRASTRUCTURE - CPU restatement of the QuantLSTM forward / backward
 * arithmetic of rx-met (plain C, OpenMP over rows).  Used only by tests, the
 * smoke check and the CPU legs of the benchmark as the checker.
 *
 * Pinned against the reference's own CPU sources compiled into
 * oracle/_ref/liblstm_ref.so and against the golden JSON cases of
 * operators/quant-lstm/tests/golden/spec (tests/test_lstm_cpu.py).  The clamp
 * masks have no CPU counterpart in the reference; they restate its CUDA kernel
 * (operators/quant-lstm/src/lstm/forward_quantized_fp_cuda.cu:514-577,750-865).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "lstm_oracle.h"

/* ---- scalar building blocks ------------------------------------------------ */

static float clamp_carrier(double v, int32_t lo, int32_t hi, uint8_t *clamped) {
    /* operators/quant-lstm/include/quantization/float_carrier_ops.h:26-34 (grids of at most 24 bits) */
    if (clamped) *clamped = (v < (double)lo) || (v > (double)hi);
    if (v <= (double)lo) return (float)lo;
    if (v >= (double)hi) return (float)hi;
    return (float)v;
}

static float center(float v, int32_t zp) { return (float)((double)v - zp); }

static float apply_rescale(float v, rxmet_lstm_rescale r) {
    /* float_carrier_ops.h:77-86 */
    return r.is_m_shift ? rintf(ldexpf(v * (float)r.multiplier, -r.shift)) : rintf(ldexpf(v, -r.shift));
}

static float quantize_one(float v, float scale, int32_t zp, int32_t lo, int32_t hi, uint8_t *clamped) {
    /* float_carrier_ops.h:49-59 */
    return clamp_carrier(rint((double)v / scale) + (double)zp, lo, hi, clamped);
}

static float sigmoid_f(float v) {
    /* operators/quant-lstm/src/lstm/cuda/quantized_fp_math.cuh:15-22 */
    if (v >= 0.0f) {
        const float e = expf(-v);
        return 1.0f / (1.0f + e);
    }
    const float e = expf(v);
    return e / (1.0f + e);
}

static float real_activation(float q, float in_scale, int32_t in_zp, float out_scale, int32_t out_zp, int32_t lo,
                             int32_t hi, int is_tanh, uint8_t *clamped) {
    /* quantized_fp_math.cuh:24-62 */
    const float real_input = (float)(((double)q - (double)in_zp) * (double)in_scale);
    const float activated = is_tanh ? tanhf(real_input) : sigmoid_f(real_input);
    const double translated = rint((double)activated / (double)out_scale) + (double)out_zp;
    return clamp_carrier(translated, lo, hi, clamped);
}

static float scale_cell_product(float product, rxmet_lstm_cell_scale s) {
    /* operators/quant-lstm/include/lstm/quantized_cell_fp.h:72-80 */
    if (s.uses_fp_scale) return (float)ldexp((double)product * s.fp_mantissa, s.fp_exponent);
    const float ratio = ldexpf((float)s.multiplier, -31);
    return product * ratio;
}

/* ---- execution context ------------------------------------------------------- */

typedef struct {
    const rxmet_lstm_quant_params *p;
    rxmet_lstm_execution e;
    int32_t lo[RXMET_LSTM_NUM_OPS], hi[RXMET_LSTM_NUM_OPS];
    int exact_sums; /* 1: the two linear stages add up exactly in integers and round to float once */
} ctx_t;

static int ctx_init(ctx_t *c, const rxmet_lstm_quant_params *p) {
    const size_t ch = 4 * (size_t)p->hidden_size;
    memset(c, 0, sizeof(*c));
    c->p = p;
    c->e.ih_accumulator_to_output = malloc(ch * sizeof(rxmet_lstm_rescale));
    c->e.hh_accumulator_to_output = malloc(ch * sizeof(rxmet_lstm_rescale));
    c->e.ih_bias_to_accumulator = malloc(ch * sizeof(rxmet_lstm_rescale));
    c->e.hh_bias_to_accumulator = malloc(ch * sizeof(rxmet_lstm_rescale));
    for (int op = 0; op < RXMET_LSTM_NUM_OPS; ++op) orc_lstm_type_range(&p->config, op, &c->lo[op], &c->hi[op]);
    return orc_lstm_derive_execution(p, 0, &c->e);
}

static void ctx_free(ctx_t *c) {
    free(c->e.ih_accumulator_to_output);
    free(c->e.hh_accumulator_to_output);
    free(c->e.ih_bias_to_accumulator);
    free(c->e.hh_bias_to_accumulator);
}

/* ---- stages (each follows operators/quant-lstm/src/lstm/forward_quantized_fp_cpu.cc) ------------ */

static void stage_linear(const ctx_t *c, int hh, long rows, const float *q_in, const float *q_w, const float *q_b,
                         float *lin, uint8_t *mask) {
    /* forward_quantized_fp_cpu.cc:17-45 */
    const rxmet_lstm_quant_params *p = c->p;
    const int K = hh ? p->hidden_size : p->input_size, C = 4 * p->hidden_size;
    const int in_op = hh ? RXMET_LSTM_OUTPUT : RXMET_LSTM_INPUT;
    const int out_op = hh ? RXMET_LSTM_WEIGHT_HH_LINEAR : RXMET_LSTM_WEIGHT_IH_LINEAR;
    const rxmet_lstm_rescale *b2a = hh ? c->e.hh_bias_to_accumulator : c->e.ih_bias_to_accumulator;
    const rxmet_lstm_rescale *a2o = hh ? c->e.hh_accumulator_to_output : c->e.ih_accumulator_to_output;
    const int32_t zin = p->zero_point[in_op], zout = p->zero_point[out_op];
#pragma omp parallel for schedule(static)
    for (long r = 0; r < rows; ++r) {
        const float *v = q_in + r * K;
        for (int ch = 0; ch < C; ++ch) {
            const float *w = q_w + (size_t)ch * K;
            float acc = 0.0f;
            if (c->exact_sums) {
                /* The same sum without the intermediate float roundings: what the reference's float
                 * accumulation yields whenever every partial sum stays below 2^24 (its
                 * exact_integer_range class), and the correctly rounded sum beyond that.  This is the
                 * arithmetic of the CUDA library's linear stages. */
                int64_t total = 0;
                for (int k = 0; k < K; ++k) total += (int64_t)w[k] * ((int64_t)v[k] - zin);
                if (q_b) total += (int64_t)apply_rescale(center(q_b[ch], 0), b2a[ch]);
                acc = (float)total;
            } else {
                for (int k = 0; k < K; ++k) acc += center(w[k], 0) * center(v[k], zin);
                if (q_b) acc += apply_rescale(center(q_b[ch], 0), b2a[ch]);
            }
            uint8_t m;
            lin[r * C + ch] = clamp_carrier((double)apply_rescale(acc, a2o[ch]) + zout, c->lo[out_op], c->hi[out_op], &m);
            if (mask) mask[r * C + ch] = m;
        }
    }
}

static void stage_gate_inputs(const ctx_t *c, long rows, const float *ih_lin, const float *hh_lin, float *gate_in,
                              uint8_t *mask) {
    /* forward_quantized_fp_cpu.cc:117-131 */
    const rxmet_lstm_quant_params *p = c->p;
    const int H = p->hidden_size, C = 4 * H;
    const int32_t zi = p->zero_point[RXMET_LSTM_WEIGHT_IH_LINEAR], zh = p->zero_point[RXMET_LSTM_WEIGHT_HH_LINEAR];
#pragma omp parallel for schedule(static)
    for (long r = 0; r < rows; ++r)
        for (int ch = 0; ch < C; ++ch) {
            const int g = ch / H, op = RXMET_LSTM_INPUT_GATE_INPUT + g;
            const float lhs = apply_rescale(center(ih_lin[r * C + ch], zi), c->e.ih_to_gate[g]);
            const float rhs = apply_rescale(center(hh_lin[r * C + ch], zh), c->e.hh_to_gate[g]);
            uint8_t m;
            gate_in[r * C + ch] = clamp_carrier((double)(lhs + rhs) + p->zero_point[op], c->lo[op], c->hi[op], &m);
            if (mask) mask[r * C + ch] = m;
        }
}

static void stage_gate_outputs(const ctx_t *c, long rows, const float *gate_in, float *gate_out, uint8_t *mask) {
    /* forward_quantized_fp_cpu.cc:132-138 */
    const rxmet_lstm_quant_params *p = c->p;
    const int H = p->hidden_size, C = 4 * H;
#pragma omp parallel for schedule(static)
    for (long r = 0; r < rows; ++r)
        for (int ch = 0; ch < C; ++ch) {
            const int g = ch / H, in_op = RXMET_LSTM_INPUT_GATE_INPUT + g, out_op = RXMET_LSTM_INPUT_GATE_OUTPUT + g;
            uint8_t m;
            gate_out[r * C + ch] =
                real_activation(gate_in[r * C + ch], p->scale[in_op], p->zero_point[in_op], p->scale[out_op],
                                p->zero_point[out_op], c->lo[out_op], c->hi[out_op], g == 2, &m);
            if (mask) mask[r * C + ch] = m;
        }
}

static void stage_cell(const ctx_t *c, long rows, const float *gate_out, const float *c_prev, float *c_next,
                       uint8_t *mask) {
    /* operators/quant-lstm/include/lstm/quantized_cell_fp.h:81-110 */
    const rxmet_lstm_quant_params *p = c->p;
    const int H = p->hidden_size, C = 4 * H;
    const int32_t zf = p->zero_point[RXMET_LSTM_FORGET_GATE_OUTPUT], zi = p->zero_point[RXMET_LSTM_INPUT_GATE_OUTPUT];
    const int32_t zg = p->zero_point[RXMET_LSTM_CELL_GATE_OUTPUT], zc = p->zero_point[RXMET_LSTM_CELL_STATE];
#pragma omp parallel for schedule(static)
    for (long r = 0; r < rows; ++r)
        for (int j = 0; j < H; ++j) {
            const float *g = gate_out + r * C + j;
            const float pf = center(g[H], zf) * center(c_prev[r * H + j], zc);
            const float pi = center(g[0], zi) * center(g[2 * H], zg);
            const float sf = scale_cell_product(pf, c->e.forget_scale);
            const float si = scale_cell_product(pi, c->e.input_scale);
            const float sum = sf + si;
            uint8_t m;
            c_next[r * H + j] = clamp_carrier((double)rintf(sum) + zc, c->lo[RXMET_LSTM_CELL_STATE],
                                              c->hi[RXMET_LSTM_CELL_STATE], &m);
            if (mask) mask[r * H + j] = m;
        }
}

static void stage_cell_tanh(const ctx_t *c, long n, const float *cell, float *cell_tanh, uint8_t *mask) {
    /* forward_quantized_fp_cpu.cc:165-169 */
    const rxmet_lstm_quant_params *p = c->p;
    const int a = RXMET_LSTM_CELL_STATE, b = RXMET_LSTM_CELL_TANH_OUTPUT;
#pragma omp parallel for schedule(static)
    for (long i = 0; i < n; ++i) {
        uint8_t m;
        cell_tanh[i] = real_activation(cell[i], p->scale[a], p->zero_point[a], p->scale[b], p->zero_point[b], c->lo[b],
                                       c->hi[b], 1, &m);
        if (mask) mask[i] = m;
    }
}

static void stage_hidden(const ctx_t *c, long rows, const float *gate_out, const float *cell_tanh, float *h,
                         uint8_t *mask) {
    /* quantized_cell_fp.h:111-124 */
    const rxmet_lstm_quant_params *p = c->p;
    const int H = p->hidden_size, C = 4 * H;
    const int32_t zo = p->zero_point[RXMET_LSTM_OUTPUT_GATE_OUTPUT], zt = p->zero_point[RXMET_LSTM_CELL_TANH_OUTPUT];
#pragma omp parallel for schedule(static)
    for (long r = 0; r < rows; ++r)
        for (int j = 0; j < H; ++j) {
            const float raw = center(gate_out[r * C + 3 * H + j], zo) * center(cell_tanh[r * H + j], zt);
            const float centered = apply_rescale(raw, c->e.product_to_output);
            uint8_t m;
            h[r * H + j] = clamp_carrier((double)centered + p->zero_point[RXMET_LSTM_OUTPUT], c->lo[RXMET_LSTM_OUTPUT],
                                         c->hi[RXMET_LSTM_OUTPUT], &m);
            if (mask) mask[r * H + j] = m;
        }
}

/* ---- exported: element-wise pieces ------------------------------------------ */

int orc_lstm_quantize(const float *src, long long n, long long row_width, const float *scales, int zero_point,
                      int bitwidth, int is_unsigned, int is_symmetric, float *dst) {
    (void)is_symmetric;
    rxmet_lstm_quant_config c;
    memset(&c, 0, sizeof(c));
    c.bitwidth[0] = bitwidth;
    c.is_unsigned[0] = (uint8_t)is_unsigned;
    int32_t lo, hi;
    orc_lstm_type_range(&c, 0, &lo, &hi);
    for (long long i = 0; i < n; ++i)
        dst[i] = quantize_one(src[i], scales[row_width > 0 ? i / row_width : 0], zero_point, lo, hi, NULL);
    return 0;
}

int orc_lstm_quantize_masked(const float *src, long long n, long long row_width, const float *scales, int zero_point,
                             int bitwidth, int is_unsigned, float *dst, uint8_t *mask) {
    rxmet_lstm_quant_config c;
    memset(&c, 0, sizeof(c));
    c.bitwidth[0] = bitwidth;
    c.is_unsigned[0] = (uint8_t)is_unsigned;
    int32_t lo, hi;
    orc_lstm_type_range(&c, 0, &lo, &hi);
    for (long long i = 0; i < n; ++i)
        dst[i] = quantize_one(src[i], scales[row_width > 0 ? i / row_width : 0], zero_point, lo, hi, mask ? mask + i : NULL);
    return 0;
}

int orc_lstm_dequantize(const float *src, long long n, long long row_width, const float *scales, int zero_point,
                        float *dst) {
    /* float_carrier_ops.h:61-70 */
    for (long long i = 0; i < n; ++i)
        dst[i] = (float)(((double)src[i] - zero_point) * (double)scales[row_width > 0 ? i / row_width : 0]);
    return 0;
}

int orc_lstm_real_activation(const float *src, long long n, float in_scale, int in_zp, int in_bits, int in_unsigned,
                             float out_scale, int out_zp, int out_bits, int out_unsigned, int is_tanh, float *dst) {
    (void)in_bits;
    (void)in_unsigned;
    rxmet_lstm_quant_config c;
    memset(&c, 0, sizeof(c));
    c.bitwidth[0] = out_bits;
    c.is_unsigned[0] = (uint8_t)out_unsigned;
    int32_t lo, hi;
    orc_lstm_type_range(&c, 0, &lo, &hi);
    for (long long i = 0; i < n; ++i)
        dst[i] = real_activation(src[i], in_scale, in_zp, out_scale, out_zp, lo, hi, is_tanh, NULL);
    return 0;
}

/* One stage on caller-supplied q-carrier inputs (used to check each stage of a device
 * trace on exactly the inputs the device saw).  stage: 0 ih linear (a = x, b = weights,
 * c = bias or NULL), 1 hh linear (a = h_prev), 2 gate inputs (a = ih_lin, b = hh_lin),
 * 3 gate outputs (a = gate_in), 4 cell (a = gate_out, b = c_prev), 5 cell tanh (a = cell,
 * rows = element count), 6 hidden (a = gate_out, b = cell_tanh). */
int orc_lstm_stage(const rxmet_lstm_quant_params *p, int stage, long long rows, const float *a, const float *b,
                   const float *c3, float *out, uint8_t *mask) {
    ctx_t c;
    if (ctx_init(&c, p) != 0) return -1;
    switch (stage) {
        case 0: stage_linear(&c, 0, rows, a, b, c3, out, mask); break;
        case 1: stage_linear(&c, 1, rows, a, b, c3, out, mask); break;
        case 2: stage_gate_inputs(&c, rows, a, b, out, mask); break;
        case 3: stage_gate_outputs(&c, rows, a, out, mask); break;
        case 4: stage_cell(&c, rows, a, b, out, mask); break;
        case 5: stage_cell_tanh(&c, rows, a, out, mask); break;
        case 6: stage_hidden(&c, rows, a, b, out, mask); break;
        default: ctx_free(&c); return -1;
    }
    ctx_free(&c);
    return 0;
}

/* ---- exported: whole q-carrier forward ---------------------------------------- */

static int forward_quantized_masked(const rxmet_lstm_quant_params *p, int exact_sums, int T, int B, const float *q_w_ih,
                                    const float *q_w_hh, const float *q_b_ih, const float *q_b_hh, const float *q_x,
                                    const float *q_h0, const float *q_c0, float *out, float *hn, float *cn,
                                    const rxmet_lstm_trace *tr) {
    /* forward_quantized_fp_cpu.cc:70-198 */
    ctx_t c;
    if (ctx_init(&c, p) != 0) return -1;
    c.exact_sums = exact_sums;
    const int I = p->input_size, H = p->hidden_size, C = 4 * H;
    const size_t BH = (size_t)B * H, BC = (size_t)B * C;
    float *h = malloc(BH * sizeof(float)), *cell = malloc(BH * sizeof(float));
    float *ih = malloc(BC * sizeof(float)), *hh = malloc(BC * sizeof(float));
    float *gi = malloc(BC * sizeof(float)), *go = malloc(BC * sizeof(float));
    float *ct = malloc(BH * sizeof(float)), *cnew = malloc(BH * sizeof(float)), *hnew = malloc(BH * sizeof(float));
    const float hz = quantize_one(0.0f, p->scale[RXMET_LSTM_OUTPUT], p->zero_point[RXMET_LSTM_OUTPUT],
                                  c.lo[RXMET_LSTM_OUTPUT], c.hi[RXMET_LSTM_OUTPUT], NULL);
    const float cz = quantize_one(0.0f, p->scale[RXMET_LSTM_CELL_STATE], p->zero_point[RXMET_LSTM_CELL_STATE],
                                  c.lo[RXMET_LSTM_CELL_STATE], c.hi[RXMET_LSTM_CELL_STATE], NULL);
    for (size_t i = 0; i < BH; ++i) {
        h[i] = q_h0 ? q_h0[i] : hz;
        cell[i] = q_c0 ? q_c0[i] : cz;
    }
#define MASK(field) (tr && tr->field ? tr->field + off : NULL)
#define COPY(field, src, count) \
    if (tr && tr->field) memcpy(tr->field + off, src, (count) * sizeof(float))
    for (int t = 0; t < T; ++t) {
        size_t off = (size_t)t * BC;
        stage_linear(&c, 0, B, q_x + (size_t)t * B * I, q_w_ih, q_b_ih, ih, MASK(weight_ih_linear_clamped));
        stage_linear(&c, 1, B, h, q_w_hh, q_b_hh, hh, MASK(weight_hh_linear_clamped));
        stage_gate_inputs(&c, B, ih, hh, gi, MASK(gate_inputs_clamped));
        stage_gate_outputs(&c, B, gi, go, MASK(gate_outputs_clamped));
        COPY(weight_ih_linear, ih, BC);
        COPY(weight_hh_linear, hh, BC);
        COPY(gate_inputs, gi, BC);
        COPY(gate_outputs, go, BC);
        off = (size_t)t * BH;
        stage_cell(&c, B, go, cell, cnew, MASK(cell_states_clamped));
        stage_cell_tanh(&c, (long)BH, cnew, ct, MASK(cell_tanh_outputs_clamped));
        stage_hidden(&c, B, go, ct, hnew, MASK(hidden_outputs_clamped));
        memcpy(cell, cnew, BH * sizeof(float));
        memcpy(h, hnew, BH * sizeof(float));
        COPY(cell_states, cell, BH);
        COPY(cell_tanh_outputs, ct, BH);
        COPY(hidden_outputs, h, BH);
        if (out) memcpy(out + off, h, BH * sizeof(float));
    }
#undef MASK
#undef COPY
    memcpy(hn, h, BH * sizeof(float));
    memcpy(cn, cell, BH * sizeof(float));
    free(h); free(cell); free(ih); free(hh); free(gi); free(go); free(ct); free(cnew); free(hnew);
    ctx_free(&c);
    return 0;
}

int orc_lstm_forward_quantized_masked(const rxmet_lstm_quant_params *p, int T, int B, const float *q_w_ih,
                                      const float *q_w_hh, const float *q_b_ih, const float *q_b_hh, const float *q_x,
                                      const float *q_h0, const float *q_c0, float *out, float *hn, float *cn,
                                      const rxmet_lstm_trace *tr) {
    return forward_quantized_masked(p, 0, T, B, q_w_ih, q_w_hh, q_b_ih, q_b_hh, q_x, q_h0, q_c0, out, hn, cn, tr);
}

/* The q-carrier forward with exactly accumulated linear stages (see stage_linear). */
int orc_lstm_forward_quantized_exact_sums(const rxmet_lstm_quant_params *p, int T, int B, const float *q_w_ih,
                                          const float *q_w_hh, const float *q_b_ih, const float *q_b_hh,
                                          const float *q_x, const float *q_h0, const float *q_c0, float *out,
                                          float *hn, float *cn, const rxmet_lstm_trace *tr) {
    return forward_quantized_masked(p, 1, T, B, q_w_ih, q_w_hh, q_b_ih, q_b_hh, q_x, q_h0, q_c0, out, hn, cn, tr);
}

/* Same argument list as the reference shim's entry point. */
int orc_lstm_forward_quantized(const rxmet_lstm_quant_params *p, int exact, int T, int B, const float *q_w_ih,
                               const float *q_w_hh, const float *q_b_ih, const float *q_b_hh, const float *q_x,
                               const float *q_h0, const float *q_c0, float *out, float *hn, float *cn, float *ih_lin,
                               float *hh_lin, float *gate_in, float *gate_out, float *cell, float *cell_tanh,
                               float *hidden) {
    (void)exact;
    rxmet_lstm_trace tr;
    memset(&tr, 0, sizeof(tr));
    tr.weight_ih_linear = ih_lin;
    tr.weight_hh_linear = hh_lin;
    tr.gate_inputs = gate_in;
    tr.gate_outputs = gate_out;
    tr.cell_states = cell;
    tr.cell_tanh_outputs = cell_tanh;
    tr.hidden_outputs = hidden;
    return orc_lstm_forward_quantized_masked(p, T, B, q_w_ih, q_w_hh, q_b_ih, q_b_hh, q_x, q_h0, q_c0, out, hn, cn, &tr);
}
