/*
 * TEST INFRASTRUCTURE - not part of the shipped library (see gru_oracle.h).
 *
 * Scalar primitives, encodings from ranges, rescale multipliers and the
 * piecewise-linear activation tables of the reference's QuantGRU, restated in
 * plain C.  Citations are <file under operators/quant-gru/>:<line>.
 */
#include <float.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "gru_oracle.h"

/* ---- primitives -------------------------------------------------------- */

/* include/quantize_ops_helper.h:201-224 : shift right with round-half-even on
 * the magnitude; n <= 0 shifts left. */
int64_t orc_rshift_round(int64_t x, int n) {
    if (n <= 0) return x << (-n);
    const int neg = x < 0;
    const int64_t a = neg ? -x : x;
    const int64_t half = (int64_t)1 << (n - 1);
    const int64_t mask = ((int64_t)1 << n) - 1;
    const int64_t q = a >> n;
    const int64_t r = a & mask;
    int64_t res;
    if (r > half) res = q + 1;
    else if (r < half) res = q;
    else res = (q & 1) ? q + 1 : q;
    return neg ? -res : res;
}

/* include/quantize_ops_helper.h:242-248 */
static int64_t apply_rescale(int64_t x, orc_rescale r) {
    return orc_rshift_round(x * r.multiplier, r.shift);
}

/* include/quantize_bitwidth_config.h:16-24 */
int32_t orc_qmin(orc_bitwidth b) {
    if (b.bits >= 32) return INT32_MIN;
    return b.is_unsigned ? 0 : -(1 << (b.bits - 1));
}
int32_t orc_qmax(orc_bitwidth b) {
    if (b.bits >= 32) return INT32_MAX;
    return b.is_unsigned ? (int32_t)((1u << b.bits) - 1u) : (1 << (b.bits - 1)) - 1;
}

/* include/quantize_ops_helper.h:133-140,280-292,357-365 : divide in float,
 * round half even, add the zero point afterwards (in double), saturate before
 * the integer cast.  *keep = 1 when the value was not clamped. */
int32_t orc_quantize(float v, float scale, int32_t zp, orc_bitwidth b, uint8_t *keep) {
    const double code = (double)rintf(v / scale) + (double)zp;
    const int32_t lo = orc_qmin(b), hi = orc_qmax(b);
    if (keep) *keep = (code < lo || code > hi) ? 0 : 1;
    return code < lo ? lo : (code > hi ? hi : (int32_t)code);
}

/* include/scale_encoding.h:87-106 : scale ~= M * 2^-shift, M in [32768,65535]. */
int orc_encode_mshift(float scale, int32_t *multiplier, int32_t *shift) {
    if (!(scale > 0.0f)) return -1;
    int e = 0;
    const double mant = frexp((double)scale, &e);
    uint32_t m = (uint32_t)llround(mant * 65536.0);
    if (m == 65536u) { m = 32768u; e += 1; }
    if (m < 32768u) m = 32768u;
    const int s = 16 - e;
    if (s < -128 || s > 127) return -1;
    *multiplier = (int32_t)m;
    *shift = s;
    return 0;
}

/* include/scale_encoding.h:114-117 */
static int pot2_shift(float scale) {
    if (!(scale > 0.0f)) return 0;
    return (int)(int8_t)lround(-log2((double)scale));
}

/* include/scale_encoding.h:122-125 + quantize_ops_helper.h:99-105 : the scale
 * the quantize/dequantize boundary actually uses. */
static int effective_scale(float scale, int use_pot2, float *out) {
    if (use_pot2) {
        *out = 1.0f * ldexpf(1.0f, -pot2_shift(scale));
        return 0;
    }
    int32_t m, s;
    if (orc_encode_mshift(scale, &m, &s)) return -1;
    *out = (float)m * ldexpf(1.0f, -s);
    return 0;
}

int orc_gru_decode_effective_scale(float scale, int use_pot2, float *out) {
    if (!(scale > 0.0f)) return -1;
    return effective_scale(scale, use_pot2, out);
}

/* include/scale_encoding.h:138-192 : rescale between grids.  ratio_mode 0:
 * src/dst, 1: (a*b)/dst, 2: src/(a*b); all ratios are formed in float. */
static int make_rescale(int use_pot2, int mode, float s0, float s1, float s2, orc_rescale *out) {
    if (use_pot2) {
        int sh;
        if (mode == 0) sh = pot2_shift(s0) - pot2_shift(s1);
        else if (mode == 1) sh = pot2_shift(s0) + pot2_shift(s1) - pot2_shift(s2);
        else sh = pot2_shift(s0) - (pot2_shift(s1) + pot2_shift(s2));
        out->multiplier = 1;
        out->shift = (int)(int8_t)sh;
        return 0;
    }
    float ratio;
    if (mode == 0) ratio = s0 / s1;
    else if (mode == 1) ratio = (s0 * s1) / s2;
    else ratio = s0 / (s1 * s2);
    int32_t m, s;
    if (orc_encode_mshift(ratio, &m, &s)) return -1;
    out->multiplier = m;
    out->shift = s;
    return 0;
}

/* ---- encodings from ranges -------------------------------------------- */

/* include/histogram_collector.h:34-38 */
static float minimum_scale(int64_t num_steps) {
    const float eps = 1.19209290e-07f;
    const float r = 0.01f / (float)num_steps;
    return eps < r ? eps : r;
}

typedef struct { float scale, min, max; } cont_scale;

/* include/pot_sqnr_calibrator.h:372-439 */
static int continuous_from_range(float mn, float mx, orc_bitwidth b, int symmetric, cont_scale *out) {
    const int32_t qmin = orc_qmin(b), qmax = orc_qmax(b);
    const int64_t steps = (int64_t)qmax - (int64_t)qmin;
    if (steps <= 0) return -1;
    const float ms = minimum_scale(steps);
    const float lo0 = (0.0f < mn) ? 0.0f : mn; /* std::min(mn, 0.0f) */
    const float hi0 = (mx < 0.0f) ? 0.0f : mx; /* std::max(mx, 0.0f) */
    const float diff = (hi0 - lo0) / (float)steps;
    const float adj = (diff < ms) ? ms : 0.0f;
    float umin = lo0, umax = hi0;
    if (symmetric) {
        if (b.is_unsigned) {
            umax = hi0 + (float)steps * adj;
            umin = 0.0f;
        } else {
            umax = hi0 + floorf((float)steps / 2.0f) * adj;
            umin = lo0 - ceilf((float)steps / 2.0f) * adj;
        }
    } else {
        umax = hi0 + (float)steps * adj;
    }
    float s = ms, amin = umin, amax = umax;
    if (symmetric) {
        if (b.is_unsigned) {
            const float dmax = umax > ms ? umax : ms;
            const float c = dmax / (float)qmax;
            s = c > ms ? c : ms;
            amin = 0.0f;
            amax = s * (float)qmax;
        } else {
            const int64_t pos = steps / 2, neg = (steps + 1) / 2;
            const int add = (steps == 3) ? 1 : 0;
            const float dmax = (pos + add > 0) ? umax / (float)(pos + add) : 0.0f;
            const float dmin = (neg > 0) ? -umin / (float)neg : 0.0f;
            const float d = dmax > dmin ? dmax : dmin;
            s = d > ms ? d : ms;
            amin = -(float)neg * s;
            amax = (float)pos * s;
        }
    } else {
        float range = umax - umin;
        const float floor_range = ms * (float)steps;
        if (!(range > floor_range)) range = floor_range; /* std::max(range, floor) */
        const float c = range / (float)steps;
        s = c > ms ? c : ms;
        amin = umin;
        amax = umin + s * (float)steps;
    }
    out->scale = s;
    out->min = amin;
    out->max = amax;
    return 0;
}

/* include/pot_scale_encode.h:63-103 */
static int near_power_of_two(float v, float tol) {
    if (!(v > 0.0f)) return 0;
    const float l = log2f(v);
    const float nearest = powf(2.0f, roundf(l));
    return fabsf(v - nearest) / nearest < tol;
}
static int scale_to_pot(float scale, int method, float rmin, float rmax, float tol, float *po2, int *n_out) {
    if (!(scale > 0.0f)) return -1;
    const float n = -log2f(scale);
    float chosen;
    if (method == RXMET_POT_ROUND) chosen = roundf(n);
    else if (method == RXMET_POT_FLOOR) chosen = floorf(n);
    else chosen = near_power_of_two(fabsf(rmax - rmin), tol) ? roundf(n) : floorf(n);
    if (chosen < -128.0f || chosen > 127.0f) return -1;
    const int8_t n8 = (int8_t)chosen;
    *po2 = powf(2.0f, -(float)n8);
    *n_out = n8;
    return 0;
}

/* include/scale_encoding.h:207-320 (encodeScaleResult and what it calls) plus
 * storedScaleForMode (:74-76): returns the scale to store and the zero point. */
static int encode_from_range(float mn, float mx, orc_bitwidth b, int symmetric,
                             const rxmet_gru_quant_config *cfg, float *scale_out, int32_t *zp_out) {
    cont_scale c;
    if (continuous_from_range(mn, mx, b, symmetric, &c)) return -1;
    const int32_t qmin = orc_qmin(b);
    if (cfg->use_pot2) {
        float po2;
        int n;
        if (scale_to_pot(c.scale, cfg->pot_scale_method, c.min, c.max, cfg->pot_scale_tolerance, &po2, &n)) return -1;
        int32_t zp = 0;
        if (!symmetric) {
            if (cfg->pot_scale_method == RXMET_POT_FLOOR) {
                const float aligned = floorf(c.min / po2) * po2;
                zp = (int32_t)rintf((float)qmin - aligned / po2);
            } else {
                zp = (int32_t)rintf((float)qmin - c.min / po2);
            }
        }
        *scale_out = po2;
        *zp_out = zp;
        return 0;
    }
    int32_t m, s;
    if (orc_encode_mshift(c.scale, &m, &s)) return -1;
    const float eff = (float)m * ldexpf(1.0f, -s);
    *zp_out = symmetric ? 0 : (int32_t)rintf((float)qmin - c.min / eff);
    *scale_out = c.scale; /* affine mode stores the continuous scale */
    return 0;
}

static orc_bitwidth bw_of(const rxmet_gru_quant_config *c, int op) {
    orc_bitwidth b;
    b.bits = c->bits[op];
    b.is_unsigned = (c->bits[op] >= 32) ? 0 : (c->is_unsigned[op] != 0);
    return b;
}

/* src/gru_host.cc:41-69 : weights by granularity. */
static int calibrate_weight(float *out, int hidden, int gran, orc_bitwidth b, int symmetric,
                            const float *mins, const float *maxs, const rxmet_gru_quant_config *cfg) {
    const int c3 = 3 * hidden;
    const int group = gran == RXMET_PER_TENSOR ? c3 : (gran == RXMET_PER_GATE ? hidden : 1);
    for (int begin = 0; begin < c3; begin += group) {
        float mn = mins[begin], mx = maxs[begin];
        if (gran == RXMET_PER_GATE) { mn = FLT_MAX; mx = -FLT_MAX; }
        for (int c = begin; c < begin + group; ++c) {
            if (mins[c] < mn) mn = mins[c];
            if (maxs[c] > mx) mx = maxs[c];
        }
        float s;
        int32_t zp;
        if (encode_from_range(mn, mx, b, symmetric, cfg, &s, &zp)) return -1;
        for (int c = begin; c < begin + group; ++c) out[c] = s;
    }
    return 0;
}

/* include/gru_calibration_helpers.h:33-62 : bias headroom, 2x the extent. */
static int calibrate_bias(float *out, int hidden, int gran, orc_bitwidth b, int use_pot2,
                          const float *mins, const float *maxs) {
    const int c3 = 3 * hidden;
    const int group = gran == RXMET_PER_TENSOR ? c3 : (gran == RXMET_PER_GATE ? hidden : 1);
    for (int begin = 0; begin < c3; begin += group) {
        double extent = 0.0;
        for (int c = begin; c < begin + group; ++c) {
            if (!isfinite(mins[c]) || !isfinite(maxs[c]) || mins[c] > maxs[c]) return -1;
            const double a = fabs((double)mins[c]), z = fabs((double)maxs[c]);
            const double m = a > z ? a : z;
            if (m > extent) extent = m;
        }
        double num = 2.0 * extent;
        if (!(num > 0.01)) num = 0.01;
        double scale = num / (double)orc_qmax(b);
        if (use_pot2) scale = exp2(ceil(log2(scale)));
        if (!isfinite(scale) || scale > FLT_MAX) return -1;
        for (int c = begin; c < begin + group; ++c) out[c] = (float)scale;
    }
    return 0;
}

/* src/gru_host.cc:13-125 */
int orc_gru_params_from_ranges(const rxmet_gru_ranges *r, const rxmet_gru_quant_config *cfg,
                               rxmet_gru_quant_params *out) {
    if (!cfg->symmetric[RXMET_GRU_W] || !cfg->symmetric[RXMET_GRU_R] ||
        !cfg->symmetric[RXMET_GRU_BW] || !cfg->symmetric[RXMET_GRU_BR]) return -1;
    out->hidden = r->hidden;
    out->config = *cfg;
    for (int i = 0; i < RXMET_GRU_NUM_OPS; ++i) { out->scale[i] = 0.0f; out->zero_point[i] = 0; }
    static const int scalar_ops[] = {
        RXMET_GRU_X, RXMET_GRU_H, RXMET_GRU_WEIGHT_IH_LINEAR, RXMET_GRU_WEIGHT_HH_LINEAR,
        RXMET_GRU_UPDATE_GATE_INPUT, RXMET_GRU_RESET_GATE_INPUT, RXMET_GRU_NEW_GATE_INPUT,
        RXMET_GRU_UPDATE_GATE_OUTPUT, RXMET_GRU_RESET_GATE_OUTPUT, RXMET_GRU_NEW_GATE_OUTPUT,
        RXMET_GRU_MUL_RESET_HIDDEN, RXMET_GRU_MUL_NEW_CONTRIBUTION, RXMET_GRU_MUL_OLD_CONTRIBUTION};
    for (unsigned k = 0; k < sizeof(scalar_ops) / sizeof(scalar_ops[0]); ++k) {
        const int op = scalar_ops[k];
        float mn = r->min[op], mx = r->max[op];
        if (op == RXMET_GRU_UPDATE_GATE_OUTPUT || op == RXMET_GRU_RESET_GATE_OUTPUT ||
            op == RXMET_GRU_NEW_GATE_OUTPUT) {
            /* include/calibration_utils.h:26-43 with threshold 0.5 (gru_host.cc:95-110) */
            const float range = mx - mn;
            if (range < 0.5f) {
                const float center = (mn + mx) / 2.0f;
                mn = center - 0.5f / 2.0f;
                mx = center + 0.5f / 2.0f;
            }
        }
        if (encode_from_range(mn, mx, bw_of(cfg, op), cfg->symmetric[op], cfg,
                              &out->scale[op], &out->zero_point[op])) return -1;
    }
    if (calibrate_weight(out->scale_W, r->hidden, cfg->W_granularity, bw_of(cfg, RXMET_GRU_W),
                         cfg->symmetric[RXMET_GRU_W], r->min_W, r->max_W, cfg)) return -1;
    if (calibrate_weight(out->scale_R, r->hidden, cfg->R_granularity, bw_of(cfg, RXMET_GRU_R),
                         cfg->symmetric[RXMET_GRU_R], r->min_R, r->max_R, cfg)) return -1;
    if (calibrate_bias(out->scale_bw, r->hidden, cfg->bw_granularity, bw_of(cfg, RXMET_GRU_BW),
                       cfg->use_pot2, r->min_bw, r->max_bw)) return -1;
    if (calibrate_bias(out->scale_br, r->hidden, cfg->br_granularity, bw_of(cfg, RXMET_GRU_BR),
                       cfg->use_pot2, r->min_br, r->max_br)) return -1;
    return 0;
}

/* ---- activation tables -------------------------------------------------- */

static int cmp_float(const void *a, const void *b) {
    const float x = *(const float *)a, y = *(const float *)b;
    return (x > y) - (x < y);
}

/* src/quantize_lut.cc:79-174 : 17 break points, denser around x = 0.  The
 * sigmoid-derivative weighting is used for the tanh table as well. */
static void segment_points(float x_min, float x_max, float *points /* [17] */) {
    enum { NS = 1000, SEG = 16 };
    static const float center_weight = 5.0f, center_range = 2.0f;
    float xs[NS], w[NS - 1], cum[NS - 1];
    for (int i = 0; i < NS; ++i) xs[i] = x_min + (x_max - x_min) * (float)i / (float)(NS - 1);
    for (int i = 0; i < NS - 1; ++i) {
        const float x = xs[i], xn = xs[i + 1];
        const float y = 1.0f / (1.0f + expf(-x));
        const float yn = 1.0f / (1.0f + expf(-xn));
        const float slope = fabsf(yn - y) / (xn - x + 1e-9f);
        const float dist = fabsf(x);
        if (dist < center_range) w[i] = center_weight * (1.0f - dist / center_range) + 1.0f;
        else w[i] = 1.0f + slope * 0.5f;
    }
    float sum = 0.0f;
    for (int i = 0; i < NS - 1; ++i) sum += w[i];
    for (int i = 0; i < NS - 1; ++i) w[i] /= sum;
    cum[0] = w[0];
    for (int i = 1; i < NS - 1; ++i) cum[i] = cum[i - 1] + w[i];

    float pts[SEG + 1 + 4];
    int n = 0;
    pts[n++] = x_min;
    for (int i = 1; i < SEG; ++i) {
        const float target = (float)i / (float)SEG;
        int lo = 0, hi = NS - 1; /* lower_bound: first cum[idx] >= target */
        while (lo < hi) {
            const int mid = (lo + hi) / 2;
            if (cum[mid] < target) lo = mid + 1; else hi = mid;
        }
        int idx = lo;
        if (idx >= NS - 1) idx = NS - 2;
        pts[n++] = xs[idx];
    }
    pts[n++] = x_max;
    qsort(pts, (size_t)n, sizeof(float), cmp_float);
    /* std::unique with |a-b| < 1e-9 against the last kept element */
    int kept = 0;
    for (int i = 1; i < n; ++i) {
        if (!(fabsf(pts[kept] - pts[i]) < 1e-9f)) pts[++kept] = pts[i];
    }
    n = kept + 1;
    while (n < SEG + 1) { /* refill by halving the widest gap */
        float gap_max = 0.0f;
        int at = 0;
        for (int i = 0; i < n - 1; ++i) {
            const float gap = pts[i + 1] - pts[i];
            if (gap > gap_max) { gap_max = gap; at = i; }
        }
        const float mid = (pts[at] + pts[at + 1]) / 2.0f;
        for (int i = n; i > at + 1; --i) pts[i] = pts[i - 1];
        pts[at + 1] = mid;
        ++n;
    }
    memcpy(points, pts, sizeof(float) * (SEG + 1));
}

/* src/quantize_lut.cc:53-76 : least squares over 100 samples, float sums. */
static void line_fit(const float *x, const float *y, int n, float *b, float *c) {
    float sx = 0.0f, sy = 0.0f, sxy = 0.0f, sx2 = 0.0f;
    for (int i = 0; i < n; ++i) {
        sx += x[i];
        sy += y[i];
        sxy += x[i] * y[i];
        sx2 += x[i] * x[i];
    }
    const float denom = (float)n * sx2 - sx * sx;
    if (fabsf(denom) < 1e-9f) {
        *b = 0.0f;
        *c = sy / (float)n;
        return;
    }
    *b = ((float)n * sxy - sx * sy) / denom;
    *c = (sy - *b * sx) / (float)n;
}

/* src/quantize_lut.cc:190-364 : is_tanh selects tanh (range +-4) over sigmoid
 * (range +-8). */
static void build_lut(int is_tanh, float scale_x, int32_t zp_x, float scale_y, int32_t zp_y,
                      orc_bitwidth in_bw, orc_bitwidth out_bw, orc_lut *lut) {
    const int32_t qlo = orc_qmin(in_bw), qhi = orc_qmax(in_bw);
    const float limit = is_tanh ? 4.0f : 8.0f;
    float x_min = (float)(qlo - zp_x) * scale_x;
    float x_max = (float)(qhi - zp_x) * scale_x;
    if (!(x_min > -limit)) x_min = -limit; /* std::max(x_min, -limit) */
    if (!(x_max < limit)) x_max = limit;   /* std::min(x_max, limit)  */
    lut->zp_x = zp_x;
    float pts[17];
    segment_points(x_min, x_max, pts);
    for (int i = 0; i < 16; ++i) {
        const float xs = pts[i], xe = pts[i + 1];
        float sx[100], sy[100];
        for (int j = 0; j < 100; ++j) {
            const float xv = xs + (xe - xs) * (float)j / 99.0f;
            sx[j] = xv;
            sy[j] = is_tanh ? tanhf(xv) : 1.0f / (1.0f + expf(-xv));
        }
        float b, c;
        line_fit(sx, sy, 100, &b, &c);
        const float m_real = b * (scale_x / scale_y);
        int32_t q_b = 0;
        int n_bx = 0;
        if (!(fabsf(m_real) < 1e-12f)) { /* :190-199 */
            const int32_t max_q = orc_qmax(out_bw);
            n_bx = (int)(int8_t)floor(log2((double)max_q / fabsf(m_real)));
            int64_t q = (int64_t)rint((double)m_real * ldexp(1.0, n_bx));
            if (q > max_q) q = max_q;
            if (q < -(int64_t)max_q) q = -(int64_t)max_q;
            q_b = (int32_t)q;
        }
        int32_t thr = (int32_t)rintf(xe / scale_x + (float)zp_x);
        if (thr < qlo) thr = qlo;
        if (thr > qhi) thr = qhi;
        lut->seg[i].q_b = q_b;
        lut->seg[i].n_bx_total = n_bx;
        lut->seg[i].term_c = (int32_t)rintf(c / scale_y + (float)zp_y);
        lut->seg[i].threshold = thr;
    }
}

/* src/quantize_lut.cc:17-48 : tables are built from the stored scales. */
static void build_all_luts(const rxmet_gru_quant_params *p, orc_lut *u, orc_lut *r, orc_lut *n) {
    const rxmet_gru_quant_config *c = &p->config;
    build_lut(0, p->scale[RXMET_GRU_UPDATE_GATE_INPUT], p->zero_point[RXMET_GRU_UPDATE_GATE_INPUT],
              p->scale[RXMET_GRU_UPDATE_GATE_OUTPUT], p->zero_point[RXMET_GRU_UPDATE_GATE_OUTPUT],
              bw_of(c, RXMET_GRU_UPDATE_GATE_INPUT), bw_of(c, RXMET_GRU_UPDATE_GATE_OUTPUT), u);
    build_lut(0, p->scale[RXMET_GRU_RESET_GATE_INPUT], p->zero_point[RXMET_GRU_RESET_GATE_INPUT],
              p->scale[RXMET_GRU_RESET_GATE_OUTPUT], p->zero_point[RXMET_GRU_RESET_GATE_OUTPUT],
              bw_of(c, RXMET_GRU_RESET_GATE_INPUT), bw_of(c, RXMET_GRU_RESET_GATE_OUTPUT), r);
    build_lut(1, p->scale[RXMET_GRU_NEW_GATE_INPUT], p->zero_point[RXMET_GRU_NEW_GATE_INPUT],
              p->scale[RXMET_GRU_NEW_GATE_OUTPUT], p->zero_point[RXMET_GRU_NEW_GATE_OUTPUT],
              bw_of(c, RXMET_GRU_NEW_GATE_INPUT), bw_of(c, RXMET_GRU_NEW_GATE_OUTPUT), n);
}

int orc_gru_build_luts(const rxmet_gru_quant_params *params, rxmet_lut_segment out[3][16]) {
    orc_lut u, r, n;
    build_all_luts(params, &u, &r, &n);
    memcpy(out[0], u.seg, sizeof(u.seg));
    memcpy(out[1], r.seg, sizeof(r.seg));
    memcpy(out[2], n.seg, sizeof(n.seg));
    return 0;
}

/* ---- execution parameters ---------------------------------------------- */

void orc_gru_exec_free(orc_gru_exec *e) {
    free(e->eff_W); free(e->eff_R); free(e->eff_bw); free(e->eff_br);
    free(e->gemm_x); free(e->bias_x); free(e->gemm_h); free(e->bias_h);
    memset(e, 0, sizeof(*e));
}

/* src/gru_forward_cpu_quant.cc:220-310 (fillLinearParamsCPU, fillGateParamsCPU) */
int orc_gru_exec_init(orc_gru_exec *e, const rxmet_gru_quant_params *p) {
    memset(e, 0, sizeof(*e));
    const int H = p->hidden, C = 3 * H;
    const int pot = p->config.use_pot2 != 0;
    e->hidden = H;
    for (int i = 0; i < RXMET_GRU_NUM_OPS; ++i) {
        e->bw[i] = bw_of(&p->config, i);
        e->zp[i] = p->zero_point[i];
        e->eff_scale[i] = 0.0f;
        if (p->scale[i] > 0.0f && effective_scale(p->scale[i], pot, &e->eff_scale[i])) return -1;
    }
    const float *S = p->scale;
    int bad = 0;
    bad |= make_rescale(pot, 0, S[RXMET_GRU_WEIGHT_IH_LINEAR], S[RXMET_GRU_UPDATE_GATE_INPUT], 0, &e->ih_to_update);
    bad |= make_rescale(pot, 0, S[RXMET_GRU_WEIGHT_HH_LINEAR], S[RXMET_GRU_UPDATE_GATE_INPUT], 0, &e->hh_to_update);
    bad |= make_rescale(pot, 0, S[RXMET_GRU_WEIGHT_IH_LINEAR], S[RXMET_GRU_RESET_GATE_INPUT], 0, &e->ih_to_reset);
    bad |= make_rescale(pot, 0, S[RXMET_GRU_WEIGHT_HH_LINEAR], S[RXMET_GRU_RESET_GATE_INPUT], 0, &e->hh_to_reset);
    bad |= make_rescale(pot, 0, S[RXMET_GRU_WEIGHT_IH_LINEAR], S[RXMET_GRU_NEW_GATE_INPUT], 0, &e->ih_to_new);
    bad |= make_rescale(pot, 1, S[RXMET_GRU_RESET_GATE_OUTPUT], S[RXMET_GRU_WEIGHT_HH_LINEAR],
                        S[RXMET_GRU_NEW_GATE_INPUT], &e->rh_to_new);
    bad |= make_rescale(pot, 0, S[RXMET_GRU_NEW_GATE_OUTPUT], S[RXMET_GRU_H], 0, &e->new_to_h);
    bad |= make_rescale(pot, 1, S[RXMET_GRU_UPDATE_GATE_OUTPUT], S[RXMET_GRU_H], S[RXMET_GRU_H], &e->update_old_to_h);
    if (bad) return -1;
    e->quant_one = (int32_t)rintf(1.0f / S[RXMET_GRU_UPDATE_GATE_OUTPUT]) + p->zero_point[RXMET_GRU_UPDATE_GATE_OUTPUT];
    build_all_luts(p, &e->lut_update, &e->lut_reset, &e->lut_new);
    e->eff_W = (float *)malloc(sizeof(float) * C);
    e->eff_R = (float *)malloc(sizeof(float) * C);
    e->eff_bw = (float *)malloc(sizeof(float) * C);
    e->eff_br = (float *)malloc(sizeof(float) * C);
    e->gemm_x = (orc_rescale *)malloc(sizeof(orc_rescale) * C);
    e->bias_x = (orc_rescale *)malloc(sizeof(orc_rescale) * C);
    e->gemm_h = (orc_rescale *)malloc(sizeof(orc_rescale) * C);
    e->bias_h = (orc_rescale *)malloc(sizeof(orc_rescale) * C);
    for (int c = 0; c < C; ++c) {
        bad |= effective_scale(p->scale_W[c], pot, &e->eff_W[c]);
        bad |= effective_scale(p->scale_R[c], pot, &e->eff_R[c]);
        bad |= effective_scale(p->scale_bw[c], pot, &e->eff_bw[c]);
        bad |= effective_scale(p->scale_br[c], pot, &e->eff_br[c]);
        bad |= make_rescale(pot, 1, p->scale_W[c], S[RXMET_GRU_X], S[RXMET_GRU_WEIGHT_IH_LINEAR], &e->gemm_x[c]);
        bad |= make_rescale(pot, 2, p->scale_bw[c], p->scale_W[c], S[RXMET_GRU_X], &e->bias_x[c]);
        bad |= make_rescale(pot, 1, p->scale_R[c], S[RXMET_GRU_H], S[RXMET_GRU_WEIGHT_HH_LINEAR], &e->gemm_h[c]);
        bad |= make_rescale(pot, 2, p->scale_br[c], p->scale_R[c], S[RXMET_GRU_H], &e->bias_h[c]);
    }
    if (bad) {
        orc_gru_exec_free(e);
        return -1;
    }
    return 0;
}

/* Shared with the forward file. */
int64_t orc_apply_rescale(int64_t x, orc_rescale r) { return apply_rescale(x, r); }
