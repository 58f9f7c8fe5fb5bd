// Device-side integer primitives of the QuantGRU integer carrier.  Bit-level
// behaviour follows operators/quant-gru/include/quantize_ops_helper.h of the
// reference (cited per function); the code is organised for the GPU: 32-bit
// fast paths where the operands provably fit, tables in shared memory.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

#include "gru_params.h"

namespace rxmet {
namespace gru {

// Gate rescales the input projection may apply on top of its own output rescale: when enabled, what it
// stores is rescale(code - zero point) with the rescale of the gate the column belongs to (the ih
// contribution to the gate input, which does not depend on the recurrent state).
struct PreRescale {
    int enabled;
    int hidden;
    Rescale toGate[3];
};

// round_half_even(x / 2^n) on the magnitude, sign restored afterwards; n <= 0
// shifts left (quantize_ops_helper.h:201-224).
__device__ __forceinline__ int64_t rshiftRound(int64_t x, int n) {
    if (n <= 0) return x << (-n);
    // floor quotient q = x >> n and non-negative remainder r: the result is q + (r > half || (r == half && q odd)).
    // Adding half - 1 + (q & 1) before the shift carries in exactly those cases (a remainder above half always,
    // one equal to half only into an odd quotient, a smaller one never), which equals the reference's
    // round-the-magnitude-then-negate formulation for every x (round-half-even is symmetric).  |x| < 2^62.
    const int64_t roundAdd = (static_cast<int64_t>(1) << (n - 1)) - 1;
    return (x + roundAdd + ((x >> n) & 1)) >> n;
}

// The same rounding shift for 1 <= n <= 62 as one add and one shift:
// floor((x + 2^(n-1) - 1 + odd(floor(x / 2^n))) / 2^n); roundAdd = 2^(n-1) - 1 is a constant of
// the caller (per channel).  A remainder above half carries, one equal to half carries only into
// an odd quotient, a smaller one never does.
__device__ __forceinline__ int64_t rshiftRoundConst(int64_t x, int n, int64_t roundAdd) {
    return (x + roundAdd + ((x >> n) & 1)) >> n;
}

// quantize_ops_helper.h:242-248
__device__ __forceinline__ int64_t applyRescale(int64_t x, Rescale r) {
    return rshiftRound(x * static_cast<int64_t>(r.mult), r.shift);
}

// 32-bit variant for operands whose product with the multiplier provably fits 31 bits
// (|x| < 2^15 and mult < 2^16).  Same rounding rule.
__device__ __forceinline__ int32_t rshiftRound32(int32_t x, int n) {
    if (n <= 0) return x << (-n);
    if (n > 31) return 0;  // |x| < 2^30 < half : rounds to zero
    const int32_t q = x >> n;
    const uint32_t r = static_cast<uint32_t>(x) & ((1u << n) - 1u);
    const uint32_t half = 1u << (n - 1);
    return q + static_cast<int32_t>((r > half) || (r == half && (q & 1)));
}

// 32-bit operand times 16-bit multiplier in one widening multiply, then the 64-bit rounding shift.
__device__ __forceinline__ int32_t rescaleWide(int32_t x, Rescale r) {
    return static_cast<int32_t>(rshiftRound(static_cast<int64_t>(x) * static_cast<int64_t>(r.mult), r.shift));
}

// Rescale of a small operand (a grid difference): 32-bit when Narrow, else 64-bit.
template <bool Narrow>
__device__ __forceinline__ int32_t rescaleSmall(int32_t x, Rescale r) {
    if constexpr (Narrow) return rshiftRound32(x * r.mult, r.shift);
    else return static_cast<int32_t>(rshiftRound(static_cast<int64_t>(x) * r.mult, r.shift));
}

// quantize_ops_helper.h:267-278 ; keep = 1 when the value was inside the grid.
__device__ __forceinline__ int32_t clampCode(int32_t v, int32_t lo, int32_t hi, uint8_t &keep) {
    keep = (v < lo || v > hi) ? 0 : 1;
    return max(lo, min(v, hi));
}

// Float -> code: divide, round half even, add the zero point afterwards,
// saturate (quantize_ops_helper.h:133-140,280-292,357-365).  The rounded
// quotient is saturated to +-2^31 before the integer add; that cannot change
// the clamped result because |zp| < 2^31 and the grid is at most 32 bit.
__device__ __forceinline__ int32_t quantizeValue(float v, float scale, int32_t zp, int32_t lo, int32_t hi,
                                                 uint8_t &keep) {
    float r = rintf(v / scale);
    r = fminf(fmaxf(r, -4294967296.0f), 4294967296.0f);
    const int64_t code = static_cast<int64_t>(r) + zp;
    keep = (code < lo || code > hi) ? 0 : 1;
    return static_cast<int32_t>(code < lo ? lo : (code > hi ? hi : code));
}

// 16-segment table: first segment whose threshold exceeds q_x, else the last
// (quantize_ops_helper.h:503-532).
template <bool Narrow = false>
__device__ __forceinline__ int32_t lutEval(int32_t qx, const Lut &lut) {
    int seg = kSegments - 1;
#pragma unroll
    for (int i = kSegments - 2; i >= 0; --i) seg = (qx < lut.threshold[i]) ? i : seg;
    const int n = lut.n_bx[seg];
    int32_t term;
    if constexpr (Narrow) {
        term = rshiftRound32(lut.q_b[seg] * (qx - lut.zp_x), n);
    } else {
        const int64_t bx = static_cast<int64_t>(lut.q_b[seg]) * static_cast<int64_t>(qx - lut.zp_x);
        term = (n >= 0) ? static_cast<int32_t>(rshiftRound(bx, n)) : static_cast<int32_t>(bx << (-n));
    }
    return term + lut.term_c[seg];
}

struct GateMasks {
    uint8_t in[3];   // update, reset, new : gate-input clamp
    uint8_t out[3];  // update, reset, new : gate-output clamp
    uint8_t h;       // hidden-state clamp
};

struct GateCodes {
    int32_t z, r, n, h;
};

// One (batch, hidden) element of a GRU step on the integer grids
// (quantize_ops_helper.h:683-1023).  ih* / hh* are the linear-stage codes of
// the three gates, hOld the previous hidden code.  Narrow = true computes the
// grid-to-grid rescales and the table products in 32 bit; the host enables it
// only when every such operand is below 2^15 in magnitude and every table
// slope times its operand is below 2^31 (true for all grids of 8 bit or less).
template <bool Narrow = false>
__device__ __forceinline__ GateCodes gruCell(int32_t ihz, int32_t ihr, int32_t ihn, int32_t hhz, int32_t hhr,
                                             int32_t hhn, int32_t hOld, const GateExec &g, GateMasks &m) {
    const int32_t zpIh = g.zp[RXMET_GRU_WEIGHT_IH_LINEAR], zpHh = g.zp[RXMET_GRU_WEIGHT_HH_LINEAR];
    GateCodes c;
    {   // update gate
        const int32_t a = rescaleSmall<Narrow>(ihz - zpIh, g.ih_to_update);
        const int32_t b = rescaleSmall<Narrow>(hhz - zpHh, g.hh_to_update);
        const int32_t pre = clampCode(a + b + g.zp[RXMET_GRU_UPDATE_GATE_INPUT], g.qlo[RXMET_GRU_UPDATE_GATE_INPUT],
                                      g.qhi[RXMET_GRU_UPDATE_GATE_INPUT], m.in[0]);
        c.z = clampCode(lutEval<Narrow>(pre, g.lut_update), g.qlo[RXMET_GRU_UPDATE_GATE_OUTPUT],
                        g.qhi[RXMET_GRU_UPDATE_GATE_OUTPUT], m.out[0]);
    }
    {   // reset gate
        const int32_t a = rescaleSmall<Narrow>(ihr - zpIh, g.ih_to_reset);
        const int32_t b = rescaleSmall<Narrow>(hhr - zpHh, g.hh_to_reset);
        const int32_t pre = clampCode(a + b + g.zp[RXMET_GRU_RESET_GATE_INPUT], g.qlo[RXMET_GRU_RESET_GATE_INPUT],
                                      g.qhi[RXMET_GRU_RESET_GATE_INPUT], m.in[1]);
        c.r = clampCode(lutEval<Narrow>(pre, g.lut_reset), g.qlo[RXMET_GRU_RESET_GATE_OUTPUT],
                        g.qhi[RXMET_GRU_RESET_GATE_OUTPUT], m.out[1]);
    }
    {   // candidate: the reset product goes straight to the gate-input grid
        const int64_t prod = (static_cast<int64_t>(c.r) - g.zp[RXMET_GRU_RESET_GATE_OUTPUT]) *
                             (static_cast<int64_t>(hhn) - zpHh);
        const int32_t rh = static_cast<int32_t>(applyRescale(prod, g.rh_to_new));
        const int32_t a = rescaleSmall<Narrow>(ihn - zpIh, g.ih_to_new);
        const int32_t pre = clampCode(a + rh + g.zp[RXMET_GRU_NEW_GATE_INPUT], g.qlo[RXMET_GRU_NEW_GATE_INPUT],
                                      g.qhi[RXMET_GRU_NEW_GATE_INPUT], m.in[2]);
        c.n = clampCode(lutEval<Narrow>(pre, g.lut_new), g.qlo[RXMET_GRU_NEW_GATE_OUTPUT], g.qhi[RXMET_GRU_NEW_GATE_OUTPUT],
                        m.out[2]);
    }
    {   // h' = z*h + (1-z)*n on the h grid, one rounding for the sum
        const int32_t zpH = g.zp[RXMET_GRU_H];
        const int32_t nAligned = rescaleSmall<Narrow>(c.n - g.zp[RXMET_GRU_NEW_GATE_OUTPUT], g.new_to_h) + zpH;
        const int64_t oldPart = (static_cast<int64_t>(c.z) - g.zp[RXMET_GRU_UPDATE_GATE_OUTPUT]) *
                                (static_cast<int64_t>(hOld) - zpH);
        const int64_t newPart = (static_cast<int64_t>(g.quant_one) - c.z) * (static_cast<int64_t>(nAligned) - zpH);
        const int32_t hNew = static_cast<int32_t>(applyRescale(oldPart + newPart, g.update_old_to_h)) + zpH;
        c.h = clampCode(hNew, g.qlo[RXMET_GRU_H], g.qhi[RXMET_GRU_H], m.h);
    }
    return c;
}

// Direct activation tables: entry [q - lo] = (output code << 1) | keep, for every gate-input code.
struct DirectTables {
    const int32_t *update, *reset, *fresh;
};

// The same cell for small grids (the host checks: linear, gate-input and gate-output grids of at
// most 10 bits, zero points on their grids, non-negative shifts): 32-bit rescales, widening
// multiplies for the two products, activations read from direct tables.  az/ar/an are the ih
// contributions ALREADY rescaled to the three gate-input grids (the input projection does that
// once for all steps, since it does not depend on the state).
__device__ __forceinline__ GateCodes gruCellFast(int32_t az, int32_t ar, int32_t an, int32_t hhz, int32_t hhr,
                                                 int32_t hhn, int32_t hOld, const GateExec &g, const DirectTables &tab,
                                                 GateMasks &m) {
    const int32_t zpHh = g.zp[RXMET_GRU_WEIGHT_HH_LINEAR];
    GateCodes c;
    {
        const int32_t b = rshiftRound32((hhz - zpHh) * g.hh_to_update.mult, g.hh_to_update.shift);
        const int32_t lo = g.qlo[RXMET_GRU_UPDATE_GATE_INPUT];
        const int32_t pre = clampCode(az + b + g.zp[RXMET_GRU_UPDATE_GATE_INPUT], lo, g.qhi[RXMET_GRU_UPDATE_GATE_INPUT], m.in[0]);
        const int32_t e = tab.update[pre - lo];
        c.z = e >> 1;
        m.out[0] = static_cast<uint8_t>(e & 1);
    }
    {
        const int32_t b = rshiftRound32((hhr - zpHh) * g.hh_to_reset.mult, g.hh_to_reset.shift);
        const int32_t lo = g.qlo[RXMET_GRU_RESET_GATE_INPUT];
        const int32_t pre = clampCode(ar + b + g.zp[RXMET_GRU_RESET_GATE_INPUT], lo, g.qhi[RXMET_GRU_RESET_GATE_INPUT], m.in[1]);
        const int32_t e = tab.reset[pre - lo];
        c.r = e >> 1;
        m.out[1] = static_cast<uint8_t>(e & 1);
    }
    {
        const int32_t prod = (c.r - g.zp[RXMET_GRU_RESET_GATE_OUTPUT]) * (hhn - zpHh);
        const int32_t rh = rescaleWide(prod, g.rh_to_new);
        const int32_t lo = g.qlo[RXMET_GRU_NEW_GATE_INPUT];
        const int32_t pre = clampCode(an + rh + g.zp[RXMET_GRU_NEW_GATE_INPUT], lo, g.qhi[RXMET_GRU_NEW_GATE_INPUT], m.in[2]);
        const int32_t e = tab.fresh[pre - lo];
        c.n = e >> 1;
        m.out[2] = static_cast<uint8_t>(e & 1);
    }
    {
        const int32_t zpH = g.zp[RXMET_GRU_H];
        const int32_t nAligned = rshiftRound32((c.n - g.zp[RXMET_GRU_NEW_GATE_OUTPUT]) * g.new_to_h.mult, g.new_to_h.shift) + zpH;
        const int32_t sum = (c.z - g.zp[RXMET_GRU_UPDATE_GATE_OUTPUT]) * (hOld - zpH) + (g.quant_one - c.z) * (nAligned - zpH);
        c.h = clampCode(rescaleWide(sum, g.update_old_to_h) + zpH, g.qlo[RXMET_GRU_H], g.qhi[RXMET_GRU_H], m.h);
    }
    return c;
}

// round_half_even(p / 2^n) for 1 <= n <= 31 when the quotient fits 32 bits: floor quotient by
// funnel shift, remainder r < 2^n, and (r + odd(q)) > half is exactly "above half, or half into
// an odd quotient".
__device__ __forceinline__ int32_t rshiftRoundNarrow(int64_t p, int n, uint32_t remMask, uint32_t half) {
    const uint32_t lo = static_cast<uint32_t>(p), hi = static_cast<uint32_t>(static_cast<uint64_t>(p) >> 32);
    const int32_t q = static_cast<int32_t>(__funnelshift_r(lo, hi, n));
    const uint32_t r = lo & remMask;
    return q + static_cast<int32_t>((r + static_cast<uint32_t>(q & 1)) > half);
}

// One rescale of the fast cell with its constants in registers.  Small operands (grid
// differences times a 16-bit multiplier, product below 2^31): shift in [0, 31], branch free
// (shift 0 has an empty remainder and a half nothing exceeds).  Products: `narrow` says that the
// 64-bit product can be rounded with 32-bit pieces (multiplier at most 2^shift, shift in [1, 31]).
struct PreparedRescale {
    int32_t mult, shift;
    uint32_t remMask, half;
    bool narrow;
};
__device__ __forceinline__ PreparedRescale prepareRescale(Rescale r) {
    PreparedRescale p;
    p.mult = r.mult;
    p.shift = r.shift;
    const int n = r.shift & 31;
    p.remMask = (1u << n) - 1u;
    p.half = n ? (1u << (n - 1)) : 0x7fffffffu;
    p.narrow = r.shift >= 1 && r.shift <= 31 && r.mult > 0 && static_cast<int64_t>(r.mult) <= (1ll << r.shift);
    return p;
}
__device__ __forceinline__ int32_t rescaleSmallPrepared(int32_t x, const PreparedRescale &p) {
    const int32_t v = x * p.mult, q = v >> p.shift;
    const uint32_t r = static_cast<uint32_t>(v) & p.remMask;
    return q + static_cast<int32_t>((r + static_cast<uint32_t>(q & 1)) > p.half);
}
// The general rounding shift behind a call: a call is never evaluated speculatively, so code that
// picks between it and the 32-bit form per value pays for the 64-bit form only when it is taken.
static __device__ __noinline__ int32_t rshiftRoundCalled(int64_t x, int n) { return static_cast<int32_t>(rshiftRound(x, n)); }

__device__ __forceinline__ int32_t rescaleProductPrepared(int32_t x, const PreparedRescale &p) {
    const int64_t prod = static_cast<int64_t>(x) * p.mult;
    if (p.narrow) return rshiftRoundNarrow(prod, p.shift, p.remMask, p.half);
    return rshiftRoundCalled(prod, p.shift);
}

// Constants of gruCellFast gathered in registers once per thread (the cell otherwise re-reads
// them from the shared copy of the parameters in every step).
struct FastCell {
    PreparedRescale hhToUpdate, hhToReset, rhToNew, newToH, updateOldToH;
    int32_t zpHh, zpR, zpN, zpZ, zpH, quantOne;
    int32_t zpIn[3], loIn[3], hiIn[3];
    int32_t loH, hiH;
};
__device__ __forceinline__ FastCell prepareFastCell(const GateExec &g) {
    FastCell f;
    f.hhToUpdate = prepareRescale(g.hh_to_update);
    f.hhToReset = prepareRescale(g.hh_to_reset);
    f.rhToNew = prepareRescale(g.rh_to_new);
    f.newToH = prepareRescale(g.new_to_h);
    f.updateOldToH = prepareRescale(g.update_old_to_h);
    f.zpHh = g.zp[RXMET_GRU_WEIGHT_HH_LINEAR];
    f.zpR = g.zp[RXMET_GRU_RESET_GATE_OUTPUT];
    f.zpN = g.zp[RXMET_GRU_NEW_GATE_OUTPUT];
    f.zpZ = g.zp[RXMET_GRU_UPDATE_GATE_OUTPUT];
    f.zpH = g.zp[RXMET_GRU_H];
    f.quantOne = g.quant_one;
    const int ops[3] = {RXMET_GRU_UPDATE_GATE_INPUT, RXMET_GRU_RESET_GATE_INPUT, RXMET_GRU_NEW_GATE_INPUT};
#pragma unroll
    for (int i = 0; i < 3; ++i) {
        f.zpIn[i] = g.zp[ops[i]];
        f.loIn[i] = g.qlo[ops[i]];
        f.hiIn[i] = g.qhi[ops[i]];
    }
    f.loH = g.qlo[RXMET_GRU_H];
    f.hiH = g.qhi[RXMET_GRU_H];
    return f;
}

// gruCellFast with prepared constants: the same arithmetic, value for value.
__device__ __forceinline__ GateCodes gruCellPrepared(int32_t az, int32_t ar, int32_t an, int32_t hhz, int32_t hhr, int32_t hhn,
                                                     int32_t hOld, const FastCell &f, const DirectTables &tab, GateMasks &m) {
    GateCodes c;
    {
        const int32_t b = rescaleSmallPrepared(hhz - f.zpHh, f.hhToUpdate);
        const int32_t pre = clampCode(az + b + f.zpIn[0], f.loIn[0], f.hiIn[0], m.in[0]);
        const int32_t e = tab.update[pre - f.loIn[0]];
        c.z = e >> 1;
        m.out[0] = static_cast<uint8_t>(e & 1);
    }
    {
        const int32_t b = rescaleSmallPrepared(hhr - f.zpHh, f.hhToReset);
        const int32_t pre = clampCode(ar + b + f.zpIn[1], f.loIn[1], f.hiIn[1], m.in[1]);
        const int32_t e = tab.reset[pre - f.loIn[1]];
        c.r = e >> 1;
        m.out[1] = static_cast<uint8_t>(e & 1);
    }
    {
        const int32_t prod = (c.r - f.zpR) * (hhn - f.zpHh);
        const int32_t rh = rescaleProductPrepared(prod, f.rhToNew);
        const int32_t pre = clampCode(an + rh + f.zpIn[2], f.loIn[2], f.hiIn[2], m.in[2]);
        const int32_t e = tab.fresh[pre - f.loIn[2]];
        c.n = e >> 1;
        m.out[2] = static_cast<uint8_t>(e & 1);
    }
    {
        const int32_t nAligned = rescaleSmallPrepared(c.n - f.zpN, f.newToH) + f.zpH;
        const int32_t sum = (c.z - f.zpZ) * (hOld - f.zpH) + (f.quantOne - c.z) * (nAligned - f.zpH);
        c.h = clampCode(rescaleProductPrepared(sum, f.updateOldToH) + f.zpH, f.loH, f.hiH, m.h);
    }
    return c;
}

// Accumulate a[k] * w[k] exactly.  int8 x int8 packs four products per dp4a.
template <class AccT>
__device__ __forceinline__ void macCodes(AccT &acc, int32_t w, int32_t a) {
    acc += static_cast<AccT>(w) * static_cast<AccT>(a);
}

}  // namespace gru
}  // namespace rxmet
