// LSTM backward through time on real values, with the optional clamp masks of the QAT path.
//
// Launch plan (the reference runs T x (pointwise kernel + cuBLAS GEMM) and three cuBLAS GEMMs,
// operators/quant-lstm/src/lstm/backward_float_cuda.cu:50-104,189-330):
//   dequantWeights x2  : QAT only - q-carrier weight codes x per-channel scale -> real weights
//   recurrentBackward  : ONE launch for all T steps; a CTA owns BT batch rows, walks t = T-1..0,
//                        keeps dc in registers and dh in shared memory, writes the masked gate
//                        gradients of both linear branches, and propagates dh through weight_hh
//                        (rows resident in shared memory as far as they fit, the rest in registers)
//   gemmRowsTN + reduce: dW_ih = G_ih^T x, dW_hh = G_hh^T h_prev as split-K tile GEMMs over the T*B
//                        rows with fixed-order reduction (bit-reproducible), masks applied there
//   gemmNN             : dx = G_ih W_ih with the input clamp mask
//   columnSums + reduce: bias gradients
// Saved q-carrier tensors are dequantized while they are loaded: real = (value - zp) * scale.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstdlib>

#include "common.h"
#include "input_grad_umma.h"
#include "lstm_kernels.h"
#include "umma_device.cuh"
#include "weight_grad_mma.h"

namespace rxmet {
namespace lstm {
namespace {

__device__ __forceinline__ void prefetchL2(const void *p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
__device__ __forceinline__ float keepOf(const uint8_t *mask, size_t i) { return (mask == nullptr || mask[i] == 0) ? 1.0f : 0.0f; }
__device__ __forceinline__ float realOf(float v, Dequant d) { return (v - d.zeroPoint) * d.scale; }

__global__ void dequantWeights(const float *__restrict__ codes, const float *__restrict__ channelScale, int rows, int cols,
                               float *__restrict__ out) {
    const size_t n = static_cast<size_t>(rows) * cols;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<size_t>(gridDim.x) * blockDim.x)
        out[i] = codes[i] * channelScale[i / cols];
}

// One word of keep/drop flags per (t, b, j): bit 0 hidden, 1 tanh(cell), 2 cell, 3-6 gate outputs,
// 7-10 gate inputs, 11-14 ih linear, 15-18 hh linear (a set bit = clamped = no gradient).  Packing them
// once in a bandwidth-bound pass takes 19 byte loads per element off every step of the recurrence.
__global__ void packStepMasks(const rxmet_lstm_backward_masks mk, size_t rows, int H, uint32_t *__restrict__ out) {
    const size_t n = rows * H;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t row = i / H, j = i % H, go = row * 4 * H + j;
        auto bit = [](const uint8_t *m, size_t idx) -> uint32_t { return (m != nullptr && m[idx] != 0) ? 1u : 0u; };
        uint32_t w = bit(mk.hidden_outputs, i) | (bit(mk.cell_tanh_outputs, i) << 1) | (bit(mk.cell_states, i) << 2);
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            const size_t o = go + static_cast<size_t>(g) * H;
            w |= (bit(mk.gate_outputs, o) << (3 + g)) | (bit(mk.gate_inputs, o) << (7 + g)) |
                 (bit(mk.weight_ih_linear, o) << (11 + g)) | (bit(mk.weight_hh_linear, o) << (15 + g));
        }
        out[i] = w;
    }
}

// The same packing, four hidden units per thread (H a multiple of 4, flag bytes 0 or 1, as every
// forward of this library writes them): 32-bit loads of four flag bytes, byte permutes spread them
// over the 16-bit lanes of two words and a multiply-add moves each pair into its bit position.
// Bits 0..14 are gathered in one pair of words, bits 15..18 in a second pair.
__global__ void packStepMasks4(const rxmet_lstm_backward_masks mk, size_t quads, int H, uint4 *__restrict__ out) {
    for (size_t q = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; q < quads;
         q += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t i = q * 4, row = i / H, j = i % H, go = row * 4 * H + j;
        uint32_t low01 = 0, low23 = 0, high01 = 0, high23 = 0;
        auto add = [](const void *m, size_t at, int pos, uint32_t &a01, uint32_t &a23) {
            const uint32_t w = m ? *reinterpret_cast<const uint32_t *>(static_cast<const uint8_t *>(m) + at) : 0u;
            a01 += __byte_perm(w, 0u, 0x4140) * (1u << pos);
            a23 += __byte_perm(w, 0u, 0x4342) * (1u << pos);
        };
        add(mk.hidden_outputs, i, 0, low01, low23);
        add(mk.cell_tanh_outputs, i, 1, low01, low23);
        add(mk.cell_states, i, 2, low01, low23);
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            const size_t o = go + static_cast<size_t>(g) * H;
            add(mk.gate_outputs, o, 3 + g, low01, low23);
            add(mk.gate_inputs, o, 7 + g, low01, low23);
            add(mk.weight_ih_linear, o, 11 + g, low01, low23);
            add(mk.weight_hh_linear, o, g, high01, high23);
        }
        out[q] = make_uint4((low01 & 0xffffu) | ((high01 & 0xffffu) << 15), (low01 >> 16) | ((high01 >> 16) << 15),
                            (low23 & 0xffffu) | ((high23 & 0xffffu) << 15), (low23 >> 16) | ((high23 >> 16) << 15));
    }
}

struct RecurrentArgs {
    int T, B, H, smemRows;  // smemRows: leading rows of each gate block held in shared memory
    int smemStride;         // floats between consecutive columns of the transposed copy (odd multiple of 4)
    const uint32_t *stepMasks;  // packed flags [T][B][H] or null
    const float *weightHh;  // real [4H][H]
    const float *c0;
    const float *gateOutputs, *cellStates, *cellTanh;
    const float *gradOutput, *gradFinalHidden, *gradFinalCell;
    Dequant dqC, dqGate[4], dqTanh;
    rxmet_lstm_backward_masks mk;
    float *gIh, *gHh;  // [T][B][4H]
    float *dh0, *dc0;  // [B][H] (masks applied)
};

// Rows of weight_hh that do not fit shared memory are kept in registers: thread (q, j) owns column j
// of the rows of gate q, the first smemRows of them in shared memory and up to kRegRows after that
// in registers, so that a step never goes to L2 for weights.
constexpr int kRegRows = 32;

template <int BT>
__global__ void __launch_bounds__(512) recurrentBackward(const __grid_constant__ RecurrentArgs a) {
    const int H = a.H, C = 4 * a.H, S = a.smemRows, R = H - S;
    extern __shared__ __align__(16) float smemF[];
    float *gS = smemF;               // [BT][C] gradient entering the hh branch
    float *partS = gS + BT * C;      // [4][BT][H] partial sums of dh
    float *wS = partS + 4 * BT * H;  // [4][S][H] leading rows of each gate block of weight_hh
    const int tid = threadIdx.x, nthreads = blockDim.x;
    const int b0 = blockIdx.x * BT, nb = min(BT, a.B - b0);
    // transposed per thread: the S leading rows of column j of gate block g are contiguous (stride SP),
    // so that phase A reads four of them with one 128-bit load
    const int SP = a.smemStride;
    for (int i = tid; i < 4 * S * H; i += nthreads) {
        const int g = i / (S * H), r = (i / H) % S, j = i % H;
        wS[(static_cast<size_t>(g) * H + j) * SP + r] = a.weightHh[(static_cast<size_t>(g) * H + r) * H + j];
    }
    for (int i = tid; i < 4 * BT * H; i += nthreads) partS[i] = 0.0f;
    for (int i = tid; i < BT * C; i += nthreads) gS[i] = 0.0f;

    const int elems = nb * H;
    const bool hasElem = tid < elems;
    const int eb = hasElem ? tid / H : 0, ej = hasElem ? tid % H : 0;
    const size_t stateIdx = static_cast<size_t>(b0 + eb) * H + ej;
    float dhCarry = hasElem ? a.gradFinalHidden[stateIdx] : 0.0f;
    float dc = hasElem ? a.gradFinalCell[stateIdx] : 0.0f;
    // phase A ownership: gate block q of the channels, hidden column j
    const bool hasColumn = tid < C;
    const int q = hasColumn ? tid / H : 0, cj = tid % H;
    float wr[kRegRows];
#pragma unroll
    for (int r = 0; r < kRegRows; ++r)
        wr[r] = (hasColumn && r < R) ? a.weightHh[(static_cast<size_t>(q) * H + S + r) * H + cj] : 0.0f;
    const bool vec = (H % 4 == 0) && (S % 4 == 0) && (SP % 4 == 0);
    __syncthreads();

    // inputs of one step for this thread's element, fetched one step ahead of their use
    struct StepIn {
        float gate[4], ct, cPrev, gradOut;
        uint32_t bits;
    };
    auto fetch = [&](int t, StepIn &in) {
        if (!hasElem) return;
        const size_t row = static_cast<size_t>(t) * a.B + b0 + eb, so = row * H + ej, go = row * C + ej;
#pragma unroll
        for (int g = 0; g < 4; ++g) in.gate[g] = a.gateOutputs[go + static_cast<size_t>(g) * H];
        in.ct = a.cellTanh[so];
        in.cPrev = t > 0 ? a.cellStates[so - static_cast<size_t>(a.B) * H] : (a.c0 ? a.c0[stateIdx] : a.dqC.zeroPoint);
        in.gradOut = a.gradOutput[so];
        in.bits = a.stepMasks ? a.stepMasks[so] : 0u;
    };
    StepIn cur{}, nxt{};
    fetch(a.T - 1, cur);

    for (int t = a.T - 1; t >= 0; --t) {
        const size_t rowBase = static_cast<size_t>(t) * a.B + b0;
        if (t > 0) fetch(t - 1, nxt);
        if (hasElem) {
            const size_t row = rowBase + eb, go = row * C + ej;
            auto keepBit = [&](int b) { return (cur.bits >> b) & 1u ? 0.0f : 1.0f; };
            const float ig = realOf(cur.gate[0], a.dqGate[0]), fg = realOf(cur.gate[1], a.dqGate[1]);
            const float cg = realOf(cur.gate[2], a.dqGate[2]), og = realOf(cur.gate[3], a.dqGate[3]);
            const float ct = realOf(cur.ct, a.dqTanh);
            const float cPrev = realOf(cur.cPrev, a.dqC);
            const float incoming = dhCarry + partS[(0 * BT + eb) * H + ej] + partS[(1 * BT + eb) * H + ej] +
                                   partS[(2 * BT + eb) * H + ej] + partS[(3 * BT + eb) * H + ej];
            const float dh = (incoming + cur.gradOut) * keepBit(0);
            const float gOut = dh * ct;
            const float gTanh = dh * og * keepBit(1);
            const float dcAll = dc + gTanh * (1.0f - ct * ct);
            const float mdc = dcAll * keepBit(2);
            const float go4[4] = {mdc * cg * keepBit(3), mdc * cPrev * keepBit(4), mdc * ig * keepBit(5), gOut * keepBit(6)};
            const float gi4[4] = {go4[0] * ig * (1.0f - ig), go4[1] * fg * (1.0f - fg), go4[2] * (1.0f - cg * cg),
                                  go4[3] * og * (1.0f - og)};
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                const size_t o = go + static_cast<size_t>(g) * H;
                const float grad = gi4[g] * keepBit(7 + g);
                const float hh = grad * keepBit(15 + g);
                a.gIh[o] = grad * keepBit(11 + g);
                a.gHh[o] = hh;
                gS[eb * C + g * H + ej] = hh;
            }
            dc = mdc * fg;
            dhCarry = 0.0f;
        }
        cur = nxt;
        __syncthreads();
        if (hasColumn) {
            float acc[BT];
#pragma unroll
            for (int b = 0; b < BT; ++b) acc[b] = 0.0f;
            const float *wq = wS + (static_cast<size_t>(q) * H + cj) * SP;
            const float *gq = gS + q * H;
            if (vec) {
#pragma unroll 4
                for (int r = 0; r < S; r += 4) {
                    const float4 wv = *reinterpret_cast<const float4 *>(wq + r);
#pragma unroll
                    for (int b = 0; b < BT; ++b) {
                        const float4 gv = *reinterpret_cast<const float4 *>(gq + b * C + r);
                        acc[b] = fmaf(gv.x, wv.x, acc[b]);
                        acc[b] = fmaf(gv.y, wv.y, acc[b]);
                        acc[b] = fmaf(gv.z, wv.z, acc[b]);
                        acc[b] = fmaf(gv.w, wv.w, acc[b]);
                    }
                }
#pragma unroll
                for (int r = 0; r < kRegRows; r += 4) {
                    if (r < R) {
#pragma unroll
                        for (int b = 0; b < BT; ++b) {
                            const float4 gv = *reinterpret_cast<const float4 *>(gq + b * C + S + r);
                            acc[b] = fmaf(gv.x, wr[r], acc[b]);
                            acc[b] = fmaf(gv.y, wr[r + 1], acc[b]);
                            acc[b] = fmaf(gv.z, wr[r + 2], acc[b]);
                            acc[b] = fmaf(gv.w, wr[r + 3], acc[b]);
                        }
                    }
                }
            } else {
                for (int r = 0; r < S; ++r) {
                    const float w = wq[r];
#pragma unroll
                    for (int b = 0; b < BT; ++b) acc[b] = fmaf(gq[b * C + r], w, acc[b]);
                }
#pragma unroll
                for (int r = 0; r < kRegRows; ++r) {
                    if (r < R) {
#pragma unroll
                        for (int b = 0; b < BT; ++b) acc[b] = fmaf(gq[b * C + S + r], wr[r], acc[b]);
                    }
                }
            }
#pragma unroll
            for (int b = 0; b < BT; ++b) partS[(q * BT + b) * H + cj] = acc[b];
        }
        __syncthreads();
    }
    if (hasElem) {
        const float dh0 = dhCarry + partS[(0 * BT + eb) * H + ej] + partS[(1 * BT + eb) * H + ej] +
                          partS[(2 * BT + eb) * H + ej] + partS[(3 * BT + eb) * H + ej];
        a.dh0[stateIdx] = dh0 * keepOf(a.mk.initial_hidden, stateIdx);
        a.dc0[stateIdx] = dc * keepOf(a.mk.initial_cell, stateIdx);
    }
}

// ---- hidden sizes above 128 -------------------------------------------------------------------
//
// Thread (j, s) owns hidden unit j for RB batch rows of row group s: the pointwise derivative of its
// elements, then dh[b][j] = sum_c G_hh[b][c] * weight_hh[c][j] with column j of weight_hh streamed
// from L2 (coalesced over j) and the CTA's gate gradients read from shared memory as 16-byte
// broadcasts; dh and dc never leave the thread's registers.
template <int RB>
__global__ void __launch_bounds__(512, 1) recurrentBackwardWide(const __grid_constant__ RecurrentArgs a, const int HP) {
    const int H = a.H, C = 4 * a.H;
    extern __shared__ __align__(16) float smemF[];
    float *gS = smemF;  // [BT][C]
    const int tid = threadIdx.x, j = tid % HP, sg = tid / HP;
    const int BT = (blockDim.x / HP) * RB;
    const bool active = j < H;
    const int b0 = blockIdx.x * BT + sg * RB;
    for (int i = tid; i < BT * C; i += blockDim.x) gS[i] = 0.0f;
    float dhCarry[RB], dc[RB];
#pragma unroll
    for (int r = 0; r < RB; ++r) {
        const bool valid = active && b0 + r < a.B;
        const size_t stateIdx = static_cast<size_t>(b0 + r) * H + j;
        dhCarry[r] = valid ? a.gradFinalHidden[stateIdx] : 0.0f;
        dc[r] = valid ? a.gradFinalCell[stateIdx] : 0.0f;
    }
    __syncthreads();
    for (int t = a.T - 1; t >= 0; --t) {
        if (active) {
#pragma unroll
            for (int r = 0; r < RB; ++r) {
                const int b = b0 + r;
                if (b >= a.B) continue;
                const size_t row = static_cast<size_t>(t) * a.B + b, so = row * H + j, go = row * C + j;
                const size_t stateIdx = static_cast<size_t>(b) * H + j;
                const uint32_t bits = a.stepMasks ? a.stepMasks[so] : 0u;
                auto keepBit = [&](int bit) { return (bits >> bit) & 1u ? 0.0f : 1.0f; };
                const float ig = realOf(a.gateOutputs[go], a.dqGate[0]);
                const float fg = realOf(a.gateOutputs[go + static_cast<size_t>(H)], a.dqGate[1]);
                const float cg = realOf(a.gateOutputs[go + 2 * static_cast<size_t>(H)], a.dqGate[2]);
                const float og = realOf(a.gateOutputs[go + 3 * static_cast<size_t>(H)], a.dqGate[3]);
                const float ct = realOf(a.cellTanh[so], a.dqTanh);
                const float cPrevCode = t > 0 ? a.cellStates[so - static_cast<size_t>(a.B) * H]
                                              : (a.c0 ? a.c0[stateIdx] : a.dqC.zeroPoint);
                const float cPrev = realOf(cPrevCode, a.dqC);
                const float dh = (dhCarry[r] + a.gradOutput[so]) * keepBit(0);
                const float gOut = dh * ct;
                const float gTanh = dh * og * keepBit(1);
                const float dcAll = dc[r] + gTanh * (1.0f - ct * ct);
                const float mdc = dcAll * keepBit(2);
                const float go4[4] = {mdc * cg * keepBit(3), mdc * cPrev * keepBit(4), mdc * ig * keepBit(5), gOut * keepBit(6)};
                const float gi4[4] = {go4[0] * ig * (1.0f - ig), go4[1] * fg * (1.0f - fg), go4[2] * (1.0f - cg * cg),
                                      go4[3] * og * (1.0f - og)};
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const size_t o = go + static_cast<size_t>(g) * H;
                    const float grad = gi4[g] * keepBit(7 + g);
                    const float hh = grad * keepBit(15 + g);
                    a.gIh[o] = grad * keepBit(11 + g);
                    a.gHh[o] = hh;
                    gS[(sg * RB + r) * C + g * H + j] = hh;
                }
                dc[r] = mdc * fg;
            }
        }
        __syncthreads();
        if (active) {
            float acc[RB];
#pragma unroll
            for (int r = 0; r < RB; ++r) acc[r] = 0.0f;
            const float *wp = a.weightHh + j;
            const float *gRows = gS + sg * RB * C;
            for (int c = 0; c < C; c += 4) {  // C = 4H is a multiple of 4
                float w[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) w[i] = __ldg(wp + static_cast<size_t>(c + i) * H);
#pragma unroll
                for (int r = 0; r < RB; ++r) {
                    const float4 gv = *reinterpret_cast<const float4 *>(gRows + r * C + c);
                    acc[r] = fmaf(gv.x, w[0], acc[r]);
                    acc[r] = fmaf(gv.y, w[1], acc[r]);
                    acc[r] = fmaf(gv.z, w[2], acc[r]);
                    acc[r] = fmaf(gv.w, w[3], acc[r]);
                }
            }
#pragma unroll
            for (int r = 0; r < RB; ++r) dhCarry[r] = acc[r];
        }
        __syncthreads();
    }
    if (active) {
#pragma unroll
        for (int r = 0; r < RB; ++r) {
            if (b0 + r >= a.B) continue;
            const size_t stateIdx = static_cast<size_t>(b0 + r) * H + j;
            a.dh0[stateIdx] = dhCarry[r] * keepOf(a.mk.initial_hidden, stateIdx);
            a.dc0[stateIdx] = dc[r] * keepOf(a.mk.initial_cell, stateIdx);
        }
    }
}

// ---- dh = G_hh W_hh on tensor cores (QAT with weight grids of at most 8 bits) ------------------
//
// Same data flow as recurrentBackward, but the per-step product runs as mma.sync m16n8k16 with
// M = hidden column k, N = batch tile (padded to 8), K = the 4H channels.  Warp w owns two m16 tiles
// (hidden columns 32*(w/4) .. +31) and the K range of gate w%4; its A fragments - the integer weight
// codes, exact in bf16 - stay in registers for the whole sequence.  The gate gradient, multiplied by
// the channel's weight scale, is split into three bf16 terms in shared memory so that every product
// is exact and only the fp32 accumulation rounds.
__device__ __forceinline__ uint32_t packBf16(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ float bf16Lo(uint32_t v) { return __uint_as_float(v << 16); }

struct RecurrentMmaArgs {
    RecurrentArgs base;
    const float *weightCodes;   // q-carrier codes [4H][H]
    const float *channelScale;  // [4H] scale of weight_hh per channel
};

template <int HT, int BT>  // H = 32*HT, blockDim = 128*HT
__global__ void __launch_bounds__(128 * HT) recurrentBackwardMma(const __grid_constant__ RecurrentMmaArgs args) {
    const RecurrentArgs &a = args.base;
    constexpr int H = 32 * HT, C = 4 * H, KS = 2 * HT;  // k16 steps per warp
    constexpr int CP = C + 8;                           // padded row of the bf16 gradient tiles
    __shared__ __align__(16) uint16_t gB[3][8][CP];     // [split][batch row][channel]
    __shared__ float partS[4][BT][H];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nthreads = blockDim.x;
    const int g8 = lane >> 2, t4 = lane & 3;
    const int grp = warp % 4, mpair = warp / 4;
    const int b0 = blockIdx.x * BT, nb = min(BT, a.B - b0);

    // A fragments: element (m = hidden column, k = channel) = code[channel][hidden column]
    uint32_t afrag[2][KS][4];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int ks = 0; ks < KS; ++ks)
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int row = mpair * 32 + mt * 16 + g8 + (q & 1) * 8;
                const int col = grp * H + ks * 16 + 2 * t4 + (q >> 1) * 8;
                const float w0 = args.weightCodes[static_cast<size_t>(col) * H + row];
                const float w1 = args.weightCodes[static_cast<size_t>(col + 1) * H + row];
                afrag[mt][ks][q] = (__float_as_uint(w0) >> 16) | (__float_as_uint(w1) & 0xffff0000u);
            }
    for (int i = tid; i < 3 * 8 * CP; i += nthreads) (&gB[0][0][0])[i] = 0;
    for (int i = tid; i < 4 * BT * H; i += nthreads) (&partS[0][0][0])[i] = 0.0f;

    const int elems = nb * H;
    const bool hasElem = tid < elems;
    const int eb = hasElem ? tid / H : 0, ej = hasElem ? tid % H : 0;
    const size_t stateIdx = static_cast<size_t>(b0 + eb) * H + ej;
    float dhCarry = hasElem ? a.gradFinalHidden[stateIdx] : 0.0f;
    float dc = hasElem ? a.gradFinalCell[stateIdx] : 0.0f;
    float scale[4];
#pragma unroll
    for (int g = 0; g < 4; ++g) scale[g] = args.channelScale[g * H + ej];

    struct StepIn {
        float gate[4], ct, cPrev, gradOut;
        uint32_t bits;
    };
    auto fetch = [&](int t, StepIn &in) {
        if (!hasElem) return;
        const size_t row = static_cast<size_t>(t) * a.B + b0 + eb, so = row * H + ej, go = row * C + ej;
#pragma unroll
        for (int g = 0; g < 4; ++g) in.gate[g] = a.gateOutputs[go + static_cast<size_t>(g) * H];
        in.ct = a.cellTanh[so];
        in.cPrev = t > 0 ? a.cellStates[so - static_cast<size_t>(a.B) * H] : (a.c0 ? a.c0[stateIdx] : a.dqC.zeroPoint);
        in.gradOut = a.gradOutput[so];
        in.bits = a.stepMasks ? a.stepMasks[so] : 0u;
    };
    auto splitStore = [&](int b, int c, float v) {
        const float hi = bf16Lo(packBf16(v, 0.0f));
        const float r1 = v - hi;
        const float mid = bf16Lo(packBf16(r1, 0.0f));
        const float lo = r1 - mid;
        gB[0][b][c] = static_cast<uint16_t>(__float_as_uint(hi) >> 16);
        gB[1][b][c] = static_cast<uint16_t>(__float_as_uint(mid) >> 16);
        gB[2][b][c] = static_cast<uint16_t>(packBf16(lo, 0.0f) & 0xffffu);
    };
    StepIn cur{}, nxt{};
    fetch(a.T - 1, cur);
    __syncthreads();

    for (int t = a.T - 1; t >= 0; --t) {
        const size_t rowBase = static_cast<size_t>(t) * a.B + b0;
        if (t > 0) fetch(t - 1, nxt);
        if (hasElem) {
            const size_t row = rowBase + eb, go = row * C + ej;
            auto keepBit = [&](int b) { return (cur.bits >> b) & 1u ? 0.0f : 1.0f; };
            const float ig = realOf(cur.gate[0], a.dqGate[0]), fg = realOf(cur.gate[1], a.dqGate[1]);
            const float cg = realOf(cur.gate[2], a.dqGate[2]), og = realOf(cur.gate[3], a.dqGate[3]);
            const float ct = realOf(cur.ct, a.dqTanh);
            const float cPrev = realOf(cur.cPrev, a.dqC);
            const float incoming = dhCarry + partS[0][eb][ej] + partS[1][eb][ej] + partS[2][eb][ej] + partS[3][eb][ej];
            const float dh = (incoming + cur.gradOut) * keepBit(0);
            const float gOut = dh * ct;
            const float gTanh = dh * og * keepBit(1);
            const float dcAll = dc + gTanh * (1.0f - ct * ct);
            const float mdc = dcAll * keepBit(2);
            const float go4[4] = {mdc * cg * keepBit(3), mdc * cPrev * keepBit(4), mdc * ig * keepBit(5), gOut * keepBit(6)};
            const float gi4[4] = {go4[0] * ig * (1.0f - ig), go4[1] * fg * (1.0f - fg), go4[2] * (1.0f - cg * cg),
                                  go4[3] * og * (1.0f - og)};
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                const size_t o = go + static_cast<size_t>(g) * H;
                const float grad = gi4[g] * keepBit(7 + g);
                const float hh = grad * keepBit(15 + g);
                a.gIh[o] = grad * keepBit(11 + g);
                a.gHh[o] = hh;
                splitStore(eb, g * H + ej, hh * scale[g]);
            }
            dc = mdc * fg;
            dhCarry = 0.0f;
        }
        cur = nxt;
        __syncthreads();
        {
            float acc[2][3][4];
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int sp = 0; sp < 3; ++sp) acc[mt][sp][0] = acc[mt][sp][1] = acc[mt][sp][2] = acc[mt][sp][3] = 0.0f;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                const int c0 = grp * H + ks * 16 + 2 * t4;
#pragma unroll
                for (int sp = 0; sp < 3; ++sp) {
                    const uint32_t bf0 = *reinterpret_cast<const uint32_t *>(&gB[sp][g8][c0]);
                    const uint32_t bf1 = *reinterpret_cast<const uint32_t *>(&gB[sp][g8][c0 + 8]);
#pragma unroll
                    for (int mt = 0; mt < 2; ++mt) {
                        asm volatile(
                            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                            "{%0,%1,%2,%3};"
                            : "+f"(acc[mt][sp][0]), "+f"(acc[mt][sp][1]), "+f"(acc[mt][sp][2]), "+f"(acc[mt][sp][3])
                            : "r"(afrag[mt][ks][0]), "r"(afrag[mt][ks][1]), "r"(afrag[mt][ks][2]), "r"(afrag[mt][ks][3]),
                              "r"(bf0), "r"(bf1));
                    }
                }
            }
            // D fragment: rows g8 / g8+8 are hidden columns, columns 2*t4 / 2*t4+1 are batch rows
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int n = 2 * t4 + (q & 1);
                    const int k = mpair * 32 + mt * 16 + g8 + (q >> 1) * 8;
                    if (n < BT) partS[grp][n][k] = (acc[mt][2][q] + acc[mt][1][q]) + acc[mt][0][q];
                }
        }
        __syncthreads();
    }
    if (hasElem) {
        const float dh0 = dhCarry + partS[0][eb][ej] + partS[1][eb][ej] + partS[2][eb][ej] + partS[3][eb][ej];
        a.dh0[stateIdx] = dh0 * keepOf(a.mk.initial_hidden, stateIdx);
        a.dc0[stateIdx] = dc * keepOf(a.mk.initial_cell, stateIdx);
    }
}

// ---- hidden sizes above 128 on the tcgen05 tensor cores (QAT with weight grids of at most 8 bits) ---------
//
// dh[b][j] = sum_c G_hh[b][c] * code[c][j] * scale[c] needs every channel of a row for every hidden unit, and
// weight_hh (4H x H) fits no single SM.  The contraction is therefore split over the CTAs of a row tile:
//   * CTA (row tile of 128 batch rows, unit tile of 32 hidden units) owns the pointwise derivative of its
//     128 x 32 elements - which yields exactly the 128 channels (4 gates x 32 units) of G_hh that form ITS
//     K slice - and keeps rows [its 128 channels] x [all H units] of the weight codes in shared memory as an
//     exact bf16 operand (K-major canonical layout, loaded once);
//   * per step it writes the slice of G_hh, multiplied by the channel scale and split into three bf16 terms
//     (products exact, only the fp32 accumulation rounds), straight into the A operand tiles in shared memory
//     (nothing is exchanged for the product), one thread issues 3 x 8 MMAs (M 128, N H or 2 x H/2, K 16) per
//     accumulator half into tensor memory, and all warps move the [128][H] partial sums to a global array;
//   * the CTAs of a row tile then meet at a counter (cooperative launch, bounded polling) and the next step's
//     pointwise stage adds the H/32 partial sums of its elements in a fixed order (bit-reproducible).
// dc never leaves the registers of the thread that owns the element.  A wait that runs out sets the status
// word, ends all further waiting of the CTA and turns its dh0 into NaN.
constexpr int kBwdUnits = 32, kBwdRows = 128, kBwdSlice = 4 * kBwdUnits;
constexpr int kBwdSpinLimit = 1 << 22;
constexpr uint32_t kBwdSplitBytes = kBwdRows * kBwdSlice * 2;   // one bf16 term of the A operand

struct RecurrentUmmaArgs {
    RecurrentArgs base;
    const uint4 *tiles;          // [H / 32] weight tiles: [H / 8][16][8 units][8 channels] bf16
    const float *channelScale;   // [4H] scale of weight_hh per channel
    float *partial;              // [2][rowTiles][H / 32][128][H]
    unsigned int *counters;      // [rowTiles], zero at launch
    int *status;                 // set to 1 when a bounded wait gave up
    int rowBase, rowTiles;       // this launch covers batch rows [rowBase, rowBase + tileRows * rowTiles)
    int tileRows;                // batch rows of a row tile: 32, 64 or 128 (the accumulator tile always has 128 rows)
};

__global__ void packBackwardTiles(const float *__restrict__ codes, int H, uint4 *__restrict__ tiles) {
    const size_t total = static_cast<size_t>(H / kBwdUnits) * 16 * H;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int n = static_cast<int>(i % H), kg = static_cast<int>((i / H) % 16), ut = static_cast<int>(i / (static_cast<size_t>(16) * H));
        const int c0 = (kg / 4) * H + ut * kBwdUnits + (kg % 4) * 8;   // first of eight consecutive channels of one gate
        uint32_t v[4];
#pragma unroll
        for (int e = 0; e < 4; ++e)
            v[e] = umma::packBf16(codes[static_cast<size_t>(c0 + 2 * e) * H + n], codes[static_cast<size_t>(c0 + 2 * e + 1) * H + n]);
        tiles[static_cast<size_t>(ut) * (static_cast<size_t>(H) * 16) + static_cast<size_t>(n / 8) * 128 + kg * 8 + n % 8] =
            make_uint4(v[0], v[1], v[2], v[3]);
    }
}

__global__ void __launch_bounds__(512, 1) recurrentBackwardUmma(const __grid_constant__ RecurrentUmmaArgs args) {
    const RecurrentArgs &a = args.base;
    extern __shared__ __align__(128) uint8_t smemBwd[];
    __shared__ __align__(8) uint64_t bar;
    __shared__ uint32_t tmemSlot;
    __shared__ int failed;
    __shared__ __align__(16) float scaleS[kBwdSlice];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int H = a.H, C = 4 * H;
    const int tilesPerRow = H / kBwdUnits;
    const int ut = blockIdx.x % tilesPerRow, rt = blockIdx.x / tilesPerRow;
    // The product runs transposed: M = 128 hidden units per accumulator tile (weights as the A operand), N = the row
    // tile's batch rows (gate gradients as the B operand).  A row tile of 32 batch rows then costs an eighth of the
    // tensor time of 128-row accumulators, and an accumulator lane holds ONE unit's sums for neighbouring batch
    // rows, so that a warp's stores of a batch row are 128 contiguous bytes.
    const int unitTiles = H / 128, N = args.tileRows;
    uint32_t tmemCols = 32;
    while (tmemCols < static_cast<uint32_t>(unitTiles * N)) tmemCols *= 2;
    uint8_t *wTile = smemBwd;                                   // H x 128 bf16
    uint8_t *gTiles = smemBwd + static_cast<size_t>(H) * 256;   // 3 x [128 batch rows][128 channels] bf16 (the first N rows are used)
    volatile int *failFlag = &failed;

    if (tid == 0) {
        failed = 0;
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(umma::smemAddr(&bar)), "r"(H / 128) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(umma::smemAddr(&tmemSlot)), "r"(tmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    {
        const uint4 *src = args.tiles + static_cast<size_t>(ut) * (static_cast<size_t>(H) * 16);
        for (int i = tid; i < H * 16; i += blockDim.x) reinterpret_cast<uint4 *>(wTile)[i] = __ldg(src + i);
        if (tid < kBwdSlice) scaleS[tid] = args.channelScale[(tid / kBwdUnits) * H + ut * kBwdUnits + tid % kBwdUnits];
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmemSlot;

    // pointwise role: warp = four neighbouring batch rows (twice: rows 4 warp + {0, 64}), eight lanes per row, four
    // neighbouring units per lane, so that a warp's 16-byte loads cover whole 128-byte lines
    const int rowInPass = warp * 4 + (lane >> 3), j0 = ut * kBwdUnits + (lane & 7) * 4;
    const int ug = (lane & 7) >> 1, sub = lane & 1;   // eight-channel group of a gate, and which half of it
    // operand rows of batch rows beyond the batch hold whatever was there: they only reach accumulator columns that
    // nobody reads (column n of the product depends on row n of the B operand alone)
    struct RowSlot {
        int i, b;
        bool valid;
        size_t stateIdx;
        uint32_t aOffset;
    };
    auto slotOf = [&](int ps) {
        RowSlot rs;
        rs.i = ps * 64 + rowInPass;
        rs.b = args.rowBase + rt * args.tileRows + rs.i;
        rs.valid = rs.i < args.tileRows && rs.b < a.B;
        rs.stateIdx = static_cast<size_t>(rs.valid ? rs.b : 0) * H + j0;
        rs.aOffset = static_cast<uint32_t>(rs.i / 8) * 2048u + static_cast<uint32_t>(rs.i % 8) * 16u;
        return rs;
    };
    // epilogue role: accumulator tile warp / 4 (128 units), lanes 32 * (warp % 4) .. + 31: unit jOut
    const int outTile = warp >> 2, quarter = warp & 3, jOut = outTile * 128 + quarter * 32 + lane;
    const int rowsValid = max(0, min(N, a.B - (args.rowBase + rt * N)));   // batch rows of this row tile that exist
    const size_t partialTile = static_cast<size_t>(N) * H;                      // floats of one CTA's partial sums
    const size_t partialStep = static_cast<size_t>(args.rowTiles) * tilesPerRow * partialTile;
    const uint32_t idesc = umma::instructionDescriptor(N, false, false);
    const uint64_t descW0 = umma::operandDescriptor(umma::smemAddr(wTile), umma::kCore, 2048u);
    const uint64_t descG0 = umma::operandDescriptor(umma::smemAddr(gTiles), umma::kCore, 2048u);

    // dc of the thread's elements: [pass][unit]; the pass loop stays rolled (the kernel's code must stay small
    // enough for the instruction caches), so the two sets are picked by selects
    float dcA[4], dcB[4];
    {
        const RowSlot s0 = slotOf(0), s1 = slotOf(1);
        const float4 v0 = s0.valid ? *reinterpret_cast<const float4 *>(a.gradFinalCell + s0.stateIdx) : make_float4(0.f, 0.f, 0.f, 0.f);
        const float4 v1 = s1.valid ? *reinterpret_cast<const float4 *>(a.gradFinalCell + s1.stateIdx) : make_float4(0.f, 0.f, 0.f, 0.f);
        dcA[0] = v0.x; dcA[1] = v0.y; dcA[2] = v0.z; dcA[3] = v0.w;
        dcB[0] = v1.x; dcB[1] = v1.y; dcB[2] = v1.z; dcB[3] = v1.w;
    }
    // the carried gradient of four units: the final-state gradient before the last step, afterwards the sum of
    // the row tile's partial products of the step above
    auto carried = [&](int t, const RowSlot &rs) -> float4 {
        if (t == a.T - 1) return *reinterpret_cast<const float4 *>(a.gradFinalHidden + rs.stateIdx);
        const float *p = args.partial + static_cast<size_t>((t + 1) & 1) * partialStep + static_cast<size_t>(rt) * tilesPerRow * partialTile +
                         static_cast<size_t>(rs.i) * H + j0;
        // eight loads in flight at a time: a rolled loop would pay one L2 round trip per slice
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s0 = 0; s0 < tilesPerRow; s0 += 8) {
            float4 v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i)
                v[i] = s0 + i < tilesPerRow ? __ldcg(reinterpret_cast<const float4 *>(p + static_cast<size_t>(s0 + i) * partialTile))
                                            : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int i = 0; i < 8; ++i) { sum.x += v[i].x; sum.y += v[i].y; sum.z += v[i].z; sum.w += v[i].w; }
        }
        return sum;
    };
    auto groupBarrier = [&](int stepsDone) {
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            __threadfence();   // cumulative: what the other threads wrote before the barrier is ordered before the arrival
            atomicAdd(args.counters + rt, 1u);
            const unsigned int want = static_cast<unsigned int>(tilesPerRow) * stepsDone;
            bool arrived = *failFlag != 0;
            for (int spin = 0; !arrived && spin < kBwdSpinLimit; ++spin) {
                unsigned int seen;
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(args.counters + rt) : "memory");
                arrived = seen >= want;
            }
            if (!arrived) *failFlag = 1;
        }
        __syncthreads();
        __threadfence();
    };

    uint32_t parity = 0;
    int stepsDone = 0;
    for (int t = a.T - 1; t >= 0; --t) {
        // ---- pointwise derivative of this thread's eight elements, four at a time
#pragma unroll 1
        for (int ps = 0; ps < 2; ++ps) {
            const RowSlot rs = slotOf(ps);
            if (rs.valid) {
                float dc[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) dc[e] = ps ? dcB[e] : dcA[e];
                const size_t row = static_cast<size_t>(t) * a.B + rs.b;
                const size_t so = row * H + j0, go = row * C + j0;
                const float4 dhIn = carried(t, rs);
                const uint4 bits4 = a.stepMasks ? *reinterpret_cast<const uint4 *>(a.stepMasks + so) : make_uint4(0u, 0u, 0u, 0u);
                const float4 gi = *reinterpret_cast<const float4 *>(a.gateOutputs + go);
                const float4 gf = *reinterpret_cast<const float4 *>(a.gateOutputs + go + static_cast<size_t>(H));
                const float4 gc = *reinterpret_cast<const float4 *>(a.gateOutputs + go + 2 * static_cast<size_t>(H));
                const float4 gq = *reinterpret_cast<const float4 *>(a.gateOutputs + go + 3 * static_cast<size_t>(H));
                const float4 ct4 = *reinterpret_cast<const float4 *>(a.cellTanh + so);
                const float4 gradOut = *reinterpret_cast<const float4 *>(a.gradOutput + so);
                float4 cp4;
                if (t > 0) cp4 = *reinterpret_cast<const float4 *>(a.cellStates + so - static_cast<size_t>(a.B) * H);
                else if (a.c0) cp4 = *reinterpret_cast<const float4 *>(a.c0 + rs.stateIdx);
                else cp4 = make_float4(a.dqC.zeroPoint, a.dqC.zeroPoint, a.dqC.zeroPoint, a.dqC.zeroPoint);
                const float dhv[4] = {dhIn.x, dhIn.y, dhIn.z, dhIn.w};
                const uint32_t bitv[4] = {bits4.x, bits4.y, bits4.z, bits4.w};
                const float igv[4] = {gi.x, gi.y, gi.z, gi.w}, fgv[4] = {gf.x, gf.y, gf.z, gf.w};
                const float cgv[4] = {gc.x, gc.y, gc.z, gc.w}, ogv[4] = {gq.x, gq.y, gq.z, gq.w};
                const float ctv[4] = {ct4.x, ct4.y, ct4.z, ct4.w}, gov[4] = {gradOut.x, gradOut.y, gradOut.z, gradOut.w};
                const float cpv[4] = {cp4.x, cp4.y, cp4.z, cp4.w};
                float outIh[4][4], outHh[4][4];   // [gate][unit]
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const uint32_t bits = bitv[e];
                    auto keepBit = [&](int bit) { return (bits >> bit) & 1u ? 0.0f : 1.0f; };
                    const float ig = realOf(igv[e], a.dqGate[0]), fg = realOf(fgv[e], a.dqGate[1]);
                    const float cg = realOf(cgv[e], a.dqGate[2]), og = realOf(ogv[e], a.dqGate[3]);
                    const float ct = realOf(ctv[e], a.dqTanh), cPrev = realOf(cpv[e], a.dqC);
                    const float dh = (dhv[e] + gov[e]) * keepBit(0);
                    const float gOut = dh * ct;
                    const float gTanh = dh * og * keepBit(1);
                    const float dcAll = dc[e] + gTanh * (1.0f - ct * ct);
                    const float mdc = dcAll * keepBit(2);
                    const float go4[4] = {mdc * cg * keepBit(3), mdc * cPrev * keepBit(4), mdc * ig * keepBit(5), gOut * keepBit(6)};
                    const float gi4[4] = {go4[0] * ig * (1.0f - ig), go4[1] * fg * (1.0f - fg), go4[2] * (1.0f - cg * cg),
                                          go4[3] * og * (1.0f - og)};
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        const float grad = gi4[g] * keepBit(7 + g);
                        outIh[g][e] = grad * keepBit(11 + g);
                        outHh[g][e] = grad * keepBit(15 + g);
                    }
                    dc[e] = mdc * fg;
                }
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const size_t o = go + static_cast<size_t>(g) * H;
                    *reinterpret_cast<float4 *>(a.gIh + o) = make_float4(outIh[g][0], outIh[g][1], outIh[g][2], outIh[g][3]);
                    *reinterpret_cast<float4 *>(a.gHh + o) = make_float4(outHh[g][0], outHh[g][1], outHh[g][2], outHh[g][3]);
                    // scaled by the channel's weight scale and split into three bf16 terms: channels g*32 + 4*(lane%8) ..
                    const float4 sc = *reinterpret_cast<const float4 *>(scaleS + g * kBwdUnits + (lane & 7) * 4);
                    const float v[4] = {outHh[g][0] * sc.x, outHh[g][1] * sc.y, outHh[g][2] * sc.z, outHh[g][3] * sc.w};
                    uint32_t hi2[2], mid2[2], lo2[2];
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        hi2[i] = packBf16(v[2 * i], v[2 * i + 1]);
                        const float r0 = v[2 * i] - bf16Lo(hi2[i]), r1 = v[2 * i + 1] - umma::bf16Hi(hi2[i]);
                        mid2[i] = packBf16(r0, r1);
                        lo2[i] = packBf16(r0 - bf16Lo(mid2[i]), r1 - umma::bf16Hi(mid2[i]));
                    }
                    uint8_t *dst = gTiles + rs.aOffset + static_cast<uint32_t>(g * 4 + ug) * umma::kCore + 8u * sub;
                    *reinterpret_cast<uint2 *>(dst) = make_uint2(hi2[0], hi2[1]);
                    *reinterpret_cast<uint2 *>(dst + kBwdSplitBytes) = make_uint2(mid2[0], mid2[1]);
                    *reinterpret_cast<uint2 *>(dst + 2 * kBwdSplitBytes) = make_uint2(lo2[0], lo2[1]);
                }
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    dcA[e] = ps ? dcA[e] : dc[e];
                    dcB[e] = ps ? dc[e] : dcB[e];
                }
            }
        }
        // the saved tensors of the step below come from HBM: ask their lines into L2 now, one lane per 128-byte line
        if (t > 0 && (lane & 7) == 0) {
#pragma unroll 1
            for (int ps = 0; ps < 2; ++ps) {
                const RowSlot rs = slotOf(ps);
                if (!rs.valid) continue;
                const size_t row = static_cast<size_t>(t - 1) * a.B + rs.b;
                const size_t so = row * H + ut * kBwdUnits, go = row * C + ut * kBwdUnits;
                if (a.stepMasks) prefetchL2(a.stepMasks + so);
#pragma unroll
                for (int g = 0; g < 4; ++g) prefetchL2(a.gateOutputs + go + static_cast<size_t>(g) * H);
                prefetchL2(a.cellTanh + so);
                prefetchL2(a.gradOutput + so);
                if (t > 1) prefetchL2(a.cellStates + so - static_cast<size_t>(a.B) * H);
            }
        }
        // ---- dh partial sums of this K slice: [128 rows][H units] into tensor memory
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        // One thread per accumulator tile issues that tile's MMAs (a single issuer spends more time on descriptor
        // arithmetic than the tensor pipe needs for N = 32); its lane siblings wait at the warp barrier instead of
        // polling beside it.  Each issuer commits to the same barrier (initialised to the number of tiles).
        if (warp < unitTiles) {
            if (lane == 0) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d = tmem + static_cast<uint32_t>(warp * N);
                const uint64_t w0 = descW0 + static_cast<uint64_t>(warp) * ((16u * 2048u) >> 4);
#pragma unroll
                for (int sp = 0; sp < 3; ++sp)
#pragma unroll
                    for (int ks = 0; ks < kBwdSlice / 16; ++ks)
                        umma::mmaBf16(d, w0 + static_cast<uint64_t>(ks * 16), descG0 + static_cast<uint64_t>(sp * (kBwdSplitBytes >> 4) + ks * 16), idesc,
                                      (sp | ks) ? 1u : 0u);
                umma::commitTo(umma::smemAddr(&bar));
            }
            __syncwarp();
        }
        if (!*failFlag && !umma::waitPhase(umma::smemAddr(&bar), parity)) *failFlag = 1;
        parity ^= 1u;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (outTile < unitTiles) {
            float *dst = args.partial + static_cast<size_t>(t & 1) * partialStep + (static_cast<size_t>(rt) * tilesPerRow + ut) * partialTile + jOut;
            for (int c = 0; c < rowsValid; c += 32) {
                uint32_t v[32];
                umma::tmemLoad32(tmem + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(outTile * N + c), v);
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (c + i < rowsValid) __stcg(dst + static_cast<size_t>(c + i) * H, __uint_as_float(v[i]));
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        // ---- publish the step and wait for the other K slices of this row tile
        ++stepsDone;
        groupBarrier(stepsDone);
    }
#pragma unroll 1
    for (int ps = 0; ps < 2; ++ps) {
        const RowSlot rs = slotOf(ps);
        if (!rs.valid) continue;
        const float nan = __int_as_float(0x7fc00000);
        const float4 dh0 = *failFlag ? make_float4(nan, nan, nan, nan) : carried(-1, rs);
        const float out[4] = {dh0.x, dh0.y, dh0.z, dh0.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const size_t o = rs.stateIdx + e;
            a.dh0[o] = out[e] * keepOf(a.mk.initial_hidden, o);
            a.dc0[o] = (ps ? dcB[e] : dcA[e]) * keepOf(a.mk.initial_cell, o);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tmemCols) : "memory");
    if (tid == 0 && failed && args.status) atomicExch(args.status, 1);
}

// Rows of a [rows, cols] operand that switches source after `split` rows (h_prev = [h0 ; hidden[0..T-2]]).
struct RowSource {
    const float *first;  // rows [0, split) ; null = zeros
    const float *rest;   // rows [split, ...) start here
    int split;
    Dequant dq;
    __device__ __forceinline__ float at(int row, int col, int cols) const {
        if (row < split) return first ? realOf(first[static_cast<size_t>(row) * cols + col], dq) : 0.0f;
        return realOf(rest[static_cast<size_t>(row - split) * cols + col], dq);
    }
};

constexpr int kTile = 64, kDepth = 16;

// partial[s][m][n] = sum over the s-th chunk of rows k of G[k][m] * X[k][n].
__global__ void __launch_bounds__(256) gemmRowsTN(const float *__restrict__ G, const RowSource X, int K, int M, int N,
                                                  int chunk, float *__restrict__ partial) {
    __shared__ float As[kDepth][kTile + 4];
    __shared__ float Bs[kDepth][kTile + 4];
    const int m0 = blockIdx.y * kTile, n0 = blockIdx.x * kTile;
    const int kBegin = blockIdx.z * chunk, kEnd = min(K, kBegin + chunk);
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    float acc[4][4] = {};
    for (int k0 = kBegin; k0 < kEnd; k0 += kDepth) {
        for (int i = threadIdx.x; i < kDepth * kTile; i += 256) {
            const int kk = i / kTile, c = i % kTile, k = k0 + kk;
            As[kk][c] = (k < kEnd && m0 + c < M) ? G[static_cast<size_t>(k) * M + m0 + c] : 0.0f;
            Bs[kk][c] = (k < kEnd && n0 + c < N) ? X.at(k, n0 + c, N) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kDepth; ++kk) {
            float av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { av[i] = As[kk][ty * 4 + i]; bv[i] = Bs[kk][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
    float *out = partial + static_cast<size_t>(blockIdx.z) * M * N;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
            if (m < M && n < N) out[static_cast<size_t>(m) * N + n] = acc[i][j];
        }
}

// out[i] = keep[i] * sum_s partial[s][i], s ascending.
__global__ void reduceSplits(const float *__restrict__ partial, int splits, size_t n, const uint8_t *__restrict__ mask,
                             float *__restrict__ out) {
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float s = 0.0f;
        for (int p = 0; p < splits; ++p) s += partial[static_cast<size_t>(p) * n + i];
        out[i] = s * keepOf(mask, i);
    }
}

// out[m][n] = keep * sum_k A[m][k] * W[k][n]   (dx = G_ih W_ih: M = T*B, K = 4H, N = I).
__global__ void __launch_bounds__(256) gemmNN(const float *__restrict__ A, const float *__restrict__ W, int M, int N, int K,
                                              const uint8_t *__restrict__ mask, float *__restrict__ out) {
    __shared__ float As[kDepth][kTile + 1];
    __shared__ float Ws[kDepth][kTile + 4];
    const int m0 = blockIdx.x * kTile, n0 = blockIdx.y * kTile;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += kDepth) {
        for (int i = threadIdx.x; i < kTile * kDepth; i += 256) {
            const int r = i / kDepth, kk = i % kDepth;
            As[kk][r] = (m0 + r < M && k0 + kk < K) ? A[static_cast<size_t>(m0 + r) * K + k0 + kk] : 0.0f;
            const int wk = i / kTile, wc = i % kTile;
            Ws[wk][wc] = (k0 + wk < K && n0 + wc < N) ? W[static_cast<size_t>(k0 + wk) * N + n0 + wc] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kDepth; ++kk) {
            float av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { av[i] = As[kk][ty * 4 + i]; bv[i] = Ws[kk][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
            if (m < M && n < N) {
                const size_t o = static_cast<size_t>(m) * N + n;
                out[o] = acc[i][j] * keepOf(mask, o);
            }
        }
}

// weight[c][m] = scale * keep * sum_s partial[s][m][c] (m < M); bias[c] = keep * sum_s partial[s][M][c]:
// reduces the split-K partials of the tensor-core GEMM and writes the transposed [4H][M] layout.
// A CTA owns 32 channels x 8 rows; its four thread layers each sum every fourth split, and layer 0
// adds the four sums in layer order, so the result does not depend on the launch.
// A set status word (a bounded wait of the producing kernel gave up) turns the results into NaN.
// One launch reduces both problems of a step (blockIdx.z: 0 = weight_ih, 1 = weight_hh).
constexpr int kReduceLayers = 4, kReduceRows = 8;
struct ReduceJob {
    const float *partial;
    int splits, M;
    float scale;
    const uint8_t *weightMask, *biasMask;
    float *weight, *bias;
};
__global__ void __launch_bounds__(32 * kReduceRows * kReduceLayers)
reduceWeightGradT(const ReduceJob jobIh, const ReduceJob jobHh, int C, const int *__restrict__ status) {
    __shared__ float layer[kReduceLayers][kReduceRows][32];
    const ReduceJob &job = blockIdx.z == 0 ? jobIh : jobHh;
    const float *__restrict__ partial = job.partial;
    const int splits = job.splits, M = job.M;
    const float scale = job.scale;
    const uint8_t *__restrict__ weightMask = job.weightMask, *__restrict__ biasMask = job.biasMask;
    float *__restrict__ weight = job.weight, *__restrict__ bias = job.bias;
    if (static_cast<int>(blockIdx.y) * kReduceRows > M) return;  // the other problem has more rows
    const size_t slab = static_cast<size_t>(M + 1) * C;
    const int c = blockIdx.x * 32 + threadIdx.x, m = blockIdx.y * kReduceRows + threadIdx.y;
    const bool inside = m <= M && c < C;
    float s = 0.0f;
    if (inside) {
        const float *src = partial + static_cast<size_t>(m) * C + c;
#pragma unroll 4
        for (int sp = threadIdx.z; sp < splits; sp += kReduceLayers) s += src[static_cast<size_t>(sp) * slab];
    }
    layer[threadIdx.z][threadIdx.y][threadIdx.x] = s;
    __syncthreads();
    if (threadIdx.z != 0 || !inside) return;
    s = layer[0][threadIdx.y][threadIdx.x];
#pragma unroll
    for (int l = 1; l < kReduceLayers; ++l) s += layer[l][threadIdx.y][threadIdx.x];
    if (status && *status) s = __int_as_float(0x7fc00000);
    if (m < M) {
        const size_t o = static_cast<size_t>(c) * M + m;
        weight[o] = s * scale * keepOf(weightMask, o);
    } else if (bias) {
        bias[c] = s * keepOf(biasMask, c);
    }
}

// dx = G_ih W_ih for a narrow N (= input size <= 128): a CTA owns 64 rows, thread (row, quarter) keeps
// NO consecutive outputs in registers and walks K in chunks of 32 staged in shared memory (the G chunk
// transposed so that neighbouring rows read neighbouring banks, the W chunk read as warp-wide
// broadcasts).  The 64x64-tile kernel above wastes a third of its tile at N = 40.
constexpr int kDxRows = 64, kDxChunk = 32;
template <int NO>
__global__ void __launch_bounds__(256) inputGradNarrow(const float *__restrict__ G, const float *__restrict__ W, int M, int N,
                                                       int K, const uint8_t *__restrict__ mask, float *__restrict__ out) {
    __shared__ float Gs[kDxChunk][kDxRows + 1];
    __shared__ __align__(16) float Ws[kDxChunk][4 * NO];
    const int tid = threadIdx.x, r = tid % kDxRows, p = tid / kDxRows;
    const int row0 = blockIdx.x * kDxRows;
    float acc[NO];
#pragma unroll
    for (int i = 0; i < NO; ++i) acc[i] = 0.0f;
    for (int k0 = 0; k0 < K; k0 += kDxChunk) {
#pragma unroll
        for (int v = 0; v < 2; ++v) {
            const int lr = tid / 8 + v * 32, c4 = (tid % 8) * 4;
            float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
            if (row0 + lr < M && k0 + c4 < K) g = *reinterpret_cast<const float4 *>(G + static_cast<size_t>(row0 + lr) * K + k0 + c4);
            Gs[c4][lr] = g.x; Gs[c4 + 1][lr] = g.y; Gs[c4 + 2][lr] = g.z; Gs[c4 + 3][lr] = g.w;
        }
        for (int i = tid; i < kDxChunk * 4 * NO; i += 256) {
            const int kk = i / (4 * NO), n = i % (4 * NO);
            Ws[kk][n] = (k0 + kk < K && n < N) ? W[static_cast<size_t>(k0 + kk) * N + n] : 0.0f;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < kDxChunk; ++kk) {
            const float g = Gs[kk][r];
#pragma unroll
            for (int i4 = 0; i4 < NO / 4; ++i4) {
                const float4 w = *reinterpret_cast<const float4 *>(&Ws[kk][p * NO + i4 * 4]);
                acc[i4 * 4 + 0] = fmaf(g, w.x, acc[i4 * 4 + 0]);
                acc[i4 * 4 + 1] = fmaf(g, w.y, acc[i4 * 4 + 1]);
                acc[i4 * 4 + 2] = fmaf(g, w.z, acc[i4 * 4 + 2]);
                acc[i4 * 4 + 3] = fmaf(g, w.w, acc[i4 * 4 + 3]);
            }
        }
        __syncthreads();
    }
    const int row = row0 + r;
    if (row >= M) return;
#pragma unroll
    for (int i = 0; i < NO; ++i) {
        const int n = p * NO + i;
        if (n < N) {
            const size_t o = static_cast<size_t>(row) * N + n;
            out[o] = acc[i] * keepOf(mask, o);
        }
    }
}

// partial[which][s][c] = sum over the s-th chunk of rows of g[n][c]; blockIdx.y selects G_ih or G_hh.
__global__ void columnSums(const float *__restrict__ gIh, const float *__restrict__ gHh, int rows, int C, int chunk,
                           float *__restrict__ partial) {
    const float *g = blockIdx.y == 0 ? gIh : gHh;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int n0 = blockIdx.z * chunk, n1 = min(rows, n0 + chunk);
    float s = 0.0f;
    for (int n = n0; n < n1; ++n) s += g[static_cast<size_t>(n) * C + c];
    partial[(static_cast<size_t>(blockIdx.y) * gridDim.z + blockIdx.z) * C + c] = s;
}

int gridFor(size_t n, int block) { return static_cast<int>(std::min<size_t>((n + block - 1) / block, 148 * 8)); }

int splitsFor(int K, int tiles) {
    const int want = std::max(1, (2 * 148 + tiles - 1) / tiles);
    return std::max(1, std::min(want, (K + 255) / 256));
}
int tilesOf(int M, int N) { return ((M + kTile - 1) / kTile) * ((N + kTile - 1) / kTile); }

constexpr int kBiasSplits = 64;
constexpr int kMaxTensorSplits = 40;

}  // namespace

// The tcgen05 recurrence of wide layers takes hidden sizes whose accumulator quarters are whole 32-column pieces.
bool wideTensorShape(int H) { return H > 128 && H <= 512 && H % 128 == 0; }
// Row tiles (128 batch rows) one cooperative launch holds: every CTA must be resident, one per SM.
int wideTensorRowTiles(int B, int H) {
    const int tilesPerRow = H / kBwdUnits;
    return std::max(1, std::min((B + kBwdRows - 1) / kBwdRows, std::max(1, 148 / tilesPerRow)));
}

// Splits of the tensor-core weight-gradient partial arrays: the one-tile plan for at most 128 rows, the slab plan
// (128-row slabs of both problems in one launch) beyond.
int tensorSplitBound(int rows, int I, int H, int M, int C) {
    const int single = M <= 143 ? wgrad::splitBound(rows, M, C) : 1;
    return std::max(single, wgrad::slabPathTakes(I, H, C) ? wgrad::slabSplitBound(I, H, C) : 1);
}

size_t backwardWorkspaceBytes(int T, int B, int I, int H) {
    const size_t rows = static_cast<size_t>(T) * B, C = 4 * static_cast<size_t>(H);
    WorkspaceSizer ws;
    ws.take<float>(rows * C);  // G_ih
    ws.take<float>(rows * C);  // G_hh
    ws.take<float>(C * I);     // real weight_ih (QAT)
    ws.take<float>(C * H);     // real weight_hh (QAT)
    ws.take<float>(static_cast<size_t>(splitsFor(static_cast<int>(rows), tilesOf(static_cast<int>(C), I))) * C * I);
    ws.take<float>(static_cast<size_t>(splitsFor(static_cast<int>(rows), tilesOf(static_cast<int>(C), H))) * C * H);
    ws.take<float>(2 * kBiasSplits * C);
    ws.take<float>(2 * C);     // per-channel weight scales (QAT)
    ws.take<float>(rows * H);  // h_prev codes for the tensor-core weight gradient (QAT)
    ws.take<float>(static_cast<size_t>(tensorSplitBound(static_cast<int>(rows), I, H, I, static_cast<int>(C))) * (I + 1) * C);
    ws.take<float>(static_cast<size_t>(tensorSplitBound(static_cast<int>(rows), I, H, H, static_cast<int>(C))) * (H + 1) * C);
    ws.take<int>(1);              // status word of the tensor-memory weight-gradient kernel
    ws.take<uint32_t>(rows * H);  // packed per-step clamp flags
    ws.take<uint8_t>(igrad::widePackedBytes(static_cast<int>(C), I) + 256);   // weight operand of the streaming input-gradient kernel
    if (wideTensorShape(H)) {   // tensor-core recurrence of wide layers: weight tiles, partial sums, counters
        ws.take<uint4>(C * H / 8);
        ws.take<float>(2 * static_cast<size_t>(wideTensorRowTiles(B, H)) * (H / kBwdUnits) * kBwdRows * H);
        ws.take<unsigned int>(256);
    }
    return ws.used() + 1024;
}

void backward(const BackwardCall &call, void *workspace, size_t workspaceBytes, cudaStream_t st) {
    const int T = call.T, B = call.B, I = call.I, H = call.H, C = 4 * H;
    if (H > 512) fail(RXMET_ERR_UNSUPPORTED, "hidden sizes up to 512 are built (got %d)", H);
    const bool wide = C > 512;
    const size_t rows = static_cast<size_t>(T) * B;
    Workspace ws(workspace, workspaceBytes);
    float *gIh = ws.take<float>(rows * C);
    float *gHh = ws.take<float>(rows * C);
    float *wIhReal = ws.take<float>(static_cast<size_t>(C) * I);
    float *wHhReal = ws.take<float>(static_cast<size_t>(C) * H);
    const int splitIh = splitsFor(static_cast<int>(rows), tilesOf(C, I));
    const int splitHh = splitsFor(static_cast<int>(rows), tilesOf(C, H));
    float *partIh = ws.take<float>(static_cast<size_t>(splitIh) * C * I);
    float *partHh = ws.take<float>(static_cast<size_t>(splitHh) * C * H);
    float *partBias = ws.take<float>(2 * kBiasSplits * static_cast<size_t>(C));
    float *channelScales = ws.take<float>(2 * static_cast<size_t>(C));
    float *hPrev = ws.take<float>(rows * H);
    float *tensorIh = ws.take<float>(static_cast<size_t>(tensorSplitBound(static_cast<int>(rows), I, H, I, C)) * (I + 1) * C);
    float *tensorHh = ws.take<float>(static_cast<size_t>(tensorSplitBound(static_cast<int>(rows), I, H, H, C)) * (H + 1) * C);
    int *tensorStatus = ws.take<int>(1);
    uint32_t *stepMasks = ws.take<uint32_t>(rows * H);

    // Which kernels multiply by the saved integer weight codes directly (QAT on 8-bit grids); the
    // others read real-valued weights rebuilt here.
    const bool tensorPath = !wide && call.quantized && call.weightCodesFitBf16 && H % 32 == 0 && H <= 128 &&
                            std::getenv("RXMET_LSTM_BWD_SIMT") == nullptr;
    // Wide layers: the tcgen05 recurrence (float4 loads of the saved tensors and of the incoming gradients)
    uint4 *wideTiles = nullptr;
    float *widePartial = nullptr;
    unsigned int *wideCounters = nullptr;
    if (wideTensorShape(H)) {
        wideTiles = ws.take<uint4>(static_cast<size_t>(C) * H / 8);
        widePartial = ws.take<float>(2 * static_cast<size_t>(wideTensorRowTiles(B, H)) * (H / kBwdUnits) * kBwdRows * H);
        wideCounters = ws.take<unsigned int>(256);
    }
    const size_t wideSmem = static_cast<size_t>(H) * 256 + 3 * kBwdSplitBytes;
    int cooperative = 0;
    RXMET_CUDA(cudaDeviceGetAttribute(&cooperative, cudaDevAttrCooperativeLaunch, currentDevice().device));
    const bool wideTensor = wide && wideTensorShape(H) && call.quantized && call.weightCodesFitBf16 && cooperative != 0 &&
                            H / kBwdUnits <= smsPerPass() && wideSmem <= static_cast<size_t>(currentDevice().smemMax) &&
                            alignedTo(call.gateOutputs, 16) && alignedTo(call.cellStates, 16) && alignedTo(call.cellTanhOutputs, 16) &&
                            alignedTo(call.gradOutput, 16) && alignedTo(call.gradFinalHidden, 16) && alignedTo(call.gradFinalCell, 16) &&
                            alignedTo(call.c0, 16) && std::getenv("RXMET_LSTM_BWD_SIMT") == nullptr;
    // 16-byte copies of the caller's weight codes, float4 stores of dx and 8-byte loads of the input mask
    const bool tensorInputGrad = call.quantized && call.weightIhCodesFitBf16 && igrad::eligible(C, I) &&
                                 alignedTo(call.grads.input, 16) && alignedTo(call.weightIh, 16) &&
                                 (call.masks == nullptr || alignedTo(call.masks->input, 8));
    const float *wIh = call.weightIh, *wHh = call.weightHh;
    if (call.quantized) {
        RXMET_REQUIRE(call.weightIhScale && call.weightHhScale, "per-channel weight scales missing");
        RXMET_CUDA(cudaMemcpyAsync(channelScales, call.weightIhScale, sizeof(float) * C, cudaMemcpyHostToDevice, st));
        RXMET_CUDA(cudaMemcpyAsync(channelScales + C, call.weightHhScale, sizeof(float) * C, cudaMemcpyHostToDevice, st));
        if (!tensorInputGrad) {
            KernelTimer timer__("lstmDequantWeights", st);
            dequantWeights<<<gridFor(static_cast<size_t>(C) * I, 256), 256, 0, st>>>(call.weightIh, channelScales, C, I, wIhReal);
            afterLaunch("lstmDequantWeights");
        }
        if (!tensorPath && !wideTensor) {
            KernelTimer timer__("lstmDequantWeights", st);
            dequantWeights<<<gridFor(static_cast<size_t>(C) * H, 256), 256, 0, st>>>(call.weightHh, channelScales + C, C, H, wHhReal);
            afterLaunch("lstmDequantWeights");
        }
        wIh = wIhReal;
        wHh = wHhReal;
    }
    const rxmet_lstm_backward_masks none{};
    const rxmet_lstm_backward_masks &mk = call.masks ? *call.masks : none;
    const bool anyStepMask = mk.hidden_outputs || mk.cell_tanh_outputs || mk.cell_states || mk.gate_outputs ||
                             mk.gate_inputs || mk.weight_ih_linear || mk.weight_hh_linear;
    if (anyStepMask) {
        {
            KernelTimer timer__("lstmPackStepMasks", st);
            auto aligned4 = [](const void *ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 3u) == 0; };
            if (H % 4 == 0 && aligned4(mk.hidden_outputs) && aligned4(mk.cell_tanh_outputs) && aligned4(mk.cell_states) &&
                aligned4(mk.gate_outputs) && aligned4(mk.gate_inputs) && aligned4(mk.weight_ih_linear) &&
                aligned4(mk.weight_hh_linear))
                packStepMasks4<<<gridFor(rows * H / 4, 256), 256, 0, st>>>(mk, rows * H / 4, H, reinterpret_cast<uint4 *>(stepMasks));
            else
                packStepMasks<<<gridFor(rows * H, 256), 256, 0, st>>>(mk, rows, H, stepMasks);
        }
        afterLaunch("lstmPackStepMasks");
    }
    {
        RecurrentArgs a{};
        a.T = T; a.B = B; a.H = H;
        a.stepMasks = anyStepMask ? stepMasks : nullptr;
        a.weightHh = wHh; a.c0 = call.c0;
        a.gateOutputs = call.gateOutputs; a.cellStates = call.cellStates; a.cellTanh = call.cellTanhOutputs;
        a.gradOutput = call.gradOutput; a.gradFinalHidden = call.gradFinalHidden; a.gradFinalCell = call.gradFinalCell;
        a.dqC = call.dqC; a.dqTanh = call.dqTanh;
        for (int g = 0; g < 4; ++g) a.dqGate[g] = call.dqGate[g];
        a.mk = mk; a.gIh = gIh; a.gHh = gHh; a.dh0 = call.grads.initial_hidden; a.dc0 = call.grads.initial_cell;
        const int smemMax = currentDevice().smemMax, sms = currentDevice().sms;
        const int bt = (B >= 4 * sms) ? 4 : ((B > sms) ? 2 : 1);
        const int block = (C + 31) / 32 * 32;
        if (tensorPath) {
            RecurrentMmaArgs m{};
            m.base = a;
            m.weightCodes = call.weightHh;  // q-carrier codes as saved by the forward
            m.channelScale = channelScales + C;
            bool launched = false;
#define RXMET_LSTM_MMA(HTV, BTV)                                                     \
    if (!launched && H == 32 * HTV && bt == BTV) {                                    \
        KernelTimer timer__("lstmRecurrentBackwardMma", st);                         \
        recurrentBackwardMma<HTV, BTV><<<(B + BTV - 1) / BTV, 128 * HTV, 0, st>>>(m); \
        launched = true;                                                              \
    }
            RXMET_LSTM_MMA(1, 1) RXMET_LSTM_MMA(1, 2) RXMET_LSTM_MMA(1, 4)
            RXMET_LSTM_MMA(2, 1) RXMET_LSTM_MMA(2, 2) RXMET_LSTM_MMA(2, 4)
            RXMET_LSTM_MMA(3, 1) RXMET_LSTM_MMA(3, 2) RXMET_LSTM_MMA(3, 4)
            RXMET_LSTM_MMA(4, 1) RXMET_LSTM_MMA(4, 2) RXMET_LSTM_MMA(4, 4)
#undef RXMET_LSTM_MMA
            afterLaunch("lstmRecurrentBackwardMma");
        }
        if (wideTensor) {
            {
                KernelTimer timer__("lstmPackBackwardTiles", st);
                packBackwardTiles<<<gridFor(static_cast<size_t>(H / kBwdUnits) * 16 * H, 256), 256, 0, st>>>(call.weightHh, H, wideTiles);
            }
            afterLaunch("lstmPackBackwardTiles");
            const int tilesPerRow = H / kBwdUnits;
            // Rows per row tile: the per-step exchange of partial sums is bound by what one SM moves, so the batch is
            // spread over as many SMs as one cooperative launch holds (smaller row tiles leave accumulator rows unused).
            const int tilesHeld = std::max(1, smsPerPass() / tilesPerRow);
            int tileRows = kBwdRows;
            for (int rows : {64, 32})
                if ((B + rows - 1) / rows <= tilesHeld) tileRows = rows;
            const int rowTilesAll = (B + tileRows - 1) / tileRows;
            const int perLaunch = std::max(1, std::min(rowTilesAll, tilesHeld));
            ensureDynamicSmem(reinterpret_cast<const void *>(recurrentBackwardUmma), wideSmem);
            RXMET_CUDA(cudaMemsetAsync(wideCounters + 255, 0, sizeof(unsigned int), st));
            for (int first = 0; first < rowTilesAll; first += perLaunch) {
                RecurrentUmmaArgs u{};
                u.base = a;
                u.tiles = wideTiles; u.channelScale = channelScales + C; u.partial = widePartial;
                u.counters = wideCounters; u.status = reinterpret_cast<int *>(wideCounters + 255);
                u.tileRows = tileRows; u.rowBase = first * tileRows; u.rowTiles = std::min(perLaunch, rowTilesAll - first);
                RXMET_CUDA(cudaMemsetAsync(wideCounters, 0, sizeof(unsigned int) * 255, st));
                void *params[] = {&u};
                KernelTimer timer__("lstmRecurrentBackwardWide", st);
                RXMET_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(recurrentBackwardUmma), dim3(u.rowTiles * tilesPerRow),
                                                       dim3(512), params, wideSmem, st));
            }
            afterLaunch("lstmRecurrentBackwardUmma");
        } else if (wide) {
            const int HP = (H + 31) / 32 * 32;
            const int groupsMax = std::max(1, 512 / HP);
            const int want = std::max(1, (B + smsPerPass() - 1) / smsPerPass());
            int rb = 1;
            while (rb < 8 && rb * groupsMax < want) rb *= 2;
            const int groups = std::max(1, std::min(groupsMax, (want + rb - 1) / rb));
            const int btWide = groups * rb;
            const size_t smem = sizeof(float) * static_cast<size_t>(btWide) * C;
            auto launchWide = [&](auto kernel) {
                ensureDynamicSmem(reinterpret_cast<const void *>(kernel), smem);
                KernelTimer timer__("lstmRecurrentBackwardWide", st);
                kernel<<<(B + btWide - 1) / btWide, groups * HP, smem, st>>>(a, HP);
            };
            if (rb == 1) launchWide(recurrentBackwardWide<1>);
            else if (rb == 2) launchWide(recurrentBackwardWide<2>);
            else if (rb == 4) launchWide(recurrentBackwardWide<4>);
            else launchWide(recurrentBackwardWide<8>);
            afterLaunch("lstmRecurrentBackwardWide");
        }
        auto launch = [&](auto kernel, int BT) {
            if (tensorPath || wide) return;
            const size_t base = sizeof(float) * (static_cast<size_t>(BT) * C + 4 * static_cast<size_t>(BT) * H);
            const size_t room = static_cast<size_t>(smemMax) > base + 1024 ? static_cast<size_t>(smemMax) - base - 1024 : 0;
            // rows per gate block in shared memory; the remaining rows of a block live in registers
            // column stride of the transposed copy: a multiple of 4 floats whose quarter is odd keeps the
            // 128-bit loads of eight neighbouring threads on distinct bank groups
            auto strideFor = [](int rows) {
                int sp = (rows + 3) / 4 * 4;
                if ((sp / 4) % 2 == 0) sp += 4;
                return sp;
            };
            int perGate = (H % 4 == 0) ? H : H / 4 * 4;
            while (perGate > 0 && sizeof(float) * 4 * static_cast<size_t>(H) * strideFor(perGate) > room) perGate -= 4;
            if (perGate < 0) perGate = 0;
            if (H - perGate > kRegRows)
                fail(RXMET_ERR_UNSUPPORTED, "hidden size %d leaves %d weight rows per gate outside shared memory and registers", H, H - perGate);
            a.smemRows = perGate;
            a.smemStride = strideFor(std::max(perGate, 1));
            const size_t smem = base + sizeof(float) * 4 * static_cast<size_t>(H) * a.smemStride;
            ensureDynamicSmem(reinterpret_cast<const void *>(kernel), smem);
            {
                KernelTimer timer__("lstmRecurrentBackward", st);
                kernel<<<(B + BT - 1) / BT, block, smem, st>>>(a);
            }
            afterLaunch("lstmRecurrentBackward");
        };
        if (bt == 4) launch(recurrentBackward<4>, 4);
        else if (bt == 2) launch(recurrentBackward<2>, 2);
        else launch(recurrentBackward<1>, 1);
    }
    if (call.quantized) RXMET_CUDA(cudaMemsetAsync(tensorStatus, 0, sizeof(int), st));
    if (tensorInputGrad) {
        // QAT: gradients times the integer weight codes on the tensor cores, scales folded into the gradients
        const int sms = currentDevice().sms;
        igrad::Problem pg{};
        pg.G = gIh; pg.kScale = channelScales; pg.codesKN = call.weightIh; pg.rows = static_cast<int>(rows); pg.K = C; pg.N = I;
        pg.mask = static_cast<const uint8_t *>(mk.input); pg.maskKeeps = 0; pg.out = call.grads.input; pg.status = tensorStatus;
        if (const size_t bytes = igrad::widePackedBytes(C, I)) pg.packed = ws.take<uint8_t>(bytes);
        igrad::launch(pg, sms, st);
        afterLaunch("inputGradUmma");
    } else if (I <= 128 && C % 4 == 0) {
        const int perThread = (I + 3) / 4;  // outputs per thread, four threads share a row
        const unsigned grid = static_cast<unsigned>((rows + kDxRows - 1) / kDxRows);
        const uint8_t *inputMask = static_cast<const uint8_t *>(mk.input);
        {
            KernelTimer timer__("lstmInputGradNarrow", st);
            if (perThread <= 4) inputGradNarrow<4><<<grid, 256, 0, st>>>(gIh, wIh, static_cast<int>(rows), I, C, inputMask, call.grads.input);
            else if (perThread <= 8) inputGradNarrow<8><<<grid, 256, 0, st>>>(gIh, wIh, static_cast<int>(rows), I, C, inputMask, call.grads.input);
            else if (perThread <= 12) inputGradNarrow<12><<<grid, 256, 0, st>>>(gIh, wIh, static_cast<int>(rows), I, C, inputMask, call.grads.input);
            else if (perThread <= 16) inputGradNarrow<16><<<grid, 256, 0, st>>>(gIh, wIh, static_cast<int>(rows), I, C, inputMask, call.grads.input);
            else if (perThread <= 24) inputGradNarrow<24><<<grid, 256, 0, st>>>(gIh, wIh, static_cast<int>(rows), I, C, inputMask, call.grads.input);
            else inputGradNarrow<32><<<grid, 256, 0, st>>>(gIh, wIh, static_cast<int>(rows), I, C, inputMask, call.grads.input);
        }
        afterLaunch("lstmInputGradNarrow");
    } else {
        {
            KernelTimer timer__("lstmGemmNN", st);
            gemmNN<<<dim3(static_cast<unsigned>((rows + kTile - 1) / kTile), (I + kTile - 1) / kTile), 256, 0, st>>>(
                gIh, wIh, static_cast<int>(rows), I, C, static_cast<const uint8_t *>(mk.input), call.grads.input);
        }
        afterLaunch("lstmGemmNN");
    }
    // QAT on 8-bit activation grids: x and h_prev are integer codes, which the tensor-core GEMM
    // multiplies exactly; its ones row also yields the bias gradients.
    if (call.quantized && call.codesFitTensorPath && I % 4 == 0 && H % 4 == 0 && I <= 140 && H <= 140 &&
        alignedTo(call.x, 16)) {
        const size_t stateBytes = sizeof(float) * static_cast<size_t>(B) * H;
        if (call.h0) RXMET_CUDA(cudaMemcpyAsync(hPrev, call.h0, stateBytes, cudaMemcpyDeviceToDevice, st));
        else RXMET_CUDA(cudaMemsetAsync(hPrev, 0, stateBytes, st));
        if (T > 1)
            RXMET_CUDA(cudaMemcpyAsync(hPrev + static_cast<size_t>(B) * H, call.hiddenOutputs, stateBytes * (T - 1),
                                       cudaMemcpyDeviceToDevice, st));
        const int sms = currentDevice().sms;
        auto planFor = [&](int M) {
            wgrad::Plan pl = wgrad::plan(static_cast<int>(rows), M, C, sms);
            if (!pl.tensorMemory && pl.splits > kMaxTensorSplits) {
                pl.chunkK = ((static_cast<int>(rows) + kMaxTensorSplits - 1) / kMaxTensorSplits + 31) / 32 * 32;
                pl.splits = (static_cast<int>(rows) + pl.chunkK - 1) / pl.chunkK;
            }
            return pl;
        };
        const wgrad::Plan planX = planFor(I), planH = planFor(H);
        wgrad::Problem px{}, ph{};
        px.aFloat = call.x; px.aFloatZero = call.dqX.zeroPoint; px.M = I; px.B = gIh; px.partial = tensorIh;
        ph.aFloat = hPrev; ph.aFloatZero = call.h0 ? call.dqH.zeroPoint : 0.0f; ph.M = H; ph.B = gHh; ph.partial = tensorHh;
        if (!call.h0 && call.dqH.zeroPoint != 0.0f) {
            // a missing h0 means real zeros, i.e. the zero-point code: fill instead of zeroing
            fail(RXMET_ERR_INVALID_ARGUMENT, "the QAT backward needs the quantized initial hidden state");
        }
        px.status = ph.status = tensorStatus;
        wgrad::launchPair(px, planX, ph, planH, static_cast<int>(rows), C, st);
        afterLaunch("weightGrad");
        {
            const ReduceJob jobIh{tensorIh, planX.splits, I, call.dqX.scale, static_cast<const uint8_t *>(mk.weight_ih),
                                  static_cast<const uint8_t *>(mk.bias_ih), call.grads.weight_ih, call.grads.bias_ih};
            const ReduceJob jobHh{tensorHh, planH.splits, H, call.dqH.scale, static_cast<const uint8_t *>(mk.weight_hh),
                                  static_cast<const uint8_t *>(mk.bias_hh), call.grads.weight_hh, call.grads.bias_hh};
            const int rowBlocks = (std::max(I, H) + 1 + kReduceRows - 1) / kReduceRows;
            KernelTimer timer__("lstmReduceWeightGradT", st);
            reduceWeightGradT<<<dim3((C + 31) / 32, rowBlocks, 2), dim3(32, kReduceRows, kReduceLayers), 0, st>>>(jobIh, jobHh, C,
                                                                                                                  tensorStatus);
        }
        afterLaunch("lstmReduceWeightGradT");
        return;
    }
    // Larger layers or 16-bit activation grids: the same tcgen05 kernel over 128-row slabs of both problems in one
    // launch, a code as two exact bf16 terms when its grid is wider than 8 bits.
    if (call.quantized && call.codesFitTwoTerms && I % 4 == 0 && H % 4 == 0 && alignedTo(call.x, 16) && (call.h0 || call.dqH.zeroPoint == 0.0f) &&
        wgrad::slabPathTakes(I, H, C) && std::getenv("RXMET_LSTM_WGRAD_SIMT") == nullptr) {
        const size_t stateBytes = sizeof(float) * static_cast<size_t>(B) * H;
        if (call.h0) RXMET_CUDA(cudaMemcpyAsync(hPrev, call.h0, stateBytes, cudaMemcpyDeviceToDevice, st));
        else RXMET_CUDA(cudaMemsetAsync(hPrev, 0, stateBytes, st));
        if (T > 1)
            RXMET_CUDA(cudaMemcpyAsync(hPrev + static_cast<size_t>(B) * H, call.hiddenOutputs, stateBytes * (T - 1),
                                       cudaMemcpyDeviceToDevice, st));
        int chunkK = 0;
        const int splits = wgrad::slabSplits(static_cast<int>(rows), I, H, C, currentDevice().sms, &chunkK);
        wgrad::Problem px{}, ph{};
        px.aFloat = call.x; px.aFloatZero = call.dqX.zeroPoint; px.M = I; px.B = gIh; px.partial = tensorIh;
        ph.aFloat = hPrev; ph.aFloatZero = call.h0 ? call.dqH.zeroPoint : 0.0f; ph.M = H; ph.B = gHh; ph.partial = tensorHh;
        px.status = ph.status = tensorStatus;
        wgrad::launchSlabs(px, ph, static_cast<int>(rows), C, chunkK, splits, !call.codesFitTensorPath, st);
        afterLaunch("weightGrad");
        {
            const ReduceJob jobIh{tensorIh, splits, I, call.dqX.scale, static_cast<const uint8_t *>(mk.weight_ih),
                                  static_cast<const uint8_t *>(mk.bias_ih), call.grads.weight_ih, call.grads.bias_ih};
            const ReduceJob jobHh{tensorHh, splits, H, call.dqH.scale, static_cast<const uint8_t *>(mk.weight_hh),
                                  static_cast<const uint8_t *>(mk.bias_hh), call.grads.weight_hh, call.grads.bias_hh};
            const int rowBlocks = (std::max(I, H) + 1 + kReduceRows - 1) / kReduceRows;
            KernelTimer timer__("lstmReduceWeightGradT", st);
            reduceWeightGradT<<<dim3((C + 31) / 32, rowBlocks, 2), dim3(32, kReduceRows, kReduceLayers), 0, st>>>(jobIh, jobHh, C,
                                                                                                                  tensorStatus);
        }
        afterLaunch("lstmReduceWeightGradT");
        return;
    }
    auto weightGrad = [&](const float *G, RowSource X, int N, int splits, float *partial, const uint8_t *mask, float *out) {
        const int chunk = ((static_cast<int>(rows) + splits - 1) / splits + kDepth - 1) / kDepth * kDepth;
        {
            KernelTimer timer__("lstmGemmRowsTN", st);
            gemmRowsTN<<<dim3((N + kTile - 1) / kTile, (C + kTile - 1) / kTile, splits), 256, 0, st>>>(
                G, X, static_cast<int>(rows), C, N, chunk, partial);
        }
        afterLaunch("lstmGemmRowsTN");
        {
            KernelTimer timer__("lstmReduceSplits", st);
            reduceSplits<<<gridFor(static_cast<size_t>(C) * N, 256), 256, 0, st>>>(partial, splits, static_cast<size_t>(C) * N, mask, out);
        }
        afterLaunch("lstmReduceSplits");
    };
    weightGrad(gIh, RowSource{call.x, call.x, 0, call.dqX}, I, splitIh, partIh, static_cast<const uint8_t *>(mk.weight_ih),
               call.grads.weight_ih);
    weightGrad(gHh, RowSource{call.h0, call.hiddenOutputs, B, call.dqH}, H, splitHh, partHh,
               static_cast<const uint8_t *>(mk.weight_hh), call.grads.weight_hh);
    if (call.grads.bias_ih || call.grads.bias_hh) {
        const int chunk = (static_cast<int>(rows) + kBiasSplits - 1) / kBiasSplits;
        {
            KernelTimer timer__("lstmColumnSums", st);
            columnSums<<<dim3((C + 127) / 128, 2, kBiasSplits), 128, 0, st>>>(gIh, gHh, static_cast<int>(rows), C, chunk, partBias);
        }
        afterLaunch("lstmColumnSums");
        float *dst[2] = {call.grads.bias_ih, call.grads.bias_hh};
        const uint8_t *msk[2] = {static_cast<const uint8_t *>(mk.bias_ih), static_cast<const uint8_t *>(mk.bias_hh)};
        for (int k = 0; k < 2; ++k) {
            if (!dst[k]) continue;
            {
                KernelTimer timer__("lstmReduceSplits", st);
                reduceSplits<<<gridFor(C, 128), 128, 0, st>>>(partBias + static_cast<size_t>(k) * kBiasSplits * C, kBiasSplits, C, msk[k], dst[k]);
            }
            afterLaunch("lstmReduceSplits");
        }
    }
}

}  // namespace lstm
}  // namespace rxmet
