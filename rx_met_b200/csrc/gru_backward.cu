// GRU backward through time (float arithmetic on dequantized saved values, straight-through
// clamp masks) and the weight / input / bias gradients.
//
//   recurrentBackward : ONE launch for all T steps in reverse.  Like the forward, each CTA owns a
//                       batch tile for the whole sequence (dh is independent per sequence) and
//                       keeps R resident in shared memory; per step it forms dp/dq with every
//                       mask applied and then dh += R dq.
//   gemmTN + reduce   : dW = x^T dp and dR = h^T dq as split-K tile GEMMs whose partial sums are
//                       added in a fixed order, so gradients are reproducible run to run.
//   gemmNT            : dx = dp W^T with the input clamp mask.
//   columnSums        : bias gradients as fixed-order column sums (the reference uses float
//                       atomics here, gru_backward_gpu_quant.cu:258-264).
//
// Reference: operators/quant-gru/src/gru_backward_gpu_quant.cu:93-493 and, for the float path,
// src/gru_backward_gpu.cu.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstdlib>

#include "common.h"
#include "gru_backward.h"
#include "gru_forward_quant.h"
#include "input_grad_umma.h"
#include "weight_grad_mma.h"

namespace rxmet {
namespace gru {
namespace {

__device__ __forceinline__ float keepOf(const uint8_t *m, size_t i) { return m ? static_cast<float>(m[i]) : 1.0f; }

// Pulls the line holding *p into L2 without occupying a register or blocking the warp.
__device__ __forceinline__ void prefetchL2(const void *p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// out[i] = (codes[i] - zp) * scale, scale per column when channelScale is set
// (gru_interface_binding.cc:842-856).
__global__ void dequantCodes(const int32_t *__restrict__ q, size_t n, int cols, const float *__restrict__ channelScale,
                             float scalarScale, int32_t zp, float *__restrict__ out) {
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const float s = channelScale ? channelScale[i % cols] : scalarScale;
        out[i] = (static_cast<float>(q[i]) - static_cast<float>(zp)) * s;
    }
}

struct BackwardArgs {
    int T, B, H;
    int weightsInSmem;
    int parts;            // the 3H contraction of dh += R dq is split into this many thread groups
    const float *RT;      // [3H][H] : R transposed
    const float *h;       // [T+1][B][H]
    const float *v;       // [T][B][4H]
    const float *dhNew;   // [T+1][B][H]
    float *dp, *dq;       // [T][B][3H]
    float *dh0;           // [B][H]
    const uint8_t *mIh, *mHh, *mGateIn, *mGateOut, *mH, *mH0;
};

template <int BT>
__global__ void __launch_bounds__(768) recurrentBackward(const __grid_constant__ BackwardArgs a) {
    const int H = a.H, C = 3 * a.H, P = a.parts;
    extern __shared__ float smemB[];
    float *dhS = smemB;                   // [BT][H]   gradient flowing to the previous step
    float *dqS = dhS + BT * H;            // [BT][C]
    float *partS = dqS + BT * C;          // [P][BT][H]
    float *RS = partS + P * BT * H;       // [C][H] when resident
    const int tid = threadIdx.x, nthreads = blockDim.x;
    const int b0 = blockIdx.x * BT, nb = min(BT, a.B - b0);

    const float *RT = a.RT;
    if (a.weightsInSmem) {
        for (int i = tid; i < C * H; i += nthreads) RS[i] = a.RT[i];
        RT = RS;
    }
    for (int i = tid; i < BT * H; i += nthreads) dhS[i] = 0.0f;
    for (int i = tid; i < BT * C; i += nthreads) dqS[i] = 0.0f;
    __syncthreads();

    for (int t = a.T - 1; t >= 0; --t) {
        const size_t rowBase = static_cast<size_t>(t) * a.B + b0;
        // ---- pointwise derivative with masks (gru_backward_gpu_quant.cu:110-240)
        for (int i = tid; i < nb * H; i += nthreads) {
            const int b = i / H, j = i % H;
            const size_t row = rowBase + b;
            const size_t hi = row * H + j, gi = row * C + j;
            const float *vRow = a.v + row * 4 * H;
            float dhTotal = a.dhNew[hi + static_cast<size_t>(a.B) * H] + dhS[b * H + j];
            dhTotal *= keepOf(a.mH, hi);
            const float z = vRow[j], r = vRow[H + j], g = vRow[2 * H + j], qg = vRow[3 * H + j];
            dhS[b * H + j] = z * dhTotal;
            const float dg = (1.0f - z) * dhTotal;
            const float dz = (a.h[hi] - g) * dhTotal;
            float dpG = (1.0f - g * g) * dg;
            dpG *= keepOf(a.mGateOut, gi + 2 * H);
            dpG *= keepOf(a.mGateIn, gi + 2 * H);
            const float dqG = dpG * r;
            const float dr = dpG * qg;
            const float dpR = (r * (1.0f - r)) * dr;
            const float dpZ = (z * (1.0f - z)) * dz;
            const float kz = keepOf(a.mGateOut, gi) * keepOf(a.mGateIn, gi);
            const float kr = keepOf(a.mGateOut, gi + H) * keepOf(a.mGateIn, gi + H);
            const float pz = dpZ * kz * keepOf(a.mIh, gi);
            const float pr = dpR * kr * keepOf(a.mIh, gi + H);
            const float pg = dpG * keepOf(a.mIh, gi + 2 * H);
            const float qz = dpZ * kz * keepOf(a.mHh, gi);
            const float qr = dpR * kr * keepOf(a.mHh, gi + H);
            const float qn = dqG * keepOf(a.mHh, gi + 2 * H);
            a.dp[gi] = pz; a.dp[gi + H] = pr; a.dp[gi + 2 * H] = pg;
            a.dq[gi] = qz; a.dq[gi + H] = qr; a.dq[gi + 2 * H] = qn;
            float *dqRow = dqS + b * C;
            dqRow[j] = qz; dqRow[H + j] = qr; dqRow[2 * H + j] = qn;
        }
        __syncthreads();
        // ---- dh[b,k] += sum_c R[k,c] dq[b,c], contraction split over P thread groups
        for (int item = tid; item < H * P; item += nthreads) {
            const int k = item % H, part = item / H;
            const int c0 = static_cast<int>(static_cast<long long>(C) * part / P);
            const int c1 = static_cast<int>(static_cast<long long>(C) * (part + 1) / P);
            float acc[BT];
#pragma unroll
            for (int b = 0; b < BT; ++b) acc[b] = 0.0f;
            for (int c = c0; c < c1; ++c) {
                const float w = RT[static_cast<size_t>(c) * H + k];
#pragma unroll
                for (int b = 0; b < BT; ++b) acc[b] = fmaf(w, dqS[b * C + c], acc[b]);
            }
#pragma unroll
            for (int b = 0; b < BT; ++b) partS[(part * BT + b) * H + k] = acc[b];
        }
        __syncthreads();
        for (int i = tid; i < BT * H; i += nthreads) {
            float s = dhS[i];
            for (int p = 0; p < P; ++p) s += partS[p * BT * H + i];
            dhS[i] = s;
        }
        __syncthreads();
    }
    for (int i = tid; i < nb * H; i += nthreads) {
        const size_t o = static_cast<size_t>(b0 + i / H) * H + (i % H);
        a.dh0[o] = dhS[i] * keepOf(a.mH0, o);
    }
}

// bf16 helpers: exact conversions of small integers, round-to-nearest splits of fp32 values
__device__ __forceinline__ uint32_t packBf16(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ float bf16Lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16Hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

// ---- quantized weights in registers -------------------------------------------
//
// For weight grids of at most 8 bits the codes are exact in bf16, so R[k][c] = code * scale[c]
// can live in registers as packed bf16 code pairs with the per-channel scale folded into dq.
// Thread (k, p) owns row k of gate p: H codes = CW packed words, resident for the whole sequence;
// a step's dh += R dq then reads shared memory only for the broadcast of dq (128-bit loads).
// All per-step operands (v, h, dh_new, 13 mask bytes) are fetched one step ahead.

// RB[(p*CW + jj)*H + k] = bf16x2(code[k][p*H + 2jj], code[k][p*H + 2jj + 1])
__global__ void packRecurrentBf16(const int32_t *__restrict__ Rq, int H, int CW, uint32_t *__restrict__ RB) {
    const int total = 3 * CW * H;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int k = i % H, jj = (i / H) % CW, p = i / (H * CW);
        const int j0 = 2 * jj, j1 = 2 * jj + 1;
        const float c0 = j0 < H ? static_cast<float>(Rq[static_cast<size_t>(k) * 3 * H + p * H + j0]) : 0.0f;
        const float c1 = j1 < H ? static_cast<float>(Rq[static_cast<size_t>(k) * 3 * H + p * H + j1]) : 0.0f;
        // |code| <= 256 has at most 9 significant bits with a trailing zero beyond 8: exact in bf16
        RB[i] = (__float_as_uint(c0) >> 16) | (__float_as_uint(c1) & 0xffff0000u);
    }
}

// One 16-bit word per (t, b, j) with the 13 keep flags the pointwise derivative of hidden unit j
// needs: bits 0..2 gate_output (z,r,n), 3..5 gate_input, 6..8 weight_hh_linear, 9..11
// weight_ih_linear, 12 h.  Packing them once, outside the serial time loop, replaces 13 byte loads
// per element and step on the critical path by one.
__global__ void packStepMasks(const uint8_t *__restrict__ mIh, const uint8_t *__restrict__ mHh,
                              const uint8_t *__restrict__ mGateIn, const uint8_t *__restrict__ mGateOut,
                              const uint8_t *__restrict__ mH, size_t rows, int H, uint16_t *__restrict__ out) {
    const size_t total = rows * H;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t row = i / H, j = i % H, gi = row * 3 * H + j;
        auto bit = [](const uint8_t *m, size_t at, int pos) -> uint32_t { return (m ? (m[at] ? 1u : 0u) : 1u) << pos; };
        out[i] = static_cast<uint16_t>(
            bit(mGateOut, gi, 0) | bit(mGateOut, gi + H, 1) | bit(mGateOut, gi + 2 * H, 2) | bit(mGateIn, gi, 3) |
            bit(mGateIn, gi + H, 4) | bit(mGateIn, gi + 2 * H, 5) | bit(mHh, gi, 6) | bit(mHh, gi + H, 7) |
            bit(mHh, gi + 2 * H, 8) | bit(mIh, gi, 9) | bit(mIh, gi + H, 10) | bit(mIh, gi + 2 * H, 11) | bit(mH, i, 12));
    }
}

// The same packing, four hidden units per thread (H a multiple of 4, flag bytes 0 or 1, as every
// forward of this library writes them): 32-bit loads of four flag bytes, two byte permutes spread
// them over the 16-bit lanes of two words, and a multiply-add moves each pair into its bit position.
__global__ void packStepMasks4(const uint8_t *__restrict__ mIh, const uint8_t *__restrict__ mHh,
                               const uint8_t *__restrict__ mGateIn, const uint8_t *__restrict__ mGateOut,
                               const uint8_t *__restrict__ mH, size_t quads, int H, uint2 *__restrict__ out) {
    for (size_t q = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; q < quads;
         q += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t i = q * 4, row = i / H, j = i % H, gi = row * 3 * H + j;
        uint32_t lanes01 = 0, lanes23 = 0;
        auto add = [&](const uint8_t *m, size_t at, int pos) {
            const uint32_t w = m ? *reinterpret_cast<const uint32_t *>(m + at) : 0x01010101u;
            lanes01 += __byte_perm(w, 0u, 0x4140) * (1u << pos);
            lanes23 += __byte_perm(w, 0u, 0x4342) * (1u << pos);
        };
#pragma unroll
        for (int g = 0; g < 3; ++g) {
            add(mGateOut, gi + static_cast<size_t>(g) * H, g);
            add(mGateIn, gi + static_cast<size_t>(g) * H, 3 + g);
            add(mHh, gi + static_cast<size_t>(g) * H, 6 + g);
            add(mIh, gi + static_cast<size_t>(g) * H, 9 + g);
        }
        add(mH, i, 12);
        out[q] = make_uint2(lanes01, lanes23);
    }
}

struct BackwardQArgs {
    int T, B, H;
    const uint32_t *RB;      // packed codes, see packRecurrentBf16
    const float *scaleR;     // [3H] effective scale per column
    const float *h, *v, *dhNew;
    float *dp, *dq, *dh0;
    const uint8_t *mIh, *mHh, *mGateIn, *mGateOut, *mH, *mH0;
    const uint16_t *stepBits;  // packed keep flags, see packStepMasks; null = nothing was clamped
    // a sequence cut into time chunks (recurrentBackwardMma only): the gradient that flows into the chunk's last
    // step from the later chunk, and whether dh0 receives this chunk's outgoing gradient as it is (1) or, at
    // the start of the sequence, under the h0 mask (0)
    const float *dhIn;
    int carryOut;
};

struct StepOperands {
    float z, r, g, qg, hOld, dhNew;
    uint32_t keepBits;  // bit i = keep flag: 0..2 gate_out(z,r,n) 3..5 gate_in 6..8 hh 9..11 ih 12 h
};

template <int CW, int BT>
__global__ void __launch_bounds__(384) recurrentBackwardQ(const __grid_constant__ BackwardQArgs a) {
    const int H = a.H, C = 3 * a.H;
    constexpr int HP = 2 * CW;           // padded hidden size
    extern __shared__ __align__(16) float smemB[];
    float *dqS = smemB;                  // [BT][3][HP]  dq scaled by the column scale, gate-major
    float *partS = dqS + BT * 3 * HP;    // [3][BT][H]
    const int tid = threadIdx.x, nthreads = blockDim.x;
    const int b0 = blockIdx.x * BT, nb = min(BT, a.B - b0);
    const int k = tid % H, p = tid / H;  // blockDim == 3H

    uint32_t rw[CW];
#pragma unroll
    for (int jj = 0; jj < CW; ++jj) rw[jj] = a.RB[static_cast<size_t>(p * CW + jj) * H + k];
    for (int i = tid; i < BT * 3 * HP; i += nthreads) dqS[i] = 0.0f;
    for (int i = tid; i < 3 * BT * H; i += nthreads) partS[i] = 0.0f;

    constexpr int kSlots = (BT + 2) / 3;  // ceil(BT*H / 3H) gate elements per thread
    const int elems = nb * H;
    float dhBase[kSlots];
    float scale[kSlots][3];
    StepOperands cur[kSlots], nxt[kSlots];
#pragma unroll
    for (int s2 = 0; s2 < kSlots; ++s2) {
        dhBase[s2] = 0.0f;
        const int e = tid + s2 * nthreads;
        const int j = e % H;
        scale[s2][0] = a.scaleR[j]; scale[s2][1] = a.scaleR[H + j]; scale[s2][2] = a.scaleR[2 * H + j];
    }
    auto fetch = [&](int t, StepOperands (&dst)[kSlots]) {
#pragma unroll
        for (int s2 = 0; s2 < kSlots; ++s2) {
            const int e = tid + s2 * nthreads;
            if (e < elems) {
                const int b = e / H, j = e % H;
                const size_t row = static_cast<size_t>(t) * a.B + b0 + b;
                const size_t hi = row * H + j;
                const float *vRow = a.v + row * 4 * H;
                StepOperands o;
                o.z = vRow[j]; o.r = vRow[H + j]; o.g = vRow[2 * H + j]; o.qg = vRow[3 * H + j];
                o.hOld = a.h[hi];
                o.dhNew = a.dhNew[hi + static_cast<size_t>(a.B) * H];
                o.keepBits = a.stepBits ? a.stepBits[hi] : 0x1fffu;
                dst[s2] = o;
            }
        }
    };
    fetch(a.T - 1, cur);
    __syncthreads();

    for (int t = a.T - 1; t >= 0; --t) {
        if (t > 0) fetch(t - 1, nxt);
        const size_t rowBase = static_cast<size_t>(t) * a.B + b0;
        // ---- pointwise derivative with masks (gru_backward_gpu_quant.cu:110-240)
#pragma unroll
        for (int s2 = 0; s2 < kSlots; ++s2) {
            const int e = tid + s2 * nthreads;
            if (e < elems) {
                const int b = e / H, j = e % H;
                const size_t gi = (rowBase + b) * C + j;
                const StepOperands o = cur[s2];
                auto keep = [&](int pos) { return static_cast<float>((o.keepBits >> pos) & 1u); };
                const float carried = dhBase[s2] + partS[(0 * BT + b) * H + j] + partS[(1 * BT + b) * H + j] +
                                      partS[(2 * BT + b) * H + j];
                const float dhTotal = (o.dhNew + carried) * keep(12);
                dhBase[s2] = o.z * dhTotal;
                const float dg = (1.0f - o.z) * dhTotal;
                const float dz = (o.hOld - o.g) * dhTotal;
                const float dpG = (1.0f - o.g * o.g) * dg * keep(2) * keep(5);
                const float dqG = dpG * o.r;
                const float dr = dpG * o.qg;
                const float dpR = (o.r * (1.0f - o.r)) * dr;
                const float dpZ = (o.z * (1.0f - o.z)) * dz;
                const float kz = keep(0) * keep(3), kr = keep(1) * keep(4);
                const float pz = dpZ * kz * keep(9), pr = dpR * kr * keep(10), pg = dpG * keep(11);
                const float qz = dpZ * kz * keep(6), qr = dpR * kr * keep(7), qn = dqG * keep(8);
                a.dp[gi] = pz; a.dp[gi + H] = pr; a.dp[gi + 2 * H] = pg;
                a.dq[gi] = qz; a.dq[gi + H] = qr; a.dq[gi + 2 * H] = qn;
                float *dqRow = dqS + b * 3 * HP;
                dqRow[j] = qz * scale[s2][0]; dqRow[HP + j] = qr * scale[s2][1]; dqRow[2 * HP + j] = qn * scale[s2][2];
            }
        }
        __syncthreads();
        // ---- part p of dh[b,k] = sum_j R[k][pH + j] dq'[b][pH + j]
        {
            float acc[BT];
#pragma unroll
            for (int b = 0; b < BT; ++b) acc[b] = 0.0f;
            const float4 *dq4 = reinterpret_cast<const float4 *>(dqS + p * HP);
#pragma unroll
            for (int j4 = 0; j4 < CW / 2; ++j4) {
                const float w0 = __uint_as_float(rw[2 * j4] << 16), w1 = __uint_as_float(rw[2 * j4] & 0xffff0000u);
                const float w2 = __uint_as_float(rw[2 * j4 + 1] << 16), w3 = __uint_as_float(rw[2 * j4 + 1] & 0xffff0000u);
#pragma unroll
                for (int b = 0; b < BT; ++b) {
                    const float4 d = dq4[b * (3 * HP / 4) + j4];
                    acc[b] = fmaf(w0, d.x, acc[b]);
                    acc[b] = fmaf(w1, d.y, acc[b]);
                    acc[b] = fmaf(w2, d.z, acc[b]);
                    acc[b] = fmaf(w3, d.w, acc[b]);
                }
            }
#pragma unroll
            for (int b = 0; b < BT; ++b) partS[(p * BT + b) * H + k] = acc[b];
        }
#pragma unroll
        for (int s2 = 0; s2 < kSlots; ++s2) cur[s2] = nxt[s2];
        __syncthreads();
    }
#pragma unroll
    for (int s2 = 0; s2 < kSlots; ++s2) {
        const int e = tid + s2 * nthreads;
        if (e < elems) {
            const int b = e / H, j = e % H;
            const size_t o = static_cast<size_t>(b0 + b) * H + j;
            const float carried = dhBase[s2] + partS[(0 * BT + b) * H + j] + partS[(1 * BT + b) * H + j] +
                                  partS[(2 * BT + b) * H + j];
            a.dh0[o] = carried * keepOf(a.mH0, o);
        }
    }
}

// ---- hidden sizes above 128: recurrent weight codes in shared memory ---------------------------
//
// For H > 128 the weight rows no longer fit the registers of recurrentBackwardQ / the fragments of the
// tensor-core kernel, and as fp32 or bf16 they do not fit shared memory either (3H x H values; 393 KB as
// bf16 at H = 256).  As 8-bit codes they do (196 KB at H = 256): word (c / 4, k) holds the codes
// R[k][4 (c / 4) .. + 3], stored with bit 7 flipped so that a byte permute builds the float 2^23 + (code + 128)
// directly and one subtraction yields the code (two full-rate instructions per weight, no integer-to-float
// conversion).  The per-column scale is folded into dq as in the kernels above.  Thread (k, part) sums a
// part of the 3H columns for hidden row k; the parts meet in shared memory.  Per-step operands are fetched
// one step ahead.
struct BackwardCodesArgs {
    BackwardQArgs q;
    const int32_t *Rq;  // [H][3H] integer codes as saved by the forward
    int HP, parts;
};

template <int RB>
__global__ void __launch_bounds__(512, 1) recurrentBackwardCodes(const __grid_constant__ BackwardCodesArgs ca) {
    const BackwardQArgs &a = ca.q;
    const int H = a.H, C = 3 * a.H, CW = C / 4, HP = ca.HP, P = ca.parts;
    extern __shared__ __align__(16) unsigned char smemRawB[];
    uint32_t *Rw = reinterpret_cast<uint32_t *>(smemRawB);             // [CW][H]
    float *dqS = reinterpret_cast<float *>(Rw + static_cast<size_t>(CW) * H);  // [RB][C]
    float *partS = dqS + RB * C;                                        // [P][RB][H]
    const int tid = threadIdx.x, k = tid % HP, part = tid / HP;
    const bool active = k < H;
    const int b0 = blockIdx.x * RB;
    for (int i = tid; i < CW * H; i += blockDim.x) {
        const int cw = i / H, row = i - cw * H;
        const int4 c4 = *reinterpret_cast<const int4 *>(ca.Rq + static_cast<size_t>(row) * C + 4 * cw);
        const uint32_t word = (static_cast<uint32_t>(c4.x) & 0xffu) | ((static_cast<uint32_t>(c4.y) & 0xffu) << 8) |
                              ((static_cast<uint32_t>(c4.z) & 0xffu) << 16) | ((static_cast<uint32_t>(c4.w) & 0xffu) << 24);
        Rw[i] = word ^ 0x80808080u;
    }
    for (int i = tid; i < RB * C; i += blockDim.x) dqS[i] = 0.0f;
    for (int i = tid; i < P * RB * H; i += blockDim.x) partS[i] = 0.0f;
    const bool owner = active && part == 0;  // the pointwise derivative of (rows, k) runs in part 0
    float scale[3] = {1.0f, 1.0f, 1.0f};
    if (owner) {
        scale[0] = a.scaleR[k]; scale[1] = a.scaleR[H + k]; scale[2] = a.scaleR[2 * H + k];
    }
    float dhBase[RB];
    StepOperands cur[RB], nxt[RB];
#pragma unroll
    for (int r = 0; r < RB; ++r) dhBase[r] = 0.0f;
    auto fetch = [&](int t, StepOperands (&dst)[RB]) {
        if (!owner) return;
#pragma unroll
        for (int r = 0; r < RB; ++r) {
            const int b = b0 + r;
            if (b >= a.B) continue;
            const size_t row = static_cast<size_t>(t) * a.B + b, hi = row * H + k;
            const float *vRow = a.v + row * 4 * H;
            StepOperands o;
            o.z = vRow[k]; o.r = vRow[H + k]; o.g = vRow[2 * H + k]; o.qg = vRow[3 * H + k];
            o.hOld = a.h[hi];
            o.dhNew = a.dhNew[hi + static_cast<size_t>(a.B) * H];
            o.keepBits = a.stepBits ? a.stepBits[hi] : 0x1fffu;
            dst[r] = o;
        }
    };
    fetch(a.T - 1, cur);
    __syncthreads();

    const int cwBegin = CW * part / P, cwEnd = CW * (part + 1) / P;
    for (int t = a.T - 1; t >= 0; --t) {
        if (t > 0) fetch(t - 1, nxt);
        if (owner) {
#pragma unroll
            for (int r = 0; r < RB; ++r) {
                const int b = b0 + r;
                if (b >= a.B) continue;
                const size_t gi = (static_cast<size_t>(t) * a.B + b) * C + k;
                const StepOperands o = cur[r];
                auto keep = [&](int pos) { return static_cast<float>((o.keepBits >> pos) & 1u); };
                float carried = dhBase[r];
                for (int p2 = 0; p2 < P; ++p2) carried += partS[(p2 * RB + r) * H + k];
                const float dhTotal = (o.dhNew + carried) * keep(12);
                dhBase[r] = o.z * dhTotal;
                const float dg = (1.0f - o.z) * dhTotal;
                const float dz = (o.hOld - o.g) * dhTotal;
                const float dpG = (1.0f - o.g * o.g) * dg * keep(2) * keep(5);
                const float dqG = dpG * o.r;
                const float dr = dpG * o.qg;
                const float dpR = (o.r * (1.0f - o.r)) * dr;
                const float dpZ = (o.z * (1.0f - o.z)) * dz;
                const float kz = keep(0) * keep(3), kr = keep(1) * keep(4);
                const float pz = dpZ * kz * keep(9), pr = dpR * kr * keep(10), pg = dpG * keep(11);
                const float qz = dpZ * kz * keep(6), qr = dpR * kr * keep(7), qn = dqG * keep(8);
                a.dp[gi] = pz; a.dp[gi + H] = pr; a.dp[gi + 2 * H] = pg;
                a.dq[gi] = qz; a.dq[gi + H] = qr; a.dq[gi + 2 * H] = qn;
                float *dqRow = dqS + r * C;
                dqRow[k] = qz * scale[0]; dqRow[H + k] = qr * scale[1]; dqRow[2 * H + k] = qn * scale[2];
            }
        }
        __syncthreads();
        if (active) {
            float acc[RB];
#pragma unroll
            for (int r = 0; r < RB; ++r) acc[r] = 0.0f;
            const float bias = 8388736.0f;  // 2^23 + 128
#pragma unroll 4
            for (int cw = cwBegin; cw < cwEnd; ++cw) {
                const uint32_t w = Rw[static_cast<size_t>(cw) * H + k];
                const float w0 = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540)) - bias;
                const float w1 = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7541)) - bias;
                const float w2 = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7542)) - bias;
                const float w3 = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7543)) - bias;
#pragma unroll
                for (int r = 0; r < RB; ++r) {
                    const float4 d = *reinterpret_cast<const float4 *>(dqS + r * C + 4 * cw);
                    acc[r] = fmaf(w0, d.x, acc[r]);
                    acc[r] = fmaf(w1, d.y, acc[r]);
                    acc[r] = fmaf(w2, d.z, acc[r]);
                    acc[r] = fmaf(w3, d.w, acc[r]);
                }
            }
#pragma unroll
            for (int r = 0; r < RB; ++r) partS[(part * RB + r) * H + k] = acc[r];
        }
#pragma unroll
        for (int r = 0; r < RB; ++r) cur[r] = nxt[r];
        __syncthreads();
    }
    if (owner) {
#pragma unroll
        for (int r = 0; r < RB; ++r) {
            if (b0 + r >= a.B) continue;
            const size_t o = static_cast<size_t>(b0 + r) * H + k;
            float carried = dhBase[r];
            for (int p2 = 0; p2 < P; ++p2) carried += partS[(p2 * RB + r) * H + k];
            a.dh0[o] = carried * keepOf(a.mH0, o);
        }
    }
}

// ---- the same recurrence over a cluster of eight CTAs ------------------------------------------
//
// For hidden sizes whose recurrent weights fit no single SM as fp32, the eight CTAs of a cluster share a tile
// of RB batch rows: CTA c owns the hidden units [c H/8, (c+1) H/8) and keeps ITS rows of R (H/8 x 3H values,
// exact integer codes as fp32) in registers for the whole sequence — thread (unit, part) holds the 3H/8
// columns of part `part` — so the per-step product needs no weight traffic and no widening of codes at all.
// Per step every CTA computes the pointwise derivative of its units, stores the scaled gate gradients of its
// 3 H/8 columns into the dq tile of ALL eight CTAs through distributed shared memory, and after one hardware
// cluster barrier (release / acquire; every CTA runs the same T iterations) multiplies the complete tile with
// its register-resident weights.  The dq tile is double-buffered: a CTA can only write the tile of step t-2
// after every CTA of the cluster has arrived at the barrier of step t-1, that is after it has finished
// reading the tile of step t.
struct BackwardClusterArgs {
    BackwardQArgs q;
    const int32_t *Rq;  // [H][3H] integer codes as saved by the forward
};

constexpr int kClusterCtas = 8, kClusterParts = 8;

__device__ __forceinline__ void clusterBarrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

template <int WPT, int RB>  // WPT = 3H / 8 weights per thread, RB batch rows per cluster (a multiple of 8)
__global__ void __launch_bounds__(256, 1)   // launched with a cluster dimension of kClusterCtas
recurrentBackwardCluster(const __grid_constant__ BackwardClusterArgs ca) {
    constexpr int NC = kClusterCtas, P = kClusterParts, RPT = RB / P;
    const BackwardQArgs &a = ca.q;
    const int H = a.H, C = 3 * a.H, HS = H / NC;
    extern __shared__ __align__(16) unsigned char smemRawC[];
    float *dqS = reinterpret_cast<float *>(smemRawC);       // [2][RB][C]: scaled gate gradients of the whole tile
    float *partS = dqS + 2 * RB * C;                        // [P][RB][HS]
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const int tid = threadIdx.x, jl = tid % HS, part = tid / HS;
    const int j = static_cast<int>(rank) * HS + jl;
    const int b0 = static_cast<int>(blockIdx.x / NC) * RB;

    float w[WPT];
#pragma unroll
    for (int i = 0; i < WPT; ++i) w[i] = static_cast<float>(ca.Rq[static_cast<size_t>(j) * C + part * WPT + i]);
    for (int i = tid; i < 2 * RB * C; i += blockDim.x) dqS[i] = 0.0f;
    for (int i = tid; i < P * RB * HS; i += blockDim.x) partS[i] = 0.0f;
    const float scale[3] = {a.scaleR[j], a.scaleR[H + j], a.scaleR[2 * H + j]};
    // this CTA's view of the same dq element in every CTA of the cluster
    uint32_t tile[NC];
    {
        const uint32_t local = static_cast<uint32_t>(__cvta_generic_to_shared(dqS));
#pragma unroll
        for (int d = 0; d < NC; ++d) asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(tile[d]) : "r"(local), "r"(d));
    }

    float dhBase[RPT];
    StepOperands cur[RPT], nxt[RPT];
#pragma unroll
    for (int i = 0; i < RPT; ++i) dhBase[i] = 0.0f;
    auto fetch = [&](int t, StepOperands (&dst)[RPT]) {
#pragma unroll
        for (int i = 0; i < RPT; ++i) {
            const int b = b0 + part + P * i;
            if (b >= a.B) continue;
            const size_t row = static_cast<size_t>(t) * a.B + b, hi = row * H + j;
            const float *vRow = a.v + row * 4 * H;
            StepOperands o;
            o.z = vRow[j]; o.r = vRow[H + j]; o.g = vRow[2 * H + j]; o.qg = vRow[3 * H + j];
            o.hOld = a.h[hi];
            o.dhNew = a.dhNew[hi + static_cast<size_t>(a.B) * H];
            o.keepBits = a.stepBits ? a.stepBits[hi] : 0x1fffu;
            dst[i] = o;
        }
    };
    fetch(a.T - 1, cur);
    clusterBarrier();  // every CTA has cleared its tiles before anyone stores into them

    for (int t = a.T - 1; t >= 0; --t) {
        const int buf = t & 1;
        if (t > 0) fetch(t - 1, nxt);
#pragma unroll
        for (int i = 0; i < RPT; ++i) {
            const int r = part + P * i, b = b0 + r;
            float q3[3] = {0.0f, 0.0f, 0.0f};
            if (b < a.B) {
                const size_t gi = (static_cast<size_t>(t) * a.B + b) * C + j;
                const StepOperands o = cur[i];
                auto keep = [&](int pos) { return static_cast<float>((o.keepBits >> pos) & 1u); };
                float carried = dhBase[i];
#pragma unroll
                for (int p2 = 0; p2 < P; ++p2) carried += partS[(p2 * RB + r) * HS + jl];
                const float dhTotal = (o.dhNew + carried) * keep(12);
                dhBase[i] = o.z * dhTotal;
                const float dg = (1.0f - o.z) * dhTotal;
                const float dz = (o.hOld - o.g) * dhTotal;
                const float dpG = (1.0f - o.g * o.g) * dg * keep(2) * keep(5);
                const float dqG = dpG * o.r;
                const float dr = dpG * o.qg;
                const float dpR = (o.r * (1.0f - o.r)) * dr;
                const float dpZ = (o.z * (1.0f - o.z)) * dz;
                const float kz = keep(0) * keep(3), kr = keep(1) * keep(4);
                const float pz = dpZ * kz * keep(9), pr = dpR * kr * keep(10), pg = dpG * keep(11);
                const float qz = dpZ * kz * keep(6), qr = dpR * kr * keep(7), qn = dqG * keep(8);
                a.dp[gi] = pz; a.dp[gi + H] = pr; a.dp[gi + 2 * H] = pg;
                a.dq[gi] = qz; a.dq[gi + H] = qr; a.dq[gi + 2 * H] = qn;
                q3[0] = qz * scale[0]; q3[1] = qr * scale[1]; q3[2] = qn * scale[2];
            }
            const uint32_t at = static_cast<uint32_t>(sizeof(float)) * static_cast<uint32_t>((buf * RB + r) * C + j);
#pragma unroll
            for (int d = 0; d < NC; ++d)
#pragma unroll
                for (int g = 0; g < 3; ++g)
                    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(tile[d] + at + static_cast<uint32_t>(sizeof(float)) * g * H), "f"(q3[g])
                                 : "memory");
        }
        clusterBarrier();  // the tile of step t is complete in every CTA

        float acc[RB];
#pragma unroll
        for (int r = 0; r < RB; ++r) acc[r] = 0.0f;
        const float *tileRow = dqS + static_cast<size_t>(buf) * RB * C + part * WPT;
#pragma unroll
        for (int i4 = 0; i4 < WPT / 4; ++i4) {
#pragma unroll
            for (int r = 0; r < RB; ++r) {
                const float4 d = *reinterpret_cast<const float4 *>(tileRow + r * C + 4 * i4);
                acc[r] = fmaf(w[4 * i4], d.x, acc[r]);
                acc[r] = fmaf(w[4 * i4 + 1], d.y, acc[r]);
                acc[r] = fmaf(w[4 * i4 + 2], d.z, acc[r]);
                acc[r] = fmaf(w[4 * i4 + 3], d.w, acc[r]);
            }
        }
#pragma unroll
        for (int r = 0; r < RB; ++r) partS[(part * RB + r) * HS + jl] = acc[r];
#pragma unroll
        for (int i = 0; i < RPT; ++i) cur[i] = nxt[i];
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
        const int r = part + P * i, b = b0 + r;
        if (b >= a.B) continue;
        const size_t o = static_cast<size_t>(b) * H + j;
        float carried = dhBase[i];
#pragma unroll
        for (int p2 = 0; p2 < P; ++p2) carried += partS[(p2 * RB + r) * HS + jl];
        a.dh0[o] = carried * keepOf(a.mH0, o);
    }
}

// ---- dh += R dq on tensor cores -------------------------------------------------
//
// Same data flow as recurrentBackwardQ, but the per-step product runs as mma.sync m16n8k16:
// M = hidden rows k, N = batch tile (padded to 8), K = the 3H columns.  Warp w owns two m16 tiles
// (rows 32*(w/3) .. +31) and the K range of gate w%3; its A fragments (exact bf16 weight codes)
// stay in registers for the whole sequence.  dq, scaled per column, is split into three bf16
// terms in shared memory so that the products are exact and only the fp32 accumulation rounds.
template <int HT, int BT>  // H = 32*HT, blockDim = 96*HT
__global__ void __launch_bounds__(96 * HT) recurrentBackwardMma(const __grid_constant__ BackwardQArgs a,
                                                                const int32_t *__restrict__ Rq) {
    constexpr int H = 32 * HT, C = 3 * H, KS = 2 * HT;  // k16 steps per warp
    constexpr int CP = C + 8;                           // padded row of the bf16 dq tiles
    __shared__ __align__(16) uint16_t dqB[3][8][CP];    // [split][batch row][column]
    __shared__ float partS[3][BT][H];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nthreads = blockDim.x;
    const int g = lane >> 2, t4 = lane & 3;
    const int grp = warp % 3, mpair = warp / 3;
    const int b0 = blockIdx.x * BT, nb = min(BT, a.B - b0);

    // A fragments: rows mpair*32 + {0,16} + g (+8), columns grp*H + ks*16 + 2*t4 (+8)
    uint32_t afrag[2][KS][4];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int ks = 0; ks < KS; ++ks)
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int row = mpair * 32 + mt * 16 + g + (q & 1) * 8;
                const int col = grp * H + ks * 16 + 2 * t4 + (q >> 1) * 8;
                const int2 w = *reinterpret_cast<const int2 *>(Rq + static_cast<size_t>(row) * C + col);
                afrag[mt][ks][q] = (__float_as_uint(static_cast<float>(w.x)) >> 16) |
                                   (__float_as_uint(static_cast<float>(w.y)) & 0xffff0000u);
            }
    for (int i = tid; i < 3 * 8 * CP; i += nthreads) (&dqB[0][0][0])[i] = 0;
    for (int i = tid; i < 3 * BT * H; i += nthreads) (&partS[0][0][0])[i] = 0.0f;

    constexpr int kSlots = (BT + 2) / 3;
    const int elems = nb * H;
    float dhBase[kSlots];
    float scale[kSlots][3];
    StepOperands cur[kSlots], nxt[kSlots];
#pragma unroll
    for (int s2 = 0; s2 < kSlots; ++s2) {
        const int e = tid + s2 * nthreads;
        const int j = e % H;
        dhBase[s2] = (a.dhIn != nullptr && e < elems) ? a.dhIn[static_cast<size_t>(b0 + e / H) * H + j] : 0.0f;
        scale[s2][0] = a.scaleR[j]; scale[s2][1] = a.scaleR[H + j]; scale[s2][2] = a.scaleR[2 * H + j];
    }
    auto fetch = [&](int t, StepOperands (&dst)[kSlots]) {
#pragma unroll
        for (int s2 = 0; s2 < kSlots; ++s2) {
            const int e = tid + s2 * nthreads;
            if (e < elems) {
                const int b = e / H, j = e % H;
                const size_t row = static_cast<size_t>(t) * a.B + b0 + b;
                const size_t hi = row * H + j;
                const float *vRow = a.v + row * 4 * H;
                StepOperands o;
                o.z = vRow[j]; o.r = vRow[H + j]; o.g = vRow[2 * H + j]; o.qg = vRow[3 * H + j];
                o.hOld = a.h[hi];
                o.dhNew = a.dhNew[hi + static_cast<size_t>(a.B) * H];
                o.keepBits = a.stepBits ? a.stepBits[hi] : 0x1fffu;
                dst[s2] = o;
            }
        }
    };
    // Operands of a step several iterations ahead are pulled into L2, so that the register
    // prefetch of the next step is an L2 hit instead of an HBM round trip on the serial chain.
    constexpr int kAhead = 4;
    auto warmL2 = [&](int t) {
#pragma unroll
        for (int s2 = 0; s2 < kSlots; ++s2) {
            const int e = tid + s2 * nthreads;
            if (e < elems) {
                const int b = e / H, j = e % H;
                const size_t row = static_cast<size_t>(t) * a.B + b0 + b;
                const size_t hi = row * H + j;
                const float *vRow = a.v + row * 4 * H;
                prefetchL2(vRow + j); prefetchL2(vRow + H + j); prefetchL2(vRow + 2 * H + j); prefetchL2(vRow + 3 * H + j);
                prefetchL2(a.h + hi);
                prefetchL2(a.dhNew + hi + static_cast<size_t>(a.B) * H);
                if (a.stepBits) prefetchL2(a.stepBits + hi);
            }
        }
    };
    auto splitStore = [&](int b, int c, float v) {
        const float hi = bf16Lo(packBf16(v, 0.0f));
        const float r1 = v - hi;
        const float mid = bf16Lo(packBf16(r1, 0.0f));
        const float lo = r1 - mid;
        dqB[0][b][c] = static_cast<uint16_t>(__float_as_uint(hi) >> 16);
        dqB[1][b][c] = static_cast<uint16_t>(__float_as_uint(mid) >> 16);
        dqB[2][b][c] = static_cast<uint16_t>(packBf16(lo, 0.0f) & 0xffffu);
    };
    for (int t = a.T - 2; t >= 0 && t >= a.T - 1 - kAhead; --t) warmL2(t);
    fetch(a.T - 1, cur);
    __syncthreads();

    for (int t = a.T - 1; t >= 0; --t) {
        if (t > 0) fetch(t - 1, nxt);
        if (t - 1 - kAhead >= 0) warmL2(t - 1 - kAhead);
        const size_t rowBase = static_cast<size_t>(t) * a.B + b0;
#pragma unroll
        for (int s2 = 0; s2 < kSlots; ++s2) {
            const int e = tid + s2 * nthreads;
            if (e < elems) {
                const int b = e / H, j = e % H;
                const size_t gi = (rowBase + b) * C + j;
                const StepOperands o = cur[s2];
                auto keep = [&](int pos) { return static_cast<float>((o.keepBits >> pos) & 1u); };
                const float carried = dhBase[s2] + partS[0][b][j] + partS[1][b][j] + partS[2][b][j];
                const float dhTotal = (o.dhNew + carried) * keep(12);
                dhBase[s2] = o.z * dhTotal;
                const float dg = (1.0f - o.z) * dhTotal;
                const float dz = (o.hOld - o.g) * dhTotal;
                const float dpG = (1.0f - o.g * o.g) * dg * keep(2) * keep(5);
                const float dqG = dpG * o.r;
                const float dr = dpG * o.qg;
                const float dpR = (o.r * (1.0f - o.r)) * dr;
                const float dpZ = (o.z * (1.0f - o.z)) * dz;
                const float kz = keep(0) * keep(3), kr = keep(1) * keep(4);
                const float pz = dpZ * kz * keep(9), pr = dpR * kr * keep(10), pg = dpG * keep(11);
                const float qz = dpZ * kz * keep(6), qr = dpR * kr * keep(7), qn = dqG * keep(8);
                a.dp[gi] = pz; a.dp[gi + H] = pr; a.dp[gi + 2 * H] = pg;
                a.dq[gi] = qz; a.dq[gi + H] = qr; a.dq[gi + 2 * H] = qn;
                splitStore(b, j, qz * scale[s2][0]);
                splitStore(b, H + j, qr * scale[s2][1]);
                splitStore(b, 2 * H + j, qn * scale[s2][2]);
            }
        }
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
                    const uint32_t bf0 = *reinterpret_cast<const uint32_t *>(&dqB[sp][g][c0]);
                    const uint32_t bf1 = *reinterpret_cast<const uint32_t *>(&dqB[sp][g][c0 + 8]);
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
            // D fragment: (row g, cols 2*t4, 2*t4+1) and (row g+8, same cols); columns are batch rows
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int n = 2 * t4 + (q & 1);
                    const int k = mpair * 32 + mt * 16 + g + (q >> 1) * 8;
                    if (n < BT) partS[grp][n][k] = (acc[mt][2][q] + acc[mt][1][q]) + acc[mt][0][q];
                }
        }
#pragma unroll
        for (int s2 = 0; s2 < kSlots; ++s2) cur[s2] = nxt[s2];
        __syncthreads();
    }
#pragma unroll
    for (int s2 = 0; s2 < kSlots; ++s2) {
        const int e = tid + s2 * nthreads;
        if (e < elems) {
            const int b = e / H, j = e % H;
            const size_t o = static_cast<size_t>(b0 + b) * H + j;
            const float carried = dhBase[s2] + partS[0][b][j] + partS[1][b][j] + partS[2][b][j];
            a.dh0[o] = a.carryOut ? carried : carried * keepOf(a.mH0, o);
        }
    }
}

__global__ void transposeMatrix(const float *__restrict__ in, int rows, int cols, float *__restrict__ out) {
    __shared__ float tile[32][33];
    const int x = blockIdx.x * 32 + threadIdx.x, y0 = blockIdx.y * 32;
    for (int dy = threadIdx.y; dy < 32; dy += blockDim.y)
        if (x < cols && y0 + dy < rows) tile[dy][threadIdx.x] = in[static_cast<size_t>(y0 + dy) * cols + x];
    __syncthreads();
    const int ox = blockIdx.y * 32 + threadIdx.x, oy0 = blockIdx.x * 32;
    for (int dy = threadIdx.y; dy < 32; dy += blockDim.y)
        if (ox < rows && oy0 + dy < cols) out[static_cast<size_t>(oy0 + dy) * rows + ox] = tile[threadIdx.x][dy];
}

// partial[s][m][n] = sum over the s-th K chunk of A[k][m] * B[k][n].  64x64 tile, 16-deep K
// steps, 4x4 outputs per thread.
constexpr int kTile = 64, kDepth = 16;
__global__ void __launch_bounds__(256) gemmTN(const float *__restrict__ A, const float *__restrict__ Bm, int K, int M,
                                              int N, int chunk, float *__restrict__ partial) {
    __shared__ float As[kDepth][kTile + 4];
    __shared__ float Bs[kDepth][kTile + 4];
    const int m0 = blockIdx.y * kTile, n0 = blockIdx.x * kTile;
    const int kBegin = blockIdx.z * chunk, kEnd = min(K, kBegin + chunk);
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    float acc[4][4] = {};
    for (int k0 = kBegin; k0 < kEnd; k0 += kDepth) {
        for (int i = threadIdx.x; i < kDepth * kTile; i += 256) {
            const int kk = i / kTile, c = i % kTile;
            const int k = k0 + kk;
            As[kk][c] = (k < kEnd && m0 + c < M) ? A[static_cast<size_t>(k) * M + m0 + c] : 0.0f;
            Bs[kk][c] = (k < kEnd && n0 + c < N) ? Bm[static_cast<size_t>(k) * N + n0 + c] : 0.0f;
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

// ---- weight and bias gradients on tensor cores --------------------------------
//
// dW = x^T dp and dR = h^T dq contract over the T*B rows.  With activation grids of at most 8
// bits the left operand is an integer of magnitude <= 255 times one scale: exact in bf16.  The
// right operand (fp32 gradients) is split into three bf16 terms that carry all 24 significand
// bits, so every product is exact and only the fp32 accumulation rounds, as in an fp32 GEMM.
// A row of ones appended to the left operand yields the column sums, i.e. the bias gradients,
// from the same pass over dp / dq.  Split-K partials are reduced in a fixed order afterwards.
//
// Tile: all M rows (MT m16-tiles) x 64 columns per CTA, 8 warps = 8 n8-tiles, K chunks of 32
// staged in shared memory as [k][m] / [k][n] and read with transposing ldmatrix.
constexpr int kWgChunk = 32, kWgCols = 64;

using WeightGradProblem = wgrad::Problem;

// Loads of the next K chunk are issued into registers before the tensor work of the current
// chunk, so the HBM latency overlaps the MMAs; one shared-memory buffer, two barriers per chunk.
template <int MT>
__global__ void __launch_bounds__(256, 2) weightGradMma(const WeightGradProblem p, int K, int N, int chunkK) {
    constexpr int MP = MT * 16 + 8;       // padded row length (bf16 elements) of the A tile
    constexpr int NP = kWgCols + 8;
    constexpr int AV = (MT + 1) / 2;      // 4-element A vectors per thread and chunk (upper bound)
    __shared__ __align__(16) uint16_t As[kWgChunk][MP];
    __shared__ __align__(16) uint16_t Bs[3][kWgChunk][NP];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n0 = blockIdx.x * kWgCols;
    const int kBegin = blockIdx.y * chunkK, kEnd = min(K, kBegin + chunkK);
    const int M = p.M, M4 = M / 4;

    // constant part of the A tile: the ones column at m == M, zeros beyond
    for (int i = tid; i < kWgChunk * (MT * 16 - M); i += 256) {
        const int kk = i / (MT * 16 - M), m = M + i % (MT * 16 - M);
        As[kk][m] = (m == M) ? 0x3f80 : 0;
    }

    // per-thread slots of the chunk loads (fixed across chunks)
    int aRow[AV], aCol[AV];
#pragma unroll
    for (int v = 0; v < AV; ++v) {
        const int idx = tid + v * 256;
        aRow[v] = idx < kWgChunk * M4 ? idx / M4 : -1;
        aCol[v] = idx < kWgChunk * M4 ? (idx % M4) * 4 : 0;
    }
    const int bRow0 = tid / 16, bCol = (tid % 16) * 4;  // two B vectors per thread: rows bRow0, bRow0+16
    const bool bColOk = n0 + bCol < N;

    float4 aReg[AV], bReg[2];
    auto loadChunk = [&](int k0) {
#pragma unroll
        for (int v = 0; v < AV; ++v) {
            aReg[v] = make_float4(0.f, 0.f, 0.f, 0.f);
            const int k = k0 + aRow[v];
            if (aRow[v] >= 0 && k < kEnd) {
                if (p.aCodes) {
                    const int4 q = *reinterpret_cast<const int4 *>(p.aCodes + static_cast<size_t>(k) * M + aCol[v]);
                    aReg[v] = make_float4(static_cast<float>(q.x - p.aZero), static_cast<float>(q.y - p.aZero),
                                          static_cast<float>(q.z - p.aZero), static_cast<float>(q.w - p.aZero));
                } else {
                    aReg[v] = *reinterpret_cast<const float4 *>(p.aFloat + static_cast<size_t>(k) * M + aCol[v]);
                }
            }
        }
#pragma unroll
        for (int v = 0; v < 2; ++v) {
            const int k = k0 + bRow0 + v * 16;
            bReg[v] = (bColOk && k < kEnd) ? *reinterpret_cast<const float4 *>(p.B + static_cast<size_t>(k) * N + n0 + bCol)
                                           : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    auto storeChunk = [&]() {
#pragma unroll
        for (int v = 0; v < AV; ++v) {
            if (aRow[v] >= 0) {
                float4 a = aReg[v];
                if (!p.aCodes) {  // recover the integer code difference from the dequantized value
                    a.x = rintf(a.x * p.aInvScale) - p.aFloatZero; a.y = rintf(a.y * p.aInvScale) - p.aFloatZero;
                    a.z = rintf(a.z * p.aInvScale) - p.aFloatZero; a.w = rintf(a.w * p.aInvScale) - p.aFloatZero;
                }
                *reinterpret_cast<uint2 *>(&As[aRow[v]][aCol[v]]) = make_uint2(packBf16(a.x, a.y), packBf16(a.z, a.w));
            }
        }
#pragma unroll
        for (int v = 0; v < 2; ++v) {
            const float4 b = bReg[v];
            const uint32_t h0 = packBf16(b.x, b.y), h1 = packBf16(b.z, b.w);
            const float rx = b.x - bf16Lo(h0), ry = b.y - bf16Hi(h0), rz = b.z - bf16Lo(h1), rw = b.w - bf16Hi(h1);
            const uint32_t m0 = packBf16(rx, ry), m1 = packBf16(rz, rw);
            const uint32_t l0 = packBf16(rx - bf16Lo(m0), ry - bf16Hi(m0)), l1 = packBf16(rz - bf16Lo(m1), rw - bf16Hi(m1));
            const int row = bRow0 + v * 16;
            *reinterpret_cast<uint2 *>(&Bs[0][row][bCol]) = make_uint2(h0, h1);
            *reinterpret_cast<uint2 *>(&Bs[1][row][bCol]) = make_uint2(m0, m1);
            *reinterpret_cast<uint2 *>(&Bs[2][row][bCol]) = make_uint2(l0, l1);
        }
    };

    float acc[MT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f;

    loadChunk(kBegin);
    storeChunk();
    __syncthreads();
    for (int k0 = kBegin; k0 < kEnd; k0 += kWgChunk) {
        const bool more = k0 + kWgChunk < kEnd;
        if (more) loadChunk(k0 + kWgChunk);
#pragma unroll
        for (int ks = 0; ks < kWgChunk; ks += 16) {
            uint32_t b[3][2];
#pragma unroll
            for (int sp = 0; sp < 3; ++sp) {
                const uint32_t addr = static_cast<uint32_t>(
                    __cvta_generic_to_shared(&Bs[sp][ks + (lane & 7) + ((lane >> 3) & 1) * 8][warp * 8]));
                asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];"
                             : "=r"(b[sp][0]), "=r"(b[sp][1]) : "r"(addr));
            }
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                uint32_t a[4];
                const int id = lane >> 3, r = lane & 7;
                const uint32_t addr = static_cast<uint32_t>(
                    __cvta_generic_to_shared(&As[ks + (id >> 1) * 8 + r][mt * 16 + (id & 1) * 8]));
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]) : "r"(addr));
#pragma unroll
                for (int sp = 0; sp < 3; ++sp) {
                    asm volatile(
                        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                        "{%0,%1,%2,%3};"
                        : "+f"(acc[mt][0]), "+f"(acc[mt][1]), "+f"(acc[mt][2]), "+f"(acc[mt][3])
                        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[sp][0]), "r"(b[sp][1]));
                }
            }
        }
        __syncthreads();
        if (more) storeChunk();
        __syncthreads();
    }
    float *out = p.partial + static_cast<size_t>(blockIdx.y) * (M + 1) * N;
    const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int m = mt * 16 + g + half * 8;
            const int n = n0 + warp * 8 + 2 * t4;
            if (m <= M && n < N)
                *reinterpret_cast<float2 *>(out + static_cast<size_t>(m) * N + n) =
                    make_float2(acc[mt][half * 2], acc[mt][half * 2 + 1]);
        }
    }
}

// weight[m][n] = scale * mask * sum_s partial[s][m][n] (m < M); bias[n] = biasMask * sum_s partial[s][M][n].
// A CTA owns 64 outputs; its four thread layers each sum every fourth split and layer 0 adds the
// four sums in layer order, so the result does not depend on the launch.
// A set status word (a bounded wait of the producing kernel gave up) turns the results into NaN.
// One launch reduces both problems of a step (blockIdx.y: 0 = input weights, 1 = recurrent weights).
constexpr int kReduceLayers = 4, kReduceWidth = 64;
struct ReduceJob {
    const float *partial;
    int splits, M;
    float scale;
    const uint8_t *weightMask, *biasMask;
    float *weight, *bias;
};
__global__ void __launch_bounds__(kReduceWidth * kReduceLayers)
reduceWeightGrad(const ReduceJob jobX, const ReduceJob jobH, int N, const int *__restrict__ status) {
    __shared__ float layer[kReduceLayers][kReduceWidth];
    const ReduceJob &job = blockIdx.y == 0 ? jobX : jobH;
    const float *__restrict__ partial = job.partial;
    const int splits = job.splits, M = job.M;
    const float scale = job.scale;
    const uint8_t *__restrict__ weightMask = job.weightMask, *__restrict__ biasMask = job.biasMask;
    float *__restrict__ weight = job.weight, *__restrict__ bias = job.bias;
    const size_t total = static_cast<size_t>(M + 1) * N;
    if (static_cast<size_t>(blockIdx.x) * kReduceWidth >= total) return;  // the other problem is larger
    const size_t i = static_cast<size_t>(blockIdx.x) * kReduceWidth + threadIdx.x;
    float s = 0.0f;
    if (i < total) {
#pragma unroll 4
        for (int sp = threadIdx.y; sp < splits; sp += kReduceLayers) s += partial[static_cast<size_t>(sp) * total + i];
    }
    layer[threadIdx.y][threadIdx.x] = s;
    __syncthreads();
    if (threadIdx.y != 0 || i >= total) return;
    s = layer[0][threadIdx.x];
#pragma unroll
    for (int l = 1; l < kReduceLayers; ++l) s += layer[l][threadIdx.x];
    if (status && *status) s = __int_as_float(0x7fc00000);
    const size_t m = i / N, n = i % N;
    if (m < static_cast<size_t>(M)) weight[i] = s * scale * keepOf(weightMask, i);
    else bias[n] = s * keepOf(biasMask, n);
}

// out[i] = mask[i] * sum_s partial[s][i], s ascending.
__global__ void reduceSplits(const float *__restrict__ partial, int splits, size_t n, const uint8_t *__restrict__ mask,
                             float *__restrict__ out) {
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float s = 0.0f;
        for (int p = 0; p < splits; ++p) s += partial[static_cast<size_t>(p) * n + i];
        out[i] = s * keepOf(mask, i);
    }
}

// out[m][n] = mask * sum_k A[m][k] * B[n][k]   (both operands K-contiguous).  Used for
// dx = dp W^T: M = T*B rows, N = I, K = 3H.  64x64 tile, 32-deep K steps, 4x4 outputs per thread;
// tiles are stored K-major in shared memory so that the inner product reads are conflict free.
constexpr int kNtDepth = 32;
__global__ void __launch_bounds__(256) gemmNT(const float *__restrict__ A, const float *__restrict__ Bm, int M, int N,
                                              int K, const uint8_t *__restrict__ mask, float *__restrict__ out) {
    __shared__ float As[kNtDepth][kTile + 1];
    __shared__ float Bs[kNtDepth][kTile + 1];
    const int m0 = blockIdx.x * kTile, n0 = blockIdx.y * kTile;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += kNtDepth) {
        for (int i = threadIdx.x; i < kTile * kNtDepth; i += 256) {
            const int r = i / kNtDepth, kk = i % kNtDepth;
            const int k = k0 + kk;
            As[kk][r] = (m0 + r < M && k < K) ? A[static_cast<size_t>(m0 + r) * K + k] : 0.0f;
            Bs[kk][r] = (n0 + r < N && k < K) ? Bm[static_cast<size_t>(n0 + r) * K + k] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kNtDepth; ++kk) {
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

// partial[s][c] = sum over the s-th row chunk of g[n][c]; blockIdx.y selects dp or dq.
__global__ void columnSums(const float *__restrict__ dp, const float *__restrict__ dq, int rows, int C, int chunk,
                           float *__restrict__ partial) {
    const float *g = blockIdx.y == 0 ? dp : dq;
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

constexpr int kBiasSplits = 64;

}  // namespace

}  // namespace gru

namespace wgrad {

constexpr int kMaxSms = 160;

Plan plan(int K, int M, int N, int sms) {
    Plan pl;
    sms = std::min(sms, kMaxSms);
    pl.tensorMemory = tensorMemoryPath(M, N);
    if (pl.tensorMemory) {
        pl.splits = planTensorMemory(K, N, sms, &pl.chunkK);
        return pl;
    }
    const int nTiles = (N + gru::kWgCols - 1) / gru::kWgCols;
    const int splits = std::max(1, std::min((2 * sms + 2 * nTiles - 1) / (2 * nTiles), (K + 255) / 256));
    pl.chunkK = ((K + splits - 1) / splits + gru::kWgChunk - 1) / gru::kWgChunk * gru::kWgChunk;
    pl.splits = (K + pl.chunkK - 1) / pl.chunkK;
    return pl;
}

int splitBound(int K, int M, int N) {
    // both kernels ask for about two CTAs per SM spread over the column tiles
    (void)M;
    return std::max(1, std::min((K + gru::kWgChunk - 1) / gru::kWgChunk, 2 * kMaxSms + 8));
}

void launch(const Problem &prob, int K, int N, const Plan &pl, cudaStream_t st) {
    if (pl.tensorMemory) {
        launchTensorMemory(prob, nullptr, K, N, pl.chunkK, pl.splits, st);
        return;
    }
    const int chunkK = pl.chunkK;
    const int mt = (prob.M + 1 + 15) / 16;
    const dim3 grid((N + gru::kWgCols - 1) / gru::kWgCols, pl.splits);
    KernelTimer timer__("weightGradMma", st);
    switch (mt) {
#define RXMET_WG_CASE(MTV) case MTV: gru::weightGradMma<MTV><<<grid, 256, 0, st>>>(prob, K, N, chunkK); break;
        RXMET_WG_CASE(1) RXMET_WG_CASE(2) RXMET_WG_CASE(3) RXMET_WG_CASE(4) RXMET_WG_CASE(5)
        RXMET_WG_CASE(6) RXMET_WG_CASE(7) RXMET_WG_CASE(8) RXMET_WG_CASE(9)
#undef RXMET_WG_CASE
        default: fail(RXMET_ERR_UNSUPPORTED, "weight gradient tile count %d", mt);
    }
}

void launchPair(const Problem &a, const Plan &planA, const Problem &b, const Plan &planB, int K, int N, cudaStream_t st) {
    if (planA.tensorMemory && planB.tensorMemory && planA.splits == planB.splits && planA.chunkK == planB.chunkK &&
        a.status == b.status) {
        if (launchPairStreamed(a, b, K, N, planA.chunkK, planA.splits, st)) return;
        const bool aFirst = a.M >= b.M;
        launchTensorMemory(aFirst ? a : b, aFirst ? &b : &a, K, N, planA.chunkK, planA.splits, st);
        return;
    }
    launch(a, K, N, planA, st);
    launch(b, K, N, planB, st);
}

}  // namespace wgrad

namespace gru {

size_t backwardWorkspaceBytes(int T, int B, int I, int H) {
    const size_t rows = static_cast<size_t>(T) * B, C = 3 * static_cast<size_t>(H);
    WorkspaceSizer ws;
    ws.take<float>(rows * C);          // dp
    ws.take<float>(rows * C);          // dq
    ws.take<float>(C * H);             // R transposed
    ws.take<uint32_t>(3 * 64 * static_cast<size_t>(H));  // packed recurrent codes
    ws.take<uint16_t>(rows * H);                         // packed per-step keep flags
    ws.take<float>(static_cast<size_t>(I) * C);  // W real-valued
    ws.take<float>(static_cast<size_t>(H) * C);  // R real-valued
    ws.take<float>(rows * I);          // x real-valued
    ws.take<float>(12 * C);            // per-channel block
    const size_t splitW = splitsFor(static_cast<int>(rows), ((I + kTile - 1) / kTile) * ((static_cast<int>(C) + kTile - 1) / kTile));
    const size_t splitR = splitsFor(static_cast<int>(rows), ((H + kTile - 1) / kTile) * ((static_cast<int>(C) + kTile - 1) / kTile));
    ws.take<float>(splitW * I * C);
    ws.take<float>(splitR * H * C);
    ws.take<float>(2 * kBiasSplits * C);
    // tensor-core path: split-K partials of (I+1) and (H+1) rows and the status word
    // (the slab form of the same kernel, for more than 128 rows or 16-bit codes, asks for fewer splits)
    ws.take<float>(static_cast<size_t>(std::max(wgrad::slabSplitBound(I, H, static_cast<int>(C)),
                                                I <= 143 ? wgrad::splitBound(static_cast<int>(rows), I, static_cast<int>(C)) : 1)) * (I + 1) * C);
    ws.take<float>(static_cast<size_t>(std::max(wgrad::slabSplitBound(I, H, static_cast<int>(C)),
                                                H <= 143 ? wgrad::splitBound(static_cast<int>(rows), H, static_cast<int>(C)) : 1)) * (H + 1) * C);
    ws.take<int>(64);
    ws.take<float>(static_cast<size_t>(B) * H);   // gradient carried between time chunks
    ws.take<uint8_t>(igrad::widePackedBytes(static_cast<int>(C), I) + 256);   // weight operand of the streaming input-gradient kernel
    return ws.used() + 4096;
}

void backward(const BackwardCall &call, void *workspace, size_t workspaceBytes, cudaStream_t st) {
    const int T = call.T, B = call.B, I = call.I, H = call.H, C = 3 * H;
    const size_t rows = static_cast<size_t>(T) * B;
    Workspace ws(workspace, workspaceBytes);
    float *dp = ws.take<float>(rows * C);
    float *dq = ws.take<float>(rows * C);
    float *RT = ws.take<float>(static_cast<size_t>(C) * H);
    const rxmet_gru_masks none{};
    const rxmet_gru_masks &mk = call.masks ? *call.masks : none;

    const int smemMax = currentDevice().smemMax, sms = currentDevice().sms;
    int bt = (B > 2 * sms) ? 4 : ((B > sms) ? 2 : 1);
    if (const char *env = std::getenv("RXMET_GRU_BWD_BT")) bt = std::atoi(env);
    if (bt != 1 && bt != 2 && bt != 4) bt = 2;

    // Which kernels take the saved integer codes directly (QAT on 8-bit grids).
    const bool qat = call.W_q != nullptr;
    if (qat) RXMET_REQUIRE(call.exec != nullptr, "backward: quantized operands need execution parameters");
    if (call.stepFlags && !(qat && call.exec->weightClass == CodeClass::I8 && H <= 128 && std::getenv("RXMET_GRU_BWD_GENERIC") == nullptr))
        fail(RXMET_ERR_UNSUPPORTED, "packed step flags are read by the 8-bit register path of the backward only");
    const bool simtGrads = std::getenv("RXMET_GRU_GRAD_SIMT") != nullptr;
    const bool registerPath = qat && call.exec->weightClass == CodeClass::I8 && H <= 128 &&
                              std::getenv("RXMET_GRU_BWD_GENERIC") == nullptr;
    // The tcgen05 kernels read the saved codes with 16-byte copies and store dx as float4 (x mask:
    // 8-byte loads); callers' buffers that are not aligned that way take the scalar kernels.
    const bool tensorInputGrad = qat && call.exec->weightClass == CodeClass::I8 && igrad::eligible(C, I) && !simtGrads &&
                                 alignedTo(call.dx, 16) && alignedTo(mk.x, 8) && alignedTo(call.W_q, 16);
    const bool tensorGrads = qat && call.exec->actClass == CodeClass::I8 && I + 1 <= 144 && H + 1 <= 144 && I % 4 == 0 &&
                             H % 4 == 0 && !simtGrads && alignedTo(call.x_q, 16) && alignedTo(call.h, 16);
    // More than 128 rows or 16-bit activation codes: the same tcgen05 kernel over 128-row slabs, two exact
    // bf16 terms per code when the grid is wider than 8 bits.
    const bool wideCodes = qat && call.exec->actClass != CodeClass::I8;
    const bool slabGrads = qat && !tensorGrads && !simtGrads && call.exec->actClass != CodeClass::I32 && I % 4 == 0 && H % 4 == 0 &&
                           alignedTo(call.x_q, 16) && alignedTo(call.h, 16) && wgrad::slabPathTakes(I, H, C);

    const float *W = call.W, *R = call.R, *x = call.x;
    const float *chanScaleR = nullptr, *chanScaleW = nullptr;
    if (qat) {  // rebuild the real-valued operands that the remaining float kernels read
        const Exec &e = *call.exec;
        float *Wf = ws.take<float>(static_cast<size_t>(I) * C);
        float *Rf = ws.take<float>(static_cast<size_t>(H) * C);
        float *xf = ws.take<float>(rows * I);
        float *chan = ws.take<float>(2 * static_cast<size_t>(C));
        // effective scales of W then R: the first two arrays of the page-locked per-channel block
        RXMET_CUDA(cudaMemcpyAsync(chan, pinnedChannelBlock(e, st), 2 * sizeof(float) * C, cudaMemcpyHostToDevice, st));
        if (!tensorInputGrad) {
            KernelTimer timer__("dequantCodes", st);
            dequantCodes<<<gridFor(static_cast<size_t>(I) * C, 256), 256, 0, st>>>(call.W_q, static_cast<size_t>(I) * C, C, chan, 0.f, 0, Wf);
            afterLaunch("dequantCodes");
        }
        if (!registerPath) {
            KernelTimer timer__("dequantCodes", st);
            dequantCodes<<<gridFor(static_cast<size_t>(H) * C, 256), 256, 0, st>>>(call.R_q, static_cast<size_t>(H) * C, C, chan + C, 0.f, 0, Rf);
            afterLaunch("dequantCodes");
        }
        if (!tensorGrads && !slabGrads) {
            KernelTimer timer__("dequantCodes", st);
            dequantCodes<<<gridFor(rows * I, 256), 256, 0, st>>>(call.x_q, rows * I, I, nullptr, e.gate.eff[RXMET_GRU_X],
                                                                e.gate.zp[RXMET_GRU_X], xf);
            afterLaunch("dequantCodes");
        }
        W = Wf; R = Rf; x = xf;
        chanScaleR = chan + C;
        chanScaleW = chan;
    }

    // H > 128 with 8-bit weight codes: the codes stay in shared memory for the whole sequence
    const int hpCodes = (H + 31) / 32 * 32;
    const int partsCodes = std::max(1, std::min(4, 512 / hpCodes));
    auto codesSmem = [&](int rb) {
        return static_cast<size_t>(C) * H + sizeof(float) * (static_cast<size_t>(rb) * C + static_cast<size_t>(partsCodes) * rb * H);
    };
    const bool codesPath = qat && !registerPath && call.exec->weightClass == CodeClass::I8 && C % 4 == 0 && hpCodes <= 512 &&
                           codesSmem(1) + 1024 <= static_cast<size_t>(smemMax) && alignedTo(call.R_q, 16) &&
                           std::getenv("RXMET_GRU_BWD_GENERIC") == nullptr;
    if (codesPath) {
        BackwardCodesArgs ca{};
        BackwardQArgs &q = ca.q;
        if (mk.weight_ih_linear || mk.weight_hh_linear || mk.gate_input || mk.gate_output || mk.h) {
            uint16_t *bits = ws.take<uint16_t>(rows * H);
            {
                KernelTimer timer__("packStepMasks", st);
                auto aligned4 = [](const void *ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 3u) == 0; };
                if (H % 4 == 0 && aligned4(mk.weight_ih_linear) && aligned4(mk.weight_hh_linear) && aligned4(mk.gate_input) &&
                    aligned4(mk.gate_output) && aligned4(mk.h))
                    packStepMasks4<<<gridFor(rows * H / 4, 256), 256, 0, st>>>(mk.weight_ih_linear, mk.weight_hh_linear, mk.gate_input,
                                                                              mk.gate_output, mk.h, rows * H / 4, H,
                                                                              reinterpret_cast<uint2 *>(bits));
                else
                    packStepMasks<<<gridFor(rows * H, 256), 256, 0, st>>>(mk.weight_ih_linear, mk.weight_hh_linear,
                                                                          mk.gate_input, mk.gate_output, mk.h, rows, H, bits);
            }
            afterLaunch("packStepMasks");
            q.stepBits = bits;
        }
        q.T = T; q.B = B; q.H = H; q.scaleR = chanScaleR;
        q.h = call.h; q.v = call.v; q.dhNew = call.dh_new; q.dp = dp; q.dq = dq; q.dh0 = call.dh0;
        q.mIh = mk.weight_ih_linear; q.mHh = mk.weight_hh_linear; q.mGateIn = mk.gate_input;
        q.mGateOut = mk.gate_output; q.mH = mk.h; q.mH0 = mk.h0;
        ca.Rq = call.R_q; ca.HP = hpCodes; ca.parts = partsCodes;
        // H = 256, opt-in (RXMET_GRU_BWD_CLUSTER): the cluster kernel, weights as fp32 in the registers of eight CTAs.
        // Correct, but measured slower than the kernel below at T = 100, B = 128 (0.59 against 0.51 ms): eight
        // warps per SM issue at 40 %, and only 15 clusters of eight are resident on this part.
        bool clusterRan = false;
        if (H == 256 && std::getenv("RXMET_GRU_BWD_CLUSTER") != nullptr) {
            BackwardClusterArgs cl{};
            cl.q = q; cl.Rq = call.R_q;
            const int rbCluster = B * concurrentPasses() * kClusterCtas > 8 * sms ? 16 : 8;
            const size_t smem = sizeof(float) * (2 * static_cast<size_t>(rbCluster) * C + static_cast<size_t>(kClusterParts) * rbCluster * (H / kClusterCtas));
            const int clusters = (B + rbCluster - 1) / rbCluster;
            auto launchCluster = [&](auto kernel) -> bool {
                ensureDynamicSmem(reinterpret_cast<const void *>(kernel), smem);
                cudaLaunchConfig_t cfg{};
                cfg.gridDim = dim3(static_cast<unsigned>(clusters * kClusterCtas));
                cfg.blockDim = dim3((H / kClusterCtas) * kClusterParts);
                cfg.dynamicSmemBytes = smem;
                cfg.stream = st;
                cudaLaunchAttribute clusterDim{};
                clusterDim.id = cudaLaunchAttributeClusterDimension;
                clusterDim.val.clusterDim.x = kClusterCtas;
                clusterDim.val.clusterDim.y = 1;
                clusterDim.val.clusterDim.z = 1;
                cfg.attrs = &clusterDim;
                cfg.numAttrs = 1;
                int resident = 0;
                if (cudaOccupancyMaxActiveClusters(&resident, kernel, &cfg) != cudaSuccess || resident < 1) {
                    cudaGetLastError();
                    return false;
                }
                if (std::getenv("RXMET_DEBUG_CLUSTER")) std::fprintf(stderr, "cluster backward: %d clusters of %d rows, %d resident at most\n", clusters, rbCluster, resident);
                KernelTimer timer__("recurrentBackward", st);
                RXMET_CUDA(cudaLaunchKernelEx(&cfg, kernel, cl));
                return true;
            };
            clusterRan = rbCluster == 16 ? launchCluster(recurrentBackwardCluster<96, 16>) : launchCluster(recurrentBackwardCluster<96, 8>);
            if (clusterRan) afterLaunch("recurrentBackwardCluster");
        }
        if (!clusterRan) {
            int rb = 1;
            const int want = std::max(1, (B + smsPerPass() - 1) / smsPerPass());
            while (rb < 4 && rb < want && codesSmem(rb * 2) + 1024 <= static_cast<size_t>(smemMax)) rb *= 2;
            auto launchCodes = [&](auto kernel) {
                const size_t smem = codesSmem(rb);
                ensureDynamicSmem(reinterpret_cast<const void *>(kernel), smem);
                KernelTimer timer__("recurrentBackward", st);
                kernel<<<(B + rb - 1) / rb, hpCodes * partsCodes, smem, st>>>(ca);
            };
            if (rb == 1) launchCodes(recurrentBackwardCodes<1>);
            else if (rb == 2) launchCodes(recurrentBackwardCodes<2>);
            else launchCodes(recurrentBackwardCodes<4>);
            afterLaunch("recurrentBackward");
        }
    } else if (registerPath) {
        const int CW = H <= 32 ? 16 : (H <= 64 ? 32 : 64);
        // The tensor-core kernel takes its fragments from the integer codes themselves; only the
        // register kernel reads the packed pairs.
        const bool mmaPath = H % 32 == 0 && std::getenv("RXMET_GRU_BWD_SIMT") == nullptr;
        uint32_t *RB = nullptr;
        if (!mmaPath) {
            RB = ws.take<uint32_t>(3 * static_cast<size_t>(CW) * H);
            KernelTimer timer__("packRecurrentBf16", st);
            packRecurrentBf16<<<gridFor(3 * static_cast<size_t>(CW) * H, 256), 256, 0, st>>>(call.R_q, H, CW, RB);
            afterLaunch("packRecurrentBf16");
        }
        BackwardQArgs q{};
        if (call.stepFlags) {
            q.stepBits = call.stepFlags;   // packed by the forward itself
        } else if (mk.weight_ih_linear || mk.weight_hh_linear || mk.gate_input || mk.gate_output || mk.h) {
            uint16_t *bits = ws.take<uint16_t>(rows * H);
            {
                KernelTimer timer__("packStepMasks", st);
                auto aligned4 = [](const void *ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 3u) == 0; };
                if (H % 4 == 0 && aligned4(mk.weight_ih_linear) && aligned4(mk.weight_hh_linear) && aligned4(mk.gate_input) &&
                    aligned4(mk.gate_output) && aligned4(mk.h))
                    packStepMasks4<<<gridFor(rows * H / 4, 256), 256, 0, st>>>(mk.weight_ih_linear, mk.weight_hh_linear, mk.gate_input,
                                                                              mk.gate_output, mk.h, rows * H / 4, H,
                                                                              reinterpret_cast<uint2 *>(bits));
                else
                    packStepMasks<<<gridFor(rows * H, 256), 256, 0, st>>>(mk.weight_ih_linear, mk.weight_hh_linear,
                                                                          mk.gate_input, mk.gate_output, mk.h, rows, H, bits);
            }
            afterLaunch("packStepMasks");
            q.stepBits = bits;
        }
        q.T = T; q.B = B; q.H = H; q.RB = RB; q.scaleR = chanScaleR;
        q.h = call.h; q.v = call.v; q.dhNew = call.dh_new; q.dp = dp; q.dq = dq; q.dh0 = call.dh0;
        q.mIh = mk.weight_ih_linear; q.mHh = mk.weight_hh_linear; q.mGateIn = mk.gate_input;
        q.mGateOut = mk.gate_output; q.mH = mk.h; q.mH0 = mk.h0;
        const size_t smem = sizeof(float) * (static_cast<size_t>(bt) * 3 * 2 * CW + 3 * static_cast<size_t>(bt) * H);
        const int grid = (B + bt - 1) / bt;
        auto launchMma = [&](const BackwardQArgs &qa) {
            KernelTimer timer__("recurrentBackward", st);
#define RXMET_BWD_CASE(HTV, BTV) \
    if (H == 32 * HTV && bt == BTV) recurrentBackwardMma<HTV, BTV><<<grid, 96 * HTV, 0, st>>>(qa, call.R_q);
            RXMET_BWD_CASE(1, 1) RXMET_BWD_CASE(1, 2) RXMET_BWD_CASE(1, 4)
            RXMET_BWD_CASE(2, 1) RXMET_BWD_CASE(2, 2) RXMET_BWD_CASE(2, 4)
            RXMET_BWD_CASE(3, 1) RXMET_BWD_CASE(3, 2) RXMET_BWD_CASE(3, 4)
            RXMET_BWD_CASE(4, 1) RXMET_BWD_CASE(4, 2) RXMET_BWD_CASE(4, 4)
#undef RXMET_BWD_CASE
        };
        // Time chunks, latest first: while the recurrence of chunk i + 1 occupies the caller's stream, the
        // gradient GEMMs of chunk i (dx rows, dW / dR partial sums) run on the library's second stream; only the
        // last (short) chunk's GEMMs and the reduction of the partial sums stay behind the recurrence.
        std::vector<int> chunks{T};
        if (mmaPath && tensorInputGrad && tensorGrads && (static_cast<size_t>(B) * I) % 8 == 0)
            chunks = overlapChunks(T, rows, true);
        std::vector<wgrad::Plan> plans;
        int totalSplits = 0;
        if (chunks.size() > 1) {
            int share = 100;
            if (const char *env = std::getenv("RXMET_GRU_CHUNK_SMS")) share = std::max(5, std::min(100, std::atoi(env)));
            for (size_t i = 0; i < chunks.size(); ++i) {
                const int K = chunks[i] * B;
                const int use = (i + 1 == chunks.size()) ? sms : std::max(4, sms * share / 100);
                const wgrad::Plan px = wgrad::plan(K, I, C, use), ph = wgrad::plan(K, H, C, use);
                if (!px.tensorMemory || !ph.tensorMemory || px.splits != ph.splits || px.chunkK != ph.chunkK) { plans.clear(); break; }
                plans.push_back(px);
                totalSplits += px.splits;
            }
            const int bound = std::min(wgrad::splitBound(static_cast<int>(rows), I, C), wgrad::splitBound(static_cast<int>(rows), H, C));
            if (plans.size() != chunks.size() || totalSplits > bound) chunks.assign(1, T);
        }
        if (chunks.size() > 1) {
            const Exec &e = *call.exec;
            OverlapLane &lane = overlapLane();
            float *carry = ws.take<float>(static_cast<size_t>(B) * H);
            int *status = ws.take<int>(1);
            RXMET_CUDA(cudaMemsetAsync(status, 0, sizeof(int), st));
            float *partialX = ws.take<float>(static_cast<size_t>(totalSplits) * (I + 1) * C);
            float *partialH = ws.take<float>(static_cast<size_t>(totalSplits) * (H + 1) * C);
            uint8_t *packedW = nullptr;
            if (const size_t bytes = igrad::widePackedBytes(C, I)) packedW = ws.take<uint8_t>(bytes);
            int tEnd = T, splitBase = 0;
            for (size_t i = 0; i < chunks.size(); ++i) {
                const int n = chunks[i], t0 = tEnd - n;
                const size_t r0 = static_cast<size_t>(t0) * B;
                const bool more = i + 1 < chunks.size();
                BackwardQArgs qa = q;
                qa.T = n;
                qa.h = q.h + r0 * H; qa.v = q.v + r0 * 4 * H; qa.dhNew = q.dhNew + r0 * H;
                qa.dp = dp + r0 * C; qa.dq = dq + r0 * C;
                if (q.stepBits) qa.stepBits = q.stepBits + r0 * H;
                qa.dhIn = i > 0 ? carry : nullptr;
                qa.carryOut = more ? 1 : 0;
                qa.dh0 = more ? carry : call.dh0;
                launchMma(qa);
                afterLaunch("recurrentBackwardMma");
                RXMET_CUDA(cudaEventRecord(lane.fork[i], st));
                RXMET_CUDA(cudaStreamWaitEvent(lane.stream, lane.fork[i], 0));
                const int K = n * B;
                igrad::Problem pg{};
                pg.G = dp + r0 * C; pg.kScale = chanScaleW; pg.codesNK = call.W_q; pg.rows = K; pg.K = C; pg.N = I;
                pg.mask = mk.x ? mk.x + r0 * I : nullptr; pg.maskKeeps = 1; pg.out = call.dx + r0 * I; pg.status = status;
                pg.packed = packedW;
                igrad::launch(pg, sms, lane.stream);
                afterLaunch("inputGradUmma");
                WeightGradProblem px{}, ph{};
                px.aCodes = call.x_q + r0 * I; px.aZero = e.gate.zp[RXMET_GRU_X]; px.M = I; px.B = dp + r0 * C;
                px.partial = partialX + static_cast<size_t>(splitBase) * (I + 1) * C;
                ph.aFloat = call.h + r0 * H; ph.aInvScale = 1.0f / e.gate.eff[RXMET_GRU_H]; ph.M = H; ph.B = dq + r0 * C;
                ph.partial = partialH + static_cast<size_t>(splitBase) * (H + 1) * C;
                px.status = ph.status = status;
                wgrad::launchPair(px, plans[i], ph, plans[i], K, C, lane.stream);
                afterLaunch("weightGrad");
                splitBase += plans[i].splits;
                tEnd = t0;
            }
            RXMET_CUDA(cudaEventRecord(lane.done[0], lane.stream));
            RXMET_CUDA(cudaStreamWaitEvent(st, lane.done[0], 0));
            {
                const ReduceJob jobX{partialX, totalSplits, I, e.gate.eff[RXMET_GRU_X], mk.W, mk.bw, call.dW, call.dbw};
                const ReduceJob jobH{partialH, totalSplits, H, e.gate.eff[RXMET_GRU_H], mk.R, mk.br, call.dR, call.dbr};
                const size_t largest = static_cast<size_t>(std::max(I, H) + 1) * C;
                KernelTimer timer__("reduceWeightGrad", st);
                reduceWeightGrad<<<dim3(static_cast<unsigned>((largest + kReduceWidth - 1) / kReduceWidth), 2),
                                   dim3(kReduceWidth, kReduceLayers), 0, st>>>(jobX, jobH, C, status);
            }
            afterLaunch("reduceWeightGrad");
            return;
        }
        if (mmaPath) {
            launchMma(q);
        } else {
            KernelTimer timer__("recurrentBackward", st);
#define RXMET_BWD_CASE(CWV, BTV) \
    if (CW == CWV && bt == BTV) recurrentBackwardQ<CWV, BTV><<<grid, 3 * H, smem, st>>>(q);
            RXMET_BWD_CASE(16, 1) RXMET_BWD_CASE(16, 2) RXMET_BWD_CASE(16, 4)
            RXMET_BWD_CASE(32, 1) RXMET_BWD_CASE(32, 2) RXMET_BWD_CASE(32, 4)
            RXMET_BWD_CASE(64, 1) RXMET_BWD_CASE(64, 2) RXMET_BWD_CASE(64, 4)
#undef RXMET_BWD_CASE
        }
        afterLaunch("recurrentBackwardQ");
    } else {
        {
            KernelTimer timer__("transposeMatrix", st);
            transposeMatrix<<<dim3((C + 31) / 32, (H + 31) / 32), dim3(32, 8), 0, st>>>(R, H, C, RT);
        }
        afterLaunch("transposeMatrix");

        BackwardArgs a{};
        a.T = T; a.B = B; a.H = H;
        a.RT = RT; a.h = call.h; a.v = call.v; a.dhNew = call.dh_new; a.dp = dp; a.dq = dq; a.dh0 = call.dh0;
        a.mIh = mk.weight_ih_linear; a.mHh = mk.weight_hh_linear; a.mGateIn = mk.gate_input;
        a.mGateOut = mk.gate_output; a.mH = mk.h; a.mH0 = mk.h0;
        const int block = std::min(std::max((C + 31) / 32 * 32, 128), 768);
        a.parts = std::max(1, std::min(block / std::max(H, 1), 8));
        auto launch = [&](auto kernel, int BT) {
            const size_t base = sizeof(float) * (static_cast<size_t>(BT) * H + static_cast<size_t>(BT) * C +
                                                 static_cast<size_t>(a.parts) * BT * H);
            const size_t full = base + sizeof(float) * static_cast<size_t>(C) * H;
            a.weightsInSmem = full <= static_cast<size_t>(smemMax) ? 1 : 0;
            const size_t smem = a.weightsInSmem ? full : base;
            if (smem > static_cast<size_t>(smemMax))
                fail(RXMET_ERR_UNSUPPORTED, "hidden size %d needs %zu bytes of shared memory per CTA", H, smem);
            ensureDynamicSmem(reinterpret_cast<const void *>(kernel), smem);
            KernelTimer timer__("recurrentBackward", st);
            kernel<<<(B + BT - 1) / BT, block, smem, st>>>(a);
        };
        if (bt == 4) launch(recurrentBackward<4>, 4);
        else if (bt == 2) launch(recurrentBackward<2>, 2);
        else launch(recurrentBackward<1>, 1);
        afterLaunch("recurrentBackward");
    }

    // dx
    int *status = ws.take<int>(1);  // set by a tcgen05 kernel whose bounded wait gave up
    if (call.W_q) RXMET_CUDA(cudaMemsetAsync(status, 0, sizeof(int), st));
    if (tensorInputGrad) {
        // QAT: gradients times the integer weight codes on the tensor cores, scales folded into the gradients
        igrad::Problem pg{};
        pg.G = dp; pg.kScale = chanScaleW; pg.codesNK = call.W_q; pg.rows = static_cast<int>(rows); pg.K = C; pg.N = I;
        pg.mask = mk.x; pg.maskKeeps = 1; pg.out = call.dx; pg.status = status;
        if (const size_t bytes = igrad::widePackedBytes(C, I)) pg.packed = ws.take<uint8_t>(bytes);
        igrad::launch(pg, sms, st);
        afterLaunch("inputGradUmma");
    } else {
        KernelTimer timer__("gemmNT", st);
        gemmNT<<<dim3(static_cast<unsigned>((rows + kTile - 1) / kTile), (I + kTile - 1) / kTile), 256, 0, st>>>(
            dp, W, static_cast<int>(rows), I, C, mk.x, call.dx);
        afterLaunch("gemmNT");
    }
    // dW, dR, dbw, dbr
    if (tensorGrads) {
        const Exec &e = *call.exec;
        const int K = static_cast<int>(rows);
        // the two problems share one launch of one CTA per SM: each is planned for half of the SMs, so that the
        // launch is a single wave (RXMET_WGRAD_FULL_SPLIT plans each for all SMs, two waves)
        const int planSms = std::getenv("RXMET_WGRAD_FULL_SPLIT") ? sms : std::max(1, sms / 2);
        const wgrad::Plan planX = wgrad::plan(K, I, C, planSms), planH = wgrad::plan(K, H, C, planSms);
        WeightGradProblem px{}, ph{};
        px.aCodes = call.x_q; px.aZero = e.gate.zp[RXMET_GRU_X]; px.M = I; px.B = dp;
        px.partial = ws.take<float>(static_cast<size_t>(planX.splits) * (I + 1) * C);
        ph.aFloat = call.h; ph.aInvScale = 1.0f / e.gate.eff[RXMET_GRU_H]; ph.M = H; ph.B = dq;
        ph.partial = ws.take<float>(static_cast<size_t>(planH.splits) * (H + 1) * C);
        px.status = ph.status = status;
        wgrad::launchPair(px, planX, ph, planH, K, C, st);
        afterLaunch("weightGrad");
        {
            const ReduceJob jobX{px.partial, planX.splits, I, e.gate.eff[RXMET_GRU_X], mk.W, mk.bw, call.dW, call.dbw};
            const ReduceJob jobH{ph.partial, planH.splits, H, e.gate.eff[RXMET_GRU_H], mk.R, mk.br, call.dR, call.dbr};
            const size_t largest = static_cast<size_t>(std::max(I, H) + 1) * C;
            KernelTimer timer__("reduceWeightGrad", st);
            reduceWeightGrad<<<dim3(static_cast<unsigned>((largest + kReduceWidth - 1) / kReduceWidth), 2),
                               dim3(kReduceWidth, kReduceLayers), 0, st>>>(jobX, jobH, C, status);
        }
        afterLaunch("reduceWeightGrad");
        return;
    }
    if (slabGrads) {
        const Exec &e = *call.exec;
        const int K = static_cast<int>(rows);
        int chunkK = 0;
        const int splits = wgrad::slabSplits(K, I, H, C, sms, &chunkK);
        WeightGradProblem px{}, ph{};
        px.aCodes = call.x_q; px.aZero = e.gate.zp[RXMET_GRU_X]; px.M = I; px.B = dp;
        px.partial = ws.take<float>(static_cast<size_t>(splits) * (I + 1) * C);
        ph.aFloat = call.h; ph.aInvScale = 1.0f / e.gate.eff[RXMET_GRU_H]; ph.M = H; ph.B = dq;
        ph.partial = ws.take<float>(static_cast<size_t>(splits) * (H + 1) * C);
        px.status = ph.status = status;
        wgrad::launchSlabs(px, ph, K, C, chunkK, splits, wideCodes, st);
        afterLaunch("weightGrad");
        {
            const ReduceJob jobX{px.partial, splits, I, e.gate.eff[RXMET_GRU_X], mk.W, mk.bw, call.dW, call.dbw};
            const ReduceJob jobH{ph.partial, splits, H, e.gate.eff[RXMET_GRU_H], mk.R, mk.br, call.dR, call.dbr};
            const size_t largest = static_cast<size_t>(std::max(I, H) + 1) * C;
            KernelTimer timer__("reduceWeightGrad", st);
            reduceWeightGrad<<<dim3(static_cast<unsigned>((largest + kReduceWidth - 1) / kReduceWidth), 2),
                               dim3(kReduceWidth, kReduceLayers), 0, st>>>(jobX, jobH, C, status);
        }
        afterLaunch("reduceWeightGrad");
        return;
    }
    auto weightGrad = [&](const float *A, int M, const float *G, const uint8_t *mask, float *out) {
        const int tilesM = (M + kTile - 1) / kTile, tilesN = (C + kTile - 1) / kTile;
        const int splits = splitsFor(static_cast<int>(rows), tilesM * tilesN);
        const int chunk = (static_cast<int>(rows) + splits - 1) / splits;
        float *partial = ws.take<float>(static_cast<size_t>(splits) * M * C);
        {
            KernelTimer timer__("gemmTN", st);
            gemmTN<<<dim3(tilesN, tilesM, splits), 256, 0, st>>>(A, G, static_cast<int>(rows), M, C, chunk, partial);
        }
        afterLaunch("gemmTN");
        {
            KernelTimer timer__("reduceSplits", st);
            reduceSplits<<<gridFor(static_cast<size_t>(M) * C, 256), 256, 0, st>>>(partial, splits, static_cast<size_t>(M) * C, mask, out);
        }
        afterLaunch("reduceSplits");
    };
    weightGrad(x, I, dp, mk.W, call.dW);
    weightGrad(call.h, H, dq, mk.R, call.dR);
    // bias gradients
    {
        float *partial = ws.take<float>(2 * static_cast<size_t>(kBiasSplits) * C);
        const int chunk = (static_cast<int>(rows) + kBiasSplits - 1) / kBiasSplits;
        {
            KernelTimer timer__("columnSums", st);
            columnSums<<<dim3((C + 127) / 128, 2, kBiasSplits), 128, 0, st>>>(dp, dq, static_cast<int>(rows), C, chunk, partial);
        }
        afterLaunch("columnSums");
        {
            KernelTimer timer__("reduceSplits", st);
            reduceSplits<<<gridFor(C, 128), 128, 0, st>>>(partial, kBiasSplits, C, mk.bw, call.dbw);
        }
        afterLaunch("reduceSplits");
        {
            KernelTimer timer__("reduceSplits", st);
            reduceSplits<<<gridFor(C, 128), 128, 0, st>>>(partial + static_cast<size_t>(kBiasSplits) * C, kBiasSplits, C, mk.br, call.dbr);
        }
        afterLaunch("reduceSplits");
    }
}

}  // namespace gru
}  // namespace rxmet
