// Quantized LSTM forward for activation grids of up to 16 bits, weight grids of up to 8 bits
// (W4 / W8), hidden sizes up to 512 and input sizes up to 256: the configurations the byte-code
// kernels of lstm_forward_quant.cu do not take.
//
// Semantics: the reference's FP32 q-carrier (operators/quant-lstm/src/lstm/forward_quantized_fp_cuda.cu:
// 690-880, CPU statement src/lstm/forward_quantized_fp_cpu.cc:71-200).  Every float rounding of the
// pointwise part is kept literally.  The two linear stages are accumulated EXACTLY in integers and
// converted to float once; that equals the reference's float accumulation whenever every partial sum
// stays below 2^24 (its "exact_integer_range" class) and is the correctly rounded value of the sum
// otherwise, where the reference's own CPU (sequential float sums) and CUDA (cuBLAS) builds differ
// from each other in the last place.
//
// Codes wider than a byte are stored as byte planes of u = code - grid minimum (0 .. 65535): a high
// and a low plane, each packed four along K, so that the products stay on dp4a (signed weight bytes
// times unsigned code bytes); sum = 256 * sum_hi + sum_lo + (grid minimum - zero point) * row sum.
//
// Launch plan for one call:
//   quantizePlanes x2    : x, h0 -> byte planes (+ optional q-carrier masters and clamp masks)
//   quantizeCodes        : c0 -> centred cell codes (lstm_forward_quant.cu)
//   prepChannelsWide     : weights -> packed byte codes, 64-bit addends (zero-point correction + bias)
//   inputLinearWide      : all T*B rows of the input projection, persistent CTAs, cp.async staging
//   recurrentWide        : ONE launch for all T steps.  Thread (j, s) owns hidden unit j - all four
//                          gates - for RB batch rows of row group s, so the gate math needs no
//                          exchange between threads; weight_hh streams from L2 (it no longer fits one
//                          SM at H = 512), the hidden codes of a CTA's rows live in shared memory
//                          (double buffered, one barrier per step), the cell state in registers.
//   Activations are table lookups (code -> code + clamp flag) built on the host with the libm calls the
//   reference's CPU path makes; for these grids the five tables (up to 65,536 entries each) sit in
//   device memory and are served by L2.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstdlib>

#include "common.h"
#include "lstm_device.cuh"
#include "plane_proj_umma.cuh"
#include "lstm_kernels.h"

namespace rxmet {
namespace lstm {
namespace {

using dev::dotSignedUnsigned;
using dev::linearCentredF;
using dev::quantizeCode;
using dev::rescaleF;
using dev::scaleCell;

// [rows][cols] floats -> [rows][PLANES][kWords] words of four unsigned bytes of (code - lo); columns
// beyond `cols` are zero.  With PLANES = 2 plane 0 holds the high bytes.  src == null stands for real
// zeros (the zero-point code).
template <int PLANES>
__global__ void quantizePlanes(const float *__restrict__ src, int rows, int cols, int kWords, float scale, int32_t zp,
                               int32_t lo, int32_t hi, uint32_t *__restrict__ planes, float *__restrict__ carrier,
                               uint8_t *__restrict__ mask) {
    const size_t total = static_cast<size_t>(rows) * kWords;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t r = i / kWords;
        const int kw = static_cast<int>(i % kWords);
        uint32_t high = 0, low = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int k = kw * 4 + e;
            if (k >= cols) continue;
            const size_t o = r * cols + k;
            uint8_t m = 0;
            const int32_t q = src ? quantizeCode(src[o], scale, zp, lo, hi, m) : min(max(zp, lo), hi);
            const uint32_t u = static_cast<uint32_t>(q - lo);
            low |= (u & 0xffu) << (8 * e);
            high |= ((u >> 8) & 0xffu) << (8 * e);
            if (carrier) carrier[o] = static_cast<float>(q);
            if (mask) mask[o] = m;
        }
        uint32_t *row = planes + r * PLANES * kWords;
        if (PLANES == 2) {
            row[kw] = high;
            row[kWords + kw] = low;
        } else {
            row[kw] = low;
        }
    }
}

struct WidePrepArgs {
    int H, I, kWordsIh, kWordsHh;
    const float *wIh, *wHh, *bIh, *bHh;  // float masters
    const float *channel;                // kChannelFields x 4H
    int32_t wLo, wHi, bLo, bHi;
    int64_t xCorrection, hCorrection;    // (grid minimum - zero point) of the x and h codes
    uint32_t *wIhWords;                  // [kWordsIh][4H]
    uint32_t *wHhWords;                  // [2 gate pairs][kWordsHh][H][2]
    int64_t *ihAddend, *hhAddend;        // correction * row sum + rescaled bias
    float *mWIh, *mWHh, *mBIh, *mBHh;    // optional q-carrier masters
    uint8_t *kWIh, *kWHh, *kBIh, *kBHh;  // optional clamp masks
};

// One warp per output channel and side (blockIdx.y: 0 = weight_ih, 1 = weight_hh).
__global__ void prepChannelsWide(const WidePrepArgs a) {
    const int C = 4 * a.H;
    const int lane = threadIdx.x & 31;
    const int c = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (c >= C) return;
    const int side = blockIdx.y;
    auto field = [&](int f) { return a.channel[static_cast<size_t>(f) * C + c]; };
    const int K = side ? a.H : a.I, kWords = side ? a.kWordsHh : a.kWordsIh;
    const float *w = (side ? a.wHh : a.wIh) + static_cast<size_t>(c) * K;
    const float scale = field(side ? kWHhScale : kWIhScale);
    float *master = side ? a.mWHh : a.mWIh;
    uint8_t *keep = side ? a.kWHh : a.kWIh;
    const int g = c / a.H, j = c % a.H;
    int32_t sum = 0;
    for (int kw = lane; kw < kWords; kw += 32) {
        uint32_t word = 0;
        for (int i = 0; i < 4; ++i) {
            const int k = kw * 4 + i;
            int32_t q = 0;
            if (k < K) {
                uint8_t m;
                q = quantizeCode(w[k], scale, 0, a.wLo, a.wHi, m);
                if (master) master[static_cast<size_t>(c) * K + k] = static_cast<float>(q);
                if (keep) keep[static_cast<size_t>(c) * K + k] = m;
            }
            sum += q;
            word |= (static_cast<uint32_t>(q) & 0xffu) << (8 * i);
        }
        if (side) a.wHhWords[((static_cast<size_t>(g >> 1) * kWords + kw) * a.H + j) * 2 + (g & 1)] = word;
        else a.wIhWords[static_cast<size_t>(kw) * C + c] = word;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane != 0) return;
    int64_t addend = (side ? a.hCorrection : a.xCorrection) * static_cast<int64_t>(sum);
    const float *b = side ? a.bHh : a.bIh;
    if (b) {
        uint8_t m;
        const int32_t q = quantizeCode(b[c], field(side ? kBHhScale : kBIhScale), 0, a.bLo, a.bHi, m);
        const DevRescale r{field(side ? kHhBiasMult : kIhBiasMult), field(side ? kHhBiasPow2 : kIhBiasPow2)};
        addend += static_cast<int64_t>(rescaleF(static_cast<float>(q), r));
        float *bm = side ? a.mBHh : a.mBIh;
        uint8_t *bk = side ? a.kBHh : a.kBIh;
        if (bm) bm[c] = static_cast<float>(q);
        if (bk) bk[c] = m;
    }
    (side ? a.hhAddend : a.ihAddend)[c] = addend;
}

__device__ __forceinline__ void copyAsync16(void *dst, const void *src, bool valid) {
    const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(valid ? 16u : 0u) : "memory");
}
__device__ __forceinline__ void commitCopies() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void waitCopies() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// 256 * high + low + addend as the float the reference's accumulator holds (rounded once).
template <int PLANES>
__device__ __forceinline__ float combine(const int32_t (&acc)[PLANES], int64_t addend) {
    int64_t total = addend;
    if (PLANES == 2) total += (static_cast<int64_t>(acc[0]) << 8) + acc[1];
    else total += acc[0];
    return __ll2float_rn(total);
}

constexpr int kWideRows = 16;
constexpr int kWideThreads = 512;

struct WideInputArgs {
    int rows, H, kWords;
    const uint32_t *x;       // [rows][PLANES][kWords]
    const uint32_t *words;   // [kWords][4H]
    const int64_t *addend;   // [4H]
    const float *channel;
    ScalarExec s;
    float *lhs;              // [rows][4H] ih contribution on each gate's input grid
    float *linear;           // optional checkpoint [rows][4H]
    uint8_t *linearClamped;  // optional
};

// Persistent over blocks of kWideRows rows (blockIdx.x strides the blocks); blockIdx.y picks a slab
// of blockDim.x output channels.  A thread keeps its channel's weight words (up to KW) in registers;
// the code rows of the next block arrive by cp.async while the current block computes and are read
// back as 16-byte broadcasts.
template <int KW, int PLANES>
__global__ void __launch_bounds__(kWideThreads) inputLinearWide(const __grid_constant__ WideInputArgs a) {
    extern __shared__ __align__(16) uint32_t wideSmem[];  // [2][kWideRows][PLANES * kWords]
    const int C = 4 * a.H, tid = threadIdx.x, c = blockIdx.y * blockDim.x + tid;
    const bool live = c < C;
    const int kWords = a.kWords, rowWords = PLANES * kWords, blockWords = kWideRows * rowWords;
    uint32_t w[KW];
#pragma unroll
    for (int kk = 0; kk < KW; ++kk) w[kk] = (live && kk < kWords) ? a.words[static_cast<size_t>(kk) * C + c] : 0u;
    const int64_t addend = live ? a.addend[c] : 0;
    const DevRescale out = live ? DevRescale{a.channel[static_cast<size_t>(kIhOutMult) * C + c],
                                             a.channel[static_cast<size_t>(kIhOutPow2) * C + c]}
                                : DevRescale{1.0f, 1.0f};
    const int op = RXMET_LSTM_WEIGHT_IH_LINEAR, g = live ? c / a.H : 0;
    const float cLo = static_cast<float>(a.s.lo[op] - a.s.zp[op]), cHi = static_cast<float>(a.s.hi[op] - a.s.zp[op]);
    const DevRescale toGate = a.s.ihToGate[g];
    const float zp = a.s.zpF[op];

    const int blocks = (a.rows + kWideRows - 1) / kWideRows;
    const size_t limit = static_cast<size_t>(a.rows) * rowWords;
    auto stage = [&](int blk, int buf) {
        const size_t base = static_cast<size_t>(blk) * blockWords;
        uint32_t *dst = wideSmem + buf * blockWords;
        for (int i = tid * 4; i < blockWords; i += blockDim.x * 4) {
            const bool valid = blk < blocks && base + i < limit;
            copyAsync16(dst + i, a.x + (valid ? base + i : 0), valid);
        }
        commitCopies();
    };
    stage(blockIdx.x, 0);
    int buf = 0;
    for (int blk = blockIdx.x; blk < blocks; blk += gridDim.x, buf ^= 1) {
        stage(blk + gridDim.x, buf ^ 1);
        waitCopies<1>();
        __syncthreads();
        const int row0 = blk * kWideRows, nRows = min(kWideRows, a.rows - row0);
        if (live) {
            size_t o = static_cast<size_t>(row0) * C + c;
            const uint32_t *xr = wideSmem + buf * blockWords;
            for (int r = 0; r < nRows; ++r, o += C, xr += rowWords) {
                int32_t acc[PLANES];
#pragma unroll
                for (int p = 0; p < PLANES; ++p) acc[p] = 0;
#pragma unroll
                for (int k4 = 0; k4 < KW / 4; ++k4) {
                    if (4 * k4 < kWords) {
#pragma unroll
                        for (int p = 0; p < PLANES; ++p) {
                            const uint4 xv = *reinterpret_cast<const uint4 *>(xr + p * kWords + 4 * k4);
                            acc[p] = dotSignedUnsigned(w[4 * k4 + 0], xv.x, acc[p]);
                            acc[p] = dotSignedUnsigned(w[4 * k4 + 1], xv.y, acc[p]);
                            acc[p] = dotSignedUnsigned(w[4 * k4 + 2], xv.z, acc[p]);
                            acc[p] = dotSignedUnsigned(w[4 * k4 + 3], xv.w, acc[p]);
                        }
                    }
                }
                uint8_t m;
                const float cen = linearCentredF(combine<PLANES>(acc, addend), out, cLo, cHi, m);
                a.lhs[o] = rescaleF(cen, toGate);
                if (a.linear) a.linear[o] = cen + zp;
                if (a.linearClamped) a.linearClamped[o] = m;
            }
        }
        __syncthreads();
    }
    waitCopies<0>();
}

struct WideRecurrentArgs {
    int T, B, H, HP, kWords;
    int weightBytesInSmem;   // size of the shared-memory copy of `words` (the kernel's WS variant), else 0
    const uint2 *words;      // [2 gate pairs][kWords][H]: (x, y) = gates (2 * pair, 2 * pair + 1)
    const int64_t *addend;   // [4H]
    const float *channel;
    const int32_t *tables;   // device: five tables back to back
    int tableOffset[kTables];
    const float *lhs;        // [T][B][4H]
    const uint32_t *h0;      // [B][PLANES][kWords]
    const float *c0;         // [B][H] centred cell codes
    ScalarExec s;
    float *output;           // [T][B][H] dequantized
    float *finalHidden, *finalCell;
    rxmet_lstm_trace ck;     // optional checkpoints (weight_ih_linear is written by inputLinearWide)
    const int *poison;       // status word of the tensor-core projection: non-zero turns the outputs into NaN
};

// WS: weight_hh (4H x H bytes) fits shared memory beside the code rows and is copied there once, which
// takes the L2 round trip out of every step of the serial chain (H up to about 200).
template <int PLANES, int RB, bool WS>
__global__ void __launch_bounds__(kWideThreads, 1) recurrentWide(const __grid_constant__ WideRecurrentArgs a) {
    extern __shared__ __align__(16) uint32_t wideSmemRaw[];  // [weights when WS] [2][BT][PLANES][kWords]
    uint32_t *wideSmem = wideSmemRaw + (WS ? a.weightBytesInSmem / 4 : 0);
    if (WS) {
        const uint4 *src = reinterpret_cast<const uint4 *>(a.words);
        uint4 *dst = reinterpret_cast<uint4 *>(wideSmemRaw);
        for (int i = threadIdx.x; i < a.weightBytesInSmem / 16; i += blockDim.x) dst[i] = src[i];
    }
    const int H = a.H, C = 4 * a.H, kWords = a.kWords;
    const int tid = threadIdx.x, j = tid % a.HP, sg = tid / a.HP;
    const int BT = (blockDim.x / a.HP) * RB;
    const bool active = j < H;
    const int rowWords = PLANES * kWords, bufWords = BT * rowWords;
    const int ctaRow0 = blockIdx.x * BT, b0 = ctaRow0 + sg * RB;
    const ScalarExec &s = a.s;

    for (int i = tid; i < 2 * bufWords; i += blockDim.x) wideSmem[i] = 0u;
    __syncthreads();
    for (int i = tid; i < bufWords; i += blockDim.x) {
        const int b = ctaRow0 + i / rowWords;
        if (b < a.B) wideSmem[i] = a.h0[static_cast<size_t>(b) * rowWords + i % rowWords];
    }

    int64_t addend[4];
    DevRescale outR[4];
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        const int c = g * H + j;
        addend[g] = active ? a.addend[c] : 0;
        outR[g] = active ? DevRescale{a.channel[static_cast<size_t>(kHhOutMult) * C + c],
                                      a.channel[static_cast<size_t>(kHhOutPow2) * C + c]}
                         : DevRescale{1.0f, 1.0f};
    }
    float cellCen[RB], hiddenCen[RB];
#pragma unroll
    for (int r = 0; r < RB; ++r) {
        cellCen[r] = (active && b0 + r < a.B) ? a.c0[static_cast<size_t>(b0 + r) * H + j] : 0.0f;
        hiddenCen[r] = 0.0f;
    }

    const int opHh = RXMET_LSTM_WEIGHT_HH_LINEAR, opC = RXMET_LSTM_CELL_STATE, opO = RXMET_LSTM_OUTPUT;
    const float hhLo = static_cast<float>(s.lo[opHh] - s.zp[opHh]), hhHi = static_cast<float>(s.hi[opHh] - s.zp[opHh]);
    const float cLo = static_cast<float>(s.lo[opC] - s.zp[opC]), cHi = static_cast<float>(s.hi[opC] - s.zp[opC]);
    const float oLo = static_cast<float>(s.lo[opO] - s.zp[opO]), oHi = static_cast<float>(s.hi[opO] - s.zp[opO]);
    const int32_t cBase = s.zp[opC] - s.lo[opC], hBase = s.zp[opO] - s.lo[opO];
    const float scaleH = (a.poison && *a.poison) ? __int_as_float(0x7fc00000) : s.scale[opO];
    const size_t stepC = static_cast<size_t>(a.B) * C, stepH = static_cast<size_t>(a.B) * H;
    __syncthreads();

    for (int t = 0; t < a.T; ++t) {
        const uint32_t *cur = wideSmem + (t & 1) * bufWords;
        uint8_t *nxt = reinterpret_cast<uint8_t *>(wideSmem + ((t + 1) & 1) * bufWords);
        const size_t baseC = t * stepC, baseH = t * stepH;
        if (active) {
            float rhs[4][RB];
            // the input projection's terms of this step: loaded first, so that they arrive during the dot products
            float lhsV[4][RB];
#pragma unroll
            for (int r = 0; r < RB; ++r)
#pragma unroll
                for (int g = 0; g < 4; ++g)
                    lhsV[g][r] = b0 + r < a.B ? __ldg(a.lhs + baseC + static_cast<size_t>(b0 + r) * C + g * H + j) : 0.0f;
            // ---- hh linear stage, two gates at a time ----
#pragma unroll
            for (int pair = 0; pair < 2; ++pair) {
                int32_t acc[2][RB][PLANES];
#pragma unroll
                for (int gg = 0; gg < 2; ++gg)
#pragma unroll
                    for (int r = 0; r < RB; ++r)
#pragma unroll
                        for (int p = 0; p < PLANES; ++p) acc[gg][r][p] = 0;
                const uint2 *wp = (WS ? reinterpret_cast<const uint2 *>(wideSmemRaw) : a.words) + static_cast<size_t>(pair) * kWords * H + j;
                const uint4 *hRows = reinterpret_cast<const uint4 *>(cur + sg * RB * rowWords);
#pragma unroll 2
                for (int k4 = 0; k4 < kWords / 4; ++k4) {
                    uint2 w[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) w[i] = WS ? wp[static_cast<size_t>(4 * k4 + i) * H] : __ldg(wp + static_cast<size_t>(4 * k4 + i) * H);
#pragma unroll
                    for (int r = 0; r < RB; ++r)
#pragma unroll
                        for (int p = 0; p < PLANES; ++p) {
                            const uint4 hv = hRows[(r * PLANES + p) * (kWords / 4) + k4];
                            acc[0][r][p] = dotSignedUnsigned(w[0].x, hv.x, acc[0][r][p]);
                            acc[1][r][p] = dotSignedUnsigned(w[0].y, hv.x, acc[1][r][p]);
                            acc[0][r][p] = dotSignedUnsigned(w[1].x, hv.y, acc[0][r][p]);
                            acc[1][r][p] = dotSignedUnsigned(w[1].y, hv.y, acc[1][r][p]);
                            acc[0][r][p] = dotSignedUnsigned(w[2].x, hv.z, acc[0][r][p]);
                            acc[1][r][p] = dotSignedUnsigned(w[2].y, hv.z, acc[1][r][p]);
                            acc[0][r][p] = dotSignedUnsigned(w[3].x, hv.w, acc[0][r][p]);
                            acc[1][r][p] = dotSignedUnsigned(w[3].y, hv.w, acc[1][r][p]);
                        }
                }
#pragma unroll
                for (int gg = 0; gg < 2; ++gg) {
                    const int g = 2 * pair + gg;
#pragma unroll
                    for (int r = 0; r < RB; ++r) {
                        uint8_t m;
                        const float cen = linearCentredF(combine<PLANES>(acc[gg][r], addend[g]), outR[g], hhLo, hhHi, m);
                        rhs[g][r] = rescaleF(cen, s.hhToGate[g]);
                        if (b0 + r < a.B) {
                            const size_t o = baseC + static_cast<size_t>(b0 + r) * C + g * H + j;
                            if (a.ck.weight_hh_linear) a.ck.weight_hh_linear[o] = cen + s.zpF[opHh];
                            if (a.ck.weight_hh_linear_clamped) a.ck.weight_hh_linear_clamped[o] = m;
                        }
                    }
                }
            }
            // ---- gates, cell and hidden for this thread's (row, j) elements ----
#pragma unroll
            for (int r = 0; r < RB; ++r) {
                const int b = b0 + r;
                if (b >= a.B) continue;
                const size_t rowC = baseC + static_cast<size_t>(b) * C + j, so = baseH + static_cast<size_t>(b) * H + j;
                float outCen[4];
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const int opIn = RXMET_LSTM_INPUT_GATE_INPUT + g;
                    const float giLo = static_cast<float>(s.lo[opIn] - s.zp[opIn]), giHi = static_cast<float>(s.hi[opIn] - s.zp[opIn]);
                    const float sum = lhsV[g][r] + rhs[g][r];
                    const float cen = fminf(fmaxf(sum, giLo), giHi);
                    const int32_t e = __ldg(a.tables + a.tableOffset[g] + static_cast<int32_t>(cen) + (s.zp[opIn] - s.lo[opIn]));
                    outCen[g] = static_cast<float>(e >> 1);
                    const size_t o = rowC + g * H;
                    if (a.ck.gate_inputs) a.ck.gate_inputs[o] = cen + s.zpF[opIn];
                    if (a.ck.gate_inputs_clamped) a.ck.gate_inputs_clamped[o] = (sum < giLo) || (sum > giHi);
                    if (a.ck.gate_outputs) a.ck.gate_outputs[o] = outCen[g] + s.zpF[RXMET_LSTM_INPUT_GATE_OUTPUT + g];
                    if (a.ck.gate_outputs_clamped) a.ck.gate_outputs_clamped[o] = static_cast<uint8_t>(e & 1);
                }
                const float pf = __fmul_rn(outCen[1], cellCen[r]), pi = __fmul_rn(outCen[0], outCen[2]);
                const float sf = scaleCell(pf, s.forgetRatio, s.forgetMantissa, s.forgetExponent, s.forgetUsesFp);
                const float si = scaleCell(pi, s.inputRatio, s.inputMantissa, s.inputExponent, s.inputUsesFp);
                const float rounded = rintf(__fadd_rn(sf, si));
                cellCen[r] = fminf(fmaxf(rounded, cLo), cHi);
                const int32_t te = __ldg(a.tables + a.tableOffset[4] + static_cast<int32_t>(cellCen[r]) + cBase);
                const float tanhCen = static_cast<float>(te >> 1);
                const float raw = __fmul_rn(outCen[3], tanhCen);
                const float hr = rescaleF(raw, s.productToOutput);
                hiddenCen[r] = fminf(fmaxf(hr, oLo), oHi);
                const uint32_t u = static_cast<uint32_t>(static_cast<int32_t>(hiddenCen[r]) + hBase);
                uint8_t *rowBytes = nxt + static_cast<size_t>(sg * RB + r) * rowWords * 4;
                if (PLANES == 2) {
                    rowBytes[j] = static_cast<uint8_t>(u >> 8);
                    rowBytes[kWords * 4 + j] = static_cast<uint8_t>(u & 0xffu);
                } else {
                    rowBytes[j] = static_cast<uint8_t>(u);
                }
                a.output[so] = __fmul_rn(hiddenCen[r], scaleH);
                if (a.ck.cell_states) a.ck.cell_states[so] = cellCen[r] + s.zpF[opC];
                if (a.ck.cell_states_clamped) a.ck.cell_states_clamped[so] = (rounded < cLo) || (rounded > cHi);
                if (a.ck.cell_tanh_outputs) a.ck.cell_tanh_outputs[so] = tanhCen + s.zpF[RXMET_LSTM_CELL_TANH_OUTPUT];
                if (a.ck.cell_tanh_outputs_clamped) a.ck.cell_tanh_outputs_clamped[so] = static_cast<uint8_t>(te & 1);
                if (a.ck.hidden_outputs) a.ck.hidden_outputs[so] = hiddenCen[r] + s.zpF[opO];
                if (a.ck.hidden_outputs_clamped) a.ck.hidden_outputs_clamped[so] = (hr < oLo) || (hr > oHi);
            }
        }
        __syncthreads();
    }
    if (active) {
#pragma unroll
        for (int r = 0; r < RB; ++r) {
            if (b0 + r >= a.B) continue;
            const size_t o = static_cast<size_t>(b0 + r) * H + j;
            a.finalHidden[o] = __fmul_rn(hiddenCen[r], scaleH);
            a.finalCell[o] = __fmul_rn(cellCen[r], s.scale[opC]);
        }
    }
}

// ---- the recurrence with the per-step product on the tensor cores --------------------------------------------
//
// For hidden sizes whose weight_hh fits no single SM (and for large batches, where dp4a is the bound), the
// 4H x H product of every step runs as tcgen05.mma kind::i8.  The hidden units are cut into tiles of 32: a
// CTA owns one unit tile - its 128 gate channels (lane 32 g + u of tensor memory = gate g of unit u) with their
// 128 x H weight bytes resident in shared memory as the canonical K-major A operand - for the rows of one ROW
// GROUP, and the H / 32 CTAs of a row group together advance those rows one step at a time:
//
//   * the hidden codes of step t - 1 (byte planes, [rows][planes][K]) lie in a global exchange buffer; a CTA
//     stages them 64 rows at a time into shared memory (cp.async straight into the canonical B layout, next
//     sub-block in flight), one thread issues PLANES x K / 32 MMAs into one of two accumulator buffers, and
//     the epilogue of the previous sub-block runs meanwhile;
//   * epilogue, phase A (warp = gate, lane = unit): accumulators -> exact sum -> the reference's float rescale,
//     clamp, gate-grid rescale, + the input projection's term, clamp, activation table -> gate output, kept
//     in shared memory; phase B (after a barrier of the four warps of a row chunk; warp = four rows, lane =
//     unit): cell update, tanh table, hidden code; the new hidden bytes go to the other half of the exchange
//     buffer, 32 neighbouring units per store;
//   * after its last sub-block a CTA publishes the step (fence, one atomic increment of the group's counter)
//     and waits until all CTAs of its group have published it.  The launch is cooperative (all CTAs are
//     resident); the wait is bounded and, when it gives up, sets the status word, stops all further waiting
//     of the CTA and poisons its outputs with NaN.
constexpr int kUnitTile = 32, kSubRows = 64, kGroupSpinLimit = 1 << 22;

struct UmmaRecurrentArgs {
    int T, B, H, kWords;
    int groups, rowsPerGroup;     // row groups and rows of each (a multiple of 16)
    const uint4 *tiles;           // [H / 32][128 x kPad bytes]: weight_hh tiles, canonical K-major
    const int64_t *addend;        // [4H]
    const float *channel;
    const int32_t *tables;
    int tableOffset[kTables];
    const float *lhs;             // [T][B][4H]
    uint32_t *exchange[2];        // 2 x [B][PLANES][kWords] hidden byte planes; [0] holds h0 at launch
    float *cell;                  // [B][H] centred cell codes, c0 at launch, updated in place
    ScalarExec s;
    float *output, *finalHidden, *finalCell;
    rxmet_lstm_trace ck;
    unsigned int *counters;       // [groups], zero at launch
    int *status;                  // set to 1 when a bounded wait gave up
    const int *poison;
};

static __global__ void packHhTiles(const uint2 *__restrict__ words, int kWords, int H, int kPad, uint4 *__restrict__ tiles) {
    const int groups = kPad / 16, C = 4 * H;
    const size_t total = static_cast<size_t>(C) * groups;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int kg = static_cast<int>(i / C), c = static_cast<int>(i % C);
        const int g = c / H, j = c % H;   // consecutive threads -> consecutive units of one gate
        uint32_t v[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int kw = 4 * kg + e;
            uint32_t word = 0u;
            if (kw < kWords) {
                const uint2 pair = words[(static_cast<size_t>(g >> 1) * kWords + kw) * H + j];
                word = (g & 1) ? pair.y : pair.x;
            }
            v[e] = word;
        }
        const int tile = j / kUnitTile, lane = 32 * g + j % kUnitTile;
        const size_t at = static_cast<size_t>(tile) * (128 * static_cast<size_t>(kPad) / 16) + static_cast<size_t>(lane / 8) * (groups * 8) +
                          static_cast<size_t>(kg) * 8 + lane % 8;
        tiles[at] = make_uint4(v[0], v[1], v[2], v[3]);
    }
}

template <int PLANES>
__global__ void __launch_bounds__(512, 1) recurrentWideUmma(const __grid_constant__ UmmaRecurrentArgs a) {
    using namespace umma;
    constexpr uint32_t kBufCols = PLANES * kSubRows;
    constexpr uint32_t kTmemCols = 2 * kBufCols;
    constexpr uint32_t kIdesc = planeproj::instructionDescriptor(kSubRows);
    extern __shared__ __align__(128) uint8_t smemU[];
    __shared__ __align__(8) uint64_t bars[2];
    __shared__ uint32_t tmemSlot;
    __shared__ int failed;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int H = a.H, C = 4 * H, kWords = a.kWords, kPad = planeproj::paddedK(kWords);
    const int tilesPerGroup = H / kUnitTile;
    const int ut = blockIdx.x % tilesPerGroup, group = blockIdx.x / tilesPerGroup;
    const int rowBegin = group * a.rowsPerGroup, rowEnd = min(a.B, rowBegin + a.rowsPerGroup);
    const int subBlocks = (max(rowEnd - rowBegin, 0) + kSubRows - 1) / kSubRows;
    const uint32_t groupStride = static_cast<uint32_t>(kPad / 16) * kCore;
    const uint32_t tileBytes = 128u * kPad, planeBytes = static_cast<uint32_t>(kSubRows) * kPad;
    uint8_t *aTile = smemU;                                   // [16][kPad / 16][8][16]
    uint8_t *bPlanes = smemU + tileBytes;                     // 2 x PLANES x [8][kPad / 16][8][16]
    float *gateS = reinterpret_cast<float *>(bPlanes + 2 * PLANES * planeBytes);   // [4 chunks][4 gates][16 rows][32 units]
    const ScalarExec &s = a.s;
    volatile int *failFlag = &failed;

    if (tid == 0) {
        failed = 0;
        for (int i = 0; i < 2; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smemAddr(&bars[i])), "r"(PLANES) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(&tmemSlot)), "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    {
        const uint4 *src = a.tiles + static_cast<size_t>(ut) * (tileBytes / 16);
        for (uint32_t i = tid; i < tileBytes / 16; i += blockDim.x) reinterpret_cast<uint4 *>(aTile)[i] = __ldg(src + i);
        for (uint32_t i = tid; i < 2 * PLANES * planeBytes / 16; i += blockDim.x) reinterpret_cast<uint4 *>(bPlanes)[i] = make_uint4(0u, 0u, 0u, 0u);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmemSlot;

    // phase A role: gate `gate` of unit j for the 16 rows of chunk `chunk`; phase B role: rows 4 gate .. + 3 of the chunk
    const int gate = warp & 3, chunk = warp >> 2;
    const int j = ut * kUnitTile + lane, c = gate * H + j;
    const int64_t addend = a.addend[c];
    const DevRescale outR{a.channel[static_cast<size_t>(kHhOutMult) * C + c], a.channel[static_cast<size_t>(kHhOutPow2) * C + c]};
    const DevRescale toGate = s.hhToGate[gate];
    const int opHh = RXMET_LSTM_WEIGHT_HH_LINEAR, opC = RXMET_LSTM_CELL_STATE, opO = RXMET_LSTM_OUTPUT, opIn = RXMET_LSTM_INPUT_GATE_INPUT + gate;
    const float hhLo = static_cast<float>(s.lo[opHh] - s.zp[opHh]), hhHi = static_cast<float>(s.hi[opHh] - s.zp[opHh]);
    const float giLo = static_cast<float>(s.lo[opIn] - s.zp[opIn]), giHi = static_cast<float>(s.hi[opIn] - s.zp[opIn]);
    const float cLo = static_cast<float>(s.lo[opC] - s.zp[opC]), cHi = static_cast<float>(s.hi[opC] - s.zp[opC]);
    const float oLo = static_cast<float>(s.lo[opO] - s.zp[opO]), oHi = static_cast<float>(s.hi[opO] - s.zp[opO]);
    const int32_t cBase = s.zp[opC] - s.lo[opC], hBase = s.zp[opO] - s.lo[opO], giBase = s.zp[opIn] - s.lo[opIn];
    const float scaleH = (a.poison && *a.poison) ? __int_as_float(0x7fc00000) : s.scale[opO];
    const size_t stepC = static_cast<size_t>(a.B) * C, stepH = static_cast<size_t>(a.B) * H;
    const int rowWords = PLANES * kWords;

    // hidden planes of sub-block `sb` of the exchange half `src` -> plane buffer `buf`
    // Rows beyond the group's last row are not copied: their operand rows keep whatever they held, which only
    // reaches accumulator columns that nobody reads (column n of the product depends on operand row n alone).
    const int perRow = PLANES * (kWords / 4);                       // 16-byte pieces of one row
    const int perRowShift = (perRow & (perRow - 1)) == 0 ? 31 - __clz(perRow) : -1;
    const int perPlaneShift = 31 - __clz(kWords / 4);               // used with perRowShift only (both powers of two then)
    auto stage = [&](const uint32_t *src, int sb, int buf) {
        const int row0 = rowBegin + sb * kSubRows;
        const int pieces = min(kSubRows, rowEnd - row0) * perRow;
        for (int i = tid; i < pieces; i += blockDim.x) {
            int r, pl, kg;
            if (perRowShift >= 0) {
                r = i >> perRowShift;
                const int rest = i & (perRow - 1);
                pl = rest >> perPlaneShift;
                kg = rest & ((kWords / 4) - 1);
            } else {
                r = i / perRow;
                const int rest = i - r * perRow;
                pl = rest / (kWords / 4);
                kg = rest - pl * (kWords / 4);
            }
            const uint32_t *from = src + (static_cast<size_t>(row0 + r) * rowWords + pl * kWords + 4 * kg);
            copyAsync16(bPlanes + (buf * PLANES + pl) * planeBytes + (r >> 3) * groupStride + kg * kCore + (r & 7) * 16, from, true);
        }
        commitCopies();
    };

    // one sub-block per step: this thread meets the same four (row, unit) cells every step and keeps them in registers
    const bool cellInRegisters = subBlocks == 1;
    float cellReg[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int b = rowBegin + 16 * chunk + 4 * gate + i;
        cellReg[i] = (cellInRegisters && b < rowEnd) ? a.cell[static_cast<size_t>(b) * H + j] : 0.0f;
    }
    uint32_t batch = 0;   // MMA batches issued so far: accumulator / plane buffer = batch & 1
    // nextSb >= 0: once the batch's MMAs are known to be complete, the planes of sub-block nextSb are staged into
    // the buffer those MMAs read (they then fly during this epilogue)
    auto epilogue = [&](int t, int sb, uint32_t m, const uint32_t *current, int nextSb) {
        const int buf = m & 1;
        const int row0 = rowBegin + sb * kSubRows + 16 * chunk;
        const size_t baseC = t * stepC, baseH = t * stepH;
        // the input projection's terms do not depend on the product: their loads fly while the MMAs finish
        const bool chunkHasRows = row0 < rowEnd;   // uniform over the four warps of a chunk
        float lhsV[16];
#pragma unroll
        for (int r = 0; r < 16; ++r) lhsV[r] = row0 + r < rowEnd ? __ldg(a.lhs + baseC + static_cast<size_t>(row0 + r) * C + c) : 0.0f;
        if (!*failFlag && !waitPhase(smemAddr(&bars[buf]), (m >> 1) & 1)) *failFlag = 1;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (nextSb >= 0) stage(current, nextSb, buf);
        if (!chunkHasRows) {   // nothing to do for this chunk; the accumulator buffer is not read
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            return;
        }
        // ---- phase A: all loads of the 16 rows before any store, so that their latencies overlap
        uint32_t acc[PLANES][16];
#pragma unroll
        for (int pl = 0; pl < PLANES; ++pl) {
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
                : "=r"(acc[pl][0]), "=r"(acc[pl][1]), "=r"(acc[pl][2]), "=r"(acc[pl][3]), "=r"(acc[pl][4]), "=r"(acc[pl][5]),
                  "=r"(acc[pl][6]), "=r"(acc[pl][7]), "=r"(acc[pl][8]), "=r"(acc[pl][9]), "=r"(acc[pl][10]), "=r"(acc[pl][11]),
                  "=r"(acc[pl][12]), "=r"(acc[pl][13]), "=r"(acc[pl][14]), "=r"(acc[pl][15])
                : "r"(tmem + (static_cast<uint32_t>(32 * gate) << 16) + static_cast<uint32_t>(buf * kBufCols + pl * kSubRows + 16 * chunk)));
        }
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        float hhCen[16], gi[16];
        int32_t entry[16];
        uint32_t flags = 0;   // bit r: hh clamp, bit 16 + r: gate-input clamp
#pragma unroll
        for (int r = 0; r < 16; ++r) {
            int32_t v[PLANES];
#pragma unroll
            for (int pl = 0; pl < PLANES; ++pl) v[pl] = static_cast<int32_t>(acc[pl][r]);
            uint8_t m8;
            hhCen[r] = linearCentredF(combine<PLANES>(v, addend), outR, hhLo, hhHi, m8);
            const float sum = lhsV[r] + rescaleF(hhCen[r], toGate);
            gi[r] = fminf(fmaxf(sum, giLo), giHi);
            flags |= (static_cast<uint32_t>(m8) << r) | (static_cast<uint32_t>((sum < giLo) || (sum > giHi)) << (16 + r));
        }
#pragma unroll
        for (int r = 0; r < 16; ++r) entry[r] = __ldg(a.tables + a.tableOffset[gate] + static_cast<int32_t>(gi[r]) + giBase);
        float *mine = gateS + ((chunk * 4 + gate) * 16) * 32 + lane;
#pragma unroll
        for (int r = 0; r < 16; ++r) {
            const int b = row0 + r;
            const float outCen = static_cast<float>(entry[r] >> 1);
            mine[r * 32] = b < rowEnd ? outCen : 0.0f;
            if (b < rowEnd) {
                const size_t o = baseC + static_cast<size_t>(b) * C + c;
                if (a.ck.weight_hh_linear) a.ck.weight_hh_linear[o] = hhCen[r] + s.zpF[opHh];
                if (a.ck.weight_hh_linear_clamped) a.ck.weight_hh_linear_clamped[o] = static_cast<uint8_t>((flags >> r) & 1u);
                if (a.ck.gate_inputs) a.ck.gate_inputs[o] = gi[r] + s.zpF[opIn];
                if (a.ck.gate_inputs_clamped) a.ck.gate_inputs_clamped[o] = static_cast<uint8_t>((flags >> (16 + r)) & 1u);
                if (a.ck.gate_outputs) a.ck.gate_outputs[o] = outCen + s.zpF[RXMET_LSTM_INPUT_GATE_OUTPUT + gate];
                if (a.ck.gate_outputs_clamped) a.ck.gate_outputs_clamped[o] = static_cast<uint8_t>(entry[r] & 1);
            }
        }
        asm volatile("bar.sync %0, 128;" ::"r"(1 + chunk) : "memory");   // the four warps of this row chunk
        // ---- phase B: the same discipline for this warp's four rows
        uint32_t *next = a.exchange[(t + 1) & 1];
        float cOld[4], cNew[4], rounded[4], gO[4];
        int32_t te[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int b = row0 + 4 * gate + i;
            cOld[i] = cellInRegisters ? cellReg[i] : (b < rowEnd ? a.cell[static_cast<size_t>(b) * H + j] : 0.0f);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float *g4 = gateS + (chunk * 4 * 16 + 4 * gate + i) * 32 + lane;
            const float gI = g4[0], gF = g4[16 * 32], gG = g4[2 * 16 * 32];
            gO[i] = g4[3 * 16 * 32];
            const float pf = __fmul_rn(gF, cOld[i]), pi = __fmul_rn(gI, gG);
            const float sf = scaleCell(pf, s.forgetRatio, s.forgetMantissa, s.forgetExponent, s.forgetUsesFp);
            const float si = scaleCell(pi, s.inputRatio, s.inputMantissa, s.inputExponent, s.inputUsesFp);
            rounded[i] = rintf(__fadd_rn(sf, si));
            cNew[i] = fminf(fmaxf(rounded[i], cLo), cHi);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) te[i] = __ldg(a.tables + a.tableOffset[4] + static_cast<int32_t>(cNew[i]) + cBase);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int b = row0 + 4 * gate + i;
            if (b >= rowEnd) continue;
            const size_t so = baseH + static_cast<size_t>(b) * H + j, cell = static_cast<size_t>(b) * H + j;
            if (cellInRegisters) cellReg[i] = cNew[i];
            else a.cell[cell] = cNew[i];
            const float tanhCen = static_cast<float>(te[i] >> 1);
            const float raw = __fmul_rn(gO[i], tanhCen);
            const float hr = rescaleF(raw, s.productToOutput);
            const float hCen = fminf(fmaxf(hr, oLo), oHi);
            const uint32_t u = static_cast<uint32_t>(static_cast<int32_t>(hCen) + hBase);
            uint8_t *rowBytes = reinterpret_cast<uint8_t *>(next + static_cast<size_t>(b) * rowWords);
            if (PLANES == 2) {
                rowBytes[j] = static_cast<uint8_t>(u >> 8);
                rowBytes[kWords * 4 + j] = static_cast<uint8_t>(u & 0xffu);
            } else {
                rowBytes[j] = static_cast<uint8_t>(u);
            }
            const float hOut = __fmul_rn(hCen, scaleH);
            a.output[so] = hOut;
            if (a.ck.cell_states) a.ck.cell_states[so] = cNew[i] + s.zpF[opC];
            if (a.ck.cell_states_clamped) a.ck.cell_states_clamped[so] = (rounded[i] < cLo) || (rounded[i] > cHi);
            if (a.ck.cell_tanh_outputs) a.ck.cell_tanh_outputs[so] = tanhCen + s.zpF[RXMET_LSTM_CELL_TANH_OUTPUT];
            if (a.ck.cell_tanh_outputs_clamped) a.ck.cell_tanh_outputs_clamped[so] = static_cast<uint8_t>(te[i] & 1);
            if (a.ck.hidden_outputs) a.ck.hidden_outputs[so] = hCen + s.zpF[opO];
            if (a.ck.hidden_outputs_clamped) a.ck.hidden_outputs_clamped[so] = (hr < oLo) || (hr > oHi);
            if (t == a.T - 1) {
                a.finalHidden[cell] = hOut;
                a.finalCell[cell] = __fmul_rn(cNew[i], s.scale[opC]);
            }
        }
        asm volatile("bar.sync %0, 128;" ::"r"(1 + chunk) : "memory");   // gateS of this chunk is free again
    };

    // operand descriptors of the resident weight tile and of the two plane buffers, without the k-step offset
    const uint64_t descA0 = operandDescriptor(smemAddr(aTile), kCore, groupStride);
    uint64_t descB0[2][PLANES];
#pragma unroll
    for (int bufI = 0; bufI < 2; ++bufI)
#pragma unroll
        for (int pl = 0; pl < PLANES; ++pl) descB0[bufI][pl] = operandDescriptor(smemAddr(bPlanes + (bufI * PLANES + pl) * planeBytes), kCore, groupStride);

    for (int t = 0; t < a.T; ++t) {
        const uint32_t *current = a.exchange[t & 1];
        if (subBlocks > 0) stage(current, 0, batch & 1);
        int pendingSb = -1;
        uint32_t pendingBatch = 0;
        for (int sb = 0; sb < subBlocks; ++sb, ++batch) {
            waitCopies<0>();
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncthreads();
            // One thread per byte plane issues that plane's MMAs (its accumulator columns are its own) and commits to
            // the batch's barrier, which counts PLANES arrivals; the issuer's lane siblings wait at the warp barrier
            // instead of polling the barrier beside it.
            if (warp < PLANES) {
                if (lane == 0) {
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const int buf = batch & 1;
                    const uint64_t kStep = static_cast<uint64_t>((2 * kCore) >> 4);   // start-address field advances by two k-groups
                    const uint64_t descB = warp == 0 ? descB0[buf][0] : descB0[buf][PLANES - 1];
                    for (int ks = 0; ks < kPad / 32; ++ks)
                        planeproj::mmaI8(tmem + buf * kBufCols + warp * kSubRows, descA0 + ks * kStep, descB + ks * kStep, kIdesc, ks > 0 ? 1u : 0u);
                    commitTo(smemAddr(&bars[buf]));
                }
                __syncwarp();
            }
            // The plane buffer of the next batch was read by the MMAs of the previous one: once those are known to be
            // complete the next sub-block's copies start, and they fly during the previous sub-block's epilogue.
            if (pendingSb >= 0) epilogue(t, pendingSb, pendingBatch, current, sb + 1 < subBlocks ? sb + 1 : -1);
            else if (sb + 1 < subBlocks) stage(current, sb + 1, (batch + 1) & 1);
            pendingSb = sb;
            pendingBatch = batch;
        }
        if (pendingSb >= 0) epilogue(t, pendingSb, pendingBatch, current, -1);

        // ---- publish step t and wait for the other unit tiles of this row group
        if (t + 1 < a.T) {
            __threadfence();
            __syncthreads();
            if (tid == 0) {
                __threadfence();   // cumulative: what the other threads wrote before the barrier is ordered before the arrival
                atomicAdd(a.counters + group, 1u);
                const unsigned int want = static_cast<unsigned int>(tilesPerGroup) * (t + 1);
                bool arrived = *failFlag != 0;
                for (int spin = 0; !arrived && spin < kGroupSpinLimit; ++spin) {
                    unsigned int seen;
                    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(a.counters + group) : "memory");
                    arrived = seen >= want;
                }
                if (!arrived) *failFlag = 1;
            }
            __syncthreads();
            __threadfence();
        }
    }
    if (*failFlag) {   // loud: the last outputs of this CTA's units become NaN
        for (int i = tid; i < (rowEnd - rowBegin) * kUnitTile; i += blockDim.x) {
            const int b = rowBegin + i / kUnitTile, jj = ut * kUnitTile + i % kUnitTile;
            a.finalHidden[static_cast<size_t>(b) * H + jj] = __int_as_float(0x7fc00000);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    if (tid == 0 && failed && a.status) atomicExch(a.status, 1);
}

int gridFor(size_t n, int block) { return static_cast<int>(std::min<size_t>((n + block - 1) / block, 148 * 8)); }

// words per code row: K padded to a multiple of 16 bytes so that rows are read as 16-byte pieces
int wordsFor(int k) { return (k + 15) / 16 * 4; }

struct WideLayout {
    uint32_t *x, *h0, *wIh, *wHh;
    float *c0, *channel, *lhs;
    int64_t *addIh, *addHh;
    uint4 *ihTiles;    // weight_ih as canonical tensor-core tiles (plane_proj_umma.cuh)
    int *projStatus;
    uint4 *hhTiles;    // weight_hh as unit tiles for the tensor-core recurrence
    uint32_t *exchange;      // second half of the hidden-plane exchange buffer (the first is h0)
    unsigned int *counters;  // step counters of the row groups, then the status word of the recurrence
};

// Epilogue of the tensor-core input projection: the exact sum of the planes and the addend rounded once to
// float, then the reference's float rescale, clamp and gate-grid rescale (the same lines as inputLinearWide).
template <int PLANES>
struct WidePlaneEpilogue {
    const int64_t *addend;
    const float *fields;     // the per-channel float block (kChannelFields x 4H)
    ScalarExec s;
    int H;
    float *lhs, *linear;
    uint8_t *linearClamped;
    struct Channel {
        int64_t addend;
        DevRescale out, toGate;
    };
    __device__ Channel channel(int c) const {
        const size_t C = 4 * static_cast<size_t>(H);
        return Channel{addend[c], DevRescale{fields[static_cast<size_t>(kIhOutMult) * C + c], fields[static_cast<size_t>(kIhOutPow2) * C + c]},
                       s.ihToGate[c / H]};
    }
    __device__ void store(const Channel &ch, size_t row, int c, const int32_t (&acc)[PLANES]) const {
        const int op = RXMET_LSTM_WEIGHT_IH_LINEAR;
        const float cLo = static_cast<float>(s.lo[op] - s.zp[op]), cHi = static_cast<float>(s.hi[op] - s.zp[op]);
        uint8_t m;
        const float cen = linearCentredF(combine<PLANES>(acc, ch.addend), ch.out, cLo, cHi, m);
        const size_t o = row * (4 * static_cast<size_t>(H)) + c;
        lhs[o] = rescaleF(cen, ch.toGate);
        if (linear) linear[o] = cen + s.zpF[op];
        if (linearClamped) linearClamped[o] = m;
    }
};

template <class W>
WideLayout layoutWide(W &ws, int T, int B, int I, int H, int planes) {
    const size_t rows = static_cast<size_t>(T) * B, C = 4 * static_cast<size_t>(H);
    const size_t kIh = wordsFor(I), kHh = wordsFor(H);
    WideLayout l{};
    l.x = ws.template take<uint32_t>(rows * planes * kIh);
    l.h0 = ws.template take<uint32_t>(static_cast<size_t>(B) * planes * kHh);
    l.c0 = ws.template take<float>(static_cast<size_t>(B) * H);
    l.wIh = ws.template take<uint32_t>(kIh * C);
    l.wHh = ws.template take<uint32_t>(kHh * C);
    l.addIh = ws.template take<int64_t>(C);
    l.addHh = ws.template take<int64_t>(C);
    l.channel = ws.template take<float>(kChannelFields * C);
    l.lhs = ws.template take<float>(rows * C);
    l.ihTiles = ws.template take<uint4>(C * planeproj::paddedK(static_cast<int>(kIh)) / 16);
    l.projStatus = ws.template take<int>(1);
    l.hhTiles = ws.template take<uint4>(C * planeproj::paddedK(static_cast<int>(kHh)) / 16);
    l.exchange = ws.template take<uint32_t>(static_cast<size_t>(B) * planes * kHh);
    l.counters = ws.template take<unsigned int>(256);
    return l;
}

struct SizerAdapter {
    WorkspaceSizer ws;
    template <class T>
    T *take(size_t n) {
        ws.take<T>(n);
        return nullptr;
    }
};

}  // namespace

bool forwardQuantWideTakes(const Exec &e, int I, int H, const char **why) {
    const char *reason = nullptr;
    if (!e.weightsFitBytes) reason = "weight grids wider than 8 bits are not built";
    else if (e.activationPlanes == 0) reason = "input / output grids wider than 16 bits are not built";
    else if (e.wide.entries.empty()) reason = "gate-input and cell-state grids wider than 16 bits are not built";
    else if (H > 512) reason = "hidden sizes above 512 are not built";
    else if (I > 256) reason = "input sizes above 256 are not built";
    else {
        for (int op : {RXMET_LSTM_WEIGHT_IH_LINEAR, RXMET_LSTM_WEIGHT_HH_LINEAR})
            if (static_cast<int64_t>(e.scalar.hi[op]) - e.scalar.lo[op] >= (int64_t{1} << 24))
                reason = "linear-output grids wider than 24 bits are not built";
    }
    if (why) *why = reason;
    return reason == nullptr;
}

size_t forwardQuantWideWorkspaceBytes(int T, int B, int I, int H) {
    SizerAdapter s;
    layoutWide(s, T, B, I, H, 2);
    return s.ws.used() + 1024;
}

void forwardQuantWide(const ForwardQuantCall &call, const Exec &e, void *workspace, size_t workspaceBytes, cudaStream_t st) {
    const int T = call.T, B = call.B, I = call.I, H = call.H, C = 4 * H;
    const ScalarExec &s = e.scalar;
    const char *why = nullptr;
    if (!forwardQuantWideTakes(e, I, H, &why)) fail(RXMET_ERR_UNSUPPORTED, "quantized LSTM forward: %s (I=%d, H=%d)", why, I, H);
    const int planes = e.activationPlanes;
    const int kIh = wordsFor(I), kHh = wordsFor(H);
    const size_t rows = static_cast<size_t>(T) * B;
    Workspace ws(workspace, workspaceBytes);
    const WideLayout l = layoutWide(ws, T, B, I, H, planes);
    const int32_t *tables = e.wideTablesOnDevice();
    RXMET_CUDA(cudaMemcpyAsync(l.channel, e.channel.data(), e.channel.size() * sizeof(float), cudaMemcpyHostToDevice, st));

    const rxmet_lstm_masters none{};
    const rxmet_lstm_masters &m = call.masters ? *call.masters : none;
    auto quantize = [&](const float *src, size_t nRows, int cols, int kWords, int op, uint32_t *dst, float *carrier, uint8_t *mask) {
        const size_t total = nRows * kWords;
        {
            KernelTimer timer__("lstmQuantizePlanes", st);
            if (planes == 2)
                quantizePlanes<2><<<gridFor(total, 256), 256, 0, st>>>(src, static_cast<int>(nRows), cols, kWords, s.scale[op], s.zp[op],
                                                                      s.lo[op], s.hi[op], dst, carrier, mask);
            else
                quantizePlanes<1><<<gridFor(total, 256), 256, 0, st>>>(src, static_cast<int>(nRows), cols, kWords, s.scale[op], s.zp[op],
                                                                      s.lo[op], s.hi[op], dst, carrier, mask);
        }
        afterLaunch("lstmQuantizePlanes");
    };
    quantize(call.x, rows, I, kIh, RXMET_LSTM_INPUT, l.x, m.input, m.input_clamped);
    quantize(call.h0, static_cast<size_t>(B), H, kHh, RXMET_LSTM_OUTPUT, l.h0, m.initial_hidden, m.initial_hidden_clamped);
    quantizeCellCodes(call.c0, B, H, s, l.c0, m.initial_cell, m.initial_cell_clamped, st);
    if (!call.h0) {
        if (m.initial_hidden_clamped) RXMET_CUDA(cudaMemsetAsync(m.initial_hidden_clamped, 0, static_cast<size_t>(B) * H, st));
        if (m.initial_cell_clamped) RXMET_CUDA(cudaMemsetAsync(m.initial_cell_clamped, 0, static_cast<size_t>(B) * H, st));
    }

    WidePrepArgs pa{};
    pa.H = H; pa.I = I; pa.kWordsIh = kIh; pa.kWordsHh = kHh;
    pa.wIh = call.weightIh; pa.wHh = call.weightHh; pa.bIh = call.biasIh; pa.bHh = call.biasHh;
    pa.channel = l.channel;
    pa.wLo = s.lo[RXMET_LSTM_WEIGHT_IH]; pa.wHi = s.hi[RXMET_LSTM_WEIGHT_IH];
    pa.bLo = s.lo[RXMET_LSTM_BIAS_IH]; pa.bHi = s.hi[RXMET_LSTM_BIAS_IH];
    pa.xCorrection = static_cast<int64_t>(s.lo[RXMET_LSTM_INPUT]) - s.zp[RXMET_LSTM_INPUT];
    pa.hCorrection = static_cast<int64_t>(s.lo[RXMET_LSTM_OUTPUT]) - s.zp[RXMET_LSTM_OUTPUT];
    pa.wIhWords = l.wIh; pa.wHhWords = l.wHh; pa.ihAddend = l.addIh; pa.hhAddend = l.addHh;
    pa.mWIh = m.weight_ih; pa.mWHh = m.weight_hh; pa.mBIh = m.bias_ih; pa.mBHh = m.bias_hh;
    pa.kWIh = m.weight_ih_clamped; pa.kWHh = m.weight_hh_clamped; pa.kBIh = m.bias_ih_clamped; pa.kBHh = m.bias_hh_clamped;
    {
        KernelTimer timer__("lstmPrepChannelsWide", st);
        prepChannelsWide<<<dim3((C + 7) / 8, 2), 256, 0, st>>>(pa);
    }
    afterLaunch("lstmPrepChannelsWide");

    const rxmet_lstm_trace noTrace{};
    const rxmet_lstm_trace &ck = call.checkpoints ? *call.checkpoints : noTrace;
    const int sms = currentDevice().sms;
    // Input projection: the tcgen05 kind::i8 kernel when 4H tiles by 128 and the operands fit shared memory
    // (RXMET_IPROJ_SIMT turns it off), else the dp4a kernel.
    const int kPadIh = planeproj::paddedK(kIh);
    const int rowsPerTile = planeproj::sharedBytes(kPadIh, planes, 128) <= 200 * 1024 ? 128 : 64;
    const bool tensorProjection = C % planeproj::kChannelTile == 0 && planeproj::sharedBytes(kPadIh, planes, rowsPerTile) <= 200 * 1024 &&
                                  std::getenv("RXMET_IPROJ_SIMT") == nullptr;
    if (tensorProjection) {
        RXMET_CUDA(cudaMemsetAsync(l.projStatus, 0, sizeof(int), st));
        {
            KernelTimer timer__("lstmPrepChannelsWide", st);
            planeproj::packTiles<<<gridFor(static_cast<size_t>(C) * kPadIh / 16, 256), 256, 0, st>>>(l.wIh, kIh, C, kPadIh, l.ihTiles);
        }
        afterLaunch("packTiles");
        planeproj::Problem pp{};
        pp.planes = l.x; pp.rows = static_cast<int>(rows); pp.kWords = kIh; pp.tiles = l.ihTiles; pp.C = C; pp.status = l.projStatus;
        const size_t smem = planeproj::sharedBytes(kPadIh, planes, rowsPerTile);
        const int rowTiles = static_cast<int>((rows + rowsPerTile - 1) / rowsPerTile);
        const int grid = std::max(1, std::min(rowTiles, smsPerPass()));
        auto launchTensor = [&](auto kernel, auto epi) {
            epi.addend = l.addIh; epi.fields = l.channel; epi.s = s; epi.H = H; epi.lhs = l.lhs;
            epi.linear = ck.weight_ih_linear; epi.linearClamped = ck.weight_ih_linear_clamped;
            ensureDynamicSmem(reinterpret_cast<const void *>(kernel), smem);
            KernelTimer timer__("lstmInputLinearWide", st);
            kernel<<<grid, planeproj::kThreads, smem, st>>>(pp, epi);
        };
        if (planes == 2 && rowsPerTile == 128) launchTensor(planeproj::planeProjUmma<WidePlaneEpilogue<2>, 2, 128>, WidePlaneEpilogue<2>{});
        else if (planes == 2) launchTensor(planeproj::planeProjUmma<WidePlaneEpilogue<2>, 2, 64>, WidePlaneEpilogue<2>{});
        else if (rowsPerTile == 128) launchTensor(planeproj::planeProjUmma<WidePlaneEpilogue<1>, 1, 128>, WidePlaneEpilogue<1>{});
        else launchTensor(planeproj::planeProjUmma<WidePlaneEpilogue<1>, 1, 64>, WidePlaneEpilogue<1>{});
        afterLaunch("lstmInputLinearWide");
    } else {
        WideInputArgs a{};
        a.rows = static_cast<int>(rows); a.H = H; a.kWords = kIh;
        a.x = l.x; a.words = l.wIh; a.addend = l.addIh; a.channel = l.channel; a.s = s; a.lhs = l.lhs;
        a.linear = ck.weight_ih_linear; a.linearClamped = ck.weight_ih_linear_clamped;
        const int block = std::min(kWideThreads, (C + 31) / 32 * 32);
        const int slabs = (C + block - 1) / block;
        const int blocks = static_cast<int>((rows + kWideRows - 1) / kWideRows);
        const size_t smem = sizeof(uint32_t) * 2 * kWideRows * planes * kIh;
        auto launch = [&](auto kernel) {
            ensureDynamicSmem(reinterpret_cast<const void *>(kernel), smem);
            const int perSm = residentPerSm(reinterpret_cast<const void *>(kernel), block, smem);
            const int grid = std::max(1, std::min(blocks, std::max(1, sms * perSm / slabs)));
            KernelTimer timer__("lstmInputLinearWide", st);
            kernel<<<dim3(grid, slabs), block, smem, st>>>(a);
        };
#define RXMET_WIDE_IH(KW)                                     \
    do {                                                       \
        if (planes == 2) launch(inputLinearWide<KW, 2>);       \
        else launch(inputLinearWide<KW, 1>);                   \
    } while (0)
        if (kIh <= 16) RXMET_WIDE_IH(16);
        else if (kIh <= 32) RXMET_WIDE_IH(32);
        else RXMET_WIDE_IH(64);
#undef RXMET_WIDE_IH
        afterLaunch("lstmInputLinearWide");
    }
    // Recurrence: per-step product on the tensor cores for hidden sizes whose weights fit no single SM
    // (RXMET_LSTM_REC_SIMT turns it off, RXMET_LSTM_REC_UMMA forces it for every eligible shape).
    {
        const int kPadHh = planeproj::paddedK(kHh);
        const int tilesPerGroup = H / kUnitTile;
        const size_t smemU = 128 * static_cast<size_t>(kPadHh) + 2 * static_cast<size_t>(planes) * kSubRows * kPadHh + sizeof(float) * 4 * 4 * 16 * 32;
        int cooperative = 0;
        RXMET_CUDA(cudaDeviceGetAttribute(&cooperative, cudaDevAttrCooperativeLaunch, currentDevice().device));
        const bool eligible = H % kUnitTile == 0 && tilesPerGroup <= smsPerPass() && smemU <= static_cast<size_t>(currentDevice().smemMax) &&
                              cooperative != 0 && std::getenv("RXMET_LSTM_REC_SIMT") == nullptr;
        if (eligible && (H >= 256 || std::getenv("RXMET_LSTM_REC_UMMA") != nullptr)) {
            int groups = std::max(1, std::min(smsPerPass() / tilesPerGroup, (B + 15) / 16));
            const int rowsPerGroup = ((B + groups - 1) / groups + 15) / 16 * 16;
            groups = (B + rowsPerGroup - 1) / rowsPerGroup;
            {
                KernelTimer timer__("lstmPrepChannelsWide", st);
                packHhTiles<<<gridFor(static_cast<size_t>(C) * kPadHh / 16, 256), 256, 0, st>>>(reinterpret_cast<const uint2 *>(l.wHh), kHh, H, kPadHh,
                                                                                                l.hhTiles);
            }
            afterLaunch("packHhTiles");
            RXMET_CUDA(cudaMemsetAsync(l.counters, 0, sizeof(unsigned int) * 256, st));
            UmmaRecurrentArgs u{};
            u.T = T; u.B = B; u.H = H; u.kWords = kHh; u.groups = groups; u.rowsPerGroup = rowsPerGroup;
            u.tiles = l.hhTiles; u.addend = l.addHh; u.channel = l.channel; u.tables = tables;
            for (int t = 0; t < kTables; ++t) u.tableOffset[t] = e.wide.offset[t];
            u.lhs = l.lhs; u.exchange[0] = l.h0; u.exchange[1] = l.exchange; u.cell = l.c0; u.s = s;
            u.output = call.output; u.finalHidden = call.finalHidden; u.finalCell = call.finalCell; u.ck = ck;
            u.counters = l.counters; u.status = reinterpret_cast<int *>(l.counters + 255);
            u.poison = tensorProjection ? l.projStatus : nullptr;
            auto launchU = [&](auto kernel) {
                ensureDynamicSmem(reinterpret_cast<const void *>(kernel), smemU);
                void *params[] = {&u};
                KernelTimer timer__("lstmRecurrentWide", st);
                RXMET_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(kernel), dim3(groups * tilesPerGroup), dim3(512), params, smemU, st));
            };
            if (planes == 2) launchU(recurrentWideUmma<2>);
            else launchU(recurrentWideUmma<1>);
            afterLaunch("lstmRecurrentWideUmma");
            return;
        }
    }
    {
        WideRecurrentArgs a{};
        a.T = T; a.B = B; a.H = H; a.HP = (H + 31) / 32 * 32; a.kWords = kHh;
        a.words = reinterpret_cast<const uint2 *>(l.wHh); a.addend = l.addHh; a.channel = l.channel; a.tables = tables;
        for (int t = 0; t < kTables; ++t) a.tableOffset[t] = e.wide.offset[t];
        a.lhs = l.lhs; a.h0 = l.h0; a.c0 = l.c0; a.s = s;
        a.output = call.output; a.finalHidden = call.finalHidden; a.finalCell = call.finalCell; a.ck = ck;
        a.poison = tensorProjection ? l.projStatus : nullptr;
        // rows per CTA: enough CTAs to occupy the SMs first, then more rows per thread so that a weight
        // word fetched from L2 serves several rows
        const int groupsMax = std::max(1, kWideThreads / a.HP);
        const int want = std::max(1, (B + smsPerPass() - 1) / smsPerPass());
        int rb = 1;
        while (rb < 8 && rb * groupsMax < want) rb *= 2;
        const int groups = std::max(1, std::min(groupsMax, (want + rb - 1) / rb));
        const int bt = groups * rb;
        const int block = groups * a.HP;
        const size_t planeBytes = sizeof(uint32_t) * 2 * bt * planes * kHh;
        const size_t weightBytes = sizeof(uint32_t) * static_cast<size_t>(kHh) * C;  // a multiple of 16
        const bool weightsInSmem = planeBytes + weightBytes + 1024 <= static_cast<size_t>(currentDevice().smemMax);
        a.weightBytesInSmem = weightsInSmem ? static_cast<int>(weightBytes) : 0;
        const size_t smem = planeBytes + (weightsInSmem ? weightBytes : 0);
        auto launch = [&](auto kernel) {
            ensureDynamicSmem(reinterpret_cast<const void *>(kernel), smem);
            KernelTimer timer__("lstmRecurrentWide", st);
            kernel<<<(B + bt - 1) / bt, block, smem, st>>>(a);
        };
#define RXMET_WIDE_REC(RBV)                                                        \
    do {                                                                            \
        if (planes == 2 && weightsInSmem) launch(recurrentWide<2, RBV, true>);      \
        else if (planes == 2) launch(recurrentWide<2, RBV, false>);                 \
        else if (weightsInSmem) launch(recurrentWide<1, RBV, true>);                \
        else launch(recurrentWide<1, RBV, false>);                                  \
    } while (0)
        if (rb == 1) RXMET_WIDE_REC(1);
        else if (rb == 2) RXMET_WIDE_REC(2);
        else if (rb == 4) RXMET_WIDE_REC(4);
        else RXMET_WIDE_REC(8);
#undef RXMET_WIDE_REC
        afterLaunch("lstmRecurrentWide");
    }
}

}  // namespace lstm
}  // namespace rxmet
