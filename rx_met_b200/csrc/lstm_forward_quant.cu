// Quantized LSTM forward on 8-bit grids (the reference's FP32 q-carrier semantics, computed on
// integer codes).
//
// Launch plan for one call (the reference runs T x (cuBLAS GEMM + pointwise kernel),
// operators/quant-lstm/src/lstm/forward_quantized_fp_cuda.cu:690-880,1050-1230):
//   quantizeCodes  x3  : x, h0, c0 -> signed-byte codes (+ optional q-carrier masters and clamp masks)
//   prepChannels       : weight_ih / weight_hh -> packed byte codes laid out for register residency,
//                        row sums for the zero-point correction, rescaled bias terms
//   inputLinearQ       : all T*B rows of the input projection with dp4a; leaves the gate-input
//                        contribution of the ih branch already rescaled to each gate's grid
//   recurrentQ         : ONE launch for all T steps.  A CTA owns BT batch rows for the whole
//                        sequence; thread c keeps row c of weight_hh in registers, the hidden codes
//                        live in shared memory, the cell state in registers, activations are table
//                        lookups, and the ih contribution of step t+1 is fetched during step t.
//
// Float semantics that decide codes are kept literally: rescale = rint((v * M) * 2^-shift) in
// float with the product rounded once, cell update = rint(pf * rf + pi * ri) without contraction.
// Integer accumulators are required to stay below 2^24, where the reference's float accumulation is
// exact and therefore order independent.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>

#include "common.h"
#include "lstm_device.cuh"
#include "lstm_kernels.h"

namespace rxmet {
namespace lstm {
namespace {

using dev::quantizeCode;
using dev::rescaleF;
using dev::scaleCell;

// Activation tensors: [rows][cols] floats -> [rows][colsPadded] signed bytes (code - shift, zero
// padded), optional q-carrier copy, optional clamp mask, optional centred float copy (code - zp).
__global__ void quantizeCodes(const float *__restrict__ src, int rows, int cols, int colsPadded, float scale, int32_t zp,
                              int32_t lo, int32_t hi, int32_t shift, int8_t *__restrict__ codes,
                              float *__restrict__ carrier, uint8_t *__restrict__ mask, float *__restrict__ centred) {
    const size_t total = static_cast<size_t>(rows) * colsPadded;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int r = static_cast<int>(i / colsPadded), c = static_cast<int>(i % colsPadded);
        if (c >= cols) {
            if (codes) codes[i] = 0;
            continue;
        }
        const size_t o = static_cast<size_t>(r) * cols + c;
        uint8_t m = 0;
        const int32_t q = src ? quantizeCode(src[o], scale, zp, lo, hi, m) : min(max(zp, lo), hi);
        if (codes) codes[i] = static_cast<int8_t>(q - shift);
        if (carrier) carrier[o] = static_cast<float>(q);
        if (mask) mask[o] = m;
        if (centred) centred[o] = static_cast<float>(q - zp);
    }
}

struct PrepArgs {
    int H, I, kWordsIh, kWordsHh;
    const float *wIh, *wHh, *bIh, *bHh;  // float masters
    const float *channel;                // kChannelFields x 4H
    int32_t wLo, wHi, bLo, bHi;
    int32_t xCorrection, hCorrection;    // (shift - zero point) of the x and h codes
    uint32_t *wIhWords, *wHhWords;       // [kWords][4H]
    int32_t *ihAddend, *hhAddend;        // correction * row sum + rescaled bias
    float *mWIh, *mWHh, *mBIh, *mBHh;    // optional q-carrier masters
    uint8_t *kWIh, *kWHh, *kBIh, *kBHh;  // optional clamp masks
};

// One warp per output channel and side (blockIdx.y: 0 = weight_ih, 1 = weight_hh): lanes quantize
// consecutive words of the channel's weight row (coalesced), the row sum is reduced by shuffles, lane
// 0 adds the rescaled bias term.
__global__ void prepChannels(const PrepArgs a) {
    const int C = 4 * a.H;
    const int lane = threadIdx.x & 31;
    const int c = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (c >= C) return;
    const int side = blockIdx.y;
    auto field = [&](int f) { return a.channel[static_cast<size_t>(f) * C + c]; };
    const int K = side ? a.H : a.I, kWords = side ? a.kWordsHh : a.kWordsIh;
    const float *w = (side ? a.wHh : a.wIh) + static_cast<size_t>(c) * K;
    const float scale = field(side ? kWHhScale : kWIhScale);
    uint32_t *words = side ? a.wHhWords : a.wIhWords;
    float *master = side ? a.mWHh : a.mWIh;
    uint8_t *keep = side ? a.kWHh : a.kWIh;
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
        words[static_cast<size_t>(kw) * C + c] = word;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane != 0) return;
    int32_t addend = (side ? a.hCorrection : a.xCorrection) * sum;
    const float *b = side ? a.bHh : a.bIh;
    if (b) {
        uint8_t m;
        const int32_t q = quantizeCode(b[c], field(side ? kBHhScale : kBIhScale), 0, a.bLo, a.bHi, m);
        const DevRescale r{field(side ? kHhBiasMult : kIhBiasMult), field(side ? kHhBiasPow2 : kIhBiasPow2)};
        addend += static_cast<int32_t>(rescaleF(static_cast<float>(q), r));
        float *bm = side ? a.mBHh : a.mBIh;
        uint8_t *bk = side ? a.kBHh : a.kBIh;
        if (bm) bm[c] = static_cast<float>(q);
        if (bk) bk[c] = m;
    }
    (side ? a.hhAddend : a.ihAddend)[c] = addend;
}

// accumulator -> centred linear code (code - zero point) and its clamp flag.
__device__ __forceinline__ float linearCentred(int32_t total, DevRescale out, float cLo, float cHi, uint8_t &clamped) {
    return dev::linearCentredF(static_cast<float>(total), out, cLo, cHi, clamped);
}

constexpr int kIhRows = 16;

struct InputLinearArgs {
    int rows, H, kWords;
    const int8_t *x;         // [rows][kWords*4]
    const uint32_t *words;   // [kWords][4H]
    const int32_t *addend;   // [4H]
    const float *channel;
    ScalarExec s;
    float *lhs;              // [rows][4H] ih contribution on each gate's input grid
    float *linear;           // optional checkpoint [rows][4H]
    uint8_t *linearClamped;  // optional
};

// Persistent: a CTA keeps its threads' weight rows and channel constants in registers and walks
// blocks of kIhRows rows; the codes of the next block are loaded while the current one computes
// (each staging thread carries one 32-bit word) and read back as 16-byte broadcasts.
// Requires blockDim.x >= kIhRows * KW (the words of one block) and blockDim.x >= 4H.
template <int KW>
__global__ void __launch_bounds__(512) inputLinearQ(const __grid_constant__ InputLinearArgs a) {
    __shared__ __align__(16) int32_t xs[2][kIhRows][KW];
    const int C = 4 * a.H, c = threadIdx.x, tid = threadIdx.x;
    const bool live = c < C;
    uint32_t w[KW];
#pragma unroll
    for (int kk = 0; kk < KW; ++kk) w[kk] = (live && kk < a.kWords) ? a.words[static_cast<size_t>(kk) * C + c] : 0u;
    const int32_t addend = live ? a.addend[c] : 0;
    const DevRescale out = live ? DevRescale{a.channel[static_cast<size_t>(kIhOutMult) * C + c],
                                             a.channel[static_cast<size_t>(kIhOutPow2) * C + c]}
                                : DevRescale{1.0f, 1.0f};
    const int op = RXMET_LSTM_WEIGHT_IH_LINEAR, g = live ? c / a.H : 0;
    const float cLo = static_cast<float>(a.s.lo[op] - a.s.zp[op]), cHi = static_cast<float>(a.s.hi[op] - a.s.zp[op]);
    const DevRescale toGate = a.s.ihToGate[g];
    const float zp = a.s.zpF[op];

    const int blocks = (a.rows + kIhRows - 1) / kIhRows;
    const int sRow = tid / KW, sWord = tid % KW;  // the word of a block this thread stages
    const bool stager = tid < kIhRows * KW;
    const int32_t *xWords = reinterpret_cast<const int32_t *>(a.x);  // [rows][kWords]
    auto fetch = [&](int blk) -> int32_t {
        const int row = blk * kIhRows + sRow;
        return (stager && blk < blocks && row < a.rows && sWord < a.kWords) ? xWords[static_cast<size_t>(row) * a.kWords + sWord] : 0;
    };
    int buf = 0;
    if (stager) xs[0][sRow][sWord] = fetch(blockIdx.x);
    __syncthreads();
    for (int blk = blockIdx.x; blk < blocks; blk += gridDim.x) {
        const int32_t pending = fetch(blk + gridDim.x);
        const int row0 = blk * kIhRows, nRows = min(kIhRows, a.rows - row0);
        if (live) {
            size_t o = static_cast<size_t>(row0) * C + c;
            for (int r = 0; r < nRows; ++r, o += C) {
                int32_t acc = 0;
#pragma unroll
                for (int k4 = 0; k4 < KW / 4; ++k4) {
                    const int4 xv = *reinterpret_cast<const int4 *>(&xs[buf][r][4 * k4]);
                    acc = __dp4a(static_cast<int32_t>(w[4 * k4 + 0]), xv.x, acc);
                    acc = __dp4a(static_cast<int32_t>(w[4 * k4 + 1]), xv.y, acc);
                    acc = __dp4a(static_cast<int32_t>(w[4 * k4 + 2]), xv.z, acc);
                    acc = __dp4a(static_cast<int32_t>(w[4 * k4 + 3]), xv.w, acc);
                }
                uint8_t m;
                const float cen = linearCentred(acc + addend, out, cLo, cHi, m);
                a.lhs[o] = rescaleF(cen, toGate);
                if (a.linear) a.linear[o] = cen + zp;
                if (a.linearClamped) a.linearClamped[o] = m;
            }
        }
        if (stager) xs[buf ^ 1][sRow][sWord] = pending;
        __syncthreads();
        buf ^= 1;
    }
}

struct RecurrentArgs {
    int T, B, H, kWords;
    const uint32_t *words;   // [kWords][4H] weight_hh codes
    const int32_t *addend;   // [4H]
    const float *channel;
    const int32_t *tables;   // kTables x kTableSize
    const float *lhs;        // [T][B][4H]
    const int8_t *h0;        // [B][kWords*4] codes - hShift
    const float *c0;         // [B][H] centred cell codes
    ScalarExec s;
    float *output;           // [T][B][H] dequantized
    float *finalHidden, *finalCell;
    rxmet_lstm_trace ck;     // optional checkpoints (weight_ih_linear is written by inputLinearQ)
};

template <int KW, int BT>
__global__ void __launch_bounds__(KW * 16) recurrentQ(const __grid_constant__ RecurrentArgs a) {
    const int H = a.H, C = 4 * a.H;
    constexpr int kPadded = KW * 4;
    __shared__ __align__(16) int8_t hS[BT][kPadded];
    __shared__ int32_t tabS[kTables * kTableSize];
    extern __shared__ __align__(16) unsigned char smemRaw[];
    float *rhsS = reinterpret_cast<float *>(smemRaw);  // [BT][C]

    const int tid = threadIdx.x, nthreads = blockDim.x;
    const int b0 = blockIdx.x * BT, nb = min(BT, a.B - b0);
    const ScalarExec &s = a.s;
    for (int i = tid; i < kTables * kTableSize; i += nthreads) tabS[i] = a.tables[i];

    // phase A ownership: row c of weight_hh
    const bool hasChannel = tid < C;
    uint32_t rw[KW];
    int32_t addend = 0;
    DevRescale outR{1.0f, 1.0f}, toGate{1.0f, 1.0f};
#pragma unroll
    for (int kk = 0; kk < KW; ++kk) rw[kk] = (hasChannel && kk < a.kWords) ? a.words[static_cast<size_t>(kk) * C + tid] : 0u;
    if (hasChannel) {
        addend = a.addend[tid];
        outR = {a.channel[static_cast<size_t>(kHhOutMult) * C + tid], a.channel[static_cast<size_t>(kHhOutPow2) * C + tid]};
        toGate = s.hhToGate[tid / H];
    }
    const int srcPadded = a.kWords * 4;
    for (int i = tid; i < BT * kPadded; i += nthreads) {
        const int b = i / kPadded, k = i % kPadded;
        hS[b][k] = (b < nb && k < srcPadded) ? a.h0[static_cast<size_t>(b0 + b) * srcPadded + k] : int8_t(0);
    }

    // phase B ownership: element (b, j) with its cell state in a register
    const int elems = nb * H;
    const bool hasElem = tid < elems;
    const int eb = hasElem ? tid / H : 0, ej = hasElem ? tid % H : 0;
    float cellCen = hasElem ? a.c0[static_cast<size_t>(b0 + eb) * H + ej] : 0.0f;
    float hiddenCen = 0.0f;

    const int opHh = RXMET_LSTM_WEIGHT_HH_LINEAR;
    const float hhLo = static_cast<float>(s.lo[opHh] - s.zp[opHh]), hhHi = static_cast<float>(s.hi[opHh] - s.zp[opHh]);
    const float zHh = static_cast<float>(s.zp[opHh]);
    float giLo[4], giHi[4];
    int32_t giBase[4];
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        const int op = RXMET_LSTM_INPUT_GATE_INPUT + g;
        giLo[g] = static_cast<float>(s.lo[op] - s.zp[op]);
        giHi[g] = static_cast<float>(s.hi[op] - s.zp[op]);
        giBase[g] = s.zp[op] - s.lo[op];
    }
    const int opC = RXMET_LSTM_CELL_STATE, opO = RXMET_LSTM_OUTPUT;
    const float cLo = static_cast<float>(s.lo[opC] - s.zp[opC]), cHi = static_cast<float>(s.hi[opC] - s.zp[opC]);
    const float oLo = static_cast<float>(s.lo[opO] - s.zp[opO]), oHi = static_cast<float>(s.hi[opO] - s.zp[opO]);
    const int32_t cBase = s.zp[opC] - s.lo[opC];
    const int32_t hStore = s.zp[opO] - s.hShift;  // centred hidden code -> stored byte
    const float scaleH = s.scale[opO];

    // offsets of this thread's element and channel inside one step; a step adds its base
    const size_t elemC = static_cast<size_t>(b0 + eb) * C + ej, elemH = static_cast<size_t>(b0 + eb) * H + ej;
    const size_t chanC = static_cast<size_t>(b0) * C + tid;
    const size_t stepC = static_cast<size_t>(a.B) * C, stepH = static_cast<size_t>(a.B) * H;
    size_t baseC = 0, baseH = 0;  // t * step

    float lhsCur[4] = {0, 0, 0, 0}, lhsNext[4] = {0, 0, 0, 0};
    auto fetch = [&](size_t stepBase, float (&dst)[4]) {
        if (hasElem) {
            const float *row = a.lhs + stepBase + elemC;
#pragma unroll
            for (int g = 0; g < 4; ++g) dst[g] = row[g * H];
        }
    };
    fetch(0, lhsCur);
    __syncthreads();

    const int4 *hS4 = reinterpret_cast<const int4 *>(&hS[0][0]);
    for (int t = 0; t < a.T; ++t, baseC += stepC, baseH += stepH) {
        if (t + 1 < a.T) fetch(baseC + stepC, lhsNext);

        if (hasChannel) {
            int32_t acc[BT];
#pragma unroll
            for (int b = 0; b < BT; ++b) acc[b] = 0;
#pragma unroll
            for (int k4 = 0; k4 < KW / 4; ++k4) {
#pragma unroll
                for (int b = 0; b < BT; ++b) {
                    const int4 hv = hS4[b * (KW / 4) + k4];
                    acc[b] = __dp4a(static_cast<int32_t>(rw[4 * k4 + 0]), hv.x, acc[b]);
                    acc[b] = __dp4a(static_cast<int32_t>(rw[4 * k4 + 1]), hv.y, acc[b]);
                    acc[b] = __dp4a(static_cast<int32_t>(rw[4 * k4 + 2]), hv.z, acc[b]);
                    acc[b] = __dp4a(static_cast<int32_t>(rw[4 * k4 + 3]), hv.w, acc[b]);
                }
            }
#pragma unroll
            for (int b = 0; b < BT; ++b) {
                uint8_t m;
                const float cen = linearCentred(acc[b] + addend, outR, hhLo, hhHi, m);
                rhsS[b * C + tid] = rescaleF(cen, toGate);
                if (b < nb) {
                    const size_t o = baseC + chanC + static_cast<size_t>(b) * C;
                    if (a.ck.weight_hh_linear) a.ck.weight_hh_linear[o] = cen + zHh;
                    if (a.ck.weight_hh_linear_clamped) a.ck.weight_hh_linear_clamped[o] = m;
                }
            }
        }
        __syncthreads();

        if (hasElem) {
            float outCen[4];
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                const float sum = lhsCur[g] + rhsS[eb * C + g * H + ej];
                const float cen = fminf(fmaxf(sum, giLo[g]), giHi[g]);
                const int32_t e = tabS[g * kTableSize + static_cast<int32_t>(cen) + giBase[g]];
                outCen[g] = static_cast<float>(e >> 1);
                const size_t o = baseC + elemC + g * H;
                if (a.ck.gate_inputs) a.ck.gate_inputs[o] = cen + s.zpF[RXMET_LSTM_INPUT_GATE_INPUT + g];
                if (a.ck.gate_inputs_clamped) a.ck.gate_inputs_clamped[o] = (sum < giLo[g]) || (sum > giHi[g]);
                if (a.ck.gate_outputs) a.ck.gate_outputs[o] = outCen[g] + s.zpF[RXMET_LSTM_INPUT_GATE_OUTPUT + g];
                if (a.ck.gate_outputs_clamped) a.ck.gate_outputs_clamped[o] = static_cast<uint8_t>(e & 1);
            }
            const float pf = __fmul_rn(outCen[1], cellCen), pi = __fmul_rn(outCen[0], outCen[2]);
            const float sf = scaleCell(pf, s.forgetRatio, s.forgetMantissa, s.forgetExponent, s.forgetUsesFp);
            const float si = scaleCell(pi, s.inputRatio, s.inputMantissa, s.inputExponent, s.inputUsesFp);
            const float rounded = rintf(__fadd_rn(sf, si));
            cellCen = fminf(fmaxf(rounded, cLo), cHi);
            const int32_t te = tabS[4 * kTableSize + static_cast<int32_t>(cellCen) + cBase];
            const float tanhCen = static_cast<float>(te >> 1);
            const float raw = __fmul_rn(outCen[3], tanhCen);
            const float hr = rescaleF(raw, s.productToOutput);
            hiddenCen = fminf(fmaxf(hr, oLo), oHi);
            hS[eb][ej] = static_cast<int8_t>(static_cast<int32_t>(hiddenCen) + hStore);
            const size_t so = baseH + elemH;
            a.output[so] = __fmul_rn(hiddenCen, scaleH);
            if (a.ck.cell_states) a.ck.cell_states[so] = cellCen + s.zpF[opC];
            if (a.ck.cell_states_clamped) a.ck.cell_states_clamped[so] = (rounded < cLo) || (rounded > cHi);
            if (a.ck.cell_tanh_outputs) a.ck.cell_tanh_outputs[so] = tanhCen + s.zpF[RXMET_LSTM_CELL_TANH_OUTPUT];
            if (a.ck.cell_tanh_outputs_clamped) a.ck.cell_tanh_outputs_clamped[so] = static_cast<uint8_t>(te & 1);
            if (a.ck.hidden_outputs) a.ck.hidden_outputs[so] = hiddenCen + s.zpF[opO];
            if (a.ck.hidden_outputs_clamped) a.ck.hidden_outputs_clamped[so] = (hr < oLo) || (hr > oHi);
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) lhsCur[g] = lhsNext[g];
        __syncthreads();
    }
    if (hasElem) {
        const size_t o = static_cast<size_t>(b0 + eb) * H + ej;
        if (a.T == 0) hiddenCen = static_cast<float>(static_cast<int32_t>(hS[eb][ej]) - hStore);
        a.finalHidden[o] = __fmul_rn(hiddenCen, scaleH);
        a.finalCell[o] = __fmul_rn(cellCen, s.scale[opC]);
    }
}

int gridFor(size_t n, int block) { return static_cast<int>(std::min<size_t>((n + block - 1) / block, 148 * 8)); }

int wordsFor(int k) { return (k + 3) / 4; }
// register-resident word counts the kernels are instantiated for
int roundWords(int kWords) { return kWords <= 8 ? 8 : (kWords <= 16 ? 16 : 32); }

struct Plan {
    int kWordsIh, kWordsHh, kwIh, kwHh;
    size_t rows;
};

Plan planFor(int T, int B, int I, int H) {
    Plan p;
    p.kWordsIh = wordsFor(I);
    p.kWordsHh = wordsFor(H);
    p.kwIh = roundWords(p.kWordsIh);
    p.kwHh = roundWords(p.kWordsHh);
    p.rows = static_cast<size_t>(T) * B;
    return p;
}

template <class W>
void layout(W &ws, int T, int B, int I, int H, int8_t **x, int8_t **h0, float **c0, uint32_t **wIh, uint32_t **wHh,
            int32_t **addIh, int32_t **addHh, float **channel, int32_t **tables, float **lhs) {
    const Plan p = planFor(T, B, I, H);
    const size_t C = 4 * static_cast<size_t>(H);
    auto set = [](auto **dst, auto *v) { if (dst) *dst = v; };
    set(x, ws.template take<int8_t>(p.rows * p.kWordsIh * 4));
    set(h0, ws.template take<int8_t>(static_cast<size_t>(B) * p.kWordsHh * 4));
    set(c0, ws.template take<float>(static_cast<size_t>(B) * H));
    set(wIh, ws.template take<uint32_t>(p.kWordsIh * C));
    set(wHh, ws.template take<uint32_t>(p.kWordsHh * C));
    set(addIh, ws.template take<int32_t>(C));
    set(addHh, ws.template take<int32_t>(C));
    set(channel, ws.template take<float>(kChannelFields * C));
    set(tables, ws.template take<int32_t>(kTables * kTableSize));
    set(lhs, ws.template take<float>(p.rows * C));
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

void quantizeCellCodes(const float *c0, int B, int H, const ScalarExec &s, float *centred, float *carrier, uint8_t *mask,
                       cudaStream_t st) {
    const int op = RXMET_LSTM_CELL_STATE;
    const size_t total = static_cast<size_t>(B) * H;
    {
        KernelTimer timer__("lstmQuantizeCodes", st);
        quantizeCodes<<<gridFor(total, 256), 256, 0, st>>>(c0, B, H, H, s.scale[op], s.zp[op], s.lo[op], s.hi[op], 0, nullptr,
                                                         carrier, mask, centred);
    }
    afterLaunch("lstmQuantizeCodes");
}

size_t forwardQuantWorkspaceBytes(int T, int B, int I, int H) {
    SizerAdapter s;
    layout(s, T, B, I, H, static_cast<int8_t **>(nullptr), static_cast<int8_t **>(nullptr), static_cast<float **>(nullptr),
           static_cast<uint32_t **>(nullptr), static_cast<uint32_t **>(nullptr), static_cast<int32_t **>(nullptr),
           static_cast<int32_t **>(nullptr), static_cast<float **>(nullptr), static_cast<int32_t **>(nullptr),
           static_cast<float **>(nullptr));
    return std::max(s.ws.used() + 1024, forwardQuantWideWorkspaceBytes(T, B, I, H));
}

void forwardQuant(const ForwardQuantCall &call, const Exec &e, void *workspace, size_t workspaceBytes, cudaStream_t st) {
    const int T = call.T, B = call.B, I = call.I, H = call.H, C = 4 * H;
    const ScalarExec &s = e.scalar;
    // The byte-code kernels below take grids of at most 8 bits whose accumulators stay below 2^24 and
    // I, H <= 128 (weight rows live in registers); everything else goes to the wide kernels.
    bool bytePath = e.exactAccumulators && H <= 128 && I <= 128 && !e.tables.empty();
    for (int op = 0; op < kOps; ++op) bytePath = bytePath && (static_cast<int64_t>(s.hi[op]) - s.lo[op] <= 255);
    if (!bytePath) {
        forwardQuantWide(call, e, workspace, workspaceBytes, st);
        return;
    }
    const Plan p = planFor(T, B, I, H);
    Workspace ws(workspace, workspaceBytes);
    int8_t *xq, *h0q;
    float *c0c, *channel, *lhs;
    uint32_t *wIh, *wHh;
    int32_t *addIh, *addHh, *tables;
    layout(ws, T, B, I, H, &xq, &h0q, &c0c, &wIh, &wHh, &addIh, &addHh, &channel, &tables, &lhs);
    RXMET_CUDA(cudaMemcpyAsync(channel, e.channel.data(), e.channel.size() * sizeof(float), cudaMemcpyHostToDevice, st));
    RXMET_CUDA(cudaMemcpyAsync(tables, e.tables.data(), e.tables.size() * sizeof(int32_t), cudaMemcpyHostToDevice, st));

    const rxmet_lstm_masters none{};
    const rxmet_lstm_masters &m = call.masters ? *call.masters : none;
    auto quantize = [&](const float *src, int rows, int cols, int colsPadded, int op, int shift, int8_t *codes,
                        float *carrier, uint8_t *mask, float *centred) {
        const size_t total = static_cast<size_t>(rows) * colsPadded;
        {
            KernelTimer timer__("lstmQuantizeCodes", st);
            quantizeCodes<<<gridFor(total, 256), 256, 0, st>>>(src, rows, cols, colsPadded, s.scale[op], s.zp[op], s.lo[op],
                                                             s.hi[op], shift, codes, carrier, mask, centred);
        }
        afterLaunch("lstmQuantizeCodes");
    };
    quantize(call.x, static_cast<int>(p.rows), I, p.kWordsIh * 4, RXMET_LSTM_INPUT, s.xShift, xq, m.input, m.input_clamped, nullptr);
    quantize(call.h0, B, H, p.kWordsHh * 4, RXMET_LSTM_OUTPUT, s.hShift, h0q, m.initial_hidden, m.initial_hidden_clamped, nullptr);
    quantize(call.c0, B, H, H, RXMET_LSTM_CELL_STATE, 0, nullptr, m.initial_cell, m.initial_cell_clamped, c0c);
    if (!call.h0) {
        if (m.initial_hidden_clamped) RXMET_CUDA(cudaMemsetAsync(m.initial_hidden_clamped, 0, static_cast<size_t>(B) * H, st));
        if (m.initial_cell_clamped) RXMET_CUDA(cudaMemsetAsync(m.initial_cell_clamped, 0, static_cast<size_t>(B) * H, st));
    }

    PrepArgs pa{};
    pa.H = H; pa.I = I; pa.kWordsIh = p.kWordsIh; pa.kWordsHh = p.kWordsHh;
    pa.wIh = call.weightIh; pa.wHh = call.weightHh; pa.bIh = call.biasIh; pa.bHh = call.biasHh;
    pa.channel = channel;
    pa.wLo = s.lo[RXMET_LSTM_WEIGHT_IH]; pa.wHi = s.hi[RXMET_LSTM_WEIGHT_IH];
    pa.bLo = s.lo[RXMET_LSTM_BIAS_IH]; pa.bHi = s.hi[RXMET_LSTM_BIAS_IH];
    pa.xCorrection = s.xShift - s.zp[RXMET_LSTM_INPUT];
    pa.hCorrection = s.hShift - s.zp[RXMET_LSTM_OUTPUT];
    pa.wIhWords = wIh; pa.wHhWords = wHh; pa.ihAddend = addIh; pa.hhAddend = addHh;
    pa.mWIh = m.weight_ih; pa.mWHh = m.weight_hh; pa.mBIh = m.bias_ih; pa.mBHh = m.bias_hh;
    pa.kWIh = m.weight_ih_clamped; pa.kWHh = m.weight_hh_clamped; pa.kBIh = m.bias_ih_clamped; pa.kBHh = m.bias_hh_clamped;
    {
        KernelTimer timer__("lstmPrepChannels", st);
        prepChannels<<<dim3((C + 7) / 8, 2), 256, 0, st>>>(pa);
    }
    afterLaunch("lstmPrepChannels");

    const rxmet_lstm_trace noTrace{};
    const rxmet_lstm_trace &ck = call.checkpoints ? *call.checkpoints : noTrace;
    const int block = (C + 31) / 32 * 32;
    {
        InputLinearArgs a{};
        a.rows = static_cast<int>(p.rows); a.H = H; a.kWords = p.kWordsIh;
        a.x = xq; a.words = wIh; a.addend = addIh; a.channel = channel; a.s = s; a.lhs = lhs;
        a.linear = ck.weight_ih_linear; a.linearClamped = ck.weight_ih_linear_clamped;
        const int blocks = static_cast<int>((p.rows + kIhRows - 1) / kIhRows);
        // the staging of a block needs kIhRows * KW threads
        const int blockIh = std::max(block, kIhRows * p.kwIh);
        auto launchIh = [&](auto kernel) {
            const int perSm = residentPerSm(reinterpret_cast<const void *>(kernel), blockIh, 0);
            const int grid = std::max(1, std::min(blocks, currentDevice().sms * std::max(1, perSm)));
            kernel<<<grid, blockIh, 0, st>>>(a);
        };
        {
            KernelTimer timer__("lstmInputLinearQ", st);
            if (p.kwIh == 8) launchIh(inputLinearQ<8>);
            else if (p.kwIh == 16) launchIh(inputLinearQ<16>);
            else launchIh(inputLinearQ<32>);
        }
        afterLaunch("lstmInputLinearQ");
    }
    {
        RecurrentArgs a{};
        a.T = T; a.B = B; a.H = H; a.kWords = p.kWordsHh;
        a.words = wHh; a.addend = addHh; a.channel = channel; a.tables = tables; a.lhs = lhs; a.h0 = h0q; a.c0 = c0c;
        a.s = s; a.output = call.output; a.finalHidden = call.finalHidden; a.finalCell = call.finalCell; a.ck = ck;
        const int sms = currentDevice().sms;
        // BT*H elements must not exceed the 4H threads of a CTA
        const int bt = (B >= 4 * sms) ? 4 : ((B > sms) ? 2 : 1);
        auto launch = [&](auto kernel, int BT) {
            const size_t smem = sizeof(float) * static_cast<size_t>(BT) * C;
            {
                KernelTimer timer__("lstmRecurrentQ", st);
                kernel<<<(B + BT - 1) / BT, block, smem, st>>>(a);
            }
            afterLaunch("lstmRecurrentQ");
        };
#define RXMET_LSTM_DISPATCH(KW)                          \
    do {                                                  \
        if (bt == 4) launch(recurrentQ<KW, 4>, 4);        \
        else if (bt == 2) launch(recurrentQ<KW, 2>, 2);   \
        else launch(recurrentQ<KW, 1>, 1);                \
    } while (0)
        if (p.kwHh == 8) RXMET_LSTM_DISPATCH(8);
        else if (p.kwHh == 16) RXMET_LSTM_DISPATCH(16);
        else RXMET_LSTM_DISPATCH(32);
#undef RXMET_LSTM_DISPATCH
    }
}

}  // namespace lstm
}  // namespace rxmet
