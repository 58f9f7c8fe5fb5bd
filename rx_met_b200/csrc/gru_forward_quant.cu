// Quantized GRU forward on the integer carrier.
//
// Data flow (one direction, one call):
//   1. quantizeTensor       : float master weights / biases / x / h0 -> integer codes in the
//                             narrowest storage class, optional int32 copy and clamp mask.
//   2. channelPrep          : per output channel, zero-point compensation sum_k W[k,c]*zp and
//                             the bias term already moved to the accumulator grid.
//   3. inputLinear          : ih[n,c] for all T*B rows at once (the recurrence does not need it
//                             step by step), stored as 16-bit codes when the grid allows.
//   4. recurrentForward     : ONE launch for all T steps.  Sequences are independent, so each
//                             CTA owns a small batch tile and keeps the whole recurrent weight
//                             matrix resident in shared memory for the entire sequence; no
//                             grid-wide barrier exists.  Each step is a tile GEMM (dp4a for
//                             8-bit grids), the hh-linear epilogue, the integer gates and the
//                             dequantized outputs, fused.
//
// Reference: operators/quant-gru/src/gru_forward_gpu_quant.cu (per-step GEMM + pointwise
// launches) and src/gru_forward_cpu_quant.cc (CPU integer core).
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <mutex>
#include <type_traits>
#include <vector>

#include "common.h"
#include "gru_device.cuh"
#include "gru_forward_quant.h"
#include "gru_forward_wide.h"
#include "input_proj_umma.h"

namespace rxmet {
namespace gru {

// The block is page-locked host memory owned by the Exec, and the Exec lives in a small cache that
// evicts old entries.  A copy recorded into a CUDA graph reads the block again at every replay, long
// after the call returned, so a block handed out while the stream is being captured is kept for the
// life of the process (one block per captured parameter set; a few tens of KB each).
const int32_t *pinnedChannelBlock(const Exec &e, cudaStream_t st) {
    std::call_once(e.pinnedOnce, [&] {
        const size_t C = 3 * static_cast<size_t>(e.hidden);
        int32_t *host = nullptr;
        RXMET_CUDA(cudaHostAlloc(reinterpret_cast<void **>(&host), 12 * C * sizeof(int32_t), cudaHostAllocDefault));
        e.pinnedChannels = std::shared_ptr<int32_t>(host, [](int32_t *ptr) { cudaFreeHost(ptr); });
        auto putF = [&](size_t slot, const std::vector<float> &v) { std::memcpy(host + slot * C, v.data(), C * 4); };
        auto putR = [&](size_t slot, const std::vector<Rescale> &v) { std::memcpy(host + slot * C, v.data(), C * 8); };
        putF(0, e.chan.eff_W); putF(1, e.chan.eff_R); putF(2, e.chan.eff_bw); putF(3, e.chan.eff_br);
        putR(4, e.chan.gemm_x); putR(6, e.chan.bias_x); putR(8, e.chan.gemm_h); putR(10, e.chan.bias_h);
    });
    cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &capture) == cudaSuccess && capture != cudaStreamCaptureStatusNone) {
        static std::mutex mutex;
        static std::vector<std::shared_ptr<int32_t>> captured;
        std::lock_guard<std::mutex> lock(mutex);
        if (std::find(captured.begin(), captured.end(), e.pinnedChannels) == captured.end()) captured.push_back(e.pinnedChannels);
    }
    return e.pinnedChannels.get();
}

namespace {

// ---- exact dot products ---------------------------------------------------

// Generic: one code per element, 64-bit accumulation (never overflows).
template <class WT, class AT>
struct Dot {
    using Acc = int64_t;
    using WWord = WT;
    using AWord = AT;
    static constexpr int kPack = 1;
    static __device__ __forceinline__ void mac(Acc &acc, WWord w, AWord a) {
        acc += static_cast<int64_t>(w) * static_cast<int64_t>(a);
    }
};
// 8-bit x 8-bit: four codes per 32-bit word, dp4a, 32-bit accumulation.  Exact for K < 2^16.
template <>
struct Dot<int8_t, int8_t> {
    using Acc = int32_t;
    using WWord = int32_t;
    using AWord = int32_t;
    static constexpr int kPack = 4;
    static __device__ __forceinline__ void mac(Acc &acc, WWord w, AWord a) { acc = __dp4a(w, a, acc); }
};

__host__ __device__ inline int padTo(int v, int m) { return (v + m - 1) / m * m; }

// ---- 1. quantize ----------------------------------------------------------

// dst layout: row-major [rowsPadded, cols] when pack == 1; [rowsPadded/pack, cols, pack] when the
// tensor is a packed weight (pack consecutive rows of one column share a word).  For activations
// (transposedPack == false) rows are samples and cols is the padded feature count.
template <class CodeT>
__global__ void quantizeTensor(const float *__restrict__ src, int rows, int cols, int rowsPadded, int colsPadded,
                               const float *__restrict__ channelScale, float scalarScale, int32_t zp, int32_t lo,
                               int32_t hi, int weightPack, CodeT *__restrict__ codes, int32_t *__restrict__ codes32,
                               uint8_t *__restrict__ mask) {
    const size_t total = static_cast<size_t>(rowsPadded) * colsPadded;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int r = static_cast<int>(i / colsPadded), c = static_cast<int>(i % colsPadded);
        int32_t q = 0;
        if (r < rows && c < cols) {
            const size_t s = static_cast<size_t>(r) * cols + c;
            uint8_t keep;
            q = quantizeValue(src[s], channelScale ? channelScale[c] : scalarScale, zp, lo, hi, keep);
            if (codes32) codes32[s] = q;
            if (mask) mask[s] = keep;
        }
        const size_t d = weightPack > 1
                             ? (static_cast<size_t>(r / weightPack) * colsPadded + c) * weightPack + (r % weightPack)
                             : i;
        codes[d] = static_cast<CodeT>(q);
    }
}

// Fills a code tensor with a constant (initial state = zero point).
template <class CodeT>
__global__ void fillCodes(CodeT *dst, size_t n, int32_t value) {
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<size_t>(gridDim.x) * blockDim.x)
        dst[i] = static_cast<CodeT>(value);
}

// int32 codes handed in by the caller -> storage class, padded rows.
template <class CodeT>
__global__ void narrowCodes(const int32_t *__restrict__ src, int rows, int cols, int colsPadded,
                            CodeT *__restrict__ dst) {
    const size_t total = static_cast<size_t>(rows) * colsPadded;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int r = static_cast<int>(i / colsPadded), c = static_cast<int>(i % colsPadded);
        dst[i] = c < cols ? static_cast<CodeT>(src[static_cast<size_t>(r) * cols + c]) : CodeT(0);
    }
}

// ---- 2. per-channel preparation --------------------------------------------

// comp[c] = zpIn * sum_k W[k,c]; biasAcc[c] = rescale(bias[c]) on the accumulator grid
// (reference: gru_forward_cpu_quant.cc:76-111,133-134).
template <class WT, class AT>
__global__ void channelPrep(const typename Dot<WT, AT>::WWord *__restrict__ w, int kWords, int channels, int32_t zpIn,
                            const int32_t *__restrict__ biasCodes, const Rescale *__restrict__ biasRescale,
                            int64_t *__restrict__ comp, int64_t *__restrict__ biasAcc) {
    using D = Dot<WT, AT>;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    int64_t sum = 0;
    for (int kk = 0; kk < kWords; ++kk) {
        const typename D::WWord word = w[static_cast<size_t>(kk) * channels + c];
        if constexpr (D::kPack == 4) {
            sum += static_cast<int8_t>(word & 0xff) + static_cast<int8_t>((word >> 8) & 0xff) +
                   static_cast<int8_t>((word >> 16) & 0xff) + static_cast<int8_t>((word >> 24) & 0xff);
        } else {
            sum += static_cast<int64_t>(word);
        }
    }
    comp[c] = sum * zpIn;
    biasAcc[c] = applyRescale(static_cast<int64_t>(biasCodes[c]), biasRescale[c]);
}

// 8-bit weights: everything that depends on the parameters alone, in one launch.  A CTA owns 32
// channels; its thread layers share the rows of W and R (four rows = one packed word),
// quantize them, store the packed words (and the optional 32-bit codes and clamp flags) and
// sum the codes; layer 0 then adds the layers' sums, quantizes the two biases and writes the
// zero-point correction and the bias on the accumulator grid.  Same arithmetic as
// quantizeTensor + channelPrep above.  kPrepLayers thread layers keep the chain of dependent
// loads per thread short: this launch sits on the critical path of every step.
struct WeightPrepArgs {
    const float *W, *R, *bw, *br;
    int I, H, C, iWords, hWords;
    const float *effW, *effR, *effBw, *effBr;
    int32_t loW, hiW, loR, hiR, loBw, hiBw, loBr, hiBr;
    int32_t *wCodes, *rCodes, *bwCodes, *brCodes;  // packed words / bias codes
    int32_t *W_q, *R_q, *bw_q, *br_q;              // optional 32-bit copies of the codes
    uint8_t *mW, *mR, *mBw, *mBr;                  // optional clamp flags
    int32_t zpX, zpH;
    const Rescale *biasRescaleX, *biasRescaleH;
    int64_t *compX, *biasX, *compH, *biasH;
    // Optional second job of the same launch: the input tensor -> codes (blocks beyond the
    // parameter blocks; same arithmetic as quantizeTensor with one scale).  xSrc null = none.
    const float *xSrc;
    int xRows, xCols, xColsPadded;
    float xScale;
    int32_t xLo, xHi;
    int8_t *xCodes;
    int32_t *xCodes32;
    uint8_t *xMask;
    int prepBlocks;
};

constexpr int kPrepLayers = 32;
__global__ void __launch_bounds__(32 * kPrepLayers) prepareWeightsI8(const WeightPrepArgs a) {
    __shared__ int32_t sums[2][kPrepLayers][32];
    if (static_cast<int>(blockIdx.x) >= a.prepBlocks) {  // the input tensor's blocks
        const size_t total = static_cast<size_t>(a.xRows) * a.xColsPadded;
        const size_t stride = static_cast<size_t>(gridDim.x - a.prepBlocks) * blockDim.x;
        for (size_t i = static_cast<size_t>(blockIdx.x - a.prepBlocks) * blockDim.x + threadIdx.x; i < total; i += stride) {
            const int r = static_cast<int>(i / a.xColsPadded), col = static_cast<int>(i % a.xColsPadded);
            int32_t q = 0;
            if (col < a.xCols) {
                const size_t at = static_cast<size_t>(r) * a.xCols + col;
                uint8_t keep;
                q = quantizeValue(a.xSrc[at], a.xScale, a.zpX, a.xLo, a.xHi, keep);
                if (a.xCodes32) a.xCodes32[at] = q;
                if (a.xMask) a.xMask[at] = keep;
            }
            a.xCodes[i] = static_cast<int8_t>(q);
        }
        return;
    }
    const int cl = threadIdx.x & 31, layer = threadIdx.x >> 5, c = blockIdx.x * 32 + cl;
    const bool live = c < a.C;
    auto pass = [&](const float *__restrict__ src, int rowsK, int words, float scale, int32_t lo, int32_t hi,
                    int32_t *__restrict__ codes, int32_t *__restrict__ codes32, uint8_t *__restrict__ mask) {
        int32_t sum = 0;
        for (int kk = layer; kk < words; kk += kPrepLayers) {
            float v[4];
#pragma unroll
            for (int b = 0; b < 4; ++b) v[b] = 4 * kk + b < rowsK ? src[static_cast<size_t>(4 * kk + b) * a.C + c] : 0.0f;
            uint32_t word = 0;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const int k = 4 * kk + b;
                int32_t q = 0;
                if (k < rowsK) {
                    const size_t at = static_cast<size_t>(k) * a.C + c;
                    uint8_t keep;
                    q = quantizeValue(v[b], scale, 0, lo, hi, keep);
                    if (codes32) codes32[at] = q;
                    if (mask) mask[at] = keep;
                }
                sum += q;
                word |= static_cast<uint32_t>(q & 0xff) << (8 * b);
            }
            codes[static_cast<size_t>(kk) * a.C + c] = static_cast<int32_t>(word);
        }
        return sum;
    };
    int32_t sumW = 0, sumR = 0;
    if (live) {
        sumW = pass(a.W, a.I, a.iWords, a.effW[c], a.loW, a.hiW, a.wCodes, a.W_q, a.mW);
        sumR = pass(a.R, a.H, a.hWords, a.effR[c], a.loR, a.hiR, a.rCodes, a.R_q, a.mR);
    }
    sums[0][layer][cl] = sumW;
    sums[1][layer][cl] = sumR;
    __syncthreads();
    if (layer != 0 || !live) return;
    int64_t totalW = 0, totalR = 0;
#pragma unroll
    for (int l = 0; l < kPrepLayers; ++l) {
        totalW += sums[0][l][cl];
        totalR += sums[1][l][cl];
    }
    uint8_t keep;
    const int32_t qBw = quantizeValue(a.bw[c], a.effBw[c], 0, a.loBw, a.hiBw, keep);
    a.bwCodes[c] = qBw;
    if (a.bw_q) a.bw_q[c] = qBw;
    if (a.mBw) a.mBw[c] = keep;
    const int32_t qBr = quantizeValue(a.br[c], a.effBr[c], 0, a.loBr, a.hiBr, keep);
    a.brCodes[c] = qBr;
    if (a.br_q) a.br_q[c] = qBr;
    if (a.mBr) a.mBr[c] = keep;
    a.compX[c] = totalW * a.zpX;
    a.biasX[c] = applyRescale(static_cast<int64_t>(qBw), a.biasRescaleX[c]);
    a.compH[c] = totalR * a.zpH;
    a.biasH[c] = applyRescale(static_cast<int64_t>(qBr), a.biasRescaleH[c]);
}

// Epilogue shared by both linear stages (gru_forward_gpu_quant.cu:163-178).
__device__ __forceinline__ int32_t linearEpilogue(int64_t acc, int64_t comp, int64_t biasAcc, Rescale r, int32_t zpOut,
                                                  int32_t lo, int32_t hi, uint8_t &keep) {
    const int64_t res = applyRescale(acc - comp + biasAcc, r) + zpOut;
    return clampCode(static_cast<int32_t>(res), lo, hi, keep);
}

// ---- 3. input projection for all steps -------------------------------------

constexpr int kLinearRows = 8;

// When `pre.enabled`, the stored value is not the ih code itself but its contribution to the gate
// input, rescale(code - zp) with the rescale of the gate the column belongs to: that term does not
// depend on the recurrent state, so it is computed here once instead of in every step.
template <class WT, class AT, class LT>
__global__ void inputLinear(const typename Dot<WT, AT>::AWord *__restrict__ x, int rows, int kWords, int channels,
                            const typename Dot<WT, AT>::WWord *__restrict__ w, const int64_t *__restrict__ comp,
                            const int64_t *__restrict__ biasAcc, const Rescale *__restrict__ rescale, int32_t zpOut,
                            int32_t lo, int32_t hi, LT *__restrict__ out, uint8_t *__restrict__ mask,
                            const PreRescale pre) {
    using D = Dot<WT, AT>;
    extern __shared__ __align__(16) unsigned char smemRaw[];
    auto *xs = reinterpret_cast<typename D::AWord *>(smemRaw);  // [kLinearRows][kWords]
    const int row0 = blockIdx.x * kLinearRows;
    const int nRows = min(kLinearRows, rows - row0);
    for (int i = threadIdx.x; i < kLinearRows * kWords; i += blockDim.x) {
        const int r = i / kWords;
        xs[i] = r < nRows ? x[static_cast<size_t>(row0 + r) * kWords + (i % kWords)] : typename D::AWord(0);
    }
    __syncthreads();
    for (int c = threadIdx.x; c < channels; c += blockDim.x) {
        typename D::Acc acc[kLinearRows];
#pragma unroll
        for (int r = 0; r < kLinearRows; ++r) acc[r] = 0;
        for (int kk = 0; kk < kWords; ++kk) {
            const typename D::WWord word = w[static_cast<size_t>(kk) * channels + c];
#pragma unroll
            for (int r = 0; r < kLinearRows; ++r) D::mac(acc[r], word, xs[r * kWords + kk]);
        }
        const int64_t cmp = comp[c], bias = biasAcc[c];
        const Rescale rs = rescale[c];
        const Rescale gateRs = pre.enabled ? pre.toGate[c / pre.hidden] : Rescale{1, 0};
        // Channel constants of the two rounding shifts.  With 32-bit accumulators, shifts in
        // [1, 40] and multipliers below 2^24 (every practical parameter set; no 64-bit overflow) the epilogue is one widening multiply, one
        // 64-bit add and one shift per rescale; anything else takes the general functions.
        const int64_t offset = bias - cmp;
        const bool quick = sizeof(typename D::Acc) == 4 && rs.shift >= 1 && rs.shift <= 40 && offset > -(1ll << 30) &&
                           offset < (1ll << 30) && rs.mult > 0 && rs.mult < (1 << 24) && zpOut > -(1 << 20) && zpOut < (1 << 20) &&
                           (!pre.enabled || (gateRs.shift >= 1 && gateRs.shift <= 40 && gateRs.mult > 0 && gateRs.mult < (1 << 24)));
        // (acc + offset) * mult = acc * mult + offset * mult: the constant rides in the widening
        // multiply-add; the output zero point rides in the rounding constant (it is a multiple of
        // 2^shift there, so it does not disturb the remainder)
        const int64_t mulAddOut = quick ? offset * rs.mult : 0;
        const int64_t roundOut = quick ? (1ll << (rs.shift - 1)) - 1 + (static_cast<int64_t>(zpOut) << rs.shift) : 0;
        const int64_t mulAddGate = (quick && pre.enabled) ? -static_cast<int64_t>(zpOut) * gateRs.mult : 0;
        const int64_t roundGate = (quick && pre.enabled) ? (1ll << (gateRs.shift - 1)) - 1 : 0;
#pragma unroll
        for (int r = 0; r < kLinearRows; ++r) {
            if (r < nRows) {
                uint8_t keep;
                int32_t q;
                if (quick) {
                    const int64_t prod = static_cast<int64_t>(static_cast<int32_t>(acc[r])) * rs.mult + mulAddOut;
                    q = clampCode(static_cast<int32_t>(rshiftRoundConst(prod, rs.shift, roundOut)), lo, hi, keep);
                    if (pre.enabled)
                        q = static_cast<int32_t>(
                            rshiftRoundConst(static_cast<int64_t>(q) * gateRs.mult + mulAddGate, gateRs.shift, roundGate));
                } else {
                    q = linearEpilogue(acc[r], cmp, bias, rs, zpOut, lo, hi, keep);
                    if (pre.enabled) q = rescaleWide(q - zpOut, gateRs);
                }
                const size_t o = static_cast<size_t>(row0 + r) * channels + c;
                out[o] = static_cast<LT>(q);
                if (mask) mask[o] = keep;
            }
        }
    }
}

// 8-bit grids: thread = channel with its weight words in registers; a CTA walks blocks of
// kI8Rows rows, staging the next block's codes (padded to four-word groups, read back as
// 16-byte broadcasts) while it computes the current one.  Channels whose parameters allow it
// (32-bit accumulator plus offset, multipliers that shrink, shifts in [1, 31]) round with
// 32-bit funnel-shift arithmetic; the others take the general 64-bit functions.  Requires
// blockDim.x >= kI8Rows * KW4 * 4 and blockDim.x >= channels.
constexpr int kI8Rows = 16;

template <int KW4>
__global__ void __launch_bounds__(512)
inputLinearI8(const int32_t *__restrict__ x, int rows, int kWords, int channels, const int32_t *__restrict__ w,
              const int64_t *__restrict__ comp, const int64_t *__restrict__ biasAcc, const Rescale *__restrict__ rescale,
              int32_t zpOut, int32_t lo, int32_t hi, int16_t *__restrict__ out, uint8_t *__restrict__ mask,
              const PreRescale pre) {
    constexpr int kRowWords = KW4 * 4;
    __shared__ __align__(16) int32_t xs[2][kI8Rows][kRowWords];
    const int tid = threadIdx.x, c = tid;
    const bool live = c < channels;
    int32_t wreg[kRowWords];
#pragma unroll
    for (int kk = 0; kk < kRowWords; ++kk) wreg[kk] = (live && kk < kWords) ? w[static_cast<size_t>(kk) * channels + c] : 0;

    const int64_t offset = live ? biasAcc[c] - comp[c] : 0;
    const Rescale rs = live ? rescale[c] : Rescale{1, 1};
    const Rescale gateRs = (pre.enabled && live) ? pre.toGate[c / pre.hidden] : Rescale{1, 1};
    // |acc| < 2^30 for every input size the 32-bit accumulator admits, so acc + offset fits 32 bits;
    // mult <= 2^shift keeps the quotient inside 32 bits
    const bool narrowOut = rs.shift >= 1 && rs.shift <= 31 && offset > -(1ll << 30) && offset < (1ll << 30) && rs.mult > 0 &&
                           static_cast<int64_t>(rs.mult) <= (1ll << rs.shift);
    const bool narrowGate = gateRs.shift >= 1 && gateRs.shift <= 31 && gateRs.mult > 0 &&
                            static_cast<int64_t>(gateRs.mult) <= (1ll << min(gateRs.shift + 9, 31)) && lo >= -(1 << 20) &&
                            hi <= (1 << 20) && zpOut >= -(1 << 20) && zpOut <= (1 << 20);
    const int64_t mulAddOut = offset * rs.mult;
    const uint32_t maskOut = (1u << (rs.shift & 31)) - 1u, halfOut = 1u << ((rs.shift - 1) & 31);
    const int64_t mulAddGate = -static_cast<int64_t>(zpOut) * gateRs.mult;
    const uint32_t maskGate = (1u << (gateRs.shift & 31)) - 1u, halfGate = 1u << ((gateRs.shift - 1) & 31);

    // does every live channel of this warp take the 32-bit rounding in both rescales?
    const bool warpNarrow = __all_sync(0xffffffffu, !live || (narrowOut && (!pre.enabled || narrowGate)));

    const int blocks = (rows + kI8Rows - 1) / kI8Rows;
    const int sRow = tid / kRowWords, sWord = tid % kRowWords;  // the word of a block this thread stages
    const bool stager = tid < kI8Rows * kRowWords;
    auto fetch = [&](int blk) -> int32_t {
        const int row = blk * kI8Rows + sRow;
        return (stager && blk < blocks && row < rows && sWord < kWords) ? x[static_cast<size_t>(row) * kWords + sWord] : 0;
    };
    int buf = 0;
    if (stager) xs[0][sRow][sWord] = fetch(blockIdx.x);
    __syncthreads();
    for (int blk = blockIdx.x; blk < blocks; blk += gridDim.x) {
        const int32_t pending = fetch(blk + gridDim.x);
        const int row0 = blk * kI8Rows, nRows = min(kI8Rows, rows - row0);
        if (live) {
            int16_t *outPtr = out + static_cast<size_t>(row0) * channels + c;
            uint8_t *maskPtr = mask ? mask + static_cast<size_t>(row0) * channels + c : nullptr;
            // Two copies of the row loop: when every channel of the warp qualifies, the loop holds the
            // 32-bit rounding only (a per-value choice makes the compiler evaluate both forms).
            auto rowsLoop = [&](auto narrowTag) {
                constexpr bool kNarrow = decltype(narrowTag)::value;
                for (int r = 0; r < nRows; ++r) {
                    int32_t acc = 0;
#pragma unroll
                    for (int g4 = 0; g4 < KW4; ++g4) {
                        const int4 xv = *reinterpret_cast<const int4 *>(&xs[buf][r][4 * g4]);
                        acc = __dp4a(wreg[4 * g4], xv.x, acc);
                        acc = __dp4a(wreg[4 * g4 + 1], xv.y, acc);
                        acc = __dp4a(wreg[4 * g4 + 2], xv.z, acc);
                        acc = __dp4a(wreg[4 * g4 + 3], xv.w, acc);
                    }
                    const int64_t prod = static_cast<int64_t>(acc) * rs.mult + mulAddOut;
                    int32_t res;
                    if constexpr (kNarrow) res = rshiftRoundNarrow(prod, rs.shift, maskOut, halfOut) + zpOut;
                    else res = (narrowOut ? rshiftRoundNarrow(prod, rs.shift, maskOut, halfOut)
                                          : static_cast<int32_t>(rshiftRound(prod, rs.shift))) + zpOut;
                    uint8_t keep;
                    int32_t q = clampCode(res, lo, hi, keep);
                    if (pre.enabled) {
                        const int64_t prodGate = static_cast<int64_t>(q) * gateRs.mult + mulAddGate;
                        if constexpr (kNarrow) q = rshiftRoundNarrow(prodGate, gateRs.shift, maskGate, halfGate);
                        else q = narrowGate ? rshiftRoundNarrow(prodGate, gateRs.shift, maskGate, halfGate)
                                            : static_cast<int32_t>(rshiftRound(prodGate, gateRs.shift));
                    }
                    *outPtr = static_cast<int16_t>(q);
                    outPtr += channels;
                    if (maskPtr) {
                        *maskPtr = keep;
                        maskPtr += channels;
                    }
                }
            };
            if (warpNarrow) rowsLoop(std::true_type{});
            else rowsLoop(std::false_type{});
        }
        if (stager) xs[buf ^ 1][sRow][sWord] = pending;
        __syncthreads();
        buf ^= 1;
    }
}

// ---- 4. the recurrence: one launch for all steps ----------------------------

struct RecurrentArgs {
    int T, B, H;
    int kWords;           // padded H / pack
    int weightsInSmem;    // 1: R is staged into shared memory once; 0: read through L2
    const void *R;        // [kWords][3H] words
    const void *ih;       // LT [T][B][3H]
    const void *h0;       // AT [B][kWords*pack] initial codes
    const int64_t *comp;  // [3H]
    const int64_t *biasAcc;
    const Rescale *rescale;
    float *h;             // [T+1][B][H] dequantized (row 0 written here too)
    float *v;             // [T][B][4H] dequantized
    int32_t *hq;          // optional [T+1][B][H]
    int32_t *vq;          // optional [T][B][4H]
    uint8_t *maskHh, *maskGateIn, *maskGateOut, *maskH;
    const int *poison;    // optional device word: non-zero = the ih codes are not valid, write NaN
    // packed keep flags (recurrentForwardI8 only): bit 0..2 gate output z, r, n; 3..5 gate input; 6..8 hh linear;
    // 9..11 ih linear (read from maskIh, the input projection's flags); 12 hidden state
    uint16_t *stepBits;
    const uint8_t *maskIh;
    // optional (recurrentForwardI8 only): the hidden codes after the last step, in the layout of h0, so that the
    // next launch can carry on from there (a sequence cut into time chunks)
    void *hFinal;
};

template <class WT, class AT, class LT, int BT>
__global__ void __launch_bounds__(768)
recurrentForward(const __grid_constant__ RecurrentArgs a, const __grid_constant__ GateExec gateParam) {
    using D = Dot<WT, AT>;
    using WWord = typename D::WWord;
    using AWord = typename D::AWord;
    const int H = a.H, C = 3 * a.H, kWords = a.kWords;
    const int kPadded = kWords * D::kPack;

    extern __shared__ __align__(16) unsigned char smemRaw[];
    size_t off = 0;
    auto carve = [&](size_t bytes) {
        unsigned char *p = smemRaw + off;
        off = (off + bytes + 15) & ~static_cast<size_t>(15);
        return p;
    };
    GateExec &g = *reinterpret_cast<GateExec *>(carve(sizeof(GateExec)));
    int64_t *compS = reinterpret_cast<int64_t *>(carve(sizeof(int64_t) * C));
    int64_t *biasS = reinterpret_cast<int64_t *>(carve(sizeof(int64_t) * C));
    Rescale *rescaleS = reinterpret_cast<Rescale *>(carve(sizeof(Rescale) * C));
    int32_t *hhS = reinterpret_cast<int32_t *>(carve(sizeof(int32_t) * BT * C));
    AT *hS = reinterpret_cast<AT *>(carve(sizeof(AT) * BT * kPadded));
    WWord *RS = reinterpret_cast<WWord *>(carve(a.weightsInSmem ? sizeof(WWord) * kWords * C : 0));

    const int b0 = blockIdx.x * BT;
    const int nb = min(BT, a.B - b0);
    const int tid = threadIdx.x, nthreads = blockDim.x;

    // one-time staging
    for (int i = tid; i < static_cast<int>(sizeof(GateExec) / 4); i += nthreads)
        reinterpret_cast<int32_t *>(&g)[i] = reinterpret_cast<const int32_t *>(&gateParam)[i];
    for (int c = tid; c < C; c += nthreads) {
        compS[c] = a.comp[c];
        biasS[c] = a.biasAcc[c];
        rescaleS[c] = a.rescale[c];
    }
    const WWord *Rsrc = static_cast<const WWord *>(a.R);
    if (a.weightsInSmem) {
        for (int i = tid; i < kWords * C; i += nthreads) RS[i] = Rsrc[i];
        Rsrc = RS;
    }
    const AT *h0 = static_cast<const AT *>(a.h0);
    for (int i = tid; i < BT * kPadded; i += nthreads) {
        const int b = i / kPadded;
        hS[i] = b < nb ? h0[static_cast<size_t>(b0 + b) * kPadded + (i % kPadded)] : AT(0);
    }
    __syncthreads();

    const float scaleH = g.eff[RXMET_GRU_H];
    const int32_t zpH = g.zp[RXMET_GRU_H];
    // h[0]: the (quantized) initial state, dequantized like every other step
    for (int i = tid; i < nb * H; i += nthreads) {
        const int b = i / H, j = i % H;
        const int32_t q = hS[b * kPadded + j];
        const size_t o = static_cast<size_t>(b0 + b) * H + j;
        a.h[o] = static_cast<float>(q - zpH) * scaleH;
        if (a.hq) a.hq[o] = q;
    }

    const LT *ih = static_cast<const LT *>(a.ih);
    const AWord *hWords = reinterpret_cast<const AWord *>(hS);
    const int32_t zpOut = g.zp[RXMET_GRU_WEIGHT_HH_LINEAR];
    const int32_t loOut = g.qlo[RXMET_GRU_WEIGHT_HH_LINEAR], hiOut = g.qhi[RXMET_GRU_WEIGHT_HH_LINEAR];

    for (int t = 0; t < a.T; ++t) {
        const size_t rowBase = static_cast<size_t>(t) * a.B + b0;  // first (t, b) row of this tile

        // ---- hh linear: this tile's rows times all 3H columns
        for (int c = tid; c < C; c += nthreads) {
            typename D::Acc acc[BT];
#pragma unroll
            for (int b = 0; b < BT; ++b) acc[b] = 0;
            for (int kk = 0; kk < kWords; ++kk) {
                const WWord word = Rsrc[static_cast<size_t>(kk) * C + c];
#pragma unroll
                for (int b = 0; b < BT; ++b) D::mac(acc[b], word, hWords[b * kWords + kk]);
            }
            const int64_t cmp = compS[c], bias = biasS[c];
            const Rescale rs = rescaleS[c];
#pragma unroll
            for (int b = 0; b < BT; ++b) {
                uint8_t keep;
                hhS[b * C + c] = linearEpilogue(acc[b], cmp, bias, rs, zpOut, loOut, hiOut, keep);
                if (a.maskHh && b < nb) a.maskHh[(rowBase + b) * C + c] = keep;
            }
        }
        __syncthreads();

        // ---- gates, state update, outputs
        for (int i = tid; i < nb * H; i += nthreads) {
            const int b = i / H, j = i % H;
            const size_t row = rowBase + b;
            const LT *ihRow = ih + row * C;
            const int32_t *hhRow = hhS + b * C;
            GateMasks m;
            const int32_t hOld = hS[b * kPadded + j];
            const GateCodes q = gruCell(ihRow[j], ihRow[H + j], ihRow[2 * H + j], hhRow[j], hhRow[H + j],
                                        hhRow[2 * H + j], hOld, g, m);
            hS[b * kPadded + j] = static_cast<AT>(q.h);

            const size_t ho = (row + a.B) * H + j;  // h[t+1]
            a.h[ho] = static_cast<float>(q.h - zpH) * scaleH;
            float *vRow = a.v + row * 4 * H;
            vRow[j] = static_cast<float>(q.z - g.zp[RXMET_GRU_UPDATE_GATE_OUTPUT]) * g.eff[RXMET_GRU_UPDATE_GATE_OUTPUT];
            vRow[H + j] = static_cast<float>(q.r - g.zp[RXMET_GRU_RESET_GATE_OUTPUT]) * g.eff[RXMET_GRU_RESET_GATE_OUTPUT];
            vRow[2 * H + j] = static_cast<float>(q.n - g.zp[RXMET_GRU_NEW_GATE_OUTPUT]) * g.eff[RXMET_GRU_NEW_GATE_OUTPUT];
            vRow[3 * H + j] = static_cast<float>(hhRow[2 * H + j] - zpOut) * g.eff[RXMET_GRU_WEIGHT_HH_LINEAR];
            if (a.hq) a.hq[ho] = q.h;
            if (a.vq) {
                int32_t *vq = a.vq + row * 4 * H;
                vq[j] = q.z; vq[H + j] = q.r; vq[2 * H + j] = q.n; vq[3 * H + j] = hhRow[2 * H + j];
            }
            if (a.maskGateIn) {
                uint8_t *mi = a.maskGateIn + row * C, *mo = a.maskGateOut + row * C;
                mi[j] = m.in[0]; mi[H + j] = m.in[1]; mi[2 * H + j] = m.in[2];
                mo[j] = m.out[0]; mo[H + j] = m.out[1]; mo[2 * H + j] = m.out[2];
                a.maskH[row * H + j] = m.h;
            }
        }
        __syncthreads();
    }
}

// ---- 4b. the recurrence for 8-bit grids: weights in registers ----------------
//
// Thread c owns column c of R for the whole sequence as KW packed words (four int8 codes each),
// so a step's GEMM touches shared memory only for the broadcast reads of h (128-bit loads).  The
// ih codes of step t+1 are fetched while step t computes, which takes the L2/HBM latency off the
// serial chain.  Requires 3H <= blockDim and H <= 4*KW.
// Mode 0: 64-bit gate arithmetic; 1: 32-bit where provably exact; 2: additionally direct
// activation tables in shared memory and ih contributions pre-rescaled by the input projection.
template <int KW, int BT, int Mode, bool Packed = false>
__global__ void __launch_bounds__(KW * 12)
recurrentForwardI8(const __grid_constant__ RecurrentArgs a, const __grid_constant__ GateExec gateParam) {
    const int H = a.H, C = 3 * a.H;
    constexpr int kPadded = KW * 4;
    __shared__ GateExec g;
    __shared__ __align__(16) int8_t hS[BT * kPadded];
    extern __shared__ __align__(16) unsigned char smemRaw[];
    int32_t *hhS = reinterpret_cast<int32_t *>(smemRaw);  // [BT][C]
    int32_t *tabS = hhS + BT * C;                          // Mode 2: three direct tables

    const int tid = threadIdx.x, nthreads = blockDim.x;
    const int b0 = blockIdx.x * BT, nb = min(BT, a.B - b0);
    if (a.poison != nullptr && *reinterpret_cast<const volatile int *>(a.poison) != 0) {
        // the producer of the ih codes gave up on a bounded wait: make that loud instead of computing on garbage
        const float nan = __int_as_float(0x7fc00000);
        for (int t = 0; t <= a.T; ++t)
            for (int i = tid; i < nb * H; i += nthreads)
                a.h[(static_cast<size_t>(t) * a.B + b0 + i / H) * H + i % H] = nan;
        for (int t = 0; t < a.T; ++t)
            for (int i = tid; i < nb * 4 * H; i += nthreads)
                a.v[(static_cast<size_t>(t) * a.B + b0 + i / (4 * H)) * 4 * H + i % (4 * H)] = nan;
        return;
    }
    for (int i = tid; i < static_cast<int>(sizeof(GateExec) / 4); i += nthreads)
        reinterpret_cast<int32_t *>(&g)[i] = reinterpret_cast<const int32_t *>(&gateParam)[i];
    DirectTables tab{};
    if constexpr (Mode == 2) {
        const int inOp[3] = {RXMET_GRU_UPDATE_GATE_INPUT, RXMET_GRU_RESET_GATE_INPUT, RXMET_GRU_NEW_GATE_INPUT};
        const int outOp[3] = {RXMET_GRU_UPDATE_GATE_OUTPUT, RXMET_GRU_RESET_GATE_OUTPUT, RXMET_GRU_NEW_GATE_OUTPUT};
        const Lut *luts[3] = {&gateParam.lut_update, &gateParam.lut_reset, &gateParam.lut_new};
        int32_t *base = tabS;
        const int32_t *ptrs[3];
#pragma unroll
        for (int l = 0; l < 3; ++l) {
            const int32_t lo = gateParam.qlo[inOp[l]], span = gateParam.qhi[inOp[l]] - lo + 1;
            for (int i = tid; i < span; i += nthreads) {
                uint8_t keep;
                const int32_t code = clampCode(lutEval<true>(lo + i, *luts[l]), gateParam.qlo[outOp[l]],
                                               gateParam.qhi[outOp[l]], keep);
                base[i] = code * 2 + keep;
            }
            ptrs[l] = base;
            base += span;
        }
        tab.update = ptrs[0]; tab.reset = ptrs[1]; tab.fresh = ptrs[2];
    }

    // this thread's column of R, zero point compensation and bias term
    const bool hasColumn = tid < C;
    int32_t rw[KW];
    int64_t cmp = 0, bias = 0;
    Rescale rs{1, 0};
    {
        const int32_t *Rg = static_cast<const int32_t *>(a.R);
#pragma unroll
        for (int kk = 0; kk < KW; ++kk) rw[kk] = (hasColumn && kk < a.kWords) ? Rg[static_cast<size_t>(kk) * C + tid] : 0;
        if (hasColumn) { cmp = a.comp[tid]; bias = a.biasAcc[tid]; rs = a.rescale[tid]; }
    }
    const int8_t *h0 = static_cast<const int8_t *>(a.h0);
    const int srcPadded = a.kWords * 4;
    for (int i = tid; i < BT * kPadded; i += nthreads) {
        const int b = i / kPadded, k = i % kPadded;
        hS[i] = (b < nb && k < srcPadded) ? h0[static_cast<size_t>(b0 + b) * srcPadded + k] : int8_t(0);
    }
    __syncthreads();

    const float scaleH = g.eff[RXMET_GRU_H];
    const int32_t zpH = g.zp[RXMET_GRU_H];
    for (int i = tid; i < nb * H; i += nthreads) {
        const int b = i / H, j = i % H;
        const int32_t q = hS[b * kPadded + j];
        const size_t o = static_cast<size_t>(b0 + b) * H + j;
        a.h[o] = static_cast<float>(q - zpH) * scaleH;
        if (a.hq) a.hq[o] = q;
    }

    const int16_t *ih = static_cast<const int16_t *>(a.ih);
    const int32_t zpOut = g.zp[RXMET_GRU_WEIGHT_HH_LINEAR];
    const int32_t loOut = g.qlo[RXMET_GRU_WEIGHT_HH_LINEAR], hiOut = g.qhi[RXMET_GRU_WEIGHT_HH_LINEAR];
    const float sZ = g.eff[RXMET_GRU_UPDATE_GATE_OUTPUT], sR = g.eff[RXMET_GRU_RESET_GATE_OUTPUT];
    const float sN = g.eff[RXMET_GRU_NEW_GATE_OUTPUT], sHh = g.eff[RXMET_GRU_WEIGHT_HH_LINEAR];
    const int32_t zZ = g.zp[RXMET_GRU_UPDATE_GATE_OUTPUT], zR = g.zp[RXMET_GRU_RESET_GATE_OUTPUT];
    const int32_t zN = g.zp[RXMET_GRU_NEW_GATE_OUTPUT];

    // gate phase: element e = tid + s*nthreads of this tile (at most kSlots per thread)
    constexpr int kSlots = 2;
    const int elems = nb * H;
    int16_t ihCur[kSlots][3], ihNext[kSlots][3];
    constexpr bool packed = Packed;   // the keep flags leave as one 16-bit word per element; no byte masks are written
    uint8_t ihKeepCur[kSlots][3] = {}, ihKeepNext[kSlots][3] = {};   // combined only where they are used: no wait at the loads

    // hh epilogue of this thread's channel: with |acc + bias - comp| < 2^31, a multiplier that
    // shrinks and a shift in [1, 31] the rounding rescale is one widening multiply-add and a
    // 32-bit funnel shift (rshiftRoundNarrow); otherwise the general 64-bit functions.
    const int64_t hhOffset = bias - cmp;
    const bool hhNarrow = rs.shift >= 1 && rs.shift <= 31 && rs.mult > 0 && static_cast<int64_t>(rs.mult) <= (1ll << rs.shift) &&
                          hhOffset > -(1ll << 30) && hhOffset < (1ll << 30);
    const int64_t hhMulAdd = hhOffset * rs.mult;
    const uint32_t hhRemMask = (1u << (rs.shift & 31)) - 1u, hhHalf = 1u << ((rs.shift - 1) & 31);

    FastCell fast{};
    if constexpr (Mode == 2) fast = prepareFastCell(g);

    // per-element output offsets (fixed over the steps; a step adds its own base)
    size_t offH[kSlots], offC[kSlots], offV[kSlots];
    int elemB[kSlots], elemJ[kSlots];
#pragma unroll
    for (int s2 = 0; s2 < kSlots; ++s2) {
        const int e = tid + s2 * nthreads;
        elemB[s2] = e < elems ? e / H : 0;
        elemJ[s2] = e < elems ? e % H : 0;
        offH[s2] = static_cast<size_t>(b0 + elemB[s2]) * H + elemJ[s2];
        offC[s2] = static_cast<size_t>(b0 + elemB[s2]) * C + elemJ[s2];
        offV[s2] = static_cast<size_t>(b0 + elemB[s2]) * 4 * H + elemJ[s2];
    }
    const size_t stepH = static_cast<size_t>(a.B) * H, stepC = static_cast<size_t>(a.B) * C, stepV = 4 * stepH;
    size_t baseH = 0, baseC = 0, baseV = 0;  // t * step
    // the three ih terms of an element at the step whose base offset is given
    auto fetch = [&](size_t stepBase, int16_t (&dst)[kSlots][3]) {
#pragma unroll
        for (int s2 = 0; s2 < kSlots; ++s2) {
            if (tid + s2 * nthreads < elems) {
                const int16_t *row = ih + stepBase + offC[s2];
                dst[s2][0] = row[0]; dst[s2][1] = row[H]; dst[s2][2] = row[2 * H];
            }
        }
    };
    auto fetchKeep = [&](size_t stepBase, uint8_t (&dst)[kSlots][3]) {
#pragma unroll
        for (int s2 = 0; s2 < kSlots; ++s2) {
            if (tid + s2 * nthreads < elems) {
                const uint8_t *row = a.maskIh + stepBase + offC[s2];
                dst[s2][0] = row[0]; dst[s2][1] = row[H]; dst[s2][2] = row[2 * H];
            }
        }
    };
    fetch(0, ihCur);
    if (packed) fetchKeep(0, ihKeepCur);

    const int4 *hS4 = reinterpret_cast<const int4 *>(hS);
    for (int t = 0; t < a.T; ++t, baseH += stepH, baseC += stepC, baseV += stepV) {
        if (t + 1 < a.T) {
            fetch(baseC + stepC, ihNext);
            if (packed) fetchKeep(baseC + stepC, ihKeepNext);
        }

        if (hasColumn) {
            int32_t acc[BT];
#pragma unroll
            for (int b = 0; b < BT; ++b) acc[b] = 0;
#pragma unroll
            for (int k4 = 0; k4 < KW / 4; ++k4) {
#pragma unroll
                for (int b = 0; b < BT; ++b) {
                    const int4 hv = hS4[b * (KW / 4) + k4];
                    acc[b] = __dp4a(rw[4 * k4 + 0], hv.x, acc[b]);
                    acc[b] = __dp4a(rw[4 * k4 + 1], hv.y, acc[b]);
                    acc[b] = __dp4a(rw[4 * k4 + 2], hv.z, acc[b]);
                    acc[b] = __dp4a(rw[4 * k4 + 3], hv.w, acc[b]);
                }
            }
#pragma unroll
            for (int b = 0; b < BT; ++b) {
                uint8_t keep;
                int32_t code;
                if (hhNarrow) {
                    const int64_t prod = static_cast<int64_t>(acc[b]) * rs.mult + hhMulAdd;
                    code = clampCode(rshiftRoundNarrow(prod, rs.shift, hhRemMask, hhHalf) + zpOut, loOut, hiOut, keep);
                } else {
                    const int64_t prod = (static_cast<int64_t>(acc[b]) - cmp + bias) * static_cast<int64_t>(rs.mult);
                    code = clampCode(rshiftRoundCalled(prod, rs.shift) + zpOut, loOut, hiOut, keep);
                }
                hhS[b * C + tid] = packed ? code * 2 + keep : code;   // the flag rides with the code to the cell thread
                if (!packed && a.maskHh && b < nb) a.maskHh[baseC + static_cast<size_t>(b0 + b) * C + tid] = keep;
            }
        }
        __syncthreads();

#pragma unroll
        for (int s2 = 0; s2 < kSlots; ++s2) {
            const int e = tid + s2 * nthreads;
            if (e < elems) {
                const int b = elemB[s2], j = elemJ[s2];
                const int32_t *hhRow = hhS + b * C;
                GateMasks m;
                const int32_t hOld = hS[b * kPadded + j];
                int32_t hhz = hhRow[j], hhr = hhRow[H + j], hhn = hhRow[2 * H + j];
                uint32_t hhKeep = 0;
                if (packed) {
                    hhKeep = static_cast<uint32_t>(hhz & 1) | (static_cast<uint32_t>(hhr & 1) << 1) | (static_cast<uint32_t>(hhn & 1) << 2);
                    hhz >>= 1; hhr >>= 1; hhn >>= 1;
                }
                GateCodes q;
                if constexpr (Mode == 2)
                    q = gruCellPrepared(ihCur[s2][0], ihCur[s2][1], ihCur[s2][2], hhz, hhr, hhn, hOld, fast, tab, m);
                else
                    q = gruCell<Mode == 1>(ihCur[s2][0], ihCur[s2][1], ihCur[s2][2], hhz, hhr, hhn, hOld, g, m);
                if (packed)
                    a.stepBits[baseH + offH[s2]] = static_cast<uint16_t>(
                        m.out[0] | (m.out[1] << 1) | (m.out[2] << 2) | (m.in[0] << 3) | (m.in[1] << 4) | (m.in[2] << 5) | (hhKeep << 6) |
                        (ihKeepCur[s2][0] << 9) | (ihKeepCur[s2][1] << 10) | (ihKeepCur[s2][2] << 11) | (static_cast<uint32_t>(m.h) << 12));
                hS[b * kPadded + j] = static_cast<int8_t>(q.h);
                const size_t ho = baseH + stepH + offH[s2];  // row t + 1 of h
                a.h[ho] = static_cast<float>(q.h - zpH) * scaleH;
                float *vRow = a.v + baseV + offV[s2];
                vRow[0] = static_cast<float>(q.z - zZ) * sZ;
                vRow[H] = static_cast<float>(q.r - zR) * sR;
                vRow[2 * H] = static_cast<float>(q.n - zN) * sN;
                vRow[3 * H] = static_cast<float>(hhn - zpOut) * sHh;
                if (a.hq) a.hq[ho] = q.h;
                if (a.vq) {
                    int32_t *vq = a.vq + baseV + offV[s2];
                    vq[0] = q.z; vq[H] = q.r; vq[2 * H] = q.n; vq[3 * H] = hhn;
                }
                if (!packed && a.maskGateIn) {
                    uint8_t *mi = a.maskGateIn + baseC + offC[s2], *mo = a.maskGateOut + baseC + offC[s2];
                    mi[0] = m.in[0]; mi[H] = m.in[1]; mi[2 * H] = m.in[2];
                    mo[0] = m.out[0]; mo[H] = m.out[1]; mo[2 * H] = m.out[2];
                    a.maskH[baseH + offH[s2]] = m.h;
                }
            }
        }
#pragma unroll
        for (int s2 = 0; s2 < kSlots; ++s2)
#pragma unroll
            for (int q3 = 0; q3 < 3; ++q3) ihCur[s2][q3] = ihNext[s2][q3];
#pragma unroll
        for (int s2 = 0; s2 < kSlots; ++s2)
#pragma unroll
            for (int q3 = 0; q3 < 3; ++q3) ihKeepCur[s2][q3] = ihKeepNext[s2][q3];
        __syncthreads();
    }
    if (a.hFinal != nullptr) {
        int8_t *out = static_cast<int8_t *>(a.hFinal);
        for (int i = tid; i < BT * kPadded; i += nthreads) {
            const int b = i / kPadded, k = i % kPadded;
            if (b < nb && k < srcPadded) out[static_cast<size_t>(b0 + b) * srcPadded + k] = hS[i];
        }
    }
}

size_t recurrentSmemBytes(int H, int kWords, int pack, size_t wordBytes, size_t actBytes, int BT, bool weights) {
    const int C = 3 * H;
    auto up = [](size_t v) { return (v + 15) & ~static_cast<size_t>(15); };
    size_t s = up(sizeof(GateExec)) + up(sizeof(int64_t) * C) * 2 + up(sizeof(Rescale) * C) +
               up(sizeof(int32_t) * BT * C) + up(actBytes * BT * kWords * pack);
    if (weights) s += up(wordBytes * kWords * C);
    return s;
}

int gridFor(size_t n, int block) { return static_cast<int>(std::min<size_t>((n + block - 1) / block, 148 * 8)); }

template <class CodeT>
void launchQuantize(cudaStream_t st, const float *src, int rows, int cols, int rowsPadded, int colsPadded,
                    const float *channelScale, float scalarScale, int32_t zp, int32_t lo, int32_t hi, int weightPack,
                    CodeT *codes, int32_t *codes32, uint8_t *mask) {
    const size_t total = static_cast<size_t>(rowsPadded) * colsPadded;
    {
        KernelTimer timer__("quantizeTensor", st);
        quantizeTensor<CodeT><<<gridFor(total, 256), 256, 0, st>>>(src, rows, cols, rowsPadded, colsPadded, channelScale,
                                                                    scalarScale, zp, lo, hi, weightPack, codes, codes32, mask);
    }
    afterLaunch("quantizeTensor");
}

// Device copy of the per-channel block: 4 float arrays then 4 Rescale arrays.
struct ChannelDevice {
    const float *effW, *effR, *effBw, *effBr;
    const Rescale *gemmX, *biasX, *gemmH, *biasH;
};

ChannelDevice uploadChannels(const Exec &e, Workspace &ws, cudaStream_t st) {
    const size_t C = 3 * static_cast<size_t>(e.hidden);
    auto *block = ws.take<int32_t>(12 * C);
    RXMET_CUDA(cudaMemcpyAsync(block, pinnedChannelBlock(e, st), 12 * C * sizeof(int32_t), cudaMemcpyHostToDevice, st));
    ChannelDevice d;
    d.effW = reinterpret_cast<const float *>(block);
    d.effR = d.effW + C; d.effBw = d.effW + 2 * C; d.effBr = d.effW + 3 * C;
    d.gemmX = reinterpret_cast<const Rescale *>(block + 4 * C);
    d.biasX = d.gemmX + C; d.gemmH = d.gemmX + 2 * C; d.biasH = d.gemmX + 3 * C;
    return d;
}

// 32-bit gate arithmetic is exact when every grid difference that gets rescaled is below 2^13
// in magnitude (multipliers are below 2^16) and every table slope times its operand is below
// 2^31: linear, gate-input and gate-output grids of at most 12 bits with zero points on the grid.
bool narrowGateMath(const GateExec &g) {
    const int ops[] = {RXMET_GRU_WEIGHT_IH_LINEAR, RXMET_GRU_WEIGHT_HH_LINEAR, RXMET_GRU_UPDATE_GATE_INPUT,
                       RXMET_GRU_RESET_GATE_INPUT, RXMET_GRU_NEW_GATE_INPUT, RXMET_GRU_UPDATE_GATE_OUTPUT,
                       RXMET_GRU_RESET_GATE_OUTPUT, RXMET_GRU_NEW_GATE_OUTPUT};
    for (int op : ops) {
        const int64_t span = static_cast<int64_t>(g.qhi[op]) - g.qlo[op];
        if (span >= (1 << 12) || g.zp[op] < g.qlo[op] || g.zp[op] > g.qhi[op]) return false;
    }
    const Rescale rs[] = {g.ih_to_update, g.hh_to_update, g.ih_to_reset, g.hh_to_reset, g.ih_to_new, g.new_to_h};
    for (const Rescale &r : rs)
        if (r.mult < 0 || r.mult >= (1 << 16) || r.shift < 0) return false;
    const Lut *luts[] = {&g.lut_update, &g.lut_reset, &g.lut_new};
    for (const Lut *l : luts)
        for (int s2 = 0; s2 < kSegments; ++s2)
            if (l->q_b[s2] >= (1 << 13) || l->q_b[s2] <= -(1 << 13) || l->n_bx[s2] < 0) return false;
    return true;
}

// Mode 2 of the 8-bit recurrence: small grids everywhere, so that the direct tables stay small, the
// pre-rescaled ih terms fit 16 bits and all 32-bit products are exact.
bool fastGateMath(const GateExec &g) {
    if (!narrowGateMath(g)) return false;
    const int ops[] = {RXMET_GRU_WEIGHT_IH_LINEAR, RXMET_GRU_WEIGHT_HH_LINEAR, RXMET_GRU_UPDATE_GATE_INPUT,
                       RXMET_GRU_RESET_GATE_INPUT, RXMET_GRU_NEW_GATE_INPUT, RXMET_GRU_UPDATE_GATE_OUTPUT,
                       RXMET_GRU_RESET_GATE_OUTPUT, RXMET_GRU_NEW_GATE_OUTPUT, RXMET_GRU_H};
    for (int op : ops) {
        const int64_t span = static_cast<int64_t>(g.qhi[op]) - g.qlo[op];
        if (span >= (1 << 10) || g.zp[op] < g.qlo[op] || g.zp[op] > g.qhi[op]) return false;
    }
    if (g.quant_one <= -(1 << 15) || g.quant_one >= (1 << 15)) return false;
    const int64_t spanIh = static_cast<int64_t>(g.qhi[RXMET_GRU_WEIGHT_IH_LINEAR]) - g.qlo[RXMET_GRU_WEIGHT_IH_LINEAR];
    for (const Rescale &r : {g.ih_to_update, g.ih_to_reset, g.ih_to_new})
        if (r.shift < 0 || ((spanIh * r.mult) >> r.shift) > 30000) return false;
    for (const Rescale &r : {g.rh_to_new, g.update_old_to_h})
        if (r.mult < 0 || r.mult >= (1 << 16) || r.shift < 0) return false;
    // the prepared cell shifts 32-bit products by these amounts without a range branch
    for (const Rescale &r : {g.hh_to_update, g.hh_to_reset, g.new_to_h})
        if (r.shift > 31) return false;
    return true;
}

template <class WT, class AT, class LT>
void runTyped(const ForwardQuantCall &call, const Exec &e, Workspace &ws, cudaStream_t st) {
    using D = Dot<WT, AT>;
    using WWord = typename D::WWord;
    using AWord = typename D::AWord;
    const int T = call.T, B = call.B, I = call.I, H = call.H, C = 3 * H;
    const GateExec &g = e.gate;
    const size_t rows = static_cast<size_t>(T) * B;
    const int iWords = padTo(I, D::kPack) / D::kPack, hWords = padTo(H, D::kPack) / D::kPack;
    const int iPad = iWords * D::kPack, hPad = hWords * D::kPack;
    const bool training = call.isTraining != 0;
    const rxmet_gru_masks none{};
    const rxmet_gru_masks &mk = (training && call.masks) ? *call.masks : none;

    const ChannelDevice ch = uploadChannels(e, ws, st);
    auto *wCodes = ws.take<WWord>(static_cast<size_t>(iWords) * C);
    auto *rCodes = ws.take<WWord>(static_cast<size_t>(hWords) * C);
    auto *bwCodes = ws.take<int32_t>(C);
    auto *brCodes = ws.take<int32_t>(C);
    auto *xCodes = ws.take<AT>(rows * iPad);
    auto *h0Codes = ws.take<AT>(static_cast<size_t>(B) * hPad);
    auto *ihCodes = ws.take<LT>(rows * C);
    auto *comp = ws.take<int64_t>(4 * static_cast<size_t>(C));
    int64_t *compX = comp, *biasX = comp + C, *compH = comp + 2 * C, *biasH = comp + 3 * C;
    int *projStatus = ws.take<int>(1);  // set by the tensor-core input projection when a bounded wait gave up

    // 1. codes (8-bit weights: together with the per-channel terms of step 2)
    constexpr bool kPackedWeights = std::is_same<WT, int8_t>::value && std::is_same<AT, int8_t>::value;
    const bool fusedPrep = kPackedWeights && std::getenv("RXMET_GRU_FWD_GENERIC") == nullptr;
    bool fusedInput = false;
    if (fusedPrep) {
        WeightPrepArgs p{};
        p.W = call.W; p.R = call.R; p.bw = call.bw; p.br = call.br;
        p.I = I; p.H = H; p.C = C; p.iWords = iWords; p.hWords = hWords;
        p.effW = ch.effW; p.effR = ch.effR; p.effBw = ch.effBw; p.effBr = ch.effBr;
        p.loW = g.qlo[RXMET_GRU_W]; p.hiW = g.qhi[RXMET_GRU_W]; p.loR = g.qlo[RXMET_GRU_R]; p.hiR = g.qhi[RXMET_GRU_R];
        p.loBw = g.qlo[RXMET_GRU_BW]; p.hiBw = g.qhi[RXMET_GRU_BW]; p.loBr = g.qlo[RXMET_GRU_BR]; p.hiBr = g.qhi[RXMET_GRU_BR];
        p.wCodes = reinterpret_cast<int32_t *>(wCodes); p.rCodes = reinterpret_cast<int32_t *>(rCodes);
        p.bwCodes = bwCodes; p.brCodes = brCodes;
        p.W_q = call.W_q; p.R_q = call.R_q; p.bw_q = call.bw_q; p.br_q = call.br_q;
        p.mW = mk.W; p.mR = mk.R; p.mBw = mk.bw; p.mBr = mk.br;
        p.zpX = g.zp[RXMET_GRU_X]; p.zpH = g.zp[RXMET_GRU_H];
        p.biasRescaleX = ch.biasX; p.biasRescaleH = ch.biasH;
        p.compX = compX; p.biasX = biasX; p.compH = compH; p.biasH = biasH;
        p.prepBlocks = (C + 31) / 32;
        int xBlocks = 0;
        if constexpr (kPackedWeights) {
            if (!call.x_codes_in) {  // the input tensor rides in the same launch
                p.xSrc = call.x; p.xRows = static_cast<int>(rows); p.xCols = I; p.xColsPadded = iPad;
                p.xScale = g.eff[RXMET_GRU_X]; p.xLo = g.qlo[RXMET_GRU_X]; p.xHi = g.qhi[RXMET_GRU_X];
                p.xCodes = reinterpret_cast<int8_t *>(xCodes); p.xCodes32 = call.x_q; p.xMask = mk.x;
                xBlocks = static_cast<int>(std::min<size_t>((rows * iPad + 32 * kPrepLayers - 1) / (32 * kPrepLayers), 4 * 148));
                fusedInput = true;
            }
        }
        {
            KernelTimer timer__("prepareWeights", st);
            prepareWeightsI8<<<p.prepBlocks + xBlocks, 32 * kPrepLayers, 0, st>>>(p);
        }
        afterLaunch("prepareWeights");
    } else {
        launchQuantize<WT>(st, call.W, I, C, iPad, C, ch.effW, 0.f, 0, g.qlo[RXMET_GRU_W], g.qhi[RXMET_GRU_W], D::kPack,
                           reinterpret_cast<WT *>(wCodes), call.W_q, mk.W);
        launchQuantize<WT>(st, call.R, H, C, hPad, C, ch.effR, 0.f, 0, g.qlo[RXMET_GRU_R], g.qhi[RXMET_GRU_R], D::kPack,
                           reinterpret_cast<WT *>(rCodes), call.R_q, mk.R);
        launchQuantize<int32_t>(st, call.bw, 1, C, 1, C, ch.effBw, 0.f, 0, g.qlo[RXMET_GRU_BW], g.qhi[RXMET_GRU_BW], 1,
                                bwCodes, call.bw_q, mk.bw);
        launchQuantize<int32_t>(st, call.br, 1, C, 1, C, ch.effBr, 0.f, 0, g.qlo[RXMET_GRU_BR], g.qhi[RXMET_GRU_BR], 1,
                                brCodes, call.br_q, mk.br);
    }
    if (call.x_codes_in) {
        {
            KernelTimer timer__("narrowCodes", st);
            narrowCodes<AT><<<gridFor(rows * iPad, 256), 256, 0, st>>>(call.x_codes_in, static_cast<int>(rows), I, iPad, xCodes);
        }
        afterLaunch("narrowCodes");
    } else if (!fusedInput) {
        launchQuantize<AT>(st, call.x, static_cast<int>(rows), I, static_cast<int>(rows), iPad, nullptr,
                           g.eff[RXMET_GRU_X], g.zp[RXMET_GRU_X], g.qlo[RXMET_GRU_X], g.qhi[RXMET_GRU_X], 1, xCodes,
                           call.x_q, mk.x);
    }
    if (call.h0_codes_in) {
        {
            KernelTimer timer__("narrowCodes", st);
            narrowCodes<AT><<<gridFor(static_cast<size_t>(B) * hPad, 256), 256, 0, st>>>(call.h0_codes_in, B, H, hPad, h0Codes);
        }
        afterLaunch("narrowCodes");
    } else if (call.h0) {
        launchQuantize<AT>(st, call.h0, B, H, B, hPad, nullptr, g.eff[RXMET_GRU_H], g.zp[RXMET_GRU_H],
                           g.qlo[RXMET_GRU_H], g.qhi[RXMET_GRU_H], 1, h0Codes, nullptr, mk.h0);
    } else {
        // padding columns hold the zero point too; they meet zero weights, so they do not matter
        if constexpr (sizeof(AT) == 1) {
            // one-byte codes: a memset node instead of a kernel
            RXMET_CUDA(cudaMemsetAsync(h0Codes, g.zp[RXMET_GRU_H] & 0xff, static_cast<size_t>(B) * hPad, st));
        } else {
            KernelTimer timer__("fillCodes", st);
            fillCodes<AT><<<gridFor(static_cast<size_t>(B) * hPad, 256), 256, 0, st>>>(h0Codes, static_cast<size_t>(B) * hPad,
                                                                                      g.zp[RXMET_GRU_H]);
            afterLaunch("fillCodes");
        }
    }

    // 2. per-channel terms
    if (!fusedPrep) {
        {
            KernelTimer timer__("channelPrep", st);
            channelPrep<WT, AT><<<(C + 127) / 128, 128, 0, st>>>(wCodes, iWords, C, g.zp[RXMET_GRU_X], bwCodes, ch.biasX, compX, biasX);
        }
        afterLaunch("channelPrep");
        {
            KernelTimer timer__("channelPrep", st);
            channelPrep<WT, AT><<<(C + 127) / 128, 128, 0, st>>>(rCodes, hWords, C, g.zp[RXMET_GRU_H], brCodes, ch.biasH, compH, biasH);
        }
        afterLaunch("channelPrep");
    }

    // W8 / A16: byte-plane dp4a kernels instead of the 64-bit generic ones
    if constexpr (std::is_same<WT, int8_t>::value && std::is_same<AT, int16_t>::value && std::is_same<LT, int16_t>::value) {
        if (forwardWideTakes(e, I, H)) {
            WideCall wc{};
            wc.T = T; wc.B = B; wc.I = I; wc.H = H;
            wc.wCodes = reinterpret_cast<const int8_t *>(wCodes); wc.rCodes = reinterpret_cast<const int8_t *>(rCodes);
            wc.iPad = iPad; wc.hPad = hPad;
            wc.xCodes = reinterpret_cast<const int16_t *>(xCodes); wc.h0Codes = reinterpret_cast<const int16_t *>(h0Codes);
            wc.compX = compX; wc.biasX = biasX; wc.compH = compH; wc.biasH = biasH;
            wc.gemmX = ch.gemmX; wc.gemmH = ch.gemmH;
            wc.ihCodes = reinterpret_cast<int16_t *>(ihCodes);
            wc.h = call.h; wc.v = call.v; wc.hq = call.h_q; wc.vq = call.v_q;
            wc.maskIh = mk.weight_ih_linear; wc.maskHh = mk.weight_hh_linear; wc.maskGateIn = mk.gate_input;
            wc.maskGateOut = mk.gate_output; wc.maskH = mk.h;
            if (mk.gate_input || mk.gate_output || mk.h)
                RXMET_REQUIRE(mk.gate_input && mk.gate_output && mk.h, "gate_input, gate_output and h masks come together");
            forwardWide(wc, e, ws, st);
            return;
        }
    }

    // Which recurrence runs decides what the input projection stores.
    const int smemMax = currentDevice().smemMax, sms = currentDevice().sms;
    constexpr bool kI8 = std::is_same<WT, int8_t>::value && std::is_same<AT, int8_t>::value &&
                         std::is_same<LT, int16_t>::value;
    const int blockI8 = padTo(C, 32);
    int btI8 = (B > 2 * sms) ? 4 : ((B > sms) ? 2 : 1);
    if (const char *env = std::getenv("RXMET_GRU_FWD_BT")) btI8 = std::atoi(env);
    const bool registerPath = kI8 && blockI8 <= 768 && hWords <= 64 && btI8 * H <= 2 * blockI8 &&
                              (btI8 == 1 || btI8 == 2 || btI8 == 4) && std::getenv("RXMET_GRU_FWD_GENERIC") == nullptr;
    int mode = 0;
    if (registerPath) {
        mode = fastGateMath(g) ? 2 : (narrowGateMath(g) ? 1 : 0);
        if (const char *env = std::getenv("RXMET_GRU_FWD_MODE")) mode = std::min(mode, std::atoi(env));
    }
    PreRescale pre{};
    pre.enabled = mode == 2 ? 1 : 0;
    pre.hidden = H;
    pre.toGate[0] = g.ih_to_update; pre.toGate[1] = g.ih_to_reset; pre.toGate[2] = g.ih_to_new;

    // 3. input projection, all steps
    bool tensorProjection = false;
    std::vector<int> chunks{T};   // time chunks of the overlapped pipeline (one = none)
    {
        const int block = std::min(padTo(C, 32), 512);
        const int kw4 = (iWords + 3) / 4;
        bool specialised = false;
        if constexpr (kI8) {
            if (iproj::eligible(C, H, iWords, xCodes, ihCodes, mk.weight_ih_linear) && std::getenv("RXMET_GRU_FWD_GENERIC") == nullptr) {
                // tcgen05 kind::i8 GEMM with the fused epilogue
                specialised = true;
                tensorProjection = true;
                RXMET_CUDA(cudaMemsetAsync(projStatus, 0, sizeof(int), st));
                // rows [r0, r0 + n) on stream `s`
                auto projectRows = [&](size_t r0, size_t n, cudaStream_t s) {
                    iproj::Problem pj{};
                    pj.x = reinterpret_cast<const int32_t *>(xCodes) + r0 * iWords; pj.rows = static_cast<int>(n); pj.kWords = iWords;
                    pj.w = reinterpret_cast<const int32_t *>(wCodes); pj.C = C;
                    pj.comp = compX; pj.biasAcc = biasX; pj.rescale = ch.gemmX;
                    pj.zpOut = g.zp[RXMET_GRU_WEIGHT_IH_LINEAR]; pj.lo = g.qlo[RXMET_GRU_WEIGHT_IH_LINEAR];
                    pj.hi = g.qhi[RXMET_GRU_WEIGHT_IH_LINEAR];
                    pj.pre = pre; pj.out = reinterpret_cast<int16_t *>(ihCodes) + r0 * C;
                    pj.mask = mk.weight_ih_linear ? mk.weight_ih_linear + r0 * C : nullptr; pj.status = projStatus;
                    iproj::launch(pj, sms, s);
                };
                // Cut into time chunks, the projection of chunk i + 1 runs on the library's second stream under the
                // recurrence of chunk i; only the first (short) chunk's projection stays in front of the recurrence.
                // Chunk borders must keep the 16-byte alignment of the operand rows.
                if (registerPath && (static_cast<size_t>(B) * iPad) % 16 == 0 && (static_cast<size_t>(B) * C) % 16 == 0)
                    chunks = overlapChunks(T, rows, false);
                if (chunks.size() > 1) {
                    OverlapLane &lane = overlapLane();
                    projectRows(0, static_cast<size_t>(chunks[0]) * B, st);
                    RXMET_CUDA(cudaEventRecord(lane.fork[0], st));
                    RXMET_CUDA(cudaStreamWaitEvent(lane.stream, lane.fork[0], 0));
                    int t0 = chunks[0];
                    for (size_t i = 1; i < chunks.size(); ++i) {
                        projectRows(static_cast<size_t>(t0) * B, static_cast<size_t>(chunks[i]) * B, lane.stream);
                        RXMET_CUDA(cudaEventRecord(lane.done[i], lane.stream));
                        t0 += chunks[i];
                    }
                } else {
                    projectRows(0, rows, st);
                }
            }
        }
        if constexpr (kI8) {
            if (!specialised && C <= 512 && kw4 <= 4 && block >= kI8Rows * kw4 * 4 && std::getenv("RXMET_GRU_FWD_GENERIC") == nullptr) {
                specialised = true;
                const int blocks = static_cast<int>((rows + kI8Rows - 1) / kI8Rows);
                const int32_t zp = g.zp[RXMET_GRU_WEIGHT_IH_LINEAR], qlo = g.qlo[RXMET_GRU_WEIGHT_IH_LINEAR],
                              qhi = g.qhi[RXMET_GRU_WEIGHT_IH_LINEAR];
                KernelTimer timer__("inputLinear", st);
#define RXMET_IL_CASE(N)                                                                                                   \
    case N: {                                                                                                              \
        const int perSm = residentPerSm(reinterpret_cast<const void *>(inputLinearI8<N>), block, 0);                       \
        const int grid = std::max(1, std::min(blocks, sms * std::max(1, perSm)));                                          \
        inputLinearI8<N><<<grid, block, 0, st>>>(reinterpret_cast<const int32_t *>(xCodes), static_cast<int>(rows), iWords, C, \
                                                 reinterpret_cast<const int32_t *>(wCodes), compX, biasX, ch.gemmX, zp, qlo, qhi, \
                                                 reinterpret_cast<int16_t *>(ihCodes), mk.weight_ih_linear, pre);            \
    } break;
                switch (kw4) {
                    RXMET_IL_CASE(1) RXMET_IL_CASE(2) RXMET_IL_CASE(3) RXMET_IL_CASE(4)
                }
#undef RXMET_IL_CASE
            }
        }
        if (!specialised) {
            const size_t smem = sizeof(AWord) * kLinearRows * iWords;
            const int grid = static_cast<int>((rows + kLinearRows - 1) / kLinearRows);
            KernelTimer timer__("inputLinear", st);
            inputLinear<WT, AT, LT><<<grid, block, smem, st>>>(
                reinterpret_cast<const AWord *>(xCodes), static_cast<int>(rows), iWords, C, wCodes, compX, biasX, ch.gemmX,
                g.zp[RXMET_GRU_WEIGHT_IH_LINEAR], g.qlo[RXMET_GRU_WEIGHT_IH_LINEAR], g.qhi[RXMET_GRU_WEIGHT_IH_LINEAR],
                ihCodes, mk.weight_ih_linear, pre);
        }
        afterLaunch("inputLinear");
    }

    // 4. recurrence
    RecurrentArgs a{};
    a.T = T; a.B = B; a.H = H; a.kWords = hWords;
    a.R = rCodes; a.ih = ihCodes; a.h0 = h0Codes;
    a.comp = compH; a.biasAcc = biasH; a.rescale = ch.gemmH;
    a.h = call.h; a.v = call.v; a.hq = call.h_q; a.vq = call.v_q;
    a.maskHh = mk.weight_hh_linear; a.maskGateIn = mk.gate_input; a.maskGateOut = mk.gate_output; a.maskH = mk.h;
    a.poison = tensorProjection ? projStatus : nullptr;
    a.stepBits = call.stepFlags; a.maskIh = mk.weight_ih_linear;
    if (call.stepFlags) {
        RXMET_REQUIRE(training && mk.weight_ih_linear, "packed step flags need a training forward with the weight_ih_linear mask");
        if (!registerPath || mode != 2)
            fail(RXMET_ERR_UNSUPPORTED, "packed step flags are written by the 8-bit register path with direct activation tables only");
    }
    if (mk.gate_input || mk.gate_output || mk.h)
        RXMET_REQUIRE(mk.gate_input && mk.gate_output && mk.h, "gate_input, gate_output and h masks come together");

    // Batch tile: as small as keeps every SM busy; a larger tile only amortises weight reads.
    const int bt = (B >= 4 * 2 * sms) ? 4 : ((B >= 2 * 2 * sms) ? 2 : 1);
    const int block = std::min(padTo(C, 32), 768);
    auto launch = [&](auto kernel, int BT) {
        size_t smem = recurrentSmemBytes(H, hWords, D::kPack, sizeof(WWord), sizeof(AT), BT, true);
        a.weightsInSmem = smem <= static_cast<size_t>(smemMax) ? 1 : 0;
        if (!a.weightsInSmem) smem = recurrentSmemBytes(H, hWords, D::kPack, sizeof(WWord), sizeof(AT), BT, false);
        if (smem > static_cast<size_t>(smemMax))
            fail(RXMET_ERR_UNSUPPORTED, "hidden size %d needs %zu bytes of shared memory per CTA", H, smem);
        ensureDynamicSmem(reinterpret_cast<const void *>(kernel), smem);
        {
            KernelTimer timer__("recurrentForward", st);
            kernel<<<(B + BT - 1) / BT, block, smem, st>>>(a, g);
        }
        afterLaunch("recurrentForward");
    };
    if constexpr (kI8) {
        if (registerPath) {
            // register-resident variant: one thread per column, at most two gate elements per thread
            size_t smem = sizeof(int32_t) * btI8 * C;
            if (mode == 2) {
                for (int op : {RXMET_GRU_UPDATE_GATE_INPUT, RXMET_GRU_RESET_GATE_INPUT, RXMET_GRU_NEW_GATE_INPUT})
                    smem += sizeof(int32_t) * (g.qhi[op] - g.qlo[op] + 1);
            }
            auto launchSteps = [&](const RecurrentArgs &ra) {
                auto launchI8 = [&](auto kernel) { kernel<<<(B + btI8 - 1) / btI8, blockI8, smem, st>>>(ra, g); };
                {
                    KernelTimer timer__("recurrentForward", st);
                    bool done = false;
#define RXMET_I8_CASE(KW, BT)                                                 \
    if (!done && hWords <= KW && btI8 == BT) {                                 \
        if (mode == 2 && ra.stepBits) launchI8(recurrentForwardI8<KW, BT, 2, true>); \
        else if (mode == 2) launchI8(recurrentForwardI8<KW, BT, 2>);           \
        else if (mode == 1) launchI8(recurrentForwardI8<KW, BT, 1>);           \
        else launchI8(recurrentForwardI8<KW, BT, 0>);                          \
        done = true;                                                           \
    }
                    RXMET_I8_CASE(16, 1) RXMET_I8_CASE(16, 2) RXMET_I8_CASE(16, 4)
                    RXMET_I8_CASE(32, 1) RXMET_I8_CASE(32, 2) RXMET_I8_CASE(32, 4)
                    RXMET_I8_CASE(64, 1) RXMET_I8_CASE(64, 2) RXMET_I8_CASE(64, 4)
#undef RXMET_I8_CASE
                }
                afterLaunch("recurrentForwardI8");
            };
            if (chunks.size() == 1) {
                launchSteps(a);
                return;
            }
            // one launch per time chunk: the hidden codes travel from launch to launch in the h0 buffer, every other
            // operand is the whole-sequence array moved to the chunk's first step
            OverlapLane &lane = overlapLane();
            int t0 = 0;
            for (size_t i = 0; i < chunks.size(); ++i) {
                if (i > 0) RXMET_CUDA(cudaStreamWaitEvent(st, lane.done[i], 0));
                const size_t r0 = static_cast<size_t>(t0) * B;
                RecurrentArgs ra = a;
                ra.T = chunks[i];
                ra.hFinal = (i + 1 < chunks.size()) ? h0Codes : nullptr;
                ra.ih = reinterpret_cast<const int16_t *>(ihCodes) + r0 * C;
                ra.h = a.h + r0 * H; ra.v = a.v + r0 * 4 * H;
                if (a.hq) ra.hq = a.hq + r0 * H;
                if (a.vq) ra.vq = a.vq + r0 * 4 * H;
                if (a.maskHh) ra.maskHh = a.maskHh + r0 * C;
                if (a.maskGateIn) ra.maskGateIn = a.maskGateIn + r0 * C;
                if (a.maskGateOut) ra.maskGateOut = a.maskGateOut + r0 * C;
                if (a.maskH) ra.maskH = a.maskH + r0 * H;
                if (a.stepBits) ra.stepBits = a.stepBits + r0 * H;
                if (a.maskIh) ra.maskIh = a.maskIh + r0 * C;
                launchSteps(ra);
                t0 += chunks[i];
            }
            return;
        }
    }
    if (bt == 4) launch(recurrentForward<WT, AT, LT, 4>, 4);
    else if (bt == 2) launch(recurrentForward<WT, AT, LT, 2>, 2);
    else launch(recurrentForward<WT, AT, LT, 1>, 1);
}

template <class WT, class AT, class LT>
void sizeTyped(WorkspaceSizer &ws, int T, int B, int I, int H) {
    using D = Dot<WT, AT>;
    const size_t C = 3 * static_cast<size_t>(H), rows = static_cast<size_t>(T) * B;
    const int iWords = padTo(I, D::kPack) / D::kPack, hWords = padTo(H, D::kPack) / D::kPack;
    ws.take<int32_t>(12 * C);
    ws.take<typename D::WWord>(iWords * C);
    ws.take<typename D::WWord>(hWords * C);
    ws.take<int32_t>(C);
    ws.take<int32_t>(C);
    ws.take<AT>(rows * iWords * D::kPack);
    ws.take<AT>(static_cast<size_t>(B) * hWords * D::kPack);
    ws.take<LT>(rows * C);
    ws.take<int64_t>(4 * C);
    ws.take<int>(1);
}

}  // namespace

size_t fpCarrierBytes(int T, int B, int I, int H);

size_t forwardQuantWorkspaceBytes(int T, int B, int I, int H) {
    // The widest storage classes bound every configuration; the byte-plane kernels add their operands.
    WorkspaceSizer ws;
    sizeTyped<int32_t, int32_t, int32_t>(ws, T, B, I, H);
    return std::max(ws.used() + 4096 + forwardWideExtraBytes(T, B, I, H), fpCarrierBytes(T, B, I, H));
}

// ---- FP32 carrier -------------------------------------------------------------------------------------------
//
// The reference's second quantized carrier (its CUDA default for float code storage): codes held in floats,
// rescale = rint(x * ratio) in float, the 16-segment tables evaluated in float
// (operators/quant-gru/src/gru_forward_gpu_quant_fp.cu).  The matrix products are formed exactly on the integer
// codes and converted to float once, which equals the reference's float GEMM whenever the sums stay below 2^24
// (always for 8-bit grids up to K = 512; beyond, the reference's own result depends on its GEMM's summation
// order).  Everything behind the product follows the reference's float operations one by one.
__device__ __forceinline__ float fpClamp(float v, float lo, float hi, uint8_t &keep) {
    keep = (v < lo || v > hi) ? 0 : 1;
    return fmaxf(lo, fminf(v, hi));
}
// biasRescaleInline, gru_forward_gpu_quant_fp.cu:138-163
__device__ __forceinline__ float fpLinear(float gemm, float bias, float sumZp, float invGemm, float invBias, float zpOut, float lo,
                                          float hi, uint8_t &keep) {
    const float biasTerm = rintf(__fmul_rn(bias, invBias));
    const float combined = __fadd_rn(__fsub_rn(gemm, sumZp), biasTerm);
    return fpClamp(__fadd_rn(rintf(__fmul_rn(combined, invGemm)), zpOut), lo, hi, keep);
}
// piecewiseLinearFP, gru_forward_gpu_quant_fp.cu:91-108
__device__ __forceinline__ float fpTable(float qx, const Lut &lut, float lo, float hi, uint8_t &keep) {
    int seg = kSegments - 1;
#pragma unroll
    for (int i = kSegments - 2; i >= 0; --i) seg = (qx < static_cast<float>(lut.threshold[i])) ? i : seg;
    const float product = __fmul_rn(static_cast<float>(lut.q_b[seg]), __fsub_rn(qx, static_cast<float>(lut.zp_x)));
    const float value = __fadd_rn(rintf(ldexpf(product, -lut.n_bx[seg])), static_cast<float>(lut.term_c[seg]));
    return fpClamp(value, lo, hi, keep);
}

// sums[c] = float(sum_k codes[k][c]) * zp: the zero-point compensation term (computeWeightSumKernel)
__global__ void fpWeightSums(const int32_t *__restrict__ codes, int K, int C, float zp, float *__restrict__ sums) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    int32_t sum = 0;
    for (int k = 0; k < K; ++k) sum += codes[static_cast<size_t>(k) * C + c];
    sums[c] = __fmul_rn(static_cast<float>(sum), zp);
}

struct FpLinearArgs {
    const int32_t *x;       // [rows][I]
    const int32_t *W;       // [I][C]
    const int32_t *bias;    // [C]
    const float *sumZp, *invGemm, *invBias;
    int rows, I, C;
    float zpOut, lo, hi;
    float *out;             // [rows][C] float codes
    uint8_t *mask;          // optional
};
__global__ void fpInputLinear(const FpLinearArgs a) {
    const size_t total = static_cast<size_t>(a.rows) * a.C;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t row = i / a.C;
        const int c = static_cast<int>(i % a.C);
        const int32_t *xr = a.x + row * a.I;
        int64_t acc = 0;
        for (int k = 0; k < a.I; ++k) acc += static_cast<int64_t>(xr[k]) * a.W[static_cast<size_t>(k) * a.C + c];
        uint8_t keep;
        a.out[i] = fpLinear(static_cast<float>(acc), static_cast<float>(a.bias[c]), a.sumZp[c], a.invGemm[c], a.invBias[c], a.zpOut, a.lo,
                            a.hi, keep);
        if (a.mask) a.mask[i] = keep;
    }
}

struct FpRecurrentArgs {
    int T, B, H;
    const int32_t *R;       // [H][3H]
    const int32_t *bias;    // [3H] br codes
    const float *sumZp, *invGemm, *invBias;
    const float *ih;        // [T][B][3H] float codes of the ih linear stage
    const int32_t *h0;      // [B][H] codes (the zero point when no initial state was given)
    FpCarrierScalars s;
    float *h, *v;           // dequantized outputs
    int32_t *hq, *vq;       // optional codes
    uint8_t *maskHh, *maskGateIn, *maskGateOut, *maskH;
};

template <int BT>
__global__ void __launch_bounds__(768) fpRecurrent(const __grid_constant__ FpRecurrentArgs a, const __grid_constant__ GateExec g) {
    extern __shared__ __align__(16) unsigned char fpSmem[];
    int32_t *hS = reinterpret_cast<int32_t *>(fpSmem);          // [BT][H] hidden codes
    float *hhS = reinterpret_cast<float *>(hS + BT * a.H);       // [BT][3H] hh linear codes
    const int H = a.H, C = 3 * a.H, tid = threadIdx.x, nthreads = blockDim.x;
    const int b0 = blockIdx.x * BT, nb = min(BT, a.B - b0);
    const FpCarrierScalars &s = a.s;
    const float zpH = s.zp[RXMET_GRU_H], zpHh = s.zp[RXMET_GRU_WEIGHT_HH_LINEAR], zpIh = s.zp[RXMET_GRU_WEIGHT_IH_LINEAR];
    for (int i = tid; i < BT * H; i += nthreads) {
        const int b = i / H, j = i % H;
        const int32_t q = b < nb ? a.h0[static_cast<size_t>(b0 + b) * H + j] : g.zp[RXMET_GRU_H];
        hS[i] = q;
        if (b < nb) {
            const size_t o = static_cast<size_t>(b0 + b) * H + j;
            a.h[o] = static_cast<float>(q - g.zp[RXMET_GRU_H]) * g.eff[RXMET_GRU_H];
            if (a.hq) a.hq[o] = q;
        }
    }
    __syncthreads();
    for (int t = 0; t < a.T; ++t) {
        // hh linear stage of this step: exact integer product, then the reference's float bias-and-rescale
        for (int c = tid; c < C; c += nthreads) {
            int64_t acc[BT];
#pragma unroll
            for (int b = 0; b < BT; ++b) acc[b] = 0;
            for (int k = 0; k < H; ++k) {
                const int64_t w = a.R[static_cast<size_t>(k) * C + c];
#pragma unroll
                for (int b = 0; b < BT; ++b) acc[b] += w * hS[b * H + k];
            }
            const float bias = static_cast<float>(a.bias[c]);
#pragma unroll
            for (int b = 0; b < BT; ++b) {
                uint8_t keep;
                hhS[b * C + c] = fpLinear(static_cast<float>(acc[b]), bias, a.sumZp[c], a.invGemm[c], a.invBias[c], zpHh,
                                          s.lo[RXMET_GRU_WEIGHT_HH_LINEAR], s.hi[RXMET_GRU_WEIGHT_HH_LINEAR], keep);
                if (a.maskHh && b < nb) a.maskHh[(static_cast<size_t>(t) * a.B + b0 + b) * C + c] = keep;
            }
        }
        __syncthreads();
        for (int e = tid; e < nb * H; e += nthreads) {
            const int b = e / H, j = e % H;
            const size_t row = static_cast<size_t>(t) * a.B + b0 + b;
            const float *ih = a.ih + row * C + j;
            const float *hh = hhS + b * C + j;
            uint8_t kin[3], kout[3], kh;
            // update and reset gates (computeUpdateGateFP / computeResetGateFP)
            const float zin = __fadd_rn(__fadd_rn(rintf(__fmul_rn(__fsub_rn(ih[0], zpIh), s.ihToUpdate)),
                                                  rintf(__fmul_rn(__fsub_rn(hh[0], zpHh), s.hhToUpdate))),
                                        s.zp[RXMET_GRU_UPDATE_GATE_INPUT]);
            const float z = fpTable(fpClamp(zin, s.lo[RXMET_GRU_UPDATE_GATE_INPUT], s.hi[RXMET_GRU_UPDATE_GATE_INPUT], kin[0]), g.lut_update,
                                    s.lo[RXMET_GRU_UPDATE_GATE_OUTPUT], s.hi[RXMET_GRU_UPDATE_GATE_OUTPUT], kout[0]);
            const float rin = __fadd_rn(__fadd_rn(rintf(__fmul_rn(__fsub_rn(ih[H], zpIh), s.ihToReset)),
                                                  rintf(__fmul_rn(__fsub_rn(hh[H], zpHh), s.hhToReset))),
                                        s.zp[RXMET_GRU_RESET_GATE_INPUT]);
            const float r = fpTable(fpClamp(rin, s.lo[RXMET_GRU_RESET_GATE_INPUT], s.hi[RXMET_GRU_RESET_GATE_INPUT], kin[1]), g.lut_reset,
                                    s.lo[RXMET_GRU_RESET_GATE_OUTPUT], s.hi[RXMET_GRU_RESET_GATE_OUTPUT], kout[1]);
            // candidate (computeNewGateFP)
            const float hhn = hh[2 * H];
            const float rh = rintf(__fmul_rn(__fmul_rn(__fsub_rn(r, s.zp[RXMET_GRU_RESET_GATE_OUTPUT]), __fsub_rn(hhn, zpHh)), s.rhToNew));
            const float nin = __fadd_rn(__fadd_rn(rintf(__fmul_rn(__fsub_rn(ih[2 * H], zpIh), s.ihToNew)), rh), s.zp[RXMET_GRU_NEW_GATE_INPUT]);
            const float n = fpTable(fpClamp(nin, s.lo[RXMET_GRU_NEW_GATE_INPUT], s.hi[RXMET_GRU_NEW_GATE_INPUT], kin[2]), g.lut_new,
                                    s.lo[RXMET_GRU_NEW_GATE_OUTPUT], s.hi[RXMET_GRU_NEW_GATE_OUTPUT], kout[2]);
            // new hidden code (computeHiddenStateFP): the two products are summed with one fused multiply-add, as the
            // reference's device code is compiled; both are exact below 2^24, so the order is immaterial there
            const float hOld = static_cast<float>(hS[b * H + j]);
            const float nAligned = __fadd_rn(rintf(__fmul_rn(__fsub_rn(n, s.zp[RXMET_GRU_NEW_GATE_OUTPUT]), s.newToH)), zpH);
            const float oldMul = __fmul_rn(__fsub_rn(z, s.zp[RXMET_GRU_UPDATE_GATE_OUTPUT]), __fsub_rn(hOld, zpH));
            const float sum = __fmaf_rn(__fsub_rn(s.quantOne, z), __fsub_rn(nAligned, zpH), oldMul);
            const float hNew = fpClamp(__fadd_rn(rintf(__fmul_rn(sum, s.updateOldToH)), zpH), s.lo[RXMET_GRU_H], s.hi[RXMET_GRU_H], kh);
            const int32_t hCode = static_cast<int32_t>(hNew);
            hS[b * H + j] = hCode;
            const size_t ho = (row + a.B) * H + j;
            a.h[ho] = static_cast<float>(hCode - g.zp[RXMET_GRU_H]) * g.eff[RXMET_GRU_H];
            float *vRow = a.v + row * 4 * H + j;
            const int32_t zc = static_cast<int32_t>(z), rc = static_cast<int32_t>(r), nc = static_cast<int32_t>(n), hc = static_cast<int32_t>(hhn);
            vRow[0] = static_cast<float>(zc - g.zp[RXMET_GRU_UPDATE_GATE_OUTPUT]) * g.eff[RXMET_GRU_UPDATE_GATE_OUTPUT];
            vRow[H] = static_cast<float>(rc - g.zp[RXMET_GRU_RESET_GATE_OUTPUT]) * g.eff[RXMET_GRU_RESET_GATE_OUTPUT];
            vRow[2 * H] = static_cast<float>(nc - g.zp[RXMET_GRU_NEW_GATE_OUTPUT]) * g.eff[RXMET_GRU_NEW_GATE_OUTPUT];
            vRow[3 * H] = static_cast<float>(hc - g.zp[RXMET_GRU_WEIGHT_HH_LINEAR]) * g.eff[RXMET_GRU_WEIGHT_HH_LINEAR];
            if (a.hq) a.hq[ho] = hCode;
            if (a.vq) {
                int32_t *vq = a.vq + row * 4 * H + j;
                vq[0] = zc; vq[H] = rc; vq[2 * H] = nc; vq[3 * H] = hc;
            }
            if (a.maskGateIn) {
                uint8_t *mi = a.maskGateIn + row * C + j, *mo = a.maskGateOut + row * C + j;
                mi[0] = kin[0]; mi[H] = kin[1]; mi[2 * H] = kin[2];
                mo[0] = kout[0]; mo[H] = kout[1]; mo[2 * H] = kout[2];
                a.maskH[row * H + j] = kh;
            }
        }
        __syncthreads();
    }
}

size_t fpCarrierBytes(int T, int B, int I, int H) {
    const size_t rows = static_cast<size_t>(T) * B, C = 3 * static_cast<size_t>(H);
    WorkspaceSizer ws;
    ws.take<float>(12 * C);
    ws.take<int32_t>(static_cast<size_t>(I) * C);
    ws.take<int32_t>(static_cast<size_t>(H) * C);
    ws.take<int32_t>(2 * C);
    ws.take<int32_t>(rows * I);
    ws.take<int32_t>(static_cast<size_t>(B) * H);
    ws.take<float>(rows * C);
    ws.take<float>(6 * C);
    return ws.used() + 4096;
}

void forwardFpCarrier(const ForwardQuantCall &call, const Exec &e, Workspace &ws, cudaStream_t st) {
    const int T = call.T, B = call.B, I = call.I, H = call.H, C = 3 * H;
    const GateExec &g = e.gate;
    const size_t rows = static_cast<size_t>(T) * B;
    RXMET_REQUIRE(call.x != nullptr && call.x_codes_in == nullptr && call.h0_codes_in == nullptr, "the FP32 carrier takes float inputs");
    RXMET_REQUIRE(call.stepFlags == nullptr, "the FP32 carrier writes byte masks");
    const bool training = call.isTraining != 0;
    const rxmet_gru_masks none{};
    const rxmet_gru_masks &mk = (training && call.masks) ? *call.masks : none;
    const FpCarrierParams fp = deriveFpCarrier(*call.fpCarrier);

    const ChannelDevice ch = uploadChannels(e, ws, st);
    int32_t *wq = ws.take<int32_t>(static_cast<size_t>(I) * C), *rq = ws.take<int32_t>(static_cast<size_t>(H) * C);
    int32_t *biasQ = ws.take<int32_t>(2 * static_cast<size_t>(C));
    int32_t *xq = ws.take<int32_t>(rows * I), *h0q = ws.take<int32_t>(static_cast<size_t>(B) * H);
    float *ih = ws.take<float>(rows * C);
    float *chan = ws.take<float>(6 * static_cast<size_t>(C));   // four ratio arrays, two zero-point compensation arrays
    launchQuantize<int32_t>(st, call.W, I, C, I, C, ch.effW, 0.f, 0, g.qlo[RXMET_GRU_W], g.qhi[RXMET_GRU_W], 1, wq, call.W_q, mk.W);
    launchQuantize<int32_t>(st, call.R, H, C, H, C, ch.effR, 0.f, 0, g.qlo[RXMET_GRU_R], g.qhi[RXMET_GRU_R], 1, rq, call.R_q, mk.R);
    launchQuantize<int32_t>(st, call.bw, 1, C, 1, C, ch.effBw, 0.f, 0, g.qlo[RXMET_GRU_BW], g.qhi[RXMET_GRU_BW], 1, biasQ, call.bw_q, mk.bw);
    launchQuantize<int32_t>(st, call.br, 1, C, 1, C, ch.effBr, 0.f, 0, g.qlo[RXMET_GRU_BR], g.qhi[RXMET_GRU_BR], 1, biasQ + C, call.br_q, mk.br);
    launchQuantize<int32_t>(st, call.x, static_cast<int>(rows), I, static_cast<int>(rows), I, nullptr, g.eff[RXMET_GRU_X], g.zp[RXMET_GRU_X],
                            g.qlo[RXMET_GRU_X], g.qhi[RXMET_GRU_X], 1, xq, call.x_q, mk.x);
    if (call.h0) {
        launchQuantize<int32_t>(st, call.h0, B, H, B, H, nullptr, g.eff[RXMET_GRU_H], g.zp[RXMET_GRU_H], g.qlo[RXMET_GRU_H],
                                g.qhi[RXMET_GRU_H], 1, h0q, nullptr, mk.h0);
    } else {
        fillCodes<int32_t><<<gridFor(static_cast<size_t>(B) * H, 256), 256, 0, st>>>(h0q, static_cast<size_t>(B) * H, g.zp[RXMET_GRU_H]);
        afterLaunch("fillCodes");
    }
    // pageable source: the runtime stages it before the call returns
    RXMET_CUDA(cudaMemcpyAsync(chan, fp.channel.data(), sizeof(float) * 4 * C, cudaMemcpyHostToDevice, st));
    float *sumX = chan + 4 * static_cast<size_t>(C), *sumH = chan + 5 * static_cast<size_t>(C);
    fpWeightSums<<<(C + 127) / 128, 128, 0, st>>>(wq, I, C, fp.s.zp[RXMET_GRU_X], sumX);
    afterLaunch("fpWeightSums");
    fpWeightSums<<<(C + 127) / 128, 128, 0, st>>>(rq, H, C, fp.s.zp[RXMET_GRU_H], sumH);
    afterLaunch("fpWeightSums");
    {
        FpLinearArgs a{};
        a.x = xq; a.W = wq; a.bias = biasQ; a.sumZp = sumX; a.invGemm = chan; a.invBias = chan + C;
        a.rows = static_cast<int>(rows); a.I = I; a.C = C;
        a.zpOut = fp.s.zp[RXMET_GRU_WEIGHT_IH_LINEAR]; a.lo = fp.s.lo[RXMET_GRU_WEIGHT_IH_LINEAR]; a.hi = fp.s.hi[RXMET_GRU_WEIGHT_IH_LINEAR];
        a.out = ih; a.mask = mk.weight_ih_linear;
        KernelTimer timer__("inputLinear", st);
        fpInputLinear<<<gridFor(rows * C, 256), 256, 0, st>>>(a);
        afterLaunch("inputLinear");
    }
    {
        FpRecurrentArgs a{};
        a.T = T; a.B = B; a.H = H; a.R = rq; a.bias = biasQ + C; a.sumZp = sumH; a.invGemm = chan + 2 * static_cast<size_t>(C);
        a.invBias = chan + 3 * static_cast<size_t>(C); a.ih = ih; a.h0 = h0q; a.s = fp.s;
        a.h = call.h; a.v = call.v; a.hq = call.h_q; a.vq = call.v_q;
        a.maskHh = mk.weight_hh_linear; a.maskGateIn = mk.gate_input; a.maskGateOut = mk.gate_output; a.maskH = mk.h;
        if (mk.gate_input || mk.gate_output || mk.h)
            RXMET_REQUIRE(mk.gate_input && mk.gate_output && mk.h, "gate_input, gate_output and h masks come together");
        const int sms = currentDevice().sms;
        const int bt = B >= 4 * sms ? 4 : (B >= 2 * sms ? 2 : 1);
        const int block = std::min((C + 31) / 32 * 32, 768);
        auto launch = [&](auto kernel, int BT) {
            const size_t smem = sizeof(int32_t) * BT * H + sizeof(float) * BT * C;
            ensureDynamicSmem(reinterpret_cast<const void *>(kernel), smem);
            KernelTimer timer__("recurrentForward", st);
            kernel<<<(B + BT - 1) / BT, block, smem, st>>>(a, g);
        };
        if (bt == 4) launch(fpRecurrent<4>, 4);
        else if (bt == 2) launch(fpRecurrent<2>, 2);
        else launch(fpRecurrent<1>, 1);
        afterLaunch("recurrentForward");
    }
}

bool packedFlagsSupported(const Exec &e, int B, int I, int H) {
    (void)I;
    if (e.weightClass != CodeClass::I8 || e.actClass != CodeClass::I8 || e.linearClass == CodeClass::I32) return false;
    if (std::getenv("RXMET_GRU_FWD_GENERIC") != nullptr || std::getenv("RXMET_GRU_FWD_BT") != nullptr) return false;
    const int sms = currentDevice().sms, C = 3 * H;
    const int block = (C + 31) / 32 * 32, hWords = (H + 3) / 4;
    const int bt = (B > 2 * sms) ? 4 : ((B > sms) ? 2 : 1);
    return block <= 768 && hWords <= 64 && bt * H <= 2 * block && H <= 128 &&   // H <= 128: the backward's register path
           fastGateMath(e.gate) && std::getenv("RXMET_GRU_FWD_MODE") == nullptr;
}

void forwardQuant(const ForwardQuantCall &call, const Exec &e, void *workspace, size_t workspaceBytes,
                  cudaStream_t st) {
    if (call.stepFlags && !packedFlagsSupported(e, call.B, call.I, call.H))
        fail(RXMET_ERR_UNSUPPORTED, "packed step flags: these grids or sizes do not take the 8-bit register path");
    Workspace ws(workspace, workspaceBytes);
    if (call.fpCarrier) {
        forwardFpCarrier(call, e, ws, st);
        return;
    }
    const CodeClass w = e.weightClass, a = e.actClass, l = e.linearClass;
    if (l == CodeClass::I32 || w == CodeClass::I32 || a == CodeClass::I32) {
        runTyped<int32_t, int32_t, int32_t>(call, e, ws, st);
    } else if (w == CodeClass::I8 && a == CodeClass::I8) {
        runTyped<int8_t, int8_t, int16_t>(call, e, ws, st);
    } else if (w == CodeClass::I8) {
        runTyped<int8_t, int16_t, int16_t>(call, e, ws, st);
    } else {
        runTyped<int16_t, int16_t, int16_t>(call, e, ws, st);
    }
}

}  // namespace gru
}  // namespace rxmet
