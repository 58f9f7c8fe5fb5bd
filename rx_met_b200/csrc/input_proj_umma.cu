// Input projection of the 8-bit QuantGRU path on the 5th-generation tensor cores:
//   ih[row][c] = epilogue( sum_k x_q[row][k] * W_q[k][c] )        for all T*B rows at once
// as tcgen05.mma kind::i8 (signed 8-bit codes, exact 32-bit integer accumulators in tensor memory)
// with the whole rescale / zero-point / clamp / keep-flag / gate-grid epilogue fused behind it
// (the reference runs a GEMM and a separate bias-and-rescale pass per call:
// operators/quant-gru/src/gru_forward_gpu_quant.cu:109-180, gru_forward_gpu_quant_fp.cu:1129).
//
// The product is computed TRANSPOSED, D[channel][row] = W_q^T x_q^T: the 128 lanes of tensor memory are
// 128 output channels, the columns are rows of the batch.  That puts one channel into one thread of the
// epilogue, so the per-channel constants (multiplier, shift, offset, gate rescale) live in registers, and
// for a given row the 32 lanes of a warp store 32 neighbouring channels: 64 contiguous bytes of codes.
//
// Work item = 128 channels x kRows rows; CTAs walk the items with a grid stride.  Per CTA, once: the
// weight codes of ALL channels as the K-major A operand in the un-swizzled canonical layout (core matrix
// = 8 channels x 16 k-bytes).  Per item: the code rows (contiguous in HBM) are placed into the canonical
// K-major B layout by plain 4-byte loads and stores (a row is I bytes, not a multiple of 16, so no bulk
// copy fits), one thread issues K/32 MMAs into one of two accumulator buffers and commits them to that
// buffer's mbarrier; the epilogue of the previous item runs meanwhile: tcgen05.ld (lane = channel, 16 rows
// per load), integer rescale with round-half-even, clamp, optional second rescale onto the gate-input grid.
// Every mbarrier wait is bounded; a wait that gives up sets the status word (the recurrent kernel that
// consumes the codes turns its outputs into NaN then) and the CTA still frees its tensor memory.
#include <algorithm>
#include <cstdlib>
#include <type_traits>

#include "common.h"
#include "gru_device.cuh"
#include "input_proj_umma.h"
#include "umma_device.cuh"

namespace rxmet {
namespace iproj {
namespace {

using namespace umma;
using gru::Rescale;

constexpr int kThreads = 512;

// kind::i8: 32-bit integer accumulator (bits [4,6) = 2), signed 8-bit A and B (bits [7,10) = [10,13) = 1),
// both K-major (bits 15, 16 clear), N >> 3 in [17,23), M >> 4 in [24,29).
__host__ __device__ constexpr uint32_t instructionDescriptorI8(int n) {
    return (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(kTileM >> 4) << 24);
}

__device__ __forceinline__ void mmaI8(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t"
        "}\n"
        :
        : "r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}

constexpr int kRows = 128;  // rows of the batch per work item = accumulator columns

size_t sharedBytes(int C, int kPad) { return static_cast<size_t>(C) * kPad + 2 * static_cast<size_t>(kRows) * kPad; }

__global__ void __launch_bounds__(kThreads, 2) inputProjUmma(const Problem p) {
    constexpr uint32_t kTmemCols = 2 * kRows;
    constexpr uint32_t kIdesc = instructionDescriptorI8(kRows);
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t bars[2];  // one per accumulator buffer
    __shared__ uint32_t tmemSlot;
    __shared__ int failed;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int C = p.C, kWords = p.kWords, kPad = p.kPad;
    const uint32_t groupStride = static_cast<uint32_t>(kPad / 16) * kCore;  // next 8 channels / 8 rows
    uint8_t *weights = smem;                                               // [C / 8][kPad / 16][8][16]
    uint8_t *rowStages = smem + static_cast<size_t>(C) * kPad;             // 2 x [kRows / 8][kPad / 16][8][16]
    const size_t stageBytes = static_cast<size_t>(kRows) * kPad;

    if (tid == 0) {
        failed = 0;
        for (int i = 0; i < 2; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smemAddr(&bars[i])) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(&tmemSlot)), "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // operands start as zeros: the k padding of both is never written again
    for (size_t i = tid; i < (static_cast<size_t>(C) * kPad + 2 * stageBytes) / 16; i += kThreads)
        reinterpret_cast<uint4 *>(smem)[i] = make_uint4(0u, 0u, 0u, 0u);
    __syncthreads();
    // weight word (kw, c) = codes k = 4 kw .. 4 kw + 3 of channel c -> four consecutive bytes of row c
    for (int i = tid; i < kWords * C; i += kThreads) {
        const int kw = i / C, c = i - kw * C;
        *reinterpret_cast<int32_t *>(weights + (c >> 3) * groupStride + (kw >> 2) * kCore + (c & 7) * 16 + (kw & 3) * 4) = p.w[i];
    }

    const int channelTiles = C / kTileM;
    const int rowTiles = (p.rows + kRows - 1) / kRows;
    const int items = rowTiles * channelTiles;

    // the code words of a row tile are one contiguous run of kRows * kWords words
    auto loadRows = [&](int item, int stage) {
        const int tile = item / channelTiles;
        const size_t first = static_cast<size_t>(tile) * kRows * kWords;
        const size_t limit = static_cast<size_t>(p.rows) * kWords;
        uint8_t *dst = rowStages + stage * stageBytes;
        for (int i = tid; i < kRows * kWords; i += kThreads) {
            const int r = i / kWords, kw = i - r * kWords;
            const int32_t v = first + i < limit ? p.x[first + i] : 0;
            *reinterpret_cast<int32_t *>(dst + (r >> 3) * groupStride + (kw >> 2) * kCore + (r & 7) * 16 + (kw & 3) * 4) = v;
        }
    };

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmemSlot;

    const int32_t zpOut = p.zpOut, lo = p.lo, hi = p.hi;
    const int q = warp & 3, group = warp >> 2;  // tensor-memory lane quarter (32 channels) of this warp, row-chunk group
    // second rescale: |code| and |zero point| below 2^20 keep the product inside 32-bit pieces
    const bool gridsSmall = lo >= -(1 << 20) && hi <= (1 << 20) && zpOut >= -(1 << 20) && zpOut <= (1 << 20);

    auto epilogue = [&](int item, int local) {
        const int buf = local & 1;
        if (!waitPhase(smemAddr(&bars[buf]), (local >> 1) & 1)) failed = 1;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int tile = item / channelTiles, ct = item - tile * channelTiles;
        const int c = ct * kTileM + 32 * q + lane;  // this thread's channel
        // per-channel constants in registers.  Narrow channels (|offset| < 2^30, a multiplier that shrinks,
        // shift in [1, 31]) round with 32-bit pieces of the product; the others take the 64-bit form.
        const Rescale rs = p.rescale[c];
        const int64_t offset = p.biasAcc[c] - p.comp[c];
        const bool narrow = rs.shift >= 1 && rs.shift <= 31 && rs.mult > 0 && static_cast<int64_t>(rs.mult) <= (1ll << rs.shift) &&
                            offset > -(1ll << 30) && offset < (1ll << 30);
        const int64_t mulAdd = offset * static_cast<int64_t>(rs.mult);
        const uint32_t remMask = (1u << (rs.shift & 31)) - 1u, half = 1u << ((rs.shift - 1) & 31);
        const Rescale gateRs = p.pre.enabled ? p.pre.toGate[c / p.pre.hidden] : Rescale{1, 0};
        const int64_t gateAdd = -static_cast<int64_t>(zpOut) * gateRs.mult;
        const bool gateNarrow = gridsSmall && gateRs.shift >= 1 && gateRs.shift <= 31 && gateRs.mult > 0 &&
                                static_cast<int64_t>(gateRs.mult) <= (1ll << min(gateRs.shift + 9, 31));
        const uint32_t gateMask = (1u << (gateRs.shift & 31)) - 1u, gateHalf = 1u << ((gateRs.shift - 1) & 31);
        const bool warpNarrow = __all_sync(0xffffffffu, narrow && (!p.pre.enabled || gateNarrow));
        for (int chunk = group; chunk < kRows / 16; chunk += kThreads / 128) {
            uint32_t acc[16];
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
                : "=r"(acc[0]), "=r"(acc[1]), "=r"(acc[2]), "=r"(acc[3]), "=r"(acc[4]), "=r"(acc[5]), "=r"(acc[6]), "=r"(acc[7]),
                  "=r"(acc[8]), "=r"(acc[9]), "=r"(acc[10]), "=r"(acc[11]), "=r"(acc[12]), "=r"(acc[13]), "=r"(acc[14]), "=r"(acc[15])
                : "r"(tmem + (static_cast<uint32_t>(32 * q) << 16) + static_cast<uint32_t>(buf * kRows + 16 * chunk)));
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            const int row0 = tile * kRows + 16 * chunk;
            size_t o = static_cast<size_t>(row0) * C + c;
            auto rowsLoop = [&](auto narrowTag) {
                constexpr bool kNarrow = decltype(narrowTag)::value;
#pragma unroll
                for (int j = 0; j < 16; ++j, o += C) {
                    const int64_t prod = static_cast<int64_t>(static_cast<int32_t>(acc[j])) * rs.mult + mulAdd;
                    int32_t rounded;
                    if constexpr (kNarrow) rounded = gru::rshiftRoundNarrow(prod, rs.shift, remMask, half);
                    else rounded = narrow ? gru::rshiftRoundNarrow(prod, rs.shift, remMask, half) : gru::rshiftRoundCalled(prod, rs.shift);
                    uint8_t keep;
                    int32_t code = gru::clampCode(rounded + zpOut, lo, hi, keep);
                    if (p.pre.enabled) {
                        const int64_t prodGate = static_cast<int64_t>(code) * gateRs.mult + gateAdd;
                        if constexpr (kNarrow) code = gru::rshiftRoundNarrow(prodGate, gateRs.shift, gateMask, gateHalf);
                        else code = gateNarrow ? gru::rshiftRoundNarrow(prodGate, gateRs.shift, gateMask, gateHalf)
                                               : gru::rshiftRoundCalled(prodGate, gateRs.shift);
                    }
                    if (row0 + j < p.rows) {
                        p.out[o] = static_cast<int16_t>(code);
                        if (p.mask) p.mask[o] = keep;
                    }
                }
            };
            if (warpNarrow) rowsLoop(std::true_type{});
            else rowsLoop(std::false_type{});
        }
        // the MMAs of the item after next overwrite this buffer: order them behind these loads
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    };

    int local = 0, previous = -1;
    for (int item = blockIdx.x; item < items; item += gridDim.x, ++local) {
        const int stage = local & 1;
        loadRows(item, stage);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncthreads();
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int ct = item % channelTiles;
            const uint32_t aBase = smemAddr(weights) + static_cast<uint32_t>(ct * (kTileM / 8)) * groupStride;
            const uint32_t bBase = smemAddr(rowStages + stage * stageBytes);
            for (int ks = 0; ks < kPad / 32; ++ks)
                mmaI8(tmem + stage * kRows, operandDescriptor(aBase + ks * 2 * kCore, kCore, groupStride),
                      operandDescriptor(bBase + ks * 2 * kCore, kCore, groupStride), kIdesc, ks > 0 ? 1u : 0u);
            commitTo(smemAddr(&bars[stage]));
        }
        if (previous >= 0) epilogue(previous, local - 1);
        previous = item;
    }
    if (previous >= 0) epilogue(previous, local - 1);

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    if (tid == 0 && failed && p.status) atomicExch(p.status, 1);
}

}  // namespace

int paddedK(int kWords) { return (kWords * 4 + 31) / 32 * 32; }

bool eligible(int C, int H, int kWords, const void *x, const void *out, const void *mask) {
    static const bool disabled = std::getenv("RXMET_IPROJ_SIMT") != nullptr;
    (void)H; (void)out; (void)mask;
    if (disabled || C % kTileM != 0 || kWords < 1 || !alignedTo(x, 4)) return false;
    return sharedBytes(C, paddedK(kWords)) <= 200 * 1024;  // all weight codes and two row stages in one SM
}

void launch(const Problem &problem, int sms, cudaStream_t st) {
    Problem prob = problem;
    prob.kPad = paddedK(prob.kWords);
    const size_t smem = sharedBytes(prob.C, prob.kPad);
    ensureDynamicSmem(reinterpret_cast<const void *>(inputProjUmma), smem);
    const int items = ((prob.rows + kRows - 1) / kRows) * (prob.C / kTileM);
    KernelTimer timer__("inputLinear", st);
    inputProjUmma<<<std::max(1, std::min(items, 2 * sms)), kThreads, smem, st>>>(prob);
}

}  // namespace iproj
}  // namespace rxmet
