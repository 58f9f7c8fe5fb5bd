// Input projection of the 8-bit QuantGRU path on the 5th-generation tensor cores:
//   ih[row][c] = epilogue( sum_k x_q[row][k] * W_q[k][c] )        for all T*B rows at once
// as tcgen05.mma kind::i8 (signed 8-bit codes, exact 32-bit integer accumulators in tensor memory)
// with the whole rescale / zero-point / clamp / keep-flag / gate-grid epilogue fused behind it
// (the reference runs a GEMM and a separate bias-and-rescale pass per call:
// operators/quant-gru/src/gru_forward_gpu_quant.cu:109-180, gru_forward_gpu_quant_fp.cu:1129).
//
// Work item = 128 rows x NT channels (NT = a divisor of 3H, at most 256); CTAs walk the items with a
// grid stride.  Per CTA, once: the weight codes of ALL channels as the K-major B operand in the
// un-swizzled canonical layout (core matrix = 8 channels x 16 k-bytes), and the per-channel epilogue
// constants.  Per item: the 128 code rows (contiguous in HBM) are placed into the canonical K-major A
// layout by plain 4-byte loads and stores (a row is I bytes, not a multiple of 16, so no bulk copy
// fits), one thread issues K/32 MMAs into one of two accumulator buffers and commits them to that
// buffer's mbarrier; the epilogue of the previous item runs meanwhile: tcgen05.ld (lane = row, 16
// channels per load), integer rescale with round-half-even, clamp, optional second rescale onto the
// gate-input grid, 16-bit codes and keep flags stored as 32- and 16-byte pieces.
// Every mbarrier wait is bounded; a wait that gives up sets the status word (the recurrent kernel that
// consumes the codes turns its outputs into NaN then) and the CTA still frees its tensor memory.
#include <algorithm>
#include <cstdlib>

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

// Per-channel epilogue constants in shared memory, one 16-byte entry per channel.
struct ChannelConst {
    int32_t mult, shift;
    int64_t mulAdd;  // (bias on the accumulator grid - zero-point compensation) * mult
};

size_t sharedBytes(int C, int kPad) {
    return static_cast<size_t>(C) * kPad + sizeof(ChannelConst) * C + 2 * static_cast<size_t>(kTileM) * kPad;
}

template <int NT>
__global__ void __launch_bounds__(kThreads, 1) inputProjUmma(const Problem p) {
    constexpr uint32_t kTmemCols = 2 * NT <= 256 ? 256 : 512;
    constexpr uint32_t kIdesc = instructionDescriptorI8(NT);
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t bars[2];  // one per accumulator buffer
    __shared__ uint32_t tmemSlot;
    __shared__ int failed;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int C = p.C, kWords = p.kWords, kPad = p.kPad;
    const uint32_t groupStride = static_cast<uint32_t>(kPad / 16) * kCore;  // next 8 rows / 8 channels
    uint8_t *bOperand = smem;                                              // [C / 8][kPad / 16][8][16]
    ChannelConst *consts = reinterpret_cast<ChannelConst *>(smem + static_cast<size_t>(C) * kPad);
    uint8_t *aStages = reinterpret_cast<uint8_t *>(consts + C);            // 2 x [16][kPad / 16][8][16]
    const size_t stageBytes = static_cast<size_t>(kTileM) * kPad;

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
    for (size_t i = tid; i < (static_cast<size_t>(C) * kPad + sizeof(ChannelConst) * C + 2 * stageBytes) / 16; i += kThreads)
        reinterpret_cast<uint4 *>(smem)[i] = make_uint4(0u, 0u, 0u, 0u);
    __syncthreads();
    // weight word (kw, c) = codes k = 4 kw .. 4 kw + 3 of channel c -> four consecutive bytes of row c
    for (int i = tid; i < kWords * C; i += kThreads) {
        const int kw = i / C, c = i - kw * C;
        *reinterpret_cast<int32_t *>(bOperand + (c >> 3) * groupStride + (kw >> 2) * kCore + (c & 7) * 16 + (kw & 3) * 4) = p.w[i];
    }
    for (int c = tid; c < C; c += kThreads) {
        const Rescale rs = p.rescale[c];
        consts[c] = ChannelConst{rs.mult, rs.shift, (p.biasAcc[c] - p.comp[c]) * static_cast<int64_t>(rs.mult)};
    }

    const int parts = C / NT;
    const int rowTiles = (p.rows + kTileM - 1) / kTileM;
    const int items = rowTiles * parts;

    // the code words of a row tile are one contiguous run of 128 * kWords words
    auto loadTile = [&](int item, int stage) {
        const int tile = item / parts;
        const size_t first = static_cast<size_t>(tile) * kTileM * kWords;
        const size_t limit = static_cast<size_t>(p.rows) * kWords;
        uint8_t *dst = aStages + stage * stageBytes;
        for (int i = tid; i < kTileM * kWords; i += kThreads) {
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
    const int q = warp & 3, group = warp >> 2;  // tensor-memory lane quarter of this warp, column-chunk group

    auto epilogue = [&](int item, int local) {
        const int buf = local & 1;
        if (!waitPhase(smemAddr(&bars[buf]), (local >> 1) & 1)) failed = 1;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int tile = item / parts, part = item - tile * parts;
        const int row = tile * kTileM + 32 * q + lane;
        for (int chunk = group; chunk < NT / 16; chunk += kThreads / 128) {
            const int c0 = part * NT + 16 * chunk;
            uint32_t acc[16];
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
                : "=r"(acc[0]), "=r"(acc[1]), "=r"(acc[2]), "=r"(acc[3]), "=r"(acc[4]), "=r"(acc[5]), "=r"(acc[6]), "=r"(acc[7]),
                  "=r"(acc[8]), "=r"(acc[9]), "=r"(acc[10]), "=r"(acc[11]), "=r"(acc[12]), "=r"(acc[13]), "=r"(acc[14]), "=r"(acc[15])
                : "r"(tmem + (static_cast<uint32_t>(32 * q) << 16) + static_cast<uint32_t>(buf * NT + 16 * chunk)));
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            // the 16 channels of a chunk lie inside one gate (H is a multiple of 16)
            const Rescale gateRs = p.pre.enabled ? p.pre.toGate[c0 / p.pre.hidden] : Rescale{1, 0};
            const int64_t gateAdd = -static_cast<int64_t>(zpOut) * gateRs.mult;
            uint32_t codes[8], keeps[4] = {0u, 0u, 0u, 0u};
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const ChannelConst k = consts[c0 + j];
                const int64_t prod = static_cast<int64_t>(static_cast<int32_t>(acc[j])) * k.mult + k.mulAdd;
                uint8_t keep;
                int32_t code = gru::clampCode(static_cast<int32_t>(gru::rshiftRound(prod, k.shift)) + zpOut, lo, hi, keep);
                if (p.pre.enabled)
                    code = static_cast<int32_t>(gru::rshiftRound(static_cast<int64_t>(code) * gateRs.mult + gateAdd, gateRs.shift));
                const uint32_t half = static_cast<uint32_t>(code) & 0xffffu;
                if (j & 1) codes[j >> 1] |= half << 16;
                else codes[j >> 1] = half;
                keeps[j >> 2] |= static_cast<uint32_t>(keep) << (8 * (j & 3));
            }
            if (row < p.rows) {
                const size_t o = static_cast<size_t>(row) * C + c0;
                uint4 *dst = reinterpret_cast<uint4 *>(p.out + o);
                dst[0] = make_uint4(codes[0], codes[1], codes[2], codes[3]);
                dst[1] = make_uint4(codes[4], codes[5], codes[6], codes[7]);
                if (p.mask) *reinterpret_cast<uint4 *>(p.mask + o) = make_uint4(keeps[0], keeps[1], keeps[2], keeps[3]);
            }
        }
        // the MMAs of the item after next overwrite this buffer: order them behind these loads
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    };

    int local = 0, previous = -1;
    for (int item = blockIdx.x; item < items; item += gridDim.x, ++local) {
        const int stage = local & 1;
        loadTile(item, stage);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncthreads();
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int part = item % parts;
            const uint32_t aBase = smemAddr(aStages + stage * stageBytes);
            const uint32_t bBase = smemAddr(bOperand) + static_cast<uint32_t>(part * (NT / 8)) * groupStride;
            for (int ks = 0; ks < kPad / 32; ++ks)
                mmaI8(tmem + stage * NT, operandDescriptor(aBase + ks * 2 * kCore, kCore, groupStride),
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

int tileWidth(int C) {
    for (int nt : {256, 192, 128, 96, 64})
        if (C % nt == 0) return nt;
    return 0;
}

template <int NT>
void launchTile(const Problem &prob, int sms, cudaStream_t st) {
    const size_t smem = sharedBytes(prob.C, prob.kPad);
    ensureDynamicSmem(reinterpret_cast<const void *>(inputProjUmma<NT>), smem);
    const int items = ((prob.rows + kTileM - 1) / kTileM) * (prob.C / NT);
    KernelTimer timer__("inputLinear", st);
    inputProjUmma<NT><<<std::max(1, std::min(items, sms)), kThreads, smem, st>>>(prob);
}

}  // namespace

int paddedK(int kWords) { return (kWords * 4 + 31) / 32 * 32; }

bool eligible(int C, int H, int kWords, const void *x, const void *out, const void *mask) {
    static const bool disabled = std::getenv("RXMET_IPROJ_SIMT") != nullptr;
    if (disabled || H % 16 != 0 || tileWidth(C) == 0 || kWords < 1) return false;
    // 16-byte stores of codes and keep flags; the whole problem must fit the shared memory of one SM
    if (!alignedTo(out, 16) || !alignedTo(mask, 16) || !alignedTo(x, 4)) return false;
    return sharedBytes(C, paddedK(kWords)) <= 200 * 1024;
}

void launch(const Problem &problem, int sms, cudaStream_t st) {
    Problem prob = problem;
    prob.kPad = paddedK(prob.kWords);
    switch (tileWidth(prob.C)) {
        case 256: launchTile<256>(prob, sms, st); break;
        case 192: launchTile<192>(prob, sms, st); break;
        case 128: launchTile<128>(prob, sms, st); break;
        case 96: launchTile<96>(prob, sms, st); break;
        case 64: launchTile<64>(prob, sms, st); break;
        default: fail(RXMET_ERR_UNSUPPORTED, "input projection: %d channels", prob.C);
    }
}

}  // namespace iproj
}  // namespace rxmet
