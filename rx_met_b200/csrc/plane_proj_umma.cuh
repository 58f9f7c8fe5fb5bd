// Input projection of the byte-plane paths (16-bit or 8-bit activation codes as one or two unsigned byte
// planes, signed 8-bit weight codes) as a tcgen05.mma kind::i8 GEMM with exact 32-bit integer accumulators in
// tensor memory, shared by the QuantGRU W8 / A16 forward and the wide QuantLSTM forward:
//
//   acc_p[row][c] = sum_k plane_p[row][k] * w[k][c]        (p = high, low byte plane)
//   out[row][c]   = epilogue(c, acc_high, acc_low)         (the caller's functor: exact 64-bit combine, rescale,
//                                                           clamp, masks - whatever its operator defines)
//
// The product is computed transposed, D[channel][row], so that a lane of tensor memory is a channel: the
// per-channel constants of the epilogue live in registers and, for one row, the lanes of a warp store
// neighbouring channels.  A CTA walks row tiles of NR rows with a grid stride.  Per row tile the planes are
// placed once into the canonical un-swizzled K-major B layout (core matrix = 8 rows x 16 k-bytes); per channel
// tile of 128 the weight tile - packed beforehand into the same canonical layout, contiguous per tile - is
// copied into one of two A buffers with 16-byte loads, one thread issues PLANES x K/32 MMAs into one of two
// accumulator buffers (PLANES x NR columns each) and commits them to that buffer's mbarrier, and the epilogue
// of the previous item runs meanwhile.  Every mbarrier wait is bounded; a wait that gives up sets the status
// word and the CTA still frees its tensor memory.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

#include "umma_device.cuh"

namespace rxmet {
namespace planeproj {

using namespace umma;

constexpr int kThreads = 512;
constexpr int kChannelTile = 128;

// kind::i8 with a signed A (weights) and an unsigned B (byte planes): 32-bit integer accumulator (bits [4,6)
// = 2), A format signed 8-bit (bits [7,10) = 1), B format unsigned 8-bit (bits [10,13) = 0), both K-major,
// N >> 3 in [17,23), M >> 4 in [24,29).
__host__ __device__ constexpr uint32_t instructionDescriptor(int n) {
    return (2u << 4) | (1u << 7) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(kTileM >> 4) << 24);
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

struct Problem {
    const uint32_t *planes = nullptr;   // [rows][PLANES][kWords] words of four unsigned bytes, kWords a multiple of 4
    int rows = 0, kWords = 0;
    const uint4 *tiles = nullptr;       // [C / 128][kPad / 16][16 channel groups]... = packTiles' output, 128 * kPad bytes per tile
    int C = 0;                          // a multiple of 128
    int *status = nullptr;              // device word, set to 1 when a bounded wait of the kernel gave up
};

__host__ __device__ inline int paddedK(int kWords) { return (kWords * 4 + 31) / 32 * 32; }
inline size_t sharedBytes(int kPad, int planes, int rowsPerTile) {
    return 2 * static_cast<size_t>(kChannelTile) * kPad + static_cast<size_t>(planes) * rowsPerTile * kPad;
}

// words [kWords][C] (four signed codes along k per word) -> per channel tile of 128 the canonical K-major A
// operand: byte (c, k) of tile c / 128 at ((c % 128) / 8) * (kPad / 16) * 128 + (k / 16) * 128 + (c % 8) * 16 + k % 16;
// k beyond 4 kWords is zero.  One thread per 16-byte row of a core matrix.
static __global__ void packTiles(const uint32_t *__restrict__ words, int kWords, int C, int kPad, uint4 *__restrict__ tiles) {
    const int groups = kPad / 16;
    const size_t total = static_cast<size_t>(C) * groups;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        // consecutive threads -> consecutive channels of one k-group (coalesced reads of the word rows)
        const int kg = static_cast<int>(i / C), c = static_cast<int>(i % C);
        uint32_t v[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int kw = 4 * kg + e;
            v[e] = kw < kWords ? words[static_cast<size_t>(kw) * C + c] : 0u;
        }
        const size_t tile = c / kChannelTile, within = c % kChannelTile;
        const size_t at = tile * (static_cast<size_t>(kChannelTile) * kPad / 16) + (within / 8) * (static_cast<size_t>(groups) * 8) +
                          static_cast<size_t>(kg) * 8 + within % 8;
        tiles[at] = make_uint4(v[0], v[1], v[2], v[3]);
    }
}

// Epilogue functor contract:
//   struct Channel;                                        per-channel constants
//   __device__ Channel channel(int c) const;
//   __device__ void store(const Channel &, size_t row, int c, const int32_t (&acc)[PLANES]) const;
template <class Epilogue, int PLANES, int NR>
__global__ void __launch_bounds__(kThreads, 1) planeProjUmma(const Problem p, const Epilogue epi) {
    constexpr uint32_t kBufCols = PLANES * NR;
    constexpr uint32_t kTmemCols = 2 * kBufCols;   // a power of two for the sizes instantiated (128 .. 512)
    constexpr uint32_t kIdesc = instructionDescriptor(NR);
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t bars[2];  // one per accumulator buffer
    __shared__ uint32_t tmemSlot;
    __shared__ int failed;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int C = p.C, kWords = p.kWords, kPad = paddedK(kWords);
    const uint32_t groupStride = static_cast<uint32_t>(kPad / 16) * kCore;   // next 8 channels / 8 rows
    const uint32_t tileBytes = static_cast<uint32_t>(kChannelTile) * kPad;
    const uint32_t planeBytes = static_cast<uint32_t>(NR) * kPad;
    uint8_t *aTiles = smem;                       // 2 x [16 channel groups][kPad / 16][8][16]
    uint8_t *rowPlanes = smem + 2 * tileBytes;    // PLANES x [NR / 8][kPad / 16][8][16]

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
    // the k padding of the planes is never written again
    for (uint32_t i = tid; i < PLANES * planeBytes / 16; i += kThreads) reinterpret_cast<uint4 *>(rowPlanes)[i] = make_uint4(0u, 0u, 0u, 0u);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmemSlot;
    volatile int *failFlag = &failed;

    const int channelTiles = C / kChannelTile;
    const int rowTiles = (p.rows + NR - 1) / NR;
    const int q = warp & 3, group = warp >> 2;   // tensor-memory lane quarter (32 channels) of this warp, row-chunk group

    auto epilogue = [&](int rowTile, int ct, int local) {
        const int buf = local & 1;
        if (!*failFlag && !waitPhase(smemAddr(&bars[buf]), (local >> 1) & 1)) *failFlag = 1;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int c = ct * kChannelTile + 32 * q + lane;
        const typename Epilogue::Channel ch = epi.channel(c);
        for (int chunk = group; chunk < NR / 16; chunk += kThreads / 128) {
            uint32_t acc[PLANES][16];
#pragma unroll
            for (int pl = 0; pl < PLANES; ++pl) {
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                    "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
                    : "=r"(acc[pl][0]), "=r"(acc[pl][1]), "=r"(acc[pl][2]), "=r"(acc[pl][3]), "=r"(acc[pl][4]), "=r"(acc[pl][5]),
                      "=r"(acc[pl][6]), "=r"(acc[pl][7]), "=r"(acc[pl][8]), "=r"(acc[pl][9]), "=r"(acc[pl][10]), "=r"(acc[pl][11]),
                      "=r"(acc[pl][12]), "=r"(acc[pl][13]), "=r"(acc[pl][14]), "=r"(acc[pl][15])
                    : "r"(tmem + (static_cast<uint32_t>(32 * q) << 16) + static_cast<uint32_t>(buf * kBufCols + pl * NR + 16 * chunk)));
            }
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            const int row0 = rowTile * NR + 16 * chunk;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                if (row0 + j >= p.rows) break;
                int32_t a[PLANES];
#pragma unroll
                for (int pl = 0; pl < PLANES; ++pl) a[pl] = static_cast<int32_t>(acc[pl][j]);
                epi.store(ch, static_cast<size_t>(row0 + j), c, a);
            }
        }
        // the MMAs of the item after next overwrite this buffer: order them behind these loads
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    };

    int local = 0, prevTile = -1, prevCt = -1;
    for (int rowTile = blockIdx.x; rowTile < rowTiles; rowTile += gridDim.x) {
        // The planes of the previous row tile may still be read by the MMAs of its last item: finish that item
        // (its epilogue waits for the commit) before the planes are overwritten.
        if (prevTile >= 0) {
            epilogue(prevTile, prevCt, local - 1);
            prevTile = -1;
        }
        {
            const size_t first = static_cast<size_t>(rowTile) * NR * PLANES * kWords;
            const size_t limit = static_cast<size_t>(p.rows) * PLANES * kWords;
            for (int i = tid; i < NR * PLANES * kWords; i += kThreads) {
                const int r = i / (PLANES * kWords), rest = i - r * (PLANES * kWords);
                const int pl = rest / kWords, kw = rest - pl * kWords;
                const uint32_t v = first + i < limit ? p.planes[first + i] : 0u;
                *reinterpret_cast<uint32_t *>(rowPlanes + pl * planeBytes + (r >> 3) * groupStride + (kw >> 2) * kCore + (r & 7) * 16 +
                                              (kw & 3) * 4) = v;
            }
        }
        for (int ct = 0; ct < channelTiles; ++ct, ++local) {
            const int buf = local & 1;
            // A buffer `buf` was read by the MMAs of item local - 2, whose epilogue has run: free.
            {
                const uint4 *src = p.tiles + static_cast<size_t>(ct) * (tileBytes / 16);
                uint4 *dst = reinterpret_cast<uint4 *>(aTiles + buf * tileBytes);
                for (uint32_t i = tid; i < tileBytes / 16; i += kThreads) dst[i] = __ldg(src + i);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncthreads();
            if (tid == 0) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t aBase = smemAddr(aTiles + buf * tileBytes);
#pragma unroll
                for (int pl = 0; pl < PLANES; ++pl) {
                    const uint32_t bBase = smemAddr(rowPlanes + pl * planeBytes);
                    for (int ks = 0; ks < kPad / 32; ++ks)
                        mmaI8(tmem + buf * kBufCols + pl * NR, operandDescriptor(aBase + ks * 2 * kCore, kCore, groupStride),
                              operandDescriptor(bBase + ks * 2 * kCore, kCore, groupStride), kIdesc, ks > 0 ? 1u : 0u);
                }
                commitTo(smemAddr(&bars[buf]));
            }
            if (prevTile >= 0) epilogue(prevTile, prevCt, local - 1);
            prevTile = rowTile;
            prevCt = ct;
        }
    }
    if (prevTile >= 0) epilogue(prevTile, prevCt, local - 1);

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    if (tid == 0 && failed && p.status) atomicExch(p.status, 1);
}

}  // namespace planeproj
}  // namespace rxmet
