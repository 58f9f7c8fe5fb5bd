// Weight-gradient GEMM on tcgen05.mma, warp-specialised (the streaming form of weightGradUmma):
//   partial[s][m][n] = sum over the s-th range of the K rows of A[k][m] * B[k][n],  partial[s][M][n] = column sums of B.
// Both operands stream through shared memory once; the [128][NT] accumulator lives in tensor memory.
//
//   * warp 16, one lane: TMA (cp.async.bulk.tensor.2d, 128-byte swizzle) brings a chunk of 32 K rows of both raw
//     operands - boxes of 32 rows x 32 four-byte values: NT / 32 boxes of gradients, up to four boxes of A - into
//     a ring of three buffers, all boxes of a chunk on one mbarrier;
//   * warps 0-15 convert (lane = K row of the chunk, a warp owns fixed 8-column groups, so the swizzled reads
//     and the operand stores are free of bank conflicts): gradients -> three bf16 terms, A -> the exact integer
//     (code minus zero point) as one bf16 term, both into the MN-major canonical layout of one of two stages;
//     the column sums of the gradients accumulate in the converters' registers;
//   * warp 17, one lane: 2 k-steps x 3 terms MMAs per chunk, committed to the barrier that frees the stage.
// Full / empty mbarriers connect the roles; the only CTA-wide barriers are at the start and the end.  After the
// last chunk warps 0-15 carry the accumulator rows out (turned round in shared memory so that a store covers whole
// 128-byte row segments) and write the bias row.  Every wait is bounded: a wait that gives up sets a flag that
// ends all further waiting of the CTA and sets the status word (the reduction that follows turns its outputs
// into NaN); the CTA still waits for its copies in flight and frees its tensor memory.
#include <cuda.h>

#include <algorithm>
#include <cstdlib>

#include "common.h"
#include "umma_device.cuh"
#include "weight_grad_mma.h"

namespace rxmet {
namespace wgrad {
namespace {

using namespace umma;

constexpr int kConvWarps = 16;
constexpr int kThreadsStream = (kConvWarps + 2) * 32;
constexpr int kChunkRows = 32;                       // K rows per chunk: two MMA k-steps
constexpr int kRing = 3, kStages = 2;
constexpr uint32_t kBoxBytes = kChunkRows * 128;     // one TMA box: 32 rows x 32 four-byte values
constexpr int kMaxABoxes = 4;                        // M <= 128
constexpr uint32_t kAKStride = (kTileM / 8) * kCore; // bytes between the k-groups of the A tile
constexpr uint32_t kABytes = (kChunkRows / 8) * kAKStride;

template <int NT>
struct StreamGeometry {
    static constexpr int kBBoxes = NT / 32;
    static constexpr uint32_t kRawBytes = (kMaxABoxes + kBBoxes) * kBoxBytes;
    static constexpr uint32_t kBKStride = (NT / 8) * kCore;
    static constexpr uint32_t kBBytes = (kChunkRows / 8) * kBKStride;
    static constexpr uint32_t kStageBytes = kABytes + 3 * kBBytes;
    static constexpr size_t kSmem = 1024 + kRing * kRawBytes + kStages * kStageBytes;
    static_assert(kSmem <= 227 * 1024, "shared memory of one SM");
};

struct StreamProblem {
    Problem p;
    CUtensorMap mapA, mapB;
    int aBoxes;
};
struct StreamSet {
    StreamProblem prob[2];
};

template <int NT>
__global__ void __launch_bounds__(kThreadsStream, 1)
weightGradStreamUmma(const __grid_constant__ StreamSet set, int K, int N, int chunkK, int *status) {
    using G = StreamGeometry<NT>;
    const StreamProblem &sp = set.prob[blockIdx.z];
    const Problem &p = sp.p;
    constexpr uint32_t kTmemCols = NT > 128 ? 256 : 128;
    constexpr uint32_t kIdesc = instructionDescriptor(NT, true, true);
    constexpr int kGroups = NT / 8;                                            // 8-column groups of the gradient tile
    constexpr int kGroupsPerWarp = (kGroups + kConvWarps - 1) / kConvWarps;   // ... a converter warp owns at most

    extern __shared__ __align__(1024) uint8_t smemRaw[];
    __shared__ __align__(8) uint64_t rawFull[kRing], rawEmpty[kRing], stageFull[kStages], stageEmpty[kStages], accFull;
    __shared__ uint32_t tmemSlot;
    __shared__ int failed;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n0 = blockIdx.x * NT;
    const int kBegin = blockIdx.y * chunkK, kEnd = min(K, kBegin + chunkK);
    const int chunks = (kEnd - kBegin + kChunkRows - 1) / kChunkRows;
    const int M = p.M, aGroups = M / 8;
    uint8_t *base = smemRaw + ((1024u - (smemAddr(smemRaw) & 1023u)) & 1023u);   // the swizzled boxes need 1024-byte alignment
    uint8_t *raw = base;                                  // [kRing][A boxes, then B boxes]
    uint8_t *stages = raw + kRing * G::kRawBytes;         // [kStages][A tile, three B terms]
    volatile int *failFlag = &failed;

    if (tid == 0) {
        failed = 0;
        for (int i = 0; i < kRing; ++i) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smemAddr(&rawFull[i])) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smemAddr(&rawEmpty[i])), "r"(kConvWarps) : "memory");
        }
        for (int i = 0; i < kStages; ++i) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smemAddr(&stageFull[i])), "r"(kConvWarps) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smemAddr(&stageEmpty[i])) : "memory");
        }
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smemAddr(&accFull)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    // rows of the A tile beyond M stay zero for the whole kernel
    for (uint32_t i = tid; i < kStages * kABytes / 16; i += kThreadsStream) {
        const uint32_t stage = i / (kABytes / 16), off = i % (kABytes / 16);
        *reinterpret_cast<uint4 *>(stages + stage * G::kStageBytes + off * 16) = make_uint4(0u, 0u, 0u, 0u);
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(&tmemSlot)), "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmemSlot;

    auto await = [&](uint64_t *bar, uint32_t parity) {
        if (*failFlag) return;
        if (!waitPhase(smemAddr(bar), parity)) *failFlag = 1;
    };

    float csum[kGroupsPerWarp][8];
#pragma unroll
    for (int g = 0; g < kGroupsPerWarp; ++g)
#pragma unroll
        for (int j = 0; j < 8; ++j) csum[g][j] = 0.0f;

    if (warp == kConvWarps) {
        // ---- both raw operands: the boxes of a chunk on one barrier
        if (lane == 0) {
            int issued = 0;
            const uint32_t chunkBytes = static_cast<uint32_t>(sp.aBoxes + G::kBBoxes) * kBoxBytes;
            for (int c = 0; c < chunks && !*failFlag; ++c) {
                const int slot = c % kRing;
                if (c >= kRing) await(&rawEmpty[slot], (c / kRing - 1) & 1);
                if (*failFlag) break;
                const uint32_t bar = smemAddr(&rawFull[slot]);
                const int k0 = kBegin + c * kChunkRows;
                uint8_t *dst = raw + slot * G::kRawBytes;
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(chunkBytes) : "memory");
                for (int b = 0; b < sp.aBoxes; ++b)
                    asm volatile(
                        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                        ::"r"(smemAddr(dst + b * kBoxBytes)), "l"(&sp.mapA), "r"(32 * b), "r"(k0), "r"(bar)
                        : "memory");
#pragma unroll
                for (int b = 0; b < G::kBBoxes; ++b)
                    asm volatile(
                        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                        ::"r"(smemAddr(dst + (kMaxABoxes + b) * kBoxBytes)), "l"(&sp.mapB), "r"(n0 + 32 * b), "r"(k0), "r"(bar)
                        : "memory");
                issued = c + 1;
            }
            if (*failFlag)   // copies in flight must land before the CTA's shared memory is given up
                for (int c = max(0, issued - kRing); c < issued; ++c) waitPhase(smemAddr(&rawFull[c % kRing]), (c / kRing) & 1);
        }
    } else if (warp == kConvWarps + 1) {
        // ---- MMA issue
        if (lane == 0) {
            for (int c = 0; c < chunks; ++c) {
                const int s = c % kStages;
                await(&stageFull[s], (c / kStages) & 1);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t stage = smemAddr(stages + s * G::kStageBytes);
#pragma unroll
                for (int ks = 0; ks < kChunkRows / 16; ++ks) {
                    const uint64_t descA = operandDescriptor(stage + ks * 2 * kAKStride, kAKStride, kCore);
#pragma unroll
                    for (int term = 0; term < 3; ++term) {
                        const uint64_t descB = operandDescriptor(stage + kABytes + term * G::kBBytes + ks * 2 * G::kBKStride, G::kBKStride, kCore);
                        mmaBf16(tmem, descA, descB, kIdesc, (c > 0 || ks > 0 || term > 0) ? 1u : 0u);
                    }
                }
                commitTo(smemAddr(&stageEmpty[s]));
            }
            commitTo(smemAddr(&accFull));
        }
    } else {
        // ---- converters: lane = K row of the chunk; warp w owns the gradient column groups w and w + 16 and the
        // A row group w
        const int r = lane;
        for (int c = 0; c < chunks; ++c) {
            const int slot = c % kRing, s = c % kStages;
            await(&rawFull[slot], (c / kRing) & 1);
            const uint8_t *src = raw + slot * G::kRawBytes;
            // unit u (16 bytes) of row r of a box sits at unit u ^ (r & 7)
            auto loadGroup = [&](const uint8_t *boxes, int group, uint4 &lo, uint4 &hi) {
                const uint8_t *row = boxes + (group >> 2) * kBoxBytes + r * 128;
                const int u = 2 * (group & 3);
                lo = *reinterpret_cast<const uint4 *>(row + ((u ^ (r & 7)) << 4));
                hi = *reinterpret_cast<const uint4 *>(row + (((u + 1) ^ (r & 7)) << 4));
            };
            uint4 bl[kGroupsPerWarp], bh[kGroupsPerWarp], al, ah;
#pragma unroll
            for (int g = 0; g < kGroupsPerWarp; ++g)
                if (warp + kConvWarps * g < kGroups) loadGroup(src + kMaxABoxes * kBoxBytes, warp + kConvWarps * g, bl[g], bh[g]);
            if (warp < aGroups) loadGroup(src, warp, al, ah);
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smemAddr(&rawEmpty[slot])) : "memory");
            if (c >= kStages) await(&stageEmpty[s], (c / kStages - 1) & 1);
            uint8_t *stage = stages + s * G::kStageBytes;
            const uint32_t rowOffset = static_cast<uint32_t>(r >> 3) * 1u /* k-group */;
#pragma unroll
            for (int g = 0; g < kGroupsPerWarp; ++g) {
                if (warp + kConvWarps * g >= kGroups) continue;
                const float4 u = make_float4(__uint_as_float(bl[g].x), __uint_as_float(bl[g].y), __uint_as_float(bl[g].z), __uint_as_float(bl[g].w));
                const float4 v = make_float4(__uint_as_float(bh[g].x), __uint_as_float(bh[g].y), __uint_as_float(bh[g].z), __uint_as_float(bh[g].w));
                csum[g][0] += u.x; csum[g][1] += u.y; csum[g][2] += u.z; csum[g][3] += u.w;
                csum[g][4] += v.x; csum[g][5] += v.y; csum[g][6] += v.z; csum[g][7] += v.w;
                const Converted cv = splitThree(u, v);
                uint8_t *dst = stage + kABytes + rowOffset * G::kBKStride + (warp + kConvWarps * g) * kCore + (r & 7) * 16;
                *reinterpret_cast<uint4 *>(dst) = cv.hi;
                *reinterpret_cast<uint4 *>(dst + G::kBBytes) = cv.mid;
                *reinterpret_cast<uint4 *>(dst + 2 * G::kBBytes) = cv.lo;
            }
            if (warp < aGroups) {   // the A tile has at most 16 groups of 8 rows: one per converter warp
                const uint32_t q[8] = {al.x, al.y, al.z, al.w, ah.x, ah.y, ah.z, ah.w};
                float x[8];
                // rows beyond the tensor read as zero bits: they decode to some finite value and meet zero gradients
                if (p.aCodes) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) x[i] = static_cast<float>(static_cast<int32_t>(q[i]) - p.aZero);
                } else {  // recover the integer code difference from the dequantized value
#pragma unroll
                    for (int i = 0; i < 8; ++i) x[i] = rintf(__uint_as_float(q[i]) * p.aInvScale) - p.aFloatZero;
                }
                uint8_t *dst = stage + rowOffset * kAKStride + warp * kCore + (r & 7) * 16;
                *reinterpret_cast<uint4 *>(dst) =
                    make_uint4(packBf16(x[0], x[1]), packBf16(x[2], x[3]), packBf16(x[4], x[5]), packBf16(x[6], x[7]));
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smemAddr(&stageFull[s])) : "memory");
        }

        // ---- accumulators -> partial sums.  Warp w reads the tensor-memory lanes [32 (w % 4), + 32) and the column
        // blocks w / 4, w / 4 + 2, ...
        if (chunks > 0) await(&accFull, 0);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int totalRows = p.totalRows ? p.totalRows : M + 1;
        float *slice = p.partial + static_cast<size_t>(blockIdx.y) * totalRows * N;
        float *out = slice + static_cast<size_t>(p.rowBase) * N;
        const int q = warp & 3;
        if (32 * q < M && chunks > 0) {
            float4 *tile = reinterpret_cast<float4 *>(raw + warp * 4096);   // the raw ring is idle now
            for (int j = warp >> 2; j < NT / 32; j += kConvWarps / 4) {
                uint32_t acc[32];
                tmemLoad32(tmem + (static_cast<uint32_t>(32 * q) << 16) + 32 * j, acc);
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    tile[lane * 8 + (i ^ (lane & 7))] = make_float4(__uint_as_float(acc[4 * i]), __uint_as_float(acc[4 * i + 1]),
                                                                    __uint_as_float(acc[4 * i + 2]), __uint_as_float(acc[4 * i + 3]));
                __syncwarp();
#pragma unroll
                for (int pass = 0; pass < 8; ++pass) {
                    const int row = 4 * pass + (lane >> 3), i = lane & 7;
                    const float4 v = tile[row * 8 + (i ^ (row & 7))];
                    if (32 * q + row < M)
                        *reinterpret_cast<float4 *>(out + static_cast<size_t>(32 * q + row) * N + n0 + 32 * j + 4 * i) = v;
                }
                __syncwarp();
            }
        }
        // bias row: the column sums of this warp's groups over the 32 K-row lanes, fixed order
        if (p.writeBias) {
#pragma unroll
            for (int g = 0; g < kGroupsPerWarp; ++g) {
                if (warp + kConvWarps * g >= kGroups) continue;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    float v = csum[g][j];
#pragma unroll
                    for (int off = 1; off < 32; off <<= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
                    csum[g][j] = v;
                }
                if (lane == 0) {
                    float4 *dst = reinterpret_cast<float4 *>(slice + static_cast<size_t>(totalRows - 1) * N + n0 + 8 * (warp + kConvWarps * g));
                    dst[0] = make_float4(csum[g][0], csum[g][1], csum[g][2], csum[g][3]);
                    dst[1] = make_float4(csum[g][4], csum[g][5], csum[g][6], csum[g][7]);
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    if (tid == 0 && failed && status) atomicExch(status, 1);
}

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against the driver library).
using EncodeTiled = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                 const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiled encodeTiled() {
    static EncodeTiled fn = [] {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult status = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &status) != cudaSuccess ||
            status != cudaDriverEntryPointSuccess)
            ptr = nullptr;
        return reinterpret_cast<EncodeTiled>(ptr);
    }();
    return fn;
}

// [rows][cols] four-byte values in boxes of 32 rows x 32 values with the 128-byte swizzle; what lies beyond the tensor
// reads as zero bits.  The x coordinate of every copy is a multiple of 32 values.
CUtensorMap boxMap(const void *data, int rows, int cols) {
    CUtensorMap map;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 4};
    const cuuint32_t box[2] = {32, kChunkRows};
    const cuuint32_t elementStrides[2] = {1, 1};
    const CUresult rc = encodeTiled()(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void *>(data), dims, strides, box, elementStrides,
                                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) fail(RXMET_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d", static_cast<int>(rc));
    return map;
}

bool takes(const Problem &p, int N) {
    return p.M >= 8 && p.M <= kTileM && p.M % 8 == 0 && p.lda == 0 && p.rowBase == 0 && p.wideCodes == 0 &&
           (p.aCodes != nullptr || p.aFloat != nullptr) && alignedTo(p.aCodes, 16) && alignedTo(p.aFloat, 16) && alignedTo(p.B, 16) &&
           alignedTo(p.partial, 16) && N % 4 == 0;
}

template <int NT>
void launchStream(const Problem &a, const Problem &b, int K, int N, int chunkK, int splits, cudaStream_t st) {
    StreamSet set;
    int count = 0;
    for (const Problem *p : {&a, &b}) {
        StreamProblem &sp = set.prob[count++];
        sp.p = *p;
        sp.aBoxes = (p->M + 31) / 32;
        sp.mapA = boxMap(p->aCodes ? static_cast<const void *>(p->aCodes) : static_cast<const void *>(p->aFloat), K, p->M);
        sp.mapB = boxMap(p->B, K, N);
    }
    constexpr size_t smem = StreamGeometry<NT>::kSmem;
    ensureDynamicSmem(reinterpret_cast<const void *>(weightGradStreamUmma<NT>), smem);
    KernelTimer timer__("weightGradUmma", st);
    weightGradStreamUmma<NT><<<dim3(N / NT, splits, count), kThreadsStream, smem, st>>>(set, K, N, chunkK, a.status);
}

}  // namespace

// Two problems over the same K rows and N columns (the input and the recurrent weights of a step) on the streaming
// kernel; false when a shape, an alignment or the driver entry point rules it out (the caller then takes
// weightGradUmma).  RXMET_WGRAD_NO_STREAM switches it off.
bool launchPairStreamed(const Problem &a, const Problem &b, int K, int N, int chunkK, int splits, cudaStream_t st) {
    static const bool disabled = std::getenv("RXMET_WGRAD_NO_STREAM") != nullptr;
    if (disabled || !takes(a, N) || !takes(b, N) || a.status != b.status || chunkK % kChunkRows != 0 || encodeTiled() == nullptr) return false;
    if (N % 192 == 0 && N % 256 != 0) launchStream<192>(a, b, K, N, chunkK, splits, st);
    else if (N % 128 == 0 && N % 256 != 0) launchStream<128>(a, b, K, N, chunkK, splits, st);
    else return false;
    return true;
}

}  // namespace wgrad
}  // namespace rxmet
