// dx = (G * kScale) code for wide inputs (up to 512 columns, any K that is a multiple of 32) on
// tcgen05.mma, warp-specialised: nothing of either operand stays resident, both stream through
// shared memory once per 128-row tile while the whole [128][N] accumulator lives in tensor memory.
//
//   * one lane of the warp behind the converters: TMA (cp.async.bulk.tensor.2d, 128-byte swizzle) brings chunk after
//     chunk of raw fp32 gradients (boxes of [128 rows][32 channels] = 16 KB; one or two per chunk) into a ring;
//   * one lane of the next warp: one bulk copy per chunk brings the chunk's slice of the weight operand,
//     packed beforehand by packWideWeights into the canonical un-swizzled K-major layout, into a
//     ring of three buffers that the MMAs read directly;
//   * the converter warps (8, or 16 with 64-channel chunks): read a raw chunk (the swizzle makes the reads conflict-free), fold the
//     per-channel scale in, split every value into three bf16 terms and store them as the A operand
//     of one of two stages;
//   * one lane of the last warp: issues the MMAs of a chunk (2 or 4 k-steps x 3 terms x column blocks of at most
//     256) and commits them to the barriers that free the A stage and the weight buffer.
// Full / empty mbarriers connect the roles; the only CTA-wide barriers are at the start and the end.
// After the last chunk the converter warps read the accumulators (lane = row), apply the mask and store.
// Every wait is bounded: a wait that gives up sets a flag that ends all further waiting, poisons the
// CTA's outputs with NaN and sets the status word; the CTA still waits for its copies in flight and
// frees its tensor memory.
#include <cuda.h>

#include <algorithm>
#include <cstdlib>

#include "common.h"
#include "input_grad_umma.h"
#include "umma_device.cuh"

namespace rxmet {
namespace igrad {
namespace {

using namespace umma;

// CH channels per chunk (32 or 64: one or two 128-byte spans of a raw row), CW converter warps.  The wider chunk halves
// the number of hand-overs between the roles per tile; it fits beside the weight ring for up to 128 columns.
template <int CH, int CW>
struct WideGeometry {
    static constexpr int kConvWarps = CW;
    static constexpr int kThreads = (CW + 3) * 32;
    static constexpr int kBoxes = CH / 32;                                  // TMA boxes (128 rows x 32 channels) per chunk
    static constexpr int kRawRing = CH == 32 ? 4 : 3, kAStages = 2, kBRing = 3;
    static constexpr uint32_t kBoxBytes = kTileM * 32 * 4;                  // 16 KB
    static constexpr uint32_t kRawChunkBytes = kBoxes * kBoxBytes;
    static constexpr uint32_t kTermChunkBytes = kTileM * CH * 2;            // one bf16 term of a chunk
    static constexpr uint32_t kAStageBytes = 3 * kTermChunkBytes;
    static constexpr uint32_t kRowGroupStride = (CH / 8) * kCore;           // next 8 rows (A) or 8 columns (B) inside a chunk
    static size_t sharedBytes(int NP) {
        return 1024 + kRawRing * kRawChunkBytes + kAStages * kAStageBytes + static_cast<size_t>(kBRing) * NP * CH * 2;
    }
};
constexpr int kChunk = 32;          // granularity of K that every variant takes
constexpr int kMaxColumns = 512;

// codes -> bf16, chunk by chunk of CH channels: packed[chunk][n / 8][k-group of 8][n % 8][8 k]; one thread per 16-byte row.
__global__ void packWideWeights(const int32_t *codesNK, const float *codesKN, int ldCodesKN, int K, int N, int NP, int CH, uint4 *packed) {
    const int item = blockIdx.x * blockDim.x + threadIdx.x;
    if (item >= (K / 8) * NP) return;
    const int groups = CH / 8;   // k-groups of a chunk
    const int nr = item & 7, kg = (item >> 3) % groups, n8 = ((item >> 3) / groups) % (NP / 8), kc = ((item >> 3) / groups) / (NP / 8);
    const int n = 8 * n8 + nr, k0 = kc * CH + 8 * kg;
    float c[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
        c[j] = n >= N ? 0.0f
                      : (codesNK ? static_cast<float>(codesNK[static_cast<size_t>(n) * K + k0 + j])
                                 : codesKN[static_cast<size_t>(k0 + j) * ldCodesKN + n]);
    packed[item] = make_uint4(packBf16(c[0], c[1]), packBf16(c[2], c[3]), packBf16(c[4], c[5]), packBf16(c[6], c[7]));
}

struct WideShape {
    int NP;        // padded columns
    int blocks;    // MMA column blocks (1 or 2)
    int NB;        // columns per block (multiple of 16, at most 256)
    int tmemCols;  // power of two that holds NP columns
};

template <int CH, int CW>
__global__ void __launch_bounds__((CW + 3) * 32, 1)
inputGradWideUmma(const Problem p, const WideShape shape, const __grid_constant__ CUtensorMap gradients) {
    using G = WideGeometry<CH, CW>;
    constexpr int kConvWarps = CW, kRawRing = G::kRawRing, kAStages = G::kAStages, kBRing = G::kBRing;
    constexpr uint32_t kRawChunkBytes = G::kRawChunkBytes, kTermChunkBytes = G::kTermChunkBytes, kAStageBytes = G::kAStageBytes,
                       kRowGroupStride = G::kRowGroupStride;
    extern __shared__ __align__(1024) uint8_t smemRaw[];
    __shared__ __align__(8) uint64_t rawFull[kRawRing], rawEmpty[kRawRing], aFull[kAStages], aEmpty[kAStages], bFull[kBRing],
        bEmpty[kBRing], accFull;
    __shared__ uint32_t tmemSlot;
    __shared__ int failed;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = p.K, N = p.N, NP = shape.NP, chunks = K / CH;
    const int ldN = p.ldN ? p.ldN : N;
    const uint32_t bBytes = static_cast<uint32_t>(NP) * CH * 2;
    uint8_t *base = smemRaw + ((1024u - (smemAddr(smemRaw) & 1023u)) & 1023u);   // the swizzled TMA boxes need 1024-byte alignment
    uint8_t *raw = base;
    uint8_t *aStages = raw + kRawRing * kRawChunkBytes;
    uint8_t *bRing = aStages + kAStages * kAStageBytes;
    const int row0 = static_cast<int>(blockIdx.x) * kTileM;
    volatile int *failFlag = &failed;

    if (tid == 0) {
        failed = 0;
        for (int i = 0; i < kRawRing; ++i) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smemAddr(&rawFull[i])) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smemAddr(&rawEmpty[i])), "r"(kConvWarps) : "memory");
        }
        for (int i = 0; i < kAStages; ++i) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smemAddr(&aFull[i])), "r"(kConvWarps) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smemAddr(&aEmpty[i])) : "memory");
        }
        for (int i = 0; i < kBRing; ++i) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smemAddr(&bFull[i])) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smemAddr(&bEmpty[i])) : "memory");
        }
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smemAddr(&accFull)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(&tmemSlot)), "r"(shape.tmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmemSlot;

    // a wait that gives up ends all further waiting of the CTA
    auto await = [&](uint64_t *bar, uint32_t parity) {
        if (*failFlag) return;
        if (!waitPhase(smemAddr(bar), parity)) *failFlag = 1;
    };

    if (warp == kConvWarps) {
        // ---- raw gradients: one TMA box per chunk
        if (lane == 0) {
            int issued = 0;
            for (int c = 0; c < chunks && !*failFlag; ++c) {
                const int slot = c % kRawRing;
                if (c >= kRawRing) await(&rawEmpty[slot], (c / kRawRing - 1) & 1);
                if (*failFlag) break;
                const uint32_t bar = smemAddr(&rawFull[slot]);
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(kRawChunkBytes) : "memory");
#pragma unroll
                for (int b = 0; b < G::kBoxes; ++b)
                    asm volatile(
                        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                        ::"r"(smemAddr(raw + slot * kRawChunkBytes + b * G::kBoxBytes)), "l"(&gradients), "r"(c * CH + 32 * b), "r"(row0), "r"(bar)
                        : "memory");
                issued = c + 1;
            }
            if (*failFlag)   // copies in flight must land before the CTA's shared memory is given up
                for (int c = max(0, issued - kRawRing); c < issued; ++c) waitPhase(smemAddr(&rawFull[c % kRawRing]), (c / kRawRing) & 1);
        }
    } else if (warp == kConvWarps + 1) {
        // ---- weight operand: one bulk copy per chunk
        if (lane == 0) {
            int issued = 0;
            const uint8_t *src = static_cast<const uint8_t *>(p.packed);
            for (int c = 0; c < chunks && !*failFlag; ++c) {
                const int slot = c % kBRing;
                if (c >= kBRing) await(&bEmpty[slot], (c / kBRing - 1) & 1);
                if (*failFlag) break;
                const uint32_t bar = smemAddr(&bFull[slot]);
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bBytes) : "memory");
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(smemAddr(bRing + static_cast<size_t>(slot) * bBytes)), "l"(src + static_cast<size_t>(c) * bBytes),
                             "r"(bBytes), "r"(bar)
                             : "memory");
                issued = c + 1;
            }
            if (*failFlag)
                for (int c = max(0, issued - kBRing); c < issued; ++c) waitPhase(smemAddr(&bFull[c % kBRing]), (c / kBRing) & 1);
        }
    } else if (warp == kConvWarps + 2) {
        // ---- MMA issue
        if (lane == 0) {
            const uint32_t idesc = instructionDescriptor(shape.NB, false, false);
            for (int c = 0; c < chunks; ++c) {
                const int sa = c % kAStages, sb = c % kBRing;
                await(&aFull[sa], (c / kAStages) & 1);
                await(&bFull[sb], (c / kBRing) & 1);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t aBase = smemAddr(aStages + sa * kAStageBytes), bBase = smemAddr(bRing + static_cast<size_t>(sb) * bBytes);
#pragma unroll
                for (int ks = 0; ks < CH / 16; ++ks) {
                    for (int nb = 0; nb < shape.blocks; ++nb) {
                        const uint64_t descB =
                            operandDescriptor(bBase + nb * (shape.NB / 8) * kRowGroupStride + ks * 2 * kCore, kCore, kRowGroupStride);
#pragma unroll
                        for (int term = 0; term < 3; ++term) {
                            const uint64_t descA =
                                operandDescriptor(aBase + term * kTermChunkBytes + ks * 2 * kCore, kCore, kRowGroupStride);
                            mmaBf16(tmem + nb * shape.NB, descA, descB, idesc, (c > 0 || ks > 0 || term > 0) ? 1u : 0u);
                        }
                    }
                }
                commitTo(smemAddr(&aEmpty[sa]));
                commitTo(smemAddr(&bEmpty[sb]));
            }
            commitTo(smemAddr(&accFull));
        }
    } else {
        // ---- converters: warp w owns the row groups w, w + CW, ... of the tile (8 rows each); lane -> row lane % 8,
        // channels [8 (lane / 8), + 8) of each 32-channel box of the chunk
        const int rm = lane & 7, cq = lane >> 3;
        constexpr int kGroupsPerWarp = 16 / CW, kPieces = kGroupsPerWarp * G::kBoxes;
        float4 suNext[G::kBoxes], svNext[G::kBoxes];
        auto loadScales = [&](int chunk) {
#pragma unroll
            for (int b = 0; b < G::kBoxes; ++b) {
                suNext[b] = svNext[b] = make_float4(1.0f, 1.0f, 1.0f, 1.0f);
                if (p.kScale) {
                    suNext[b] = __ldg(reinterpret_cast<const float4 *>(p.kScale + chunk * CH + 32 * b + 8 * cq));
                    svNext[b] = __ldg(reinterpret_cast<const float4 *>(p.kScale + chunk * CH + 32 * b + 8 * cq + 4));
                }
            }
        };
        loadScales(0);
        for (int c = 0; c < chunks; ++c) {
            const int slot = c % kRawRing, sa = c % kAStages;
            await(&rawFull[slot], (c / kRawRing) & 1);
            const uint8_t *src = raw + slot * kRawChunkBytes;
            uint4 ru[kPieces], rv[kPieces];
#pragma unroll
            for (int h = 0; h < kGroupsPerWarp; ++h)
#pragma unroll
                for (int b = 0; b < G::kBoxes; ++b) {
                    const uint8_t *row = src + b * G::kBoxBytes + (8 * (warp + kConvWarps * h) + rm) * 128;
                    ru[h * G::kBoxes + b] = *reinterpret_cast<const uint4 *>(row + (((2 * cq) ^ rm) << 4));
                    rv[h * G::kBoxes + b] = *reinterpret_cast<const uint4 *>(row + (((2 * cq + 1) ^ rm) << 4));
                }
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smemAddr(&rawEmpty[slot])) : "memory");
            // this chunk's scales were asked for one chunk ago; the next chunk's go out now, so that their L2 round
            // trip does not sit between the raw chunk and the operand stores
            float4 su[G::kBoxes], sv[G::kBoxes];
#pragma unroll
            for (int b = 0; b < G::kBoxes; ++b) {
                su[b] = suNext[b];
                sv[b] = svNext[b];
            }
            if (c + 1 < chunks) loadScales(c + 1);
            if (c >= kAStages) await(&aEmpty[sa], (c / kAStages - 1) & 1);
            uint8_t *stage = aStages + sa * kAStageBytes;
#pragma unroll
            for (int h = 0; h < kGroupsPerWarp; ++h)
#pragma unroll
                for (int b = 0; b < G::kBoxes; ++b) {
                    const uint4 qu = ru[h * G::kBoxes + b], qv = rv[h * G::kBoxes + b];
                    const float4 u = make_float4(__uint_as_float(qu.x) * su[b].x, __uint_as_float(qu.y) * su[b].y,
                                                 __uint_as_float(qu.z) * su[b].z, __uint_as_float(qu.w) * su[b].w);
                    const float4 v = make_float4(__uint_as_float(qv.x) * sv[b].x, __uint_as_float(qv.y) * sv[b].y,
                                                 __uint_as_float(qv.z) * sv[b].z, __uint_as_float(qv.w) * sv[b].w);
                    const Converted cv = splitThree(u, v);
                    uint8_t *dst = stage + (warp + kConvWarps * h) * kRowGroupStride + (4 * b + cq) * kCore + rm * 16;
                    *reinterpret_cast<uint4 *>(dst) = cv.hi;
                    *reinterpret_cast<uint4 *>(dst + kTermChunkBytes) = cv.mid;
                    *reinterpret_cast<uint4 *>(dst + 2 * kTermChunkBytes) = cv.lo;
                }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smemAddr(&aFull[sa])) : "memory");
        }

        // ---- accumulators -> out: warp w reads lanes [32 (w % 4), + 32) and half of the columns
        await(&accFull, 0);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const bool poison = *failFlag != 0;
        const int q = warp & 3, part = ((NP + CW / 4 - 1) / (CW / 4) + 15) / 16 * 16;   // columns per warp of a lane quarter
        const int colBegin = (warp >> 2) * part, colEnd = min(NP, colBegin + part);
        const int row = row0 + 32 * q + lane;
        const bool wideMask = (N % 8) == 0 && (ldN % 8) == 0;
        const bool wideOut = (N % 4) == 0 && (ldN % 4) == 0;
        for (int col0 = colBegin; col0 < colEnd; col0 += 16) {
            uint32_t r[16];
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
                : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                  "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                : "r"(tmem + (static_cast<uint32_t>(32 * q) << 16) + col0));
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (row >= p.rows || col0 >= N) continue;
            const size_t o = static_cast<size_t>(row) * ldN + col0;
            uint8_t m[16];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                if (p.mask && wideMask && col0 + 8 * h + 8 <= N) {
                    const uint2 w = *reinterpret_cast<const uint2 *>(p.mask + o + 8 * h);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        m[8 * h + j] = static_cast<uint8_t>(w.x >> (8 * j));
                        m[8 * h + 4 + j] = static_cast<uint8_t>(w.y >> (8 * j));
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        m[8 * h + j] = (p.mask && col0 + 8 * h + j < N) ? p.mask[o + 8 * h + j] : static_cast<uint8_t>(p.maskKeeps);
                }
            }
            float v[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const float keep = p.maskKeeps ? static_cast<float>(m[j] != 0) : (m[j] == 0 ? 1.0f : 0.0f);
                v[j] = poison ? __int_as_float(0x7fc00000) : __uint_as_float(r[j]) * keep;
            }
#pragma unroll
            for (int h = 0; h < 4; ++h) {
                if (wideOut && col0 + 4 * h + 4 <= N) {
                    *reinterpret_cast<float4 *>(p.out + o + 4 * h) = make_float4(v[4 * h], v[4 * h + 1], v[4 * h + 2], v[4 * h + 3]);
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (col0 + 4 * h + j < N) p.out[o + 4 * h + j] = v[4 * h + j];
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(shape.tmemCols) : "memory");
    }
    if (tid == 0 && failed && p.status) atomicExch(p.status, 1);
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

// [rows][K] floats in boxes of 128 rows x 32 floats with the 128-byte swizzle; rows beyond the tensor read as zero.
// The x coordinate of every copy is a multiple of 32 floats.
CUtensorMap gradientMap(const float *G, int rows, int K) {
    CUtensorMap map;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(K) * sizeof(float)};
    const cuuint32_t box[2] = {kChunk, kTileM};
    const cuuint32_t elementStrides[2] = {1, 1};
    const CUresult rc = encodeTiled()(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(G), dims, strides, box, elementStrides,
                                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) fail(RXMET_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d", static_cast<int>(rc));
    return map;
}

WideShape shapeFor(int N) {
    WideShape s{};
    s.blocks = N > 256 ? 2 : 1;
    s.NP = (N + 16 * s.blocks - 1) / (16 * s.blocks) * (16 * s.blocks);
    s.NB = s.NP / s.blocks;
    s.tmemCols = 32;
    while (s.tmemCols < s.NP) s.tmemCols *= 2;
    return s;
}

}  // namespace

size_t widePackedBytes(int K, int N) { return (N > kMaxColumns || K % kChunk != 0) ? 0 : static_cast<size_t>(shapeFor(N).NP) * K * 2; }

bool wideTakes(int K, int N) {
    static const bool disabled = std::getenv("RXMET_IGRAD_SIMT") != nullptr || std::getenv("RXMET_IGRAD_NARROW") != nullptr;
    static const int least = std::getenv("RXMET_IGRAD_STREAM_ALL") != nullptr ? 1 : 65;
    return !disabled && N >= least && N <= kMaxColumns && K >= kChunk && K % kChunk == 0 && encodeTiled() != nullptr;
}

bool wideEligible(const Problem &p) {
    return wideTakes(p.K, p.N) && p.packed != nullptr && alignedTo(p.G, 16) && alignedTo(p.packed, 16) &&
           (p.kScale == nullptr || alignedTo(p.kScale, 16));
}

template <int CH, int CW>
void launchWideAs(const Problem &prob, const WideShape &shape, cudaStream_t st) {
    using G = WideGeometry<CH, CW>;
    const size_t smem = G::sharedBytes(shape.NP);
    ensureDynamicSmem(reinterpret_cast<const void *>(inputGradWideUmma<CH, CW>), smem);
    const CUtensorMap map = gradientMap(prob.G, prob.rows, prob.K);
    const int items = (prob.K / 8) * shape.NP;
    KernelTimer timer__("inputGradUmma", st);
    packWideWeights<<<(items + 255) / 256, 256, 0, st>>>(prob.codesNK, prob.codesKN, prob.ldCodesKN ? prob.ldCodesKN : prob.N, prob.K, prob.N,
                                                         shape.NP, CH, static_cast<uint4 *>(prob.packed));
    inputGradWideUmma<CH, CW><<<(prob.rows + kTileM - 1) / kTileM, G::kThreads, smem, st>>>(prob, shape, map);
}

void launchWide(const Problem &prob, cudaStream_t st) {
    const WideShape shape = shapeFor(prob.N);
    // up to 80 columns leave room for 64-channel chunks and sixteen converter warps (half as many hand-overs per tile)
    static const bool narrowChunks = std::getenv("RXMET_IGRAD_CHUNK32") != nullptr;
    if (prob.K % 64 == 0 && !narrowChunks && WideGeometry<64, 16>::sharedBytes(shape.NP) <= static_cast<size_t>(currentDevice().smemMax))
        launchWideAs<64, 16>(prob, shape, st);
    else launchWideAs<32, 8>(prob, shape, st);
}

}  // namespace igrad
}  // namespace rxmet
