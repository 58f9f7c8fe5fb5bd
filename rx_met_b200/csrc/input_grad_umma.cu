// dx = (G * kScale) code on tcgen05.mma with the accumulator tile in tensor memory.
//
// One CTA per SM owns a contiguous range of rows and walks it in tiles of 128 rows (= the 128
// lanes of tensor memory).  For a tile the accumulator D[128][NP] (NP = N padded to 16) sums
// over K in chunks of 32 channels:
//   * A = the chunk of G, K-major as it lies in HBM ([row][k]).  Warp w copies rows [8w, 8w + 8)
//     of the chunk (8 x 128 bytes) into a ring of raw buffers with cp.async, several chunks ahead,
//     then scales, splits into three bf16 terms and stores 16-byte pieces into the un-swizzled
//     canonical K-major layout (core matrix = 8 rows x 8 k).
//   * B = the weight codes as bf16, converted once per CTA into the same canonical layout and
//     kept in shared memory for all tiles.
//   * one thread issues the six MMAs of the chunk (2 k-steps x 3 terms) and commits them to the
//     mbarrier of the operand stage; kStages stages rotate.
// After the last chunk of a tile the accumulators are read back with tcgen05.ld (lane = row),
// masked and stored.  Every mbarrier wait is bounded; a wait that gives up poisons the CTA's
// outputs with NaN and sets the status word, and the CTA still frees its tensor memory.
#include <algorithm>
#include <cstdlib>

#include "common.h"
#include "input_grad_umma.h"
#include "umma_device.cuh"

namespace rxmet {
namespace igrad {
namespace {

using namespace umma;

constexpr int kThreads = 512, kWarps = kThreads / 32;
constexpr int kChunkK = 64;                      // channels per chunk: four MMA k-steps
constexpr int kSpans = kChunkK / 32;             // 128-byte spans of a row per chunk
constexpr int kRing = 2;                         // raw chunks in flight
constexpr int kStages = 2;                       // operand stages: chunks whose MMAs may be pending
constexpr uint32_t kRawBytes = kTileM * kChunkK * 4;         // 16 x kSpans pieces of 8 rows x 128 bytes
constexpr uint32_t kTermBytes = kTileM * kChunkK * 2;        // 8 KB: one bf16 term of a chunk
constexpr uint32_t kStageBytes = 3 * kTermBytes;
constexpr uint32_t kAKStride = kCore;                        // next k-group of the same 8 rows
constexpr uint32_t kAMStride = (kChunkK / 8) * kCore;        // next 8 rows
constexpr int kMaxK = 768;

size_t sharedBytes(int K, int NP) {
    return kStages * kStageBytes + kRing * kRawBytes + static_cast<size_t>(NP) * K * 2 + sizeof(float) * K;
}

// gridDim.y = column slabs of the output: slab s works on columns [NP s, NP s + NP) with its own copy of the
// weight operand; every slab walks all rows (the gradient rows are re-read from L2 once per slab).
template <int NP>
__global__ void __launch_bounds__(kThreads, 1) inputGradUmma(const Problem whole, int rowsPerCta) {
    Problem p = whole;
    {
        const int n0 = static_cast<int>(blockIdx.y) * NP;
        if (p.ldN == 0) p.ldN = p.N;
        if (p.ldCodesKN == 0) p.ldCodesKN = p.N;
        if (gridDim.y > 1) {
            p.N = min(NP, whole.N - n0);
            if (p.codesNK) p.codesNK += static_cast<size_t>(n0) * p.K;
            if (p.codesKN) p.codesKN += n0;
            if (p.mask) p.mask += n0;
            p.out += n0;
        }
    }
    constexpr uint32_t kTmemCols = NP <= 32 ? 32 : 64;
    constexpr uint32_t kIdesc = instructionDescriptor(NP, false, false);
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t bars[kStages + 1];  // one per operand stage, the last for "tile complete"
    __shared__ uint32_t tmemSlot;
    __shared__ int failed;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int rm = lane & 7, cq = lane >> 3;
    const int K = p.K, N = p.N, chunksPerTile = K / kChunkK;
    const uint32_t kBNStride = static_cast<uint32_t>(K / 8) * kCore;  // next 8 columns of the weight operand
    uint8_t *stages = smem;
    uint4 *raw = reinterpret_cast<uint4 *>(smem + kStages * kStageBytes);   // [kRing][16 warps][kSpans][64]
    uint8_t *weights = smem + kStages * kStageBytes + kRing * kRawBytes;
    float *scale = reinterpret_cast<float *>(weights + static_cast<size_t>(NP) * K * 2);

    const int rowBegin = min(p.rows, static_cast<int>(blockIdx.x) * rowsPerCta);
    const int rowEnd = min(p.rows, rowBegin + rowsPerCta);
    const int tiles = (rowEnd - rowBegin + kTileM - 1) / kTileM;
    const int totalChunks = tiles * chunksPerTile;

    if (tid == 0) {
        failed = 0;
        for (int i = 0; i <= kStages; ++i)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smemAddr(&bars[i])) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(&tmemSlot)), "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }

    // Warp w copies rows [8w, 8w + 8) of linear chunk `chunk` (tile chunk / chunksPerTile) into
    // ring entry `slot`.  A copy instruction covers four whole 128-byte rows (lane -> row
    // lane / 8, 16-byte part lane % 8); part q of row r is kept at r * 8 + (q ^ r), which keeps
    // these writes and the converting reads free of bank conflicts.
    auto issueChunk = [&](int chunk, int slot) {
        const int tile = chunk / chunksPerTile, kc = chunk - tile * chunksPerTile;
        uint4 *dst = raw + (static_cast<size_t>(slot) * kWarps + warp) * kSpans * 64;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int wrow = 4 * i + (lane >> 3), part = lane & 7;
            const int row = rowBegin + tile * kTileM + 8 * warp + wrow;
            const bool ok = chunk < totalChunks && row < rowEnd;
            const float *src = ok ? p.G + static_cast<size_t>(row) * K + kc * kChunkK + 4 * part : p.G;
#pragma unroll
            for (int sp = 0; sp < kSpans; ++sp) copyAsync16(dst + sp * 64 + wrow * 8 + (part ^ wrow), ok ? src + 32 * sp : src, ok);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
#pragma unroll
    for (int r = 0; r < kRing; ++r) issueChunk(r, r);

    // the weight operand: column n, channels [8 j, 8 j + 8) -> one 16-byte row of a core matrix
    // (consecutive threads walk the contiguous index of whichever code layout was given)
    for (int item = tid; item < NP * (K / 8); item += kThreads) {
        const int n = p.codesNK ? item / (K / 8) : item % NP, k8 = p.codesNK ? item % (K / 8) : item / NP;
        float c[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int k = 8 * k8 + j;
            c[j] = n >= N ? 0.0f
                          : (p.codesNK ? static_cast<float>(p.codesNK[static_cast<size_t>(n) * K + k])
                                       : p.codesKN[static_cast<size_t>(k) * p.ldCodesKN + n]);
        }
        *reinterpret_cast<uint4 *>(weights + (n / 8) * kBNStride + k8 * kCore + (n % 8) * 16) =
            make_uint4(packBf16(c[0], c[1]), packBf16(c[2], c[3]), packBf16(c[4], c[5]), packBf16(c[6], c[7]));
    }
    for (int k = tid; k < K; k += kThreads) scale[k] = p.kScale ? p.kScale[k] : 1.0f;

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmemSlot;

    for (int g = 0; g < totalChunks; ++g) {
        const int s = g % kStages, slot = g % kRing;
        const int tile = g / chunksPerTile, kc = g - tile * chunksPerTile;
        uint8_t *stage = stages + s * kStageBytes;
        asm volatile("cp.async.wait_group %0;" ::"n"(kRing - 1) : "memory");
        __syncwarp();  // the lanes of a warp convert what other lanes of it copied
        // the MMAs that read this stage kStages chunks ago must have finished
        if (g >= kStages && !waitPhase(smemAddr(&bars[s]), (g / kStages - 1) & 1)) failed = 1;
#pragma unroll
        for (int span = 0; span < kSpans; ++span) {
            const uint4 *src = raw + ((static_cast<size_t>(slot) * kWarps + warp) * kSpans + span) * 64;
            const uint4 ru = src[rm * 8 + ((2 * cq) ^ rm)], rv = src[rm * 8 + ((2 * cq + 1) ^ rm)];
            const float4 su = *reinterpret_cast<const float4 *>(scale + kc * kChunkK + 32 * span + 8 * cq);
            const float4 sv = *reinterpret_cast<const float4 *>(scale + kc * kChunkK + 32 * span + 8 * cq + 4);
            const float4 u = make_float4(__uint_as_float(ru.x) * su.x, __uint_as_float(ru.y) * su.y,
                                         __uint_as_float(ru.z) * su.z, __uint_as_float(ru.w) * su.w);
            const float4 v = make_float4(__uint_as_float(rv.x) * sv.x, __uint_as_float(rv.y) * sv.y,
                                         __uint_as_float(rv.z) * sv.z, __uint_as_float(rv.w) * sv.w);
            const Converted c = splitThree(u, v);
            uint8_t *dst = stage + warp * kAMStride + (4 * span + cq) * kAKStride + rm * 16;
            *reinterpret_cast<uint4 *>(dst) = c.hi;
            *reinterpret_cast<uint4 *>(dst + kTermBytes) = c.mid;
            *reinterpret_cast<uint4 *>(dst + 2 * kTermBytes) = c.lo;
        }
        __syncwarp();
        issueChunk(g + kRing, slot);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncthreads();
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t aBase = smemAddr(stage), bBase = smemAddr(weights) + kc * (kChunkK / 8) * kCore;
#pragma unroll
            for (int ks = 0; ks < kChunkK / 16; ++ks) {
                const uint64_t descB = operandDescriptor(bBase + ks * 2 * kCore, kCore, kBNStride);
#pragma unroll
                for (int sp = 0; sp < 3; ++sp) {
                    const uint64_t descA = operandDescriptor(aBase + sp * kTermBytes + ks * 2 * kAKStride, kAKStride, kAMStride);
                    mmaBf16(tmem, descA, descB, kIdesc, (kc > 0 || ks > 0 || sp > 0) ? 1u : 0u);
                }
            }
            commitTo(smemAddr(&bars[s]));
            if (kc + 1 == chunksPerTile) commitTo(smemAddr(&bars[kStages]));
        }
        if (kc + 1 < chunksPerTile) continue;

        // the tile is complete: accumulator rows -> out.  Warp w reads lanes [32 (w % 4), + 32) and
        // the 16 columns [16 (w / 4), + 16).
        if (!waitPhase(smemAddr(&bars[kStages]), tile & 1)) failed = 1;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int q = warp & 3, col0 = 16 * (warp >> 2);
        if (col0 < NP) {
            uint32_t r[16];
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
                : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                  "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                : "r"(tmem + (static_cast<uint32_t>(32 * q) << 16) + col0));
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            const int row = rowBegin + tile * kTileM + 32 * q + lane;
            const bool poison = *reinterpret_cast<volatile int *>(&failed) != 0;
            if (row < rowEnd) {
                const size_t o = static_cast<size_t>(row) * p.ldN + col0;
                float v[16];
                uint8_t m[16];
                const bool wide = (N % 8) == 0 && (p.ldN % 8) == 0 && col0 + 8 <= N;  // whole 8-column groups, aligned
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    if (p.mask && wide && col0 + 8 * h + 8 <= N) {
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
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const float keep = p.maskKeeps ? static_cast<float>(m[j]) : (m[j] == 0 ? 1.0f : 0.0f);
                    v[j] = poison ? __int_as_float(0x7fc00000) : __uint_as_float(r[j]) * keep;
                }
#pragma unroll
                for (int h = 0; h < 4; ++h) {
                    if ((N % 4) == 0 && (p.ldN % 4) == 0 && col0 + 4 * h + 4 <= N) {
                        *reinterpret_cast<float4 *>(p.out + o + 4 * h) = make_float4(v[4 * h], v[4 * h + 1], v[4 * h + 2], v[4 * h + 3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            if (col0 + 4 * h + j < N) p.out[o + 4 * h + j] = v[4 * h + j];
                    }
                }
            }
        }
        // the next tile's first MMA overwrites the accumulators: order it behind these loads
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
    if (tid == 0 && failed && p.status) atomicExch(p.status, 1);
}

template <int NP>
void launchPadded(const Problem &prob, int sms, cudaStream_t st) {
    const size_t smem = sharedBytes(prob.K, NP);
    ensureDynamicSmem(reinterpret_cast<const void *>(inputGradUmma<NP>), smem);  // per device
    const int slabs = (prob.N + NP - 1) / NP;
    const int groups = (prob.rows + 7) / 8;
    const int grid = std::max(1, std::min(std::max(1, sms / slabs), groups));
    const int rowsPerCta = (groups + grid - 1) / grid * 8;
    KernelTimer timer__("inputGradUmma", st);
    inputGradUmma<NP><<<dim3(grid, slabs), kThreads, smem, st>>>(prob, rowsPerCta);
}

}  // namespace

bool wideTakes(int K, int N);

bool eligible(int K, int N) {
    static const bool disabled = std::getenv("RXMET_IGRAD_SIMT") != nullptr;
    if (disabled || N < 1) return false;
    if (K >= kChunkK && K % kChunkK == 0 && K <= kMaxK) return true;
    return wideTakes(K, N);   // only with Problem::packed
}

bool wideTakes(int K, int N);
bool wideEligible(const Problem &p);
void launchWide(const Problem &prob, cudaStream_t st);

void launch(const Problem &prob, int sms, cudaStream_t st) {
    if (wideEligible(prob)) {
        launchWide(prob, st);
        return;
    }
    if (prob.K > kMaxK || prob.K % kChunkK != 0)
        fail(RXMET_ERR_UNSUPPORTED, "input gradient: %d channels need the streaming kernel (scratch, 16-byte aligned operands)", prob.K);
    // widest slab whose weight operand fits shared memory beside the stages and the ring
    const int widest = prob.K <= 512 ? 64 : 32;
    const int np = prob.N > widest ? widest : (prob.N + 15) / 16 * 16;
    switch (np) {
        case 16: launchPadded<16>(prob, sms, st); break;
        case 32: launchPadded<32>(prob, sms, st); break;
        case 48: launchPadded<48>(prob, sms, st); break;
        case 64: launchPadded<64>(prob, sms, st); break;
        default: fail(RXMET_ERR_UNSUPPORTED, "input gradient: %d columns", prob.N);
    }
}

}  // namespace igrad
}  // namespace rxmet
