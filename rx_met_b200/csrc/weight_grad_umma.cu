// Weight-gradient GEMM on the fifth-generation tensor cores (tcgen05.mma, accumulators in
// tensor memory).
//
//   partial[s][m][n] = sum over the K rows of split s of A[k][m] * B[k][n]      (m < M)
//   partial[s][M][n] = sum over the same rows of B[k][n]                        (bias gradient)
//
// A holds small integers (activation codes minus their zero point), exact in bf16.  B (fp32
// gradients) is split into three bf16 terms that together carry all 24 significand bits, and the
// three products accumulate into the same fp32 accumulator, so every product is exact and only
// the accumulation rounds, as in an fp32 GEMM.
//
// One CTA owns a 128 x NT accumulator tile (NT columns of tensor memory) over one K split.
// Both operands arrive from HBM with the contraction index outermost ([k][m], [k][n]), which is
// the "MN-major" operand form of the instruction: no transposition anywhere.  The producer
// threads load fp32 / int32 rows, convert, and store 16-byte pieces straight into the
// un-swizzled canonical operand layout (8 k-rows x 8 mn-elements per 128-byte core matrix);
// one thread then issues the MMAs for the stage and commits them to an mbarrier.  Two operand
// stages alternate, so the conversion of one 32-row chunk overlaps the tensor work of the
// previous one.  One CTA per SM: the raw rows reach shared memory through a ring of cp.async
// copies issued several chunks ahead, which keeps enough bytes in flight to cover the HBM
// latency from a single CTA and halves the number of K splits (and partial tiles) against two
// CTAs per SM.
//
// Every mbarrier wait is bounded: when a wait gives up the CTA records it in the status word and
// carries on with the same control flow (the results are then wrong, and the reduction that
// follows turns them into NaN), so the kernel always reaches the point where it gives its tensor
// memory back.
#include <algorithm>
#include <cstdlib>

#include "common.h"
#include "umma_device.cuh"
#include "weight_grad_mma.h"

namespace rxmet {
namespace wgrad {
namespace {

using namespace umma;

constexpr int kStageRows = 32;          // K rows per stage: two MMA k-steps of 16

// Depth of the ring of raw (unconverted) chunks, chosen so that ring + operand stages fill the
// shared memory of an SM.
template <int NT, int ATERMS = 1>
struct Geometry {
    static constexpr int kThreads = 2 * NT;                      // two thread halves, two k-groups of B each
    static constexpr int kWarps = kThreads / 32;
    static constexpr int kAPieces = (16 + kWarps - 1) / kWarps;  // A pieces (k-group x 32 rows of m) per warp
    static constexpr uint32_t kAKStride = (kTileM / 8) * kCore;  // bytes between k-groups of the A tile
    static constexpr uint32_t kBKStride = (NT / 8) * kCore;
    static constexpr uint32_t kABytes = (kStageRows / 8) * kAKStride;
    static constexpr uint32_t kBBytes = (kStageRows / 8) * kBKStride;
    static constexpr uint32_t kStageBytes = ATERMS * kABytes + 3 * kBBytes;
    static constexpr uint32_t kRawPieces = 2 * kWarps + 16;      // 1 KB pieces of a raw chunk: B per warp, then A
    static constexpr uint32_t kRawBytes = kRawPieces * 1024;
    static constexpr int kRing = NT <= 128 ? 4 : (NT <= 192 ? (ATERMS == 1 ? 3 : 2) : 2);
    static_assert(2 * kStageBytes + kRing * kRawBytes <= 227 * 1024, "shared memory of one SM");
    static constexpr size_t kSmem = 2 * kStageBytes + static_cast<size_t>(kRing) * kRawBytes;
};

// blockDim.x == 2 NT, one CTA per SM.  Warp w produces the B columns [32 (w % (NT/32)), + 32) of
// the tile for two of the four k-groups of a chunk (which two: w / (NT/32)): lane -> k-row
// (lane % 8) of a k-group and 8-column piece (lane / 8), so a warp's 16-byte operand stores cover
// four whole core matrices (512 contiguous bytes) and its loads cover 8 rows x 128 contiguous bytes.  Each thread copies its own pieces of the next chunks into a
// ring of raw buffers with cp.async, kRing chunks ahead; a warp later converts exactly the pieces
// it copied, so the ring needs no CTA-wide barrier of its own.
template <int NT, int ATERMS>
__global__ void __launch_bounds__(2 * NT, 1)
weightGradUmma(const __grid_constant__ ProblemSet set, int K, int N, int chunkK, int *status) {
    const Problem &p = set.slab[blockIdx.z];  // gridDim.z problems / slabs share one launch
    using G = Geometry<NT, ATERMS>;
    constexpr int NW = G::kWarps, CW = NT / 32, AT = G::kAPieces, R = G::kRing, TH = G::kThreads;
    constexpr uint32_t kAKStride = G::kAKStride, kBKStride = G::kBKStride, kABytes = G::kABytes, kBBytes = G::kBBytes;
    constexpr uint32_t kStageBytes = G::kStageBytes;
    constexpr uint32_t kTmemCols = NT > 128 ? 256 : 128;
    constexpr uint32_t kIdesc = instructionDescriptor(NT, true, true);

    extern __shared__ __align__(128) uint8_t stages[];
    __shared__ __align__(8) uint64_t bars[3];
    __shared__ uint32_t tmemSlot;
    __shared__ int failed;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int rk = lane & 7, cq = lane >> 3;
    const int cw = warp % CW, half = warp / CW;  // column warp and k-group half of the B pieces
    const int n0 = blockIdx.x * NT;
    const int kBegin = blockIdx.y * chunkK, kEnd = min(K, kBegin + chunkK);
    const int chunks = (kEnd - kBegin + kStageRows - 1) / kStageRows;
    const int M = p.M, quads = (M + 31) / 32;
    uint4 *raw = reinterpret_cast<uint4 *>(stages + 2 * kStageBytes);  // [R][kRawPieces][64]

    if (tid == 0) {
        failed = 0;
        for (int i = 0; i < 3; ++i)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smemAddr(&bars[i])) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // rows of A beyond M stay zero for the whole kernel
    for (uint32_t i = tid; i < 2 * ATERMS * kABytes / 16; i += TH) {
        const uint32_t stage = i / (ATERMS * kABytes / 16), off = i % (ATERMS * kABytes / 16);
        *reinterpret_cast<uint4 *>(stages + stage * kStageBytes + off * 16) = make_uint4(0u, 0u, 0u, 0u);
    }
    const int lda = p.lda ? p.lda : M;
    const int totalRows = p.totalRows ? p.totalRows : M + 1;
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(&tmemSlot)), "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }

    const void *aBase = p.aCodes ? static_cast<const void *>(p.aCodes) : static_cast<const void *>(p.aFloat);
    // Copies this warp's pieces of chunk `chunk` into ring entry `slot` and closes the group.  A
    // piece is 8 k-rows x 128 bytes; one copy instruction of the warp covers four whole rows of
    // it (lane -> row lane / 8, 16-byte part lane % 8), so every request is a full 128-byte line.
    // Part p of row r is kept at position r * 8 + (p ^ r) of the piece, which makes both these
    // writes and the converting reads (lane -> row lane % 8, parts 2 (lane / 8) and + 1) free of
    // bank conflicts.
    auto issueChunk = [&](int chunk, int slot) {
        const int k0 = kBegin + chunk * kStageRows;
        uint4 *dstB = raw + (static_cast<size_t>(slot) * G::kRawPieces + 2 * warp) * 64;
        uint4 *dstA = raw + (static_cast<size_t>(slot) * G::kRawPieces + 2 * NW) * 64;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int wrow = 4 * i + (lane >> 3), part = lane & 7, pos = wrow * 8 + (part ^ wrow);
#pragma unroll
            for (int gi = 0; gi < 2; ++gi) {
                const int k = k0 + 8 * (2 * half + gi) + wrow;
                const bool ok = k < kEnd;
                copyAsync16(dstB + gi * 64 + pos, ok ? p.B + static_cast<size_t>(k) * N + n0 + 32 * cw + 4 * part : p.B, ok);
            }
#pragma unroll
            for (int t = 0; t < AT; ++t) {
                const int task = warp + t * NW, m = 32 * (task >> 2) + 4 * part;
                const int k = k0 + 8 * (task & 3) + wrow;
                if (task >= 16) continue;
                const bool ok = task < 4 * quads && k < kEnd && m < M;
                const size_t at = ok ? static_cast<size_t>(k) * lda + m : 0;
                copyAsync16(dstA + task * 64 + pos, static_cast<const uint32_t *>(aBase) + at, ok);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
#pragma unroll
    for (int r = 0; r < R; ++r) issueChunk(r, r);

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmemSlot;

    float csum[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) csum[j] = 0.0f;

    // converts ring entry `slot` into the operand stage
    auto convertChunk = [&](int slot, uint8_t *stage) {
        const uint4 *srcB = raw + (static_cast<size_t>(slot) * G::kRawPieces + 2 * warp) * 64;
        const uint4 *srcA = raw + (static_cast<size_t>(slot) * G::kRawPieces + 2 * NW) * 64;
        const int posU = rk * 8 + ((2 * cq) ^ rk), posV = rk * 8 + ((2 * cq + 1) ^ rk);
#pragma unroll
        for (int gi = 0; gi < 2; ++gi) {
            const int g = 2 * half + gi;
            const uint4 ru = srcB[gi * 64 + posU], rv = srcB[gi * 64 + posV];
            const float4 u = make_float4(__uint_as_float(ru.x), __uint_as_float(ru.y), __uint_as_float(ru.z), __uint_as_float(ru.w));
            const float4 v = make_float4(__uint_as_float(rv.x), __uint_as_float(rv.y), __uint_as_float(rv.z), __uint_as_float(rv.w));
            csum[0] += u.x; csum[1] += u.y; csum[2] += u.z; csum[3] += u.w;
            csum[4] += v.x; csum[5] += v.y; csum[6] += v.z; csum[7] += v.w;
            const Converted c = splitThree(u, v);
            uint8_t *dst = stage + ATERMS * kABytes + (4 * cw + cq) * kCore + rk * 16 + g * kBKStride;
            *reinterpret_cast<uint4 *>(dst) = c.hi;
            *reinterpret_cast<uint4 *>(dst + kBBytes) = c.mid;
            *reinterpret_cast<uint4 *>(dst + 2 * kBBytes) = c.lo;
        }
#pragma unroll
        for (int t = 0; t < AT; ++t) {
            const int task = warp + t * NW, g = task & 3, quad = task >> 2;
            if (task >= 4 * quads) continue;
            const uint4 ru = srcA[task * 64 + posU], rv = srcA[task * 64 + posV];
            float x[8];
            // zero-filled pieces decode to some finite value: they only meet zero rows of B or
            // accumulator rows that are never stored
            if (p.aCodes) {
                const uint32_t q[8] = {ru.x, ru.y, ru.z, ru.w, rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                for (int i = 0; i < 8; ++i) x[i] = static_cast<float>(static_cast<int32_t>(q[i]) - p.aZero);
            } else {  // recover the integer code difference from the dequantized value
                const uint32_t q[8] = {ru.x, ru.y, ru.z, ru.w, rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                for (int i = 0; i < 8; ++i) x[i] = rintf(__uint_as_float(q[i]) * p.aInvScale) - p.aFloatZero;
            }
            uint8_t *dstA = stage + (4 * quad + cq) * kCore + rk * 16 + g * kAKStride;
            if (ATERMS == 2) {
                // a = 256 * floor(a / 256) + (a mod 256): both terms are exact in bf16 for |a| < 2^17
                float hi[8], lo[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    hi[i] = floorf(x[i] * (1.0f / 256.0f)) * 256.0f;
                    lo[i] = x[i] - hi[i];
                }
                *reinterpret_cast<uint4 *>(dstA) =
                    make_uint4(packBf16(hi[0], hi[1]), packBf16(hi[2], hi[3]), packBf16(hi[4], hi[5]), packBf16(hi[6], hi[7]));
                *reinterpret_cast<uint4 *>(dstA + kABytes) =
                    make_uint4(packBf16(lo[0], lo[1]), packBf16(lo[2], lo[3]), packBf16(lo[4], lo[5]), packBf16(lo[6], lo[7]));
            } else {
                *reinterpret_cast<uint4 *>(dstA) =
                    make_uint4(packBf16(x[0], x[1]), packBf16(x[2], x[3]), packBf16(x[4], x[5]), packBf16(x[6], x[7]));
            }
        }
    };

    for (int c = 0; c < chunks; ++c) {
        const int s = c & 1, slot = c % R;
        uint8_t *stage = stages + s * kStageBytes;
        asm volatile("cp.async.wait_group %0;" ::"n"(R - 1) : "memory");
        __syncwarp();  // the lanes of a warp convert what other lanes of it copied
        // the MMAs that read this stage two chunks ago must have finished
        if (c >= 2 && !waitPhase(smemAddr(&bars[s]), ((c >> 1) - 1) & 1)) failed = 1;
        convertChunk(slot, stage);
        __syncwarp();
        issueChunk(c + R, slot);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncthreads();
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t base = smemAddr(stage);
#pragma unroll
            for (int ks = 0; ks < kStageRows / 16; ++ks) {
#pragma unroll
                for (int at = 0; at < ATERMS; ++at) {
                    const uint64_t descA = operandDescriptor(base + at * kABytes + ks * 2 * kAKStride, kAKStride, kCore);
#pragma unroll
                    for (int sp = 0; sp < 3; ++sp) {
                        const uint64_t descB =
                            operandDescriptor(base + ATERMS * kABytes + sp * kBBytes + ks * 2 * kBKStride, kBKStride, kCore);
                        mmaBf16(tmem, descA, descB, kIdesc, (c > 0 || ks > 0 || sp > 0 || at > 0) ? 1u : 0u);
                    }
                }
            }
            commitTo(smemAddr(&bars[s]));
            if (c + 1 == chunks) commitTo(smemAddr(&bars[2]));
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (chunks > 0 && !waitPhase(smemAddr(&bars[2]), 0)) failed = 1;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

    float *slice = p.partial + static_cast<size_t>(blockIdx.y) * totalRows * N;
    float *out = slice + static_cast<size_t>(p.rowBase) * N;
    // accumulator rows: warp w may read the tensor-memory lanes [32 (w % 4), 32 (w % 4) + 32)
    {
        const int q = warp & 3, sharing = (NW - q + 3) / 4;
        if (32 * q < M && chunks > 0) {
            float4 *tile = reinterpret_cast<float4 *>(stages + warp * 4096);  // the operand stages are idle now
            for (int j = warp >> 2; j < CW; j += sharing) {
                uint32_t r[32];
                tmemLoad32(tmem + (static_cast<uint32_t>(32 * q) << 16) + 32 * j, r);
                // lane = accumulator row here; turn the 32 x 32 block through shared memory so that a
                // store instruction of the warp writes four whole 128-byte row segments
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    tile[lane * 8 + (i ^ (lane & 7))] = make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]),
                                                                    __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
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
    }
    // column sums of B: fold the eight k-row lanes, fixed order
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        float v = csum[j];
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        csum[j] = v;
    }
    // ... then the two thread halves, through the (now idle) first operand stage
    float *scratch = reinterpret_cast<float *>(stages + NW * 4096);  // behind the warps' epilogue tiles
    if (half == 1 && rk == 0) {
#pragma unroll
        for (int j = 0; j < 8; ++j) scratch[32 * cw + 8 * cq + j] = csum[j];
    }
    __syncthreads();
    if (half == 0 && rk == 0 && p.writeBias) {
#pragma unroll
        for (int j = 0; j < 8; ++j) csum[j] += scratch[32 * cw + 8 * cq + j];
        float4 *dst = reinterpret_cast<float4 *>(slice + static_cast<size_t>(totalRows - 1) * N + n0 + 32 * cw + 8 * cq);
        dst[0] = make_float4(csum[0], csum[1], csum[2], csum[3]);
        dst[1] = make_float4(csum[4], csum[5], csum[6], csum[7]);
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
    if (tid == 0 && failed && status) atomicExch(status, 1);
}

template <int NT, int ATERMS>
void launchSet(const ProblemSet &set, int K, int N, int chunkK, int splits, cudaStream_t st) {
    constexpr size_t smem = Geometry<NT, ATERMS>::kSmem;
    ensureDynamicSmem(reinterpret_cast<const void *>(weightGradUmma<NT, ATERMS>), smem);  // per device
    KernelTimer timer__("weightGradUmma", st);
    weightGradUmma<NT, ATERMS><<<dim3(N / NT, splits, set.count), Geometry<NT, ATERMS>::kThreads, smem, st>>>(
        set, K, N, chunkK, set.slab[0].status);
}

template <int NT>
void launchTile(const Problem &prob, const Problem *other, int K, int N, int chunkK, int splits, cudaStream_t st) {
    ProblemSet set;
    set.slab[0] = prob;
    set.count = 1;
    if (other) set.slab[set.count++] = *other;
    launchSet<NT, 1>(set, K, N, chunkK, splits, st);
}

int tileColumns(int N) {
    for (int nt : {256, 192, 128})
        if (N % nt == 0) return nt;
    return 0;
}

}  // namespace

bool tensorMemoryPath(int M, int N) {
    static const bool disabled = std::getenv("RXMET_WGRAD_MMA_SYNC") != nullptr;
    return !disabled && M >= 4 && M <= kTileM && M % 4 == 0 && N % 4 == 0 && tileColumns(N) != 0;
}

int planTensorMemory(int K, int N, int sms, int *chunkK, int slabs) {
    const int tiles = (N / tileColumns(N)) * std::max(1, slabs);
    const int want = std::max(1, sms / tiles);  // one CTA per SM
    *chunkK = ((K + want - 1) / want + kStageRows - 1) / kStageRows * kStageRows;
    return (K + *chunkK - 1) / *chunkK;
}

void launchTensorMemory(const Problem &prob, const Problem *other, int K, int N, int chunkK, int splits, cudaStream_t st) {
    switch (tileColumns(N)) {
        case 256: launchTile<256>(prob, other, K, N, chunkK, splits, st); break;
        case 192: launchTile<192>(prob, other, K, N, chunkK, splits, st); break;
        case 128: launchTile<128>(prob, other, K, N, chunkK, splits, st); break;
        default: fail(RXMET_ERR_UNSUPPORTED, "no tensor-memory tile for %d columns", N);
    }
}

int slabsOf(int M) { return (M + kTileM - 1) / kTileM; }

bool slabPathTakes(int Ma, int Mb, int N) {
    static const bool disabled = std::getenv("RXMET_WGRAD_MMA_SYNC") != nullptr;
    if (disabled || tileColumns(N) == 0 || Ma % 4 != 0 || Mb % 4 != 0 || Ma < 0 || Mb < 0) return false;
    return slabsOf(Ma) + slabsOf(Mb) >= 1 && slabsOf(Ma) + slabsOf(Mb) <= kMaxSlabs;
}

int slabSplits(int K, int Ma, int Mb, int N, int sms, int *chunkK) {
    return planTensorMemory(K, N, sms, chunkK, slabsOf(Ma) + slabsOf(Mb));
}

int slabSplitBound(int Ma, int Mb, int N) {
    const int nt = tileColumns(N);
    if (nt == 0) return 1;
    return std::max(1, 160 / ((N / nt) * std::max(1, slabsOf(Ma) + slabsOf(Mb))));
}

void launchSlabs(const Problem &a, const Problem &b, int K, int N, int chunkK, int splits, bool wide, cudaStream_t st) {
    ProblemSet set;
    for (const Problem *prob : {&a, &b}) {
        for (int m0 = 0; m0 < prob->M; m0 += kTileM) {
            Problem s = *prob;
            s.M = std::min(kTileM, prob->M - m0);
            s.lda = prob->M;
            s.rowBase = m0;
            s.totalRows = prob->M + 1;
            s.writeBias = m0 == 0 ? 1 : 0;
            s.wideCodes = wide ? 1 : 0;
            if (s.aCodes) s.aCodes += m0;
            if (s.aFloat) s.aFloat += m0;
            set.slab[set.count++] = s;
        }
    }
    RXMET_REQUIRE(set.count >= 1 && set.count <= kMaxSlabs, "weight gradient: %d slabs", set.count);
    switch (tileColumns(N)) {
        case 256: wide ? launchSet<256, 2>(set, K, N, chunkK, splits, st) : launchSet<256, 1>(set, K, N, chunkK, splits, st); break;
        case 192: wide ? launchSet<192, 2>(set, K, N, chunkK, splits, st) : launchSet<192, 1>(set, K, N, chunkK, splits, st); break;
        case 128: wide ? launchSet<128, 2>(set, K, N, chunkK, splits, st) : launchSet<128, 1>(set, K, N, chunkK, splits, st); break;
        default: fail(RXMET_ERR_UNSUPPORTED, "no tensor-memory tile for %d columns", N);
    }
}

}  // namespace wgrad

namespace {

// One warp polls a barrier that nothing completes, with the poll loop of the tcgen05 kernels.
__global__ void boundedWaitProbe(int *status, unsigned int *polls) {
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(umma::smemAddr(&bar)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    uint32_t made = 0;
    const bool completed = umma::waitPhase(umma::smemAddr(&bar), 0, &made);
    if (threadIdx.x == 0) {
        *polls = made;
        if (!completed) atomicExch(status, 1);
    }
}

}  // namespace
}  // namespace rxmet

extern "C" int rxmet_selftest_bounded_wait(int *status_dev, unsigned int *polls_out, void *stream) {
    using namespace rxmet;
    return guarded([&] {
        RXMET_REQUIRE(status_dev != nullptr, "status_dev must not be null");
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        unsigned int *pollsDev = reinterpret_cast<unsigned int *>(status_dev + 1);
        RXMET_CUDA(cudaMemsetAsync(status_dev, 0, 2 * sizeof(int), st));
        boundedWaitProbe<<<1, 32, 0, st>>>(status_dev, pollsDev);
        afterLaunch("boundedWaitProbe");
        int status = 0;
        unsigned int polls = 0;
        RXMET_CUDA(cudaMemcpyAsync(&status, status_dev, sizeof(int), cudaMemcpyDeviceToHost, st));
        RXMET_CUDA(cudaMemcpyAsync(&polls, pollsDev, sizeof(unsigned int), cudaMemcpyDeviceToHost, st));
        RXMET_CUDA(cudaStreamSynchronize(st));
        if (polls_out) *polls_out = polls;
        if (status != 0) fail(RXMET_ERR_DEVICE_TIMEOUT, "a bounded device-side wait ran out after %u polls", polls);
    });
}
