// Device helpers shared by the tcgen05 kernels: operand and instruction descriptors, MMA issue
// and commit, bounded mbarrier waits, tensor-memory loads, the three-way bf16 split of fp32
// values, and 16-byte asynchronous copies.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

namespace rxmet {
namespace umma {

constexpr int kTileM = 128;             // accumulator rows = tensor-memory lanes
constexpr uint32_t kCore = 128;         // bytes of one core matrix: 8 rows of 16 bytes
constexpr uint32_t kSpinLimit = 1u << 20;  // about 0.13 s of polling; a legitimate wait lasts microseconds

__device__ __forceinline__ uint32_t smemAddr(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ uint32_t packBf16(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ float bf16Lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16Hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

// Shared-memory operand descriptor, no swizzle, 16-bit elements.  A core matrix is 128
// contiguous bytes: 8 rows of 16 bytes.
//   MN-major operand: element (mn, k) lives at
//     (mn / 8) * mnGroupStride + (k / 8) * kGroupStride + (k % 8) * 16 + (mn % 8) * 2   bytes,
//   K-major operand:  element (mn, k) lives at
//     (mn / 8) * mnGroupStride + (k / 8) * kGroupStride + (mn % 8) * 16 + (k % 8) * 2   bytes.
// Bits: start address >> 4 in [0,14), k-group stride >> 4 in [16,30) ("leading byte offset"),
// mn-group stride >> 4 in [32,46) ("stride byte offset"), descriptor version 1 in [46,48).
__device__ __forceinline__ uint64_t operandDescriptor(uint32_t addr, uint32_t kGroupStride, uint32_t mnGroupStride) {
    return static_cast<uint64_t>((addr >> 4) & 0x3fffu) | (static_cast<uint64_t>((kGroupStride >> 4) & 0x3fffu) << 16) |
           (static_cast<uint64_t>((mnGroupStride >> 4) & 0x3fffu) << 32) | (1ull << 46);
}

// Instruction descriptor of kind::f16 for a 128-row accumulator tile: fp32 accumulator (bits
// [4,6) = 1), bf16 A and B ([7,10) = [10,13) = 1), operand majors in bits 15 (A) and 16 (B),
// 1 = MN-major, N >> 3 in [17,23), M >> 4 in [24,29).
__host__ __device__ constexpr uint32_t instructionDescriptor(int n, bool aMnMajor, bool bMnMajor) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (aMnMajor ? (1u << 15) : 0u) | (bMnMajor ? (1u << 16) : 0u) |
           (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(kTileM >> 4) << 24);
}

__device__ __forceinline__ void mmaBf16(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t"
        "}\n"
        :
        : "r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}

__device__ __forceinline__ void commitTo(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// Polls the barrier phase of the given parity; false when the limit ran out.  `polls`
// (optional) receives the number of polls made.
__device__ __forceinline__ bool waitPhase(uint32_t bar, uint32_t parity, uint32_t *polls = nullptr) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t"
            "}\n"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
        if (done) {
            if (polls) *polls = i + 1;
            return true;
        }
    }
    if (polls) *polls = kSpinLimit;
    return false;
}

__device__ __forceinline__ void tmemLoad32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

struct Converted {
    uint4 hi, mid, lo;
};

// Eight fp32 values -> three bf16x8 vectors whose sum is the input exactly.
__device__ __forceinline__ Converted splitThree(const float4 &u, const float4 &v) {
    const float x[8] = {u.x, u.y, u.z, u.w, v.x, v.y, v.z, v.w};
    uint32_t h[4], m[4], l[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        h[i] = packBf16(x[2 * i], x[2 * i + 1]);
        const float r0 = x[2 * i] - bf16Lo(h[i]), r1 = x[2 * i + 1] - bf16Hi(h[i]);
        m[i] = packBf16(r0, r1);
        l[i] = packBf16(r0 - bf16Lo(m[i]), r1 - bf16Hi(m[i]));
    }
    Converted c;
    c.hi = make_uint4(h[0], h[1], h[2], h[3]);
    c.mid = make_uint4(m[0], m[1], m[2], m[3]);
    c.lo = make_uint4(l[0], l[1], l[2], l[3]);
    return c;
}

// 16-byte asynchronous copy global -> shared; `valid` false writes zeros instead.
__device__ __forceinline__ void copyAsync16(void *dst, const void *src, bool valid) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smemAddr(dst)), "l"(src), "r"(valid ? 16u : 0u)
                 : "memory");
}

}  // namespace umma
}  // namespace rxmet
