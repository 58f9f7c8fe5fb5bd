// Host -> device staging of a step's inputs by a kernel that reads page-locked, device-mapped
// host memory directly (PCIe reads issued by a few CTAs) instead of a copy-engine transfer.
// Meant to run on a side stream next to a training step: a narrow grid leaves the SMs of the
// step alone, the loads bypass L1 and the stores are marked evict-first, so the staged bytes
// do not displace the step's working set in L2.
#include "common.h"

namespace rxmet {
namespace {

__global__ void __launch_bounds__(256) stageFromHost(const uint4 *__restrict__ src, uint4 *__restrict__ dst, size_t vectors,
                                                     const unsigned char *__restrict__ srcTail, unsigned char *__restrict__ dstTail,
                                                     int tailBytes) {
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    // eight independent 16-byte loads per thread and pass: a PCIe read takes microseconds, and the bytes in flight
    // (CTAs x 256 threads x 128 B) decide the rate
    constexpr int kInFlight = 8;
    size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    for (; i + (kInFlight - 1) * stride < vectors; i += kInFlight * stride) {
        uint4 v[kInFlight];
#pragma unroll
        for (int k = 0; k < kInFlight; ++k)
            asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(v[k].x), "=r"(v[k].y), "=r"(v[k].z), "=r"(v[k].w)
                         : "l"(src + i + k * stride));
#pragma unroll
        for (int k = 0; k < kInFlight; ++k)
            asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(dst + i + k * stride), "r"(v[k].x), "r"(v[k].y),
                         "r"(v[k].z), "r"(v[k].w)
                         : "memory");
    }
    for (; i < vectors; i += stride) dst[i] = src[i];
    if (blockIdx.x == 0 && static_cast<int>(threadIdx.x) < tailBytes) dstTail[threadIdx.x] = srcTail[threadIdx.x];
}

}  // namespace
}  // namespace rxmet

extern "C" int rxmet_stage_from_pinned_host(void *dst_dev, const void *src_host, size_t bytes, int ctas, void *stream) {
    using namespace rxmet;
    return guarded([&] {
        RXMET_REQUIRE(dst_dev != nullptr && src_host != nullptr, "staging: null pointer");
        RXMET_REQUIRE((reinterpret_cast<uintptr_t>(dst_dev) & 15u) == 0 && (reinterpret_cast<uintptr_t>(src_host) & 15u) == 0,
                      "staging: both buffers must be 16-byte aligned");
        if (bytes == 0) return;
        void *mapped = nullptr;
        RXMET_CUDA(cudaHostGetDevicePointer(&mapped, const_cast<void *>(src_host), 0));
        const size_t vectors = bytes / 16;
        const int tail = static_cast<int>(bytes % 16);
        const int grid = std::max(1, std::min(ctas > 0 ? ctas : 16, 1024));
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        KernelTimer timer__("stageFromHost", st);
        stageFromHost<<<grid, 256, 0, st>>>(static_cast<const uint4 *>(mapped), static_cast<uint4 *>(dst_dev), vectors,
                                            static_cast<const unsigned char *>(mapped) + vectors * 16,
                                            static_cast<unsigned char *>(dst_dev) + vectors * 16, tail);
        afterLaunch("stageFromHost");
    });
}
