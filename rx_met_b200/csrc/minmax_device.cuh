// Device helpers for running min/max statistics: per-thread accumulators, warp and block
// reduction, and order-preserving float atomics for the final commit.
#pragma once

#include <cuda_runtime.h>

#include <cfloat>

namespace rxmet {
namespace stats {

// Valid for any finite value (-0.0 included) as long as the slot starts at +FLT_MAX / -FLT_MAX.
__device__ __forceinline__ void atomicMinFloat(float *addr, float v) {
    if (v >= 0.0f) atomicMin(reinterpret_cast<int *>(addr), __float_as_int(v));
    else atomicMax(reinterpret_cast<unsigned int *>(addr), __float_as_uint(v));
}
__device__ __forceinline__ void atomicMaxFloat(float *addr, float v) {
    if (v >= 0.0f) atomicMax(reinterpret_cast<int *>(addr), __float_as_int(v));
    else atomicMin(reinterpret_cast<unsigned int *>(addr), __float_as_uint(v));
}

struct MinMax {
    float lo = FLT_MAX, hi = -FLT_MAX;
    __device__ __forceinline__ void see(float v) {
        if (isfinite(v)) {
            lo = fminf(lo, v);
            hi = fmaxf(hi, v);
        }
    }
};

__device__ __forceinline__ MinMax warpReduce(MinMax m) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        m.lo = fminf(m.lo, __shfl_xor_sync(0xffffffffu, m.lo, o));
        m.hi = fmaxf(m.hi, __shfl_xor_sync(0xffffffffu, m.hi, o));
    }
    return m;
}

// Block-wide reduce of N per-thread statistics, then one atomic pair per statistic.
// scratch: 2 * N * (blockDim/32) floats of shared memory.  All threads of the block must call it.
template <int N>
__device__ void commit(MinMax (&local)[N], const int (&slot)[N], float *mins, float *maxs, float *scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int i = 0; i < N; ++i) {
        const MinMax m = warpReduce(local[i]);
        if (lane == 0) {
            scratch[(2 * i) * warps + warp] = m.lo;
            scratch[(2 * i + 1) * warps + warp] = m.hi;
        }
    }
    __syncthreads();
    if (threadIdx.x < N) {
        float lo = FLT_MAX, hi = -FLT_MAX;
        for (int w = 0; w < warps; ++w) {
            lo = fminf(lo, scratch[(2 * threadIdx.x) * warps + w]);
            hi = fmaxf(hi, scratch[(2 * threadIdx.x + 1) * warps + w]);
        }
        if (lo <= hi) {
            atomicMinFloat(&mins[slot[threadIdx.x]], lo);
            atomicMaxFloat(&maxs[slot[threadIdx.x]], hi);
        }
    }
    __syncthreads();
}

}  // namespace stats
}  // namespace rxmet
