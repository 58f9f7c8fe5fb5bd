// AIMET native quantize-dequantize, fixed-point quantize, min/max and PDF histogram kernels.
//
// All of these are HBM-bound elementwise or reduction passes; they are written for bandwidth:
// 128-bit loads and stores where alignment allows, grid-stride loops over a grid that is a
// multiple of the SM count, warp-shuffle + one-atomic-per-CTA reductions, CTA-private shared
// memory histograms.  Arithmetic follows the reference's CPU definitions to the bit
// (native/common/src/quantize_dequantize.hpp:36-46, trim_functions.cpp:143-167,
// math_functions.cpp:355-412); the reference's CUDA build compiles the same expressions with
// fast-math division for the fixed-point path, which this code deliberately does not.
#include <cuda_runtime.h>

#include <algorithm>
#include <cfloat>
#include <cmath>
#include <cstdint>

#include <vector>

#include "common.h"
#include "rxmet_b200.h"

namespace rxmet {
namespace aimet {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxDims = 8;

int smCount() { return currentDevice().sms; }
int gridFor(uint64_t work, int perSm = 8) {
    const uint64_t blocks = (work + kThreads - 1) / kThreads;
    return static_cast<int>(std::max<uint64_t>(1, std::min<uint64_t>(blocks, static_cast<uint64_t>(smCount()) * perSm)));
}

// counter-based uniform in [0,1): one hash per element, reproducible for a given seed
__device__ __forceinline__ float uniform01(uint64_t seed, uint64_t i) {
    uint64_t z = seed + 0x9E3779B97F4A7C15ull * (i + 1);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return static_cast<float>(z >> 40) * (1.0f / 16777216.0f);
}

template <class T> struct Math;
template <> struct Math<float> {
    static __device__ __forceinline__ float recip(float s) { return __fdiv_rn(1.0f, s); }
    static __device__ __forceinline__ float clampTo(float v, float lo, float hi) { return fmaxf(fminf(v, hi), lo); }
    static __device__ __forceinline__ float rne(float v) { return nearbyintf(v); }
    static __device__ __forceinline__ float flr(float v) { return floorf(v); }
    static __device__ __forceinline__ float away(float v) { return roundf(v); }
    static __device__ __forceinline__ float div(float a, float b) { return __fdiv_rn(a, b); }
};
template <> struct Math<double> {
    static __device__ __forceinline__ double recip(double s) { return __ddiv_rn(1.0, s); }
    static __device__ __forceinline__ double clampTo(double v, double lo, double hi) { return fmax(fmin(v, hi), lo); }
    static __device__ __forceinline__ double rne(double v) { return nearbyint(v); }
    static __device__ __forceinline__ double flr(double v) { return floor(v); }
    static __device__ __forceinline__ double away(double v) { return round(v); }
    static __device__ __forceinline__ double div(double a, double b) { return __ddiv_rn(a, b); }
};

// quantize_dequantize.hpp:36-46 ; invScale is the rounded reciprocal, computed once per grid point
template <class T>
__device__ __forceinline__ T qdqValue(T v, T lo, T hi, T scale, T invScale, bool stochastic, T noise) {
    if (v != v) return v;
    const T scaled = Math<T>::clampTo(v, lo, hi) * invScale;
    const T rounded = stochastic ? Math<T>::flr(scaled + noise) : Math<T>::rne(scaled);
    return rounded * scale;
}

template <class T> struct Vec;
template <> struct Vec<float> { using type = float4; static constexpr int n = 4; };
template <> struct Vec<double> { using type = double2; static constexpr int n = 2; };

// Per-tensor QDQ: 16-byte vectors over the aligned body, scalars for head and tail.
template <class T>
__global__ void __launch_bounds__(kThreads) qdqTensor(const T *__restrict__ in, uint64_t n, T lo, T hi, T scale,
                                                      int stochastic, uint64_t seed, T *__restrict__ out) {
    using V = typename Vec<T>::type;
    constexpr int W = Vec<T>::n;
    const T inv = Math<T>::recip(scale);
    const uint64_t tid = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x;
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    auto one = [&](uint64_t i) {
        out[i] = qdqValue<T>(in[i], lo, hi, scale, inv, stochastic != 0, stochastic ? static_cast<T>(uniform01(seed, i)) : T(0));
    };
    const bool aligned = ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0;
    if (!aligned) {
        for (uint64_t i = tid; i < n; i += stride) one(i);
        return;
    }
    const uint64_t nv = n / W;
    const V *in4 = reinterpret_cast<const V *>(in);
    V *out4 = reinterpret_cast<V *>(out);
    for (uint64_t v = tid; v < nv; v += stride) {
        V q = in4[v];
        T *e = reinterpret_cast<T *>(&q);
#pragma unroll
        for (int k = 0; k < W; ++k)
            e[k] = qdqValue<T>(e[k], lo, hi, scale, inv, stochastic != 0,
                               stochastic ? static_cast<T>(uniform01(seed, v * W + k)) : T(0));
        out4[v] = q;
    }
    for (uint64_t i = nv * W + tid; i < n; i += stride) one(i);
}

// trim_functions.cu:75-86
template <class T>
__global__ void __launch_bounds__(kThreads) qdqPerChannel(const T *__restrict__ in, int channels, int64_t n,
                                                          int64_t perChannel, const T *__restrict__ lo,
                                                          const T *__restrict__ hi, const T *__restrict__ delta,
                                                          T *__restrict__ out) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n; i += stride) {
        const int c = static_cast<int>((i / perChannel) % channels);
        const T s = delta[c];
        out[i] = qdqValue<T>(in[i], lo[c], hi[c], s, Math<T>::recip(s), false, T(0));
    }
}

struct BroadcastDims {
    int nd;
    int64_t inStride[kMaxDims];
    int64_t encStride[kMaxDims];
};

// trim_functions.cu:90-116
template <class T>
__global__ void __launch_bounds__(kThreads) qdqBroadcast(const T *__restrict__ in, T *__restrict__ out, int64_t n,
                                                         const BroadcastDims dims, const T *__restrict__ lo,
                                                         const T *__restrict__ hi, const T *__restrict__ delta) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n; i += stride) {
        int64_t e = 0, rem = i;
        for (int d = 0; d < dims.nd; ++d) {
            const int64_t idx = rem / dims.inStride[d];
            rem -= idx * dims.inStride[d];
            e += dims.encStride[d] * idx;
        }
        const T s = delta[e];
        out[i] = qdqValue<T>(in[i], lo[e], hi[e], s, Math<T>::recip(s), false, T(0));
    }
}

// trim_functions.cuh:122-149 and trim_functions.cu:60-73
template <class T>
__global__ void __launch_bounds__(kThreads) toFxp(const T *__restrict__ in, uint64_t n, T lo, T hi, T delta, T offset,
                                                  T shift, T *__restrict__ out) {
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t i = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x; i < n; i += stride) {
        T v = Math<T>::clampTo(in[i], lo, hi);
        v = Math<T>::div(v, delta) - offset;
        out[i] = Math<T>::away(v) - shift;
    }
}

// ---- min / max ------------------------------------------------------------------
template <class T>
struct Extremes {
    T lo, hi;
    __device__ __forceinline__ void see(T v) {  // NaN never wins (math_functions.cpp:355-375)
        lo = (v < lo) ? v : lo;
        hi = (hi < v) ? v : hi;
    }
    __device__ __forceinline__ void merge(const Extremes &o) {
        lo = (o.lo < lo) ? o.lo : lo;
        hi = (hi < o.hi) ? o.hi : hi;
    }
};
template <class T> __device__ __forceinline__ T posInf();
template <> __device__ __forceinline__ float posInf<float>() { return __int_as_float(0x7f800000); }
template <> __device__ __forceinline__ double posInf<double>() { return __longlong_as_double(0x7ff0000000000000ll); }

template <class T>
__device__ __forceinline__ Extremes<T> blockReduce(Extremes<T> m, Extremes<T> *scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Extremes<T> other{__shfl_xor_sync(0xffffffffu, m.lo, o), __shfl_xor_sync(0xffffffffu, m.hi, o)};
        m.merge(other);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) scratch[warp] = m;
    __syncthreads();
    if (warp == 0) {
        m = lane < (blockDim.x >> 5) ? scratch[lane] : Extremes<T>{posInf<T>(), -posInf<T>()};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            Extremes<T> other{__shfl_xor_sync(0xffffffffu, m.lo, o), __shfl_xor_sync(0xffffffffu, m.hi, o)};
            m.merge(other);
        }
    }
    __syncthreads();
    return m;  // valid in warp 0
}

// Stage 1 of the whole-tensor reduction: one (min, max) pair per CTA.
template <class T>
__global__ void __launch_bounds__(kThreads) minMaxPartial(const T *__restrict__ x, uint64_t n, T *__restrict__ partial) {
    using V = typename Vec<T>::type;
    constexpr int W = Vec<T>::n;
    __shared__ Extremes<T> scratch[kThreads / 32];
    Extremes<T> m{posInf<T>(), -posInf<T>()};
    const uint64_t tid = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x;
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    if ((reinterpret_cast<uintptr_t>(x) & 15u) == 0) {
        const V *x4 = reinterpret_cast<const V *>(x);
        const uint64_t nv = n / W;
        for (uint64_t v = tid; v < nv; v += stride) {
            const V q = x4[v];
            const T *e = reinterpret_cast<const T *>(&q);
#pragma unroll
            for (int k = 0; k < W; ++k) m.see(e[k]);
        }
        for (uint64_t i = nv * W + tid; i < n; i += stride) m.see(x[i]);
    } else {
        for (uint64_t i = tid; i < n; i += stride) m.see(x[i]);
    }
    m = blockReduce<T>(m, scratch);
    if (threadIdx.x == 0) {
        partial[2 * blockIdx.x] = m.lo;
        partial[2 * blockIdx.x + 1] = m.hi;
    }
}

template <class T>
__global__ void __launch_bounds__(kThreads) minMaxFinal(const T *__restrict__ partial, int count, T *mins, T *maxs) {
    __shared__ Extremes<T> scratch[kThreads / 32];
    Extremes<T> m{posInf<T>(), -posInf<T>()};
    for (int i = threadIdx.x; i < count; i += blockDim.x) {
        m.lo = (partial[2 * i] < m.lo) ? partial[2 * i] : m.lo;
        m.hi = (m.hi < partial[2 * i + 1]) ? partial[2 * i + 1] : m.hi;
    }
    m = blockReduce<T>(m, scratch);
    if (threadIdx.x == 0) {
        mins[0] = m.lo;
        maxs[0] = m.hi;
    }
}

// Segmented form (math_functions.cu:81-139): one CTA per block of `blockSize` elements.
template <class T>
__global__ void __launch_bounds__(kThreads) minMaxBlocks(const T *__restrict__ x, uint64_t blockSize, uint64_t blocks,
                                                         T *__restrict__ mins, T *__restrict__ maxs) {
    __shared__ Extremes<T> scratch[kThreads / 32];
    for (uint64_t b = blockIdx.x; b < blocks; b += gridDim.x) {
        Extremes<T> m{posInf<T>(), -posInf<T>()};
        const T *seg = x + b * blockSize;
        for (uint64_t i = threadIdx.x; i < blockSize; i += blockDim.x) m.see(seg[i]);
        m = blockReduce<T>(m, scratch);
        if (threadIdx.x == 0) {
            mins[b] = m.lo;
            maxs[b] = m.hi;
        }
    }
}

// ---- PDF histogram (math_functions.cpp:395-412) ------------------------------------
constexpr int kPdfSize = 512 * 3;

template <class T>
__global__ void __launch_bounds__(kThreads) pdfHistogram(const T *__restrict__ x, uint64_t n, T invBucket, int pdfOffset,
                                                         uint32_t *__restrict__ hist) {
    // Four private copies per CTA, selected by lane: values cluster around the mode of the
    // distribution, and replication divides the shared-memory atomic contention on those buckets.
    constexpr int kCopies = 4;
    __shared__ uint32_t local[kCopies][kPdfSize];
    for (int i = threadIdx.x; i < kCopies * kPdfSize; i += blockDim.x) (&local[0][0])[i] = 0;
    __syncthreads();
    uint32_t *mine = local[threadIdx.x & (kCopies - 1)];
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    auto count = [&](T v) {
        const T slot = Math<T>::flr(v * invBucket) - static_cast<T>(pdfOffset);
        if (slot >= T(0) && slot < static_cast<T>(kPdfSize)) atomicAdd(&mine[static_cast<int>(slot)], 1u);
    };
    using V = typename Vec<T>::type;
    constexpr int W = Vec<T>::n;
    const uint64_t tid = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x;
    if ((reinterpret_cast<uintptr_t>(x) & 15u) == 0) {
        const V *x4 = reinterpret_cast<const V *>(x);
        const uint64_t nv = n / W;
        for (uint64_t v = tid; v < nv; v += stride) {
            const V q = x4[v];
            const T *e = reinterpret_cast<const T *>(&q);
#pragma unroll
            for (int k = 0; k < W; ++k) count(e[k]);
        }
        for (uint64_t i = nv * W + tid; i < n; i += stride) count(x[i]);
    } else {
        for (uint64_t i = tid; i < n; i += stride) count(x[i]);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < kPdfSize; i += blockDim.x) {
        const uint32_t total = local[0][i] + local[1][i] + local[2][i] + local[3][i];
        if (total) atomicAdd(&hist[i], total);
    }
}

__global__ void zeroWords(uint32_t *p, int n) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) p[i] = 0;
}

template <class F>
void dispatch(int dtype, F &&f) {
    if (dtype == 0) f(float{});
    else if (dtype == 1) f(double{});
    else fail(RXMET_ERR_INVALID_ARGUMENT, "dtype must be 0 (float32) or 1 (float64), got %d", dtype);
}

}  // namespace
}  // namespace aimet
}  // namespace rxmet

using namespace rxmet;
using namespace rxmet::aimet;

extern "C" {

int rxmet_aimet_pdf_size(void) { return kPdfSize; }

int rxmet_aimet_qdq(const void *in_dev, uint64_t count, int dtype, double enc_min, double enc_max, double delta,
                    int stochastic, uint64_t seed, void *out_dev, void *stream) {
    return guarded([&] {
        if (count == 0) return;
        RXMET_REQUIRE(in_dev && out_dev, "qdq: null tensor");
        RXMET_REQUIRE(delta > 0.0, "qdq: delta must be > 0");
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        dispatch(dtype, [&](auto tag) {
            using T = decltype(tag);
            KernelTimer timer__("qdqTensor", st);
            qdqTensor<T><<<gridFor(count / Vec<T>::n + 1), kThreads, 0, st>>>(
                static_cast<const T *>(in_dev), count, static_cast<T>(enc_min), static_cast<T>(enc_max),
                static_cast<T>(delta), stochastic, seed, static_cast<T *>(out_dev));
        });
        afterLaunch("qdqTensor");
    });
}

int rxmet_aimet_qdq_per_channel(const void *in_dev, int num_channels, int64_t num_elements,
                                int64_t elements_per_channel, int dtype, const void *min_dev, const void *max_dev,
                                const void *delta_dev, void *out_dev, void *stream) {
    return guarded([&] {
        if (num_elements == 0) return;
        RXMET_REQUIRE(in_dev && out_dev && min_dev && max_dev && delta_dev, "qdq_per_channel: null pointer");
        RXMET_REQUIRE(num_channels > 0 && elements_per_channel > 0 && num_elements > 0, "qdq_per_channel: bad sizes");
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        dispatch(dtype, [&](auto tag) {
            using T = decltype(tag);
            KernelTimer timer__("qdqPerChannel", st);
            qdqPerChannel<T><<<gridFor(num_elements), kThreads, 0, st>>>(
                static_cast<const T *>(in_dev), num_channels, num_elements, elements_per_channel,
                static_cast<const T *>(min_dev), static_cast<const T *>(max_dev), static_cast<const T *>(delta_dev),
                static_cast<T *>(out_dev));
        });
        afterLaunch("qdqPerChannel");
    });
}

int rxmet_aimet_qdq_broadcast(const void *in_dev, void *out_dev, int64_t num_elements, int num_dims,
                              const int64_t *input_strides, const int64_t *encoding_strides, int dtype,
                              const void *min_dev, const void *max_dev, const void *delta_dev, void *stream) {
    return guarded([&] {
        if (num_elements == 0) return;
        RXMET_REQUIRE(in_dev && out_dev && min_dev && max_dev && delta_dev && input_strides && encoding_strides,
                      "qdq_broadcast: null pointer");
        RXMET_REQUIRE(num_dims >= 1 && num_dims <= kMaxDims, "qdq_broadcast: 1..%d dimensions supported", kMaxDims);
        BroadcastDims dims{};
        dims.nd = num_dims;
        for (int d = 0; d < num_dims; ++d) {
            RXMET_REQUIRE(input_strides[d] > 0, "qdq_broadcast: input strides must be positive");
            dims.inStride[d] = input_strides[d];
            dims.encStride[d] = encoding_strides[d];
        }
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        dispatch(dtype, [&](auto tag) {
            using T = decltype(tag);
            KernelTimer timer__("qdqBroadcast", st);
            qdqBroadcast<T><<<gridFor(num_elements), kThreads, 0, st>>>(
                static_cast<const T *>(in_dev), static_cast<T *>(out_dev), num_elements, dims,
                static_cast<const T *>(min_dev), static_cast<const T *>(max_dev), static_cast<const T *>(delta_dev));
        });
        afterLaunch("qdqBroadcast");
    });
}

int rxmet_aimet_quantize_to_fxp(const void *in_dev, uint64_t count, int dtype, double enc_min, double enc_max,
                                double delta, double offset, int bitwidth, int shift_to_signed, void *out_dev,
                                void *stream) {
    return guarded([&] {
        if (count == 0) return;
        RXMET_REQUIRE(in_dev && out_dev, "quantize_to_fxp: null tensor");
        RXMET_REQUIRE(bitwidth >= 1 && bitwidth <= 32, "quantize_to_fxp: bitwidth 1..32");
        const double shift = shift_to_signed ? std::pow(2.0, bitwidth - 1) : 0.0;
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        dispatch(dtype, [&](auto tag) {
            using T = decltype(tag);
            KernelTimer timer__("toFxp", st);
            toFxp<T><<<gridFor(count), kThreads, 0, st>>>(static_cast<const T *>(in_dev), count, static_cast<T>(enc_min),
                                                          static_cast<T>(enc_max), static_cast<T>(delta),
                                                          static_cast<T>(offset), static_cast<T>(shift),
                                                          static_cast<T *>(out_dev));
        });
        afterLaunch("toFxp");
    });
}

size_t rxmet_aimet_minmax_workspace_bytes(void) { return sizeof(double) * 2 * 148 * 16 + 256; }

int rxmet_aimet_minmax(const void *data_dev, uint64_t count, uint64_t block_size, int dtype, void *min_out_dev,
                       void *max_out_dev, void *workspace_dev, size_t workspace_bytes, void *stream) {
    return guarded([&] {
        RXMET_REQUIRE(data_dev && min_out_dev && max_out_dev, "minmax: null pointer");
        RXMET_REQUIRE(count > 0 && block_size > 0 && block_size <= count, "minmax: need 0 < block_size <= count");
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        const uint64_t blocks = count / block_size;
        dispatch(dtype, [&](auto tag) {
            using T = decltype(tag);
            if (blocks == 1) {
                const int grid = gridFor(count / Vec<T>::n + 1, 4);
                if (workspace_dev == nullptr || workspace_bytes < sizeof(T) * 2 * grid)
                    fail(RXMET_ERR_WORKSPACE, "minmax: workspace too small: need %zu bytes", sizeof(T) * 2 * grid);
                {
                    KernelTimer timer__("minMaxPartial", st);
                    minMaxPartial<T><<<grid, kThreads, 0, st>>>(static_cast<const T *>(data_dev), block_size,
                                                               static_cast<T *>(workspace_dev));
                }
                afterLaunch("minMaxPartial");
                minMaxFinal<T><<<1, kThreads, 0, st>>>(static_cast<const T *>(workspace_dev), grid,
                                                      static_cast<T *>(min_out_dev), static_cast<T *>(max_out_dev));
                afterLaunch("minMaxFinal");
            } else {
                KernelTimer timer__("minMaxBlocks", st);
                const int grid = static_cast<int>(std::min<uint64_t>(blocks, static_cast<uint64_t>(smCount()) * 8));
                minMaxBlocks<T><<<grid, kThreads, 0, st>>>(static_cast<const T *>(data_dev), block_size, blocks,
                                                          static_cast<T *>(min_out_dev), static_cast<T *>(max_out_dev));
                afterLaunch("minMaxBlocks");
            }
        });
    });
}

int rxmet_aimet_histogram(const void *data_dev, uint64_t count, int dtype, double bucket_size, int pdf_offset,
                          uint32_t *histogram_dev, void *stream) {
    return guarded([&] {
        RXMET_REQUIRE(histogram_dev, "histogram: null output");
        RXMET_REQUIRE(bucket_size > 0.0, "histogram: bucket_size must be > 0");
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        zeroWords<<<6, kThreads, 0, st>>>(histogram_dev, kPdfSize);
        afterLaunch("zeroWords");
        if (count == 0) return;
        RXMET_REQUIRE(data_dev, "histogram: null tensor");
        dispatch(dtype, [&](auto tag) {
            using T = decltype(tag);
            KernelTimer timer__("pdfHistogram", st);
            pdfHistogram<T><<<gridFor(count / Vec<T>::n + 1, 4), kThreads, 0, st>>>(
                static_cast<const T *>(data_dev), count, static_cast<T>(1 / bucket_size), pdf_offset, histogram_dev);
        });
        afterLaunch("pdfHistogram");
    });
}

size_t rxmet_aimet_pdf_workspace_bytes(void) {
    return rxmet_aimet_minmax_workspace_bytes() + 256 + sizeof(uint32_t) * kPdfSize + 256;
}

int rxmet_aimet_pdf_update(rxmet_aimet_pdf *pdf, const float *data_dev, uint64_t count, int signed_values,
                           void *workspace_dev, size_t workspace_bytes, void *stream) {
    return guarded([&] {
        RXMET_REQUIRE(pdf != nullptr && data_dev != nullptr && count > 0, "pdf update: null pdf or empty tensor");
        RXMET_REQUIRE(workspace_dev != nullptr && workspace_bytes >= rxmet_aimet_pdf_workspace_bytes(),
                      "pdf update: workspace too small");
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        char *base = static_cast<char *>(workspace_dev);
        float *extremes = reinterpret_cast<float *>(base);
        uint32_t *histogram = reinterpret_cast<uint32_t *>(base + 256);
        void *scratch = base + 256 + alignUp(sizeof(uint32_t) * kPdfSize, 256);
        auto check = [](int rc) {
            if (rc != 0) fail(rc, "%s", std::string(rxmet_last_error()).c_str());
        };
        float host[2] = {1.0f, 1.0f};  // only the first batches need the extremes: they fix the range
        if (!pdf->initialized) {
            check(rxmet_aimet_minmax(data_dev, count, count, 0, extremes, extremes + 1, scratch,
                                     rxmet_aimet_minmax_workspace_bytes(), stream));
            RXMET_CUDA(cudaMemcpyAsync(host, extremes, sizeof(host), cudaMemcpyDeviceToHost, st));
            RXMET_CUDA(cudaStreamSynchronize(st));
        }
        double bucket = 0;
        int offset = 0, skip = 0;
        check(rxmet_aimet_pdf_plan(pdf, host[0], host[1], signed_values, &bucket, &offset, &skip));
        if (skip) return;
        check(rxmet_aimet_histogram(data_dev, count, 0, bucket, offset, histogram, stream));
        std::vector<uint32_t> counts(kPdfSize);
        RXMET_CUDA(cudaMemcpyAsync(counts.data(), histogram, sizeof(uint32_t) * kPdfSize, cudaMemcpyDeviceToHost, st));
        RXMET_CUDA(cudaStreamSynchronize(st));
        check(rxmet_aimet_pdf_commit(pdf, counts.data(), count));
    });
}

}  // extern "C"
