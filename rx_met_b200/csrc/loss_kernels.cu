// Mean-squared-error loss of a training step and its gradient with respect to the output, in one pass over
// the output and the target: grad = (out - target) * (2 / n), loss = sum (out - target)^2 / n.
//
// HBM-bound: 8 bytes read and 4 written per element, against four eager passes (difference, square, mean, scaled
// copy).  The gradient is bit-identical to the eager expressions (one subtraction and one multiplication by the
// float32 value of 2 / n); the loss is a float sum in a fixed order (per-CTA partials, then one CTA in double).
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>

#include "common.h"
#include "rxmet_b200.h"

namespace rxmet {
namespace {

constexpr int kLossThreads = 256;
constexpr int kLossCtasPerSm = 8;

__global__ void __launch_bounds__(kLossThreads) mseLossGrad(const float *__restrict__ out, const float *__restrict__ target,
                                                            uint64_t count, float factor, int vector,
                                                            float *__restrict__ grad, float *__restrict__ partial) {
    float acc = 0.0f;
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kLossThreads;
    const uint64_t first = static_cast<uint64_t>(blockIdx.x) * kLossThreads + threadIdx.x;
    if (vector) {
        const float4 *o4 = reinterpret_cast<const float4 *>(out);
        const float4 *t4 = reinterpret_cast<const float4 *>(target);
        float4 *g4 = reinterpret_cast<float4 *>(grad);
#pragma unroll 2
        for (uint64_t v = first; v < count / 4; v += stride) {
            const float4 a = __ldcs(o4 + v), b = __ldcs(t4 + v);
            const float d0 = __fsub_rn(a.x, b.x), d1 = __fsub_rn(a.y, b.y), d2 = __fsub_rn(a.z, b.z), d3 = __fsub_rn(a.w, b.w);
            acc += d0 * d0 + d1 * d1 + d2 * d2 + d3 * d3;
            g4[v] = make_float4(__fmul_rn(d0, factor), __fmul_rn(d1, factor), __fmul_rn(d2, factor), __fmul_rn(d3, factor));
        }
        for (uint64_t i = (count / 4) * 4 + first; i < count; i += stride) {
            const float d = __fsub_rn(out[i], target[i]);
            acc += d * d;
            grad[i] = __fmul_rn(d, factor);
        }
    } else {
        for (uint64_t i = first; i < count; i += stride) {
            const float d = __fsub_rn(out[i], target[i]);
            acc += d * d;
            grad[i] = __fmul_rn(d, factor);
        }
    }
    __shared__ float part[kLossThreads / 32];
    for (int d = 16; d > 0; d >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, d);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.0f;
        for (int w = 0; w < kLossThreads / 32; ++w) total += part[w];
        partial[blockIdx.x] = total;
    }
}

__global__ void __launch_bounds__(256) mseLossFinish(const float *__restrict__ partial, int parts, double count, float *loss) {
    double acc = 0.0;
    for (int i = threadIdx.x; i < parts; i += blockDim.x) acc += static_cast<double>(partial[i]);
    __shared__ double part[8];
    for (int d = 16; d > 0; d >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, d);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        double total = 0.0;
        for (int w = 0; w < 8; ++w) total += part[w];
        *loss = static_cast<float>(total / count);
    }
}

constexpr int kLossMaxCtas = 2048;   // the workspace holds one float per CTA
int lossGrid() { return std::min(currentDevice().sms * kLossCtasPerSm, kLossMaxCtas); }

}  // namespace
}  // namespace rxmet

using namespace rxmet;

extern "C" {

size_t rxmet_mse_loss_workspace_bytes(void) { return static_cast<size_t>(kLossMaxCtas) * sizeof(float); }

int rxmet_mse_loss_grad(const float *out_dev, const float *target_dev, uint64_t count, float *grad_dev, float *loss_dev,
                        void *workspace_dev, size_t workspace_bytes, void *stream) {
    return guarded([&] {
        RXMET_REQUIRE(count > 0, "mse loss: empty tensors");
        RXMET_REQUIRE(out_dev && target_dev && grad_dev && loss_dev, "mse loss: null tensor");
        const int grid = static_cast<int>(std::min<uint64_t>(static_cast<uint64_t>(lossGrid()), (count + kLossThreads - 1) / kLossThreads));
        RXMET_REQUIRE(workspace_dev && workspace_bytes >= static_cast<size_t>(grid) * sizeof(float),
                      "mse loss: workspace of %zu bytes needed", static_cast<size_t>(kLossMaxCtas) * sizeof(float));
        const bool vector = ((reinterpret_cast<uintptr_t>(out_dev) | reinterpret_cast<uintptr_t>(target_dev) |
                              reinterpret_cast<uintptr_t>(grad_dev)) & 15) == 0;
        const float factor = static_cast<float>(2.0 / static_cast<double>(count));
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        float *partial = static_cast<float *>(workspace_dev);
        mseLossGrad<<<grid, kLossThreads, 0, st>>>(out_dev, target_dev, count, factor, vector ? 1 : 0, grad_dev, partial);
        afterLaunch("mseLossGrad");
        mseLossFinish<<<1, 256, 0, st>>>(partial, grid, static_cast<double>(count), loss_dev);
        afterLaunch("mseLossFinish");
    });
}

}  // extern "C"
