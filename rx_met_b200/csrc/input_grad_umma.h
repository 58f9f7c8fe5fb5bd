// Input gradient of a quantized linear stage on the tcgen05 tensor cores:
//
//   out[r][n] = keep[r][n] * sum_k (G[r][k] * kScale[k]) * code[k][n]
//
// G holds the fp32 gradients of the stage's outputs ([rows][K], K = gate channels), code the
// integer weight codes (magnitude at most 256, exact in bf16) and kScale their per-channel
// scales, folded into G so that the weight operand stays exact.  G * kScale is split into three
// bf16 terms that carry all 24 significand bits; only the fp32 accumulation rounds.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

namespace rxmet {
namespace igrad {

struct Problem {
    const float *G = nullptr;           // [rows][K]
    const float *kScale = nullptr;      // [K]
    const int32_t *codesNK = nullptr;   // [N][K] integer codes, or
    const float *codesKN = nullptr;     // [K][N] integer-valued floats
    int rows = 0, K = 0, N = 0;
    const uint8_t *mask = nullptr;      // [rows][N], optional
    int maskKeeps = 1;                  // 1: a nonzero byte keeps the gradient; 0: a nonzero byte drops it
    float *out = nullptr;               // [rows][N]
    int *status = nullptr;              // device word, set to 1 when a bounded wait of the kernel gave up
};

// K a multiple of 32 up to 512, N up to 64.  RXMET_IGRAD_SIMT in the environment turns the path off.
bool eligible(int K, int N);
void launch(const Problem &problem, int sms, cudaStream_t stream);

}  // namespace igrad
}  // namespace rxmet
