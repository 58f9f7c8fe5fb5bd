// Tensor-core weight-gradient GEMM shared by the GRU and LSTM backward passes.
//
// partial[s][m][n] = sum over the s-th chunk of the K rows of A[k][m] * B[k][n], for m < M, and
// partial[s][M][n] = the column sums of B (a row of ones appended to A), i.e. the bias gradient.
// A holds small integers (activation codes minus their zero point, magnitude at most 256), which
// bf16 represents exactly; B (fp32 gradients) is split into three bf16 terms that together carry
// all 24 significand bits, so every product is exact and only the fp32 accumulation rounds.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

namespace rxmet {
namespace wgrad {

struct Problem {
    const int32_t *aCodes = nullptr;  // [K][M] integer codes, or
    const float *aFloat = nullptr;    // [K][M] floats: the integer is rint(value * aInvScale) - aFloatZero
    float aInvScale = 1.0f;
    float aFloatZero = 0.0f;
    int32_t aZero = 0;                // zero point of aCodes
    int M = 0;                        // real rows (multiple of 4, at most 143); row M is the ones row
    const float *B = nullptr;         // [K][N] gradients, N a multiple of 4
    float *partial = nullptr;         // [splits][M+1][N]
};

// Number of K splits for a problem with N output columns on a device with `sms` SMs; chunkK
// receives the rows per split (a multiple of the kernel's K tile).
int plan(int K, int N, int sms, int *chunkK);
void launch(const Problem &problem, int K, int N, int chunkK, int splits, cudaStream_t stream);

}  // namespace wgrad
}  // namespace rxmet
