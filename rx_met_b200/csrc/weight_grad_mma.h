// Tensor-core weight-gradient GEMM shared by the GRU and LSTM backward passes.
//
// partial[s][m][n] = sum over the s-th chunk of the K rows of A[k][m] * B[k][n], for m < M, and
// partial[s][M][n] = the column sums of B over the same rows, i.e. the bias gradient.
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
    int *status = nullptr;            // device word, set to 1 when a bounded wait of the kernel gave up
};

// How a problem is cut: K splits of chunkK rows each (a multiple of the kernel's K tile), and
// which kernel runs it.  The tcgen05 kernel (accumulators in tensor memory) takes problems with
// at most 128 rows whose column count is a multiple of 128, 192 or 256; the others run on the
// mma.sync kernel.  Setting RXMET_WGRAD_MMA_SYNC in the environment forces the latter.
struct Plan {
    int splits = 0;
    int chunkK = 0;
    bool tensorMemory = false;
};
Plan plan(int K, int M, int N, int sms);
// Upper bound of plan(...).splits over every device, for sizing the partial buffers.
int splitBound(int K, int M, int N);
void launch(const Problem &problem, int K, int N, const Plan &plan, cudaStream_t stream);
// Two problems over the same K rows and N columns (the input and the recurrent weights of a step).
// When both take the tcgen05 kernel with the same split they share ONE launch, the larger problem's
// CTAs scheduled first; otherwise two launches.
void launchPair(const Problem &a, const Plan &planA, const Problem &b, const Plan &planB, int K, int N, cudaStream_t stream);

// The tcgen05 kernel (weight_grad_umma.cu).
bool tensorMemoryPath(int M, int N);
int planTensorMemory(int K, int N, int sms, int *chunkK);
void launchTensorMemory(const Problem &problem, const Problem *other, int K, int N, int chunkK, int splits,
                        cudaStream_t stream);

}  // namespace wgrad
}  // namespace rxmet
