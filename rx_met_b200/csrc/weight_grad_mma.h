// Tensor-core weight-gradient GEMM shared by the GRU and LSTM backward passes.
//
// partial[s][m][n] = sum over the s-th chunk of the K rows of A[k][m] * B[k][n], for m < M, and
// partial[s][M][n] = the column sums of B over the same rows, i.e. the bias gradient.
// A holds small integers (activation codes minus their zero point), which bf16 represents exactly:
// magnitude at most 256 as one term, or - for 16-bit activation grids - up to 2^17 as the two terms
// 256 * floor(a / 256) and a mod 256; B (fp32 gradients) is split into three bf16 terms that together
// carry all 24 significand bits, so every product is exact and only the fp32 accumulation rounds.
// Problems with more than 128 rows are cut into slabs of 128 rows that share one launch.
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
    // Slabs (tcgen05 kernel only; the defaults describe a whole problem of at most 128 rows).  A slab covers
    // rows [rowBase, rowBase + M) of a problem of totalRows - 1 real rows: aCodes / aFloat point at its first
    // column, consecutive K rows lie `lda` elements apart, and its accumulator rows land at row rowBase of the
    // [splits][totalRows][N] partial array; the slab with writeBias set also writes row totalRows - 1.
    int lda = 0;                      // 0 = M
    int rowBase = 0;
    int totalRows = 0;                // 0 = M + 1
    int writeBias = 1;
    int wideCodes = 0;                // 1: |code - zero point| may exceed 256 (two A terms)
};

constexpr int kMaxSlabs = 12;
struct ProblemSet {
    Problem slab[kMaxSlabs];
    int count = 0;
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

// The warp-specialised tcgen05 kernel (weight_grad_stream_umma.cu): both problems of a pair with at most 128 rows
// (a multiple of 8) each, whole arrays (no slabs), 8-bit codes, N a multiple of 128 or 192 but not of 256.  Returns
// false without launching when it does not take the pair.
bool launchPairStreamed(const Problem &a, const Problem &b, int K, int N, int chunkK, int splits, cudaStream_t stream);

// The tcgen05 kernel (weight_grad_umma.cu).
bool tensorMemoryPath(int M, int N);
int planTensorMemory(int K, int N, int sms, int *chunkK, int slabs = 1);
void launchTensorMemory(const Problem &problem, const Problem *other, int K, int N, int chunkK, int splits,
                        cudaStream_t stream);
// Any number of rows: cuts `a` and `b` (either may have M = 0) into 128-row slabs, plans one K split for
// all of them and runs them in ONE launch.  wide = two-term A operands for 16-bit codes.  Returns the
// number of splits (the partial arrays hold [splits][M + 1][N]); slabsOf(M) slabs per problem.
bool slabPathTakes(int Ma, int Mb, int N);
int slabSplits(int K, int Ma, int Mb, int N, int sms, int *chunkK);
// Upper bound of slabSplits over every device, for sizing the partial arrays.
int slabSplitBound(int Ma, int Mb, int N);
void launchSlabs(const Problem &a, const Problem &b, int K, int N, int chunkK, int splits, bool wide, cudaStream_t stream);

}  // namespace wgrad
}  // namespace rxmet
