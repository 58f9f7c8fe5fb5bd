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
    int ldN = 0;                        // elements between rows of `out` and `mask` (0 = N); wider than N when the
                                        // problem is one 64-column slab of a larger output
    int ldCodesKN = 0;                  // elements between k rows of codesKN (0 = N)
    void *packed = nullptr;             // scratch of widePackedBytes(K, N) bytes, 16-byte aligned: with it, outputs wider
                                        // than 64 columns (up to 512) take the warp-specialised kernel that streams
                                        // both operands and keeps the whole [128][N] accumulator in tensor memory
};

// Resident-weight kernel: K a multiple of 64 up to 768; any N: more than 64 columns (32 when K > 512, where the
// weight operand of a wider slab no longer fits shared memory) run as column slabs that share one launch.
// Streaming kernel (Problem::packed given, 64 < N <= 512): any K that is a multiple of 32.
// RXMET_IGRAD_SIMT in the environment turns both off, RXMET_IGRAD_NARROW the streaming kernel.
bool eligible(int K, int N);
size_t widePackedBytes(int K, int N);   // 0 when the streaming kernel does not take N
void launch(const Problem &problem, int sms, cudaStream_t stream);

}  // namespace igrad
}  // namespace rxmet
