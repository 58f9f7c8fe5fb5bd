// Input projection of the 8-bit QuantGRU path as a tcgen05 kind::i8 GEMM with the fused integer
// epilogue (input_proj_umma.cu).
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

#include "gru_device.cuh"

namespace rxmet {
namespace iproj {

struct Problem {
    const int32_t *x = nullptr;        // [rows][kWords] words of four signed 8-bit codes, rows back to back
    int rows = 0, kWords = 0, kPad = 0;  // kPad (bytes of k per row in shared memory) is filled in by launch()
    const int32_t *w = nullptr;        // [kWords][C] words of four signed 8-bit weight codes
    int C = 0;
    const int64_t *comp = nullptr;     // [C] zero-point compensation sum_k W * zp_x
    const int64_t *biasAcc = nullptr;  // [C] bias on the accumulator grid
    const gru::Rescale *rescale = nullptr;  // [C] accumulator -> output grid
    int32_t zpOut = 0, lo = 0, hi = 0;
    gru::PreRescale pre{};
    int16_t *out = nullptr;            // [rows][C]
    uint8_t *mask = nullptr;           // [rows][C] keep flags, optional
    int *status = nullptr;             // device word, set to 1 when a bounded wait of the kernel gave up
};

// H a multiple of 16, 3H a multiple of 64 .. 256, operands that fit one SM's shared memory and output
// pointers that take 16-byte stores.  RXMET_IPROJ_SIMT in the environment turns the path off.
bool eligible(int C, int H, int kWords, const void *x, const void *out, const void *mask);
void launch(const Problem &problem, int sms, cudaStream_t stream);

}  // namespace iproj
}  // namespace rxmet
