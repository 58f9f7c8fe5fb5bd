// W8 / A16 forward of the QuantGRU integer carrier on byte planes (gru_forward_wide.cu).
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

#include "common.h"
#include "gru_params.h"

namespace rxmet {
namespace gru {

// Everything the shared front of the forward has prepared: one code per element for the weights (int8,
// [K padded][3H]), x and h0 (int16), the zero-point compensation and bias terms of both linear stages.
struct WideCall {
    int T, B, I, H;
    const int8_t *wCodes, *rCodes;      // [iPad][3H], [hPad][3H]
    int iPad, hPad;
    const int16_t *xCodes, *h0Codes;    // [T*B][iPad], [B][hPad]
    const int64_t *compX, *biasX, *compH, *biasH;
    const Rescale *gemmX, *gemmH;
    int16_t *ihCodes;                   // [T*B][3H] workspace
    float *h, *v;
    int32_t *hq, *vq;                   // optional
    uint8_t *maskIh, *maskHh, *maskGateIn, *maskGateOut, *maskH;  // optional keep flags
};

// Weight grids of at most 8 bits, x / h grids of 9..16 bits, linear grids of at most 16 bits, H <= 512.
bool forwardWideTakes(const Exec &exec, int I, int H);
size_t forwardWideExtraBytes(int T, int B, int I, int H);
void forwardWide(const WideCall &call, const Exec &exec, Workspace &workspace, cudaStream_t stream);

}  // namespace gru
}  // namespace rxmet
