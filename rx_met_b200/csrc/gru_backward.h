// Host entry of the GRU backward (QAT and float).
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "gru_params.h"
#include "rxmet_b200.h"

namespace rxmet {
namespace gru {

// Device pointers.  Either the real-valued operands (W, R, x) or the saved
// integer codes (W_q, R_q, x_q together with exec) are given.
struct BackwardCall {
    int T = 0, B = 0, I = 0, H = 0;
    const float *W = nullptr, *R = nullptr, *x = nullptr;
    const int32_t *W_q = nullptr, *R_q = nullptr, *x_q = nullptr;
    const Exec *exec = nullptr;
    const float *dh_new = nullptr, *h = nullptr, *v = nullptr;
    const rxmet_gru_masks *masks = nullptr;
    const uint16_t *stepFlags = nullptr;    // optional [T,B,H]: packed per-step keep flags as the forward wrote them
    float *dx = nullptr, *dW = nullptr, *dR = nullptr, *dbw = nullptr, *dbr = nullptr, *dh0 = nullptr;
};

size_t backwardWorkspaceBytes(int T, int B, int I, int H);
void backward(const BackwardCall &call, void *workspace, size_t workspaceBytes, cudaStream_t stream);

}  // namespace gru
}  // namespace rxmet
