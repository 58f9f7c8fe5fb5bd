// Host entry of the float GRU forward and of the calibration forward.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>

#include "gru_params.h"

namespace rxmet {
namespace gru {

// All pointers are device pointers.  stats, when set, receives the packed
// statistics: [mins | maxs], each half = 17 scalar slots (indexed by
// quantization point; the W/R/bw/br slots stay at their initial value)
// followed by the per-channel ranges of W, R, bw, br (3*H each).
struct ForwardFloatCall {
    int T = 0, B = 0, I = 0, H = 0;
    const float *W = nullptr, *R = nullptr, *bw = nullptr, *br = nullptr, *x = nullptr, *h0 = nullptr;
    float *h = nullptr, *v = nullptr;
    float *stats = nullptr;
    // optional per-step tensors for the histogram calibration, each [T,B,3H]:
    // W x + bw; R h + br; (z, r, n) pre-activations; (r*(Rh)_n, (1-z)*n, z*h_old)
    float *traceWx = nullptr, *traceRh = nullptr, *tracePre = nullptr, *traceMul = nullptr;
};

size_t statsFloats(int H);
size_t forwardFloatWorkspaceBytes(int T, int B, int I, int H);
void forwardFloat(const ForwardFloatCall &call, void *workspace, size_t workspaceBytes, cudaStream_t stream);
// Scratch of the histogram calibration forward (float forward + four [T,B,3H] traces + bin counters).
size_t histCalibrationWorkspaceBytes(int T, int B, int I, int H, int bins);

}  // namespace gru
}  // namespace rxmet
