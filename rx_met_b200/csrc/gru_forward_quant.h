// Host entry of the quantized GRU forward (integer carrier).
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "gru_params.h"
#include "rxmet_b200.h"

namespace rxmet {
namespace gru {

// All pointers are device pointers; optional ones may be null.
struct ForwardQuantCall {
    int isTraining = 0;
    int T = 0, B = 0, I = 0, H = 0;
    const float *W = nullptr, *R = nullptr, *bw = nullptr, *br = nullptr;
    const float *x = nullptr;               // [T,B,I] float input, or
    const int32_t *x_codes_in = nullptr;    // [T,B,I] codes already on the x grid
    const float *h0 = nullptr;              // [B,H] float initial state, or
    const int32_t *h0_codes_in = nullptr;   // [B,H] codes already on the h grid (else zero point)
    float *h = nullptr;                     // [T+1,B,H] dequantized
    float *v = nullptr;                     // [T,B,4H] dequantized
    int32_t *W_q = nullptr, *R_q = nullptr, *bw_q = nullptr, *br_q = nullptr, *x_q = nullptr;
    int32_t *h_q = nullptr, *v_q = nullptr;
    const rxmet_gru_masks *masks = nullptr;
    uint16_t *stepFlags = nullptr;          // optional [T,B,H]: the 13 per-step keep flags of an element packed into 16 bits
    const rxmet_gru_quant_params *fpCarrier = nullptr;   // set: run the FP32 carrier with these (raw) scales
};

// Whether forwardQuant can write stepFlags for these parameters and sizes (the register-resident 8-bit path).
bool packedFlagsSupported(const Exec &exec, int B, int I, int H);

// Page-locked host copy of the per-channel block of `exec`, 12 arrays of 3H 32-bit words: effective
// scales of W, R, bw, br (floats), then the Rescale pairs gemm_x, bias_x, gemm_h, bias_h.  Built on
// first use and owned by `exec`.
const int32_t *pinnedChannelBlock(const Exec &exec, cudaStream_t stream);

size_t forwardQuantWorkspaceBytes(int T, int B, int I, int H);
void forwardQuant(const ForwardQuantCall &call, const Exec &exec, void *workspace, size_t workspaceBytes,
                  cudaStream_t stream);

}  // namespace gru
}  // namespace rxmet
