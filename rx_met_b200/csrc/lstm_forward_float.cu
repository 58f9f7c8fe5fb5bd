// Float LSTM forward, optionally with the calibration statistics of all 18 quantization points
// and the three product contributions reduced on the device.
//
// Launch plan (the reference runs T x (cuBLAS GEMM + pointwise) and, for calibration, one
// reduction per statistic, operators/quant-lstm/src/lstm/forward_float_cuda.cu and
// src/lstm/calibration_cuda.cu; what is observed is defined by src/lstm/calibration.cc:128-232):
//   transposeWeights   : weight_hh [4H,H] -> [H,4H] so that thread c streams its row coalesced
//   inputLinearFloat   : W_ih x + b_ih for all T*B rows
//   recurrentFloat     : ONE launch for all T steps; a CTA owns BT batch rows, keeps as many rows
//                        of the transposed recurrent weights in shared memory as fit and streams the
//                        rest from L2; statistics stay in registers until the last step.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>

#include "common.h"
#include "lstm_kernels.h"
#include "minmax_device.cuh"

namespace rxmet {
namespace lstm {
namespace {

using stats::MinMax;

__global__ void fillStats(float *stats, size_t half) {
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < 2 * half;
         i += static_cast<size_t>(gridDim.x) * blockDim.x)
        stats[i] = i < half ? FLT_MAX : -FLT_MAX;
}

__global__ void tensorMinMax(const float *__restrict__ x, size_t n, float *minSlot, float *maxSlot) {
    __shared__ float scratch[2 * 32];
    MinMax m[1];
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<size_t>(gridDim.x) * blockDim.x)
        m[0].see(x[i]);
    const int slot[1] = {0};
    stats::commit<1>(m, slot, minSlot, maxSlot, scratch);
}

// Per-row min/max of a [rows, cols] matrix (one row = one output channel).
__global__ void rowMinMax(const float *__restrict__ w, int rows, int cols, float *mins, float *maxs) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    MinMax m;
    for (int c = 0; c < cols; ++c) m.see(w[static_cast<size_t>(r) * cols + c]);
    mins[r] = m.lo;
    maxs[r] = m.hi;
}

__global__ void transposeWeights(const float *__restrict__ in, int rows, int cols, float *__restrict__ out) {
    __shared__ float tile[32][33];
    const int x = blockIdx.x * 32 + threadIdx.x, y0 = blockIdx.y * 32;
    for (int dy = threadIdx.y; dy < 32; dy += blockDim.y)
        if (x < cols && y0 + dy < rows) tile[dy][threadIdx.x] = in[static_cast<size_t>(y0 + dy) * cols + x];
    __syncthreads();
    const int ox = blockIdx.y * 32 + threadIdx.x, oy0 = blockIdx.x * 32;
    for (int dy = threadIdx.y; dy < 32; dy += blockDim.y)
        if (ox < rows && oy0 + dy < cols) out[static_cast<size_t>(oy0 + dy) * rows + ox] = tile[threadIdx.x][dy];
}

constexpr int kRowsPerBlock = 8;

// out[n, c] = b[c] + sum_k x[n,k] wT[k,c]
__global__ void inputLinearFloat(const float *__restrict__ x, int rows, int K, int C, const float *__restrict__ wT,
                                 const float *__restrict__ bias, float *__restrict__ out, float *__restrict__ traceOut,
                                 float *mins, float *maxs, int slot) {
    extern __shared__ float smemF[];
    float *xs = smemF;                           // [kRowsPerBlock][K]
    float *scratch = smemF + kRowsPerBlock * K;  // 2 * warps
    const int row0 = blockIdx.x * kRowsPerBlock, nRows = min(kRowsPerBlock, rows - row0);
    for (int i = threadIdx.x; i < kRowsPerBlock * K; i += blockDim.x) {
        const int r = i / K;
        xs[i] = r < nRows ? x[static_cast<size_t>(row0 + r) * K + (i % K)] : 0.0f;
    }
    __syncthreads();
    MinMax m[1];
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float acc[kRowsPerBlock];
        const float b = bias ? bias[c] : 0.0f;
#pragma unroll
        for (int r = 0; r < kRowsPerBlock; ++r) acc[r] = b;
        for (int k = 0; k < K; ++k) {
            const float w = wT[static_cast<size_t>(k) * C + c];
#pragma unroll
            for (int r = 0; r < kRowsPerBlock; ++r) acc[r] = fmaf(xs[r * K + k], w, acc[r]);
        }
#pragma unroll
        for (int r = 0; r < kRowsPerBlock; ++r)
            if (r < nRows) {
                const size_t o = static_cast<size_t>(row0 + r) * C + c;
                out[o] = acc[r];
                if (traceOut) traceOut[o] = acc[r];
                m[0].see(acc[r]);
            }
    }
    if (mins) {
        const int slots[1] = {slot};
        stats::commit<1>(m, slots, mins, maxs, scratch);
    }
}

struct FloatRecurrentArgs {
    int T, B, H, smemRows;
    const float *wT;    // [H][4H] transposed weight_hh
    const float *bias;  // [4H] or null
    const float *ih;    // [T][B][4H]
    const float *h0, *c0;
    float *output, *finalHidden, *finalCell;
    rxmet_lstm_trace tr;
    float *mins, *maxs;
};

__device__ __forceinline__ float sigmoidStable(float v) {
    if (v >= 0.0f) {
        const float e = expf(-v);
        return 1.0f / (1.0f + e);
    }
    const float e = expf(v);
    return e / (1.0f + e);
}

constexpr int kRecurrentStats = 15;

template <int BT>
__global__ void __launch_bounds__(512) recurrentFloat(const __grid_constant__ FloatRecurrentArgs a) {
    const int H = a.H, C = 4 * a.H;
    extern __shared__ float smemF[];
    float *hS = smemF;                               // [BT][H]
    float *hhS = hS + BT * H;                        // [BT][C]
    float *scratch = hhS + BT * C;                   // 2 * kRecurrentStats * 16
    float *wS = scratch + 2 * kRecurrentStats * 16;  // [smemRows][C]
    const int tid = threadIdx.x, nthreads = blockDim.x;
    const int b0 = blockIdx.x * BT, nb = min(BT, a.B - b0);
    for (int i = tid; i < a.smemRows * C; i += nthreads) wS[i] = a.wT[i];
    for (int i = tid; i < BT * H; i += nthreads) {
        const int b = i / H;
        hS[i] = (b < nb && a.h0) ? a.h0[static_cast<size_t>(b0 + b) * H + (i % H)] : 0.0f;
    }
    const int elems = nb * H;
    const bool hasElem = tid < elems;
    const int eb = hasElem ? tid / H : 0, ej = hasElem ? tid % H : 0;
    float cell = (hasElem && a.c0) ? a.c0[static_cast<size_t>(b0 + eb) * H + ej] : 0.0f;
    float hidden = 0.0f;
    // order: hh linear, 4 gate inputs, 4 gate outputs, cell, tanh(cell), hidden, f*c, i*g, o*tanh
    MinMax st[kRecurrentStats];
    __syncthreads();
    if (hasElem) {
        hidden = hS[eb * H + ej];
        st[11].see(hidden);  // the initial states are observed too (zeros when absent)
        st[9].see(cell);
    }
    const bool hasChannel = tid < C;
    const float bias = (hasChannel && a.bias) ? a.bias[tid] : 0.0f;
    for (int t = 0; t < a.T; ++t) {
        const size_t rowBase = static_cast<size_t>(t) * a.B + b0;
        if (hasChannel) {
            float acc[BT];
#pragma unroll
            for (int b = 0; b < BT; ++b) acc[b] = bias;
            for (int k = 0; k < a.smemRows; ++k) {
                const float w = wS[k * C + tid];
#pragma unroll
                for (int b = 0; b < BT; ++b) acc[b] = fmaf(hS[b * H + k], w, acc[b]);
            }
            for (int k = a.smemRows; k < H; ++k) {
                const float w = a.wT[static_cast<size_t>(k) * C + tid];
#pragma unroll
                for (int b = 0; b < BT; ++b) acc[b] = fmaf(hS[b * H + k], w, acc[b]);
            }
#pragma unroll
            for (int b = 0; b < BT; ++b) {
                hhS[b * C + tid] = acc[b];
                if (b < nb) {
                    st[0].see(acc[b]);
                    if (a.tr.weight_hh_linear) a.tr.weight_hh_linear[(rowBase + b) * C + tid] = acc[b];
                }
            }
        }
        __syncthreads();
        if (hasElem) {
            const size_t row = rowBase + eb;
            const float *ih = a.ih + row * C + ej;
            float pre[4], act[4];
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                pre[g] = ih[g * H] + hhS[eb * C + g * H + ej];
                act[g] = g == 2 ? tanhf(pre[g]) : sigmoidStable(pre[g]);
                st[1 + g].see(pre[g]);
                st[5 + g].see(act[g]);
                if (a.tr.gate_inputs) a.tr.gate_inputs[row * C + g * H + ej] = pre[g];
                if (a.tr.gate_outputs) a.tr.gate_outputs[row * C + g * H + ej] = act[g];
            }
            const float keepOld = act[1] * cell, writeNew = act[0] * act[2];
            cell = keepOld + writeNew;
            const float ct = tanhf(cell);
            hidden = act[3] * ct;
            st[9].see(cell); st[10].see(ct); st[11].see(hidden);
            st[12].see(keepOld); st[13].see(writeNew); st[14].see(hidden);
            const size_t so = row * H + ej;
            a.output[so] = hidden;
            if (a.tr.cell_states) a.tr.cell_states[so] = cell;
            if (a.tr.cell_tanh_outputs) a.tr.cell_tanh_outputs[so] = ct;
            if (a.tr.hidden_outputs) a.tr.hidden_outputs[so] = hidden;
        }
        __syncthreads();
        if (hasElem) hS[eb * H + ej] = hidden;
        __syncthreads();
    }
    if (hasElem) {
        const size_t o = static_cast<size_t>(b0 + eb) * H + ej;
        a.finalHidden[o] = hidden;
        a.finalCell[o] = cell;
    }
    if (a.mins) {
        const int slots[kRecurrentStats] = {
            RXMET_LSTM_WEIGHT_HH_LINEAR, RXMET_LSTM_INPUT_GATE_INPUT, RXMET_LSTM_FORGET_GATE_INPUT,
            RXMET_LSTM_CELL_GATE_INPUT, RXMET_LSTM_OUTPUT_GATE_INPUT, RXMET_LSTM_INPUT_GATE_OUTPUT,
            RXMET_LSTM_FORGET_GATE_OUTPUT, RXMET_LSTM_CELL_GATE_OUTPUT, RXMET_LSTM_OUTPUT_GATE_OUTPUT,
            RXMET_LSTM_CELL_STATE, RXMET_LSTM_CELL_TANH_OUTPUT, RXMET_LSTM_OUTPUT, kOps + 0, kOps + 1, kOps + 2};
        stats::commit<kRecurrentStats>(st, slots, a.mins, a.maxs, scratch);
    }
}

// ---- hidden sizes above 128 -------------------------------------------------------------------
//
// 4H no longer fits the one-thread-per-channel layout above.  Here thread (j, s) owns hidden unit j -
// all four gates - for RB batch rows of row group s, so the pointwise part needs no exchange between
// threads: per step one 16-byte load per k brings the four gate weights of (k, j) from L2 (weight_hh
// interleaved to [k][j][gate] once per call), the hidden state of the CTA's rows is double buffered
// in shared memory (one barrier per step), the cell state stays in registers.  The sums run in the
// same order (bias first, k ascending, one fused multiply-add per term) as in recurrentFloat.
__global__ void interleaveGates(const float *__restrict__ w, int H, float *__restrict__ out) {
    const size_t n = static_cast<size_t>(4) * H * H;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int g = static_cast<int>(i % 4), j = static_cast<int>((i / 4) % H), k = static_cast<int>(i / (4 * static_cast<size_t>(H)));
        out[i] = w[(static_cast<size_t>(g) * H + j) * H + k];
    }
}

struct FloatWideArgs {
    FloatRecurrentArgs base;  // wT is unused
    const float4 *w4;         // [H][H] float4: gates (i, f, g, o) of (k, j)
    int HP;
};

template <int RB>
__global__ void __launch_bounds__(512, 1) recurrentFloatWide(const __grid_constant__ FloatWideArgs wa) {
    const FloatRecurrentArgs &a = wa.base;
    const int H = a.H, C = 4 * a.H, HP = wa.HP;
    extern __shared__ __align__(16) float smemF[];
    const int tid = threadIdx.x, j = tid % HP, sg = tid / HP;
    const int BT = (blockDim.x / HP) * RB;
    const int HS = (H + 3) / 4 * 4;                       // row stride of the state buffers
    float *hS = smemF;                                    // [2][BT][HS]
    float *scratch = smemF + 2 * BT * HS;                 // 2 * kRecurrentStats * 16
    const bool active = j < H;
    const int ctaRow0 = blockIdx.x * BT, b0 = ctaRow0 + sg * RB;
    for (int i = tid; i < 2 * BT * HS; i += blockDim.x) hS[i] = 0.0f;
    __syncthreads();
    for (int i = tid; i < BT * H; i += blockDim.x) {
        const int r = i / H, k = i % H, b = ctaRow0 + r;
        if (b < a.B && a.h0) hS[r * HS + k] = a.h0[static_cast<size_t>(b) * H + k];
    }
    float cell[RB], hidden[RB];
    // order: hh linear, 4 gate inputs, 4 gate outputs, cell, tanh(cell), hidden, f*c, i*g, o*tanh
    MinMax st[kRecurrentStats];
    __syncthreads();
#pragma unroll
    for (int r = 0; r < RB; ++r) {
        const bool valid = active && b0 + r < a.B;
        cell[r] = (valid && a.c0) ? a.c0[static_cast<size_t>(b0 + r) * H + j] : 0.0f;
        hidden[r] = valid ? hS[(sg * RB + r) * HS + j] : 0.0f;
        if (valid) {
            st[11].see(hidden[r]);  // the initial states are observed too (zeros when absent)
            st[9].see(cell[r]);
        }
    }
    float bias[4];
#pragma unroll
    for (int g = 0; g < 4; ++g) bias[g] = (active && a.bias) ? a.bias[g * H + j] : 0.0f;

    for (int t = 0; t < a.T; ++t) {
        const float *cur = hS + (t & 1) * BT * HS + sg * RB * HS;
        float *nxt = hS + ((t + 1) & 1) * BT * HS + sg * RB * HS;
        if (active) {
            float acc[4][RB];
#pragma unroll
            for (int g = 0; g < 4; ++g)
#pragma unroll
                for (int r = 0; r < RB; ++r) acc[g][r] = bias[g];
            const float4 *wp = wa.w4 + j;
            int k = 0;
            for (; k + 4 <= H; k += 4) {
                float4 w[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) w[i] = __ldg(wp + static_cast<size_t>(k + i) * H);
#pragma unroll
                for (int r = 0; r < RB; ++r) {
                    const float4 hv = *reinterpret_cast<const float4 *>(cur + r * HS + k);
                    const float hk[4] = {hv.x, hv.y, hv.z, hv.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        acc[0][r] = fmaf(hk[i], w[i].x, acc[0][r]);
                        acc[1][r] = fmaf(hk[i], w[i].y, acc[1][r]);
                        acc[2][r] = fmaf(hk[i], w[i].z, acc[2][r]);
                        acc[3][r] = fmaf(hk[i], w[i].w, acc[3][r]);
                    }
                }
            }
            for (; k < H; ++k) {
                const float4 w = __ldg(wp + static_cast<size_t>(k) * H);
#pragma unroll
                for (int r = 0; r < RB; ++r) {
                    const float hk = cur[r * HS + k];
                    acc[0][r] = fmaf(hk, w.x, acc[0][r]);
                    acc[1][r] = fmaf(hk, w.y, acc[1][r]);
                    acc[2][r] = fmaf(hk, w.z, acc[2][r]);
                    acc[3][r] = fmaf(hk, w.w, acc[3][r]);
                }
            }
#pragma unroll
            for (int r = 0; r < RB; ++r) {
                const int b = b0 + r;
                if (b >= a.B) continue;
                const size_t row = static_cast<size_t>(t) * a.B + b;
                const float *ih = a.ih + row * C + j;
                float pre[4], act[4];
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    st[0].see(acc[g][r]);
                    if (a.tr.weight_hh_linear) a.tr.weight_hh_linear[row * C + g * H + j] = acc[g][r];
                    pre[g] = ih[g * H] + acc[g][r];
                    act[g] = g == 2 ? tanhf(pre[g]) : sigmoidStable(pre[g]);
                    st[1 + g].see(pre[g]);
                    st[5 + g].see(act[g]);
                    if (a.tr.gate_inputs) a.tr.gate_inputs[row * C + g * H + j] = pre[g];
                    if (a.tr.gate_outputs) a.tr.gate_outputs[row * C + g * H + j] = act[g];
                }
                const float keepOld = act[1] * cell[r], writeNew = act[0] * act[2];
                cell[r] = keepOld + writeNew;
                const float ct = tanhf(cell[r]);
                hidden[r] = act[3] * ct;
                st[9].see(cell[r]); st[10].see(ct); st[11].see(hidden[r]);
                st[12].see(keepOld); st[13].see(writeNew); st[14].see(hidden[r]);
                const size_t so = row * H + j;
                a.output[so] = hidden[r];
                if (a.tr.cell_states) a.tr.cell_states[so] = cell[r];
                if (a.tr.cell_tanh_outputs) a.tr.cell_tanh_outputs[so] = ct;
                if (a.tr.hidden_outputs) a.tr.hidden_outputs[so] = hidden[r];
                nxt[r * HS + j] = hidden[r];
            }
        }
        __syncthreads();
    }
    if (active) {
#pragma unroll
        for (int r = 0; r < RB; ++r) {
            if (b0 + r >= a.B) continue;
            const size_t o = static_cast<size_t>(b0 + r) * H + j;
            a.finalHidden[o] = hidden[r];
            a.finalCell[o] = cell[r];
        }
    }
    if (a.mins) {
        const int slots[kRecurrentStats] = {
            RXMET_LSTM_WEIGHT_HH_LINEAR, RXMET_LSTM_INPUT_GATE_INPUT, RXMET_LSTM_FORGET_GATE_INPUT,
            RXMET_LSTM_CELL_GATE_INPUT, RXMET_LSTM_OUTPUT_GATE_INPUT, RXMET_LSTM_INPUT_GATE_OUTPUT,
            RXMET_LSTM_FORGET_GATE_OUTPUT, RXMET_LSTM_CELL_GATE_OUTPUT, RXMET_LSTM_OUTPUT_GATE_OUTPUT,
            RXMET_LSTM_CELL_STATE, RXMET_LSTM_CELL_TANH_OUTPUT, RXMET_LSTM_OUTPUT, kOps + 0, kOps + 1, kOps + 2};
        stats::commit<kRecurrentStats>(st, slots, a.mins, a.maxs, scratch);
    }
}

int gridFor(size_t n, int block) { return static_cast<int>(std::min<size_t>((n + block - 1) / block, 148 * 8)); }

}  // namespace

size_t forwardFloatWorkspaceBytes(int T, int B, int I, int H) {
    WorkspaceSizer ws;
    const size_t C = 4 * static_cast<size_t>(H);
    ws.take<float>(static_cast<size_t>(T) * B * C);  // ih linear
    ws.take<float>(static_cast<size_t>(I) * C);      // weight_ih transposed
    ws.take<float>(static_cast<size_t>(H) * C);      // weight_hh transposed (H > 128: interleaved by gate)
    return ws.used() + 1024;
}

void forwardFloat(const ForwardFloatCall &call, void *workspace, size_t workspaceBytes, cudaStream_t st) {
    const int T = call.T, B = call.B, I = call.I, H = call.H, C = 4 * H;
    if (H > 512) fail(RXMET_ERR_UNSUPPORTED, "hidden sizes up to 512 are built (got %d)", H);
    const bool wide = C > 512;
    const size_t rows = static_cast<size_t>(T) * B;
    Workspace ws(workspace, workspaceBytes);
    float *ih = ws.take<float>(rows * C);
    float *wIhT = ws.take<float>(static_cast<size_t>(I) * C);
    float *wHhT = ws.take<float>(static_cast<size_t>(H) * C);
    float *mins = nullptr, *maxs = nullptr;
    const rxmet_lstm_trace none{};
    const rxmet_lstm_trace &tr = call.trace ? *call.trace : none;
    if (call.stats) {
        const size_t half = statsFloats(H) / 2;
        mins = call.stats;
        maxs = call.stats + half;
        {
            KernelTimer timer__("lstmFillStats", st);
            fillStats<<<gridFor(2 * half, 256), 256, 0, st>>>(call.stats, half);
        }
        afterLaunch("lstmFillStats");
        {
            KernelTimer timer__("lstmTensorMinMax", st);
            tensorMinMax<<<gridFor(rows * I, 256), 256, 0, st>>>(call.x, rows * I, mins + RXMET_LSTM_INPUT, maxs + RXMET_LSTM_INPUT);
        }
        afterLaunch("lstmTensorMinMax");
        const float *src[4] = {call.weightIh, call.weightHh, call.biasIh, call.biasHh};
        const int cols[4] = {I, H, 1, 1};
        for (int k = 0; k < 4; ++k) {
            if (!src[k]) continue;
            {
                KernelTimer timer__("lstmRowMinMax", st);
                rowMinMax<<<(C + 127) / 128, 128, 0, st>>>(src[k], C, cols[k], mins + kOps + 3 + k * C, maxs + kOps + 3 + k * C);
            }
            afterLaunch("lstmRowMinMax");
        }
    }
    auto transpose = [&](const float *in, int rowsIn, int colsIn, float *out) {
        {
            KernelTimer timer__("lstmTransposeWeights", st);
            transposeWeights<<<dim3((colsIn + 31) / 32, (rowsIn + 31) / 32), dim3(32, 8), 0, st>>>(in, rowsIn, colsIn, out);
        }
        afterLaunch("lstmTransposeWeights");
    };
    transpose(call.weightIh, C, I, wIhT);
    if (wide) {
        KernelTimer timer__("lstmInterleaveGates", st);
        interleaveGates<<<gridFor(static_cast<size_t>(C) * H, 256), 256, 0, st>>>(call.weightHh, H, wHhT);
        afterLaunch("lstmInterleaveGates");
    } else {
        transpose(call.weightHh, C, H, wHhT);
    }
    {
        const int block = std::min((C + 31) / 32 * 32, 512);
        const size_t smem = sizeof(float) * (kRowsPerBlock * I + 2 * 32);
        {
            KernelTimer timer__("lstmInputLinearFloat", st);
            inputLinearFloat<<<static_cast<int>((rows + kRowsPerBlock - 1) / kRowsPerBlock), block, smem, st>>>(
                call.x, static_cast<int>(rows), I, C, wIhT, call.biasIh, ih, tr.weight_ih_linear, mins, maxs,
                RXMET_LSTM_WEIGHT_IH_LINEAR);
        }
        afterLaunch("lstmInputLinearFloat");
    }
    FloatRecurrentArgs a{};
    a.T = T; a.B = B; a.H = H;
    a.wT = wHhT; a.bias = call.biasHh; a.ih = ih; a.h0 = call.h0; a.c0 = call.c0;
    a.output = call.output; a.finalHidden = call.finalHidden; a.finalCell = call.finalCell;
    a.tr = tr; a.mins = mins; a.maxs = maxs;
    const int smemMax = currentDevice().smemMax, sms = currentDevice().sms;
    if (wide) {
        FloatWideArgs wa{};
        wa.base = a;
        wa.w4 = reinterpret_cast<const float4 *>(wHhT);
        wa.HP = (H + 31) / 32 * 32;
        const int groupsMax = std::max(1, 512 / wa.HP);
        const int want = std::max(1, (B + sms - 1) / sms);
        int rb = 1;
        while (rb < 4 && rb * groupsMax < want) rb *= 2;
        const int groups = std::max(1, std::min(groupsMax, (want + rb - 1) / rb));
        const int btWide = groups * rb, blockWide = groups * wa.HP;
        const size_t smem = sizeof(float) * (2 * static_cast<size_t>(btWide) * ((H + 3) / 4 * 4) + 2 * kRecurrentStats * 16);
        auto launchWide = [&](auto kernel) {
            ensureDynamicSmem(reinterpret_cast<const void *>(kernel), smem);
            KernelTimer timer__("lstmRecurrentFloatWide", st);
            kernel<<<(B + btWide - 1) / btWide, blockWide, smem, st>>>(wa);
        };
        if (rb == 1) launchWide(recurrentFloatWide<1>);
        else if (rb == 2) launchWide(recurrentFloatWide<2>);
        else launchWide(recurrentFloatWide<4>);
        afterLaunch("lstmRecurrentFloatWide");
        return;
    }
    const int bt = (B >= 4 * sms) ? 4 : ((B > sms) ? 2 : 1);
    const int block = (C + 31) / 32 * 32;
    auto launch = [&](auto kernel, int BT) {
        const size_t base = sizeof(float) * (static_cast<size_t>(BT) * H + static_cast<size_t>(BT) * C + 2 * kRecurrentStats * 16);
        const size_t room = static_cast<size_t>(smemMax) > base + 1024 ? static_cast<size_t>(smemMax) - base - 1024 : 0;
        a.smemRows = static_cast<int>(std::min<size_t>(H, room / (sizeof(float) * C)));
        const size_t smem = base + sizeof(float) * static_cast<size_t>(a.smemRows) * C;
        RXMET_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        {
            KernelTimer timer__("lstmRecurrentFloat", st);
            kernel<<<(B + BT - 1) / BT, block, smem, st>>>(a);
        }
        afterLaunch("lstmRecurrentFloat");
    };
    if (bt == 4) launch(recurrentFloat<4>, 4);
    else if (bt == 2) launch(recurrentFloat<2>, 2);
    else launch(recurrentFloat<1>, 1);
}

}  // namespace lstm
}  // namespace rxmet
