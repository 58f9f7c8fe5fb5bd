// Float GRU forward and the calibration forward (float forward + min/max statistics).
//
// Same shape as the quantized path: the input projection for all steps is one kernel, the
// recurrence is ONE launch in which each CTA owns a batch tile for the whole sequence with the
// recurrent weights resident in shared memory when they fit.  The 13 activation statistics are
// accumulated in registers across all steps and leave the kernel as one atomic per CTA and
// statistic, so calibration never re-reads the activations from HBM and never returns to the
// host per tensor.
//
// Reference: operators/quant-gru/src/gru_forward_gpu.cu:359-431 (T x (SGEMM + pointwise)),
// src/calibration_gpu.cu:1847-1953 (one reduction + D2H copy per statistic) and the CPU
// definition of what is observed, src/gru_forward_cpu.cc:58-151.
#include <cuda_runtime.h>

#include <algorithm>
#include <cfloat>
#include <cstdint>

#include "common.h"
#include "gru_forward_float.h"

namespace rxmet {
namespace gru {
namespace {

constexpr int kRowsPerBlock = 8;

// Order-preserving float atomics (valid for any finite value, -0.0 included, as long as the
// slot starts at +FLT_MAX / -FLT_MAX).
__device__ __forceinline__ void atomicMinFloat(float *addr, float v) {
    if (v >= 0.0f) atomicMin(reinterpret_cast<int *>(addr), __float_as_int(v));
    else atomicMax(reinterpret_cast<unsigned int *>(addr), __float_as_uint(v));
}
__device__ __forceinline__ void atomicMaxFloat(float *addr, float v) {
    if (v >= 0.0f) atomicMax(reinterpret_cast<int *>(addr), __float_as_int(v));
    else atomicMin(reinterpret_cast<unsigned int *>(addr), __float_as_uint(v));
}

struct MinMax {
    float lo = FLT_MAX, hi = -FLT_MAX;
    __device__ __forceinline__ void see(float v) {
        if (isfinite(v)) {  // only finite values are observed (gru_forward_cpu.cc:17-22)
            lo = fminf(lo, v);
            hi = fmaxf(hi, v);
        }
    }
};

__device__ __forceinline__ MinMax warpReduce(MinMax m) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        m.lo = fminf(m.lo, __shfl_xor_sync(0xffffffffu, m.lo, o));
        m.hi = fmaxf(m.hi, __shfl_xor_sync(0xffffffffu, m.hi, o));
    }
    return m;
}

// Block-wide reduce of `count` statistics held per thread, then one atomic pair per statistic.
// scratch: 2 * count * (blockDim/32) floats of shared memory.
template <int N>
__device__ void commitStats(MinMax (&local)[N], const int (&slot)[N], float *mins, float *maxs, float *scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int i = 0; i < N; ++i) {
        const MinMax m = warpReduce(local[i]);
        if (lane == 0) {
            scratch[(2 * i) * warps + warp] = m.lo;
            scratch[(2 * i + 1) * warps + warp] = m.hi;
        }
    }
    __syncthreads();
    if (threadIdx.x < N) {
        float lo = FLT_MAX, hi = -FLT_MAX;
        for (int w = 0; w < warps; ++w) {
            lo = fminf(lo, scratch[(2 * threadIdx.x) * warps + w]);
            hi = fmaxf(hi, scratch[(2 * threadIdx.x + 1) * warps + w]);
        }
        if (lo <= hi) {
            atomicMinFloat(&mins[slot[threadIdx.x]], lo);
            atomicMaxFloat(&maxs[slot[threadIdx.x]], hi);
        }
    }
    __syncthreads();
}

__global__ void fillStats(float *stats, size_t half) {
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < 2 * half;
         i += static_cast<size_t>(gridDim.x) * blockDim.x)
        stats[i] = i < half ? FLT_MAX : -FLT_MAX;
}

// min/max of a flat tensor: 128-bit loads, warp shuffles, one atomic pair per CTA.
__global__ void tensorMinMax(const float *__restrict__ x, size_t n, float *minSlot, float *maxSlot) {
    __shared__ float scratch[2 * 32];
    MinMax m[1];
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    const size_t i0 = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    if ((reinterpret_cast<uintptr_t>(x) & 15u) == 0) {
        const float4 *x4 = reinterpret_cast<const float4 *>(x);
        const size_t n4 = n / 4;
        for (size_t i = i0; i < n4; i += stride) {
            const float4 q = x4[i];
            m[0].see(q.x); m[0].see(q.y); m[0].see(q.z); m[0].see(q.w);
        }
        for (size_t i = n4 * 4 + i0; i < n; i += stride) m[0].see(x[i]);
    } else {
        for (size_t i = i0; i < n; i += stride) m[0].see(x[i]);
    }
    const int slot[1] = {0};
    commitStats<1>(m, slot, minSlot, maxSlot, scratch);
}

// Per-column min/max of a [rows, cols] matrix (weights and biases per output channel).
__global__ void columnMinMax(const float *__restrict__ w, int rows, int cols, float *mins, float *maxs) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    MinMax m;
    for (int r = 0; r < rows; ++r) m.see(w[static_cast<size_t>(r) * cols + c]);
    if (m.lo > m.hi) m.lo = m.hi = 0.0f;  // nothing finite: observes 0 (gru_forward_cpu.cc:24)
    mins[c] = m.lo;
    maxs[c] = m.hi;
}

// wx[n, c] = sum_k x[n,k] W[k,c] + bw[c] for all T*B rows.
__global__ void inputLinearFloat(const float *__restrict__ x, int rows, int K, int C, const float *__restrict__ W,
                                 const float *__restrict__ bw, float *__restrict__ out, float *mins, float *maxs,
                                 int slot) {
    extern __shared__ float smemF[];
    float *xs = smemF;                        // [kRowsPerBlock][K]
    float *scratch = smemF + kRowsPerBlock * K;  // 2 * warps
    const int row0 = blockIdx.x * kRowsPerBlock;
    const int nRows = min(kRowsPerBlock, rows - row0);
    for (int i = threadIdx.x; i < kRowsPerBlock * K; i += blockDim.x) {
        const int r = i / K;
        xs[i] = r < nRows ? x[static_cast<size_t>(row0 + r) * K + (i % K)] : 0.0f;
    }
    __syncthreads();
    MinMax m[1];
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float acc[kRowsPerBlock];
#pragma unroll
        for (int r = 0; r < kRowsPerBlock; ++r) acc[r] = 0.0f;
        for (int k = 0; k < K; ++k) {
            const float w = W[static_cast<size_t>(k) * C + c];
#pragma unroll
            for (int r = 0; r < kRowsPerBlock; ++r) acc[r] = fmaf(xs[r * K + k], w, acc[r]);
        }
        const float b = bw[c];
#pragma unroll
        for (int r = 0; r < kRowsPerBlock; ++r) {
            if (r < nRows) {
                const float val = acc[r] + b;
                out[static_cast<size_t>(row0 + r) * C + c] = val;
                m[0].see(val);
            }
        }
    }
    if (mins) {
        const int slots[1] = {slot};
        commitStats<1>(m, slots, mins, maxs, scratch);
    }
}

struct FloatRecurrentArgs {
    int T, B, H;
    int weightsInSmem;
    const float *R;   // [H][3H]
    const float *br;  // [3H]
    const float *wx;  // [T][B][3H] = W x + bw
    const float *h0;  // [B][H] or null
    float *h;         // [T+1][B][H]
    float *v;         // [T][B][4H]
    float *mins, *maxs;  // packed statistics or null
    float *trRh, *trPre, *trMul;  // optional [T][B][3H] traces
};

template <int BT>
__global__ void __launch_bounds__(768) recurrentFloat(const __grid_constant__ FloatRecurrentArgs a) {
    const int H = a.H, C = 3 * a.H;
    extern __shared__ float smemF[];
    float *hS = smemF;                 // [BT][H]
    float *rhS = hS + BT * H;          // [BT][C] = R h + br
    float *scratch = rhS + BT * C;     // 2 * 12 * warps
    float *RS = scratch + 2 * 12 * 32; // [H][C] when resident
    const int tid = threadIdx.x, nthreads = blockDim.x;
    const int b0 = blockIdx.x * BT, nb = min(BT, a.B - b0);

    const float *Rsrc = a.R;
    if (a.weightsInSmem) {
        for (int i = tid; i < H * C; i += nthreads) RS[i] = a.R[i];
        Rsrc = RS;
    }
    for (int i = tid; i < BT * H; i += nthreads) {
        const int b = i / H;
        hS[i] = (b < nb && a.h0) ? a.h0[static_cast<size_t>(b0 + b) * H + (i % H)] : 0.0f;
    }
    __syncthreads();
    for (int i = tid; i < nb * H; i += nthreads) a.h[static_cast<size_t>(b0 + i / H) * H + (i % H)] = hS[i];

    // statistic order: h, Rh, z_pre, r_pre, n_pre, z, r, n, r*rec, (1-z)*n, z*h_old  (+ unused)
    MinMax st[12];
    for (int t = 0; t < a.T; ++t) {
        const size_t rowBase = static_cast<size_t>(t) * a.B + b0;
        for (int c = tid; c < C; c += nthreads) {
            float acc[BT];
#pragma unroll
            for (int b = 0; b < BT; ++b) acc[b] = 0.0f;
            for (int k = 0; k < H; ++k) {
                const float w = Rsrc[static_cast<size_t>(k) * C + c];
#pragma unroll
                for (int b = 0; b < BT; ++b) acc[b] = fmaf(hS[b * H + k], w, acc[b]);
            }
            const float bias = a.br[c];
#pragma unroll
            for (int b = 0; b < BT; ++b) {
                const float val = acc[b] + bias;
                rhS[b * C + c] = val;
                if (b < nb) {
                    st[1].see(val);
                    if (a.trRh) a.trRh[(rowBase + b) * C + c] = val;
                }
            }
        }
        __syncthreads();
        for (int i = tid; i < nb * H; i += nthreads) {
            const int b = i / H, j = i % H;
            const size_t row = rowBase + b;
            const float *wx = a.wx + row * C;
            const float *rh = rhS + b * C;
            const float zPre = wx[j] + rh[j];
            const float rPre = wx[H + j] + rh[H + j];
            const float z = 1.0f / (1.0f + expf(-zPre));
            const float r = 1.0f / (1.0f + expf(-rPre));
            const float rec = rh[2 * H + j];
            const float rm = r * rec;
            const float nPre = wx[2 * H + j] + rm;
            const float n = tanhf(nPre);
            const float hOld = hS[b * H + j];
            const float oldC = z * hOld;
            const float newC = (1.0f - z) * n;
            const float hNew = oldC + newC;
            hS[b * H + j] = hNew;
            a.h[(row + a.B) * H + j] = hNew;
            float *vRow = a.v + row * 4 * H;
            vRow[j] = z; vRow[H + j] = r; vRow[2 * H + j] = n; vRow[3 * H + j] = rec;
            if (a.trPre) {
                float *pre = a.trPre + row * C, *mul = a.trMul + row * C;
                pre[j] = zPre; pre[H + j] = rPre; pre[2 * H + j] = nPre;
                mul[j] = rm; mul[H + j] = newC; mul[2 * H + j] = oldC;
            }
            st[0].see(hNew); st[2].see(zPre); st[3].see(rPre); st[4].see(nPre);
            st[5].see(z); st[6].see(r); st[7].see(n); st[8].see(rm); st[9].see(newC); st[10].see(oldC);
        }
        __syncthreads();
    }
    if (a.mins) {
        const int slots[12] = {RXMET_GRU_H, RXMET_GRU_WEIGHT_HH_LINEAR, RXMET_GRU_UPDATE_GATE_INPUT,
                               RXMET_GRU_RESET_GATE_INPUT, RXMET_GRU_NEW_GATE_INPUT, RXMET_GRU_UPDATE_GATE_OUTPUT,
                               RXMET_GRU_RESET_GATE_OUTPUT, RXMET_GRU_NEW_GATE_OUTPUT, RXMET_GRU_MUL_RESET_HIDDEN,
                               RXMET_GRU_MUL_NEW_CONTRIBUTION, RXMET_GRU_MUL_OLD_CONTRIBUTION, RXMET_GRU_H};
        commitStats<12>(st, slots, a.mins, a.maxs, scratch);
    }
}

int gridFor(size_t n, int block) { return static_cast<int>(std::min<size_t>((n + block - 1) / block, 148 * 8)); }

}  // namespace

size_t statsFloats(int H) { return 2 * (static_cast<size_t>(kOps) + 12 * static_cast<size_t>(H)); }

size_t forwardFloatWorkspaceBytes(int T, int B, int I, int H) {
    (void)I;
    WorkspaceSizer ws;
    ws.take<float>(static_cast<size_t>(T) * B * 3 * H);
    ws.take<float>(statsFloats(H));
    return ws.used() + 1024;
}

void forwardFloat(const ForwardFloatCall &call, void *workspace, size_t workspaceBytes, cudaStream_t st) {
    const int T = call.T, B = call.B, I = call.I, H = call.H, C = 3 * H;
    const size_t rows = static_cast<size_t>(T) * B;
    Workspace ws(workspace, workspaceBytes);
    float *wx = ws.take<float>(rows * C);
    if (call.traceWx) wx = call.traceWx;
    float *mins = nullptr, *maxs = nullptr;
    const size_t half = statsFloats(H) / 2;
    if (call.stats) {
        mins = call.stats;
        maxs = call.stats + half;
        {
            KernelTimer timer__("fillStats", st);
            fillStats<<<gridFor(2 * half, 256), 256, 0, st>>>(call.stats, half);
        }
        afterLaunch("fillStats");
        {
            KernelTimer timer__("tensorMinMax", st);
            tensorMinMax<<<gridFor(rows * I / 4 + 1, 256), 256, 0, st>>>(call.x, rows * I, mins + RXMET_GRU_X,
                                                                        maxs + RXMET_GRU_X);
        }
        afterLaunch("tensorMinMax");
        // per-channel blocks follow the 17 scalar slots: W, R, bw, br
        const float *src[4] = {call.W, call.R, call.bw, call.br};
        const int srcRows[4] = {I, H, 1, 1};
        for (int k = 0; k < 4; ++k) {
            {
                KernelTimer timer__("columnMinMax", st);
                columnMinMax<<<(C + 127) / 128, 128, 0, st>>>(src[k], srcRows[k], C, mins + kOps + k * C, maxs + kOps + k * C);
            }
            afterLaunch("columnMinMax");
        }
    }
    {
        const int block = std::min((C + 31) / 32 * 32, 512);
        const size_t smem = sizeof(float) * (kRowsPerBlock * I + 2 * 32);
        {
            KernelTimer timer__("inputLinearFloat", st);
            inputLinearFloat<<<static_cast<int>((rows + kRowsPerBlock - 1) / kRowsPerBlock), block, smem, st>>>(
                call.x, static_cast<int>(rows), I, C, call.W, call.bw, wx, mins, maxs, RXMET_GRU_WEIGHT_IH_LINEAR);
        }
        afterLaunch("inputLinearFloat");
    }
    FloatRecurrentArgs a{};
    a.T = T; a.B = B; a.H = H;
    a.R = call.R; a.br = call.br; a.wx = wx; a.h0 = call.h0; a.h = call.h; a.v = call.v;
    a.mins = mins; a.maxs = maxs;
    a.trRh = call.traceRh; a.trPre = call.tracePre; a.trMul = call.traceMul;
    RXMET_REQUIRE((call.tracePre == nullptr) == (call.traceMul == nullptr), "pre-activation and product traces go together");
    int device = 0, smemMax = 0, sms = 0;
    RXMET_CUDA(cudaGetDevice(&device));
    RXMET_CUDA(cudaDeviceGetAttribute(&smemMax, cudaDevAttrMaxSharedMemoryPerBlockOptin, device));
    RXMET_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    const int bt = (B >= 8 * sms) ? 4 : ((B >= 4 * sms) ? 2 : 1);
    const int block = std::min((C + 31) / 32 * 32, 768);
    auto launch = [&](auto kernel, int BT) {
        const size_t base = sizeof(float) * (static_cast<size_t>(BT) * H + static_cast<size_t>(BT) * C + 2 * 12 * 32);
        const size_t full = base + sizeof(float) * static_cast<size_t>(H) * C;
        a.weightsInSmem = full <= static_cast<size_t>(smemMax) ? 1 : 0;
        const size_t smem = a.weightsInSmem ? full : base;
        if (smem > static_cast<size_t>(smemMax))
            fail(RXMET_ERR_UNSUPPORTED, "hidden size %d needs %zu bytes of shared memory per CTA", H, smem);
        RXMET_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        {
            KernelTimer timer__("recurrentFloat", st);
            kernel<<<(B + BT - 1) / BT, block, smem, st>>>(a);
        }
        afterLaunch("recurrentFloat");
    };
    if (bt == 4) launch(recurrentFloat<4>, 4);
    else if (bt == 2) launch(recurrentFloat<2>, 2);
    else launch(recurrentFloat<1>, 1);
}

}  // namespace gru
}  // namespace rxmet
