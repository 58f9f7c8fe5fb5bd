// Quantized GRU forward for weight grids of at most 8 bits with activation grids (x, h) of 9 to 16 bits -
// the W8 / A16 configurations - on the integer carrier (operators/quant-gru/src/gru_forward_cpu_quant.cc:
// 113-348, CUDA statement src/gru_forward_gpu_quant.cu:109-180,789-841).
//
// The generic kernels accumulate one 64-bit multiply-add per code.  Here a 16-bit code is stored as two
// byte planes of u = code - grid minimum (0 .. 65535), packed four along K, so both linear stages run on
// dp4a (signed weight bytes times unsigned code bytes):
//   sum_k w * code = 256 * sum_hi + sum_lo + grid minimum * sum_k w
// with the last term, the zero-point compensation and the bias folded into one 64-bit addend per channel.
// Everything after the sum is the reference's integer arithmetic unchanged (64-bit rounding rescales,
// piecewise-linear activation tables, clamp flags).
//
// Launches (after the shared quantization of weights, x and h0 into one code per element):
//   packWeightWords  : int8 codes [K][3H] -> words of four along K, per-channel addends
//   planesFromCodes  : int16 codes -> byte planes (x for all steps, h0)
//   inputLinearPlanes: all T*B rows of the input projection, persistent CTAs, cp.async staging
//   recurrentPlanes  : ONE launch for all T steps; thread (j, s) owns hidden unit j - all three gates - for
//                      RB batch rows of row group s, keeps those rows' hidden codes in registers, reads the
//                      packed recurrent weights from shared memory (3H x H bytes: fits up to H = 256) or
//                      from L2, and exchanges the hidden byte planes of the CTA's rows through shared
//                      memory (double buffered, one barrier per step).
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstdlib>

#include "common.h"
#include "gru_device.cuh"
#include "gru_forward_wide.h"
#include "plane_proj_umma.cuh"

namespace rxmet {
namespace gru {
namespace {

__device__ __forceinline__ int32_t dotSignedUnsigned(uint32_t signedBytes, uint32_t unsignedBytes, int32_t acc) {
    int32_t d;
    asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(signedBytes), "r"(unsignedBytes), "r"(acc));
    return d;
}
__device__ __forceinline__ void copyAsync16(void *dst, const void *src, bool valid) {
    const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(valid ? 16u : 0u) : "memory");
}

int gridFor(size_t n, int block) { return static_cast<int>(std::min<size_t>((n + block - 1) / block, 148 * 8)); }
int wordsFor(int k) { return (k + 15) / 16 * 4; }  // K padded to 16 bytes so that rows are read as 16-byte pieces

// codes [K rows (padded to kPadRows)][C] int8 -> words [kWords][C], four consecutive k per word; one warp
// per channel sums the codes: addend = (gridMin - zeroPoint) * sum + bias on the accumulator grid, where
// comp = zeroPoint * sum was computed with the codes (so gridMin * sum - comp + bias).
__global__ void packWeightWords(const int8_t *__restrict__ codes, int K, int C, int kWords, int32_t gridMin,
                                const int64_t *__restrict__ comp, const int64_t *__restrict__ biasAcc,
                                uint32_t *__restrict__ words, int64_t *__restrict__ addend) {
    const int lane = threadIdx.x & 31;
    const int c = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (c >= C) return;
    int32_t sum = 0;
    for (int kw = lane; kw < kWords; kw += 32) {
        uint32_t word = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int k = 4 * kw + i;
            const int32_t q = k < K ? codes[static_cast<size_t>(k) * C + c] : 0;
            sum += q;
            word |= (static_cast<uint32_t>(q) & 0xffu) << (8 * i);
        }
        words[static_cast<size_t>(kw) * C + c] = word;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) addend[c] = static_cast<int64_t>(gridMin) * sum - comp[c] + biasAcc[c];
}

// int16 codes [rows][colsPadded] -> [rows][2][kWords] words of four bytes of u = code - gridMin (plane 0 = high
// bytes); columns beyond `cols` are zero.
__global__ void planesFromCodes(const int16_t *__restrict__ codes, size_t rows, int cols, int colsPadded, int kWords,
                                int32_t gridMin, uint32_t *__restrict__ planes) {
    const size_t total = rows * kWords;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t r = i / kWords;
        const int kw = static_cast<int>(i % kWords);
        uint32_t high = 0, low = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int k = 4 * kw + e;
            if (k >= cols) continue;
            const uint32_t u = static_cast<uint32_t>(static_cast<int32_t>(codes[r * colsPadded + k]) - gridMin);
            low |= (u & 0xffu) << (8 * e);
            high |= ((u >> 8) & 0xffu) << (8 * e);
        }
        planes[(2 * r) * kWords + kw] = high;
        planes[(2 * r + 1) * kWords + kw] = low;
    }
}

__device__ __forceinline__ int64_t combine(int32_t high, int32_t low, int64_t addend) {
    return (static_cast<int64_t>(high) << 8) + low + addend;
}

constexpr int kRowsPerBlock = 16;
constexpr int kThreads = 512;

struct InputArgs {
    int rows, C, kWords;
    const uint32_t *x;       // [rows][2][kWords]
    const uint32_t *words;   // [kWords][C]
    const int64_t *addend;   // [C]
    const Rescale *rescale;  // [C]
    int32_t zpOut, lo, hi;
    int16_t *out;            // [rows][C]
    uint8_t *mask;           // optional keep flags
};

// KW = weight words a thread keeps in registers.  CHUNKED = false: the whole K fits (kWords <= KW) and the
// words are loaded once per CTA.  CHUNKED = true: K is walked in chunks of KW words per row block, the
// chunk's words re-read from L2 (a block of 16 rows amortises them) and the sums kept in registers.
template <int KW, bool CHUNKED>
__global__ void __launch_bounds__(kThreads) inputLinearPlanes(const __grid_constant__ InputArgs a) {
    extern __shared__ __align__(16) uint32_t planeSmem[];  // [2][kRowsPerBlock][2 * kWords]
    const int C = a.C, tid = threadIdx.x, c = blockIdx.y * blockDim.x + tid;
    const bool live = c < C;
    const int kWords = a.kWords, rowWords = 2 * kWords, blockWords = kRowsPerBlock * rowWords;
    uint32_t w[KW];
    if (!CHUNKED) {
#pragma unroll
        for (int kk = 0; kk < KW; ++kk) w[kk] = (live && kk < kWords) ? a.words[static_cast<size_t>(kk) * C + c] : 0u;
    }
    const int64_t addend = live ? a.addend[c] : 0;
    const Rescale rs = live ? a.rescale[c] : Rescale{1, 0};
    const int blocks = (a.rows + kRowsPerBlock - 1) / kRowsPerBlock;
    const size_t limit = static_cast<size_t>(a.rows) * rowWords;
    auto stage = [&](int blk, int buf) {
        const size_t base = static_cast<size_t>(blk) * blockWords;
        uint32_t *dst = planeSmem + buf * blockWords;
        for (int i = tid * 4; i < blockWords; i += blockDim.x * 4) {
            const bool valid = blk < blocks && base + i < limit;
            copyAsync16(dst + i, a.x + (valid ? base + i : 0), valid);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    stage(blockIdx.x, 0);
    int buf = 0;
    for (int blk = blockIdx.x; blk < blocks; blk += gridDim.x, buf ^= 1) {
        stage(blk + gridDim.x, buf ^ 1);
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();
        const int row0 = blk * kRowsPerBlock, nRows = min(kRowsPerBlock, a.rows - row0);
        if (live) {
            const uint32_t *xb = planeSmem + buf * blockWords;
            int32_t high[kRowsPerBlock], low[kRowsPerBlock];
#pragma unroll
            for (int r = 0; r < kRowsPerBlock; ++r) high[r] = low[r] = 0;
            for (int kc = 0; kc < (CHUNKED ? kWords : 1); kc += KW) {
                if (CHUNKED) {
#pragma unroll
                    for (int kk = 0; kk < KW; ++kk)
                        w[kk] = kc + kk < kWords ? __ldg(a.words + static_cast<size_t>(kc + kk) * C + c) : 0u;
                }
#pragma unroll
                for (int r = 0; r < kRowsPerBlock; ++r) {
                    const uint32_t *xr = xb + r * rowWords + kc;
#pragma unroll
                    for (int k4 = 0; k4 < KW / 4; ++k4) {
                        if (kc + 4 * k4 < kWords) {
                            const uint4 xh = *reinterpret_cast<const uint4 *>(xr + 4 * k4);
                            const uint4 xl = *reinterpret_cast<const uint4 *>(xr + kWords + 4 * k4);
                            high[r] = dotSignedUnsigned(w[4 * k4 + 0], xh.x, high[r]);
                            high[r] = dotSignedUnsigned(w[4 * k4 + 1], xh.y, high[r]);
                            high[r] = dotSignedUnsigned(w[4 * k4 + 2], xh.z, high[r]);
                            high[r] = dotSignedUnsigned(w[4 * k4 + 3], xh.w, high[r]);
                            low[r] = dotSignedUnsigned(w[4 * k4 + 0], xl.x, low[r]);
                            low[r] = dotSignedUnsigned(w[4 * k4 + 1], xl.y, low[r]);
                            low[r] = dotSignedUnsigned(w[4 * k4 + 2], xl.z, low[r]);
                            low[r] = dotSignedUnsigned(w[4 * k4 + 3], xl.w, low[r]);
                        }
                    }
                }
            }
            size_t o = static_cast<size_t>(row0) * C + c;
#pragma unroll
            for (int r = 0; r < kRowsPerBlock; ++r, o += C) {
                if (r >= nRows) break;
                uint8_t keep;
                const int32_t q = clampCode(static_cast<int32_t>(applyRescale(combine(high[r], low[r], addend), rs)) + a.zpOut, a.lo, a.hi, keep);
                a.out[o] = static_cast<int16_t>(q);
                if (a.mask) a.mask[o] = keep;
            }
        }
        __syncthreads();
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
}

struct RecurrentArgs {
    int T, B, H, HP, kWords;
    int weightBytesInSmem;   // size of the shared-memory copy of `words` (WS variant), else 0
    const uint32_t *words;   // [kWords][3H]
    const int64_t *addend;   // [3H]
    const Rescale *rescale;  // [3H]
    const int16_t *ih;       // [T][B][3H]
    const int16_t *h0;       // [B][hPad] codes
    int hPad;
    const uint32_t *h0Planes;  // [B][2][kWords]
    float *h;                // [T+1][B][H] dequantized
    float *v;                // [T][B][4H] dequantized
    int32_t *hq, *vq;        // optional codes
    uint8_t *maskHh, *maskGateIn, *maskGateOut, *maskH;
    const int *poison;       // status word of the tensor-core projection: non-zero turns the hidden outputs into NaN
};

template <int RB, bool WS>
__global__ void __launch_bounds__(kThreads, 1)
recurrentPlanes(const __grid_constant__ RecurrentArgs a, const __grid_constant__ GateExec gateParam) {
    // The cell reads table entries at per-lane segment indices: from the constant bank such a read is replayed once
    // per distinct index in the warp, from shared memory it is one banked access.
    __shared__ GateExec g;
    for (int i = threadIdx.x; i < static_cast<int>(sizeof(GateExec) / 4); i += blockDim.x)
        reinterpret_cast<int32_t *>(&g)[i] = reinterpret_cast<const int32_t *>(&gateParam)[i];
    extern __shared__ __align__(16) uint32_t planeSmemRaw[];  // [weights when WS] [2][BT][2][kWords]
    uint32_t *planeSmem = planeSmemRaw + (WS ? a.weightBytesInSmem / 4 : 0);
    const int H = a.H, C = 3 * a.H, kWords = a.kWords;
    const int tid = threadIdx.x, j = tid % a.HP, sg = tid / a.HP;
    const int BT = (blockDim.x / a.HP) * RB;
    const bool active = j < H;
    const int rowWords = 2 * kWords, bufWords = BT * rowWords;
    const int ctaRow0 = blockIdx.x * BT, b0 = ctaRow0 + sg * RB;
    if (WS) {
        const uint4 *src = reinterpret_cast<const uint4 *>(a.words);
        uint4 *dst = reinterpret_cast<uint4 *>(planeSmemRaw);
        for (int i = tid; i < a.weightBytesInSmem / 16; i += blockDim.x) dst[i] = src[i];
    }
    for (int i = tid; i < 2 * bufWords; i += blockDim.x) planeSmem[i] = 0u;
    __syncthreads();
    for (int i = tid; i < bufWords; i += blockDim.x) {
        const int b = ctaRow0 + i / rowWords;
        if (b < a.B) planeSmem[i] = a.h0Planes[static_cast<size_t>(b) * rowWords + i % rowWords];
    }
    int64_t addend[3];
    Rescale rs[3];
#pragma unroll
    for (int gate = 0; gate < 3; ++gate) {
        addend[gate] = active ? a.addend[gate * H + j] : 0;
        rs[gate] = active ? a.rescale[gate * H + j] : Rescale{1, 0};
    }
    const int32_t zpH = g.zp[RXMET_GRU_H], loH = g.qlo[RXMET_GRU_H];
    // a projection whose bounded wait gave up left unusable codes: make that loud
    const float scaleH = (a.poison && *a.poison) ? __int_as_float(0x7fc00000) : g.eff[RXMET_GRU_H];
    int32_t hOld[RB];
#pragma unroll
    for (int r = 0; r < RB; ++r) {
        const int b = b0 + r;
        hOld[r] = (active && b < a.B) ? a.h0[static_cast<size_t>(b) * a.hPad + j] : zpH;
        if (active && b < a.B) {
            const size_t o = static_cast<size_t>(b) * H + j;
            a.h[o] = static_cast<float>(hOld[r] - zpH) * scaleH;
            if (a.hq) a.hq[o] = hOld[r];
        }
    }
    const int32_t zpOut = g.zp[RXMET_GRU_WEIGHT_HH_LINEAR], loOut = g.qlo[RXMET_GRU_WEIGHT_HH_LINEAR],
                  hiOut = g.qhi[RXMET_GRU_WEIGHT_HH_LINEAR];
    const size_t stepH = static_cast<size_t>(a.B) * H, stepC = static_cast<size_t>(a.B) * C;
    __syncthreads();

    for (int t = 0; t < a.T; ++t) {
        const uint32_t *cur = planeSmem + (t & 1) * bufWords;
        uint8_t *nxt = reinterpret_cast<uint8_t *>(planeSmem + ((t + 1) & 1) * bufWords);
        if (active) {
            // the input projection's codes of this step: loaded first, so that they arrive during the dot products
            int32_t ihV[RB][3];
#pragma unroll
            for (int r = 0; r < RB; ++r) {
                const int b = b0 + r;
                const int16_t *ihRow = a.ih + (static_cast<size_t>(t) * a.B + (b < a.B ? b : 0)) * C;
#pragma unroll
                for (int gate = 0; gate < 3; ++gate) ihV[r][gate] = __ldg(ihRow + gate * H + j);
            }
            int32_t acc[3][RB][2];
#pragma unroll
            for (int gate = 0; gate < 3; ++gate)
#pragma unroll
                for (int r = 0; r < RB; ++r) acc[gate][r][0] = acc[gate][r][1] = 0;
            const uint32_t *wp = (WS ? planeSmemRaw : a.words) + j;
            const uint4 *hRows = reinterpret_cast<const uint4 *>(cur + sg * RB * rowWords);
#pragma unroll 2
            for (int k4 = 0; k4 < kWords / 4; ++k4) {
                uint32_t w[3][4];
#pragma unroll
                for (int gate = 0; gate < 3; ++gate)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t *src = wp + static_cast<size_t>(4 * k4 + i) * C + gate * H;
                        w[gate][i] = WS ? *src : __ldg(src);
                    }
#pragma unroll
                for (int r = 0; r < RB; ++r)
#pragma unroll
                    for (int p = 0; p < 2; ++p) {
                        const uint4 hv = hRows[(r * 2 + p) * (kWords / 4) + k4];
#pragma unroll
                        for (int gate = 0; gate < 3; ++gate) {
                            acc[gate][r][p] = dotSignedUnsigned(w[gate][0], hv.x, acc[gate][r][p]);
                            acc[gate][r][p] = dotSignedUnsigned(w[gate][1], hv.y, acc[gate][r][p]);
                            acc[gate][r][p] = dotSignedUnsigned(w[gate][2], hv.z, acc[gate][r][p]);
                            acc[gate][r][p] = dotSignedUnsigned(w[gate][3], hv.w, acc[gate][r][p]);
                        }
                    }
            }
#pragma unroll
            for (int r = 0; r < RB; ++r) {
                const int b = b0 + r;
                if (b >= a.B) continue;
                const size_t row = static_cast<size_t>(t) * a.B + b;
                int32_t hh[3];
                uint8_t keepHh[3];
#pragma unroll
                for (int gate = 0; gate < 3; ++gate)
                    hh[gate] = clampCode(static_cast<int32_t>(applyRescale(combine(acc[gate][r][0], acc[gate][r][1], addend[gate]), rs[gate])) + zpOut,
                                         loOut, hiOut, keepHh[gate]);
                GateMasks m;
                const GateCodes q = gruCell(ihV[r][0], ihV[r][1], ihV[r][2], hh[0], hh[1], hh[2], hOld[r], g, m);
                hOld[r] = q.h;
                const uint32_t u = static_cast<uint32_t>(q.h - loH);
                uint8_t *rowBytes = nxt + static_cast<size_t>(sg * RB + r) * rowWords * 4;
                rowBytes[j] = static_cast<uint8_t>(u >> 8);
                rowBytes[kWords * 4 + j] = static_cast<uint8_t>(u & 0xffu);

                const size_t ho = (row + a.B) * H + j;  // h[t+1]
                a.h[ho] = static_cast<float>(q.h - zpH) * scaleH;
                float *vRow = a.v + row * 4 * H;
                vRow[j] = static_cast<float>(q.z - g.zp[RXMET_GRU_UPDATE_GATE_OUTPUT]) * g.eff[RXMET_GRU_UPDATE_GATE_OUTPUT];
                vRow[H + j] = static_cast<float>(q.r - g.zp[RXMET_GRU_RESET_GATE_OUTPUT]) * g.eff[RXMET_GRU_RESET_GATE_OUTPUT];
                vRow[2 * H + j] = static_cast<float>(q.n - g.zp[RXMET_GRU_NEW_GATE_OUTPUT]) * g.eff[RXMET_GRU_NEW_GATE_OUTPUT];
                vRow[3 * H + j] = static_cast<float>(hh[2] - zpOut) * g.eff[RXMET_GRU_WEIGHT_HH_LINEAR];
                if (a.hq) a.hq[ho] = q.h;
                if (a.vq) {
                    int32_t *vq = a.vq + row * 4 * H;
                    vq[j] = q.z; vq[H + j] = q.r; vq[2 * H + j] = q.n; vq[3 * H + j] = hh[2];
                }
                if (a.maskHh) {
                    uint8_t *mh = a.maskHh + row * C;
                    mh[j] = keepHh[0]; mh[H + j] = keepHh[1]; mh[2 * H + j] = keepHh[2];
                }
                if (a.maskGateIn) {
                    uint8_t *mi = a.maskGateIn + row * C, *mo = a.maskGateOut + row * C;
                    mi[j] = m.in[0]; mi[H + j] = m.in[1]; mi[2 * H + j] = m.in[2];
                    mo[j] = m.out[0]; mo[H + j] = m.out[1]; mo[2 * H + j] = m.out[2];
                    a.maskH[row * H + j] = m.h;
                }
            }
        }
        __syncthreads();
    }
    (void)stepH;
    (void)stepC;
}

struct Layout {
    uint32_t *xPlanes, *h0Planes, *wWords, *rWords;
    int64_t *addX, *addH;
    uint4 *wTiles;     // input weights as canonical tensor-core tiles (plane_proj_umma.cuh)
    int *projStatus;
};

// Epilogue of the tensor-core input projection: exact 64-bit sum of the two planes and the addend, the
// rounding rescale onto the linear-output grid, clamp, code and keep flag.
struct PlaneEpilogue {
    const int64_t *addend;
    const Rescale *rescale;
    int32_t zpOut, lo, hi;
    int16_t *out;
    uint8_t *mask;
    int C;
    struct Channel {
        int64_t addend;
        Rescale rs;
    };
    __device__ Channel channel(int c) const { return Channel{addend[c], rescale[c]}; }
    __device__ void store(const Channel &ch, size_t row, int c, const int32_t (&acc)[2]) const {
        uint8_t keep;
        const int32_t q = clampCode(static_cast<int32_t>(applyRescale(combine(acc[0], acc[1], ch.addend), ch.rs)) + zpOut, lo, hi, keep);
        const size_t o = row * C + c;
        out[o] = static_cast<int16_t>(q);
        if (mask) mask[o] = keep;
    }
};

template <class W>
Layout layoutWide(W &ws, int T, int B, int I, int H) {
    const size_t rows = static_cast<size_t>(T) * B, C = 3 * static_cast<size_t>(H);
    const size_t kI = wordsFor(I), kH = wordsFor(H);
    Layout l{};
    l.xPlanes = ws.template take<uint32_t>(rows * 2 * kI);
    l.h0Planes = ws.template take<uint32_t>(static_cast<size_t>(B) * 2 * kH);
    l.wWords = ws.template take<uint32_t>(kI * C);
    l.rWords = ws.template take<uint32_t>(kH * C);
    l.addX = ws.template take<int64_t>(C);
    l.addH = ws.template take<int64_t>(C);
    l.wTiles = ws.template take<uint4>(C * planeproj::paddedK(static_cast<int>(kI)) / 16);
    l.projStatus = ws.template take<int>(1);
    return l;
}

struct SizerAdapter {
    WorkspaceSizer ws;
    template <class T>
    T *take(size_t n) {
        ws.take<T>(n);
        return nullptr;
    }
};

}  // namespace

size_t forwardWideExtraBytes(int T, int B, int I, int H) {
    SizerAdapter s;
    layoutWide(s, T, B, I, H);
    return s.ws.used() + 2048;
}

bool forwardWideTakes(const Exec &e, int I, int H) {
    static const bool disabled = std::getenv("RXMET_GRU_FWD_GENERIC") != nullptr;
    if (disabled || e.weightClass != CodeClass::I8 || e.actClass != CodeClass::I16 || e.linearClass != CodeClass::I16) return false;
    const GateExec &g = e.gate;
    for (int op : {RXMET_GRU_X, RXMET_GRU_H})
        if (static_cast<int64_t>(g.qhi[op]) - g.qlo[op] > 65535) return false;
    return H <= 512 && I <= 1024;
}

void forwardWide(const WideCall &call, const Exec &e, Workspace &ws, cudaStream_t st) {
    const int T = call.T, B = call.B, I = call.I, H = call.H, C = 3 * H;
    const GateExec &g = e.gate;
    const size_t rows = static_cast<size_t>(T) * B;
    const int kI = wordsFor(I), kH = wordsFor(H);
    const Layout l = layoutWide(ws, T, B, I, H);
    const int sms = currentDevice().sms;

    {
        KernelTimer timer__("packWeightWords", st);
        packWeightWords<<<(C + 7) / 8, 256, 0, st>>>(call.wCodes, I, C, kI, g.qlo[RXMET_GRU_X], call.compX, call.biasX, l.wWords, l.addX);
        afterLaunch("packWeightWords");
        packWeightWords<<<(C + 7) / 8, 256, 0, st>>>(call.rCodes, H, C, kH, g.qlo[RXMET_GRU_H], call.compH, call.biasH, l.rWords, l.addH);
        afterLaunch("packWeightWords");
    }
    {
        KernelTimer timer__("planesFromCodes", st);
        planesFromCodes<<<gridFor(rows * kI, 256), 256, 0, st>>>(call.xCodes, rows, I, call.iPad, kI, g.qlo[RXMET_GRU_X], l.xPlanes);
        afterLaunch("planesFromCodes");
        planesFromCodes<<<gridFor(static_cast<size_t>(B) * kH, 256), 256, 0, st>>>(call.h0Codes, static_cast<size_t>(B), H, call.hPad, kH,
                                                                                   g.qlo[RXMET_GRU_H], l.h0Planes);
        afterLaunch("planesFromCodes");
    }
    // Input projection: the tcgen05 kind::i8 kernel when the channel count tiles by 128 and the operands fit
    // shared memory (RXMET_IPROJ_SIMT turns it off), else the dp4a kernel.
    const int kPadI = planeproj::paddedK(kI);
    const int rowsPerTile = planeproj::sharedBytes(kPadI, 2, 128) <= 200 * 1024 ? 128 : 64;
    const bool tensorProjection = C % planeproj::kChannelTile == 0 && planeproj::sharedBytes(kPadI, 2, rowsPerTile) <= 200 * 1024 &&
                                  std::getenv("RXMET_IPROJ_SIMT") == nullptr;
    if (tensorProjection) {
        RXMET_CUDA(cudaMemsetAsync(l.projStatus, 0, sizeof(int), st));
        {
            KernelTimer timer__("packWeightWords", st);
            planeproj::packTiles<<<gridFor(static_cast<size_t>(C) * kPadI / 16, 256), 256, 0, st>>>(l.wWords, kI, C, kPadI, l.wTiles);
            afterLaunch("packTiles");
        }
        planeproj::Problem pp{};
        pp.planes = l.xPlanes; pp.rows = static_cast<int>(rows); pp.kWords = kI; pp.tiles = l.wTiles; pp.C = C; pp.status = l.projStatus;
        PlaneEpilogue epi{};
        epi.addend = l.addX; epi.rescale = call.gemmX;
        epi.zpOut = g.zp[RXMET_GRU_WEIGHT_IH_LINEAR]; epi.lo = g.qlo[RXMET_GRU_WEIGHT_IH_LINEAR]; epi.hi = g.qhi[RXMET_GRU_WEIGHT_IH_LINEAR];
        epi.out = call.ihCodes; epi.mask = call.maskIh; epi.C = C;
        const size_t smem = planeproj::sharedBytes(kPadI, 2, rowsPerTile);
        const int rowTiles = static_cast<int>((rows + rowsPerTile - 1) / rowsPerTile);
        const int grid = std::max(1, std::min(rowTiles, smsPerPass()));
        auto launchTensor = [&](auto kernel) {
            ensureDynamicSmem(reinterpret_cast<const void *>(kernel), smem);
            KernelTimer timer__("inputLinear", st);
            kernel<<<grid, planeproj::kThreads, smem, st>>>(pp, epi);
        };
        if (rowsPerTile == 128) launchTensor(planeproj::planeProjUmma<PlaneEpilogue, 2, 128>);
        else launchTensor(planeproj::planeProjUmma<PlaneEpilogue, 2, 64>);
        afterLaunch("inputLinear");
    } else {
        InputArgs a{};
        a.rows = static_cast<int>(rows); a.C = C; a.kWords = kI;
        a.x = l.xPlanes; a.words = l.wWords; a.addend = l.addX; a.rescale = call.gemmX;
        a.zpOut = g.zp[RXMET_GRU_WEIGHT_IH_LINEAR]; a.lo = g.qlo[RXMET_GRU_WEIGHT_IH_LINEAR]; a.hi = g.qhi[RXMET_GRU_WEIGHT_IH_LINEAR];
        a.out = call.ihCodes; a.mask = call.maskIh;
        const int block = std::min(kThreads, (C + 31) / 32 * 32);
        const int slabs = (C + block - 1) / block;
        const int blocks = static_cast<int>((rows + kRowsPerBlock - 1) / kRowsPerBlock);
        const size_t smem = sizeof(uint32_t) * 2 * kRowsPerBlock * 2 * kI;
        auto launch = [&](auto kernel) {
            ensureDynamicSmem(reinterpret_cast<const void *>(kernel), smem);
            const int perSm = residentPerSm(reinterpret_cast<const void *>(kernel), block, smem);
            const int grid = std::max(1, std::min(blocks, std::max(1, sms * perSm / slabs)));
            KernelTimer timer__("inputLinear", st);
            kernel<<<dim3(grid, slabs), block, smem, st>>>(a);
        };
        if (kI <= 16) launch(inputLinearPlanes<16, false>);
        else if (kI <= 32) launch(inputLinearPlanes<32, false>);
        else launch(inputLinearPlanes<32, true>);
        afterLaunch("inputLinear");
    }
    {
        RecurrentArgs a{};
        a.T = T; a.B = B; a.H = H; a.HP = (H + 31) / 32 * 32; a.kWords = kH;
        a.words = l.rWords; a.addend = l.addH; a.rescale = call.gemmH; a.ih = call.ihCodes;
        a.h0 = call.h0Codes; a.hPad = call.hPad; a.h0Planes = l.h0Planes;
        a.h = call.h; a.v = call.v; a.hq = call.hq; a.vq = call.vq;
        a.maskHh = call.maskHh; a.maskGateIn = call.maskGateIn; a.maskGateOut = call.maskGateOut; a.maskH = call.maskH;
        a.poison = tensorProjection ? l.projStatus : nullptr;
        const int groupsMax = std::max(1, kThreads / a.HP);
        const int want = std::max(1, (B + smsPerPass() - 1) / smsPerPass());
        int rb = 1;
        while (rb < 4 && rb * groupsMax < want) rb *= 2;
        const int groups = std::max(1, std::min(groupsMax, (want + rb - 1) / rb));
        const int bt = groups * rb, block = groups * a.HP;
        const size_t planeBytes = sizeof(uint32_t) * 2 * bt * 2 * kH;
        const size_t weightBytes = sizeof(uint32_t) * static_cast<size_t>(kH) * C;
        const bool weightsInSmem = planeBytes + weightBytes + 2048 <= static_cast<size_t>(currentDevice().smemMax);   // + the kernel's static copy of the gate parameters
        a.weightBytesInSmem = weightsInSmem ? static_cast<int>(weightBytes) : 0;
        const size_t smem = planeBytes + (weightsInSmem ? weightBytes : 0);
        auto launch = [&](auto kernel) {
            ensureDynamicSmem(reinterpret_cast<const void *>(kernel), smem);
            KernelTimer timer__("recurrentForward", st);
            kernel<<<(B + bt - 1) / bt, block, smem, st>>>(a, g);
        };
#define RXMET_GRU_WIDE(RBV)                                         \
    do {                                                             \
        if (weightsInSmem) launch(recurrentPlanes<RBV, true>);       \
        else launch(recurrentPlanes<RBV, false>);                    \
    } while (0)
        if (rb == 1) RXMET_GRU_WIDE(1);
        else if (rb == 2) RXMET_GRU_WIDE(2);
        else RXMET_GRU_WIDE(4);
#undef RXMET_GRU_WIDE
        afterLaunch("recurrentForward");
    }
}

}  // namespace gru
}  // namespace rxmet
