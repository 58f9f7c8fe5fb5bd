// Learned-grid quantize-dequantize of the affine quantizers (aimet_torch.v2), forward and backward,
// one pass over the tensor each.
//
//   divide form      (QuantDequantFunc, torch_builtins.py:618-691)
//     t = rne(x / s) - o;  keep = qmin <= t <= qmax;  y = (clamp(t, qmin, qmax) + o) * s
//     dx = g * keep
//     ds = sum g * (clamp(rne(x / s), o + qmin, o + qmax) - (x / s) * keep)
//     do = sum g * (!keep * s)
//   reciprocal form  (the fake-quantize fast path taken when the grid is not trained, torch_builtins.py:199-250)
//     q = int64(rne(x * (1 / s)) + zp), zp = -int32(o);  keep = qmin <= q <= qmax
//     y = float(clamp(q, qmin, qmax) - zp) * s;  NaN inputs stay NaN;  dx = g * keep
//
// Every float operation is a separately rounded IEEE operation, as in the eager reference (no fused
// multiply-add, no approximate division), so y, keep and dx are bit-exact; ds and do are float sums whose
// order differs from the reference's.
//
// The tensor is viewed as [outer][channels][inner] with one (s, o) pair per channel; channels == 1 is the
// per-tensor grid.  HBM-bound: the forward moves 8 bytes per element, the backward 12, and the sums ride
// along: per-CTA partials land in a small workspace and a second launch adds them in a fixed order, so the
// result does not change from run to run.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <mutex>
#include <unordered_map>

#include "common.h"
#include "rxmet_b200.h"

namespace rxmet {
namespace affine {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxResident = 2048 / kThreads;   // CTAs of kThreads threads an SM can hold
constexpr int kSegment = 8192;     // elements of one row handled by one CTA pass (long rows)
constexpr int kChunkRows = 32;     // rows of one CTA tile (short rows)
constexpr int kBatchForward = 4;   // rows whose loads are in flight together (short rows)
constexpr int kBatchBackward = 2;  // two tensors are read there
constexpr int kLongRow = 256;      // rows at least this long take the row kernel

struct Grid {
    const float *scale;
    const float *offset;
    float lo, hi;        // qmin, qmax as floats (|q| < 2^24 is checked on the host)
    int qmin, qmax;
};

struct Element {
    float y;
    float keep;   // 1 or 0
};

template <bool kReciprocal>
__device__ __forceinline__ Element quantDequant(float x, float s, float inv, float o, float zp, const Grid &g) {
    Element e;
    if constexpr (kReciprocal) {
        // The reference converts r to int64 (saturating), clamps and subtracts zp as integers.  r is an integer
        // or infinite, qmin / qmax / zp are exact floats, and both float(int64 difference) and the float
        // subtraction round the same exact integer, so the float domain gives the same bits without 64-bit work.
        const float r = __fadd_rn(nearbyintf(__fmul_rn(x, inv)), zp);
        const bool nan = x != x;
        const bool keep = g.lo <= r && r <= g.hi;    // false for NaN
        const float c = fminf(fmaxf(r, g.lo), g.hi);
        e.y = nan ? x : __fmul_rn(__fsub_rn(c, zp), s);
        e.keep = keep ? 1.0f : 0.0f;
    } else {
        const float t = __fsub_rn(nearbyintf(__fdiv_rn(x, s)), o);
        const bool keep = g.lo <= t && t <= g.hi;    // false for NaN
        const float c = t != t ? t : fminf(fmaxf(t, g.lo), g.hi);
        e.y = __fmul_rn(__fadd_rn(c, o), s);
        e.keep = keep ? 1.0f : 0.0f;
    }
    return e;
}

struct Sums {
    float scale = 0.0f, offset = 0.0f;
};

// Backward of one element in the divide form; returns dx.
__device__ __forceinline__ float backwardOne(float x, float gr, float s, float o, const Grid &g, Sums &acc) {
    const float xs = __fdiv_rn(x, s);
    const float q = nearbyintf(xs);
    const float t = __fsub_rn(q, o);
    const bool keep = g.lo <= t && t <= g.hi;
    const float m = keep ? 1.0f : 0.0f;
    const float lo = __fadd_rn(o, g.lo), hi = __fadd_rn(o, g.hi);
    const float qc = fminf(fmaxf(q, lo), hi);   // a NaN input reaches the sum through xs * m below
    acc.scale = __fadd_rn(acc.scale, __fmul_rn(gr, __fsub_rn(qc, __fmul_rn(xs, m))));
    acc.offset = __fadd_rn(acc.offset, __fmul_rn(gr, keep ? 0.0f : s));
    return __fmul_rn(gr, m);
}

// One partial per warp: no CTA-wide barrier between work items.
__device__ __forceinline__ void writeWarpPartial(Sums acc, float *partial, uint64_t at) {
    for (int d = 16; d > 0; d >>= 1) {
        acc.scale += __shfl_down_sync(0xffffffffu, acc.scale, d);
        acc.offset += __shfl_down_sync(0xffffffffu, acc.offset, d);
    }
    if ((threadIdx.x & 31) == 0) {
        partial[2 * at] = acc.scale;
        partial[2 * at + 1] = acc.offset;
    }
}

struct Pass {
    const float *x;
    const float *grad;      // backward only
    float *out;             // y (forward) or dx (backward); may be null in a backward that only wants sums
    uint8_t *keep;          // forward, optional: 1 where the value was inside the grid
    float *partial;         // backward, optional: [items][2]
    float *dscale, *doffset;   // backward, block pass only: the sums of a row are the final result
    uint64_t outer, channels, inner;
    int wantSums;
};

// Long rows: one work item = one segment of one row (a row is `inner` contiguous elements of one channel).
template <bool kBackward, bool kReciprocal>
__global__ void __launch_bounds__(kThreads) rowPass(Pass p, Grid g, uint64_t segments, int vector) {
    const uint64_t rows = p.outer * p.channels;
    // A per-tensor grid has one channel, so a warp keeps its sums across all its work items and writes one
    // partial at the end; otherwise every work item writes its own.
    const bool perTensor = rows == 1;
    Sums acc;
    for (uint64_t item = blockIdx.x; item < rows * segments; item += gridDim.x) {
        const uint64_t row = item / segments, seg = item - row * segments;
        const uint64_t c = row % p.channels;
        const float s = __ldg(g.scale + c), o = __ldg(g.offset + c);
        const float inv = __fdiv_rn(1.0f, s);
        const float zp = static_cast<float>(-static_cast<int>(o));   // zero point of the fast form: -int32(o)
        const uint64_t begin = row * p.inner + seg * kSegment;
        const int count = static_cast<int>(min(static_cast<uint64_t>(kSegment), p.inner - seg * kSegment));
        if (!perTensor) acc = Sums();
        if (vector) {
            // restrict: the loads of the next iterations may move above this iteration's store, so several
            // 16-byte requests per thread are in flight
            const float4 *__restrict__ x4 = reinterpret_cast<const float4 *>(p.x + begin);
            const float4 *__restrict__ g4 = kBackward ? reinterpret_cast<const float4 *>(p.grad + begin) : nullptr;
            float4 *__restrict__ o4 = p.out ? reinterpret_cast<float4 *>(p.out + begin) : nullptr;
            uint32_t *__restrict__ k4 = p.keep ? reinterpret_cast<uint32_t *>(p.keep + begin) : nullptr;
#pragma unroll(kBackward ? 2 : 1)
            for (int v = threadIdx.x; v < count / 4; v += kThreads) {
                const float4 xv = __ldcs(x4 + v);
                float in[4] = {xv.x, xv.y, xv.z, xv.w}, res[4];
                if constexpr (kBackward) {
                    const float4 gv = __ldcs(g4 + v);
                    const float gr[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        if (kReciprocal) res[k] = __fmul_rn(gr[k], quantDequant<true>(in[k], s, inv, o, zp, g).keep);
                        else res[k] = backwardOne(in[k], gr[k], s, o, g, acc);
                    }
                } else {
                    uint32_t bits = 0;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const Element e = quantDequant<kReciprocal>(in[k], s, inv, o, zp, g);
                        res[k] = e.y;
                        bits |= (e.keep != 0.0f ? 1u : 0u) << (8 * k);
                    }
                    if (k4) k4[v] = bits;
                }
                if (o4) __stcs(o4 + v, make_float4(res[0], res[1], res[2], res[3]));
            }
        } else {
            for (int i = threadIdx.x; i < count; i += kThreads) {
                const float xv = p.x[begin + i];
                float res;
                if constexpr (kBackward) {
                    const float gr = p.grad[begin + i];
                    if (kReciprocal) res = __fmul_rn(gr, quantDequant<true>(xv, s, inv, o, zp, g).keep);
                    else res = backwardOne(xv, gr, s, o, g, acc);
                } else {
                    const Element e = quantDequant<kReciprocal>(xv, s, inv, o, zp, g);
                    res = e.y;
                    if (p.keep) p.keep[begin + i] = e.keep != 0.0f;
                }
                if (p.out) p.out[begin + i] = res;
            }
        }
        if constexpr (kBackward) {
            if (p.wantSums && !perTensor) writeWarpPartial(acc, p.partial, item * kWarps + (threadIdx.x >> 5));
        }
    }
    if constexpr (kBackward) {
        if (p.wantSums && perTensor)
            writeWarpPartial(acc, p.partial, static_cast<uint64_t>(blockIdx.x) * kWarps + (threadIdx.x >> 5));
    }
}

// Short rows: the tensor is a matrix [outer][channels * inner].  A thread owns kVec adjacent columns (their
// channels, scales and sums stay in registers) and walks down kChunkRows rows, so a warp reads 128 * kVec
// contiguous bytes per row and nothing is reduced across threads.  Narrow matrices fold several row chunks
// into one CTA: colThreads threads across, 256 / colThreads chunks down.
template <bool kBackward, bool kReciprocal, int kVec>
__global__ void __launch_bounds__(kThreads, 4) columnPass(Pass p, Grid g, int colThreads) {
    const uint64_t period = p.channels * p.inner;
    const int tx = threadIdx.x % colThreads, ty = threadIdx.x / colThreads, down = kThreads / colThreads;
    const uint64_t col = (static_cast<uint64_t>(blockIdx.x) * colThreads + tx) * kVec;
    if (col >= period) return;
    float s[kVec], o[kVec], inv[kVec], zp[kVec];
#pragma unroll
    for (int k = 0; k < kVec; ++k) {
        const uint64_t c = (col + k) / p.inner;
        s[k] = __ldg(g.scale + c);
        o[k] = __ldg(g.offset + c);
        inv[k] = __fdiv_rn(1.0f, s[k]);
        zp[k] = static_cast<float>(-static_cast<int>(o[k]));
    }
    constexpr int kBatch = kBackward ? kBatchBackward : kBatchForward;
    const float *__restrict__ xIn = p.x;
    const float *__restrict__ gIn = p.grad;
    float *__restrict__ out = p.out;
    uint8_t *__restrict__ keepOut = p.keep;
    const uint64_t chunks = (p.outer + kChunkRows - 1) / kChunkRows;
    for (uint64_t chunk = static_cast<uint64_t>(blockIdx.y) * down + ty; chunk < chunks;
         chunk += static_cast<uint64_t>(gridDim.y) * down) {
        const uint64_t first = chunk * kChunkRows, last = min(first + kChunkRows, p.outer);
        Sums acc[kVec];
        for (uint64_t r0 = first; r0 < last; r0 += kBatch) {
            // all loads of a batch of rows are issued before the first result is needed
            float in[kBatch][kVec], gr[kBatch][kVec];
#pragma unroll
            for (int b = 0; b < kBatch; ++b) {
                if (r0 + b >= last) break;
                const uint64_t at = (r0 + b) * period + col;
                if constexpr (kVec == 4) {
                    const float4 xv = __ldcs(reinterpret_cast<const float4 *>(xIn + at));
                    in[b][0] = xv.x; in[b][1] = xv.y; in[b][2] = xv.z; in[b][3] = xv.w;
                    if constexpr (kBackward) {
                        const float4 gv = __ldcs(reinterpret_cast<const float4 *>(gIn + at));
                        gr[b][0] = gv.x; gr[b][1] = gv.y; gr[b][2] = gv.z; gr[b][3] = gv.w;
                    }
                } else {
                    in[b][0] = __ldcs(xIn + at);
                    if constexpr (kBackward) gr[b][0] = __ldcs(gIn + at);
                }
            }
#pragma unroll
            for (int b = 0; b < kBatch; ++b) {
                if (r0 + b >= last) break;
                const uint64_t at = (r0 + b) * period + col;
                float res[kVec];
                uint32_t bits = 0;
#pragma unroll
                for (int k = 0; k < kVec; ++k) {
                    if constexpr (kBackward) {
                        if (kReciprocal) res[k] = __fmul_rn(gr[b][k], quantDequant<true>(in[b][k], s[k], inv[k], o[k], zp[k], g).keep);
                        else res[k] = backwardOne(in[b][k], gr[b][k], s[k], o[k], g, acc[k]);
                    } else {
                        const Element e = quantDequant<kReciprocal>(in[b][k], s[k], inv[k], o[k], zp[k], g);
                        res[k] = e.y;
                        bits |= (e.keep != 0.0f ? 1u : 0u) << (8 * k);
                    }
                }
                if constexpr (!kBackward) {
                    if (keepOut) {
                        if constexpr (kVec == 4) *reinterpret_cast<uint32_t *>(keepOut + at) = bits;
                        else keepOut[at] = static_cast<uint8_t>(bits);
                    }
                }
                if (out) {
                    if constexpr (kVec == 4) __stcs(reinterpret_cast<float4 *>(out + at), make_float4(res[0], res[1], res[2], res[3]));
                    else __stcs(out + at, res[0]);
                }
            }
        }
        if constexpr (kBackward) {
            if (p.wantSums) {
#pragma unroll
                for (int k = 0; k < kVec; ++k) {
                    p.partial[2 * (chunk * period + col + k)] = acc[k].scale;
                    p.partial[2 * (chunk * period + col + k) + 1] = acc[k].offset;
                }
            }
        }
    }
}

// Short rows that are whole grid entries (outer == 1: blockwise weights, per-channel grids of short rows): a
// group of lanesPerRow lanes (a power of two up to 32) owns one row, so a warp reads 32 / lanesPerRow adjacent
// rows = one contiguous stretch, and the sums of a row, reduced with shuffles inside the group, are the final
// dscale / doffset of its entry: no workspace, no second launch.
template <bool kBackward, bool kReciprocal>
__global__ void __launch_bounds__(kThreads) blockPass(Pass p, Grid g, int lanesPerRow, int vector) {
    const uint64_t rows = p.channels;   // outer == 1
    const int lane = threadIdx.x & 31, sub = lane / lanesPerRow, sl = lane % lanesPerRow;
    const int rowsPerWarp = 32 / lanesPerRow;
    const uint64_t warps = static_cast<uint64_t>(gridDim.x) * kWarps;
    const float *__restrict__ xIn = p.x;
    const float *__restrict__ gIn = p.grad;
    float *__restrict__ out = p.out;
    uint8_t *__restrict__ keepOut = p.keep;
    const uint64_t warpId = static_cast<uint64_t>(blockIdx.x) * kWarps + (threadIdx.x >> 5);
    if (vector && p.inner / 4 <= static_cast<uint64_t>(lanesPerRow)) {
        // At most one 16-byte piece per lane and row (rows of up to 128 elements): a warp takes two adjacent
        // stretches of rows per turn and issues all their loads before the first result is needed.
        const bool has = static_cast<uint64_t>(sl) < p.inner / 4;
        for (uint64_t base = warpId * rowsPerWarp * 2; base < rows; base += warps * rowsPerWarp * 2) {
            uint64_t row[2], at[2];
            bool live[2];
            float4 xv[2], gv[2];
            float s[2], o[2];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                row[j] = base + static_cast<uint64_t>(j) * rowsPerWarp + sub;
                live[j] = has && row[j] < rows;
                at[j] = row[j] * p.inner + 4 * static_cast<uint64_t>(sl);
                if (live[j]) {
                    xv[j] = __ldcs(reinterpret_cast<const float4 *>(xIn + at[j]));
                    if constexpr (kBackward) gv[j] = __ldcs(reinterpret_cast<const float4 *>(gIn + at[j]));
                    s[j] = __ldg(g.scale + row[j]);
                    o[j] = __ldg(g.offset + row[j]);
                }
            }
            Sums acc[2];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                if (!live[j]) continue;
                const float inv = __fdiv_rn(1.0f, s[j]);
                const float zp = static_cast<float>(-static_cast<int>(o[j]));
                const float in[4] = {xv[j].x, xv[j].y, xv[j].z, xv[j].w};
                float res[4];
                if constexpr (kBackward) {
                    const float gr[4] = {gv[j].x, gv[j].y, gv[j].z, gv[j].w};
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        if (kReciprocal) res[k] = __fmul_rn(gr[k], quantDequant<true>(in[k], s[j], inv, o[j], zp, g).keep);
                        else res[k] = backwardOne(in[k], gr[k], s[j], o[j], g, acc[j]);
                    }
                } else {
                    uint32_t bits = 0;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const Element e = quantDequant<kReciprocal>(in[k], s[j], inv, o[j], zp, g);
                        res[k] = e.y;
                        bits |= (e.keep != 0.0f ? 1u : 0u) << (8 * k);
                    }
                    if (keepOut) *reinterpret_cast<uint32_t *>(keepOut + at[j]) = bits;
                }
                if (out) __stcs(reinterpret_cast<float4 *>(out + at[j]), make_float4(res[0], res[1], res[2], res[3]));
            }
            if constexpr (kBackward) {
                if (p.wantSums) {
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        for (int d = lanesPerRow >> 1; d > 0; d >>= 1) {
                            acc[j].scale += __shfl_down_sync(0xffffffffu, acc[j].scale, d, lanesPerRow);
                            acc[j].offset += __shfl_down_sync(0xffffffffu, acc[j].offset, d, lanesPerRow);
                        }
                        if (sl == 0 && row[j] < rows) {
                            if (p.dscale) p.dscale[row[j]] = acc[j].scale;
                            if (p.doffset) p.doffset[row[j]] = acc[j].offset;
                        }
                    }
                }
            }
        }
        return;
    }
    for (uint64_t base = warpId * rowsPerWarp; base < rows; base += warps * rowsPerWarp) {
        const uint64_t row = base + sub;
        const bool live = row < rows;
        Sums acc;
        if (live) {
            const float s = __ldg(g.scale + row), o = __ldg(g.offset + row);
            const float inv = __fdiv_rn(1.0f, s);
            const float zp = static_cast<float>(-static_cast<int>(o));
            const uint64_t begin = row * p.inner;
            if (vector) {
                for (uint64_t v = sl; v < p.inner / 4; v += lanesPerRow) {
                    const uint64_t at = begin + 4 * v;
                    const float4 xv = __ldcs(reinterpret_cast<const float4 *>(xIn + at));
                    const float in[4] = {xv.x, xv.y, xv.z, xv.w};
                    float res[4];
                    if constexpr (kBackward) {
                        const float4 gv = __ldcs(reinterpret_cast<const float4 *>(gIn + at));
                        const float gr[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            if (kReciprocal) res[k] = __fmul_rn(gr[k], quantDequant<true>(in[k], s, inv, o, zp, g).keep);
                            else res[k] = backwardOne(in[k], gr[k], s, o, g, acc);
                        }
                    } else {
                        uint32_t bits = 0;
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const Element e = quantDequant<kReciprocal>(in[k], s, inv, o, zp, g);
                            res[k] = e.y;
                            bits |= (e.keep != 0.0f ? 1u : 0u) << (8 * k);
                        }
                        if (keepOut) *reinterpret_cast<uint32_t *>(keepOut + at) = bits;
                    }
                    if (out) __stcs(reinterpret_cast<float4 *>(out + at), make_float4(res[0], res[1], res[2], res[3]));
                }
            } else {
                for (uint64_t i = sl; i < p.inner; i += lanesPerRow) {
                    const uint64_t at = begin + i;
                    const float xv = __ldcs(xIn + at);
                    float res;
                    if constexpr (kBackward) {
                        const float gr = __ldcs(gIn + at);
                        if (kReciprocal) res = __fmul_rn(gr, quantDequant<true>(xv, s, inv, o, zp, g).keep);
                        else res = backwardOne(xv, gr, s, o, g, acc);
                    } else {
                        const Element e = quantDequant<kReciprocal>(xv, s, inv, o, zp, g);
                        res = e.y;
                        if (keepOut) keepOut[at] = e.keep != 0.0f;
                    }
                    if (out) __stcs(out + at, res);
                }
            }
        }
        if constexpr (kBackward) {
            if (p.wantSums) {
                for (int d = lanesPerRow >> 1; d > 0; d >>= 1) {   // every lane takes part, dead rows add zeros
                    acc.scale += __shfl_down_sync(0xffffffffu, acc.scale, d, lanesPerRow);
                    acc.offset += __shfl_down_sync(0xffffffffu, acc.offset, d, lanesPerRow);
                }
                if (live && sl == 0) {
                    if (p.dscale) p.dscale[row] = acc.scale;
                    if (p.doffset) p.doffset[row] = acc.offset;
                }
            }
        }
    }
}

// dscale[c], doffset[c] = sum over a < groups, b < run of partial[a * groupStride + c * run + b], in that order
// per thread and then over the threads of the CTA: the same order on every run.
__global__ void __launch_bounds__(128) finishSums(const float *partial, uint64_t groups, uint64_t groupStride, uint64_t run,
                                                  float *dscale, float *doffset) {
    const uint64_t c = blockIdx.x;
    double s = 0.0, o = 0.0;
    for (uint64_t k = threadIdx.x; k < groups * run; k += blockDim.x) {
        const uint64_t a = k / run, b = k - a * run;
        const uint64_t at = a * groupStride + c * run + b;
        s += static_cast<double>(partial[2 * at]);
        o += static_cast<double>(partial[2 * at + 1]);
    }
    __shared__ double part[2][4];
    for (int d = 16; d > 0; d >>= 1) {
        s += __shfl_down_sync(0xffffffffu, s, d);
        o += __shfl_down_sync(0xffffffffu, o, d);
    }
    if ((threadIdx.x & 31) == 0) { part[0][threadIdx.x >> 5] = s; part[1][threadIdx.x >> 5] = o; }
    __syncthreads();
    if (threadIdx.x == 0) {
        if (dscale) dscale[c] = static_cast<float>(part[0][0] + part[0][1] + part[0][2] + part[0][3]);
        if (doffset) doffset[c] = static_cast<float>(part[1][0] + part[1][1] + part[1][2] + part[1][3]);
    }
}

struct Plan {
    bool rows;              // row kernel or column kernel
    bool blocks;            // block kernel: short rows that are whole grid entries; nothing else is set then
    uint64_t segments;      // row kernel: segments per row
    uint64_t chunks;        // column kernel: row chunks
    uint64_t items;         // partial entries
};

Plan planFor(uint64_t outer, uint64_t channels, uint64_t inner) {
    Plan plan{};
    plan.rows = channels == 1 || inner >= kLongRow;
    plan.blocks = !plan.rows && outer == 1;
    if (plan.blocks) {
        plan.items = 0;
    } else if (plan.rows) {
        plan.segments = (inner + kSegment - 1) / kSegment;
        // one partial per warp and segment; per tensor one per warp of the grid (at most kMaxResident CTAs per SM)
        plan.items = outer * channels == 1 ? static_cast<uint64_t>(currentDevice().sms) * kMaxResident * kWarps
                                           : outer * channels * plan.segments * kWarps;
    } else {
        plan.chunks = (outer + kChunkRows - 1) / kChunkRows;
        plan.items = plan.chunks * channels * inner;
    }
    return plan;
}

void checkGrid(int qmin, int qmax) {
    RXMET_REQUIRE(qmin < qmax, "affine qdq: qmin must be below qmax");
    RXMET_REQUIRE(qmin > -(1 << 24) && qmax < (1 << 24), "affine qdq: the code range must be exact in float (|q| < 2^24)");
}

// CTAs of `kernel` one SM holds; asked once per kernel.
template <class Kernel>
int residentCtas(Kernel kernel) {
    static std::mutex lock;
    static std::unordered_map<const void *, int> known;
    std::lock_guard<std::mutex> hold(lock);
    int &n = known[reinterpret_cast<const void *>(kernel)];
    if (n == 0) {
        RXMET_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, kThreads, 0));
        n = std::max(n, 1);
    }
    return n;
}

// Returns the number of CTAs of the row pass (0 for the column pass).
template <bool kBackward>
int run(Pass p, Grid g, int reciprocal, const Plan &plan, cudaStream_t st) {
    int rowGrid = 0;
    const DeviceInfo dev = currentDevice();
    if (plan.blocks) {
        const bool vector = p.inner % 4 == 0 && (reinterpret_cast<uintptr_t>(p.x) & 15) == 0 &&
                            (!p.grad || (reinterpret_cast<uintptr_t>(p.grad) & 15) == 0) &&
                            (!p.out || (reinterpret_cast<uintptr_t>(p.out) & 15) == 0) &&
                            (!p.keep || (reinterpret_cast<uintptr_t>(p.keep) & 3) == 0);
        const uint64_t lanes = vector ? p.inner / 4 : p.inner;
        int lanesPerRow = 1;
        while (lanesPerRow < 32 && static_cast<uint64_t>(lanesPerRow) < lanes) lanesPerRow *= 2;
        const uint64_t warpsNeeded = (p.channels + 32 / lanesPerRow - 1) / (32 / lanesPerRow);
        auto launch = [&](auto kernel) {
            const uint64_t ctas = (warpsNeeded + kWarps - 1) / kWarps;
            const int grid = static_cast<int>(std::min<uint64_t>(
                ctas, static_cast<uint64_t>(dev.sms) * std::min(residentCtas(kernel), kMaxResident)));
            kernel<<<grid, kThreads, 0, st>>>(p, g, lanesPerRow, vector ? 1 : 0);
        };
        if (reciprocal) launch(blockPass<kBackward, true>);
        else launch(blockPass<kBackward, false>);
        afterLaunch("affineBlockPass");
    } else if (plan.rows) {
        // per tensor the whole tensor is one row: `outer` and `channels` fold into it on the host
        const bool aligned = p.inner % 4 == 0 && (reinterpret_cast<uintptr_t>(p.x) & 15) == 0 &&
                             (!p.grad || (reinterpret_cast<uintptr_t>(p.grad) & 15) == 0) &&
                             (!p.out || (reinterpret_cast<uintptr_t>(p.out) & 15) == 0) &&
                             (!p.keep || (reinterpret_cast<uintptr_t>(p.keep) & 3) == 0);
        const uint64_t items = p.outer * p.channels * plan.segments;
        auto launch = [&](auto kernel) {
            // exactly one wave of resident CTAs, so that every CTA walks the same number of work items
            const int grid = static_cast<int>(std::min<uint64_t>(
                items, static_cast<uint64_t>(dev.sms) * std::min(residentCtas(kernel), kMaxResident)));
            kernel<<<grid, kThreads, 0, st>>>(p, g, plan.segments, aligned ? 1 : 0);
            rowGrid = grid;
        };
        if (reciprocal) launch(rowPass<kBackward, true>);
        else launch(rowPass<kBackward, false>);
        afterLaunch("affineRowPass");
    } else {
        const uint64_t period = p.channels * p.inner;
        const bool vec4 = period % 4 == 0 && (reinterpret_cast<uintptr_t>(p.x) & 15) == 0 &&
                          (!p.grad || (reinterpret_cast<uintptr_t>(p.grad) & 15) == 0) &&
                          (!p.out || (reinterpret_cast<uintptr_t>(p.out) & 15) == 0) &&
                          (!p.keep || (reinterpret_cast<uintptr_t>(p.keep) & 3) == 0);
        const uint64_t lanes = vec4 ? period / 4 : period;             // threads one row needs
        int colThreads = 32;
        while (colThreads < kThreads && static_cast<uint64_t>(colThreads) < lanes) colThreads *= 2;
        const int down = kThreads / colThreads;                        // row chunks per CTA
        const unsigned gx = static_cast<unsigned>((lanes + colThreads - 1) / colThreads);
        const uint64_t blocksDown = (plan.chunks + down - 1) / down;
        auto launch = [&](auto kernel) {
            const uint64_t want = std::max<uint64_t>(1, static_cast<uint64_t>(dev.sms) * residentCtas(kernel) / gx);
            const unsigned gy = static_cast<unsigned>(std::min<uint64_t>(std::min<uint64_t>(blocksDown, want), 65535));
            kernel<<<dim3(gx, gy), kThreads, 0, st>>>(p, g, colThreads);
        };
        if (vec4) {
            if (reciprocal) launch(columnPass<kBackward, true, 4>);
            else launch(columnPass<kBackward, false, 4>);
        } else {
            if (reciprocal) launch(columnPass<kBackward, true, 1>);
            else launch(columnPass<kBackward, false, 1>);
        }
        afterLaunch("affineColumnPass");
    }
    return rowGrid;
}

}  // namespace
}  // namespace affine
}  // namespace rxmet

using namespace rxmet;
using namespace rxmet::affine;

extern "C" {

int rxmet_affine_qdq_forward(const float *x_dev, uint64_t outer, uint64_t channels, uint64_t inner, const float *scale_dev,
                             const float *offset_dev, int qmin, int qmax, int reciprocal, float *y_dev, uint8_t *keep_dev,
                             void *stream) {
    return guarded([&] {
        if (outer * channels * inner == 0) return;
        RXMET_REQUIRE(x_dev && y_dev && scale_dev && offset_dev, "affine qdq forward: null tensor");
        checkGrid(qmin, qmax);
        Pass p{};
        p.x = x_dev; p.out = y_dev; p.keep = keep_dev;
        p.outer = outer; p.channels = channels; p.inner = inner;
        if (channels == 1) { p.inner = outer * inner; p.outer = 1; }
        const Grid g{scale_dev, offset_dev, static_cast<float>(qmin), static_cast<float>(qmax), qmin, qmax};
        run<false>(p, g, reciprocal, planFor(p.outer, p.channels, p.inner), static_cast<cudaStream_t>(stream));
    });
}

size_t rxmet_affine_qdq_backward_workspace_bytes(uint64_t outer, uint64_t channels, uint64_t inner) {
    if (channels == 1) { inner = outer * inner; outer = 1; }
    return static_cast<size_t>(planFor(outer, channels, inner).items) * 2 * sizeof(float);
}

int rxmet_affine_qdq_backward(const float *grad_dev, const float *x_dev, uint64_t outer, uint64_t channels, uint64_t inner,
                              const float *scale_dev, const float *offset_dev, int qmin, int qmax, int reciprocal,
                              float *dx_dev, float *dscale_dev, float *doffset_dev, void *workspace_dev,
                              size_t workspace_bytes, void *stream) {
    return guarded([&] {
        if (outer * channels * inner == 0) return;
        RXMET_REQUIRE(grad_dev && x_dev && scale_dev && offset_dev, "affine qdq backward: null tensor");
        RXMET_REQUIRE(dx_dev || dscale_dev || doffset_dev, "affine qdq backward: no gradient was asked for");
        checkGrid(qmin, qmax);
        const bool sums = dscale_dev || doffset_dev;
        RXMET_REQUIRE(!(sums && reciprocal), "affine qdq backward: the reciprocal form has no grid gradients");
        Pass p{};
        p.x = x_dev; p.grad = grad_dev; p.out = dx_dev;
        p.outer = outer; p.channels = channels; p.inner = inner;
        if (channels == 1) { p.inner = outer * inner; p.outer = 1; }
        const Plan plan = planFor(p.outer, p.channels, p.inner);
        if (sums && plan.blocks) {
            p.dscale = dscale_dev; p.doffset = doffset_dev;
            p.wantSums = 1;
        } else if (sums) {
            RXMET_REQUIRE(workspace_dev && workspace_bytes >= plan.items * 2 * sizeof(float),
                          "affine qdq backward: workspace of %zu bytes needed", static_cast<size_t>(plan.items * 2 * sizeof(float)));
            p.partial = static_cast<float *>(workspace_dev);
            p.wantSums = 1;
        }
        const Grid g{scale_dev, offset_dev, static_cast<float>(qmin), static_cast<float>(qmax), qmin, qmax};
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        const int rowGrid = run<true>(p, g, reciprocal, plan, st);
        if (sums && !plan.blocks) {
            if (plan.rows && p.outer * p.channels == 1)
                finishSums<<<1, 128, 0, st>>>(p.partial, 1, 0, static_cast<uint64_t>(rowGrid) * kWarps, dscale_dev, doffset_dev);
            else if (plan.rows)
                finishSums<<<static_cast<unsigned>(p.channels), 128, 0, st>>>(p.partial, p.outer, p.channels * plan.segments * kWarps,
                                                                              plan.segments * kWarps, dscale_dev, doffset_dev);
            else
                finishSums<<<static_cast<unsigned>(p.channels), 128, 0, st>>>(p.partial, plan.chunks, p.channels * p.inner,
                                                                              p.inner, dscale_dev, doffset_dev);
            afterLaunch("affineFinishSums");
        }
    });
}

}  // extern "C"
