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

#include "common.h"
#include "rxmet_b200.h"

namespace rxmet {
namespace affine {
namespace {

constexpr int kThreads = 256;
constexpr int kSegment = 8192;     // elements of one row handled by one CTA pass (long rows)
constexpr int kChunkRows = 32;     // rows of one CTA tile (short rows)
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
__device__ __forceinline__ Element quantDequant(float x, float s, float inv, float o, int zp, const Grid &g) {
    Element e;
    if constexpr (kReciprocal) {
        const float r = __fadd_rn(nearbyintf(__fmul_rn(x, inv)), static_cast<float>(zp));
        const long long q = static_cast<long long>(r);   // saturates; NaN gives 0
        const bool nan = x != x;
        const bool keep = !nan && q >= g.qmin && q <= g.qmax;
        const long long c = q < g.qmin ? g.qmin : (q > g.qmax ? g.qmax : q);
        e.y = nan ? x : __fmul_rn(static_cast<float>(c - zp), s);
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
    const float qc = q != q ? q : fminf(fmaxf(q, lo), hi);
    acc.scale = __fadd_rn(acc.scale, __fmul_rn(gr, __fsub_rn(qc, __fmul_rn(xs, m))));
    acc.offset = __fadd_rn(acc.offset, __fmul_rn(gr, keep ? 0.0f : s));
    return __fmul_rn(gr, m);
}

__device__ __forceinline__ Sums blockSum(Sums v) {
    __shared__ float part[2][kThreads / 32];
    for (int d = 16; d > 0; d >>= 1) {
        v.scale += __shfl_down_sync(0xffffffffu, v.scale, d);
        v.offset += __shfl_down_sync(0xffffffffu, v.offset, d);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();   // the buffer may still be read from the previous call
    if (lane == 0) { part[0][warp] = v.scale; part[1][warp] = v.offset; }
    __syncthreads();
    Sums out;
    if (threadIdx.x == 0) {
        for (int w = 0; w < kThreads / 32; ++w) { out.scale += part[0][w]; out.offset += part[1][w]; }
    }
    return out;
}

struct Pass {
    const float *x;
    const float *grad;      // backward only
    float *out;             // y (forward) or dx (backward); may be null in a backward that only wants sums
    uint8_t *keep;          // forward, optional: 1 where the value was inside the grid
    float *partial;         // backward, optional: [items][2]
    uint64_t outer, channels, inner;
    int wantSums;
};

// Long rows: one work item = one segment of one row (a row is `inner` contiguous elements of one channel).
template <bool kBackward, bool kReciprocal>
__global__ void __launch_bounds__(kThreads) rowPass(Pass p, Grid g, uint64_t segments, int vector) {
    const uint64_t rows = p.outer * p.channels;
    for (uint64_t item = blockIdx.x; item < rows * segments; item += gridDim.x) {
        const uint64_t row = item / segments, seg = item - row * segments;
        const uint64_t c = row % p.channels;
        const float s = __ldg(g.scale + c), o = __ldg(g.offset + c);
        const float inv = __fdiv_rn(1.0f, s);
        const int zp = -static_cast<int>(o);
        const uint64_t begin = row * p.inner + seg * kSegment;
        const int count = static_cast<int>(min(static_cast<uint64_t>(kSegment), p.inner - seg * kSegment));
        Sums acc;
        if (vector) {
            const float4 *x4 = reinterpret_cast<const float4 *>(p.x + begin);
            const float4 *g4 = kBackward ? reinterpret_cast<const float4 *>(p.grad + begin) : nullptr;
            float4 *o4 = p.out ? reinterpret_cast<float4 *>(p.out + begin) : nullptr;
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
                    if (p.keep) reinterpret_cast<uint32_t *>(p.keep + begin)[v] = bits;
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
            if (p.wantSums) {
                const Sums total = blockSum(acc);
                if (threadIdx.x == 0) { p.partial[2 * item] = total.scale; p.partial[2 * item + 1] = total.offset; }
            }
        }
    }
}

// Short rows: the tensor is a matrix [outer][channels * inner]; a thread owns one column (one channel) and
// walks down kChunkRows rows, so a warp reads 128 contiguous bytes per row and nothing is reduced across threads.
template <bool kBackward, bool kReciprocal>
__global__ void __launch_bounds__(kThreads) columnPass(Pass p, Grid g) {
    const uint64_t period = p.channels * p.inner;
    const uint64_t col = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x;
    if (col >= period) return;
    const uint64_t c = col / p.inner;
    const float s = __ldg(g.scale + c), o = __ldg(g.offset + c);
    const float inv = __fdiv_rn(1.0f, s);
    const int zp = -static_cast<int>(o);
    for (uint64_t chunk = blockIdx.y; chunk * kChunkRows < p.outer; chunk += gridDim.y) {
        const uint64_t first = chunk * kChunkRows, last = min(first + kChunkRows, p.outer);
        Sums acc;
#pragma unroll 4
        for (uint64_t r = first; r < last; ++r) {
            const uint64_t at = r * period + col;
            const float xv = __ldcs(p.x + at);
            float res;
            if constexpr (kBackward) {
                const float gr = __ldcs(p.grad + at);
                if (kReciprocal) res = __fmul_rn(gr, quantDequant<true>(xv, s, inv, o, zp, g).keep);
                else res = backwardOne(xv, gr, s, o, g, acc);
            } else {
                const Element e = quantDequant<kReciprocal>(xv, s, inv, o, zp, g);
                res = e.y;
                if (p.keep) p.keep[at] = e.keep != 0.0f;
            }
            if (p.out) __stcs(p.out + at, res);
        }
        if constexpr (kBackward) {
            if (p.wantSums) {
                p.partial[2 * (chunk * period + col)] = acc.scale;
                p.partial[2 * (chunk * period + col) + 1] = acc.offset;
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
    uint64_t segments;      // row kernel: segments per row
    uint64_t chunks;        // column kernel: row chunks
    uint64_t items;         // partial entries
};

Plan planFor(uint64_t outer, uint64_t channels, uint64_t inner) {
    Plan plan{};
    plan.rows = channels == 1 || inner >= kLongRow;
    if (plan.rows) {
        plan.segments = (inner + kSegment - 1) / kSegment;
        plan.items = outer * channels * plan.segments;
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

template <bool kBackward>
void run(Pass p, Grid g, int reciprocal, const Plan &plan, cudaStream_t st) {
    const DeviceInfo dev = currentDevice();
    if (plan.rows) {
        // per tensor the whole tensor is one row: `outer` and `channels` fold into it on the host
        const bool aligned = p.inner % 4 == 0 && (reinterpret_cast<uintptr_t>(p.x) & 15) == 0 &&
                             (!p.grad || (reinterpret_cast<uintptr_t>(p.grad) & 15) == 0) &&
                             (!p.out || (reinterpret_cast<uintptr_t>(p.out) & 15) == 0) &&
                             (!p.keep || (reinterpret_cast<uintptr_t>(p.keep) & 3) == 0);
        const uint64_t items = p.outer * p.channels * plan.segments;
        const int grid = static_cast<int>(std::min<uint64_t>(items, static_cast<uint64_t>(dev.sms) * 8));
        if (reciprocal) rowPass<kBackward, true><<<grid, kThreads, 0, st>>>(p, g, plan.segments, aligned ? 1 : 0);
        else rowPass<kBackward, false><<<grid, kThreads, 0, st>>>(p, g, plan.segments, aligned ? 1 : 0);
        afterLaunch("affineRowPass");
    } else {
        const uint64_t period = p.channels * p.inner;
        const unsigned gx = static_cast<unsigned>((period + kThreads - 1) / kThreads);
        const uint64_t want = std::max<uint64_t>(1, static_cast<uint64_t>(dev.sms) * 8 / gx);
        const unsigned gy = static_cast<unsigned>(std::min<uint64_t>(std::min<uint64_t>(plan.chunks, want), 65535));
        if (reciprocal) columnPass<kBackward, true><<<dim3(gx, gy), kThreads, 0, st>>>(p, g);
        else columnPass<kBackward, false><<<dim3(gx, gy), kThreads, 0, st>>>(p, g);
        afterLaunch("affineColumnPass");
    }
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
        if (sums) {
            RXMET_REQUIRE(workspace_dev && workspace_bytes >= plan.items * 2 * sizeof(float),
                          "affine qdq backward: workspace of %zu bytes needed", static_cast<size_t>(plan.items * 2 * sizeof(float)));
            p.partial = static_cast<float *>(workspace_dev);
            p.wantSums = 1;
        }
        const Grid g{scale_dev, offset_dev, static_cast<float>(qmin), static_cast<float>(qmax), qmin, qmax};
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        run<true>(p, g, reciprocal, plan, st);
        if (sums) {
            if (plan.rows)
                finishSums<<<static_cast<unsigned>(p.channels), 128, 0, st>>>(p.partial, p.outer, p.channels * plan.segments,
                                                                              plan.segments, dscale_dev, doffset_dev);
            else
                finishSums<<<static_cast<unsigned>(p.channels), 128, 0, st>>>(p.partial, plan.chunks, p.channels * p.inner,
                                                                              p.inner, dscale_dev, doffset_dev);
            afterLaunch("affineFinishSums");
        }
    });
}

}  // extern "C"
