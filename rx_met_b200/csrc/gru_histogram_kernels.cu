// Device side of the histogram calibration and its C entry points.
//
// A collector update is split as plan (host, from the batch extremes) -> bin (device) -> commit
// (host): the device only counts elements into a fixed range with the collector's exact float
// expression  bin = int((v - lo) * inv_width), v < lo -> first bin, v > hi -> last bin, non-finite
// skipped (operators/quant-gru/include/histogram_collector.h:289-311).  For the GRU calibration
// forward the extremes of all 13 activation points come out of the recurrent kernel itself, so a
// batch costs one pass that writes the traces and one bandwidth-bound pass that bins them (the
// reference makes a min/max pass, a histogram pass and a device-to-host round trip per tensor,
// operators/quant-gru/src/calibration_gpu.cu).
#include <cuda_runtime.h>

#include <algorithm>
#include <cfloat>
#include <cstring>
#include <vector>

#include "common.h"
#include "gru_forward_float.h"
#include "gru_histogram.h"
#include "gru_params.h"
#include "minmax_device.cuh"

namespace rxmet {
namespace hist {
namespace {

constexpr int kMaxSharedBins = 8192;

struct BinJob {
    const float *data;
    unsigned long long rows, cols, rowStride;
    float lo, hi, inv;
    uint32_t *counts;
};

// blockIdx.y selects the job; a CTA keeps a private histogram in shared memory and flushes the
// non-empty bins with one global atomic each.
__global__ void rangeHistogram(const BinJob *__restrict__ jobs, int bins) {
    extern __shared__ uint32_t local[];
    const BinJob job = jobs[blockIdx.y];
    for (int i = threadIdx.x; i < bins; i += blockDim.x) local[i] = 0u;
    __syncthreads();
    const unsigned long long n = job.rows * job.cols;
    for (unsigned long long i = blockIdx.x * static_cast<unsigned long long>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<unsigned long long>(gridDim.x) * blockDim.x) {
        const float v = job.data[(i / job.cols) * job.rowStride + (i % job.cols)];
        if (!isfinite(v)) continue;
        int idx;
        if (v < job.lo) idx = 0;
        else if (v > job.hi) idx = bins - 1;
        else idx = min(static_cast<int>(__fmul_rn(__fsub_rn(v, job.lo), job.inv)), bins - 1);
        atomicAdd(&local[idx], 1u);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < bins; i += blockDim.x)
        if (local[i]) atomicAdd(&job.counts[i], local[i]);
}

__global__ void stridedMinMax(const float *__restrict__ x, unsigned long long rows, unsigned long long cols,
                              unsigned long long rowStride, float *minSlot, float *maxSlot) {
    __shared__ float scratch[2 * 32];
    stats::MinMax m[1];
    const unsigned long long n = rows * cols;
    for (unsigned long long i = blockIdx.x * static_cast<unsigned long long>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<unsigned long long>(gridDim.x) * blockDim.x)
        m[0].see(x[(i / cols) * rowStride + (i % cols)]);
    const int slot[1] = {0};
    stats::commit<1>(m, slot, minSlot, maxSlot, scratch);
}

__global__ void initMinMax(float *mm) {
    mm[0] = FLT_MAX;
    mm[1] = -FLT_MAX;
}

int gridFor(unsigned long long n, int block) {
    return static_cast<int>(std::min<unsigned long long>((n + block - 1) / block, 148 * 4));
}

struct Pending {
    rxmet_histogram *h;
    Plan plan;
    unsigned long long elements;
};

// Bins every job on the device and commits the counts on the host.  jobsDev / countsDev are
// workspace regions for jobs.size() entries; synchronises the stream.
void runJobs(std::vector<BinJob> &jobs, std::vector<Pending> &pending, int bins, BinJob *jobsDev, uint32_t *countsDev,
             cudaStream_t st, const rxmet_exchange *exchange = nullptr) {
    if (jobs.empty()) return;
    RXMET_REQUIRE(bins <= kMaxSharedBins, "histograms of up to %d bins are built (got %d)", kMaxSharedBins, bins);
    const size_t n = jobs.size();
    for (size_t j = 0; j < n; ++j) jobs[j].counts = countsDev + j * bins;
    RXMET_CUDA(cudaMemsetAsync(countsDev, 0, n * bins * sizeof(uint32_t), st));
    RXMET_CUDA(cudaMemcpyAsync(jobsDev, jobs.data(), n * sizeof(BinJob), cudaMemcpyHostToDevice, st));
    unsigned long long largest = 0;
    for (const BinJob &j : jobs) largest = std::max(largest, j.rows * j.cols);
    {
        KernelTimer timer__("rangeHistogram", st);
        rangeHistogram<<<dim3(gridFor(largest, 256 * 8), static_cast<unsigned>(n)), 256, bins * sizeof(uint32_t), st>>>(jobsDev, bins);
    }
    afterLaunch("rangeHistogram");
    if (exchange && exchange->reduce(RXMET_REDUCE_SUM_U32, countsDev, n * bins, st, exchange->user) != 0)
        fail(RXMET_ERR_INVALID_ARGUMENT, "the exchange hook reported a failure (bin counts)");
    std::vector<uint32_t> host(n * bins);
    RXMET_CUDA(cudaMemcpyAsync(host.data(), countsDev, host.size() * sizeof(uint32_t), cudaMemcpyDeviceToHost, st));
    RXMET_CUDA(cudaStreamSynchronize(st));
    for (size_t j = 0; j < n; ++j) commit(pending[j].h, pending[j].plan, host.data() + j * bins, pending[j].elements);
}

void checkCollector(const rxmet_histogram *h) {
    RXMET_REQUIRE(h != nullptr && h->counts != nullptr && h->num_bins > 0, "histogram needs a counts array and a bin count");
}

}  // namespace
}  // namespace hist

namespace gru {

size_t histCalibrationWorkspaceBytes(int T, int B, int I, int H, int bins) {
    const size_t rows = static_cast<size_t>(T) * B, C = 3 * static_cast<size_t>(H);
    WorkspaceSizer ws;
    ws.take<char>(forwardFloatWorkspaceBytes(T, B, I, H));
    ws.take<float>(statsFloats(H));
    for (int k = 0; k < 4; ++k) ws.take<float>(rows * C);
    ws.take<hist::BinJob>(16);
    ws.take<uint32_t>(16 * static_cast<size_t>(bins));
    return ws.used() + 1024;
}

// src/gru_forward_cpu.cc:27-56 : which collectors a weight or bias tensor feeds.
void observeParameter(const std::vector<float> &values, int rows, int hidden, rxmet_histogram *channels,
                      rxmet_histogram *tensor, rxmet_histogram *gates, int granularity, bool bias) {
    const int columns = 3 * hidden;
    if (granularity == RXMET_PER_TENSOR) hist::collectHost(tensor, values.data(), rows, columns, columns);
    if (bias || granularity == RXMET_PER_CHANNEL) {
        RXMET_REQUIRE(channels != nullptr, "per-channel collectors are not set");
        for (int c = 0; c < columns; ++c) {
            rxmet_histogram *h = &channels[c];
            if (h->num_bins > 0 && h->total_count > 0) continue;  // static values are observed once
            hist::collectHost(h, values.data() + c, rows, 1, columns);
        }
    }
    if (granularity == RXMET_PER_GATE)
        for (int g = 0; g < 3; ++g) hist::collectHost(&gates[g], values.data() + g * hidden, rows, hidden, columns);
}

void forwardCalibrateHist(int T, int B, int I, int H, const float *W, const float *R, const float *bw, const float *br,
                          const float *x, const float *h0, float *h, float *v, const rxmet_gru_quant_config &cfg,
                          rxmet_gru_histograms *hs, void *workspace, size_t workspaceBytes, cudaStream_t st,
                          const rxmet_exchange *exchange) {
    const unsigned long long world = exchange ? static_cast<unsigned long long>(std::max(exchange->world_size, 1)) : 1ull;
    if (exchange) RXMET_REQUIRE(exchange->reduce != nullptr, "exchange without a reduce function");
    RXMET_REQUIRE(hs->hidden == H, "histogram collectors were made for hidden=%d, call has H=%d", hs->hidden, H);
    const int bins = hs->num_bins;
    for (int op = 0; op < kOps; ++op) {
        hist::checkCollector(&hs->point[op]);
        RXMET_REQUIRE(hs->point[op].num_bins == bins, "all collectors of a set share one bin count");
    }
    const size_t rows = static_cast<size_t>(T) * B, C = 3 * static_cast<size_t>(H);
    Workspace ws(workspace, workspaceBytes);
    const size_t fwdBytes = forwardFloatWorkspaceBytes(T, B, I, H);
    char *fwdWs = ws.take<char>(fwdBytes);
    float *stats = ws.take<float>(statsFloats(H));
    float *wx = ws.take<float>(rows * C), *rh = ws.take<float>(rows * C);
    float *pre = ws.take<float>(rows * C), *mul = ws.take<float>(rows * C);
    hist::BinJob *jobsDev = ws.take<hist::BinJob>(16);
    uint32_t *countsDev = ws.take<uint32_t>(16 * static_cast<size_t>(bins));

    ForwardFloatCall call;
    call.T = T; call.B = B; call.I = I; call.H = H;
    call.W = W; call.R = R; call.bw = bw; call.br = br; call.x = x; call.h0 = h0; call.h = h; call.v = v;
    call.stats = stats;
    call.traceWx = wx; call.traceRh = rh; call.tracePre = pre; call.traceMul = mul;
    forwardFloat(call, fwdWs, fwdBytes, st);
    if (exchange) {  // every rank bins on the extremes of the whole batch
        const size_t halfDev = statsFloats(H) / 2;
        if (exchange->reduce(RXMET_REDUCE_MIN_F32, stats, halfDev, st, exchange->user) != 0 ||
            exchange->reduce(RXMET_REDUCE_MAX_F32, stats + halfDev, halfDev, st, exchange->user) != 0)
            fail(RXMET_ERR_INVALID_ARGUMENT, "the exchange hook reported a failure (extremes)");
    }
    std::vector<float> host(statsFloats(H));
    RXMET_CUDA(cudaMemcpyAsync(host.data(), stats, host.size() * sizeof(float), cudaMemcpyDeviceToHost, st));
    const size_t wCount = static_cast<size_t>(I) * C, rCount = static_cast<size_t>(H) * C;
    std::vector<float> hW(wCount), hR(rCount), hbw(C), hbr(C);
    RXMET_CUDA(cudaMemcpyAsync(hW.data(), W, wCount * sizeof(float), cudaMemcpyDeviceToHost, st));
    RXMET_CUDA(cudaMemcpyAsync(hR.data(), R, rCount * sizeof(float), cudaMemcpyDeviceToHost, st));
    RXMET_CUDA(cudaMemcpyAsync(hbw.data(), bw, C * sizeof(float), cudaMemcpyDeviceToHost, st));
    RXMET_CUDA(cudaMemcpyAsync(hbr.data(), br, C * sizeof(float), cudaMemcpyDeviceToHost, st));
    RXMET_CUDA(cudaStreamSynchronize(st));
    const size_t half = host.size() / 2;

    // the 13 activation points: (point, data, cols, row stride)
    struct Source { int op; const float *data; unsigned long long cols, stride; };
    const unsigned long long uH = H, uC = C;
    const Source sources[13] = {
        {RXMET_GRU_X, x, static_cast<unsigned long long>(I), static_cast<unsigned long long>(I)},
        {RXMET_GRU_H, h + static_cast<size_t>(B) * H, uH, uH},  // h0 is not sampled
        {RXMET_GRU_WEIGHT_IH_LINEAR, wx, uC, uC},
        {RXMET_GRU_WEIGHT_HH_LINEAR, rh, uC, uC},
        {RXMET_GRU_UPDATE_GATE_INPUT, pre, uH, uC},
        {RXMET_GRU_RESET_GATE_INPUT, pre + H, uH, uC},
        {RXMET_GRU_NEW_GATE_INPUT, pre + 2 * H, uH, uC},
        {RXMET_GRU_UPDATE_GATE_OUTPUT, v, uH, 4 * uH},
        {RXMET_GRU_RESET_GATE_OUTPUT, v + H, uH, 4 * uH},
        {RXMET_GRU_NEW_GATE_OUTPUT, v + 2 * H, uH, 4 * uH},
        {RXMET_GRU_MUL_RESET_HIDDEN, mul, uH, uC},
        {RXMET_GRU_MUL_NEW_CONTRIBUTION, mul + H, uH, uC},
        {RXMET_GRU_MUL_OLD_CONTRIBUTION, mul + 2 * H, uH, uC},
    };
    std::vector<hist::BinJob> jobs;
    std::vector<hist::Pending> pending;
    for (const Source &s : sources) {
        float lo = host[s.op], hi = host[half + s.op];
        if (!(lo <= hi)) lo = hi = 0.0f;  // nothing finite observed
        rxmet_histogram *target = &hs->point[s.op];
        const hist::Plan p = hist::plan(*target, lo, hi);
        jobs.push_back({s.data, static_cast<unsigned long long>(rows), s.cols, s.stride, p.lo, p.hi, p.invBinWidth, nullptr});
        pending.push_back({target, p, world * static_cast<unsigned long long>(rows) * s.cols});
    }
    hist::runJobs(jobs, pending, bins, jobsDev, countsDev, st, exchange);

    observeParameter(hW, I, H, hs->channel[0], &hs->point[RXMET_GRU_W], hs->gate[0], cfg.W_granularity, false);
    observeParameter(hR, H, H, hs->channel[1], &hs->point[RXMET_GRU_R], hs->gate[1], cfg.R_granularity, false);
    observeParameter(hbw, 1, H, hs->channel[2], &hs->point[RXMET_GRU_BW], hs->gate[2], cfg.bw_granularity, true);
    observeParameter(hbr, 1, H, hs->channel[3], &hs->point[RXMET_GRU_BR], hs->gate[3], cfg.br_granularity, true);
}

}  // namespace gru
}  // namespace rxmet

using namespace rxmet;

extern "C" {

int rxmet_histogram_reset(rxmet_histogram *h) {
    return guarded([&] {
        RXMET_REQUIRE(h != nullptr, "hist must not be null");
        hist::reset(h);
    });
}

int rxmet_histogram_collect_host(rxmet_histogram *h, const float *data, uint64_t count) {
    return guarded([&] {
        hist::checkCollector(h);
        RXMET_REQUIRE(data != nullptr || count == 0, "data must not be null");
        hist::collectHost(h, data, 1, count, count);
    });
}

size_t rxmet_histogram_workspace_bytes(int num_bins) {
    if (num_bins <= 0) return 0;
    return 1024 + sizeof(hist::BinJob) + static_cast<size_t>(num_bins) * sizeof(uint32_t) + 256 * 3;
}

int rxmet_histogram_collect_dev(rxmet_histogram *h, const float *data, uint64_t rows, uint64_t cols, uint64_t rowStride,
                                void *workspace, size_t workspaceBytes, void *stream) {
    return guarded([&] {
        hist::checkCollector(h);
        if (rows * cols == 0) return;
        RXMET_REQUIRE(data != nullptr, "data must not be null");
        RXMET_REQUIRE(rowStride >= cols, "row stride is smaller than the row");
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        Workspace ws(workspace, workspaceBytes);
        float *mm = ws.take<float>(2);
        hist::BinJob *jobsDev = ws.take<hist::BinJob>(1);
        uint32_t *countsDev = ws.take<uint32_t>(h->num_bins);
        hist::initMinMax<<<1, 1, 0, st>>>(mm);
        afterLaunch("initMinMax");
        {
            KernelTimer timer__("stridedMinMax", st);
            hist::stridedMinMax<<<hist::gridFor(rows * cols, 256 * 8), 256, 0, st>>>(data, rows, cols, rowStride, mm, mm + 1);
        }
        afterLaunch("stridedMinMax");
        float host[2];
        RXMET_CUDA(cudaMemcpyAsync(host, mm, sizeof(host), cudaMemcpyDeviceToHost, st));
        RXMET_CUDA(cudaStreamSynchronize(st));
        if (!(host[0] <= host[1])) host[0] = host[1] = 0.0f;
        const hist::Plan p = hist::plan(*h, host[0], host[1]);
        std::vector<hist::BinJob> jobs{{data, rows, cols, rowStride, p.lo, p.hi, p.invBinWidth, nullptr}};
        std::vector<hist::Pending> pending{{h, p, rows * cols}};
        hist::runJobs(jobs, pending, h->num_bins, jobsDev, countsDev, st);
    });
}

int rxmet_histogram_merge(rxmet_histogram *h, const rxmet_histogram *other) {
    return guarded([&] {
        hist::checkCollector(h);
        RXMET_REQUIRE(other != nullptr, "other must not be null");
        hist::merge(h, *other);
    });
}

int rxmet_histogram_calibrate(const rxmet_histogram *h, int bits, int is_unsigned, int symmetric, int use_percentile,
                              float percentile, float *scale, float *range_min, float *range_max) {
    return guarded([&] {
        hist::checkCollector(h);
        RXMET_REQUIRE(bits >= 1 && bits <= 31, "bit width must be in [1, 31]");
        RXMET_REQUIRE(scale && range_min && range_max, "output pointers must not be null");
        const int32_t qlo = is_unsigned ? 0 : -(1 << (bits - 1));
        const int32_t qhi = is_unsigned ? static_cast<int32_t>((1u << bits) - 1u) : (1 << (bits - 1)) - 1;
        const hist::Continuous c = hist::calibrate(*h, qlo, qhi, is_unsigned != 0, symmetric != 0, use_percentile != 0, percentile);
        *scale = c.scale;
        *range_min = c.lo;
        *range_max = c.hi;
    });
}

int rxmet_gru_forward_calibrate_hist(int T, int B, int I, int H, const float *W, const float *R, const float *bw,
                                     const float *br, const float *x, const float *h0, float *h, float *v,
                                     const rxmet_gru_quant_config *config, rxmet_gru_histograms *hists, void *workspace,
                                     size_t workspace_bytes, void *stream) {
    return guarded([&] {
        RXMET_REQUIRE(T > 0 && B > 0 && I > 0 && H > 0, "GRU dimensions must be positive");
        RXMET_REQUIRE(W && R && bw && br && x && h && v && config && hists, "null argument");
        gru::forwardCalibrateHist(T, B, I, H, W, R, bw, br, x, h0, h, v, *config, hists, workspace, workspace_bytes,
                                  static_cast<cudaStream_t>(stream), nullptr);
    });
}

int rxmet_gru_forward_calibrate_hist_dp(int T, int B, int I, int H, const float *W, const float *R, const float *bw,
                                        const float *br, const float *x, const float *h0, float *h, float *v,
                                        const rxmet_gru_quant_config *config, rxmet_gru_histograms *hists, void *workspace,
                                        size_t workspace_bytes, void *stream, const rxmet_exchange *exchange) {
    return guarded([&] {
        RXMET_REQUIRE(T > 0 && B > 0 && I > 0 && H > 0, "GRU dimensions must be positive");
        RXMET_REQUIRE(W && R && bw && br && x && h && v && config && hists, "null argument");
        gru::forwardCalibrateHist(T, B, I, H, W, R, bw, br, x, h0, h, v, *config, hists, workspace, workspace_bytes,
                                  static_cast<cudaStream_t>(stream), exchange);
    });
}

int rxmet_histogram_plan_batch(const rxmet_histogram *h, float batch_min, float batch_max, rxmet_histogram_plan *out) {
    return guarded([&] {
        hist::checkCollector(h);
        RXMET_REQUIRE(out != nullptr, "plan must not be null");
        const hist::Plan p = hist::plan(*h, batch_min, batch_max);
        *out = rxmet_histogram_plan{static_cast<int32_t>(p.mode), p.lo, p.hi, p.invBinWidth, p.newMin, p.newMax,
                                    p.dataMin, p.dataMax, p.limitMin, p.limitMax};
    });
}

namespace {
hist::Plan fromC(const rxmet_histogram_plan &c) {
    hist::Plan p;
    p.mode = static_cast<hist::Plan::Mode>(c.mode);
    p.lo = c.lo; p.hi = c.hi; p.invBinWidth = c.inv_bin_width;
    p.newMin = c.new_min; p.newMax = c.new_max;
    p.dataMin = c.data_min; p.dataMax = c.data_max;
    p.limitMin = c.limit_min; p.limitMax = c.limit_max;
    return p;
}
}  // namespace

int rxmet_histogram_count_host(const rxmet_histogram_plan *plan, int num_bins, const float *data, uint64_t count,
                               uint32_t *counts) {
    return guarded([&] {
        RXMET_REQUIRE(plan && counts && num_bins > 0 && (data || count == 0), "bad arguments");
        hist::binHost(data, 1, count, count, fromC(*plan), num_bins, counts);
    });
}

int rxmet_histogram_commit_counts(rxmet_histogram *h, const rxmet_histogram_plan *plan, const uint32_t *counts,
                                  uint64_t total_elements) {
    return guarded([&] {
        hist::checkCollector(h);
        RXMET_REQUIRE(plan && counts, "bad arguments");
        if (total_elements == 0) return;
        hist::commit(h, fromC(*plan), counts, total_elements);
    });
}

int rxmet_gru_params_from_histograms(const rxmet_gru_histograms *hists, const rxmet_gru_quant_config *config,
                                     int use_percentile, float percentile, rxmet_gru_quant_params *params) {
    return guarded([&] {
        RXMET_REQUIRE(hists && config && params, "null argument");
        gru::paramsFromHistograms(*hists, *config, use_percentile != 0, percentile, params);
    });
}

}  // extern "C"
