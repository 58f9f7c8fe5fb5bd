// Device side of the QuantLSTM histogram calibration and its C entry points.
//
// One calibration batch = float forward with all seven per-step tensors kept in the workspace, then
// two batched launches over up to 16 tensors (blockIdx.y = tensor): finite min/max + finite count,
// and the binning of every tensor over its own range with the collector's double-precision index
// expression (operators/quant-lstm/src/quantization/histogram.cc:23-34).  The merges (re-binning of
// bin centres) run on the host in the order the reference's collector observes the tensors
// (operators/quant-lstm/src/lstm/calibration.cc:128-232), so that the result is the reference's.
// The reference makes one reduction and one device-to-host copy per operator group
// (operators/quant-lstm/src/lstm/calibration_cuda.cu:371-491).
#include <cuda_runtime.h>

#include <algorithm>
#include <cfloat>
#include <cmath>
#include <cstring>
#include <limits>
#include <memory>
#include <vector>

#include "common.h"
#include "lstm_histogram.h"
#include "lstm_kernels.h"
#include "lstm_params.h"

namespace rxmet {
namespace lstm {
namespace {

constexpr int kMaxJobs = 16;
constexpr int kMaxSharedBins = 8192;

struct Job {
    const float *data;
    unsigned long long rows, cols, rowStride;
    float lo, hi;  // filled in before the binning launch
};

// Finite extremes and finite count of every job; three separate arrays on the device, so that a
// data-parallel run can reduce each of them across ranks in place (MIN, MAX, SUM).
struct JobStats {
    float lo, hi;
    unsigned long long finite;
};
struct JobStatsDev {
    float *lo, *hi;
    unsigned long long *finite;
};

__device__ __forceinline__ void atomicMinFloat(float *addr, float v) {
    if (v >= 0.0f) atomicMin(reinterpret_cast<int *>(addr), __float_as_int(v));
    else atomicMax(reinterpret_cast<unsigned int *>(addr), __float_as_uint(v));
}
__device__ __forceinline__ void atomicMaxFloat(float *addr, float v) {
    if (v >= 0.0f) atomicMax(reinterpret_cast<int *>(addr), __float_as_int(v));
    else atomicMin(reinterpret_cast<unsigned int *>(addr), __float_as_uint(v));
}

__global__ void initJobStats(JobStatsDev stats, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        stats.lo[i] = FLT_MAX;
        stats.hi[i] = -FLT_MAX;
        stats.finite[i] = 0ull;
    }
}

__global__ void jobMinMax(const Job *__restrict__ jobs, JobStatsDev stats) {
    __shared__ float sLo[8], sHi[8];
    __shared__ unsigned long long sN[8];
    const Job job = jobs[blockIdx.y];
    const unsigned long long n = job.rows * job.cols;
    float lo = FLT_MAX, hi = -FLT_MAX;
    unsigned long long finite = 0;
    for (unsigned long long i = blockIdx.x * static_cast<unsigned long long>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<unsigned long long>(gridDim.x) * blockDim.x) {
        const float v = job.data[(i / job.cols) * job.rowStride + (i % job.cols)];
        if (isfinite(v)) {
            lo = fminf(lo, v);
            hi = fmaxf(hi, v);
            ++finite;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
        hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
        finite += __shfl_xor_sync(0xffffffffu, finite, o);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { sLo[warp] = lo; sHi[warp] = hi; sN[warp] = finite; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (blockDim.x >> 5); ++w) { lo = fminf(lo, sLo[w]); hi = fmaxf(hi, sHi[w]); finite += sN[w]; }
        if (finite) {
            atomicMinFloat(&stats.lo[blockIdx.y], lo);
            atomicMaxFloat(&stats.hi[blockIdx.y], hi);
            atomicAdd(&stats.finite[blockIdx.y], finite);
        }
    }
}

__global__ void jobHistogram(const Job *__restrict__ jobs, int bins, uint32_t *__restrict__ counts) {
    extern __shared__ uint32_t local[];
    const Job job = jobs[blockIdx.y];
    for (int i = threadIdx.x; i < bins; i += blockDim.x) local[i] = 0u;
    __syncthreads();
    const unsigned long long n = job.rows * job.cols;
    const double lo = static_cast<double>(job.lo), span = static_cast<double>(job.hi) - static_cast<double>(job.lo);
    for (unsigned long long i = blockIdx.x * static_cast<unsigned long long>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<unsigned long long>(gridDim.x) * blockDim.x) {
        const float v = job.data[(i / job.cols) * job.rowStride + (i % job.cols)];
        if (!isfinite(v)) continue;
        int idx;
        if (v <= job.lo) idx = 0;
        else if (v >= job.hi) idx = bins - 1;
        else {
            const double normalized = __ddiv_rn(__dsub_rn(static_cast<double>(v), lo), span);
            idx = min(static_cast<int>(__dmul_rn(normalized, static_cast<double>(bins))), bins - 1);
        }
        atomicAdd(&local[idx], 1u);
    }
    __syncthreads();
    uint32_t *out = counts + static_cast<size_t>(blockIdx.y) * bins;
    for (int i = threadIdx.x; i < bins; i += blockDim.x)
        if (local[i]) atomicAdd(&out[i], local[i]);
}

int gridFor(unsigned long long n, int block) {
    return static_cast<int>(std::max<unsigned long long>(1, std::min<unsigned long long>((n + block - 1) / block, 148 * 4)));
}

bool isBias(int op) { return op == RXMET_LSTM_BIAS_IH || op == RXMET_LSTM_BIAS_HH; }
bool isParameter(int op) { return op >= RXMET_LSTM_WEIGHT_IH && op <= RXMET_LSTM_BIAS_HH; }

// A collector with its own storage, for the per-batch collectors the reference builds before it
// merges them into the session's.
struct Scratch {
    std::vector<double> counts;
    rxmet_lstm_histogram h{};
    explicit Scratch(int bins) : counts(bins, 0.0) {
        h.counts = counts.data();
        h.num_bins = bins;
    }
    Scratch(const Scratch &) = delete;
};

void checkCollector(const rxmet_lstm_histogram *h) {
    RXMET_REQUIRE(h != nullptr && h->counts != nullptr && h->num_bins >= 2, "histogram needs a counts array and at least 2 bins");
}

// Host collection of a weight or bias tensor into the collectors of its granularity
// (LstmCalibrationCollector::observeParameter, calibration.cc:94-127).
void observeParameter(const std::vector<float> &values, int rowWidth, int H, int granularity, rxmet_lstm_histogram *tensor,
                      rxmet_lstm_histogram *gates, rxmet_lstm_histogram *channels, int bins) {
    const int C = 4 * H;
    auto collectInto = [&](rxmet_lstm_histogram *dst, const float *data, uint64_t count) {
        checkCollector(dst);
        Scratch batch(bins);
        hist::collectHost(&batch.h, data, 1, count, count);
        hist::merge(dst, batch.h);
    };
    if (granularity == RXMET_LSTM_PER_TENSOR) {
        collectInto(tensor, values.data(), static_cast<uint64_t>(C) * rowWidth);
    } else if (granularity == RXMET_LSTM_PER_GATE) {
        for (int g = 0; g < 4; ++g)
            collectInto(&gates[g], values.data() + static_cast<size_t>(g) * H * rowWidth, static_cast<uint64_t>(H) * rowWidth);
    } else {
        RXMET_REQUIRE(channels != nullptr, "per-channel collectors are not set");
        for (int ch = 0; ch < C; ++ch) collectInto(&channels[ch], values.data() + static_cast<size_t>(ch) * rowWidth, rowWidth);
    }
}

}  // namespace

size_t histCalibrationWorkspaceBytes(int T, int B, int I, int H) {
    const size_t rows = static_cast<size_t>(T) * B, C = 4 * static_cast<size_t>(H);
    WorkspaceSizer ws;
    ws.take<char>(forwardFloatWorkspaceBytes(T, B, I, H));
    ws.take<float>(statsFloats(H));
    for (int k = 0; k < 4; ++k) ws.take<float>(rows * C);
    for (int k = 0; k < 3; ++k) ws.take<float>(rows * H);
    ws.take<Job>(kMaxJobs);
    ws.take<float>(kMaxJobs);
    ws.take<float>(kMaxJobs);
    ws.take<unsigned long long>(kMaxJobs);
    ws.take<uint32_t>(static_cast<size_t>(kMaxJobs) * kMaxSharedBins);
    return ws.used() + 1024;
}

void forwardCalibrateHist(const ForwardFloatCall &user, const rxmet_lstm_quant_config &cfg, rxmet_lstm_ranges *ranges,
                          rxmet_lstm_histograms *hs, void *workspace, size_t workspaceBytes, cudaStream_t st,
                          const rxmet_exchange *exchange) {
    // Data parallel (exchange set): every rank holds a shard of the batch.  The ranks reduce the range
    // statistics and the finite extremes / counts of every observed tensor, bin on the common range and
    // sum the bin counts, so that every rank merges the histogram one process would build on the
    // concatenated batch (the per-batch collection of the reference: histogram.cc:145-193).
    const unsigned long long world = exchange ? static_cast<unsigned long long>(std::max(exchange->world_size, 1)) : 1ull;
    auto reduce = [&](int kind, void *data, uint64_t count) {
        if (!exchange) return;
        RXMET_REQUIRE(exchange->reduce != nullptr, "exchange without a reduce function");
        if (exchange->reduce(kind, data, count, st, exchange->user) != 0)
            fail(RXMET_ERR_INVALID_ARGUMENT, "the exchange hook reported a failure (kind %d)", kind);
    };
    const int T = user.T, B = user.B, I = user.I, H = user.H, C = 4 * H;
    RXMET_REQUIRE(hs->hidden_size == H, "histogram collectors were made for hidden_size=%d, call has H=%d", hs->hidden_size, H);
    const int bins = hs->num_bins;
    RXMET_REQUIRE(bins >= 2 && bins <= kMaxSharedBins, "histograms of 2..%d bins are built (got %d)", kMaxSharedBins, bins);
    const bool bias = user.biasIh != nullptr;
    const size_t rows = static_cast<size_t>(T) * B;
    Workspace ws(workspace, workspaceBytes);
    const size_t fwdBytes = forwardFloatWorkspaceBytes(T, B, I, H);
    char *fwdWs = ws.take<char>(fwdBytes);
    float *stats = ws.take<float>(statsFloats(H));
    rxmet_lstm_trace tr{};
    tr.weight_ih_linear = ws.take<float>(rows * C);
    tr.weight_hh_linear = ws.take<float>(rows * C);
    tr.gate_inputs = ws.take<float>(rows * C);
    tr.gate_outputs = ws.take<float>(rows * C);
    tr.cell_states = ws.take<float>(rows * H);
    tr.cell_tanh_outputs = ws.take<float>(rows * H);
    tr.hidden_outputs = ws.take<float>(rows * H);
    Job *jobsDev = ws.take<Job>(kMaxJobs);
    JobStatsDev statsDev{};
    statsDev.lo = ws.take<float>(kMaxJobs);
    statsDev.hi = ws.take<float>(kMaxJobs);
    statsDev.finite = ws.take<unsigned long long>(kMaxJobs);
    uint32_t *countsDev = ws.take<uint32_t>(static_cast<size_t>(kMaxJobs) * bins);

    ForwardFloatCall call = user;
    call.trace = &tr;
    call.stats = stats;
    forwardFloat(call, fwdWs, fwdBytes, st);

    // device tensors in the order the collector observes them; `target` = point, `second` marks the
    // recorded states that follow the initial state in the same collector
    struct Source { int op; const float *data; unsigned long long r, c, stride; };
    std::vector<Source> src;
    const unsigned long long uRows = rows, uH = H, uC = C, uB = B;
    src.push_back({RXMET_LSTM_INPUT, user.x, uRows, static_cast<unsigned long long>(I), static_cast<unsigned long long>(I)});
    if (user.h0) src.push_back({RXMET_LSTM_OUTPUT, user.h0, uB, uH, uH});
    src.push_back({RXMET_LSTM_OUTPUT, tr.hidden_outputs, uRows, uH, uH});
    if (user.c0) src.push_back({RXMET_LSTM_CELL_STATE, user.c0, uB, uH, uH});
    src.push_back({RXMET_LSTM_CELL_STATE, tr.cell_states, uRows, uH, uH});
    src.push_back({RXMET_LSTM_WEIGHT_IH_LINEAR, tr.weight_ih_linear, uRows, uC, uC});
    src.push_back({RXMET_LSTM_WEIGHT_HH_LINEAR, tr.weight_hh_linear, uRows, uC, uC});
    src.push_back({RXMET_LSTM_CELL_TANH_OUTPUT, tr.cell_tanh_outputs, uRows, uH, uH});
    for (int g = 0; g < 4; ++g) {
        src.push_back({RXMET_LSTM_INPUT_GATE_INPUT + g, tr.gate_inputs + g * H, uRows, uH, uC});
        src.push_back({RXMET_LSTM_INPUT_GATE_OUTPUT + g, tr.gate_outputs + g * H, uRows, uH, uC});
    }
    const int n = static_cast<int>(src.size());
    RXMET_REQUIRE(n <= kMaxJobs, "too many calibration tensors");
    std::vector<Job> jobs(n);
    unsigned long long largest = 0;
    for (int j = 0; j < n; ++j) {
        jobs[j] = {src[j].data, src[j].r, src[j].c, src[j].stride, 0.0f, 0.0f};
        largest = std::max(largest, src[j].r * src[j].c);
    }
    RXMET_CUDA(cudaMemcpyAsync(jobsDev, jobs.data(), n * sizeof(Job), cudaMemcpyHostToDevice, st));
    initJobStats<<<1, 32, 0, st>>>(statsDev, n);
    afterLaunch("lstmInitJobStats");
    {
        KernelTimer timer__("lstmJobMinMax", st);
        jobMinMax<<<dim3(gridFor(largest, 256 * 8), n), 256, 0, st>>>(jobsDev, statsDev);
    }
    afterLaunch("lstmJobMinMax");
    {
        const size_t half = statsFloats(H) / 2;
        reduce(RXMET_REDUCE_MIN_F32, stats, half);
        reduce(RXMET_REDUCE_MAX_F32, stats + half, half);
        reduce(RXMET_REDUCE_MIN_F32, statsDev.lo, n);
        reduce(RXMET_REDUCE_MAX_F32, statsDev.hi, n);
        reduce(RXMET_REDUCE_SUM_U64, statsDev.finite, n);
    }
    std::vector<JobStats> jobStats(n);
    std::vector<float> hostStats(statsFloats(H)), hostLo(n), hostHi(n);
    std::vector<unsigned long long> hostFinite(n);
    RXMET_CUDA(cudaMemcpyAsync(hostLo.data(), statsDev.lo, n * sizeof(float), cudaMemcpyDeviceToHost, st));
    RXMET_CUDA(cudaMemcpyAsync(hostHi.data(), statsDev.hi, n * sizeof(float), cudaMemcpyDeviceToHost, st));
    RXMET_CUDA(cudaMemcpyAsync(hostFinite.data(), statsDev.finite, n * sizeof(unsigned long long), cudaMemcpyDeviceToHost, st));
    RXMET_CUDA(cudaMemcpyAsync(hostStats.data(), stats, hostStats.size() * sizeof(float), cudaMemcpyDeviceToHost, st));
    // weights for the host-side parameter collectors
    std::vector<float> wIh(static_cast<size_t>(C) * I), wHh(static_cast<size_t>(C) * H), bIh(bias ? C : 0), bHh(bias ? C : 0);
    RXMET_CUDA(cudaMemcpyAsync(wIh.data(), user.weightIh, wIh.size() * sizeof(float), cudaMemcpyDeviceToHost, st));
    RXMET_CUDA(cudaMemcpyAsync(wHh.data(), user.weightHh, wHh.size() * sizeof(float), cudaMemcpyDeviceToHost, st));
    if (bias) {
        RXMET_CUDA(cudaMemcpyAsync(bIh.data(), user.biasIh, C * sizeof(float), cudaMemcpyDeviceToHost, st));
        RXMET_CUDA(cudaMemcpyAsync(bHh.data(), user.biasHh, C * sizeof(float), cudaMemcpyDeviceToHost, st));
    }
    RXMET_CUDA(cudaStreamSynchronize(st));
    for (int j = 0; j < n; ++j) jobStats[j] = {hostLo[j], hostHi[j], hostFinite[j]};

    for (int j = 0; j < n; ++j) {
        const auto range = jobStats[j].finite ? hist::batchRange(jobStats[j].lo, jobStats[j].hi) : std::pair<float, float>{0.0f, 1.0f};
        jobs[j].lo = range.first;
        jobs[j].hi = range.second;
    }
    RXMET_CUDA(cudaMemcpyAsync(jobsDev, jobs.data(), n * sizeof(Job), cudaMemcpyHostToDevice, st));
    RXMET_CUDA(cudaMemsetAsync(countsDev, 0, static_cast<size_t>(n) * bins * sizeof(uint32_t), st));
    {
        KernelTimer timer__("lstmJobHistogram", st);
        jobHistogram<<<dim3(gridFor(largest, 256 * 8), n), 256, bins * sizeof(uint32_t), st>>>(jobsDev, bins, countsDev);
    }
    afterLaunch("lstmJobHistogram");
    reduce(RXMET_REDUCE_SUM_U32, countsDev, static_cast<uint64_t>(n) * bins);
    std::vector<uint32_t> counts(static_cast<size_t>(n) * bins);
    RXMET_CUDA(cudaMemcpyAsync(counts.data(), countsDev, counts.size() * sizeof(uint32_t), cudaMemcpyDeviceToHost, st));
    RXMET_CUDA(cudaStreamSynchronize(st));

    // ranges and contributions of this batch
    foldStats(ranges, hostStats.data(), H, bias);

    // per-batch collectors, filled in observation order, then merged into the session's
    std::vector<std::unique_ptr<Scratch>> batch(kOps);
    auto batchOf = [&](int op) -> rxmet_lstm_histogram * {
        if (!batch[op]) batch[op] = std::make_unique<Scratch>(bins);
        return &batch[op]->h;
    };
    std::vector<double> asDouble(bins);
    auto zeros = [&](int op) {  // an absent initial state is observed as B*H zeros
        const auto range = hist::batchRange(0.0f, 0.0f);
        std::fill(asDouble.begin(), asDouble.end(), 0.0);
        const uint64_t zerosSeen = world * static_cast<uint64_t>(B) * H;
        asDouble[hist::binIndex(0.0f, range.first, range.second, bins)] = static_cast<double>(zerosSeen);
        hist::mergeBatch(batchOf(op), asDouble.data(), range.first, range.second, zerosSeen);
    };
    for (int j = 0; j < n; ++j) {
        if (src[j].op == RXMET_LSTM_OUTPUT && src[j].data == tr.hidden_outputs && !user.h0) zeros(RXMET_LSTM_OUTPUT);
        if (src[j].op == RXMET_LSTM_CELL_STATE && src[j].data == tr.cell_states && !user.c0) zeros(RXMET_LSTM_CELL_STATE);
        if (!jobStats[j].finite) continue;
        for (int i = 0; i < bins; ++i) asDouble[i] = static_cast<double>(counts[static_cast<size_t>(j) * bins + i]);
        hist::mergeBatch(batchOf(src[j].op), asDouble.data(), jobs[j].lo, jobs[j].hi, jobStats[j].finite);
    }
    for (int op = 0; op < kOps; ++op) {
        if (isParameter(op) || !batch[op]) continue;
        checkCollector(&hs->point[op]);
        hist::merge(&hs->point[op], batch[op]->h);
    }
    const std::vector<float> *values[4] = {&wIh, &wHh, &bIh, &bHh};
    const int widths[4] = {I, H, 1, 1};
    for (int slot = 0; slot < 4; ++slot) {
        const int op = RXMET_LSTM_WEIGHT_IH + slot;
        if (isBias(op) && !bias) continue;
        observeParameter(*values[slot], widths[slot], H, cfg.granularity[op], &hs->point[op], hs->gate[slot], hs->channel[slot], bins);
    }
}

void paramsFromHistograms(const rxmet_lstm_quant_config &cfg, const rxmet_lstm_ranges &observed, const rxmet_lstm_histograms &hs,
                          int method, float percentile, int inputSize, int hidden, bool bias, float *wIhScale,
                          float *wHhScale, float *bIhScale, float *bHhScale, rxmet_lstm_quant_params *out) {
    RXMET_REQUIRE(hs.hidden_size == hidden, "histogram collectors were made for another hidden size");
    const int C = 4 * hidden;
    rxmet_lstm_ranges selected = observed;
    std::vector<float> lo[4], hi[4];
    for (int slot = 0; slot < 4; ++slot) {
        lo[slot].assign(C, 0.0f);
        hi[slot].assign(C, 0.0f);
        if (observed.channel_min[slot] && observed.channel_max[slot]) {
            std::copy(observed.channel_min[slot], observed.channel_min[slot] + C, lo[slot].begin());
            std::copy(observed.channel_max[slot], observed.channel_max[slot] + C, hi[slot].begin());
        }
        selected.channel_min[slot] = lo[slot].data();
        selected.channel_max[slot] = hi[slot].data();
    }
    auto choose = [&](const rxmet_lstm_histogram &h, int op) {
        checkCollector(&h);
        return hist::selectRange(h, cfg.bitwidth[op], cfg.is_unsigned[op] != 0, cfg.is_symmetric[op] != 0, method, percentile);
    };
    for (int op = 0; op < kOps; ++op) {
        if (isBias(op)) continue;  // biases keep their observed range
        if (!isParameter(op)) {
            const auto r = choose(hs.point[op], op);
            selected.minimum[op] = r.first;
            selected.maximum[op] = r.second;
            continue;
        }
        const int slot = op - RXMET_LSTM_WEIGHT_IH;
        const int gran = cfg.granularity[op];
        const int span = gran == RXMET_LSTM_PER_TENSOR ? C : (gran == RXMET_LSTM_PER_GATE ? hidden : 1);
        for (int first = 0; first < C; first += span) {
            const rxmet_lstm_histogram &h = gran == RXMET_LSTM_PER_TENSOR ? hs.point[op]
                                            : (gran == RXMET_LSTM_PER_GATE ? hs.gate[slot][first / hidden] : hs.channel[slot][first]);
            const auto r = choose(h, op);
            std::fill(lo[slot].begin() + first, lo[slot].begin() + first + span, r.first);
            std::fill(hi[slot].begin() + first, hi[slot].begin() + first + span, r.second);
        }
    }
    paramsFromRanges(cfg, selected, inputSize, hidden, bias, wIhScale, wHhScale, bIhScale, bHhScale, out);
}

}  // namespace lstm
}  // namespace rxmet

using namespace rxmet;

extern "C" {

int rxmet_lstm_histogram_collect_host(rxmet_lstm_histogram *h, const float *data, uint64_t count) {
    return guarded([&] {
        lstm::checkCollector(h);
        RXMET_REQUIRE(data != nullptr || count == 0, "data must not be null");
        lstm::hist::collectHost(h, data, 1, count, count);
    });
}

int rxmet_lstm_histogram_merge(rxmet_lstm_histogram *h, const rxmet_lstm_histogram *other) {
    return guarded([&] {
        lstm::checkCollector(h);
        RXMET_REQUIRE(other != nullptr, "other must not be null");
        lstm::hist::merge(h, *other);
    });
}

int rxmet_lstm_histogram_range(const rxmet_lstm_histogram *h, int bitwidth, int is_unsigned, int is_symmetric, int method,
                               float percentile, float *range_min, float *range_max) {
    return guarded([&] {
        lstm::checkCollector(h);
        RXMET_REQUIRE(bitwidth >= 1 && bitwidth <= 31 && range_min && range_max, "bad arguments");
        const auto r = lstm::hist::selectRange(*h, bitwidth, is_unsigned != 0, is_symmetric != 0, method, percentile);
        *range_min = r.first;
        *range_max = r.second;
    });
}

int rxmet_lstm_forward_calibrate_hist(int T, int B, int I, int H, const float *weight_ih, const float *weight_hh,
                                      const float *bias_ih, const float *bias_hh, const float *x, const float *h0,
                                      const float *c0, float *output, float *final_hidden, float *final_cell,
                                      const rxmet_lstm_quant_config *config, rxmet_lstm_ranges *ranges,
                                      rxmet_lstm_histograms *hists, void *workspace, size_t workspace_bytes, void *stream) {
    return guarded([&] {
        RXMET_REQUIRE(T > 0 && B > 0 && I > 0 && H > 0, "LSTM dimensions must be positive");
        RXMET_REQUIRE(weight_ih && weight_hh && x && output && final_hidden && final_cell && config && ranges && hists, "null argument");
        RXMET_REQUIRE((bias_ih == nullptr) == (bias_hh == nullptr), "bias_ih and bias_hh are given together or not at all");
        RXMET_REQUIRE((h0 == nullptr) == (c0 == nullptr), "h0 and c0 are given together or not at all");
        lstm::ForwardFloatCall call{};
        call.T = T; call.B = B; call.I = I; call.H = H;
        call.weightIh = weight_ih; call.weightHh = weight_hh; call.biasIh = bias_ih; call.biasHh = bias_hh;
        call.x = x; call.h0 = h0; call.c0 = c0;
        call.output = output; call.finalHidden = final_hidden; call.finalCell = final_cell;
        lstm::forwardCalibrateHist(call, *config, ranges, hists, workspace, workspace_bytes, static_cast<cudaStream_t>(stream),
                                   nullptr);
    });
}

int rxmet_lstm_forward_calibrate_hist_dp(int T, int B, int I, int H, const float *weight_ih, const float *weight_hh,
                                         const float *bias_ih, const float *bias_hh, const float *x, const float *h0,
                                         const float *c0, float *output, float *final_hidden, float *final_cell,
                                         const rxmet_lstm_quant_config *config, rxmet_lstm_ranges *ranges,
                                         rxmet_lstm_histograms *hists, void *workspace, size_t workspace_bytes, void *stream,
                                         const rxmet_exchange *exchange) {
    return guarded([&] {
        RXMET_REQUIRE(T > 0 && B > 0 && I > 0 && H > 0, "LSTM dimensions must be positive");
        RXMET_REQUIRE(weight_ih && weight_hh && x && output && final_hidden && final_cell && config && ranges && hists, "null argument");
        RXMET_REQUIRE((bias_ih == nullptr) == (bias_hh == nullptr), "bias_ih and bias_hh are given together or not at all");
        RXMET_REQUIRE((h0 == nullptr) == (c0 == nullptr), "h0 and c0 are given together or not at all");
        lstm::ForwardFloatCall call{};
        call.T = T; call.B = B; call.I = I; call.H = H;
        call.weightIh = weight_ih; call.weightHh = weight_hh; call.biasIh = bias_ih; call.biasHh = bias_hh;
        call.x = x; call.h0 = h0; call.c0 = c0;
        call.output = output; call.finalHidden = final_hidden; call.finalCell = final_cell;
        lstm::forwardCalibrateHist(call, *config, ranges, hists, workspace, workspace_bytes, static_cast<cudaStream_t>(stream),
                                   exchange);
    });
}

int rxmet_lstm_histogram_batch_range(float batch_min, float batch_max, float *range_min, float *range_max) {
    return guarded([&] {
        RXMET_REQUIRE(range_min && range_max, "output pointers must not be null");
        const auto r = lstm::hist::batchRange(batch_min, batch_max);
        *range_min = r.first;
        *range_max = r.second;
    });
}

int rxmet_lstm_histogram_count_host(float range_min, float range_max, int num_bins, const float *data, uint64_t count,
                                    uint64_t *counts, uint64_t *finite) {
    return guarded([&] {
        RXMET_REQUIRE(num_bins >= 2 && counts && finite && (data || count == 0), "bad arguments");
        for (uint64_t i = 0; i < count; ++i) {
            if (!std::isfinite(data[i])) continue;
            ++counts[lstm::hist::binIndex(data[i], range_min, range_max, num_bins)];
            ++*finite;
        }
    });
}

int rxmet_lstm_histogram_merge_counts(rxmet_lstm_histogram *h, const uint64_t *counts, float range_min, float range_max,
                                      uint64_t finite) {
    return guarded([&] {
        lstm::checkCollector(h);
        RXMET_REQUIRE(counts != nullptr, "counts must not be null");
        if (finite == 0) return;
        std::vector<double> asDouble(h->num_bins);
        for (int i = 0; i < h->num_bins; ++i) asDouble[i] = static_cast<double>(counts[i]);
        lstm::hist::mergeBatch(h, asDouble.data(), range_min, range_max, finite);
    });
}

int rxmet_lstm_params_from_histograms(const rxmet_lstm_quant_config *config, const rxmet_lstm_ranges *ranges,
                                      const rxmet_lstm_histograms *hists, int method, float percentile, int input_size,
                                      int hidden_size, int bias_enabled, float *weight_ih_scale, float *weight_hh_scale,
                                      float *bias_ih_scale, float *bias_hh_scale, rxmet_lstm_quant_params *params) {
    return guarded([&] {
        RXMET_REQUIRE(config && ranges && hists && params && weight_ih_scale && weight_hh_scale, "null argument");
        lstm::paramsFromHistograms(*config, *ranges, *hists, method, percentile, input_size, hidden_size, bias_enabled != 0,
                                   weight_ih_scale, weight_hh_scale, bias_ih_scale, bias_hh_scale, params);
    });
}

}  // extern "C"
