// extern "C" surface of librxmet_b200.so (declared in include/rxmet_b200.h).  Validates
// arguments, turns exceptions into status codes and hands over to the kernel launchers.
#include <cuda_runtime.h>

#include <algorithm>
#include <cfloat>
#include <cstring>
#include <map>
#include <tuple>
#include <mutex>
#include <string>
#include <vector>

#include "common.h"
#include "gru_backward.h"
#include "gru_forward_float.h"
#include "gru_forward_quant.h"
#include "gru_params.h"
#include "rxmet_b200.h"

namespace rxmet {

std::string &lastError() {
    static thread_local std::string message;
    return message;
}
std::atomic<uint64_t> &launchCounter() {
    static std::atomic<uint64_t> counter{0};
    return counter;
}

namespace {
struct TimingState {
    std::mutex mutex;
    bool enabled = false;
    struct Pending { std::string name; cudaEvent_t start, stop; };
    std::vector<Pending> pending;
    std::map<std::string, std::pair<double, long long>> totals;  // name -> (ms, launches)
};
TimingState &timing() {
    static TimingState state;
    return state;
}
}  // namespace

bool kernelTimingEnabled() { return timing().enabled; }

const DeviceInfo &currentDevice() {
    constexpr int kMaxDevices = 64;
    static DeviceInfo table[kMaxDevices];
    static std::atomic<bool> known[kMaxDevices];
    int device = 0;
    RXMET_CUDA(cudaGetDevice(&device));
    if (device < 0 || device >= kMaxDevices) fail(RXMET_ERR_UNSUPPORTED, "device ordinal %d", device);
    if (!known[device].load(std::memory_order_acquire)) {
        DeviceInfo info;
        info.device = device;
        RXMET_CUDA(cudaDeviceGetAttribute(&info.smemMax, cudaDevAttrMaxSharedMemoryPerBlockOptin, device));
        RXMET_CUDA(cudaDeviceGetAttribute(&info.sms, cudaDevAttrMultiProcessorCount, device));
        table[device] = info;  // racing threads write the same values
        known[device].store(true, std::memory_order_release);
    }
    return table[device];
}

void ensureDynamicSmem(const void *kernel, size_t bytes) {
    static std::mutex guard;
    static std::map<std::pair<int, const void *>, size_t> granted;
    const int device = currentDevice().device;
    std::lock_guard<std::mutex> lock(guard);
    size_t &have = granted[{device, kernel}];
    if (bytes <= have) return;
    RXMET_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)));
    have = bytes;
}

int residentPerSm(const void *kernel, int block, size_t smem) {
    static std::mutex guard;
    static std::map<std::tuple<int, const void *, int, size_t>, int> known;
    const int device = currentDevice().device;
    std::lock_guard<std::mutex> lock(guard);
    int &n = known[{device, kernel, block, smem}];
    if (n == 0) {
        RXMET_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, block, smem));
        n = std::max(n, 1);
    }
    return n;
}

OverlapLane &overlapLane() {
    constexpr int kMaxDevices = 64;
    static thread_local OverlapLane lanes[kMaxDevices];
    const int device = currentDevice().device;
    OverlapLane &lane = lanes[device];
    if (lane.stream == nullptr) {
        RXMET_CUDA(cudaStreamCreateWithFlags(&lane.stream, cudaStreamNonBlocking));
        for (int i = 0; i < kLaneEvents; ++i) {
            RXMET_CUDA(cudaEventCreateWithFlags(&lane.fork[i], cudaEventDisableTiming));
            RXMET_CUDA(cudaEventCreateWithFlags(&lane.done[i], cudaEventDisableTiming));
        }
    }
    return lane;
}

std::vector<int> overlapChunks(int T, size_t rows, bool backward) {
    std::vector<int> percent;
    if (const char *env = std::getenv(backward ? "RXMET_GRU_BWD_CHUNKS" : "RXMET_GRU_FWD_CHUNKS")) {
        for (const char *p = env; *p;) {
            char *end = nullptr;
            const long v = std::strtol(p, &end, 10);
            if (end == p) break;
            if (v > 0) percent.push_back(static_cast<int>(v));
            p = (*end == ',') ? end + 1 : end;
            if (*end != ',') break;
        }
    }
    // No cut by default: on a B200 at T = 100, B = 256, I = 40, H = 128 every cut measured slower than the
    // single launches (the GEMM CTAs sharing the SMs slow the recurrence's serial chain by more than they hide).
    (void)rows;
    if (percent.size() < 2 || percent.size() > static_cast<size_t>(kLaneEvents)) return {T};
    if (backward) {
        // the backward runs the time axis downwards and its batched work FOLLOWS each chunk: the short chunk last
        std::reverse(percent.begin(), percent.end());
    }
    int total = 0;
    for (int v : percent) total += v;
    std::vector<int> steps;
    int used = 0;
    for (size_t i = 0; i < percent.size(); ++i) {
        int n = (i + 1 == percent.size()) ? T - used : static_cast<int>(static_cast<long long>(T) * percent[i] / total);
        n = std::max(0, std::min(n, T - used));
        if (n > 0) steps.push_back(n);
        used += n;
    }
    if (steps.empty()) steps.push_back(T);
    return steps;
}

void kernelTimingBegin(const char *, cudaStream_t stream, cudaEvent_t *start, cudaEvent_t *stop) {
    if (cudaEventCreate(start) != cudaSuccess || cudaEventCreate(stop) != cudaSuccess) {
        *start = *stop = nullptr;
        return;
    }
    cudaEventRecord(*start, stream);
}

void kernelTimingEnd(const char *name, cudaStream_t stream, cudaEvent_t start, cudaEvent_t stop) {
    cudaEventRecord(stop, stream);
    TimingState &t = timing();
    std::lock_guard<std::mutex> lock(t.mutex);
    t.pending.push_back({name, start, stop});
}

namespace {

void checkDims(int T, int B, int I, int H) {
    RXMET_REQUIRE(T > 0 && B > 0 && I > 0 && H > 0, "GRU dimensions must be positive (T=%d B=%d I=%d H=%d)", T, B, I, H);
    RXMET_REQUIRE(static_cast<long long>(T) * B * 4LL * H < (1LL << 40), "GRU problem too large");
}

#define RXMET_PTR(p) RXMET_REQUIRE((p) != nullptr, #p " must not be null")

float *channelArray(rxmet_gru_ranges *r, int k, bool isMax) {
    float *mins[4] = {r->min_W, r->min_R, r->min_bw, r->min_br};
    float *maxs[4] = {r->max_W, r->max_R, r->max_bw, r->max_br};
    return isMax ? maxs[k] : mins[k];
}

// Folds one call's packed statistics into the running ranges.  A point with no finite
// observation in this call observes 0, as the reference does per call.
void foldStats(rxmet_gru_ranges *r, const float *stats) {
    const int H = r->hidden, C = 3 * H;
    const size_t half = gru::statsFloats(H) / 2;
    const float *mins = stats, *maxs = stats + half;
    for (int op = 0; op < gru::kOps; ++op) {
        if (op == RXMET_GRU_W || op == RXMET_GRU_R || op == RXMET_GRU_BW || op == RXMET_GRU_BR) continue;
        float lo = mins[op], hi = maxs[op];
        if (lo > hi) lo = hi = 0.0f;
        r->min[op] = std::min(r->min[op], lo);
        r->max[op] = std::max(r->max[op], hi);
    }
    for (int k = 0; k < 4; ++k) {
        float *dstMin = channelArray(r, k, false), *dstMax = channelArray(r, k, true);
        RXMET_REQUIRE(dstMin && dstMax, "ranges: per-channel arrays are not set");
        for (int c = 0; c < C; ++c) {
            dstMin[c] = std::min(dstMin[c], mins[gru::kOps + k * C + c]);
            dstMax[c] = std::max(dstMax[c], maxs[gru::kOps + k * C + c]);
        }
    }
}

}  // namespace
}  // namespace rxmet

namespace rxmet {
std::atomic<int> &concurrentPassesSetting() {
    static std::atomic<int> passes{1};
    return passes;
}
int concurrentPasses() { return concurrentPassesSetting().load(); }
}  // namespace rxmet

using namespace rxmet;

extern "C" {

const char *rxmet_last_error(void) { return lastError().c_str(); }
const char *rxmet_version(void) { return "rxmet_b200 0.1.0 (sm_100a)"; }
uint64_t rxmet_kernel_launch_count(void) { return launchCounter().load(); }

int rxmet_set_concurrent_passes(int passes) {
    concurrentPassesSetting().store(passes < 1 ? 1 : passes);
    return RXMET_OK;
}

int rxmet_set_kernel_timing(int enabled) {
    return guarded([&] {
        TimingState &t = timing();
        std::lock_guard<std::mutex> lock(t.mutex);
        t.enabled = enabled != 0;
        if (!enabled) {
            for (auto &p : t.pending) { cudaEventDestroy(p.start); cudaEventDestroy(p.stop); }
            t.pending.clear();
            t.totals.clear();
        }
    });
}

int rxmet_get_kernel_timing(const char *kernel_name, double *total_ms, long long *launches) {
    return guarded([&] {
        RXMET_PTR(kernel_name); RXMET_PTR(total_ms); RXMET_PTR(launches);
        TimingState &t = timing();
        std::lock_guard<std::mutex> lock(t.mutex);
        for (auto &p : t.pending) {
            RXMET_CUDA(cudaEventSynchronize(p.stop));
            float ms = 0.0f;
            RXMET_CUDA(cudaEventElapsedTime(&ms, p.start, p.stop));
            auto &slot = t.totals[p.name];
            slot.first += ms;
            slot.second += 1;
            cudaEventDestroy(p.start);
            cudaEventDestroy(p.stop);
        }
        t.pending.clear();
        const auto it = t.totals.find(kernel_name);
        *total_ms = it == t.totals.end() ? 0.0 : it->second.first;
        *launches = it == t.totals.end() ? 0 : it->second.second;
    });
}

int rxmet_reset_kernel_timing(void) {
    return guarded([&] {
        TimingState &t = timing();
        std::lock_guard<std::mutex> lock(t.mutex);
        for (auto &p : t.pending) { cudaEventDestroy(p.start); cudaEventDestroy(p.stop); }
        t.pending.clear();
        t.totals.clear();
    });
}

void rxmet_gru_default_config(rxmet_gru_quant_config *cfg) {
    if (!cfg) return;
    for (int i = 0; i < RXMET_GRU_NUM_OPS; ++i) {
        cfg->bits[i] = 8;
        cfg->is_unsigned[i] = (i == RXMET_GRU_UPDATE_GATE_OUTPUT || i == RXMET_GRU_RESET_GATE_OUTPUT) ? 1 : 0;
        cfg->symmetric[i] = 1;
    }
    cfg->W_granularity = cfg->R_granularity = cfg->bw_granularity = cfg->br_granularity = RXMET_PER_CHANNEL;
    cfg->use_pot2 = 0;
    cfg->pot_scale_method = RXMET_POT_COVER_RANGE;
    cfg->pot_scale_tolerance = 0.02f;
}

int rxmet_gru_ranges_reset(rxmet_gru_ranges *r) {
    return guarded([&] {
        RXMET_PTR(r);
        RXMET_REQUIRE(r->hidden > 0, "ranges: hidden must be > 0");
        for (int i = 0; i < RXMET_GRU_NUM_OPS; ++i) {
            r->min[i] = FLT_MAX;
            r->max[i] = -FLT_MAX;
        }
        for (int k = 0; k < 4; ++k) {
            float *mn = channelArray(r, k, false), *mx = channelArray(r, k, true);
            RXMET_REQUIRE(mn && mx, "ranges: per-channel arrays are not set");
            std::fill(mn, mn + 3 * r->hidden, FLT_MAX);
            std::fill(mx, mx + 3 * r->hidden, -FLT_MAX);
        }
    });
}

int rxmet_gru_params_from_ranges(const rxmet_gru_ranges *ranges, const rxmet_gru_quant_config *cfg,
                                 rxmet_gru_quant_params *out) {
    return guarded([&] {
        RXMET_PTR(ranges); RXMET_PTR(cfg); RXMET_PTR(out);
        gru::paramsFromRanges(*ranges, *cfg, out);
    });
}

int rxmet_gru_build_luts(const rxmet_gru_quant_params *params, rxmet_lut_segment out_segments[3][16]) {
    return guarded([&] {
        RXMET_PTR(params); RXMET_PTR(out_segments);
        gru::buildLuts(*params, out_segments);
    });
}

int rxmet_gru_decode_effective_scale(float scale, int use_pot2, float *out) {
    return guarded([&] {
        RXMET_PTR(out);
        *out = gru::decodeEffectiveScale(scale, use_pot2 != 0);
    });
}

size_t rxmet_gru_workspace_bytes(int op, int T, int B, int I, int H) {
    if (T <= 0 || B <= 0 || I <= 0 || H <= 0) return 0;
    switch (op) {
        case 0: return gru::forwardFloatWorkspaceBytes(T, B, I, H);
        case 1: return gru::forwardQuantWorkspaceBytes(T, B, I, H);
        case 2: return gru::backwardWorkspaceBytes(T, B, I, H);
        case 3: return gru::histCalibrationWorkspaceBytes(T, B, I, H, 8192);
        default: return 0;
    }
}

size_t rxmet_gru_stats_floats(int H) { return H > 0 ? gru::statsFloats(H) : 0; }

static void runFloat(int T, int B, int I, int H, const float *W, const float *R, const float *bw, const float *br,
                     const float *x, const float *h0, float *h, float *v, float *stats, void *ws, size_t wsBytes,
                     void *stream) {
    checkDims(T, B, I, H);
    RXMET_PTR(W); RXMET_PTR(R); RXMET_PTR(bw); RXMET_PTR(br); RXMET_PTR(x); RXMET_PTR(h); RXMET_PTR(v);
    gru::ForwardFloatCall call;
    call.T = T; call.B = B; call.I = I; call.H = H;
    call.W = W; call.R = R; call.bw = bw; call.br = br; call.x = x; call.h0 = h0; call.h = h; call.v = v;
    call.stats = stats;
    gru::forwardFloat(call, ws, wsBytes, static_cast<cudaStream_t>(stream));
}

int rxmet_gru_forward_fp(int T, int B, int I, int H, const float *W_dev, const float *R_dev, const float *bw_dev,
                         const float *br_dev, const float *x_dev, const float *h0_dev, float *h_dev, float *v_dev,
                         void *workspace_dev, size_t workspace_bytes, void *stream) {
    return guarded([&] {
        runFloat(T, B, I, H, W_dev, R_dev, bw_dev, br_dev, x_dev, h0_dev, h_dev, v_dev, nullptr, workspace_dev,
                 workspace_bytes, stream);
    });
}

int rxmet_gru_forward_calibrate_stats(int T, int B, int I, int H, const float *W_dev, const float *R_dev,
                                      const float *bw_dev, const float *br_dev, const float *x_dev,
                                      const float *h0_dev, float *h_dev, float *v_dev, float *stats_dev,
                                      void *workspace_dev, size_t workspace_bytes, void *stream) {
    return guarded([&] {
        RXMET_PTR(stats_dev);
        runFloat(T, B, I, H, W_dev, R_dev, bw_dev, br_dev, x_dev, h0_dev, h_dev, v_dev, stats_dev, workspace_dev,
                 workspace_bytes, stream);
    });
}

int rxmet_gru_ranges_fold_stats(rxmet_gru_ranges *ranges, const float *stats_host) {
    return guarded([&] {
        RXMET_PTR(ranges); RXMET_PTR(stats_host);
        RXMET_REQUIRE(ranges->hidden > 0, "ranges: hidden must be > 0");
        foldStats(ranges, stats_host);
    });
}

int rxmet_gru_forward_calibrate_minmax(int T, int B, int I, int H, const float *W_dev, const float *R_dev,
                                       const float *bw_dev, const float *br_dev, const float *x_dev,
                                       const float *h0_dev, float *h_dev, float *v_dev, rxmet_gru_ranges *ranges,
                                       void *workspace_dev, size_t workspace_bytes, void *stream) {
    return guarded([&] {
        RXMET_PTR(ranges);
        RXMET_REQUIRE(ranges->hidden == H, "ranges were set up for hidden=%d, call has H=%d", ranges->hidden, H);
        // The packed statistics take the head of the caller's workspace, the forward the rest.
        const size_t statBytes = gru::statsFloats(H) * sizeof(float);
        const size_t head = alignUp(statBytes, 256);
        const size_t need = gru::forwardFloatWorkspaceBytes(T, B, I, H);
        if (workspace_dev == nullptr || workspace_bytes < need)
            fail(RXMET_ERR_WORKSPACE, "workspace too small: need at least %zu bytes, have %zu", need, workspace_bytes);
        float *stats = static_cast<float *>(workspace_dev);
        runFloat(T, B, I, H, W_dev, R_dev, bw_dev, br_dev, x_dev, h0_dev, h_dev, v_dev, stats,
                 static_cast<char *>(workspace_dev) + head, workspace_bytes - head, stream);
        std::vector<float> host(gru::statsFloats(H));
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        RXMET_CUDA(cudaMemcpyAsync(host.data(), stats, statBytes, cudaMemcpyDeviceToHost, st));
        RXMET_CUDA(cudaStreamSynchronize(st));
        foldStats(ranges, host.data());
    });
}

static void runQuant(gru::ForwardQuantCall &call, const rxmet_gru_quant_params *params, void *ws, size_t wsBytes,
                     void *stream) {
    checkDims(call.T, call.B, call.I, call.H);
    RXMET_PTR(params);
    RXMET_REQUIRE(params->hidden == call.H, "quant params were made for hidden=%d, call has H=%d", params->hidden, call.H);
    RXMET_PTR(call.W); RXMET_PTR(call.R); RXMET_PTR(call.bw); RXMET_PTR(call.br);
    const auto exec = gru::deriveExec(*params);
    gru::forwardQuant(call, *exec, ws, wsBytes, static_cast<cudaStream_t>(stream));
}

int rxmet_gru_forward_quant(int is_training, int T, int B, int I, int H, const float *W_dev, const float *R_dev,
                            const float *bw_dev, const float *br_dev, const float *x_dev, const float *h0_dev,
                            const rxmet_gru_quant_params *params, float *h_dev, float *v_dev, int32_t *W_q_dev,
                            int32_t *R_q_dev, int32_t *bw_q_dev, int32_t *br_q_dev, int32_t *x_q_dev, int32_t *h_q_dev,
                            int32_t *v_q_dev, const rxmet_gru_masks *masks, void *workspace_dev,
                            size_t workspace_bytes, void *stream) {
    return guarded([&] {
        RXMET_PTR(x_dev); RXMET_PTR(h_dev); RXMET_PTR(v_dev);
        gru::ForwardQuantCall call;
        call.isTraining = is_training;
        call.T = T; call.B = B; call.I = I; call.H = H;
        call.W = W_dev; call.R = R_dev; call.bw = bw_dev; call.br = br_dev; call.x = x_dev; call.h0 = h0_dev;
        call.h = h_dev; call.v = v_dev;
        call.W_q = W_q_dev; call.R_q = R_q_dev; call.bw_q = bw_q_dev; call.br_q = br_q_dev; call.x_q = x_q_dev;
        call.h_q = h_q_dev; call.v_q = v_q_dev;
        call.masks = masks;
        runQuant(call, params, workspace_dev, workspace_bytes, stream);
    });
}

int rxmet_gru_forward_quant_int_io(int T, int B, int I, int H, const float *W_dev, const float *R_dev,
                                   const float *bw_dev, const float *br_dev, const int32_t *x_q_dev,
                                   const int32_t *h0_q_dev, const rxmet_gru_quant_params *params, int32_t *h_q_dev,
                                   void *workspace_dev, size_t workspace_bytes, void *stream) {
    return guarded([&] {
        RXMET_PTR(x_q_dev); RXMET_PTR(h_q_dev);
        checkDims(T, B, I, H);
        // The dequantized outputs are not wanted here; they go to scratch behind the regular workspace.
        const size_t base = gru::forwardQuantWorkspaceBytes(T, B, I, H);
        const size_t hBytes = alignUp(sizeof(float) * (static_cast<size_t>(T) + 1) * B * H, 256);
        const size_t vBytes = alignUp(sizeof(float) * static_cast<size_t>(T) * B * 4 * H, 256);
        if (workspace_dev == nullptr || workspace_bytes < base + hBytes + vBytes)
            fail(RXMET_ERR_WORKSPACE, "workspace too small: need at least %zu bytes, have %zu", base + hBytes + vBytes,
                 workspace_bytes);
        char *tail = static_cast<char *>(workspace_dev) + alignUp(base, 256);
        gru::ForwardQuantCall call;
        call.T = T; call.B = B; call.I = I; call.H = H;
        call.W = W_dev; call.R = R_dev; call.bw = bw_dev; call.br = br_dev;
        call.x_codes_in = x_q_dev; call.h0_codes_in = h0_q_dev;
        call.h = reinterpret_cast<float *>(tail);
        call.v = reinterpret_cast<float *>(tail + hBytes);
        call.h_q = h_q_dev;
        runQuant(call, params, workspace_dev, base, stream);
    });
}

static void runBackward(gru::BackwardCall &call, void *ws, size_t wsBytes, void *stream) {
    checkDims(call.T, call.B, call.I, call.H);
    RXMET_PTR(call.dh_new); RXMET_PTR(call.h); RXMET_PTR(call.v);
    RXMET_PTR(call.dx); RXMET_PTR(call.dW); RXMET_PTR(call.dR); RXMET_PTR(call.dbw); RXMET_PTR(call.dbr);
    RXMET_PTR(call.dh0);
    gru::backward(call, ws, wsBytes, static_cast<cudaStream_t>(stream));
}

int rxmet_gru_backward_quant(int T, int B, int I, int H, const int32_t *W_q_dev, const int32_t *R_q_dev,
                             const int32_t *bw_q_dev, const int32_t *br_q_dev, const int32_t *x_q_dev,
                             const float *dh_new_dev, const float *h_dev, const float *v_dev,
                             const rxmet_gru_quant_params *params, const rxmet_gru_masks *masks, float *dx_dev,
                             float *dW_dev, float *dR_dev, float *dbw_dev, float *dbr_dev, float *dh0_dev,
                             void *workspace_dev, size_t workspace_bytes, void *stream) {
    (void)bw_q_dev; (void)br_q_dev;  // bias values do not enter the derivative, only their masks do
    return guarded([&] {
        RXMET_PTR(params); RXMET_PTR(W_q_dev); RXMET_PTR(R_q_dev); RXMET_PTR(x_q_dev);
        RXMET_REQUIRE(params->hidden == H, "quant params were made for hidden=%d, call has H=%d", params->hidden, H);
        const auto exec = gru::deriveExec(*params);
        gru::BackwardCall call;
        call.T = T; call.B = B; call.I = I; call.H = H;
        call.W_q = W_q_dev; call.R_q = R_q_dev; call.x_q = x_q_dev; call.exec = exec.get();
        call.dh_new = dh_new_dev; call.h = h_dev; call.v = v_dev; call.masks = masks;
        call.dx = dx_dev; call.dW = dW_dev; call.dR = dR_dev; call.dbw = dbw_dev; call.dbr = dbr_dev; call.dh0 = dh0_dev;
        runBackward(call, workspace_dev, workspace_bytes, stream);
    });
}

int rxmet_gru_forward_quant_fp_carrier(int is_training, int T, int B, int I, int H, const float *W_dev, const float *R_dev,
                                       const float *bw_dev, const float *br_dev, const float *x_dev, const float *h0_dev,
                                       const rxmet_gru_quant_params *params, float *h_dev, float *v_dev, int32_t *W_q_dev,
                                       int32_t *R_q_dev, int32_t *bw_q_dev, int32_t *br_q_dev, int32_t *x_q_dev,
                                       int32_t *h_q_dev, int32_t *v_q_dev, const rxmet_gru_masks *masks, void *workspace_dev,
                                       size_t workspace_bytes, void *stream) {
    return guarded([&] {
        RXMET_PTR(x_dev); RXMET_PTR(h_dev); RXMET_PTR(v_dev); RXMET_PTR(params);
        gru::ForwardQuantCall call;
        call.isTraining = is_training;
        call.T = T; call.B = B; call.I = I; call.H = H;
        call.W = W_dev; call.R = R_dev; call.bw = bw_dev; call.br = br_dev; call.x = x_dev; call.h0 = h0_dev;
        call.h = h_dev; call.v = v_dev;
        call.W_q = W_q_dev; call.R_q = R_q_dev; call.bw_q = bw_q_dev; call.br_q = br_q_dev; call.x_q = x_q_dev;
        call.h_q = h_q_dev; call.v_q = v_q_dev;
        call.masks = masks;
        call.fpCarrier = params;
        runQuant(call, params, workspace_dev, workspace_bytes, stream);
    });
}

int rxmet_gru_packed_flags_supported(const rxmet_gru_quant_params *params, int B, int I, int H) {
    int supported = 0;
    const int rc = guarded([&] {
        RXMET_PTR(params);
        RXMET_REQUIRE(params->hidden == H, "quant params were made for hidden=%d, call has H=%d", params->hidden, H);
        supported = gru::packedFlagsSupported(*gru::deriveExec(*params), B, I, H) ? 1 : 0;
    });
    return rc == RXMET_OK ? supported : 0;
}

int rxmet_gru_forward_quant_packed(int T, int B, int I, int H, const float *W_dev, const float *R_dev, const float *bw_dev,
                                   const float *br_dev, const float *x_dev, const float *h0_dev,
                                   const rxmet_gru_quant_params *params, float *h_dev, float *v_dev, int32_t *W_q_dev,
                                   int32_t *R_q_dev, int32_t *bw_q_dev, int32_t *br_q_dev, int32_t *x_q_dev,
                                   const rxmet_gru_masks *masks, uint16_t *step_flags_dev, void *workspace_dev,
                                   size_t workspace_bytes, void *stream) {
    return guarded([&] {
        RXMET_PTR(x_dev); RXMET_PTR(h_dev); RXMET_PTR(v_dev); RXMET_PTR(masks); RXMET_PTR(step_flags_dev);
        gru::ForwardQuantCall call;
        call.isTraining = 1;
        call.T = T; call.B = B; call.I = I; call.H = H;
        call.W = W_dev; call.R = R_dev; call.bw = bw_dev; call.br = br_dev; call.x = x_dev; call.h0 = h0_dev;
        call.h = h_dev; call.v = v_dev;
        call.W_q = W_q_dev; call.R_q = R_q_dev; call.bw_q = bw_q_dev; call.br_q = br_q_dev; call.x_q = x_q_dev;
        call.masks = masks;
        call.stepFlags = step_flags_dev;
        runQuant(call, params, workspace_dev, workspace_bytes, stream);
    });
}

int rxmet_gru_backward_quant_packed(int T, int B, int I, int H, const int32_t *W_q_dev, const int32_t *R_q_dev,
                                    const int32_t *x_q_dev, const float *dh_new_dev, const float *h_dev, const float *v_dev,
                                    const rxmet_gru_quant_params *params, const rxmet_gru_masks *masks,
                                    const uint16_t *step_flags_dev, float *dx_dev, float *dW_dev, float *dR_dev,
                                    float *dbw_dev, float *dbr_dev, float *dh0_dev, void *workspace_dev,
                                    size_t workspace_bytes, void *stream) {
    return guarded([&] {
        RXMET_PTR(params); RXMET_PTR(W_q_dev); RXMET_PTR(R_q_dev); RXMET_PTR(x_q_dev); RXMET_PTR(step_flags_dev);
        RXMET_REQUIRE(params->hidden == H, "quant params were made for hidden=%d, call has H=%d", params->hidden, H);
        const auto exec = gru::deriveExec(*params);
        gru::BackwardCall call;
        call.T = T; call.B = B; call.I = I; call.H = H;
        call.W_q = W_q_dev; call.R_q = R_q_dev; call.x_q = x_q_dev; call.exec = exec.get();
        call.dh_new = dh_new_dev; call.h = h_dev; call.v = v_dev; call.masks = masks;
        call.stepFlags = step_flags_dev;
        call.dx = dx_dev; call.dW = dW_dev; call.dR = dR_dev; call.dbw = dbw_dev; call.dbr = dbr_dev; call.dh0 = dh0_dev;
        runBackward(call, workspace_dev, workspace_bytes, stream);
    });
}

int rxmet_gru_backward_fp(int T, int B, int I, int H, const float *W_dev, const float *R_dev, const float *bw_dev,
                          const float *br_dev, const float *x_dev, const float *dh_new_dev, const float *h_dev,
                          const float *v_dev, float *dx_dev, float *dW_dev, float *dR_dev, float *dbw_dev,
                          float *dbr_dev, float *dh0_dev, void *workspace_dev, size_t workspace_bytes, void *stream) {
    (void)bw_dev; (void)br_dev;
    return guarded([&] {
        RXMET_PTR(W_dev); RXMET_PTR(R_dev); RXMET_PTR(x_dev);
        gru::BackwardCall call;
        call.T = T; call.B = B; call.I = I; call.H = H;
        call.W = W_dev; call.R = R_dev; call.x = x_dev;
        call.dh_new = dh_new_dev; call.h = h_dev; call.v = v_dev;
        call.dx = dx_dev; call.dW = dW_dev; call.dR = dR_dev; call.dbw = dbw_dev; call.dbr = dbr_dev; call.dh0 = dh0_dev;
        runBackward(call, workspace_dev, workspace_bytes, stream);
    });
}

}  // extern "C"
