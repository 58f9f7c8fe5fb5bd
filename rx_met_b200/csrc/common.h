// Shared host-side helpers of the CUDA library: error reporting, launch
// accounting and CUDA call checking.
#pragma once

#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <stdexcept>
#include <string>
#include <vector>

#include "rxmet_b200.h"

namespace rxmet {

// Thread-local message returned by rxmet_last_error().
std::string &lastError();
// Count of kernels launched by this library in this process.
std::atomic<uint64_t> &launchCounter();

struct Error : std::runtime_error {
    int status;
    Error(int s, const std::string &m) : std::runtime_error(m), status(s) {}
};

[[noreturn]] inline void fail(int status, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    throw Error(status, buf);
}

#define RXMET_CUDA(expr)                                                                   \
    do {                                                                                   \
        cudaError_t err__ = (expr);                                                        \
        if (err__ != cudaSuccess)                                                          \
            ::rxmet::fail(RXMET_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(err__)); \
    } while (0)

// Called after every kernel launch: counts it and surfaces launch errors.
inline void afterLaunch(const char *name) {
    launchCounter().fetch_add(1, std::memory_order_relaxed);
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) fail(RXMET_ERR_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(err));
}

#define RXMET_REQUIRE(cond, ...)                                            \
    do {                                                                    \
        if (!(cond)) ::rxmet::fail(RXMET_ERR_INVALID_ARGUMENT, __VA_ARGS__); \
    } while (0)

// Runs f and converts exceptions into status codes + last-error text.
template <class F>
int guarded(F &&f) {
    try {
        f();
        return RXMET_OK;
    } catch (const Error &e) {
        lastError() = e.what();
        return e.status;
    } catch (const std::exception &e) {
        lastError() = e.what();
        return RXMET_ERR_INVALID_ARGUMENT;
    }
}

// Optional per-kernel timing (off by default): while enabled, every launcher brackets its kernel
// with CUDA events on the launching stream; rxmet_get_kernel_timing() resolves and sums them.
bool kernelTimingEnabled();
void kernelTimingBegin(const char *name, cudaStream_t stream, cudaEvent_t *start, cudaEvent_t *stop);
void kernelTimingEnd(const char *name, cudaStream_t stream, cudaEvent_t start, cudaEvent_t stop);

class KernelTimer {
   public:
    KernelTimer(const char *name, cudaStream_t stream) : name_(name), stream_(stream) {
        if (kernelTimingEnabled()) kernelTimingBegin(name_, stream_, &start_, &stop_);
    }
    ~KernelTimer() {
        if (start_) kernelTimingEnd(name_, stream_, start_, stop_);
    }
    KernelTimer(const KernelTimer &) = delete;
    KernelTimer &operator=(const KernelTimer &) = delete;

   private:
    const char *name_;
    cudaStream_t stream_;
    cudaEvent_t start_ = nullptr, stop_ = nullptr;
};

// Properties of the current device, queried once per device and process (the attribute queries
// cost microseconds each, and the hot entry points run once per training step).
struct DeviceInfo {
    int device = 0, sms = 0, smemMax = 0;
};
const DeviceInfo &currentDevice();
// Recurrent passes the caller runs side by side on one GPU (rxmet_set_concurrent_passes); at least 1.
int concurrentPasses();
// SMs one of those passes can count on.
inline int smsPerPass() { return std::max(1, currentDevice().sms / concurrentPasses()); }
// A second stream of this thread on the current device, for work the library runs beside a recurrence that
// occupies the caller's stream, and the events that order the two.  Every user forks from the caller's stream
// (record fork[i] there, make the lane wait for it) and joins back (record done[i] on the lane, make the caller's
// stream wait for it) before it returns, so the pattern is legal inside a stream capture and the caller never
// sees the lane.
constexpr int kLaneEvents = 8;
struct OverlapLane {
    cudaStream_t stream = nullptr;
    cudaEvent_t fork[kLaneEvents] = {};
    cudaEvent_t done[kLaneEvents] = {};
};
OverlapLane &overlapLane();
// Time chunks, in processing order, that a forward (ascending time) or a backward (descending time) over T
// steps is cut into so that the batched GEMM work of one chunk runs under the recurrence of its neighbour;
// one chunk = no overlap.  RXMET_GRU_FWD_CHUNKS / RXMET_GRU_BWD_CHUNKS = "15,35,50" (per cent of the steps, in the
// order of ascending time for the forward; the backward walks the mirror image, short chunk last) override the
// default; a single number switches the cut off.
std::vector<int> overlapChunks(int T, size_t rows, bool backward);
// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) only when `bytes` exceeds what the kernel
// was last given.
void ensureDynamicSmem(const void *kernel, size_t bytes);
// Resident CTAs per SM of `kernel` at this block size and dynamic shared memory, asked once per
// device and configuration (at least 1).
int residentPerSm(const void *kernel, int block, size_t smem);

inline size_t alignUp(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Whether a caller's pointer may be read or written with `bytes`-wide vector accesses (null counts
// as aligned: an absent optional tensor is never touched).  The tensor-core paths issue 16-byte
// asynchronous copies and vector stores on the caller's buffers; a base pointer that fails this
// check sends the call to the kernels that use scalar accesses instead.
inline bool alignedTo(const void *ptr, size_t bytes) { return (reinterpret_cast<uintptr_t>(ptr) & (bytes - 1)) == 0; }

// Carves aligned sub-buffers out of a caller-provided device workspace.
class Workspace {
   public:
    Workspace(void *base, size_t bytes) : base_(static_cast<char *>(base)), bytes_(bytes) {}
    template <class T>
    T *take(size_t count) {
        const size_t off = alignUp(used_, 256);
        const size_t need = off + count * sizeof(T);
        if (base_ == nullptr || need > bytes_)
            fail(RXMET_ERR_WORKSPACE, "workspace too small: need at least %zu bytes, have %zu", need, bytes_);
        used_ = need;
        return reinterpret_cast<T *>(base_ + off);
    }
    size_t used() const { return used_; }

   private:
    char *base_;
    size_t bytes_;
    size_t used_ = 0;
};

// Same arithmetic without a buffer, for the workspace-size query.
class WorkspaceSizer {
   public:
    template <class T>
    void take(size_t count) { used_ = alignUp(used_, 256) + count * sizeof(T); }
    size_t used() const { return alignUp(used_, 256); }

   private:
    size_t used_ = 0;
};

}  // namespace rxmet
