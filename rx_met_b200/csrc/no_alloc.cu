// rxmet_gru_forward_fp_static: the float GRU forward for callers that are not allowed to
// allocate device memory.
//
// Who needs this: code that runs the GRU from inside somebody else's execution callback - an
// inference-runtime plugin's enqueue function, an audio or control loop with a hard deadline, a
// process whose memory pool was sized and frozen at start-up.  Such callers get a stream and
// their input/output buffers and nothing else: a cudaMalloc there either is forbidden outright,
// or would serialise the whole device and break the deadline, or would come out of a pool the
// host application has already handed out completely.  The regular entry point asks them for a
// workspace they cannot provide.
//
// This variant keeps the one piece of scratch the float forward needs - the input projection
// W x + bw for all T*B rows - in a fixed array that is part of the library image itself, so it
// exists as soon as the library is loaded on a device and costs no call at run time.
#include <cuda_runtime.h>

#include <mutex>

#include "common.h"
#include "gru_forward_float.h"
#include "rxmet_b200.h"

namespace {

// 8 MiB per GPU that loads the library, held until the process exits.
constexpr size_t kScratchBytes = RXMET_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
void *g_scratchAddress[kMaxDevices] = {};
std::mutex g_setupMutex;

// The name g_scratch is only a handle on the host side; the address a kernel can use has to be
// asked for, once per device, while that device is current.
void *scratchForCurrentDevice() {
    int device = 0;
    RXMET_CUDA(cudaGetDevice(&device));
    if (device < 0 || device >= kMaxDevices)
        rxmet::fail(RXMET_ERR_UNSUPPORTED, "device ordinal %d is outside the supported range", device);
    std::lock_guard<std::mutex> lock(g_setupMutex);
    if (g_scratchAddress[device] == nullptr) {
        void *ptr = nullptr;
        const cudaError_t err = cudaGetSymbolAddress(&ptr, g_scratch);
        if (err != cudaSuccess || ptr == nullptr)
            rxmet::fail(RXMET_ERR_CUDA, "cudaGetSymbolAddress for the static scratch failed: %s",
                        cudaGetErrorString(err));
        g_scratchAddress[device] = ptr;
    }
    return g_scratchAddress[device];
}

}  // namespace

extern "C" {

size_t rxmet_static_scratch_bytes(void) { return kScratchBytes; }

int rxmet_gru_forward_fp_static(int T, int B, int I, int H, const float *W_dev, const float *R_dev,
                                const float *bw_dev, const float *br_dev, const float *x_dev, const float *h0_dev,
                                float *h_dev, float *v_dev, void *stream) {
    return rxmet::guarded([&] {
        RXMET_REQUIRE(T > 0 && B > 0 && I > 0 && H > 0, "GRU dimensions must be positive (T=%d B=%d I=%d H=%d)", T, B,
                      I, H);
        RXMET_REQUIRE(W_dev && R_dev && bw_dev && br_dev && x_dev && h_dev && v_dev,
                      "weights, input and output pointers must not be null");
        const size_t need = sizeof(float) * static_cast<size_t>(T) * B * 3 * H;
        if (need > kScratchBytes)
            rxmet::fail(RXMET_ERR_WORKSPACE,
                        "T*B*3H*4 = %zu bytes of scratch needed but the built-in scratch holds %zu; split the batch "
                        "or the sequence, or use rxmet_gru_forward_fp with your own workspace",
                        need, kScratchBytes);
        rxmet::gru::ForwardFloatCall call;
        call.T = T; call.B = B; call.I = I; call.H = H;
        call.W = W_dev; call.R = R_dev; call.bw = bw_dev; call.br = br_dev; call.x = x_dev; call.h0 = h0_dev;
        call.h = h_dev; call.v = v_dev;
        // Every element of the scratch that a step reads was written earlier in the same call, so
        // nothing has to be cleared between calls.
        rxmet::gru::forwardFloat(call, scratchForCurrentDevice(), kScratchBytes, static_cast<cudaStream_t>(stream));
    });
}

}  // extern "C"
