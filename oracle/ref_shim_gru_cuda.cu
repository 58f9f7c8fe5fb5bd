// TEST INFRASTRUCTURE - not part of the shipped library.
//
// Thin extern "C" adapter around the reference's own CUDA implementation of the QuantGRU path
// (operators/quant-gru/src/*.cu and gru_interface.cc, compiled where they lie by the Makefile beside
// this file into oracle/_ref/libgru_ref_cuda.so, linked against cuBLAS).  It gives the GPU tests a
// same-device checker for the pieces the reference has only as CUDA (the QAT backward with its
// straight-through masks, the FP32-carrier forward) and gives the benchmark the reference's own GPU
// time for the same step.  Nothing of the reference is copied here: this file converts the flat C
// structs of include/rxmet_b200.h into the reference's types and calls its functions.  All array
// arguments are device pointers; every call synchronises the device before it returns.
#include <cublas_v2.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <stdexcept>
#include <string>

#include "gru_interface.h"  // reference: quantGRUForwardInt, quantGRUForwardFP, quantGRUBackward, haste*
#include "quantize_ops_helper.h"  // reference: dev::dequantificationFPInplace
#include "scale_encoding.h"       // reference: toFixedScale
#include "ref_shim_gru_convert.h"
#include "rxmet_b200.h"

namespace {

thread_local std::string g_error;
cublasHandle_t g_handle = nullptr;

const cublasHandle_t &handle() {
    if (g_handle == nullptr) init_gru_cublas(g_handle);
    return g_handle;
}

template <class F>
int guarded(F &&f) {
    try {
        f();
        const cudaError_t err = cudaDeviceSynchronize();
        if (err != cudaSuccess) throw std::runtime_error(cudaGetErrorString(err));
        return 0;
    } catch (const std::exception &e) {
        g_error = e.what();
        return -1;
    }
}

}  // namespace

extern "C" {

const char *refcuda_last_error() { return g_error.c_str(); }

// quantGRUForwardInt (gru_interface.h:261-292): float in / float out, integer carrier, int32 code caches.
int refcuda_gru_forward_quant_int(int is_training, int T, int B, int I, int H, const float *W, const float *R,
                                  const float *bw, const float *br, const float *x, const float *h0,
                                  const rxmet_gru_quant_params *params, float *h, float *v, const rxmet_gru_masks *m,
                                  int32_t *W_q, int32_t *R_q, int32_t *bw_q, int32_t *br_q, int32_t *x_q) {
    return guarded([&] {
        const GRUQuantParams qp = refshim::toRefParams(*params);
        const rxmet_gru_masks none{};
        const rxmet_gru_masks &k = m ? *m : none;
        quantGRUForwardInt(is_training != 0, T, B, I, H, W, R, bw, br, x, h0, qp, handle(), h, v, k.x, k.h0, k.W, k.R, k.bw,
                           k.br, k.weight_ih_linear, k.weight_hh_linear, k.gate_input, k.gate_output, k.h, W_q, R_q, bw_q,
                           br_q, x_q);
    });
}

// quantGRUForwardFP (gru_interface.h:483-514): the FP32-carrier forward, float code caches.
int refcuda_gru_forward_quant_fp(int is_training, int T, int B, int I, int H, const float *W, const float *R,
                                 const float *bw, const float *br, const float *x, const float *h0,
                                 const rxmet_gru_quant_params *params, float *h, float *v, const rxmet_gru_masks *m,
                                 float *W_q, float *R_q, float *bw_q, float *br_q, float *x_q) {
    return guarded([&] {
        const GRUQuantParams qp = refshim::toRefParams(*params);
        const rxmet_gru_masks none{};
        const rxmet_gru_masks &k = m ? *m : none;
        quantGRUForwardFP(is_training != 0, T, B, I, H, W, R, bw, br, x, h0, qp, handle(), h, v, W_q, R_q, bw_q, br_q, x_q,
                          k.x, k.h0, k.W, k.R, k.bw, k.br, k.weight_ih_linear, k.weight_hh_linear, k.gate_input,
                          k.gate_output, k.h);
    });
}

// quantGRUBackward (gru_interface.h:571-595) on real-valued, TRANSPOSED operands as the reference's binding
// prepares them (W_t [3H,I], R_t [3H,H], x_t [I,T,B]; gru_interface_binding.cc:842-870).  dW / dR / dbw / dbr
// must be zeroed by the caller (the reference accumulates into them).
int refcuda_gru_backward_quant(int T, int B, int I, int H, const float *W_t, const float *R_t, const float *bw,
                               const float *br, const float *x_t, const float *dh_new, const float *h, const float *v,
                               const rxmet_gru_quant_params *params, const rxmet_gru_masks *m, float *dx, float *dW,
                               float *dR, float *dbw, float *dbr, float *dh) {
    return guarded([&] {
        const rxmet_gru_masks none{};
        const rxmet_gru_masks &k = m ? *m : none;
        if (params) {
            const GRUQuantParams qp = refshim::toRefParams(*params);
            quantGRUBackward(T, B, I, H, W_t, R_t, bw, br, x_t, dh_new, h, v, handle(), dx, dW, dR, dbw, dbr, dh, &qp, k.x,
                             k.h0, k.W, k.R, k.bw, k.br, k.weight_ih_linear, k.weight_hh_linear, k.gate_input, k.gate_output,
                             k.h);
        } else {
            hasteGRUBackward(T, B, I, H, W_t, R_t, bw, br, x_t, dh_new, h, v, handle(), dx, dW, dR, dbw, dbr, dh);
        }
    });
}

// What the reference's binding does to the saved float code caches before its backward
// (gru_interface_binding.cc:842-866): weights and biases through dequantizeGRUWeights, the input codes
// through dev::dequantificationFPInplace with the decoded x scale.  All five arrays are rewritten in place.
int refcuda_gru_dequantize_saved(int I, int H, long long x_count, float *W_q, float *R_q, float *bw_q, float *br_q,
                                 float *x_q, const rxmet_gru_quant_params *params) {
    return guarded([&] {
        const GRUQuantParams qp = refshim::toRefParams(*params);
        dequantizeGRUWeights(W_q, R_q, bw_q, br_q, static_cast<size_t>(I), static_cast<size_t>(H), qp);
        dev::dequantificationFPInplace(x_q, static_cast<size_t>(x_count), toFixedScale(qp.x_, qp.bitwidth_config_.usePOT2_),
                                       qp.x_.zero_point);
    });
}

// hasteGRUForward (gru_interface.h:410-416): the float forward.
int refcuda_gru_forward_float(int is_training, int T, int B, int I, int H, const float *W, const float *R,
                              const float *bw, const float *br, const float *x, const float *h0, float *h, float *v) {
    return guarded([&] { hasteGRUForward(is_training != 0, T, B, I, H, W, R, bw, br, x, h0, handle(), h, v); });
}

}  // extern "C"
