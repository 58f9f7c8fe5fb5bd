/*
 * rxmet_b200_lstm.h - C ABI of the QuantLSTM part of the library (single layer,
 * single direction, gate order input / forget / cell / output).
 *
 * Same conventions as rxmet_b200.h: plain pointers and POD structs, "dev" =
 * CUDA device pointer on the current device, "host" = host memory, 0 on
 * success, negative rxmet_status on failure.  Every array is dense, row-major
 * and time-major: x [T,B,I], weight_ih [4H,I], weight_hh [4H,H], biases [4H],
 * states [B,H], per-step gate tensors [T,B,4H], per-step state tensors [T,B,H].
 *
 * "q-carrier" means a float array whose values are integer quantization codes
 * (the representation of the reference's FP32 carrier, operators/quant-lstm/
 * include/quantization/float_carrier_ops.h:49-60).
 *
 * Each declaration cites the reference interface it replaces as
 * <path inside rx-met>:<line>.
 */
#ifndef RXMET_B200_LSTM_H_
#define RXMET_B200_LSTM_H_

#include "rxmet_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* The 18 quantization points, in the order of the reference's QuantOperator
 * (operators/quant-lstm/include/lstm/quant_config.h:12-31). */
enum {
    RXMET_LSTM_INPUT = 0,
    RXMET_LSTM_OUTPUT = 1,
    RXMET_LSTM_CELL_STATE = 2,
    RXMET_LSTM_WEIGHT_IH = 3,
    RXMET_LSTM_WEIGHT_HH = 4,
    RXMET_LSTM_BIAS_IH = 5,
    RXMET_LSTM_BIAS_HH = 6,
    RXMET_LSTM_WEIGHT_IH_LINEAR = 7,
    RXMET_LSTM_WEIGHT_HH_LINEAR = 8,
    RXMET_LSTM_INPUT_GATE_INPUT = 9,
    RXMET_LSTM_FORGET_GATE_INPUT = 10,
    RXMET_LSTM_CELL_GATE_INPUT = 11,
    RXMET_LSTM_OUTPUT_GATE_INPUT = 12,
    RXMET_LSTM_INPUT_GATE_OUTPUT = 13,
    RXMET_LSTM_FORGET_GATE_OUTPUT = 14,
    RXMET_LSTM_CELL_GATE_OUTPUT = 15,
    RXMET_LSTM_OUTPUT_GATE_OUTPUT = 16,
    RXMET_LSTM_CELL_TANH_OUTPUT = 17,
    RXMET_LSTM_NUM_OPS = 18
};

enum { RXMET_LSTM_PER_TENSOR = 0, RXMET_LSTM_PER_GATE = 1, RXMET_LSTM_PER_CHANNEL = 2 };
enum { RXMET_LSTM_SCALE_AFFINE = 0, RXMET_LSTM_SCALE_POT2 = 1 };

/* Grid of every point (LstmOperatorQuantConfig, quant_config.h:39-52, and
 * QuantizationType, operators/quant-lstm/include/quantization/bit_width.h:16-58).
 * Granularity other than per-tensor is only legal for the four parameter points. */
typedef struct rxmet_lstm_quant_config {
    int32_t scale_mode; /* RXMET_LSTM_SCALE_* : M+shift rescales or pure shifts */
    int32_t bitwidth[RXMET_LSTM_NUM_OPS];
    uint8_t is_unsigned[RXMET_LSTM_NUM_OPS];
    uint8_t is_symmetric[RXMET_LSTM_NUM_OPS];
    uint8_t granularity[RXMET_LSTM_NUM_OPS];
} rxmet_lstm_quant_config;

/* Finalized scales and zero points (LstmQuantParams, quant_params.h:43-50): one
 * value for every activation point; the four parameter points carry one scale per
 * output channel (4H, host arrays owned by the caller, repeated bit for bit for
 * per-tensor / per-gate granularity) and a zero point of 0. */
typedef struct rxmet_lstm_quant_params {
    rxmet_lstm_quant_config config;
    int32_t input_size;
    int32_t hidden_size;
    int32_t bias_enabled;
    float scale[RXMET_LSTM_NUM_OPS];
    int32_t zero_point[RXMET_LSTM_NUM_OPS];
    const float *weight_ih_scale; /* host [4H] */
    const float *weight_hh_scale; /* host [4H] */
    const float *bias_ih_scale;   /* host [4H], NULL without bias */
    const float *bias_hh_scale;   /* host [4H], NULL without bias */
} rxmet_lstm_quant_params;

/* Observed ranges of one or more calibration batches (LstmQuantizationRanges,
 * quant_params.h:20-28, plus LstmContributionRanges, calibration.h:24-28).
 * Parameter points are kept per channel; coarser granularities are folded when
 * the parameters are finalized.  An untouched entry holds +inf / -inf. */
typedef struct rxmet_lstm_ranges {
    float minimum[RXMET_LSTM_NUM_OPS];
    float maximum[RXMET_LSTM_NUM_OPS];
    float contribution_min[3]; /* forget*old_cell, input*cell_gate, output*tanh(cell) */
    float contribution_max[3];
    float *channel_min[4];     /* host [4H] each: weight_ih, weight_hh, bias_ih, bias_hh */
    float *channel_max[4];
} rxmet_lstm_ranges;

/* Encoded rescale (ExecutionRescale, lstm_execution_params.h:16-20): the value is
 * multiplied by `multiplier` (1 for a pure shift) and shifted right by `shift`. */
typedef struct rxmet_lstm_rescale {
    int32_t is_m_shift;
    int32_t multiplier;
    int32_t shift;
} rxmet_lstm_rescale;

/* Cell-update ratio (Q31Scale, lstm_execution_params.h:42-48). */
typedef struct rxmet_lstm_cell_scale {
    int64_t multiplier;
    double fp_mantissa;
    int32_t fp_exponent;
    int32_t uses_fp_scale;
} rxmet_lstm_cell_scale;

/* Everything derived from the quantization parameters that the kernels execute
 * with (LstmExecutionParams, lstm_execution_params.h:74-83).  The four per-channel
 * arrays are host arrays of 4H entries owned by the caller (may be NULL when the
 * caller only wants the scalar part). */
typedef struct rxmet_lstm_execution {
    rxmet_lstm_rescale ih_to_gate[4];
    rxmet_lstm_rescale hh_to_gate[4];
    rxmet_lstm_cell_scale forget_scale;
    rxmet_lstm_cell_scale input_scale;
    rxmet_lstm_rescale product_to_output;
    int32_t exact_accumulation; /* 1 when every accumulator provably stays below 2^24 */
    rxmet_lstm_rescale *ih_bias_to_accumulator;
    rxmet_lstm_rescale *ih_accumulator_to_output;
    rxmet_lstm_rescale *hh_bias_to_accumulator;
    rxmet_lstm_rescale *hh_accumulator_to_output;
} rxmet_lstm_execution;

/* The seven per-step tensors of a forward pass (LstmFloatReferenceTrace,
 * operators/quant-lstm/include/lstm/forward_float.h:18-26; for the quantized pass
 * LstmQuantizedFpCudaCheckpoints, forward_quantized_fp_cuda.h:62-77, whose masks
 * hold 1 where the value left the grid before clamping).  Any pointer may be NULL. */
typedef struct rxmet_lstm_trace {
    float *weight_ih_linear;  /* dev [T,B,4H] */
    float *weight_hh_linear;  /* dev [T,B,4H] */
    float *gate_inputs;       /* dev [T,B,4H] */
    float *gate_outputs;      /* dev [T,B,4H] */
    float *cell_states;       /* dev [T,B,H]  */
    float *cell_tanh_outputs; /* dev [T,B,H]  */
    float *hidden_outputs;    /* dev [T,B,H]  */
    uint8_t *weight_ih_linear_clamped;
    uint8_t *weight_hh_linear_clamped;
    uint8_t *gate_inputs_clamped;
    uint8_t *gate_outputs_clamped;
    uint8_t *cell_states_clamped;
    uint8_t *cell_tanh_outputs_clamped;
    uint8_t *hidden_outputs_clamped;
} rxmet_lstm_trace;

/* Quantized copies of the float masters and their clamp masks
 * (LstmQuantizedFpCudaMasters, forward_quantized_fp_cuda.h:45-60).  All NULL-able. */
typedef struct rxmet_lstm_masters {
    float *input;          /* dev [T,B,I] q-carrier */
    float *weight_ih;      /* dev [4H,I] */
    float *weight_hh;      /* dev [4H,H] */
    float *bias_ih;        /* dev [4H]   */
    float *bias_hh;        /* dev [4H]   */
    float *initial_hidden; /* dev [B,H]  */
    float *initial_cell;   /* dev [B,H]  */
    uint8_t *input_clamped;
    uint8_t *weight_ih_clamped;
    uint8_t *weight_hh_clamped;
    uint8_t *bias_ih_clamped;
    uint8_t *bias_hh_clamped;
    uint8_t *initial_hidden_clamped;
    uint8_t *initial_cell_clamped;
} rxmet_lstm_masters;

/* Clamp masks consumed by the backward pass (LstmFloatCudaBackwardMasks,
 * operators/quant-lstm/include/lstm/backward_float_cuda.h:27-43): 1 = the value was
 * clamped and passes no gradient.  Any pointer may be NULL (= nothing clamped). */
typedef struct rxmet_lstm_backward_masks {
    const uint8_t *input, *weight_ih, *weight_hh, *bias_ih, *bias_hh, *initial_hidden, *initial_cell;
    const uint8_t *weight_ih_linear, *weight_hh_linear, *gate_inputs, *gate_outputs;
    const uint8_t *cell_states, *cell_tanh_outputs, *hidden_outputs;
} rxmet_lstm_backward_masks;

/* Gradients written by the backward pass (LstmFloatCudaGradients,
 * backward_float_cuda.h:17-25).  bias pointers may be NULL. */
typedef struct rxmet_lstm_gradients {
    float *input;          /* dev [T,B,I] */
    float *weight_ih;      /* dev [4H,I]  */
    float *weight_hh;      /* dev [4H,H]  */
    float *bias_ih;        /* dev [4H]    */
    float *bias_hh;        /* dev [4H]    */
    float *initial_hidden; /* dev [B,H]   */
    float *initial_cell;   /* dev [B,H]   */
} rxmet_lstm_gradients;

/* ---- host-side parameter logic ------------------------------------------- */

/* Default grid: 8-bit everywhere, symmetric signed parameters per channel,
 * asymmetric activations, unsigned sigmoid outputs. */
RXMET_API int rxmet_lstm_default_config(rxmet_lstm_quant_config *config);

/* Sets every range to "nothing observed" (LstmQuantizationRanges::reset,
 * operators/quant-lstm/src/lstm/quant_params.cc:118-131).  channel arrays hold 4H. */
RXMET_API int rxmet_lstm_ranges_reset(rxmet_lstm_ranges *ranges, int hidden_size);

/* Ranges -> scales and zero points (finalizeQuantParams, quant_params.cc:222-287;
 * calibrateMinMax / convertScaleToPot2CoverRange, operators/quant-lstm/src/
 * quantization/scale_encoding.cc:39-91,143-185).  Writes the four per-channel
 * scale arrays (host [4H], caller-owned) that `params` is then made to point to. */
RXMET_API int rxmet_lstm_params_from_ranges(const rxmet_lstm_quant_config *config, const rxmet_lstm_ranges *ranges,
                                            int input_size, int hidden_size, int bias_enabled,
                                            float *weight_ih_scale, float *weight_hh_scale, float *bias_ih_scale,
                                            float *bias_hh_scale, rxmet_lstm_quant_params *params);

/* Parameters -> executable encodings (deriveLstmExecutionParams,
 * operators/quant-lstm/src/lstm/lstm_execution_params.cc:188-326).  With
 * require_exact_accumulation != 0 a configuration whose accumulators may exceed
 * the exactly representable integer range of float is rejected. */
RXMET_API int rxmet_lstm_derive_execution(const rxmet_lstm_quant_params *params, int require_exact_accumulation,
                                          rxmet_lstm_execution *execution);

/* ---- device entry points --------------------------------------------------- */

/* Workspace bytes of: op 0 float / calibration forward, 1 quantized forward,
 * 2 backward, 3 histogram calibration forward (lstmQuantizedFpCudaWorkspaceBreakdown, forward_quantized_fp_cuda.h:133-135;
 * cudaBackwardWorkspaceElementCount, backward_float_cuda.h:45-46). */
RXMET_API size_t rxmet_lstm_workspace_bytes(int op, int T, int B, int I, int H);

/* Float forward (lstmForwardFloatCuda, operators/quant-lstm/include/lstm/
 * forward_float_cuda.h:12-31; binding lstm_forward / lstm_forward_training,
 * operators/quant-lstm/pytorch/lib/lstm_interface_binding.cc:918-926).
 * bias_ih/bias_hh and h0/c0 are given in pairs or both NULL. */
RXMET_API int rxmet_lstm_forward_float(int T, int B, int I, int H, const float *weight_ih, const float *weight_hh,
                                       const float *bias_ih, const float *bias_hh, const float *x, const float *h0,
                                       const float *c0, float *output, float *final_hidden, float *final_cell,
                                       const rxmet_lstm_trace *trace, void *workspace, size_t workspace_bytes,
                                       void *stream);

/* Number of floats of the packed calibration statistics for hidden size H:
 * [minima | maxima], each half = 18 point slots + 3 contribution slots +
 * 4 x 4H per-channel slots (weight_ih, weight_hh, bias_ih, bias_hh). */
RXMET_API size_t rxmet_lstm_stats_floats(int H);

/* Float forward that also reduces the ranges of all 18 points and the three
 * product contributions on the device (lstmForwardCalibrateCuda,
 * operators/quant-lstm/include/lstm/calibration_cuda.h:10-16; collector semantics
 * operators/quant-lstm/src/lstm/calibration.cc:128-232).  stats_dev is overwritten. */
RXMET_API int rxmet_lstm_forward_calibrate_stats(int T, int B, int I, int H, const float *weight_ih,
                                                 const float *weight_hh, const float *bias_ih, const float *bias_hh,
                                                 const float *x, const float *h0, const float *c0, float *output,
                                                 float *final_hidden, float *final_cell, float *stats_dev,
                                                 void *workspace, size_t workspace_bytes, void *stream);

/* Merges host copies of packed statistics into `ranges`
 * (LstmCalibrationCollector::merge, calibration.cc:233-276). */
RXMET_API int rxmet_lstm_ranges_fold_stats(rxmet_lstm_ranges *ranges, const float *stats_host, int H, int bias_enabled);

/* ---- histogram calibration (SQNR / percentile) ------------------------------ */

/* One collector (quantization::Histogram / HistogramCollector, operators/quant-lstm/
 * include/quantization/histogram.h:9-37): double counts over [minimum, maximum].
 * counts is a host array of num_bins doubles owned by the caller; an empty
 * collector has total_count 0. */
typedef struct rxmet_lstm_histogram {
    double *counts;
    int32_t num_bins;
    float minimum, maximum;
    uint64_t total_count;
} rxmet_lstm_histogram;

/* Collectors of a calibration session (LstmCalibrationCollector::histograms_,
 * operators/quant-lstm/include/lstm/calibration.h:113-114): one per activation
 * point; for the four parameter points the collectors of the configured
 * granularity are used: point[op] (per tensor), gate[slot] (per gate) or
 * channel[slot][4H] (per channel), slot = op - RXMET_LSTM_WEIGHT_IH. */
typedef struct rxmet_lstm_histograms {
    int32_t hidden_size;
    int32_t num_bins;
    rxmet_lstm_histogram point[RXMET_LSTM_NUM_OPS];
    rxmet_lstm_histogram gate[4][4];
    rxmet_lstm_histogram *channel[4];
} rxmet_lstm_histograms;

/* Adds host data to a collector (HistogramCollector::collect,
 * operators/quant-lstm/src/quantization/histogram.cc:129-161): the batch is binned
 * over its own finite range and merged by re-binning bin centres (:163-183). */
RXMET_API int rxmet_lstm_histogram_collect_host(rxmet_lstm_histogram *hist, const float *data_host, uint64_t count);
RXMET_API int rxmet_lstm_histogram_merge(rxmet_lstm_histogram *hist, const rxmet_lstm_histogram *other);
/* Range chosen from a collector (calibrateHistogramRange, histogram.cc:186-254):
 * method 0 = SQNR search, 1 = percentile. */
RXMET_API int rxmet_lstm_histogram_range(const rxmet_lstm_histogram *hist, int bitwidth, int is_unsigned,
                                         int is_symmetric, int method, float percentile, float *range_min,
                                         float *range_max);

/* Float forward of one calibration batch that feeds ranges AND histograms
 * (lstmForwardCalibrateCuda with a histogram-collecting session,
 * operators/quant-lstm/include/lstm/calibration_cuda.h:10-16; collection order
 * operators/quant-lstm/src/lstm/calibration.cc:128-232,233-276).  Min/max and the
 * binning run on the device, merges on the host; synchronises the stream.
 * Workspace: rxmet_lstm_workspace_bytes(3, ...). */
RXMET_API int rxmet_lstm_forward_calibrate_hist(int T, int B, int I, int H, const float *weight_ih,
                                                const float *weight_hh, const float *bias_ih, const float *bias_hh,
                                                const float *x, const float *h0, const float *c0, float *output,
                                                float *final_hidden, float *final_cell,
                                                const rxmet_lstm_quant_config *config, rxmet_lstm_ranges *ranges,
                                                rxmet_lstm_histograms *hists, void *workspace, size_t workspace_bytes,
                                                void *stream);

/* The same with the batch sharded over ranks (see rxmet_exchange in rxmet_b200.h): the range
 * statistics, the finite extremes and counts of every observed tensor and the bin counts are
 * reduced through the hook, so that every rank merges the batch histogram one process would build
 * on the concatenated batch (per-batch collection: histogram.cc:145-193).  exchange == NULL is
 * rxmet_lstm_forward_calibrate_hist. */
RXMET_API int rxmet_lstm_forward_calibrate_hist_dp(int T, int B, int I, int H, const float *weight_ih,
                                                   const float *weight_hh, const float *bias_ih, const float *bias_hh,
                                                   const float *x, const float *h0, const float *c0, float *output,
                                                   float *final_hidden, float *final_cell,
                                                   const rxmet_lstm_quant_config *config, rxmet_lstm_ranges *ranges,
                                                   rxmet_lstm_histograms *hists, void *workspace, size_t workspace_bytes,
                                                   void *stream, const rxmet_exchange *exchange);

/* One collector, data on the host, exchange by the caller: the range a batch with the given
 * global finite extremes is binned over, this rank's counts over it (added to counts[num_bins]
 * and *finite), and the merge of the summed counts (HistogramCollector::collect split in three,
 * histogram.cc:129-161). */
RXMET_API int rxmet_lstm_histogram_batch_range(float batch_min, float batch_max, float *range_min, float *range_max);
RXMET_API int rxmet_lstm_histogram_count_host(float range_min, float range_max, int num_bins, const float *data_host,
                                              uint64_t count, uint64_t *counts, uint64_t *finite);
RXMET_API int rxmet_lstm_histogram_merge_counts(rxmet_lstm_histogram *hist, const uint64_t *counts, float range_min,
                                                float range_max, uint64_t finite);

/* Ranges + histograms -> parameters (LstmCalibrationSession::finalize with
 * method sqnr / percentile, calibration.cc:312-346): every non-bias group takes
 * the range calibrateHistogramRange selects, biases keep their observed range. */
RXMET_API int rxmet_lstm_params_from_histograms(const rxmet_lstm_quant_config *config, const rxmet_lstm_ranges *ranges,
                                                const rxmet_lstm_histograms *hists, int method, float percentile,
                                                int input_size, int hidden_size, int bias_enabled,
                                                float *weight_ih_scale, float *weight_hh_scale, float *bias_ih_scale,
                                                float *bias_hh_scale, rxmet_lstm_quant_params *params);

/* Quantized forward on the FP32 q-carrier (lstmForwardQuantizedFpCuda,
 * forward_quantized_fp_cuda.h:137-169; binding lstm_forward_quantized,
 * lstm_interface_binding.cc:940-946).  Quantizes the float masters, runs all T steps
 * and writes dequantized output [T,B,H], final_hidden and final_cell [B,H].
 * `checkpoints` (q-carrier values + clamp masks) and `masters` may be NULL. */
RXMET_API int rxmet_lstm_forward_quantized(int T, int B, int I, int H, const float *weight_ih, const float *weight_hh,
                                           const float *bias_ih, const float *bias_hh, const float *x, const float *h0,
                                           const float *c0, const rxmet_lstm_quant_params *params,
                                           int require_exact_accumulation, float *output, float *final_hidden,
                                           float *final_cell, const rxmet_lstm_trace *checkpoints,
                                           const rxmet_lstm_masters *masters, void *workspace, size_t workspace_bytes,
                                           void *stream);

/* Float backward through time with optional clamp masks (lstmBackwardFloatCuda,
 * backward_float_cuda.h:48-60; binding lstm_backward_float, lstm_interface_binding.cc:927-934).
 * The trace tensors are real-valued (gate_outputs, cell_states, cell_tanh_outputs,
 * hidden_outputs of the forward). */
RXMET_API int rxmet_lstm_backward_float(int T, int B, int I, int H, const float *weight_ih, const float *weight_hh,
                                        const float *x, const float *h0, const float *c0, const float *gate_outputs,
                                        const float *cell_states, const float *cell_tanh_outputs,
                                        const float *hidden_outputs, const float *grad_output,
                                        const float *grad_final_hidden, const float *grad_final_cell,
                                        const rxmet_lstm_backward_masks *masks, const rxmet_lstm_gradients *gradients,
                                        void *workspace, size_t workspace_bytes, void *stream);

/* QAT backward (binding lstm_backward_qat, lstm_interface_binding.cc:437-480,935-939):
 * dequantizes the q-carrier masters and checkpoints saved by the quantized forward
 * and runs the masked float backward on them. */
RXMET_API int rxmet_lstm_backward_qat(int T, int B, int I, int H, const rxmet_lstm_quant_params *params,
                                      const float *q_weight_ih, const float *q_weight_hh, const float *q_x,
                                      const float *q_h0, const float *q_c0, const float *q_gate_outputs,
                                      const float *q_cell_states, const float *q_cell_tanh_outputs,
                                      const float *q_hidden_outputs, const float *grad_output,
                                      const float *grad_final_hidden, const float *grad_final_cell,
                                      const rxmet_lstm_backward_masks *masks, const rxmet_lstm_gradients *gradients,
                                      void *workspace, size_t workspace_bytes, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* RXMET_B200_LSTM_H_ */
