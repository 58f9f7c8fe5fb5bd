/*
 * rxmet_b200.h - C ABI of the B200-native quantized recurrent hot path.
 *
 * Every entry point takes plain pointers, sizes and POD structs; no C++ or
 * torch types cross this boundary.  "dev" pointers are CUDA device pointers on
 * the current device, "host" pointers are ordinary host memory.  All tensors
 * are dense and contiguous in the layouts named per argument.  All entry
 * points return 0 on success and a negative rxmet_status on failure;
 * rxmet_last_error() then holds a message for the calling thread.
 *
 * Each declaration cites the reference interface it replaces as
 * <path inside rx-met>:<line>.
 */
#ifndef RXMET_B200_H_
#define RXMET_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define RXMET_API
#else
#define RXMET_API __attribute__((visibility("default")))
#endif

typedef enum rxmet_status {
    RXMET_OK = 0,
    RXMET_ERR_INVALID_ARGUMENT = -1, /* bad size, null pointer, bad config      */
    RXMET_ERR_CUDA = -2,             /* a CUDA runtime call or launch failed    */
    RXMET_ERR_WORKSPACE = -3,        /* caller's workspace is too small         */
    RXMET_ERR_UNSUPPORTED = -4,      /* shape or bit-width outside this build   */
    RXMET_ERR_DEVICE_TIMEOUT = -5    /* a bounded device-side wait ran out      */
} rxmet_status;

/* Message of the last failure on the calling thread ("" if none). */
RXMET_API const char *rxmet_last_error(void);
/* Library version string. */
RXMET_API const char *rxmet_version(void);
/* Number of kernels this library has launched in this process so far. */
RXMET_API uint64_t rxmet_kernel_launch_count(void);

/* How many recurrent passes the caller keeps in flight at once on one GPU (the two directions of a
 * bidirectional layer on two streams: 2).  The recurrent kernels of wide layers, which hold one CTA per
 * SM, size their batch tiles so that the CTAs of all those launches are resident together instead of
 * queueing behind each other.  Default 1; values below 1 are taken as 1.  Results do not depend on
 * it.  No counterpart in the reference. */
RXMET_API int rxmet_set_concurrent_passes(int passes);

/* Per-kernel timing, off by default.  While enabled every kernel launch of the
 * library is bracketed by CUDA events on its stream;
 * rxmet_get_kernel_timing waits for the recorded events and returns the summed
 * duration and the launch count of the kernel with that name since the last
 * reset.  Plays the role of the reference's caller-supplied timing events
 * (operators/quant-lstm/include/lstm/forward_quantized_fp_cuda.h:119-131). */
RXMET_API int rxmet_set_kernel_timing(int enabled);
RXMET_API int rxmet_get_kernel_timing(const char *kernel_name, double *total_ms, long long *launches);
RXMET_API int rxmet_reset_kernel_timing(void);

/* Host -> device staging by a kernel instead of the copy engine: `ctas` CTAs (default 16 when
 * <= 0) read the page-locked, device-mapped host buffer over PCIe and write dst_dev with
 * evict-first stores.  For input staging on a side stream next to a training step, where a
 * copy-engine transfer of the same bytes slows the step's latency-bound kernels more.
 * src_host must be page-locked (cudaHostAlloc / cudaHostRegister / torch pin_memory); both
 * pointers 16-byte aligned. */
RXMET_API int rxmet_stage_from_pinned_host(void *dst_dev, const void *src_host, size_t bytes, int ctas, void *stream);

/* Self-test of the bounded device-side wait that the tcgen05 kernels use: launches one CTA that
 * polls an mbarrier nothing ever arrives on, with the kernels' own poll loop and limit.  The
 * kernel gives up when the limit runs out, sets status_dev[0] to 1 and returns; the call waits
 * for it and returns RXMET_ERR_DEVICE_TIMEOUT, the context stays usable.  status_dev: two ints of
 * device memory (status, polls made); polls_out (optional, host) receives the number of polls. */
RXMET_API int rxmet_selftest_bounded_wait(int *status_dev, unsigned int *polls_out, void *stream);

/* ------------------------------------------------------------------------ */
/* QuantGRU: configuration and encodings                                     */
/* ------------------------------------------------------------------------ */

/* The 17 quantization points of one GRU direction, in the member order of the
 * reference's OperatorQuantConfig (operators/quant-gru/include/
 * quantize_bitwidth_config.h:54-83). */
enum {
    RXMET_GRU_X = 0,
    RXMET_GRU_H = 1,
    RXMET_GRU_W = 2,
    RXMET_GRU_R = 3,
    RXMET_GRU_BW = 4,
    RXMET_GRU_BR = 5,
    RXMET_GRU_WEIGHT_IH_LINEAR = 6,
    RXMET_GRU_WEIGHT_HH_LINEAR = 7,
    RXMET_GRU_UPDATE_GATE_INPUT = 8,
    RXMET_GRU_UPDATE_GATE_OUTPUT = 9,
    RXMET_GRU_RESET_GATE_INPUT = 10,
    RXMET_GRU_RESET_GATE_OUTPUT = 11,
    RXMET_GRU_NEW_GATE_INPUT = 12,
    RXMET_GRU_NEW_GATE_OUTPUT = 13,
    RXMET_GRU_MUL_RESET_HIDDEN = 14,
    RXMET_GRU_MUL_OLD_CONTRIBUTION = 15,
    RXMET_GRU_MUL_NEW_CONTRIBUTION = 16,
    RXMET_GRU_NUM_OPS = 17
};

/* Granularity of the W / R / bw / br scales (quantize_bitwidth_config.h:56-60). */
enum { RXMET_PER_TENSOR = 0, RXMET_PER_GATE = 1, RXMET_PER_CHANNEL = 2 };
/* Power-of-two rounding policy (operators/quant-gru/include/pot_scale_encode.h:37-41). */
enum { RXMET_POT_ROUND = 0, RXMET_POT_COVER_RANGE = 1, RXMET_POT_FLOOR = 2 };

/* Mirror of OperatorQuantConfig (quantize_bitwidth_config.h:54-122): bit-width
 * 1..32, signedness and symmetry per quantization point, weight granularities
 * and the power-of-two switch. */
typedef struct rxmet_gru_quant_config {
    int8_t bits[RXMET_GRU_NUM_OPS];
    uint8_t is_unsigned[RXMET_GRU_NUM_OPS];
    uint8_t symmetric[RXMET_GRU_NUM_OPS];
    int32_t W_granularity, R_granularity, bw_granularity, br_granularity;
    uint8_t use_pot2;
    int8_t pot_scale_method;
    float pot_scale_tolerance;
} rxmet_gru_quant_config;

/* Fills *cfg with the reference defaults: 8 bit everywhere, update/reset gate
 * outputs unsigned, everything symmetric, per-channel weights, affine
 * (M * 2^-shift) rescale, CoverRange with tolerance 0.02. */
RXMET_API void rxmet_gru_default_config(rxmet_gru_quant_config *cfg);

/* Mirror of GRUQuantizationRanges (operators/quant-gru/include/
 * gru_quantization_ranges.h:20-69).  min/max are indexed by quantization
 * point; the W/R/bw/br entries of the scalar arrays are unused, their
 * per-channel ranges live in the eight host arrays of 3*hidden floats. */
typedef struct rxmet_gru_ranges {
    int32_t hidden;
    float min[RXMET_GRU_NUM_OPS];
    float max[RXMET_GRU_NUM_OPS];
    float *min_W, *max_W, *min_R, *max_R, *min_bw, *max_bw, *min_br, *max_br;
} rxmet_gru_ranges;

/* Sets every range to (FLT_MAX, -FLT_MAX) like GRUQuantizationRanges::reset
 * (gru_quantization_ranges.h:74-118).  The per-channel arrays must be set. */
RXMET_API int rxmet_gru_ranges_reset(rxmet_gru_ranges *ranges);

/* Mirror of the Python-visible GRUQuantParams (operators/quant-gru/pytorch/lib/
 * gru_interface_binding.cc:145-193): one (scale, zero point) per point, the
 * four weight/bias scale arrays always expanded to 3*hidden (zero point 0),
 * and the configuration.  LUT tables and rescale multipliers are derived
 * inside the library from these values, as the reference's to_cpp() does
 * (gru_interface_binding.cc:1261-1316). */
typedef struct rxmet_gru_quant_params {
    int32_t hidden;
    float scale[RXMET_GRU_NUM_OPS];
    int32_t zero_point[RXMET_GRU_NUM_OPS];
    float *scale_W, *scale_R, *scale_bw, *scale_br; /* host, 3*hidden each */
    rxmet_gru_quant_config config;
} rxmet_gru_quant_params;

/* Ranges -> encodings.  Replaces calculateGRUQuantitativeParameters
 * (operators/quant-gru/src/gru_host.cc:13-125).  out->scale_* must point to
 * 3*hidden floats each.  Host only. */
RXMET_API int rxmet_gru_params_from_ranges(const rxmet_gru_ranges *ranges,
                                           const rxmet_gru_quant_config *cfg,
                                           rxmet_gru_quant_params *out);

/* One segment of the 16-segment piecewise-linear activation table
 * (operators/quant-gru/include/quantize_lut_types.h:32-37). */
typedef struct rxmet_lut_segment {
    int32_t q_b;
    int32_t n_bx_total;
    int32_t term_c;
    int32_t threshold;
} rxmet_lut_segment;

/* Writes the three activation tables (update sigmoid, reset sigmoid, new-gate
 * tanh; 16 segments each) derived from params.  Replaces
 * generate_piecewise_linear_lut_to_params (operators/quant-gru/src/
 * quantize_lut.cc:17-48).  Host only; exposed so that table parity can be
 * checked on its own. */
RXMET_API int rxmet_gru_build_luts(const rxmet_gru_quant_params *params,
                                   rxmet_lut_segment out_segments[3][16]);

/* Effective scale the integer core uses for a stored scale: M*2^-shift with a
 * 16-bit M (affine) or the power of two itself.  Replaces
 * decode_effective_scale (gru_interface_binding.cc:1322-1327). */
RXMET_API int rxmet_gru_decode_effective_scale(float scale, int use_pot2, float *out);

/* ------------------------------------------------------------------------ */
/* QuantGRU: device entry points                                             */
/* ------------------------------------------------------------------------ */

/* Weights arrive as the reference's Python hands them over: gate order z,r,n
 * and transposed, W [I,3H], R [H,3H], bw/br [3H] (operators/quant-gru/pytorch/
 * quant_gru.py:714-759).  x is time-major [T,B,I]; h is [T+1,B,H] with h[0]
 * the initial state; v is [T,B,4H] = (z, r, n, (R h + br)_n). */

/* Bytes of device scratch the entry point named by `op` needs for these
 * sizes.  op: 0 forward_fp / forward_calibrate, 1 forward_quant,
 * 2 backward_quant / backward_fp, 3 forward_calibrate with histograms. */
RXMET_API size_t rxmet_gru_workspace_bytes(int op, int T, int B, int I, int H);

/* Float GRU forward.  Replaces forward_fp -> gru::ForwardPass<float>::Run
 * (gru_interface_binding.cc:656-698, operators/quant-gru/src/
 * gru_forward_gpu.cu:359-431).  h0_dev may be NULL (zero state). */
RXMET_API int rxmet_gru_forward_fp(int T, int B, int I, int H,
                                   const float *W_dev, const float *R_dev,
                                   const float *bw_dev, const float *br_dev,
                                   const float *x_dev, const float *h0_dev,
                                   float *h_dev, float *v_dev,
                                   void *workspace_dev, size_t workspace_bytes,
                                   void *stream);

/* Float forward that also folds the min/max of the 13 activation points and
 * of W/R/bw/br per channel into *ranges (host).  Replaces forward_calibrate
 * with calib_method "minmax" -> forwardWithCalibrationGPU /
 * forwardWithCalibrationCPU (gru_interface_binding.cc:710-780, operators/
 * quant-gru/src/gru_interface.cc:936-1024, src/gru_forward_cpu.cc:58-151).
 * Only finite values are observed; h[0] is not observed.  Synchronises the
 * stream before returning because the result lands in host memory. */
RXMET_API int rxmet_gru_forward_calibrate_minmax(int T, int B, int I, int H,
                                                 const float *W_dev, const float *R_dev,
                                                 const float *bw_dev, const float *br_dev,
                                                 const float *x_dev, const float *h0_dev,
                                                 float *h_dev, float *v_dev,
                                                 rxmet_gru_ranges *ranges,
                                                 void *workspace_dev, size_t workspace_bytes,
                                                 void *stream);

/* Device-side half of the above for data-parallel calibration: leaves the
 * packed statistics (see rxmet_gru_stats_floats) in stats_dev as
 * [mins..., maxs...] without touching the host, so that ranks can all-reduce
 * them (MIN on the first half, MAX on the second) before folding. */
RXMET_API size_t rxmet_gru_stats_floats(int H);
RXMET_API int rxmet_gru_forward_calibrate_stats(int T, int B, int I, int H,
                                                const float *W_dev, const float *R_dev,
                                                const float *bw_dev, const float *br_dev,
                                                const float *x_dev, const float *h0_dev,
                                                float *h_dev, float *v_dev, float *stats_dev,
                                                void *workspace_dev, size_t workspace_bytes,
                                                void *stream);
/* Folds packed statistics (host copy of stats_dev) into *ranges. */
RXMET_API int rxmet_gru_ranges_fold_stats(rxmet_gru_ranges *ranges, const float *stats_host);

/* ---- histogram calibration (SQNR / percentile) ---------------------------- */

/* One histogram collector (HistogramCollector + Histogram,
 * operators/quant-gru/include/histogram_collector.h:44-164,166-420): float counts
 * over [min_val, max_val], the observed extremes and the growth limits.  counts
 * is a host array of num_bins floats owned by the caller. */
typedef struct rxmet_histogram {
    float *counts;
    int32_t num_bins;
    float min_val, max_val;
    float observed_min, observed_max;
    int64_t total_count;
    int32_t range_limit_set;
    float range_limit_min, range_limit_max;
} rxmet_histogram;

/* Empties a collector (HistogramCollector::reset, histogram_collector.h:283-288).
 * counts and num_bins must be set. */
RXMET_API int rxmet_histogram_reset(rxmet_histogram *hist);
/* Adds host data (HistogramCollector::collect, histogram_collector.h:185-247):
 * first batch fixes the range, later batches extend it and redistribute the
 * existing counts (AIMET merge_stats rule). */
RXMET_API int rxmet_histogram_collect_host(rxmet_histogram *hist, const float *data_host, uint64_t count);
/* Same for a device tensor of `rows` rows of `cols` contiguous floats, rows
 * `row_stride` floats apart: min/max and the binning run on the device, the merge
 * on the host.  Synchronises the stream.  Workspace: rxmet_histogram_workspace_bytes. */
RXMET_API size_t rxmet_histogram_workspace_bytes(int num_bins);
RXMET_API int rxmet_histogram_collect_dev(rxmet_histogram *hist, const float *data_dev, uint64_t rows, uint64_t cols,
                                          uint64_t row_stride, void *workspace_dev, size_t workspace_bytes,
                                          void *stream);
/* Merges another collector's histogram (HistogramCollector::merge, :248-282). */
RXMET_API int rxmet_histogram_merge(rxmet_histogram *hist, const rxmet_histogram *other);
/* Continuous scale and covered range from a histogram
 * (calibrateContinuousScaleFromHistogram, operators/quant-gru/include/
 * pot_sqnr_calibrator.h:340-358: SQNR search :118-338 or percentile :19-107). */
RXMET_API int rxmet_histogram_calibrate(const rxmet_histogram *hist, int bits, int is_unsigned, int symmetric,
                                        int use_percentile, float percentile, float *scale, float *range_min,
                                        float *range_max);

/* ---- data-parallel calibration --------------------------------------------- */

/* A batch sharded over ranks must give the collectors what one process would see on the
 * concatenated batch (the collectors' range growth and binning are defined per batch,
 * operators/quant-gru/include/histogram_collector.h:185-292).  That takes two exchanges inside
 * one calibration batch: the finite extremes (MIN / MAX) before anything is binned, so that every
 * rank bins on the same range, and the bin counts (SUM) before they are committed.  The library
 * calls the hook below for each exchange; the hook reduces `count` elements at `data_dev` across
 * the ranks IN PLACE, ordered on `stream`, and returns 0 (NCCL all-reduce in the Python layer).
 * world_size scales what every rank observes identically (element totals). */
enum { RXMET_REDUCE_MIN_F32 = 0, RXMET_REDUCE_MAX_F32 = 1, RXMET_REDUCE_SUM_U32 = 2, RXMET_REDUCE_SUM_U64 = 3 };
typedef int (*rxmet_reduce_fn)(int kind, void *data_dev, uint64_t count, void *stream, void *user);
typedef struct rxmet_exchange {
    rxmet_reduce_fn reduce;
    void *user;
    int32_t world_size;
} rxmet_exchange;

/* The same three steps for one collector with the data on the host (the exchange is the
 * caller's): plan from the batch's global extremes, count this rank's elements into
 * counts[num_bins] (added to what is there), commit the summed counts with the global element
 * total.  plan + count + commit on one rank equals rxmet_histogram_collect_host. */
typedef struct rxmet_histogram_plan {
    int32_t mode; /* 0 first batch, 1 range unchanged, 2 range extended */
    float lo, hi, inv_bin_width;
    float new_min, new_max;
    float data_min, data_max;
    float limit_min, limit_max;
} rxmet_histogram_plan;
RXMET_API int rxmet_histogram_plan_batch(const rxmet_histogram *hist, float batch_min, float batch_max,
                                         rxmet_histogram_plan *plan);
RXMET_API int rxmet_histogram_count_host(const rxmet_histogram_plan *plan, int num_bins, const float *data_host,
                                         uint64_t count, uint32_t *counts);
RXMET_API int rxmet_histogram_commit_counts(rxmet_histogram *hist, const rxmet_histogram_plan *plan,
                                            const uint32_t *counts, uint64_t total_elements);

/* All collectors of one GRU direction (GRUHistogramCollectors,
 * histogram_collector.h:609-720): one per activation point (the W, R, bw, br
 * entries of `point` are the per-tensor collectors), 3*hidden per-channel
 * collectors and three per-gate collectors for each of W, R, bw, br. */
typedef struct rxmet_gru_histograms {
    int32_t hidden;
    int32_t num_bins;
    rxmet_histogram point[RXMET_GRU_NUM_OPS];
    rxmet_histogram *channel[4]; /* host arrays of 3*hidden collectors: W, R, bw, br */
    rxmet_histogram gate[4][3];
} rxmet_gru_histograms;

/* Float forward that feeds every collector (forwardWithCalibrationGPU with
 * calib_method sqnr / percentile, operators/quant-gru/src/gru_interface.cc:936-1024;
 * what is observed: src/gru_forward_cpu.cc:118-151).  Workspace:
 * rxmet_gru_workspace_bytes(3, ...).  Synchronises the stream. */
RXMET_API int rxmet_gru_forward_calibrate_hist(int T, int B, int I, int H, const float *W_dev, const float *R_dev,
                                               const float *bw_dev, const float *br_dev, const float *x_dev,
                                               const float *h0_dev, float *h_dev, float *v_dev,
                                               const rxmet_gru_quant_config *config, rxmet_gru_histograms *hists,
                                               void *workspace_dev, size_t workspace_bytes, void *stream);

/* The same with the batch sharded over ranks (exchange != NULL): statistics and bin counts of
 * the 13 activation points are reduced through the hook; weights and biases are identical on
 * every rank and are observed locally. */
RXMET_API int rxmet_gru_forward_calibrate_hist_dp(int T, int B, int I, int H, const float *W_dev, const float *R_dev,
                                                  const float *bw_dev, const float *br_dev, const float *x_dev,
                                                  const float *h0_dev, float *h_dev, float *v_dev,
                                                  const rxmet_gru_quant_config *config, rxmet_gru_histograms *hists,
                                                  void *workspace_dev, size_t workspace_bytes, void *stream,
                                                  const rxmet_exchange *exchange);

/* Histograms -> encodings (calculateGRUQuantitativeParametersFromHistograms,
 * operators/quant-gru/src/gru_host.cc:254-335).  The four scale arrays of *params
 * must point to 3*hidden floats each. */
RXMET_API int rxmet_gru_params_from_histograms(const rxmet_gru_histograms *hists, const rxmet_gru_quant_config *config,
                                               int use_percentile, float percentile, rxmet_gru_quant_params *params);

/* The 11 clamp masks of a training forward (1 = kept, 0 = clamped;
 * operators/quant-gru/include/quantize_ops_helper.h:272-276), in the order
 * the reference returns them (gru_interface_binding.cc:310-448).  Each is a
 * device uint8 array; all NULL for an inference forward. */
typedef struct rxmet_gru_masks {
    uint8_t *x;                /* [T,B,I]  */
    uint8_t *h0;               /* [B,H], NULL when no h0 is given */
    uint8_t *W;                /* [I,3H]   */
    uint8_t *R;                /* [H,3H]   */
    uint8_t *bw;               /* [3H]     */
    uint8_t *br;               /* [3H]     */
    uint8_t *weight_ih_linear; /* [T,B,3H] */
    uint8_t *weight_hh_linear; /* [T,B,3H] */
    uint8_t *gate_input;       /* [T,B,3H] */
    uint8_t *gate_output;      /* [T,B,3H] */
    uint8_t *h;                /* [T,B,H]  */
} rxmet_gru_masks;

/* Quantized GRU forward with the integer carrier: int32-exact accumulation,
 * M*2^-shift (or power-of-two) rescale with round-half-even shifts and the
 * 16-segment integer activation tables.  Replaces forward_quant_int_storage /
 * forward_quant_float_storage -> quantGRUForwardInt -> ForwardPassQuant::Run
 * (gru_interface_binding.cc:463-597, operators/quant-gru/src/
 * gru_interface.cc:430-556, src/gru_forward_gpu_quant.cu:789-841) and the CPU
 * core ForwardPassQuantCPU::Run (src/gru_forward_cpu_quant.cc:313-348).
 * h_dev / v_dev receive the dequantized values; the optional *_q_dev outputs
 * receive the integer codes (int32, NULL to skip): W_q [I,3H], R_q [H,3H],
 * bw_q/br_q [3H], x_q [T,B,I], h_q [T+1,B,H], v_q [T,B,4H]. */
RXMET_API int rxmet_gru_forward_quant(int is_training, int T, int B, int I, int H,
                                      const float *W_dev, const float *R_dev,
                                      const float *bw_dev, const float *br_dev,
                                      const float *x_dev, const float *h0_dev,
                                      const rxmet_gru_quant_params *params,
                                      float *h_dev, float *v_dev,
                                      int32_t *W_q_dev, int32_t *R_q_dev,
                                      int32_t *bw_q_dev, int32_t *br_q_dev,
                                      int32_t *x_q_dev, int32_t *h_q_dev, int32_t *v_q_dev,
                                      const rxmet_gru_masks *masks,
                                      void *workspace_dev, size_t workspace_bytes,
                                      void *stream);

/* Integer-in / integer-out inference: x_q [T,B,I] and h0_q [B,H] (or NULL)
 * are already codes on the x / h grids; h_q_dev receives [T+1,B,H] codes.
 * Replaces forward_quantized_int_io -> quantGRUForwardIntIO
 * (gru_interface_binding.cc:600-647, gru_interface.cc:566-618). */
RXMET_API int rxmet_gru_forward_quant_int_io(int T, int B, int I, int H,
                                             const float *W_dev, const float *R_dev,
                                             const float *bw_dev, const float *br_dev,
                                             const int32_t *x_q_dev, const int32_t *h0_q_dev,
                                             const rxmet_gru_quant_params *params,
                                             int32_t *h_q_dev,
                                             void *workspace_dev, size_t workspace_bytes,
                                             void *stream);

/* QAT backward: BPTT on the dequantized saved values with straight-through
 * clamp masks.  Replaces backward_quant_int_storage /
 * backward_quant_float_storage -> quantGRUBackward -> BackwardPassQuant::Run
 * (gru_interface_binding.cc:790-969, gru_interface.cc:112-153, operators/
 * quant-gru/src/gru_backward_gpu_quant.cu:93-493).  W_q..x_q are the int32
 * codes saved by the forward and are left untouched; h [T+1,B,H] and
 * v [T,B,4H] are the dequantized forward outputs; dh_new is [T+1,B,H].
 * Outputs: dx [T,B,I], dW [I,3H], dR [H,3H], dbw/dbr [3H], dh0 [B,H].  Bias
 * gradients are reduced in a fixed order (no atomics), so the result is
 * reproducible run to run.  masks may be NULL (no clamp anywhere). */
RXMET_API int rxmet_gru_backward_quant(int T, int B, int I, int H,
                                       const int32_t *W_q_dev, const int32_t *R_q_dev,
                                       const int32_t *bw_q_dev, const int32_t *br_q_dev,
                                       const int32_t *x_q_dev,
                                       const float *dh_new_dev, const float *h_dev,
                                       const float *v_dev,
                                       const rxmet_gru_quant_params *params,
                                       const rxmet_gru_masks *masks,
                                       float *dx_dev, float *dW_dev, float *dR_dev,
                                       float *dbw_dev, float *dbr_dev, float *dh0_dev,
                                       void *workspace_dev, size_t workspace_bytes,
                                       void *stream);

/* The same forward on the reference's FP32 carrier: codes held in floats, every rescale = rint(x * ratio)
 * with ratio = source scale / destination scale in float, the 16-segment tables evaluated in float.
 * Replaces forward_quant_float_storage -> quantGRUForwardFP -> ForwardPassQuantFP::Run as the reference's
 * CUDA build runs it (gru_interface_binding.cc:599-719, operators/quant-gru/src/gru_interface.cc:636-716,
 * src/gru_forward_gpu_quant_fp.cu).  Arguments and outputs as rxmet_gru_forward_quant (the code outputs
 * stay int32; the reference stores the same integers in float tensors).  The matrix products are formed
 * exactly on the integer codes, which equals the reference's float GEMM while the sums stay below 2^24
 * (every 8-bit configuration with input and hidden sizes up to 512); beyond that the reference's own result
 * depends on its GEMM's summation order and this entry returns the exactly summed one. */
RXMET_API int rxmet_gru_forward_quant_fp_carrier(int is_training, int T, int B, int I, int H,
                                                 const float *W_dev, const float *R_dev,
                                                 const float *bw_dev, const float *br_dev,
                                                 const float *x_dev, const float *h0_dev,
                                                 const rxmet_gru_quant_params *params,
                                                 float *h_dev, float *v_dev,
                                                 int32_t *W_q_dev, int32_t *R_q_dev,
                                                 int32_t *bw_q_dev, int32_t *br_q_dev,
                                                 int32_t *x_q_dev, int32_t *h_q_dev, int32_t *v_q_dev,
                                                 const rxmet_gru_masks *masks,
                                                 void *workspace_dev, size_t workspace_bytes,
                                                 void *stream);

/* The training forward / QAT backward pair with the per-step clamp flags in a compact form: instead of the
 * five byte masks weight_ih_linear, weight_hh_linear, gate_input, gate_output and h ([T,B,3H] x 4 + [T,B,H] =
 * 13 bytes per element and step) the forward writes ONE 16-bit word per (t, b, j) into step_flags_dev
 * ([T,B,H] uint16): bit 0..2 = gate_output z, r, n; 3..5 = gate_input; 6..8 = weight_hh_linear; 9..11 =
 * weight_ih_linear; 12 = h (1 = kept), and the backward reads that word.  `masks` still carries the six
 * parameter / input masks (x, h0, W, R, bw, br) and weight_ih_linear, which the input projection fills and the
 * recurrence folds into the word; its other four per-step members may be NULL and are not written then.
 * Results are identical to the byte-mask pair.  For training engines that own their save-for-backward
 * buffers (rx_met_b200.qat.GruQatStep); the reference's binding hands byte masks to Python and has no
 * counterpart.  Supported where rxmet_gru_packed_flags_supported returns 1 (8-bit grids, H <= 128);
 * RXMET_ERR_UNSUPPORTED otherwise. */
RXMET_API int rxmet_gru_packed_flags_supported(const rxmet_gru_quant_params *params, int B, int I, int H);
RXMET_API int rxmet_gru_forward_quant_packed(int T, int B, int I, int H,
                                             const float *W_dev, const float *R_dev,
                                             const float *bw_dev, const float *br_dev,
                                             const float *x_dev, const float *h0_dev,
                                             const rxmet_gru_quant_params *params,
                                             float *h_dev, float *v_dev,
                                             int32_t *W_q_dev, int32_t *R_q_dev,
                                             int32_t *bw_q_dev, int32_t *br_q_dev, int32_t *x_q_dev,
                                             const rxmet_gru_masks *masks, uint16_t *step_flags_dev,
                                             void *workspace_dev, size_t workspace_bytes, void *stream);
RXMET_API int rxmet_gru_backward_quant_packed(int T, int B, int I, int H,
                                              const int32_t *W_q_dev, const int32_t *R_q_dev,
                                              const int32_t *x_q_dev,
                                              const float *dh_new_dev, const float *h_dev, const float *v_dev,
                                              const rxmet_gru_quant_params *params,
                                              const rxmet_gru_masks *masks, const uint16_t *step_flags_dev,
                                              float *dx_dev, float *dW_dev, float *dR_dev,
                                              float *dbw_dev, float *dbr_dev, float *dh0_dev,
                                              void *workspace_dev, size_t workspace_bytes, void *stream);

/* Float backward.  Replaces backward_fp -> gru::BackwardPass<float>::Run
 * (gru_interface_binding.cc:975-1046, operators/quant-gru/src/
 * gru_backward_gpu.cu). */
RXMET_API int rxmet_gru_backward_fp(int T, int B, int I, int H,
                                    const float *W_dev, const float *R_dev,
                                    const float *bw_dev, const float *br_dev,
                                    const float *x_dev,
                                    const float *dh_new_dev, const float *h_dev,
                                    const float *v_dev,
                                    float *dx_dev, float *dW_dev, float *dR_dev,
                                    float *dbw_dev, float *dbr_dev, float *dh0_dev,
                                    void *workspace_dev, size_t workspace_bytes,
                                    void *stream);

/* ------------------------------------------------------------------------ */
/* AIMET native kernels: quantize-dequantize, min/max, PDF histogram          */
/* ------------------------------------------------------------------------ */

/* dtype: 0 = float32, 1 = float64.  Tensors are dense device arrays.  The
 * arithmetic is the reference's CPU definition, which its tests hold equal to
 * torch fake-quantize bit for bit (tests/integration/
 * test_native_qdq_alignment.py:78-131): clamp in the real domain, multiply by
 * the ROUNDED reciprocal of delta, round half to even, multiply by delta; NaN
 * passes through, infinities saturate. */

/* out = QDQ(in) with one encoding.  Replaces quantizeDequantizeGpu
 * (native/common/src/trim_functions.cu:47-58,118-127; value function
 * native/common/src/quantize_dequantize.hpp:36-46).  stochastic != 0 rounds
 * floor(x + u), u uniform in [0,1) from a counter-based generator keyed by
 * seed (statistically, not bitwise, comparable with the reference's curand). */
RXMET_API int rxmet_aimet_qdq(const void *in_dev, uint64_t count, int dtype, double enc_min,
                              double enc_max, double delta, int stochastic, uint64_t seed,
                              void *out_dev, void *stream);

/* Per-channel QDQ, channel = (i / elements_per_channel) % num_channels; the
 * encoding arrays are device arrays of the tensor's dtype.  Replaces
 * quantizeDequantizePerChannelGpu (trim_functions.cu:75-86). */
RXMET_API int rxmet_aimet_qdq_per_channel(const void *in_dev, int num_channels, int64_t num_elements,
                                          int64_t elements_per_channel, int dtype,
                                          const void *min_dev, const void *max_dev,
                                          const void *delta_dev, void *out_dev, void *stream);

/* Broadcast QDQ: strides (host arrays, num_dims <= 8) of the broadcast-aligned
 * tensor and encoding shapes, encoding stride 0 along broadcast dimensions.
 * Replaces quantizeDequantizeBroadcastGpu (trim_functions.cu:90-116). */
RXMET_API int rxmet_aimet_qdq_broadcast(const void *in_dev, void *out_dev, int64_t num_elements,
                                        int num_dims, const int64_t *input_strides,
                                        const int64_t *encoding_strides, int dtype,
                                        const void *min_dev, const void *max_dev,
                                        const void *delta_dev, void *stream);

/* Quantize to the integer index grid (values stay in the tensor's dtype):
 * round_half_away(clamp(x)/delta - offset) - (shift_to_signed ? 2^(bw-1) : 0).
 * Replaces quantizeToFxpGpu (trim_functions.cu:60-73, trim_functions.cuh:
 * 122-149); division is IEEE here, as on the reference's CPU path. */
RXMET_API int rxmet_aimet_quantize_to_fxp(const void *in_dev, uint64_t count, int dtype,
                                          double enc_min, double enc_max, double delta,
                                          double offset, int bitwidth, int shift_to_signed,
                                          void *out_dev, void *stream);

/* Min and max of each consecutive block of block_size elements (count /
 * block_size results, device arrays of the tensor's dtype); block_size ==
 * count gives the whole-tensor pair.  NaN never wins, infinities do.
 * Replaces GetMinMax_gpu (native/common/src/math_functions.cu:81-169).  The
 * whole-tensor form needs rxmet_aimet_minmax_workspace_bytes() of scratch. */
RXMET_API size_t rxmet_aimet_minmax_workspace_bytes(void);
RXMET_API int rxmet_aimet_minmax(const void *data_dev, uint64_t count, uint64_t block_size, int dtype,
                                 void *min_out_dev, void *max_out_dev, void *workspace_dev,
                                 size_t workspace_bytes, void *stream);

/* PDF histogram with rxmet_aimet_pdf_size() (= 1536) buckets: bucket of x is
 * floor(x * (1/bucket_size)) - pdf_offset, values outside are dropped;
 * histogram_dev (uint32) is overwritten.  Replaces GetHistogram_gpu
 * (math_functions.cu:232-268) with the bucket rule of the reference's CPU
 * path (native/common/src/math_functions.cpp:395-412), which is what its
 * encoding analyzers are specified against. */
RXMET_API int rxmet_aimet_pdf_size(void);
RXMET_API int rxmet_aimet_histogram(const void *data_dev, uint64_t count, int dtype, double bucket_size,
                                    int pdf_offset, uint32_t *histogram_dev, void *stream);

/* Encoding of a (min, max) range (TfEncoding, native/common/include/DlQuantization/
 * Quantization.hpp:114-121). */
typedef struct rxmet_aimet_encoding {
    double min, max, delta, offset;
    int32_t bw;
} rxmet_aimet_encoding;

/* Range -> encoding (getComputedEncodings, native/common/src/quantization_utils.cpp:59-117):
 * zero kept on the grid, symmetric / strict-symmetric / unsigned-symmetric modes,
 * delta clamped so that the dequantized range stays inside 0.99 of float32. */
RXMET_API int rxmet_aimet_compute_encoding(int bw, double range_min, double range_max, int symmetric,
                                           int strict_symmetric, int unsigned_symmetric,
                                           rxmet_aimet_encoding *encoding);

/* Min/max statistics -> encoding (MinMaxEncodingAnalyzer::computeEncoding,
 * native/common/src/MinMaxEncodingAnalyzer.cpp:80-107): zero included, maximum
 * nudged to at least minimum + 0.01 (0.01 in the analyzer's element type: dtype 0
 * = float, 1 = double).  stats_min / stats_max are the running extremes that
 * rxmet_aimet_minmax accumulates.  With dtype 1 and statistics that start at 0 / 0 this is
 * also TfEncodingAnalyzer::computeEncoding (native/common/src/TfEncodingAnalyzer.cpp:88-108),
 * whose updateStats is a running min / max in double. */
RXMET_API int rxmet_aimet_minmax_encoding(int bw, int dtype, double stats_min, double stats_max, int symmetric,
                                          int strict_symmetric, int unsigned_symmetric,
                                          rxmet_aimet_encoding *encoding);

/* Running histogram statistics of the histogram analyzers (struct PDF,
 * native/common/src/math_functions.hpp): left bucket edges and the running
 * average of the per-batch probabilities, rxmet_aimet_pdf_size() doubles each,
 * in host memory owned by the caller. */
typedef struct rxmet_aimet_pdf {
    double *x_left;
    double *pdf;
    int32_t initialized; /* the first batch that is not all zero fixes the range */
    int32_t iterations;  /* batches averaged so far */
    int32_t updated;     /* a batch was offered (all-zero batches count) */
} rxmet_aimet_pdf;

RXMET_API int rxmet_aimet_pdf_reset(rxmet_aimet_pdf *pdf);
/* UpdatePdf (native/common/src/math_functions.cpp:272-316) in three steps, so that the counting
 * can run wherever the data lives:
 *   plan   - from the batch extremes: on the first non-zero batch the range (InitializePdf,
 *            :226-269: tripled around its centre); returns the bucket size and offset for the
 *            counting, or *skip = 1 for an all-zero batch before any range exists;
 *   count  - rxmet_aimet_histogram on the device (or any exact counter);
 *   commit - pdf = (pdf * iterations + histogram / count) / (iterations + 1). */
RXMET_API int rxmet_aimet_pdf_plan(rxmet_aimet_pdf *pdf, float batch_min, float batch_max, int signed_values,
                                   double *bucket_size, int *pdf_offset, int *skip);
RXMET_API int rxmet_aimet_pdf_commit(rxmet_aimet_pdf *pdf, const uint32_t *histogram, uint64_t count);
/* All three steps on a host tensor (the reference's CPU mode). */
RXMET_API int rxmet_aimet_pdf_update_host(rxmet_aimet_pdf *pdf, const float *data, uint64_t count, int signed_values);
/* All three steps on a device float tensor: rxmet_aimet_minmax when no range exists yet,
 * rxmet_aimet_histogram, one synchronisation of the stream per step that returns to the host.
 * workspace: rxmet_aimet_pdf_workspace_bytes() device bytes. */
RXMET_API size_t rxmet_aimet_pdf_workspace_bytes(void);
RXMET_API int rxmet_aimet_pdf_update(rxmet_aimet_pdf *pdf, const float *data_dev, uint64_t count, int signed_values,
                                     void *workspace_dev, size_t workspace_bytes, void *stream);

/* TfEnhancedEncodingAnalyzer<float>::computeEncoding (native/common/src/
 * TfEnhancedEncodingAnalyzer.cpp:86-411): grid search over (delta, offset) candidates - 17 x 21
 * clamped to the observed range plus the observed range itself, or 101 deltas on the symmetric
 * grid - for the least quantization cost + 3 x saturation cost of the bucket centres. */
RXMET_API int rxmet_aimet_tf_enhanced_encoding(const rxmet_aimet_pdf *pdf, int bw, int symmetric, int strict_symmetric,
                                               int unsigned_symmetric, rxmet_aimet_encoding *encoding);
/* PercentileEncodingAnalyzer<float>::computeEncoding (native/common/src/
 * PercentileEncodingAnalyzer.cpp:86-203): range between the (100 - p) and p percentiles of the
 * collected distribution (never beyond the observed maximum), zero included, then
 * rxmet_aimet_compute_encoding. */
RXMET_API int rxmet_aimet_percentile_encoding(const rxmet_aimet_pdf *pdf, int bw, int symmetric, int strict_symmetric,
                                              int unsigned_symmetric, float percentile, rxmet_aimet_encoding *encoding);

/* ------------------------------------------------------------------------ */
/* Allocation-free variant                                                    */
/* ------------------------------------------------------------------------ */

/* Size of the scratch array built into the library image (bytes). */
#define RXMET_STATIC_SCRATCH_BYTES (8u << 20)
RXMET_API size_t rxmet_static_scratch_bytes(void);

/* Float GRU forward that needs no workspace and allocates nothing, neither on
 * the device nor on the host: same arguments and results as
 * rxmet_gru_forward_fp minus the workspace pair.  It has no counterpart in the
 * reference (whose wrappers allocate their outputs and temporaries on every
 * call); it exists for callers that must not allocate while they run, such as
 * a runtime plugin's enqueue callback, a fixed-deadline audio or control loop,
 * or a process whose memory pool is frozen after start-up.
 *   - The scratch (W x + bw for all T*B rows) lives in a fixed 8 MiB array
 *     inside the library image; every GPU that loads the library holds it
 *     until the process exits.  Calls with T*B*3H*4 > 8 MiB are rejected with
 *     RXMET_ERR_WORKSPACE and leave the outputs untouched.
 *   - The first call on each device looks up the device address of that array
 *     (a host-side query, no allocation).  Make that first call during
 *     start-up, outside any stream capture; later calls only launch kernels.
 *   - All calls on one device share the array.  Nothing in it has to be
 *     cleared between calls, but two calls whose kernels can overlap on the
 *     GPU (different streams, or threads racing on one stream) would overwrite
 *     each other's projection: serialise them. */
RXMET_API int rxmet_gru_forward_fp_static(int T, int B, int I, int H,
                                          const float *W_dev, const float *R_dev,
                                          const float *bw_dev, const float *br_dev,
                                          const float *x_dev, const float *h0_dev,
                                          float *h_dev, float *v_dev, void *stream);

/* ---- affine quantizers with a learned grid (aimet_torch.v2) ---------------------------------
 * Fused quantize-dequantize and its backward, replacing the eager tensor expressions of
 * src/aimet_torch/v2/quantization/affine/backends/torch_builtins.py (quantize_dequantize :199-285,
 * QuantDequantFunc.forward :640-669 and .backward :675-691, and the torch.fake_quantize fast path
 * :288-360 taken when the grid is not trained).
 *
 * The tensor is [outer][channels][inner], contiguous; scale_dev / offset_dev hold one float per
 * channel (channels == 1: per tensor).  reciprocal == 0 is the divide form (rne(x / s) - o), the one
 * the reference differentiates with respect to scale and offset; reciprocal == 1 is the fast path
 * (rne(x * (1 / s)) + zp on integers, NaN kept).  y, keep and dx are bit-exact; dscale / doffset are
 * float sums (fixed order, run-to-run reproducible).  Infinite inputs saturate to the nearer end of the
 * grid in both forms.  |qmin|, |qmax| < 2^24. */
RXMET_API int rxmet_affine_qdq_forward(const float *x_dev, uint64_t outer, uint64_t channels, uint64_t inner,
                                       const float *scale_dev, const float *offset_dev, int qmin, int qmax,
                                       int reciprocal, float *y_dev,
                                       uint8_t *keep_dev /* optional: 1 where inside the grid */, void *stream);
RXMET_API size_t rxmet_affine_qdq_backward_workspace_bytes(uint64_t outer, uint64_t channels, uint64_t inner);
/* Any of dx_dev, dscale_dev [channels], doffset_dev [channels] may be null; the grid gradients exist in
 * the divide form only and need the workspace. */
RXMET_API int rxmet_affine_qdq_backward(const float *grad_dev, const float *x_dev, uint64_t outer, uint64_t channels,
                                        uint64_t inner, const float *scale_dev, const float *offset_dev, int qmin,
                                        int qmax, int reciprocal, float *dx_dev, float *dscale_dev, float *doffset_dev,
                                        void *workspace_dev, size_t workspace_bytes, void *stream);

/* ---- loss of the training step -------------------------------------------------------------
 * Mean-squared-error loss between the output sequence and a target and its gradient with respect to the
 * output, fused: grad = (out - target) * (2 / count) (bit-identical to the eager float32 expressions
 * `diff = out - target; grad = diff * (2.0 / diff.numel())` of a training loop; this entry has no
 * counterpart in the reference, whose loss lives in the caller's torch code), *loss_dev =
 * sum (out - target)^2 / count (fixed summation order).  workspace: rxmet_mse_loss_workspace_bytes()
 * device bytes. */
RXMET_API size_t rxmet_mse_loss_workspace_bytes(void);
RXMET_API int rxmet_mse_loss_grad(const float *out_dev, const float *target_dev, uint64_t count, float *grad_dev,
                                  float *loss_dev, void *workspace_dev, size_t workspace_bytes, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* RXMET_B200_H_ */
