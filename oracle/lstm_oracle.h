/*
 * TEST INFRASTRUCTURE - declarations of the CPU restatement of the QuantLSTM
 * path of rx-met (plain C).  Only tests, the smoke check and the CPU legs of
 * the benchmark may load it, and only as the checker.
 */
#ifndef RXMET_LSTM_ORACLE_H_
#define RXMET_LSTM_ORACLE_H_

#include <stdint.h>

#include "rxmet_b200_lstm.h"

void orc_lstm_type_range(const rxmet_lstm_quant_config *c, int op, int32_t *lo, int32_t *hi);

int orc_lstm_params_from_ranges(const rxmet_lstm_quant_config *config, const rxmet_lstm_ranges *ranges, int I, int H,
                                int bias, float *w_ih_scale, float *w_hh_scale, float *b_ih_scale, float *b_hh_scale,
                                rxmet_lstm_quant_params *params);
int orc_lstm_derive_execution(const rxmet_lstm_quant_params *params, int exact, rxmet_lstm_execution *out);

/* Executable form used by the forward restatement: the flat struct plus owned per-channel arrays. */
typedef struct orc_lstm_exec {
    rxmet_lstm_execution e;
    int32_t lo[RXMET_LSTM_NUM_OPS], hi[RXMET_LSTM_NUM_OPS];
} orc_lstm_exec;

#endif
