"""ctypes mirrors of the QuantLSTM part of the C ABI (``include/rxmet_b200_lstm.h``)."""
from __future__ import annotations

import ctypes as C

import numpy as np

NUM_OPS = 18
(INPUT, OUTPUT, CELL_STATE, WEIGHT_IH, WEIGHT_HH, BIAS_IH, BIAS_HH, WEIGHT_IH_LINEAR, WEIGHT_HH_LINEAR,
 INPUT_GATE_INPUT, FORGET_GATE_INPUT, CELL_GATE_INPUT, OUTPUT_GATE_INPUT, INPUT_GATE_OUTPUT, FORGET_GATE_OUTPUT,
 CELL_GATE_OUTPUT, OUTPUT_GATE_OUTPUT, CELL_TANH_OUTPUT) = range(NUM_OPS)

# Names of the points in the reference's configuration and bundle JSON
# (operators/quant-lstm/src/lstm/quant_config.cc, quantOperatorName).
OP_NAMES = ("input", "output", "cell_state", "weight_ih", "weight_hh", "bias_ih", "bias_hh", "weight_ih_linear",
            "weight_hh_linear", "input_gate_input", "forget_gate_input", "cell_gate_input", "output_gate_input",
            "input_gate_output", "forget_gate_output", "cell_gate_output", "output_gate_output", "cell_tanh_output")
PARAMETER_OPS = (WEIGHT_IH, WEIGHT_HH, BIAS_IH, BIAS_HH)
BIAS_OPS = (BIAS_IH, BIAS_HH)

PER_TENSOR, PER_GATE, PER_CHANNEL = 0, 1, 2
GRANULARITY_NAMES = ("per_tensor", "per_gate", "per_channel")
SCALE_AFFINE, SCALE_POT2 = 0, 1
SCALE_MODE_NAMES = ("affine", "pot2")

_f32p = C.POINTER(C.c_float)
_u8p = C.POINTER(C.c_uint8)


class QuantConfig(C.Structure):
    _fields_ = [("scale_mode", C.c_int32), ("bitwidth", C.c_int32 * NUM_OPS), ("is_unsigned", C.c_uint8 * NUM_OPS),
                ("is_symmetric", C.c_uint8 * NUM_OPS), ("granularity", C.c_uint8 * NUM_OPS)]


class QuantParams(C.Structure):
    _fields_ = [("config", QuantConfig), ("input_size", C.c_int32), ("hidden_size", C.c_int32),
                ("bias_enabled", C.c_int32), ("scale", C.c_float * NUM_OPS), ("zero_point", C.c_int32 * NUM_OPS),
                ("weight_ih_scale", _f32p), ("weight_hh_scale", _f32p), ("bias_ih_scale", _f32p),
                ("bias_hh_scale", _f32p)]


class Ranges(C.Structure):
    _fields_ = [("minimum", C.c_float * NUM_OPS), ("maximum", C.c_float * NUM_OPS),
                ("contribution_min", C.c_float * 3), ("contribution_max", C.c_float * 3),
                ("channel_min", _f32p * 4), ("channel_max", _f32p * 4)]


class Rescale(C.Structure):
    _fields_ = [("is_m_shift", C.c_int32), ("multiplier", C.c_int32), ("shift", C.c_int32)]

    def astuple(self):
        return (self.is_m_shift, self.multiplier, self.shift)


class CellScale(C.Structure):
    _fields_ = [("multiplier", C.c_int64), ("fp_mantissa", C.c_double), ("fp_exponent", C.c_int32),
                ("uses_fp_scale", C.c_int32)]

    def astuple(self):
        return (self.multiplier, self.fp_mantissa, self.fp_exponent, self.uses_fp_scale)


_rsp = C.POINTER(Rescale)


class Execution(C.Structure):
    _fields_ = [("ih_to_gate", Rescale * 4), ("hh_to_gate", Rescale * 4), ("forget_scale", CellScale),
                ("input_scale", CellScale), ("product_to_output", Rescale), ("exact_accumulation", C.c_int32),
                ("ih_bias_to_accumulator", _rsp), ("ih_accumulator_to_output", _rsp),
                ("hh_bias_to_accumulator", _rsp), ("hh_accumulator_to_output", _rsp)]


TRACE_VALUES = ("weight_ih_linear", "weight_hh_linear", "gate_inputs", "gate_outputs", "cell_states",
                "cell_tanh_outputs", "hidden_outputs")


class Trace(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in TRACE_VALUES] + [(n + "_clamped", C.c_void_p) for n in TRACE_VALUES]


MASTER_VALUES = ("input", "weight_ih", "weight_hh", "bias_ih", "bias_hh", "initial_hidden", "initial_cell")


class Masters(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in MASTER_VALUES] + [(n + "_clamped", C.c_void_p) for n in MASTER_VALUES]


class BackwardMasks(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in MASTER_VALUES + TRACE_VALUES]


class Gradients(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in MASTER_VALUES]


class ParamsBox:
    """QuantParams plus the numpy arrays its pointers refer to."""

    def __init__(self, H: int):
        self.H = H
        self.channel_scales = [np.zeros(4 * H, np.float32) for _ in range(4)]
        self.struct = QuantParams()
        self.bind()

    def bind(self):
        s = self.struct
        ptrs = [a.ctypes.data_as(_f32p) for a in self.channel_scales]
        s.weight_ih_scale, s.weight_hh_scale = ptrs[0], ptrs[1]
        if s.bias_enabled or not s.hidden_size:
            s.bias_ih_scale, s.bias_hh_scale = ptrs[2], ptrs[3]
        else:
            s.bias_ih_scale, s.bias_hh_scale = None, None

    def scale_ptrs(self):
        return [a.ctypes.data_as(_f32p) for a in self.channel_scales]


class RangesBox:
    def __init__(self, H: int):
        self.H = H
        self.mins = [np.full(4 * H, np.inf, np.float32) for _ in range(4)]
        self.maxs = [np.full(4 * H, -np.inf, np.float32) for _ in range(4)]
        self.struct = Ranges()
        for i in range(NUM_OPS):
            self.struct.minimum[i] = np.inf
            self.struct.maximum[i] = -np.inf
        for k in range(3):
            self.struct.contribution_min[k] = np.inf
            self.struct.contribution_max[k] = -np.inf
        for k in range(4):
            self.struct.channel_min[k] = self.mins[k].ctypes.data_as(_f32p)
            self.struct.channel_max[k] = self.maxs[k].ctypes.data_as(_f32p)


class ExecutionBox:
    def __init__(self, H: int):
        self.arrays = [(Rescale * (4 * H))() for _ in range(4)]
        self.struct = Execution()
        s = self.struct
        s.ih_bias_to_accumulator = C.cast(self.arrays[0], _rsp)
        s.ih_accumulator_to_output = C.cast(self.arrays[1], _rsp)
        s.hh_bias_to_accumulator = C.cast(self.arrays[2], _rsp)
        s.hh_accumulator_to_output = C.cast(self.arrays[3], _rsp)

    def flat(self, bias: bool):
        s = self.struct
        out = [r.astuple() for r in s.ih_to_gate] + [r.astuple() for r in s.hh_to_gate]
        out += [s.forget_scale.astuple(), s.input_scale.astuple(), s.product_to_output.astuple()]
        for k, arr in enumerate(self.arrays):
            if k in (0, 2) and not bias:
                continue
            out += [r.astuple() for r in arr]
        return out


class Histogram(C.Structure):
    """``rxmet_lstm_histogram``; ``counts`` points at host doubles."""
    _fields_ = [("counts", C.POINTER(C.c_double)), ("num_bins", C.c_int32), ("minimum", C.c_float),
                ("maximum", C.c_float), ("total_count", C.c_uint64)]


class Histograms(C.Structure):
    """``rxmet_lstm_histograms``."""
    _fields_ = [("hidden_size", C.c_int32), ("num_bins", C.c_int32), ("point", Histogram * NUM_OPS),
                ("gate", (Histogram * 4) * 4), ("channel", C.POINTER(Histogram) * 4)]


class HistogramSet:
    """All collectors of a calibration session with their storage: 18 point collectors, 4 x 4 gate
    collectors and 4 x 4H channel collectors."""

    def __init__(self, hidden: int, num_bins: int = 2048):
        self.hidden, self.num_bins = int(hidden), int(num_bins)
        total = NUM_OPS + 16 + 16 * self.hidden
        self.counts = np.zeros((total, self.num_bins), np.float64)
        self.channels = [(Histogram * (4 * self.hidden))() for _ in range(4)]
        self.struct = Histograms()
        self.struct.hidden_size, self.struct.num_bins = self.hidden, self.num_bins
        for row, h in enumerate(self.all()):
            h.counts = self.counts[row].ctypes.data_as(C.POINTER(C.c_double))
            h.num_bins = self.num_bins
        for k in range(4):
            self.struct.channel[k] = C.cast(self.channels[k], C.POINTER(Histogram))

    def all(self):
        for op in range(NUM_OPS):
            yield self.struct.point[op]
        for k in range(4):
            for g in range(4):
                yield self.struct.gate[k][g]
        for k in range(4):
            for ch in range(4 * self.hidden):
                yield self.channels[k][ch]

    def states(self):
        return [(h.minimum, h.maximum, int(h.total_count)) for h in self.all()]


def default_config(scale_mode=SCALE_AFFINE, bits=8, symmetric_activations=False,
                   parameter_granularity=PER_CHANNEL) -> QuantConfig:
    """8-bit grid: symmetric signed parameters, unsigned sigmoid outputs, other activations signed."""
    cfg = QuantConfig()
    cfg.scale_mode = scale_mode
    for op in range(NUM_OPS):
        cfg.bitwidth[op] = bits
        cfg.is_unsigned[op] = 1 if op in (INPUT_GATE_OUTPUT, FORGET_GATE_OUTPUT, OUTPUT_GATE_OUTPUT) else 0
        cfg.is_symmetric[op] = 1 if (op in PARAMETER_OPS or symmetric_activations) else 0
        cfg.granularity[op] = parameter_granularity if op in PARAMETER_OPS else PER_TENSOR
    return cfg


def mixed_config(weight_bits=8, activation_bits=16, bias_bits=None, scale_mode=SCALE_AFFINE, symmetric_activations=False,
                 parameter_granularity=PER_CHANNEL) -> QuantConfig:
    """Mixed-precision grid: `weight_bits` for weight_ih / weight_hh (W4, W8), `activation_bits` for every
    activation point (input, output, cell state, the two linear outputs, gate inputs and outputs, tanh(cell));
    biases take `bias_bits` (default: the activation width)."""
    cfg = default_config(scale_mode=scale_mode, bits=activation_bits, symmetric_activations=symmetric_activations,
                         parameter_granularity=parameter_granularity)
    cfg.bitwidth[WEIGHT_IH] = cfg.bitwidth[WEIGHT_HH] = weight_bits
    cfg.bitwidth[BIAS_IH] = cfg.bitwidth[BIAS_HH] = activation_bits if bias_bits is None else bias_bits
    return cfg

