"""ctypes view of ``include/rxmet_b200.h``: the structs and the library loader.

The shared library is the product: if it is missing or cannot be loaded the
import of the operator modules fails with a clear error.  Nothing here falls
back to a CPU implementation.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

NUM_OPS = 17
(X, H, W, R, BW, BR, WEIGHT_IH_LINEAR, WEIGHT_HH_LINEAR, UPDATE_GATE_INPUT, UPDATE_GATE_OUTPUT,
 RESET_GATE_INPUT, RESET_GATE_OUTPUT, NEW_GATE_INPUT, NEW_GATE_OUTPUT, MUL_RESET_HIDDEN,
 MUL_OLD_CONTRIBUTION, MUL_NEW_CONTRIBUTION) = range(NUM_OPS)

#: quantization-point names in the order of the C enum (also the attribute stems
#: used by the reference's OperatorQuantConfig / GRUQuantParams Python classes).
OP_NAMES = (
    "x", "h", "W", "R", "bw", "br", "weight_ih_linear", "weight_hh_linear",
    "update_gate_input", "update_gate_output", "reset_gate_input", "reset_gate_output",
    "new_gate_input", "new_gate_output", "mul_reset_hidden", "mul_old_contribution",
    "mul_new_contribution",
)
SCALAR_OPS = tuple(i for i in range(NUM_OPS) if i not in (W, R, BW, BR))

PER_TENSOR, PER_GATE, PER_CHANNEL = 0, 1, 2
POT_ROUND, POT_COVER_RANGE, POT_FLOOR = 0, 1, 2

_f32p = C.POINTER(C.c_float)
_u8p = C.POINTER(C.c_uint8)
_i32p = C.POINTER(C.c_int32)


class QuantConfig(C.Structure):
    """``rxmet_gru_quant_config``."""
    _fields_ = [
        ("bits", C.c_int8 * NUM_OPS),
        ("is_unsigned", C.c_uint8 * NUM_OPS),
        ("symmetric", C.c_uint8 * NUM_OPS),
        ("W_granularity", C.c_int32),
        ("R_granularity", C.c_int32),
        ("bw_granularity", C.c_int32),
        ("br_granularity", C.c_int32),
        ("use_pot2", C.c_uint8),
        ("pot_scale_method", C.c_int8),
        ("pot_scale_tolerance", C.c_float),
    ]


class Ranges(C.Structure):
    """``rxmet_gru_ranges``."""
    _fields_ = [
        ("hidden", C.c_int32),
        ("min", C.c_float * NUM_OPS),
        ("max", C.c_float * NUM_OPS),
        ("min_W", _f32p), ("max_W", _f32p), ("min_R", _f32p), ("max_R", _f32p),
        ("min_bw", _f32p), ("max_bw", _f32p), ("min_br", _f32p), ("max_br", _f32p),
    ]


class QuantParams(C.Structure):
    """``rxmet_gru_quant_params``."""
    _fields_ = [
        ("hidden", C.c_int32),
        ("scale", C.c_float * NUM_OPS),
        ("zero_point", C.c_int32 * NUM_OPS),
        ("scale_W", _f32p), ("scale_R", _f32p), ("scale_bw", _f32p), ("scale_br", _f32p),
        ("config", QuantConfig),
    ]


class LutSegment(C.Structure):
    """``rxmet_lut_segment``."""
    _fields_ = [("q_b", C.c_int32), ("n_bx_total", C.c_int32), ("term_c", C.c_int32),
                ("threshold", C.c_int32)]


class Masks(C.Structure):
    """``rxmet_gru_masks``: eleven device (or host, for the checker) uint8 arrays."""
    _fields_ = [(n, C.c_void_p) for n in (
        "x", "h0", "W", "R", "bw", "br", "weight_ih_linear", "weight_hh_linear",
        "gate_input", "gate_output", "h")]


MASK_NAMES = tuple(n for n, _ in Masks._fields_)


class Histogram(C.Structure):
    """``rxmet_histogram``: one collector; ``counts`` points at host floats."""
    _fields_ = [("counts", _f32p), ("num_bins", C.c_int32), ("min_val", C.c_float), ("max_val", C.c_float),
                ("observed_min", C.c_float), ("observed_max", C.c_float), ("total_count", C.c_int64),
                ("range_limit_set", C.c_int32), ("range_limit_min", C.c_float), ("range_limit_max", C.c_float)]


class HistogramPlan(C.Structure):
    """``rxmet_histogram_plan``: what a batch with given global extremes does to a collector."""
    _fields_ = [("mode", C.c_int32), ("lo", C.c_float), ("hi", C.c_float), ("inv_bin_width", C.c_float),
                ("new_min", C.c_float), ("new_max", C.c_float), ("data_min", C.c_float), ("data_max", C.c_float),
                ("limit_min", C.c_float), ("limit_max", C.c_float)]


class GruHistograms(C.Structure):
    """``rxmet_gru_histograms``."""
    _fields_ = [("hidden", C.c_int32), ("num_bins", C.c_int32), ("point", Histogram * NUM_OPS),
                ("channel", C.POINTER(Histogram) * 4), ("gate", (Histogram * 3) * 4)]


class HistogramSet:
    """All collectors of one GRU direction with the storage their count pointers refer to:
    17 point collectors, 4 x 3 gate collectors and 4 x 3*hidden channel collectors."""

    def __init__(self, hidden: int, num_bins: int = 2048):
        import numpy as np
        self.hidden, self.num_bins = int(hidden), int(num_bins)
        total = NUM_OPS + 12 + 12 * self.hidden
        self.counts = np.zeros((total, self.num_bins), np.float32)
        self.channels = [(Histogram * (3 * self.hidden))() for _ in range(4)]
        self.c = GruHistograms()
        self.c.hidden, self.c.num_bins = self.hidden, self.num_bins
        row = 0
        for h in self.all():
            h.counts = self.counts[row].ctypes.data_as(_f32p)
            h.num_bins = self.num_bins
            row += 1
        for k in range(4):
            self.c.channel[k] = C.cast(self.channels[k], C.POINTER(Histogram))
        self.reset()

    def all(self):
        for op in range(NUM_OPS):
            yield self.c.point[op]
        for k in range(4):
            for g in range(3):
                yield self.c.gate[k][g]
        for k in range(4):
            for ch in range(3 * self.hidden):
                yield self.channels[k][ch]

    def reset(self):
        self.counts[:] = 0
        fmax = 3.4028234663852886e38
        for h in self.all():
            h.min_val, h.max_val = fmax, -fmax
            h.observed_min, h.observed_max = fmax, -fmax
            h.total_count = 0
            h.range_limit_set = 0
            h.range_limit_min = h.range_limit_max = 0.0

    def is_valid(self) -> bool:
        return self.hidden > 0 and self.c.point[X].total_count > 0

LIB_NAME = "librxmet_b200.so"


def library_path() -> Path:
    override = os.environ.get("RXMET_B200_LIBRARY")
    if override:
        return Path(override)
    return Path(__file__).resolve().parent / "csrc" / LIB_NAME


_lib = None


def load_library() -> C.CDLL:
    """Load the CUDA library (once).  Raises ``RuntimeError`` when it is absent."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not path.exists():
        raise RuntimeError(
            f"{path} not found: build the CUDA library first "
            "(python -c 'import __graft_entry__ as g; g.build()' or make -C rx_met_b200/csrc). "
            "There is no CPU fallback.")
    try:
        lib = C.CDLL(str(path), mode=C.RTLD_GLOBAL)
    except OSError as exc:  # pragma: no cover - depends on the machine
        raise RuntimeError(f"could not load {path}: {exc}") from exc
    lib.rxmet_last_error.restype = C.c_char_p
    lib.rxmet_version.restype = C.c_char_p
    lib.rxmet_kernel_launch_count.restype = C.c_uint64
    lib.rxmet_gru_workspace_bytes.restype = C.c_size_t
    lib.rxmet_gru_workspace_bytes.argtypes = [C.c_int] * 5
    lib.rxmet_gru_stats_floats.restype = C.c_size_t
    lib.rxmet_gru_stats_floats.argtypes = [C.c_int]
    _lib = lib
    return lib


def check(status: int, what: str) -> None:
    """Turn a negative ``rxmet_status`` into the exception the reference raises."""
    if status == 0:
        return
    msg = load_library().rxmet_last_error().decode("utf-8", "replace")
    if status == -1:
        raise ValueError(f"{what}: {msg}")
    raise RuntimeError(f"{what}: {msg} (status {status})")
