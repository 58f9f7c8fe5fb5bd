"""Drop-in for the reference's ``gru_interface_binding`` extension module.

Same names, argument meaning, return tuples and error behaviour as
``operators/quant-gru/pytorch/lib/gru_interface_binding.cc:1331-1788`` so that the
reference's ``quant_gru.py`` can import this module in its place.  Every compute
entry forwards to the C ABI of ``librxmet_b200.so`` (``include/rxmet_b200.h``);
torch only provides device memory and the current stream.  There is no CPU path:
tensors must be CUDA float32 and the library must be built.

Numerics note: both ``forward_quant_float_storage`` and
``forward_quant_int_storage`` run the integer carrier (exact integer
accumulation, M*2^-shift rescale, integer activation tables) and differ only in
the dtype of the returned code caches, exactly as the reference's CPU build does
(``gru_cpu_binding.h:66-116``).
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Tuple

import torch

from . import _cabi as cabi

cpu_only = False
use_real_activation = False

_FMAX = 3.4028234663852886e38


# Data-parallel calibration (no counterpart in the reference's module): with a process group set here, every
# rank passes its shard of each calibration batch to forward_calibrate(); min/max statistics and histogram bin
# counts are all-reduced inside the batch, so all ranks end with the collectors one process would hold after
# the concatenated batches.
_calibration_group = None
_exchange_cache = {}


def set_calibration_process_group(group) -> None:
    global _calibration_group
    _calibration_group = group
    _exchange_cache.clear()


def _exchange_for(device):
    if _calibration_group is None:
        return None
    key = str(device)
    if key not in _exchange_cache:
        from .data_parallel import make_exchange
        _exchange_cache[key] = make_exchange(_calibration_group, device)
    return _exchange_cache[key]


def init_gru_cublas() -> None:
    """Kept for interface compatibility; the kernels do not use cuBLAS."""
    cabi.load_library()


def decode_effective_scale(scale: float, usePOT2: bool) -> float:
    if not scale > 0.0:
        raise ValueError("scale must be > 0")
    out = C.c_float()
    cabi.check(cabi.load_library().rxmet_gru_decode_effective_scale(C.c_float(scale), int(bool(usePOT2)), C.byref(out)),
               "decode_effective_scale")
    return float(out.value)


# --------------------------------------------------------------------------
# configuration / parameter objects (plain Python mirrors of the pybind classes)
# --------------------------------------------------------------------------

class OperatorQuantConfig:
    """Bit-widths 1..32, symmetry and signedness of the 17 quantization points, the four
    weight granularities (0 tensor, 1 gate, 2 channel) and the power-of-two switch."""

    def __init__(self):
        for name in cabi.OP_NAMES:
            setattr(self, f"{name}_", 8)
            setattr(self, f"{name}_symmetric_", True)
            setattr(self, f"{name}_unsigned_", name in ("update_gate_output", "reset_gate_output"))
        self.W_granularity_ = self.R_granularity_ = self.bw_granularity_ = self.br_granularity_ = cabi.PER_CHANNEL
        self.usePOT2_ = False
        self.pot_scale_method_ = cabi.POT_COVER_RANGE
        self.pot_scale_tolerance_ = 0.02

    def __setattr__(self, key, value):
        # a change counter lets holders of a converted copy (GRUQuantParams) notice assignments
        object.__setattr__(self, key, value)
        if not key.startswith("_"):
            object.__setattr__(self, "_version", getattr(self, "_version", 0) + 1)

    # the reference exposes the same field under two spellings
    @property
    def usePO2_(self):
        return self.usePOT2_

    @usePO2_.setter
    def usePO2_(self, value):
        self.usePOT2_ = bool(value)

    def _to_c(self) -> cabi.QuantConfig:
        cfg = cabi.QuantConfig()
        for i, name in enumerate(cabi.OP_NAMES):
            cfg.bits[i] = int(getattr(self, f"{name}_"))
            cfg.is_unsigned[i] = int(bool(getattr(self, f"{name}_unsigned_")))
            cfg.symmetric[i] = int(bool(getattr(self, f"{name}_symmetric_")))
        cfg.W_granularity = int(self.W_granularity_)
        cfg.R_granularity = int(self.R_granularity_)
        cfg.bw_granularity = int(self.bw_granularity_)
        cfg.br_granularity = int(self.br_granularity_)
        cfg.use_pot2 = int(bool(self.usePOT2_))
        cfg.pot_scale_method = int(self.pot_scale_method_)
        cfg.pot_scale_tolerance = float(self.pot_scale_tolerance_)
        return cfg

    @classmethod
    def _from_c(cls, cfg: cabi.QuantConfig) -> "OperatorQuantConfig":
        out = cls()
        for i, name in enumerate(cabi.OP_NAMES):
            setattr(out, f"{name}_", int(cfg.bits[i]))
            setattr(out, f"{name}_unsigned_", bool(cfg.is_unsigned[i]))
            setattr(out, f"{name}_symmetric_", bool(cfg.symmetric[i]))
        out.W_granularity_, out.R_granularity_ = cfg.W_granularity, cfg.R_granularity
        out.bw_granularity_, out.br_granularity_ = cfg.bw_granularity, cfg.br_granularity
        out.usePOT2_ = bool(cfg.use_pot2)
        out.pot_scale_method_ = int(cfg.pot_scale_method)
        out.pot_scale_tolerance_ = float(cfg.pot_scale_tolerance)
        return out


# attribute stem used by the reference for each scalar range / parameter
_RANGE_STEM = {cabi.WEIGHT_IH_LINEAR: "Wx", cabi.WEIGHT_HH_LINEAR: "Rh"}
_CHANNEL_NAMES = ("W", "R", "bw", "br")


def _range_stem(op: int) -> str:
    return _RANGE_STEM.get(op, cabi.OP_NAMES[op])


class GRUQuantizationRanges:
    """min/max per quantization point (``min_x_`` ... ``max_mul_old_contribution_``) plus
    per-channel lists for W, R, bw, br; ``reset`` restores (FLT_MAX, -FLT_MAX)."""

    def __init__(self, hidden: int = 0):
        self.hidden_ = int(hidden)
        self.reset()

    def reset(self, hidden: int = -1) -> None:
        if hidden > 0:
            self.hidden_ = int(hidden)
        for op in cabi.SCALAR_OPS:
            setattr(self, f"min_{_range_stem(op)}_", _FMAX)
            setattr(self, f"max_{_range_stem(op)}_", -_FMAX)
        n = 3 * self.hidden_
        for name in _CHANNEL_NAMES:
            setattr(self, f"min_{name}_", [_FMAX] * n)
            setattr(self, f"max_{name}_", [-_FMAX] * n)

    # ---- C struct round trip
    def _to_c(self):
        n = 3 * self.hidden_
        c = cabi.Ranges()
        c.hidden = self.hidden_
        for op in cabi.SCALAR_OPS:
            c.min[op] = getattr(self, f"min_{_range_stem(op)}_")
            c.max[op] = getattr(self, f"max_{_range_stem(op)}_")
        keep = []
        for name in _CHANNEL_NAMES:
            for kind in ("min", "max"):
                values = list(getattr(self, f"{kind}_{name}_"))
                if len(values) != n:
                    raise ValueError(f"{kind}_{name}_ must hold 3*hidden = {n} values")
                arr = (C.c_float * n)(*values)
                keep.append(arr)
                setattr(c, f"{kind}_{name}", C.cast(arr, C.POINTER(C.c_float)))
        return c, keep

    def _from_c(self, c, keep) -> None:
        for op in cabi.SCALAR_OPS:
            setattr(self, f"min_{_range_stem(op)}_", float(c.min[op]))
            setattr(self, f"max_{_range_stem(op)}_", float(c.max[op]))
        it = iter(keep)
        for name in _CHANNEL_NAMES:
            for kind in ("min", "max"):
                setattr(self, f"{kind}_{name}_", list(next(it)))


class GRUHistogramCollectors:
    """Histogram (SQNR / percentile) calibration state of one direction: one 2048-bin collector per
    activation point, per-tensor / per-gate / per-channel collectors for W, R, bw, br
    (operators/quant-gru/include/histogram_collector.h:609-720).  The counts live in host memory;
    ``forward_calibrate`` fills them from device-side binning."""

    def __init__(self, hidden: int = 0, num_bins: int = 2048):
        self._hidden, self._num_bins = int(hidden), int(num_bins)
        self._set = cabi.HistogramSet(self._hidden, self._num_bins) if self._hidden > 0 else None

    def reset(self, hidden: int = -1, num_bins: int = -1) -> None:
        if hidden > 0:
            self._hidden = int(hidden)
        if num_bins > 0:
            self._num_bins = int(num_bins)
        self._set = cabi.HistogramSet(self._hidden, self._num_bins) if self._hidden > 0 else None

    def is_valid(self) -> bool:
        return self._set is not None and self._set.is_valid()

    def hidden(self) -> int:
        return self._hidden

    def num_bins(self) -> int:
        return self._num_bins

    def histogram(self, name: str):
        """(counts, min, max, total) of the collector of an activation point, by its config name."""
        h = self._set.c.point[cabi.OP_NAMES.index(name)]
        row = cabi.OP_NAMES.index(name)
        return self._set.counts[row].copy(), h.min_val, h.max_val, int(h.total_count)

    def print(self) -> None:
        print(f"GRUHistogramCollectors: hidden={self._hidden} num_bins={self._num_bins} "
              f"is_valid={'true' if self.is_valid() else 'false'}")


class GRUQuantParams:
    """(scale, zero point) per quantization point, per-channel scale lists for W/R/bw/br
    (always 3*hidden long) and the bit-width configuration."""

    def __init__(self):
        self.hidden_ = 0
        for op in cabi.SCALAR_OPS:
            setattr(self, f"scale_{cabi.OP_NAMES[op]}_", 0.0)
            setattr(self, f"zp_{cabi.OP_NAMES[op]}_", 0)
        for name in _CHANNEL_NAMES:
            setattr(self, f"scale_{name}_", [])
        self.bitwidth_config_ = OperatorQuantConfig()

    def __setattr__(self, key, value):
        object.__setattr__(self, key, value)
        if not key.startswith("_"):
            object.__setattr__(self, "_c_copy", None)

    def _to_c(self):
        """The C struct and the arrays its pointers refer to.  The conversion is kept until an
        attribute of this object or of its bit-width configuration is assigned (as with the
        reference's bound classes, editing a returned list in place changes nothing)."""
        cfg = self.bitwidth_config_
        stamp = (id(cfg), getattr(cfg, "_version", 0))
        cached = getattr(self, "_c_copy", None)
        if cached is not None and cached[0] == stamp:
            return cached[1], cached[2]
        c, keep = self._build_c()
        object.__setattr__(self, "_c_copy", (stamp, c, keep))
        return c, keep

    def _build_c(self):
        if self.hidden_ <= 0:
            raise ValueError("GRUQuantParams hidden size must be > 0")
        n = 3 * self.hidden_
        c = cabi.QuantParams()
        c.hidden = self.hidden_
        for op in cabi.SCALAR_OPS:
            c.scale[op] = float(getattr(self, f"scale_{cabi.OP_NAMES[op]}_"))
            c.zero_point[op] = int(getattr(self, f"zp_{cabi.OP_NAMES[op]}_"))
        keep = []
        for name in _CHANNEL_NAMES:
            values = list(getattr(self, f"scale_{name}_"))
            if len(values) != n:
                raise ValueError(f"{name} per-channel scale size mismatch")
            arr = (C.c_float * n)(*values)
            keep.append(arr)
            setattr(c, f"scale_{name}", C.cast(arr, C.POINTER(C.c_float)))
        c.config = self.bitwidth_config_._to_c()
        return c, keep

    @classmethod
    def _from_c(cls, c, keep) -> "GRUQuantParams":
        out = cls()
        out.hidden_ = int(c.hidden)
        for op in cabi.SCALAR_OPS:
            setattr(out, f"scale_{cabi.OP_NAMES[op]}_", float(c.scale[op]))
            setattr(out, f"zp_{cabi.OP_NAMES[op]}_", int(c.zero_point[op]))
        for name, arr in zip(_CHANNEL_NAMES, keep):
            setattr(out, f"scale_{name}_", list(arr))
        out.bitwidth_config_ = OperatorQuantConfig._from_c(c.config)
        return out


def calculate_gru_quantitative_parameters(quant_ranges: GRUQuantizationRanges,
                                          bitwidth_config: Optional[OperatorQuantConfig] = None) -> GRUQuantParams:
    cfg = (bitwidth_config or OperatorQuantConfig())._to_c()
    ranges, keep_r = quant_ranges._to_c()
    n = 3 * quant_ranges.hidden_
    out = cabi.QuantParams()
    keep = [(C.c_float * n)() for _ in range(4)]
    for name, arr in zip(_CHANNEL_NAMES, keep):
        setattr(out, f"scale_{name}", C.cast(arr, C.POINTER(C.c_float)))
    rc = cabi.load_library().rxmet_gru_params_from_ranges(C.byref(ranges), C.byref(cfg), C.byref(out))
    if rc != 0:
        msg = cabi.load_library().rxmet_last_error().decode()
        raise RuntimeError(msg)
    del keep_r
    return GRUQuantParams._from_c(out, keep)


def calculate_gru_quantitative_parameters_from_histograms(hist_collectors, bitwidth_config=None,
                                                          use_percentile=False, percentile_value=99.99):
    """Encodings from histogram collectors: SQNR search, or percentile clipping when
    ``use_percentile`` (gru_interface_binding.cc, calculate_gru_quantitative_parameters_from_histograms)."""
    if hist_collectors is None or hist_collectors._set is None:
        raise RuntimeError("hist_collectors is invalid.")
    cfg = (bitwidth_config or OperatorQuantConfig())._to_c()
    n = 3 * hist_collectors.hidden()
    out = cabi.QuantParams()
    keep = [(C.c_float * n)() for _ in range(4)]
    for name, arr in zip(_CHANNEL_NAMES, keep):
        setattr(out, f"scale_{name}", C.cast(arr, C.POINTER(C.c_float)))
    lib = cabi.load_library()
    rc = lib.rxmet_gru_params_from_histograms(C.byref(hist_collectors._set.c), C.byref(cfg), int(bool(use_percentile)),
                                              C.c_float(percentile_value), C.byref(out))
    if rc != 0:
        raise RuntimeError(lib.rxmet_last_error().decode())
    return GRUQuantParams._from_c(out, keep)


# --------------------------------------------------------------------------
# device plumbing
# --------------------------------------------------------------------------

_workspaces = {}


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """One growing scratch buffer per device and stream, reused across calls."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def _check_f32(t: torch.Tensor, name: str, shape: Optional[Tuple[int, ...]] = None) -> torch.Tensor:
    if not (t.is_cuda and t.dtype == torch.float32):
        raise RuntimeError(f"{name} must be CUDA float32 tensor")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise RuntimeError(f"{name} must have shape {list(shape)}")
    return t.contiguous()


def _ptr(t: Optional[torch.Tensor]):
    return C.c_void_p(t.data_ptr()) if t is not None and t.numel() > 0 else None


def _stream(device) -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _common_inputs(T, B, I, H, W, R, bw, br, x, h0):
    W = _check_f32(W, "W", (I, 3 * H))
    R = _check_f32(R, "R", (H, 3 * H))
    bw = _check_f32(bw, "bw", (3 * H,))
    br = _check_f32(br, "br", (3 * H,))
    x = _check_f32(x, "x", (T, B, I))
    h0v = None
    if h0 is not None and h0.numel() > 0:
        h0v = _check_f32(h0, "h0", (B, H))
    return W, R, bw, br, x, h0v


def forward_fp(is_training, time_steps, batch_size, input_size, hidden_size, W, R, bw, br, x, h0):
    """Float forward: returns (h [T+1,B,H], v [T,B,4H])."""
    T, B, I, H = int(time_steps), int(batch_size), int(input_size), int(hidden_size)
    lib = cabi.load_library()
    W, R, bw, br, x, h0v = _common_inputs(T, B, I, H, W, R, bw, br, x, h0)
    dev = x.device
    h = torch.empty((T + 1, B, H), dtype=torch.float32, device=dev)
    v = torch.empty((T, B, 4 * H), dtype=torch.float32, device=dev)
    nbytes = lib.rxmet_gru_workspace_bytes(0, T, B, I, H)
    ws = _workspace(dev, nbytes)
    with torch.cuda.device(dev):
        cabi.check(lib.rxmet_gru_forward_fp(T, B, I, H, _ptr(W), _ptr(R), _ptr(bw), _ptr(br), _ptr(x), _ptr(h0v),
                                            _ptr(h), _ptr(v), _ptr(ws), C.c_size_t(ws.numel()), _stream(dev)),
                   "forward_fp")
    return h, v


def forward_calibrate(is_training, time_steps, batch_size, input_size, hidden_size, W, R, bw, br, x, h0,
                      calib_method, bitwidth_config, quant_ranges=None, hist_collectors=None):
    """Float forward that updates ``quant_ranges`` (calib_method 'minmax') or ``hist_collectors``
    ('sqnr' / 'percentile') in place."""
    T, B, I, H = int(time_steps), int(batch_size), int(input_size), int(hidden_size)
    method = str(calib_method).lower()
    if method == "none":
        return forward_fp(is_training, T, B, I, H, W, R, bw, br, x, h0)
    if method in ("sqnr", "percentile"):
        if hist_collectors is None:
            raise ValueError("Histogram calibration requires hist_collectors")
        lib = cabi.load_library()
        W, R, bw, br, x, h0v = _common_inputs(T, B, I, H, W, R, bw, br, x, h0)
        if hist_collectors.hidden() != H or hist_collectors._set is None:
            hist_collectors.reset(H)
        dev = x.device
        h = torch.empty((T + 1, B, H), dtype=torch.float32, device=dev)
        v = torch.empty((T, B, 4 * H), dtype=torch.float32, device=dev)
        cfg = (bitwidth_config or OperatorQuantConfig())._to_c()
        ws = _workspace(dev, lib.rxmet_gru_workspace_bytes(3, T, B, I, H))
        exchange = _exchange_for(dev)
        with torch.cuda.device(dev):
            cabi.check(lib.rxmet_gru_forward_calibrate_hist_dp(
                T, B, I, H, _ptr(W), _ptr(R), _ptr(bw), _ptr(br), _ptr(x), _ptr(h0v), _ptr(h), _ptr(v), C.byref(cfg),
                C.byref(hist_collectors._set.c), _ptr(ws), C.c_size_t(ws.numel()), _stream(dev),
                C.byref(exchange) if exchange is not None else None), "forward_calibrate")
        return h, v
    if method != "minmax":
        raise ValueError(f"unknown calib_method {calib_method!r}")
    if quant_ranges is None:
        raise ValueError("MINMAX requires quant_ranges")
    lib = cabi.load_library()
    W, R, bw, br, x, h0v = _common_inputs(T, B, I, H, W, R, bw, br, x, h0)
    if quant_ranges.hidden_ != H:
        quant_ranges.reset(H)
    dev = x.device
    h = torch.empty((T + 1, B, H), dtype=torch.float32, device=dev)
    v = torch.empty((T, B, 4 * H), dtype=torch.float32, device=dev)
    ranges, keep = quant_ranges._to_c()
    nbytes = lib.rxmet_gru_workspace_bytes(0, T, B, I, H)
    ws = _workspace(dev, nbytes)
    if _calibration_group is not None:
        # sharded batch: the packed extremes of this rank's shard are all-reduced before they are folded
        import torch.distributed as dist
        stats = torch.empty(lib.rxmet_gru_stats_floats(H), dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            cabi.check(lib.rxmet_gru_forward_calibrate_stats(
                T, B, I, H, _ptr(W), _ptr(R), _ptr(bw), _ptr(br), _ptr(x), _ptr(h0v), _ptr(h), _ptr(v), _ptr(stats),
                _ptr(ws), C.c_size_t(ws.numel()), _stream(dev)), "forward_calibrate")
        half = stats.numel() // 2
        dist.all_reduce(stats[:half], op=dist.ReduceOp.MIN, group=_calibration_group)
        dist.all_reduce(stats[half:], op=dist.ReduceOp.MAX, group=_calibration_group)
        host = stats.cpu().contiguous()
        cabi.check(lib.rxmet_gru_ranges_fold_stats(C.byref(ranges), C.cast(host.data_ptr(), C.POINTER(C.c_float))),
                   "ranges_fold_stats")
    else:
        with torch.cuda.device(dev):
            cabi.check(lib.rxmet_gru_forward_calibrate_minmax(
                T, B, I, H, _ptr(W), _ptr(R), _ptr(bw), _ptr(br), _ptr(x), _ptr(h0v), _ptr(h), _ptr(v),
                C.byref(ranges), _ptr(ws), C.c_size_t(ws.numel()), _stream(dev)), "forward_calibrate")
    quant_ranges._from_c(ranges, keep)
    return h, v


_MASK_SHAPES = lambda T, B, I, H: {  # noqa: E731
    "x": (T, B, I), "h0": (B, H), "W": (I, 3 * H), "R": (H, 3 * H), "bw": (3 * H,), "br": (3 * H,),
    "weight_ih_linear": (T, B, 3 * H), "weight_hh_linear": (T, B, 3 * H), "gate_input": (T, B, 3 * H),
    "gate_output": (T, B, 3 * H), "h": (T, B, H)}


def _carve(device, dtype, shapes):
    """Tensors of the given shapes as views of ONE allocation (each starts on a 16-byte boundary):
    a forward call returns 16 small tensors, and one allocator round trip per tensor is host time
    on the critical path of a training step."""
    item = torch.empty((), dtype=dtype).element_size()
    per = 16 // item
    counts = [1 if not shape else int(torch.Size(shape).numel()) for shape in shapes]
    offsets, total = [], 0
    for n in counts:
        offsets.append(total)
        total += (n + per - 1) // per * per
    pool = torch.empty((max(total, 1),), dtype=dtype, device=device)
    return [pool[o:o + n].view(shape) for o, n, shape in zip(offsets, counts, shapes)]


_FLOAT_STORAGE_CARRIERS = ("integer", "fp32")
_float_storage_carrier = "integer"


def set_float_storage_carrier(carrier):
    """Choose what forward_quant_float_storage computes with; returns the previous choice.

    "integer" (default): the integer carrier, the same arithmetic as forward_quant_int_storage and as the
    reference's CPU build (src/quantize_ops_helper.h: multiply, add, rounding right shift), so the two storage
    modes return the same codes.  "fp32": the reference's CUDA float-code arithmetic
    (src/gru_forward_gpu_quant_fp.cu: codes held in float, rescales as rintf(x * ratio), float tables), bit
    for bit what the reference's CUDA kernels return while the integer matrix sums stay below 2^24."""
    global _float_storage_carrier
    if carrier not in _FLOAT_STORAGE_CARRIERS:
        raise ValueError(f"carrier must be one of {_FLOAT_STORAGE_CARRIERS}, got {carrier!r}")
    previous, _float_storage_carrier = _float_storage_carrier, carrier
    return previous


def float_storage_carrier():
    return _float_storage_carrier


def _forward_quant(is_training, T, B, I, H, W, R, bw, br, x, h0, quant_params, code_dtype, fp_carrier=False):
    lib = cabi.load_library()
    W, R, bw, br, x, h0v = _common_inputs(T, B, I, H, W, R, bw, br, x, h0)
    dev = x.device
    params, keep = quant_params._to_c()
    h = torch.empty((T + 1, B, H), dtype=torch.float32, device=dev)
    v = torch.empty((T, B, 4 * H), dtype=torch.float32, device=dev)
    code_shapes = {"W_q": (I, 3 * H), "R_q": (H, 3 * H), "bw_q": (3 * H,), "br_q": (3 * H,), "x_q": (T, B, I)}
    codes = dict(zip(code_shapes, _carve(dev, torch.int32, list(code_shapes.values()))))
    mask_struct = cabi.Masks()
    shapes = _MASK_SHAPES(T, B, I, H)
    wanted = [name for name in shapes if is_training and not (name == "h0" and h0v is None)]
    masks = dict(zip(wanted, _carve(dev, torch.uint8, [shapes[name] for name in wanted]))) if wanted else {}
    empty = None
    for name in shapes:
        if name in masks:
            setattr(mask_struct, name, masks[name].data_ptr())
        else:
            if empty is None:
                empty = torch.empty((0,), dtype=torch.uint8, device=dev)
            masks[name] = empty
    ws = _workspace(dev, lib.rxmet_gru_workspace_bytes(1, T, B, I, H))
    with torch.cuda.device(dev):
        entry = lib.rxmet_gru_forward_quant_fp_carrier if fp_carrier else lib.rxmet_gru_forward_quant
        cabi.check(entry(
            int(bool(is_training)), T, B, I, H, _ptr(W), _ptr(R), _ptr(bw), _ptr(br), _ptr(x), _ptr(h0v),
            C.byref(params), _ptr(h), _ptr(v), _ptr(codes["W_q"]), _ptr(codes["R_q"]), _ptr(codes["bw_q"]),
            _ptr(codes["br_q"]), _ptr(codes["x_q"]), None, None,
            C.byref(mask_struct) if is_training else None, _ptr(ws), C.c_size_t(ws.numel()), _stream(dev)),
            "forward_quant")
    del keep
    if code_dtype != torch.int32:
        codes = {k: t.to(code_dtype) for k, t in codes.items()}
    return (h, v, codes["W_q"], codes["R_q"], codes["bw_q"], codes["br_q"], codes["x_q"],
            masks["x"], masks["h0"], masks["W"], masks["R"], masks["bw"], masks["br"],
            masks["weight_ih_linear"], masks["weight_hh_linear"], masks["gate_input"], masks["gate_output"],
            masks["h"])


def forward_quant_int_storage(is_training, time_steps, batch_size, input_size, hidden_size, W, R, bw, br, x, h0,
                              quant_params):
    """18-tuple (h, v, W_q, R_q, bw_q, br_q, x_q, 11 masks); code caches are int32."""
    return _forward_quant(is_training, int(time_steps), int(batch_size), int(input_size), int(hidden_size),
                          W, R, bw, br, x, h0, quant_params, torch.int32)


def forward_quant_float_storage(is_training, time_steps, batch_size, input_size, hidden_size, W, R, bw, br, x, h0,
                                quant_params):
    """Same tuple with the code caches stored as float32 (values are still integers); computed with the
    carrier set_float_storage_carrier selected."""
    return _forward_quant(is_training, int(time_steps), int(batch_size), int(input_size), int(hidden_size),
                          W, R, bw, br, x, h0, quant_params, torch.float32,
                          fp_carrier=_float_storage_carrier == "fp32")


def forward_quantized_int_io(time_steps, batch_size, input_size, hidden_size, W, R, bw, br, x_q, h0_q, quant_params):
    """Integer in / integer out inference: returns (output_q [T,B,H], h_n_q [1,B,H]) int32."""
    T, B, I, H = int(time_steps), int(batch_size), int(input_size), int(hidden_size)
    lib = cabi.load_library()
    W = _check_f32(W, "W", (I, 3 * H)); R = _check_f32(R, "R", (H, 3 * H))
    bw = _check_f32(bw, "bw", (3 * H,)); br = _check_f32(br, "br", (3 * H,))
    if not (x_q.is_cuda and x_q.dtype == torch.int32) or tuple(x_q.shape) != (T, B, I):
        raise RuntimeError("x_q must be CUDA int32 tensor of shape [T, B, I]")
    x_q = x_q.contiguous()
    h0v = None
    if h0_q is not None and h0_q.numel() > 0:
        if not (h0_q.is_cuda and h0_q.dtype == torch.int32) or tuple(h0_q.shape) != (B, H):
            raise RuntimeError("h0_q must be CUDA int32 tensor of shape [B, H]")
        h0v = h0_q.contiguous()
    dev = x_q.device
    params, keep = quant_params._to_c()
    h_q = torch.empty((T + 1, B, H), dtype=torch.int32, device=dev)
    extra = 4 * ((T + 1) * B * H + T * B * 4 * H) + 1024
    ws = _workspace(dev, lib.rxmet_gru_workspace_bytes(1, T, B, I, H) + extra)
    with torch.cuda.device(dev):
        cabi.check(lib.rxmet_gru_forward_quant_int_io(
            T, B, I, H, _ptr(W), _ptr(R), _ptr(bw), _ptr(br), _ptr(x_q), _ptr(h0v), C.byref(params), _ptr(h_q),
            _ptr(ws), C.c_size_t(ws.numel()), _stream(dev)), "forward_quantized_int_io")
    del keep
    return h_q[1:], h_q[-1:]


def _backward_quant(T, B, I, H, W_q, R_q, bw_q, br_q, x_q, dh_new, h, v, quant_params, masks: List[torch.Tensor]):
    lib = cabi.load_library()
    dev = h.device
    codes = []
    for t, name, shape in ((W_q, "W_q", (I, 3 * H)), (R_q, "R_q", (H, 3 * H)), (bw_q, "bw_q", (3 * H,)),
                           (br_q, "br_q", (3 * H,)), (x_q, "x_q", (T, B, I))):
        if not t.is_cuda or tuple(t.shape) != shape:
            raise RuntimeError(f"{name} must be a CUDA tensor of shape {list(shape)}")
        codes.append(t.to(torch.int32).contiguous())
    dh_new = _check_f32(dh_new, "dh_new", (T + 1, B, H))
    h = _check_f32(h, "h", (T + 1, B, H))
    v = _check_f32(v, "v", (T, B, 4 * H))
    params, keep = quant_params._to_c()
    mask_struct = cabi.Masks()
    live = []
    for name, m in zip(cabi.MASK_NAMES, masks):
        if m is not None and m.numel() > 0:
            m = m.contiguous()
            live.append(m)
            setattr(mask_struct, name, m.data_ptr())
    dx, dW, dR, dbw, dbr, dh0 = _carve(dev, torch.float32,
                                       [(T, B, I), (I, 3 * H), (H, 3 * H), (3 * H,), (3 * H,), (B, H)])
    ws = _workspace(dev, lib.rxmet_gru_workspace_bytes(2, T, B, I, H))
    with torch.cuda.device(dev):
        cabi.check(lib.rxmet_gru_backward_quant(
            T, B, I, H, _ptr(codes[0]), _ptr(codes[1]), _ptr(codes[2]), _ptr(codes[3]), _ptr(codes[4]),
            _ptr(dh_new), _ptr(h), _ptr(v), C.byref(params), C.byref(mask_struct),
            _ptr(dx), _ptr(dW), _ptr(dR), _ptr(dbw), _ptr(dbr), _ptr(dh0),
            _ptr(ws), C.c_size_t(ws.numel()), _stream(dev)), "backward_quant")
    del keep, live
    return dx, dW, dR, dbw, dbr, dh0


def backward_quant_int_storage(time_steps, batch_size, input_size, hidden_size, W_q, R_q, bw_q, br_q, x_q, dh_new,
                               h, v, quant_params, x_mask, h0_mask, W_mask, R_mask, bw_mask, br_mask,
                               weight_ih_linear_mask, weight_hh_linear_mask, gate_input_mask, gate_output_mask,
                               h_mask):
    """QAT backward from int32 code caches: (dx, dW, dR, dbw, dbr, dh)."""
    return _backward_quant(int(time_steps), int(batch_size), int(input_size), int(hidden_size), W_q, R_q, bw_q,
                           br_q, x_q, dh_new, h, v, quant_params,
                           [x_mask, h0_mask, W_mask, R_mask, bw_mask, br_mask, weight_ih_linear_mask,
                            weight_hh_linear_mask, gate_input_mask, gate_output_mask, h_mask])


def backward_quant_float_storage(time_steps, batch_size, input_size, hidden_size, W_q, R_q, bw_q, br_q, x_q,
                                 dh_new, h, v, quant_params, x_mask, h0_mask, W_mask, R_mask, bw_mask, br_mask,
                                 weight_ih_linear_mask, weight_hh_linear_mask, gate_input_mask, gate_output_mask,
                                 h_mask):
    """QAT backward from float32 code caches.  Unlike the reference, the saved caches are not
    overwritten, so a second backward through the same graph sees the same inputs."""
    return _backward_quant(int(time_steps), int(batch_size), int(input_size), int(hidden_size), W_q, R_q, bw_q,
                           br_q, x_q, dh_new, h, v, quant_params,
                           [x_mask, h0_mask, W_mask, R_mask, bw_mask, br_mask, weight_ih_linear_mask,
                            weight_hh_linear_mask, gate_input_mask, gate_output_mask, h_mask])


def backward_fp(time_steps, batch_size, input_size, hidden_size, W, R, bw, br, x, dh_new, h, v):
    """Float backward: (dx, dW, dR, dbw, dbr, dh)."""
    T, B, I, H = int(time_steps), int(batch_size), int(input_size), int(hidden_size)
    lib = cabi.load_library()
    W, R, bw, br, x, _ = _common_inputs(T, B, I, H, W, R, bw, br, x, None)
    dh_new = _check_f32(dh_new, "dh_new", (T + 1, B, H))
    h = _check_f32(h, "h", (T + 1, B, H))
    v = _check_f32(v, "v", (T, B, 4 * H))
    dev = x.device
    dx, dW, dR, dbw, dbr, dh0 = _carve(dev, torch.float32,
                                       [(T, B, I), (I, 3 * H), (H, 3 * H), (3 * H,), (3 * H,), (B, H)])
    ws = _workspace(dev, lib.rxmet_gru_workspace_bytes(2, T, B, I, H))
    with torch.cuda.device(dev):
        cabi.check(lib.rxmet_gru_backward_fp(
            T, B, I, H, _ptr(W), _ptr(R), _ptr(bw), _ptr(br), _ptr(x), _ptr(dh_new), _ptr(h), _ptr(v),
            _ptr(dx), _ptr(dW), _ptr(dR), _ptr(dbw), _ptr(dbr), _ptr(dh0),
            _ptr(ws), C.c_size_t(ws.numel()), _stream(dev)), "backward_fp")
    return dx, dW, dR, dbw, dbr, dh0
