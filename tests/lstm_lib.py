"""numpy wrappers over the QuantLSTM parity checkers (test infrastructure).

``orc`` = plain-C restatement in ``oracle/librxmet_oracle.so``; ``ref`` = the reference's own CPU
sources in ``oracle/_ref/liblstm_ref.so`` (only where it was built).  Both export the same entry
points under the two prefixes.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

import oracle_lib
from rx_met_b200 import _cabi_lstm as L

LSTM_REF_SO = oracle_lib.ROOT / "oracle" / "_ref" / "liblstm_ref.so"
_f32p = C.POINTER(C.c_float)
_u8p = C.POINTER(C.c_uint8)
_ref = None


def _fp(a):
    return None if a is None else a.ctypes.data_as(_f32p)


def _up(a):
    return None if a is None else a.ctypes.data_as(_u8p)


def lib(prefix: str):
    global _ref
    if prefix == "orc":
        return oracle_lib.oracle()
    if _ref is None and LSTM_REF_SO.exists():
        _ref = C.CDLL(str(LSTM_REF_SO))
        _ref.ref_lstm_last_error.restype = C.c_char_p
    return _ref


def have_ref() -> bool:
    return lib("ref") is not None


def _call(prefix, name, *args):
    fn = getattr(lib(prefix), f"{prefix}_lstm_{name}")
    fn.restype = C.c_int
    rc = fn(*args)
    if rc != 0:
        msg = lib("ref").ref_lstm_last_error().decode(errors="replace") if prefix == "ref" else ""
        raise RuntimeError(f"{prefix}_lstm_{name} failed: {msg}")


def problem(T, B, I, H, seed=0, bias=True, state=True, wscale=0.3):
    rng = np.random.default_rng(seed)
    f = lambda *s: rng.standard_normal(s).astype(np.float32)
    p = dict(T=T, B=B, I=I, H=H, x=f(T, B, I), w_ih=f(4 * H, I) * wscale, w_hh=f(4 * H, H) * wscale,
             b_ih=f(4 * H) * 0.1 if bias else None, b_hh=f(4 * H) * 0.1 if bias else None,
             h0=f(B, H) * 0.5 if state else None, c0=f(B, H) * 0.5 if state else None)
    return p


def forward_float(prefix, p):
    T, B, I, H = p["T"], p["B"], p["I"], p["H"]
    out = np.zeros((T, B, H), np.float32)
    hn, cn = np.zeros((B, H), np.float32), np.zeros((B, H), np.float32)
    tr = {n: np.zeros((T, B, 4 * H if i < 4 else H), np.float32) for i, n in enumerate(L.TRACE_VALUES)}
    _call(prefix, "forward_float", T, B, I, H, _fp(p["w_ih"]), _fp(p["w_hh"]), _fp(p["b_ih"]), _fp(p["b_hh"]),
          _fp(p["x"]), _fp(p["h0"]), _fp(p["c0"]), _fp(out), _fp(hn), _fp(cn), *[_fp(tr[n]) for n in L.TRACE_VALUES])
    return out, hn, cn, tr


def backward_float(prefix, p, tr, g_out, g_hn, g_cn, masks: dict | None = None):
    T, B, I, H = p["T"], p["B"], p["I"], p["H"]
    g = dict(input=np.zeros((T, B, I), np.float32), weight_ih=np.zeros((4 * H, I), np.float32),
             weight_hh=np.zeros((4 * H, H), np.float32), bias_ih=np.zeros(4 * H, np.float32),
             bias_hh=np.zeros(4 * H, np.float32), initial_hidden=np.zeros((B, H), np.float32),
             initial_cell=np.zeros((B, H), np.float32))
    head = [T, B, I, H, _fp(p["w_ih"]), _fp(p["w_hh"]), _fp(p["x"]), _fp(p["h0"]), _fp(p["c0"]),
            _fp(tr["gate_outputs"]), _fp(tr["cell_states"]), _fp(tr["cell_tanh_outputs"]), _fp(tr["hidden_outputs"]),
            _fp(g_out), _fp(g_hn), _fp(g_cn)]
    tail = [_fp(g[n]) for n in L.MASTER_VALUES]
    if masks is None:
        _call(prefix, "backward_float", *head, *tail)
    else:
        m = L.BackwardMasks()
        for n, _ in L.BackwardMasks._fields_:
            a = masks.get(n)
            setattr(m, n, None if a is None else a.ctypes.data)
        _call(prefix, "backward_float_masked", *head, C.byref(m), *tail)
    return g


def params_from_ranges(prefix, cfg, ranges: L.RangesBox, I, H, bias) -> L.ParamsBox:
    box = L.ParamsBox(H)
    _call(prefix, "params_from_ranges", C.byref(cfg), C.byref(ranges.struct), I, H, int(bias), *box.scale_ptrs(),
          C.byref(box.struct))
    box.bind()
    return box


def derive(prefix, params: L.ParamsBox, exact=False) -> L.ExecutionBox:
    box = L.ExecutionBox(params.H)
    _call(prefix, "derive_execution", C.byref(params.struct), int(exact), C.byref(box.struct))
    return box


def calibrate(prefix, cfg, p, batches_x: np.ndarray):
    """batches_x: [N,T,B,I].  Returns (RangesBox, ParamsBox)."""
    T, B, I, H = p["T"], p["B"], p["I"], p["H"]
    ranges, box = L.RangesBox(H), L.ParamsBox(H)
    _call(prefix, "calibrate_minmax", C.byref(cfg), batches_x.shape[0], T, B, I, H, _fp(p["w_ih"]), _fp(p["w_hh"]),
          _fp(p["b_ih"]), _fp(p["b_hh"]), _fp(np.ascontiguousarray(batches_x)), _fp(p["h0"]), _fp(p["c0"]),
          C.byref(ranges.struct), *box.scale_ptrs(), C.byref(box.struct))
    box.bind()
    return ranges, box


def quantize(prefix, src, scales, zp, cfg, op, row_width=0):
    src = np.ascontiguousarray(src, np.float32)
    dst = np.zeros_like(src)
    scales = np.ascontiguousarray(np.atleast_1d(scales), np.float32)
    _call(prefix, "quantize", _fp(src), C.c_longlong(src.size), C.c_longlong(row_width), _fp(scales), int(zp),
          int(cfg.bitwidth[op]), int(cfg.is_unsigned[op]), int(cfg.is_symmetric[op]), _fp(dst))
    return dst


def quantize_masked(src, scales, zp, cfg, op, row_width=0):
    src = np.ascontiguousarray(src, np.float32)
    dst, mask = np.zeros_like(src), np.zeros(src.shape, np.uint8)
    scales = np.ascontiguousarray(np.atleast_1d(scales), np.float32)
    _call("orc", "quantize_masked", _fp(src), C.c_longlong(src.size), C.c_longlong(row_width), _fp(scales), int(zp),
          int(cfg.bitwidth[op]), int(cfg.is_unsigned[op]), _fp(dst), _up(mask))
    return dst, mask


def dequantize(src, scales, zp, row_width=0):
    src = np.ascontiguousarray(src, np.float32)
    dst = np.zeros_like(src)
    scales = np.ascontiguousarray(np.atleast_1d(scales), np.float32)
    _call("orc", "dequantize", _fp(src), C.c_longlong(src.size), C.c_longlong(row_width), _fp(scales), int(zp), _fp(dst))
    return dst


def quantize_masters(prefix, p, params: L.ParamsBox, with_masks=False):
    """Float masters -> q-carrier copies (as the reference's binding does before its core runs,
    operators/quant-lstm/pytorch/lib/lstm_interface_binding_cpu.cc:215-233)."""
    s, cfg = params.struct, params.struct.config
    I, H = p["I"], p["H"]
    spec = [("x", L.INPUT, [s.scale[L.INPUT]], s.zero_point[L.INPUT], 0),
            ("w_ih", L.WEIGHT_IH, params.channel_scales[0], 0, I), ("w_hh", L.WEIGHT_HH, params.channel_scales[1], 0, H),
            ("b_ih", L.BIAS_IH, params.channel_scales[2], 0, 1), ("b_hh", L.BIAS_HH, params.channel_scales[3], 0, 1),
            ("h0", L.OUTPUT, [s.scale[L.OUTPUT]], s.zero_point[L.OUTPUT], 0),
            ("c0", L.CELL_STATE, [s.scale[L.CELL_STATE]], s.zero_point[L.CELL_STATE], 0)]
    q, masks = {}, {}
    for name, op, scales, zp, rw in spec:
        if p[name] is None:
            q[name] = None
            masks[name] = None
        elif with_masks:
            q[name], masks[name] = quantize_masked(p[name], scales, zp, cfg, op, rw)
        else:
            q[name] = quantize(prefix, p[name], scales, zp, cfg, op, rw)
    return (q, masks) if with_masks else q


def forward_quantized(prefix, params: L.ParamsBox, T, B, q, exact=False):
    H = params.H
    out = np.zeros((T, B, H), np.float32)
    hn, cn = np.zeros((B, H), np.float32), np.zeros((B, H), np.float32)
    tr = {n: np.zeros((T, B, 4 * H if i < 4 else H), np.float32) for i, n in enumerate(L.TRACE_VALUES)}
    _call(prefix, "forward_quantized", C.byref(params.struct), int(exact), T, B, _fp(q["w_ih"]), _fp(q["w_hh"]),
          _fp(q["b_ih"]), _fp(q["b_hh"]), _fp(q["x"]), _fp(q["h0"]), _fp(q["c0"]), _fp(out), _fp(hn), _fp(cn),
          *[_fp(tr[n]) for n in L.TRACE_VALUES])
    return out, hn, cn, tr


def forward_int32(params: L.ParamsBox, T, B, q):
    """The reference's exact integer forward (lstmForwardInt32CpuReference) on q-carrier inputs; codes come
    back as floats.  Returns (out, hn, cn, trace)."""
    H = params.H
    out = np.zeros((T, B, H), np.float32)
    hn, cn = np.zeros((B, H), np.float32), np.zeros((B, H), np.float32)
    tr = {n: np.zeros((T, B, 4 * H if i < 4 else H), np.float32) for i, n in enumerate(L.TRACE_VALUES)}
    _call("ref", "forward_int32", C.byref(params.struct), T, B, _fp(q["w_ih"]), _fp(q["w_hh"]), _fp(q["b_ih"]),
          _fp(q["b_hh"]), _fp(q["x"]), _fp(q["h0"]), _fp(q["c0"]), _fp(out), _fp(hn), _fp(cn),
          *[_fp(tr[n]) for n in L.TRACE_VALUES])
    return out, hn, cn, tr


def forward_quantized_masked(params: L.ParamsBox, T, B, q, exact_sums=False):
    """Oracle only: q-carrier forward that also returns the seven clamp masks.  `exact_sums` accumulates the
    two linear stages exactly (the CUDA library's arithmetic) instead of in sequential float additions."""
    H = params.H
    out = np.zeros((T, B, H), np.float32)
    hn, cn = np.zeros((B, H), np.float32), np.zeros((B, H), np.float32)
    tr = {n: np.zeros((T, B, 4 * H if i < 4 else H), np.float32) for i, n in enumerate(L.TRACE_VALUES)}
    mk = {n: np.zeros((T, B, 4 * H if i < 4 else H), np.uint8) for i, n in enumerate(L.TRACE_VALUES)}
    t = L.Trace()
    for n in L.TRACE_VALUES:
        setattr(t, n, tr[n].ctypes.data)
        setattr(t, n + "_clamped", mk[n].ctypes.data)
    _call("orc", "forward_quantized_exact_sums" if exact_sums else "forward_quantized_masked", C.byref(params.struct), T, B,
          _fp(q["w_ih"]), _fp(q["w_hh"]),
          _fp(q["b_ih"]), _fp(q["b_hh"]), _fp(q["x"]), _fp(q["h0"]), _fp(q["c0"]), _fp(out), _fp(hn), _fp(cn),
          C.byref(t))
    return out, hn, cn, tr, mk


def stage(params: L.ParamsBox, which: int, rows: int, a, b=None, c=None, out_shape=None):
    """One stage of the oracle on given q-carrier inputs; returns (values, clamp mask)."""
    out = np.zeros(out_shape, np.float32)
    mask = np.zeros(out_shape, np.uint8)
    cont = lambda v: None if v is None else np.ascontiguousarray(v, np.float32)
    a, b, c = cont(a), cont(b), cont(c)
    _call("orc", "stage", C.byref(params.struct), which, C.c_longlong(rows), _fp(a), _fp(b), _fp(c), _fp(out), _up(mask))
    return out, mask


def calibrate_hist(cfg, p, batches_x: np.ndarray, method: str, percentile: float, bins: int = 2048):
    """Reference calibration session with a histogram method.  Returns (HistogramSet, ParamsBox)."""
    T, B, I, H = p["T"], p["B"], p["I"], p["H"]
    hs, box = L.HistogramSet(H, bins), L.ParamsBox(H)
    _call("ref", "calibrate_hist", C.byref(cfg), 1 if method == "sqnr" else 2, C.c_float(percentile), batches_x.shape[0],
          T, B, I, H, _fp(p["w_ih"]), _fp(p["w_hh"]), _fp(p["b_ih"]), _fp(p["b_hh"]), _fp(np.ascontiguousarray(batches_x)),
          _fp(p["h0"]), _fp(p["c0"]), C.byref(hs.struct), *box.scale_ptrs(), C.byref(box.struct))
    box.bind()
    return hs, box
