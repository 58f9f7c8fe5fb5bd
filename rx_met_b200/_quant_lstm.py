"""Drop-in for the reference's ``_quant_lstm`` extension module
(operators/quant-lstm/pytorch/lib/lstm_interface_binding.cc:917-978): same function names,
argument order, return tuples and error types, implemented over ``librxmet_b200.so``.

Every function takes CUDA float32 tensors and enqueues on torch's current stream.  There is no
CPU implementation behind this module: a missing library or a CPU tensor raises.
"""
from __future__ import annotations

import ctypes as C
import json
from typing import Optional, Sequence

import numpy as np
import torch

from . import _cabi
from . import _cabi_lstm as L

_lib = None


def _library():
    global _lib
    if _lib is None:
        lib = _cabi.load_library()
        lib.rxmet_lstm_workspace_bytes.restype = C.c_size_t
        lib.rxmet_lstm_workspace_bytes.argtypes = [C.c_int] * 5
        lib.rxmet_lstm_stats_floats.restype = C.c_size_t
        lib.rxmet_lstm_stats_floats.argtypes = [C.c_int]
        _lib = lib
    return _lib


def _check(rc: int, invalid=ValueError):
    if rc == 0:
        return
    msg = _library().rxmet_last_error().decode(errors="replace")
    raise (invalid if rc == -1 else RuntimeError)(msg)


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None or t.numel() == 0 else C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _workspace(op, T, B, I, H, device):
    n = _library().rxmet_lstm_workspace_bytes(op, T, B, I, H)
    return torch.empty(n, dtype=torch.uint8, device=device), n


# --------------------------------------------------------------------------
# argument preparation (prepareForward, lstm_interface_binding.cc:86-170)
# --------------------------------------------------------------------------

def _float_cuda(t: torch.Tensor, name: str) -> torch.Tensor:
    if not isinstance(t, torch.Tensor) or t.dtype != torch.float32:
        raise RuntimeError(f"{name} must be a float32 tensor")
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    return t.contiguous()


class _Prepared:
    def __init__(self, input, weight_ih, weight_hh, bias_ih, bias_hh, initial_hidden, initial_cell, batch_first):
        x = _float_cuda(input, "input")
        if x.dim() != 3:
            raise RuntimeError("input must have 3 dimensions")
        self.x = (x.transpose(0, 1) if batch_first else x).contiguous()
        self.T, self.B, self.I = self.x.shape
        self.w_ih = _float_cuda(weight_ih, "weight_ih")
        self.w_hh = _float_cuda(weight_hh, "weight_hh")
        if self.w_ih.dim() != 2 or self.w_hh.dim() != 2 or self.w_ih.shape[0] % 4 != 0:
            raise RuntimeError("weights must be [4H, I] and [4H, H]")
        self.H = self.w_ih.shape[0] // 4
        if tuple(self.w_ih.shape) != (4 * self.H, self.I) or tuple(self.w_hh.shape) != (4 * self.H, self.H):
            raise RuntimeError("weight shapes do not match input_size / hidden_size")
        if (bias_ih is None) != (bias_hh is None):
            raise RuntimeError("bias_ih and bias_hh must be given together")
        self.b_ih = None if bias_ih is None else _float_cuda(bias_ih, "bias_ih")
        self.b_hh = None if bias_hh is None else _float_cuda(bias_hh, "bias_hh")
        for b in (self.b_ih, self.b_hh):
            if b is not None and tuple(b.shape) != (4 * self.H,):
                raise RuntimeError("bias must be [4H]")
        if (initial_hidden is None) != (initial_cell is None):
            raise RuntimeError("initial_hidden and initial_cell must be given together")
        self.h0 = self.c0 = None
        if initial_hidden is not None:
            self.h0 = _float_cuda(initial_hidden, "initial_hidden").reshape(self.B, self.H).contiguous()
            self.c0 = _float_cuda(initial_cell, "initial_cell").reshape(self.B, self.H).contiguous()
        self.device = self.x.device

    def empty(self, *shape, dtype=torch.float32):
        return torch.empty(shape, dtype=dtype, device=self.device)

    def dims(self):
        return self.T, self.B, self.I, self.H


def _trace_struct(tensors: dict, masks: dict | None = None) -> L.Trace:
    t = L.Trace()
    for n in L.TRACE_VALUES:
        if n in tensors:
            setattr(t, n, tensors[n].data_ptr())
        if masks and n in masks:
            setattr(t, n + "_clamped", masks[n].data_ptr())
    return t


def _run_float(p: _Prepared, trace: Optional[dict], stats: Optional[torch.Tensor]):
    lib = _library()
    T, B, I, H = p.dims()
    out, hn, cn = p.empty(T, B, H), p.empty(1, B, H), p.empty(1, B, H)
    ws, n = _workspace(0, T, B, I, H, p.device)
    with torch.cuda.device(p.device):
        if stats is None:
            tr = _trace_struct(trace) if trace else None
            rc = lib.rxmet_lstm_forward_float(T, B, I, H, _ptr(p.w_ih), _ptr(p.w_hh), _ptr(p.b_ih), _ptr(p.b_hh),
                                              _ptr(p.x), _ptr(p.h0), _ptr(p.c0), _ptr(out), _ptr(hn), _ptr(cn),
                                              C.byref(tr) if tr is not None else None, _ptr(ws), C.c_size_t(n), _stream())
        else:
            rc = lib.rxmet_lstm_forward_calibrate_stats(T, B, I, H, _ptr(p.w_ih), _ptr(p.w_hh), _ptr(p.b_ih),
                                                        _ptr(p.b_hh), _ptr(p.x), _ptr(p.h0), _ptr(p.c0), _ptr(out),
                                                        _ptr(hn), _ptr(cn), _ptr(stats), _ptr(ws), C.c_size_t(n), _stream())
    _check(rc, RuntimeError)
    return out, hn, cn


def lstm_forward(input, weight_ih, weight_hh, bias_ih=None, bias_hh=None, initial_hidden=None, initial_cell=None,
                 batch_first=False):
    """Float forward: (output, h_n [1,B,H], c_n [1,B,H])."""
    p = _Prepared(input, weight_ih, weight_hh, bias_ih, bias_hh, initial_hidden, initial_cell, batch_first)
    out, hn, cn = _run_float(p, None, None)
    return (out.transpose(0, 1) if batch_first else out), hn, cn


def lstm_forward_training(input, weight_ih, weight_hh, bias_ih=None, bias_hh=None, initial_hidden=None,
                          initial_cell=None, batch_first=False):
    """Float forward that also returns the tensors the backward needs:
    (output, h_n, c_n, gate_outputs, cell_states, cell_tanh_outputs, hidden_outputs)."""
    p = _Prepared(input, weight_ih, weight_hh, bias_ih, bias_hh, initial_hidden, initial_cell, batch_first)
    T, B, I, H = p.dims()
    tr = {"gate_outputs": p.empty(T, B, 4 * H), "cell_states": p.empty(T, B, H), "cell_tanh_outputs": p.empty(T, B, H)}
    out, hn, cn = _run_float(p, tr, None)
    hidden = out
    return ((out.transpose(0, 1) if batch_first else out), hn, cn, tr["gate_outputs"], tr["cell_states"],
            tr["cell_tanh_outputs"], hidden)


def _mask_tensor(t: torch.Tensor, name: str, shape, device, allow_empty=False):
    if t.dtype not in (torch.bool, torch.uint8):
        raise RuntimeError(f"{name} must be a bool or uint8 tensor")
    if t.device != device:
        raise RuntimeError(f"{name} is on another device")
    if allow_empty and t.numel() == 0:
        return None
    if tuple(t.shape) != tuple(shape):
        raise RuntimeError(f"{name} shape mismatch")
    t = t.contiguous()
    return t.view(torch.uint8) if t.dtype == torch.bool else t


def _backward(p: _Prepared, batch_first, trace4, grad_output, grad_final_hidden, grad_final_cell, master_masks,
              checkpoint_masks, input_shape, params: Optional[L.ParamsBox]):
    lib = _library()
    T, B, I, H = p.dims()

    def shaped(t, name, shape):
        t = _float_cuda(t, name)
        if tuple(t.shape) != tuple(shape):
            raise RuntimeError(f"{name} shape mismatch")
        return t

    gates = shaped(trace4[0], "gate_outputs", (T, B, 4 * H))
    cells = shaped(trace4[1], "cell_states", (T, B, H))
    ctanh = shaped(trace4[2], "cell_tanh_outputs", (T, B, H))
    hidden = shaped(trace4[3], "hidden_outputs", (T, B, H))
    g_out = shaped(grad_output, "grad_output", (T, B, H))
    g_hn = shaped(grad_final_hidden, "grad_final_hidden", (B, H))
    g_cn = shaped(grad_final_cell, "grad_final_cell", (B, H))
    if bool(master_masks) != bool(checkpoint_masks):
        raise RuntimeError("master_masks and checkpoint_masks must be given together")
    mk, keep = None, []
    if master_masks:
        if len(master_masks) != 7 or len(checkpoint_masks) != 7:
            raise RuntimeError("master_masks and checkpoint_masks must hold 7 tensors each")
        mk = L.BackwardMasks()
        m0 = _mask_tensor(master_masks[0], "input_mask", input_shape, p.device)
        if batch_first:
            m0 = m0.transpose(0, 1).contiguous()
        prepared = [m0,
                    _mask_tensor(master_masks[1], "weight_ih_mask", p.w_ih.shape, p.device),
                    _mask_tensor(master_masks[2], "weight_hh_mask", p.w_hh.shape, p.device),
                    _mask_tensor(master_masks[3], "bias_ih_mask", (4 * H,), p.device, allow_empty=True),
                    _mask_tensor(master_masks[4], "bias_hh_mask", (4 * H,), p.device, allow_empty=True),
                    _mask_tensor(master_masks[5], "initial_hidden_mask", (1, B, H), p.device),
                    _mask_tensor(master_masks[6], "initial_cell_mask", (1, B, H), p.device)]
        for i, n in enumerate(L.TRACE_VALUES):
            prepared.append(_mask_tensor(checkpoint_masks[i], n + "_mask", (T, B, 4 * H if i < 4 else H), p.device))
        for n, t in zip(L.MASTER_VALUES + L.TRACE_VALUES, prepared):
            setattr(mk, n, None if t is None else t.data_ptr())
        keep = prepared
    grads = [p.empty(T, B, I), torch.empty_like(p.w_ih), torch.empty_like(p.w_hh), p.empty(4 * H), p.empty(4 * H),
             p.empty(B, H), p.empty(B, H)]
    gs = L.Gradients()
    for n, t in zip(L.MASTER_VALUES, grads):
        setattr(gs, n, t.data_ptr())
    ws, n = _workspace(2, T, B, I, H, p.device)
    with torch.cuda.device(p.device):
        if params is None:
            rc = lib.rxmet_lstm_backward_float(T, B, I, H, _ptr(p.w_ih), _ptr(p.w_hh), _ptr(p.x), _ptr(p.h0), _ptr(p.c0),
                                               _ptr(gates), _ptr(cells), _ptr(ctanh), _ptr(hidden), _ptr(g_out), _ptr(g_hn),
                                               _ptr(g_cn), C.byref(mk) if mk is not None else None, C.byref(gs), _ptr(ws),
                                               C.c_size_t(n), _stream())
        else:
            rc = lib.rxmet_lstm_backward_qat(T, B, I, H, C.byref(params.struct), _ptr(p.w_ih), _ptr(p.w_hh), _ptr(p.x),
                                             _ptr(p.h0), _ptr(p.c0), _ptr(gates), _ptr(cells), _ptr(ctanh), _ptr(hidden),
                                             _ptr(g_out), _ptr(g_hn), _ptr(g_cn), C.byref(mk) if mk is not None else None,
                                             C.byref(gs), _ptr(ws), C.c_size_t(n), _stream())
    _check(rc, RuntimeError)
    del keep
    if batch_first:
        grads[0] = grads[0].transpose(0, 1)
    return tuple(grads)


def lstm_backward_float(input, weight_ih, weight_hh, bias_ih, bias_hh, initial_hidden, initial_cell, batch_first,
                        gate_outputs, cell_states, cell_tanh_outputs, hidden_outputs, grad_output, grad_final_hidden,
                        grad_final_cell, master_masks: Sequence[torch.Tensor] = (),
                        checkpoint_masks: Sequence[torch.Tensor] = ()):
    """Float backward through time: (d_input, d_weight_ih, d_weight_hh, d_bias_ih, d_bias_hh, d_h0, d_c0)."""
    p = _Prepared(input, weight_ih, weight_hh, bias_ih, bias_hh, initial_hidden, initial_cell, batch_first)
    return _backward(p, batch_first, (gate_outputs, cell_states, cell_tanh_outputs, hidden_outputs), grad_output,
                     grad_final_hidden, grad_final_cell, list(master_masks), list(checkpoint_masks), input.shape, None)


# --------------------------------------------------------------------------
# parameter bundles (operators/quant-lstm/src/lstm/quant_params_io.cc)
# --------------------------------------------------------------------------

def _shortest_float(v) -> str:
    """Shortest decimal that round-trips float32 (what the reference writes with std::to_chars)."""
    v = np.float32(v)
    if not np.isfinite(v):
        raise ValueError("scale must be a finite float32")
    fixed = np.format_float_positional(v, unique=True, trim="-")
    sci = np.format_float_scientific(v, unique=True, trim="-", exp_digits=2)
    mant, exp = sci.split("e")
    sci = f"{mant}e{'-' if exp[0] == '-' else '+'}{exp.lstrip('+-')}"
    return sci if len(sci) < len(fixed) else fixed


def _parse_scale(text) -> np.float32:
    if not isinstance(text, str):
        raise ValueError("scale must be a canonical float32 string")
    try:
        v = np.float32(text)
    except ValueError as e:
        raise ValueError("scale is not a float32 decimal string") from e
    if not np.isfinite(v) or np.float32(_shortest_float(v)) != v:
        raise ValueError("scale is not a finite float32")
    return v


_BUNDLE_CACHE: dict = {}


def _bundle_to_params(bundle_json: str) -> L.ParamsBox:
    """Parsed parameters of a bundle; cached on the text, because a module passes the same bundle on
    every call (treat the returned box as read-only)."""
    box = _BUNDLE_CACHE.get(bundle_json)
    if box is None:
        box = _parse_bundle(bundle_json)
        if len(_BUNDLE_CACHE) > 64:
            _BUNDLE_CACHE.clear()
        _BUNDLE_CACHE[bundle_json] = box
    return box


def _parse_bundle(bundle_json: str) -> L.ParamsBox:
    try:
        root = json.loads(bundle_json)
    except json.JSONDecodeError as e:
        raise ValueError(f"quant params JSON does not parse: {e}") from e
    allowed = {"schema_version", "input_size", "hidden_size", "bias_enabled", "scale_mode", "operators"}
    if not isinstance(root, dict) or set(root) - allowed:
        raise ValueError("quant params root has unknown fields")
    for key in ("schema_version", "input_size", "hidden_size"):
        if not isinstance(root.get(key), int) or isinstance(root.get(key), bool):
            raise ValueError(f"{key} must be a JSON integer")
    if root["schema_version"] != 1:
        raise ValueError("only quant params bundle schema_version=1 is supported")
    if not isinstance(root.get("bias_enabled"), bool):
        raise ValueError("bias_enabled must be a boolean")
    if root.get("scale_mode") not in L.SCALE_MODE_NAMES:
        raise ValueError("scale_mode must be affine or pot2")
    H, I, bias = root["hidden_size"], root["input_size"], root["bias_enabled"]
    if H <= 0 or I <= 0:
        raise ValueError("input_size and hidden_size must be positive")
    ops = root.get("operators")
    if not isinstance(ops, dict):
        raise ValueError("operators must be an object")
    expected = [n for i, n in enumerate(L.OP_NAMES) if bias or i not in L.BIAS_OPS]
    if set(ops) != set(expected):
        raise ValueError("operators has missing, unknown or disabled fields")
    box = L.ParamsBox(H)
    s = box.struct
    s.input_size, s.hidden_size, s.bias_enabled = I, H, int(bias)
    s.config.scale_mode = L.SCALE_MODE_NAMES.index(root["scale_mode"])
    for op, name in enumerate(L.OP_NAMES):
        if name not in ops:
            s.config.bitwidth[op], s.config.is_symmetric[op], s.config.granularity[op] = 8, 1, L.PER_CHANNEL
            continue
        o = ops[name]
        if set(o) - {"bitwidth", "is_unsigned", "is_symmetric", "granularity", "scales", "zero_points"}:
            raise ValueError(f"{name} has unknown fields")
        if o.get("granularity") not in L.GRANULARITY_NAMES:
            raise ValueError(f"{name}: bad granularity")
        s.config.bitwidth[op] = int(o["bitwidth"])
        s.config.is_unsigned[op] = int(bool(o["is_unsigned"]))
        s.config.is_symmetric[op] = int(bool(o["is_symmetric"]))
        s.config.granularity[op] = L.GRANULARITY_NAMES.index(o["granularity"])
        scales, zps = o.get("scales"), o.get("zero_points")
        count = 4 * H if op in L.PARAMETER_OPS else 1
        if not isinstance(scales, list) or not isinstance(zps, list) or len(scales) != count or len(zps) != count:
            raise ValueError("quantization parameters must be given as the full 4H list or a single value")
        values = [_parse_scale(v) for v in scales]
        if op in L.PARAMETER_OPS:
            if any(z != 0 for z in zps):
                raise ValueError("weight/bias zero points must all be 0")
            box.channel_scales[op - L.WEIGHT_IH][:] = values
        else:
            s.scale[op], s.zero_point[op] = values[0], int(zps[0])
    box.bind()
    return box


def _params_to_bundle(box: L.ParamsBox) -> str:
    s = box.struct
    ops = {}
    for op, name in enumerate(L.OP_NAMES):
        if not s.bias_enabled and op in L.BIAS_OPS:
            continue
        if op in L.PARAMETER_OPS:
            scales = [_shortest_float(v) for v in box.channel_scales[op - L.WEIGHT_IH]]
            zps = [0] * (4 * box.H)
        else:
            scales, zps = [_shortest_float(s.scale[op])], [int(s.zero_point[op])]
        ops[name] = {"bitwidth": int(s.config.bitwidth[op]), "is_unsigned": bool(s.config.is_unsigned[op]),
                     "is_symmetric": bool(s.config.is_symmetric[op]),
                     "granularity": L.GRANULARITY_NAMES[s.config.granularity[op]], "scales": scales, "zero_points": zps}
    root = {"schema_version": 1, "input_size": int(s.input_size), "hidden_size": int(s.hidden_size),
            "bias_enabled": bool(s.bias_enabled), "scale_mode": L.SCALE_MODE_NAMES[s.config.scale_mode], "operators": ops}
    return json.dumps(root, separators=(",", ":"))


def _config_to_json(cfg: L.QuantConfig) -> str:
    ops = {}
    for op, name in enumerate(L.OP_NAMES):
        entry = {"bitwidth": int(cfg.bitwidth[op]), "is_unsigned": bool(cfg.is_unsigned[op]),
                 "is_symmetric": bool(cfg.is_symmetric[op]), "granularity": L.GRANULARITY_NAMES[cfg.granularity[op]]}
        ops[name] = entry
    return json.dumps({"schema_version": 1, "scale_mode": L.SCALE_MODE_NAMES[cfg.scale_mode], "operators": ops},
                      separators=(",", ":"))


def _config_from_json(text: str) -> L.QuantConfig:
    try:
        root = json.loads(text)
    except json.JSONDecodeError as e:
        raise ValueError(f"quant config JSON does not parse: {e}") from e
    if not isinstance(root, dict) or root.get("schema_version") != 1:
        raise ValueError("only quant config schema_version=1 is supported")
    if root.get("scale_mode") not in L.SCALE_MODE_NAMES:
        raise ValueError("scale_mode must be affine or pot2")
    ops = root.get("operators")
    if not isinstance(ops, dict) or set(ops) != set(L.OP_NAMES):
        raise ValueError("operators must name exactly the 18 quantization points")
    cfg = L.QuantConfig()
    cfg.scale_mode = L.SCALE_MODE_NAMES.index(root["scale_mode"])
    for op, name in enumerate(L.OP_NAMES):
        o = ops[name]
        parameter = op in L.PARAMETER_OPS
        cfg.bitwidth[op] = int(o["bitwidth"])
        cfg.is_unsigned[op] = int(bool(o.get("is_unsigned", False)))
        cfg.is_symmetric[op] = int(bool(o.get("is_symmetric", True)))
        gran = o.get("granularity", "per_channel" if parameter else "per_tensor")
        if gran not in L.GRANULARITY_NAMES:
            raise ValueError(f"{name}: bad granularity")
        cfg.granularity[op] = L.GRANULARITY_NAMES.index(gran)
    return cfg


def _execution(box: L.ParamsBox, require_exact: bool) -> L.ExecutionBox:
    cached = getattr(box, "_execution", {}).get(bool(require_exact))
    if cached is not None:
        return cached
    ex = L.ExecutionBox(box.H)
    _check(_library().rxmet_lstm_derive_execution(C.byref(box.struct), int(require_exact), C.byref(ex.struct)), ValueError)
    if not hasattr(box, "_execution"):
        box._execution = {}
    box._execution[bool(require_exact)] = ex
    return ex


def _safety_summary(ex: L.ExecutionBox) -> dict:
    exact = bool(ex.struct.exact_accumulation)
    return {"has_precision_risk": not exact, "all_exact_integer_range": exact}


def audit_quant_params_bundle(bundle_json: str, require_exact_accumulation: bool = False) -> dict:
    """Normalises a parameter bundle and re-derives its execution encodings."""
    box = _bundle_to_params(bundle_json)
    ex = _execution(box, require_exact_accumulation)
    return {"bundle_json": _params_to_bundle(box), "resolved_config_json": _config_to_json(box.struct.config),
            "safety": _safety_summary(ex), "input_size": int(box.struct.input_size),
            "hidden_size": int(box.struct.hidden_size), "bias_enabled": bool(box.struct.bias_enabled)}


def validate_resolved_quant_config(resolved_json: str) -> str:
    return _config_to_json(_config_from_json(resolved_json))


def resolve_quant_config(defaults_json: str, override_json: str) -> str:
    """Merges an override (any subset of scale_mode and per-operator fields) into a default config."""
    base = json.loads(defaults_json)
    over = json.loads(override_json) if override_json else {}
    if not isinstance(base, dict) or not isinstance(over, dict):
        raise ValueError("quant config documents must be JSON objects")
    if "scale_mode" in over:
        base["scale_mode"] = over["scale_mode"]
    for name, fields in over.get("operators", {}).items():
        if name not in L.OP_NAMES:
            raise ValueError(f"unknown operator {name}")
        base.setdefault("operators", {}).setdefault(name, {}).update(fields)
    for o in base.get("operators", {}).values():
        o.pop("comment", None)
    return _config_to_json(_config_from_json(json.dumps(base)))


# --------------------------------------------------------------------------
# quantized forward / QAT backward
# --------------------------------------------------------------------------

def lstm_forward_quantized(input, weight_ih, weight_hh, bias_ih=None, bias_hh=None, initial_hidden=None,
                           initial_cell=None, batch_first=False, bundle_json="", math_mode="pedantic",
                           require_exact_accumulation=False, save_checkpoints=False):
    """Quantized forward: (output, h_n, c_n, checkpoints, safety).  With save_checkpoints the fourth
    entry holds ``values`` / ``clamp_masks`` (7 per-step tensors each) and ``quantized_master`` /
    ``master_clamp_masks`` (the q-carrier copies of the inputs), as the QAT backward consumes them."""
    p = _Prepared(input, weight_ih, weight_hh, bias_ih, bias_hh, initial_hidden, initial_cell, batch_first)
    box = _bundle_to_params(bundle_json)
    T, B, I, H = p.dims()
    if box.struct.input_size != I or box.struct.hidden_size != H:
        raise RuntimeError("quantization parameters do not match input_size / hidden_size of the module")
    if bool(box.struct.bias_enabled) != (p.b_ih is not None):
        raise RuntimeError("quantization parameters do not match the bias setting of the module")
    if math_mode not in ("pedantic", "tf32"):
        raise ValueError("cublas_math_mode must be pedantic or tf32")
    ex = _execution(box, require_exact_accumulation)
    out, hn, cn = p.empty(T, B, H), p.empty(1, B, H), p.empty(1, B, H)
    checkpoints: dict = {}
    tr = ms = None
    if save_checkpoints:
        values = {n: p.empty(T, B, 4 * H if i < 4 else H) for i, n in enumerate(L.TRACE_VALUES)}
        masks = {n: p.empty(T, B, 4 * H if i < 4 else H, dtype=torch.uint8) for i, n in enumerate(L.TRACE_VALUES)}
        tr = _trace_struct(values, masks)
        mv = [torch.empty_like(p.x), torch.empty_like(p.w_ih), torch.empty_like(p.w_hh),
              p.empty(4 * H) if p.b_ih is not None else p.empty(0), p.empty(4 * H) if p.b_ih is not None else p.empty(0),
              p.empty(1, B, H), p.empty(1, B, H)]
        # every flag is written by the library (0 or 1), so the buffers need no zero-fill
        mm = [torch.empty(v.shape, dtype=torch.bool, device=p.device) for v in mv]
        ms = L.Masters()
        for n, v, m in zip(L.MASTER_VALUES, mv, mm):
            setattr(ms, n, v.data_ptr() if v.numel() else None)
            setattr(ms, n + "_clamped", m.data_ptr() if m.numel() else None)
    ws, n = _workspace(1, T, B, I, H, p.device)
    with torch.cuda.device(p.device):
        rc = _library().rxmet_lstm_forward_quantized(
            T, B, I, H, _ptr(p.w_ih), _ptr(p.w_hh), _ptr(p.b_ih), _ptr(p.b_hh), _ptr(p.x), _ptr(p.h0), _ptr(p.c0),
            C.byref(box.struct), int(require_exact_accumulation), _ptr(out), _ptr(hn), _ptr(cn),
            C.byref(tr) if tr is not None else None, C.byref(ms) if ms is not None else None, _ptr(ws), C.c_size_t(n),
            _stream())
    _check(rc, RuntimeError)
    if save_checkpoints:
        names = ("input", "weight_ih", "weight_hh", "bias_ih", "bias_hh", "h_0", "c_0")
        qm, qk = {}, {}
        for i, name in enumerate(names):
            if p.b_ih is None and i in (3, 4):
                continue
            v, m = mv[i], mm[i]
            if i == 0 and batch_first:
                v, m = v.transpose(0, 1), m.transpose(0, 1)
            qm[name], qk[name] = v, m
        checkpoints = {"values": values, "clamp_masks": masks, "quantized_master": qm, "master_clamp_masks": qk}
    return (out.transpose(0, 1) if batch_first else out), hn, cn, checkpoints, _safety_summary(ex)


def lstm_backward_qat(master_values, batch_first, bundle_json, checkpoint_values, grad_output, grad_final_hidden,
                      grad_final_cell, master_masks, checkpoint_masks):
    """QAT backward on the q-carrier tensors saved by ``lstm_forward_quantized``."""
    if len(master_values) != 7:
        raise RuntimeError("QAT master_values must hold 7 tensors")
    if len(checkpoint_values) != 4:
        raise RuntimeError("QAT checkpoint_values must hold the 4 trace tensors")
    box = _bundle_to_params(bundle_json)
    bias = bool(box.struct.bias_enabled)
    if not bias and (master_values[3].numel() or master_values[4].numel()):
        raise RuntimeError("bias masters must be empty when bias is disabled")
    p = _Prepared(master_values[0], master_values[1], master_values[2], master_values[3] if bias else None,
                  master_values[4] if bias else None, master_values[5], master_values[6], batch_first)
    return _backward(p, batch_first, checkpoint_values, grad_output, grad_final_hidden, grad_final_cell,
                     list(master_masks), list(checkpoint_masks), master_values[0].shape, box)


# --------------------------------------------------------------------------
# calibration
# --------------------------------------------------------------------------

class CalibrationSession:
    """Calibration over any number of batches, method "minmax", "sqnr" or "percentile"
    (CalibrationSessionBinding, lstm_interface_binding.cc:791-882).  The statistics of a batch are
    reduced (and, for the histogram methods, binned) on the device by the calibration forward and
    merged on the host; ``finalize`` turns them into a parameter bundle."""

    def __init__(self, resolved_config_json: str, input_size: int, hidden_size: int, bias_enabled: bool,
                 method: str = "minmax", percentile: float = 99.99):
        if method not in ("minmax", "sqnr", "percentile"):
            raise ValueError("calibration_method must be minmax, sqnr or percentile")
        if not (0.0 < percentile <= 100.0):
            raise RuntimeError("percentile must be in (0, 100]")
        self._config = _config_from_json(resolved_config_json)
        self._I, self._H, self._bias = int(input_size), int(hidden_size), bool(bias_enabled)
        self._method = method
        self._percentile = float(percentile)
        self.reset()

    def reset(self):
        self._ranges = L.RangesBox(self._H)
        self._hists = L.HistogramSet(self._H) if self._method != "minmax" else None
        self._batches = 0
        self._state = "empty"
        self._final = None

    @property
    def state(self) -> str:
        return self._state

    @property
    def batch_count(self) -> int:
        return self._batches

    # Data-parallel calibration (no counterpart in the reference's session): with `process_group` set, every
    # rank passes its shard of each batch to collect(); extremes and bin counts are all-reduced inside the batch,
    # so all ranks finalize the parameters one process would derive from the concatenated batches.
    process_group = None

    def _exchange_for(self, device):
        if self.process_group is None:
            return None
        key = (id(self.process_group), str(device))
        if getattr(self, "_exchange_key", None) != key:
            from .data_parallel import make_exchange
            self._exchange, self._exchange_key = make_exchange(self.process_group, device), key
        return self._exchange

    def collect(self, input, weight_ih, weight_hh, bias_ih=None, bias_hh=None, initial_hidden=None,
                initial_cell=None, batch_first=False):
        if self._state == "locked":
            raise RuntimeError("a locked calibration session accepts no further batches")
        p = _Prepared(input, weight_ih, weight_hh, bias_ih, bias_hh, initial_hidden, initial_cell, batch_first)
        if p.I != self._I or p.H != self._H:
            raise RuntimeError("calibration tensor shapes do not match the session")
        if (p.b_ih is not None) != self._bias:
            raise RuntimeError("calibration bias setting does not match the session")
        lib = _library()
        if self._hists is not None:
            T, B, I, H = p.dims()
            out, hn, cn = p.empty(T, B, H), p.empty(1, B, H), p.empty(1, B, H)
            ws, n = _workspace(3, T, B, I, H, p.device)
            exchange = self._exchange_for(p.device)
            with torch.cuda.device(p.device):
                rc = lib.rxmet_lstm_forward_calibrate_hist_dp(
                    T, B, I, H, _ptr(p.w_ih), _ptr(p.w_hh), _ptr(p.b_ih), _ptr(p.b_hh), _ptr(p.x), _ptr(p.h0), _ptr(p.c0),
                    _ptr(out), _ptr(hn), _ptr(cn), C.byref(self._config), C.byref(self._ranges.struct),
                    C.byref(self._hists.struct), _ptr(ws), C.c_size_t(n), _stream(),
                    C.byref(exchange) if exchange is not None else None)
            _check(rc, RuntimeError)
        else:
            stats = torch.empty(lib.rxmet_lstm_stats_floats(p.H), dtype=torch.float32, device=p.device)
            out, hn, cn = _run_float(p, None, stats)
            if self.process_group is not None:  # every rank folds the extremes of the whole batch
                import torch.distributed as dist
                half = stats.numel() // 2
                dist.all_reduce(stats[:half], op=dist.ReduceOp.MIN, group=self.process_group)
                dist.all_reduce(stats[half:], op=dist.ReduceOp.MAX, group=self.process_group)
            host = stats.cpu().numpy()
            _check(lib.rxmet_lstm_ranges_fold_stats(C.byref(self._ranges.struct),
                                                    host.ctypes.data_as(C.POINTER(C.c_float)), p.H, int(self._bias)),
                   RuntimeError)
        self._batches += 1
        self._state = "dirty"
        return (out.transpose(0, 1) if batch_first else out), hn, cn

    def finalize(self, require_exact_accumulation: bool = False) -> dict:
        if self._state == "empty":
            raise RuntimeError("an empty calibration session cannot be finalized")
        if self._final is None:
            box = L.ParamsBox(self._H)
            if self._hists is None:
                _check(_library().rxmet_lstm_params_from_ranges(
                    C.byref(self._config), C.byref(self._ranges.struct), self._I, self._H, int(self._bias),
                    *box.scale_ptrs(), C.byref(box.struct)), ValueError)
            else:
                _check(_library().rxmet_lstm_params_from_histograms(
                    C.byref(self._config), C.byref(self._ranges.struct), C.byref(self._hists.struct),
                    0 if self._method == "sqnr" else 1, C.c_float(self._percentile), self._I, self._H, int(self._bias),
                    *box.scale_ptrs(), C.byref(box.struct)), ValueError)
            box.bind()
            ex = _execution(box, require_exact_accumulation)
            r = self._ranges.struct
            self._final = {"bundle_json": _params_to_bundle(box), "resolved_config_json": _config_to_json(self._config),
                           "safety": _safety_summary(ex), "batch_count": self._batches, "method": self._method,
                           "activation_ranges": {n: (float(r.minimum[i]), float(r.maximum[i]))
                                                 for i, n in enumerate(L.OP_NAMES) if i not in L.PARAMETER_OPS}}
            self._state = "locked"
        return self._final
