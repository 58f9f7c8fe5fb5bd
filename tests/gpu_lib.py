"""Direct ctypes calls into librxmet_b200.so for the GPU parity tests (numpy in, numpy out)."""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from rx_met_b200 import _cabi as cabi

MASK_SHAPES = lambda T, B, I, H: {  # noqa: E731
    "x": (T, B, I), "h0": (B, H), "W": (I, 3 * H), "R": (H, 3 * H), "bw": (3 * H,), "br": (3 * H,),
    "weight_ih_linear": (T, B, 3 * H), "weight_hh_linear": (T, B, 3 * H), "gate_input": (T, B, 3 * H),
    "gate_output": (T, B, 3 * H), "h": (T, B, H)}


def dev(a):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda()


def ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def workspace(op, T, B, I, H, extra=0):
    n = cabi.load_library().rxmet_gru_workspace_bytes(op, T, B, I, H) + extra
    return torch.empty(n, dtype=torch.uint8, device="cuda"), n


def forward_quant(W, R, bw, br, x, h0, params, training=True, workspace_bytes=None, fp_carrier=False):
    """params: oracle_lib.ParamsBox.  Returns dict of numpy arrays (codes, masks, h, v).  fp_carrier: the reference's
    FP32 carrier (rxmet_gru_forward_quant_fp_carrier) instead of the integer carrier."""
    lib = cabi.load_library()
    T, B, I = x.shape
    H = R.shape[0]
    d = {k: dev(v) for k, v in dict(W=W, R=R, bw=bw, br=br, x=x, h0=h0).items()}
    f32 = dict(dtype=torch.float32, device="cuda")
    i32 = dict(dtype=torch.int32, device="cuda")
    out = {"h": torch.empty((T + 1, B, H), **f32), "v": torch.empty((T, B, 4 * H), **f32),
           "W_q": torch.empty((I, 3 * H), **i32), "R_q": torch.empty((H, 3 * H), **i32),
           "bw_q": torch.empty(3 * H, **i32), "br_q": torch.empty(3 * H, **i32),
           "x_q": torch.empty((T, B, I), **i32), "h_q": torch.empty((T + 1, B, H), **i32),
           "v_q": torch.empty((T, B, 4 * H), **i32)}
    masks, ms = {}, cabi.Masks()
    if training:
        for name, shape in MASK_SHAPES(T, B, I, H).items():
            if name == "h0" and h0 is None:
                continue
            masks[name] = torch.full(shape, 255, dtype=torch.uint8, device="cuda")
            setattr(ms, name, masks[name].data_ptr())
    ws, n = workspace(1, T, B, I, H)
    if workspace_bytes is not None:
        n = workspace_bytes
    entry = lib.rxmet_gru_forward_quant_fp_carrier if fp_carrier else lib.rxmet_gru_forward_quant
    rc = entry(
        int(training), T, B, I, H, ptr(d["W"]), ptr(d["R"]), ptr(d["bw"]), ptr(d["br"]), ptr(d["x"]), ptr(d["h0"]),
        C.byref(params.c), ptr(out["h"]), ptr(out["v"]), ptr(out["W_q"]), ptr(out["R_q"]), ptr(out["bw_q"]),
        ptr(out["br_q"]), ptr(out["x_q"]), ptr(out["h_q"]), ptr(out["v_q"]),
        C.byref(ms) if training else None, ptr(ws), C.c_size_t(n), stream())
    torch.cuda.synchronize()
    if rc != 0:
        return rc, lib.rxmet_last_error().decode()
    res = {k: v.cpu().numpy() for k, v in out.items()}
    res["masks"] = {k: v.cpu().numpy() for k, v in masks.items()}
    res["dev"] = out
    res["dev_masks"] = masks
    return 0, res


def forward_int_io(W, R, bw, br, x_q, h0_q, params):
    lib = cabi.load_library()
    T, B, I = x_q.shape
    H = R.shape[0]
    d = {k: dev(v) for k, v in dict(W=W, R=R, bw=bw, br=br, x_q=x_q, h0_q=h0_q).items()}
    h_q = torch.empty((T + 1, B, H), dtype=torch.int32, device="cuda")
    extra = 4 * ((T + 1) * B * H + T * B * 4 * H) + 4096
    ws, n = workspace(1, T, B, I, H, extra)
    rc = lib.rxmet_gru_forward_quant_int_io(T, B, I, H, ptr(d["W"]), ptr(d["R"]), ptr(d["bw"]), ptr(d["br"]),
                                            ptr(d["x_q"]), ptr(d["h0_q"]), C.byref(params.c), ptr(h_q), ptr(ws),
                                            C.c_size_t(n), stream())
    torch.cuda.synchronize()
    assert rc == 0, lib.rxmet_last_error()
    return h_q.cpu().numpy()


def forward_float(W, R, bw, br, x, h0, ranges=None):
    """ranges: oracle_lib.RangesBox updated in place when given (calibration forward)."""
    lib = cabi.load_library()
    T, B, I = x.shape
    H = R.shape[0]
    d = {k: dev(v) for k, v in dict(W=W, R=R, bw=bw, br=br, x=x, h0=h0).items()}
    h = torch.empty((T + 1, B, H), dtype=torch.float32, device="cuda")
    v = torch.empty((T, B, 4 * H), dtype=torch.float32, device="cuda")
    ws, n = workspace(0, T, B, I, H)
    args = (T, B, I, H, ptr(d["W"]), ptr(d["R"]), ptr(d["bw"]), ptr(d["br"]), ptr(d["x"]), ptr(d["h0"]), ptr(h), ptr(v))
    if ranges is None:
        rc = lib.rxmet_gru_forward_fp(*args, ptr(ws), C.c_size_t(n), stream())
    else:
        rc = lib.rxmet_gru_forward_calibrate_minmax(*args, C.byref(ranges.c), ptr(ws), C.c_size_t(n), stream())
    torch.cuda.synchronize()
    assert rc == 0, lib.rxmet_last_error()
    return h.cpu().numpy(), v.cpu().numpy()


def _grads(T, B, I, H):
    f32 = dict(dtype=torch.float32, device="cuda")
    return {"dx": torch.empty((T, B, I), **f32), "dW": torch.empty((I, 3 * H), **f32),
            "dR": torch.empty((H, 3 * H), **f32), "dbw": torch.empty(3 * H, **f32),
            "dbr": torch.empty(3 * H, **f32), "dh0": torch.empty((B, H), **f32)}


def backward_quant(codes, dh_new, h, v, params, masks):
    """codes: dict with W_q, R_q, bw_q, br_q, x_q (numpy int32); masks: dict name -> numpy uint8 or None."""
    lib = cabi.load_library()
    T, B, I = codes["x_q"].shape
    H = codes["R_q"].shape[0]
    d = {k: dev(codes[k]) for k in ("W_q", "R_q", "bw_q", "br_q", "x_q")}
    dd = {k: dev(a) for k, a in dict(dh_new=dh_new, h=h, v=v).items()}
    ms, keep = cabi.Masks(), []
    if masks:
        for name, a in masks.items():
            t = dev(a)
            keep.append(t)
            setattr(ms, name, t.data_ptr())
    g = _grads(T, B, I, H)
    ws, n = workspace(2, T, B, I, H)
    rc = lib.rxmet_gru_backward_quant(
        T, B, I, H, ptr(d["W_q"]), ptr(d["R_q"]), ptr(d["bw_q"]), ptr(d["br_q"]), ptr(d["x_q"]),
        ptr(dd["dh_new"]), ptr(dd["h"]), ptr(dd["v"]), C.byref(params.c), C.byref(ms) if masks else None,
        ptr(g["dx"]), ptr(g["dW"]), ptr(g["dR"]), ptr(g["dbw"]), ptr(g["dbr"]), ptr(g["dh0"]),
        ptr(ws), C.c_size_t(n), stream())
    torch.cuda.synchronize()
    assert rc == 0, lib.rxmet_last_error()
    return {k: t.cpu().numpy() for k, t in g.items()}


def backward_fp(W, R, bw, br, x, dh_new, h, v):
    lib = cabi.load_library()
    T, B, I = x.shape
    H = R.shape[0]
    d = {k: dev(a) for k, a in dict(W=W, R=R, bw=bw, br=br, x=x, dh_new=dh_new, h=h, v=v).items()}
    g = _grads(T, B, I, H)
    ws, n = workspace(2, T, B, I, H)
    rc = lib.rxmet_gru_backward_fp(T, B, I, H, ptr(d["W"]), ptr(d["R"]), ptr(d["bw"]), ptr(d["br"]), ptr(d["x"]),
                                   ptr(d["dh_new"]), ptr(d["h"]), ptr(d["v"]), ptr(g["dx"]), ptr(g["dW"]),
                                   ptr(g["dR"]), ptr(g["dbw"]), ptr(g["dbr"]), ptr(g["dh0"]), ptr(ws),
                                   C.c_size_t(n), stream())
    torch.cuda.synchronize()
    assert rc == 0, lib.rxmet_last_error()
    return {k: t.cpu().numpy() for k, t in g.items()}
