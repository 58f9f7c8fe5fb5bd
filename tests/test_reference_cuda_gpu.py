"""The library against the reference's own CUDA build on the same GPU (oracle/_ref/libgru_ref_cuda.so = the
reference's unmodified .cu / .cc sources of operators/quant-gru/src compiled with nvcc for sm_100a + cuBLAS).

The reference has the QAT backward (BPTT on dequantized values with the eleven straight-through masks,
gru_backward_gpu_quant.cu:316-493) only as CUDA, so this is where the backward of the library is held to the
reference itself rather than to the C restatement: same saved tensors in, gradients within 1e-5 relative.
The integer-carrier forward is compared too (codes, masks, dequantized outputs)."""
from __future__ import annotations

import ctypes as C

import numpy as np
import pytest
import torch

import gpu_lib
import oracle_lib as ol
import refcuda_lib as rc
from rx_met_b200 import _cabi as cabi

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(rc.lib() is None, reason="reference CUDA build not present")]

P = gpu_lib.ptr


def calibrated(seed, T, B, I, H, cfg, with_h0):
    W, R, bw, br, x, h0 = ol.gru_problem(seed, T, B, I, H, with_h0=with_h0)
    ranges = ol.RangesBox(H)
    gpu_lib.forward_float(W, R, bw, br, x * 0.8, h0, ranges=ranges)  # narrower calibration input: clamping happens
    params = ol.ParamsBox(H, cfg)
    assert cabi.load_library().rxmet_gru_params_from_ranges(C.byref(ranges.c), C.byref(cfg), C.byref(params.c)) == 0
    return (W, R, bw, br, x, h0), params


def reference_forward(problem, params, T, B, I, H):
    W, R, bw, br, x, h0 = [gpu_lib.dev(a) for a in problem]
    f32, i32 = dict(dtype=torch.float32, device="cuda"), dict(dtype=torch.int32, device="cuda")
    out = {"h": torch.zeros((T + 1, B, H), **f32), "v": torch.zeros((T, B, 4 * H), **f32),
           "W_q": torch.zeros((I, 3 * H), **i32), "R_q": torch.zeros((H, 3 * H), **i32), "bw_q": torch.zeros(3 * H, **i32),
           "br_q": torch.zeros(3 * H, **i32), "x_q": torch.zeros((T, B, I), **i32)}
    masks, ms = {}, cabi.Masks()
    for name, shape in gpu_lib.MASK_SHAPES(T, B, I, H).items():
        if name == "h0" and h0 is None:
            continue
        masks[name] = torch.full(shape, 255, dtype=torch.uint8, device="cuda")
        setattr(ms, name, masks[name].data_ptr())
    rc.call("refcuda_gru_forward_quant_int", 1, T, B, I, H, P(W), P(R), P(bw), P(br), P(x), P(h0), C.byref(params.c),
            P(out["h"]), P(out["v"]), C.byref(ms), P(out["W_q"]), P(out["R_q"]), P(out["bw_q"]), P(out["br_q"]), P(out["x_q"]))
    return out, masks


def reference_backward(got, dh_new, params, T, B, I, H):
    """The reference's binding, step by step: float copies of the saved codes, its own dequantization in place,
    transposes, zeroed weight gradients, quantGRUBackward with the eleven masks."""
    dev = got["dev"]
    Wf, Rf, bwf, brf, xf = [dev[k].to(torch.float32).contiguous() for k in ("W_q", "R_q", "bw_q", "br_q", "x_q")]
    rc.call("refcuda_gru_dequantize_saved", I, H, C.c_longlong(xf.numel()), P(Wf), P(Rf), P(bwf), P(brf), P(xf),
            C.byref(params.c))
    x_t, W_t, R_t = xf.permute(2, 0, 1).contiguous(), Wf.t().contiguous(), Rf.t().contiguous()
    f32 = dict(dtype=torch.float32, device="cuda")
    g = {"dx": torch.empty((T, B, I), **f32), "dW": torch.zeros((I, 3 * H), **f32), "dR": torch.zeros((H, 3 * H), **f32),
         "dbw": torch.zeros(3 * H, **f32), "dbr": torch.zeros(3 * H, **f32), "dh0": torch.zeros((B, H), **f32)}
    ms = cabi.Masks()
    for name, t in got["dev_masks"].items():
        setattr(ms, name, t.data_ptr())
    rc.call("refcuda_gru_backward_quant", T, B, I, H, P(W_t), P(R_t), P(bwf), P(brf), P(x_t), P(gpu_lib.dev(dh_new)),
            P(dev["h"]), P(dev["v"]), C.byref(params.c), C.byref(ms), P(g["dx"]), P(g["dW"]), P(g["dR"]), P(g["dbw"]),
            P(g["dbr"]), P(g["dh0"]))
    return {k: t.cpu().numpy() for k, t in g.items()}


CASES = [
    # T, B, I, H, bits, symmetric activations, h0
    (6, 5, 12, 16, 8, False, True),
    (12, 16, 40, 128, 8, False, False),    # the 8-bit fast paths (tensor-core projection and backward)
    (8, 40, 40, 64, 8, True, True),
    (5, 7, 20, 48, 16, False, True),       # 16-bit activation grids: the generic kernels
    (4, 6, 64, 256, 16, False, False),
]


@pytest.mark.parametrize("T,B,I,H,bits,sym,with_h0", CASES)
def test_forward_and_backward_against_the_reference_cuda_build(T, B, I, H, bits, sym, with_h0):
    cfg = ol.make_config(bits=8, symmetric=sym)
    if bits != 8:
        for i, name in enumerate(cabi.OP_NAMES):
            if name not in ("W", "R", "bw", "br"):
                cfg.bits[i] = bits
    problem, params = calibrated(31 + H, T, B, I, H, cfg, with_h0)
    status, got = gpu_lib.forward_quant(*problem, params, training=True)
    assert status == 0, got
    ref, ref_masks = reference_forward(problem, params, T, B, I, H)
    # integer carrier of the reference's CUDA build against the library (which is held bit for bit to the
    # reference's CPU build elsewhere): codes of the saved tensors, dequantized outputs, masks
    for k in ("W_q", "R_q", "bw_q", "br_q", "x_q"):
        np.testing.assert_array_equal(got[k], ref[k].cpu().numpy(), err_msg=k)
    for k in ("h", "v"):
        np.testing.assert_array_equal(got[k], ref[k].cpu().numpy(), err_msg=k)
    for k, m in ref_masks.items():
        np.testing.assert_array_equal(got["masks"][k] != 0, m.cpu().numpy() != 0, err_msg=f"mask {k}")
    # QAT backward
    rng = np.random.default_rng(3)
    dh_new = np.zeros((T + 1, B, H), np.float32)
    dh_new[1:] = rng.standard_normal((T, B, H)).astype(np.float32)
    mine = gpu_lib.backward_quant(got, dh_new, got["h"], got["v"], params, got["masks"])
    want = reference_backward(got, dh_new, params, T, B, I, H)
    for k in ("dx", "dW", "dR", "dbw", "dbr", "dh0"):
        err = np.abs(mine[k].astype(np.float64) - want[k]).max()
        assert err <= 2e-5 * max(np.abs(want[k]).max(), 1e-30), f"{k}: {err:.3e} against {np.abs(want[k]).max():.3e}"


def reference_forward_fp(problem, params, T, B, I, H):
    """quantGRUForwardFP of the reference's CUDA build: float code caches, dequantized h and v, byte masks."""
    W, R, bw, br, x, h0 = [gpu_lib.dev(a) for a in problem]
    f32 = dict(dtype=torch.float32, device="cuda")
    out = {"h": torch.zeros((T + 1, B, H), **f32), "v": torch.zeros((T, B, 4 * H), **f32),
           "W_q": torch.zeros((I, 3 * H), **f32), "R_q": torch.zeros((H, 3 * H), **f32), "bw_q": torch.zeros(3 * H, **f32),
           "br_q": torch.zeros(3 * H, **f32), "x_q": torch.zeros((T, B, I), **f32)}
    masks, ms = {}, cabi.Masks()
    for name, shape in gpu_lib.MASK_SHAPES(T, B, I, H).items():
        if name == "h0" and h0 is None:
            continue
        masks[name] = torch.full(shape, 255, dtype=torch.uint8, device="cuda")
        setattr(ms, name, masks[name].data_ptr())
    rc.call("refcuda_gru_forward_quant_fp", 1, T, B, I, H, P(W), P(R), P(bw), P(br), P(x), P(h0), C.byref(params.c),
            P(out["h"]), P(out["v"]), C.byref(ms), P(out["W_q"]), P(out["R_q"]), P(out["bw_q"]), P(out["br_q"]), P(out["x_q"]))
    return out, masks


FP_CASES = [
    # T, B, I, H, symmetric activations, h0, power-of-two scales
    (6, 5, 12, 16, False, True, False),
    (12, 16, 40, 128, False, False, False),
    (8, 40, 40, 64, True, True, False),
    (7, 9, 24, 96, False, True, True),
]


@pytest.mark.parametrize("T,B,I,H,sym,with_h0,pot2", FP_CASES)
def test_fp32_carrier_forward_against_the_reference_cuda_build(T, B, I, H, sym, with_h0, pot2):
    """The FP32 carrier (the reference's CUDA default behind forward_quant_float_storage) on 8-bit grids: h, v, all
    saved codes and all eleven clamp masks equal the reference's own CUDA kernels bit for bit."""
    cfg = ol.make_config(bits=8, symmetric=sym, use_pot2=pot2)
    problem, params = calibrated(31 + T, T, B, I, H, cfg, with_h0)
    want, want_masks = reference_forward_fp(problem, params, T, B, I, H)
    rc_, got = gpu_lib.forward_quant(*problem, params, training=True, fp_carrier=True)
    assert rc_ == 0, got
    for k in ("W_q", "R_q", "bw_q", "br_q", "x_q"):
        np.testing.assert_array_equal(got[k], want[k].cpu().numpy().astype(np.int32), err_msg=k)
    for k in ("h", "v"):
        np.testing.assert_array_equal(got[k], want[k].cpu().numpy(), err_msg=k)
    for k, m in want_masks.items():
        np.testing.assert_array_equal(got["masks"][k], m.cpu().numpy(), err_msg=f"mask {k}")
    # the two carriers are different contracts: they need not agree with each other
    rc_, integer = gpu_lib.forward_quant(*problem, params, training=True)
    assert rc_ == 0
    differing = float((integer["h_q"] != got["h_q"]).mean())
    print(f"FP32 carrier against integer carrier: {100 * differing:.2f} % of the hidden codes differ")
