"""QuantGRU histogram calibration on the GPU: device binning against the reference's collector
(bit-exact on identical data) and the calibration forward end to end against the reference's CPU
calibration (same totals; counts and encodings agree up to the float differences of the forward)."""
from __future__ import annotations

import ctypes as C

import numpy as np
import pytest
import torch

import oracle_lib as ol
from rx_met_b200 import _cabi as cabi
from test_gru_histogram_cpu import BATCHES, one_hist, same, state

pytestmark = pytest.mark.gpu
needs_ref = pytest.mark.skipif(ol.ref() is None, reason="compiled reference not available")
_f32p = C.POINTER(C.c_float)


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@needs_ref
@pytest.mark.parametrize("name", sorted(BATCHES))
def test_device_binning_matches_reference_collector(name):
    lib, ref = cabi.load_library(), ol.ref()
    lib.rxmet_histogram_workspace_bytes.restype = C.c_size_t
    rng = np.random.default_rng(sum(name.encode()) + 1)
    (a, sa), (b, sb) = one_hist(2048), one_hist(2048)
    ws = torch.empty(lib.rxmet_histogram_workspace_bytes(2048), dtype=torch.uint8, device="cuda")
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for data in BATCHES[name](rng):
        d = dev(data)
        rc = lib.rxmet_histogram_collect_dev(C.byref(a), C.c_void_p(d.data_ptr()), C.c_uint64(1), C.c_uint64(data.size),
                                             C.c_uint64(data.size), C.c_void_p(ws.data_ptr()), C.c_size_t(ws.numel()), st)
        assert rc == 0, lib.rxmet_last_error()
        assert ref.ref_histogram_collect_host(C.byref(b), data.ctypes.data_as(_f32p), C.c_uint64(data.size)) == 0
        same(state(a, sa), state(b, sb))


@needs_ref
def test_device_binning_of_a_strided_view():
    lib, ref = cabi.load_library(), ol.ref()
    lib.rxmet_histogram_workspace_bytes.restype = C.c_size_t
    rng = np.random.default_rng(8)
    full = rng.standard_normal((700, 48)).astype(np.float32)
    view = np.ascontiguousarray(full[:, 16:32])
    (a, sa), (b, sb) = one_hist(512), one_hist(512)
    ws = torch.empty(lib.rxmet_histogram_workspace_bytes(512), dtype=torch.uint8, device="cuda")
    d = dev(full)
    rc = lib.rxmet_histogram_collect_dev(C.byref(a), C.c_void_p(d.data_ptr() + 16 * 4), C.c_uint64(700), C.c_uint64(16),
                                         C.c_uint64(48), C.c_void_p(ws.data_ptr()), C.c_size_t(ws.numel()),
                                         C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, lib.rxmet_last_error()
    ref.ref_histogram_collect_host(C.byref(b), view.ctypes.data_as(_f32p), C.c_uint64(view.size))
    same(state(a, sa), state(b, sb))


@needs_ref
@pytest.mark.parametrize("granularity", [cabi.PER_CHANNEL, cabi.PER_TENSOR, cabi.PER_GATE])
def test_calibration_forward_fills_the_collectors_like_the_reference(granularity):
    from rx_met_b200 import gru_interface_binding as ops
    ref = ol.ref()
    T, B, I, H = 20, 16, 12, 32
    W, R, bw, br, x, h0 = ol.gru_problem(6, T, B, I, H, with_h0=True)
    cfg_c = ol.make_config(bits=8, symmetric=False, granularity=granularity)
    cfg = ops.OperatorQuantConfig._from_c(cfg_c)
    got = ops.GRUHistogramCollectors(H)
    want = cabi.HistogramSet(H, 2048)
    h = np.zeros((T + 1, B, H), np.float32)
    v = np.zeros((T, B, 4 * H), np.float32)
    fp = lambda a_: a_.ctypes.data_as(_f32p)  # noqa: E731
    for scale in (1.0, 1.5, 0.5):
        xs = np.ascontiguousarray(x * np.float32(scale))
        ops.forward_calibrate(False, T, B, I, H, dev(W), dev(R), dev(bw), dev(br), dev(xs), dev(h0), "sqnr", cfg,
                              None, got)
        assert ref.ref_gru_forward_calibrate_hist(T, B, I, H, fp(W), fp(R), fp(bw), fp(br), fp(xs), fp(h0),
                                                  C.byref(cfg_c), C.byref(want.c), fp(h), fp(v)) == 0
    assert got.is_valid()
    for ga, wa in zip(got._set.all(), want.all()):
        assert ga.total_count == wa.total_count
    for op in range(cabi.NUM_OPS):
        g, w = got._set.c.point[op], want.c.point[op]
        if w.total_count == 0:
            continue
        span = max(abs(w.max_val - w.min_val), 1e-6)
        assert abs(g.min_val - w.min_val) <= 1e-5 * span + 1e-7 and abs(g.max_val - w.max_val) <= 1e-5 * span + 1e-7, cabi.OP_NAMES[op]
        moved = np.abs(got._set.counts[op] - want.counts[op]).sum()
        assert moved <= 0.02 * w.total_count, (cabi.OP_NAMES[op], moved, w.total_count)
    # x and the weights involve no arithmetic: exact
    np.testing.assert_array_equal(got._set.counts[cabi.X], want.counts[cabi.X])
    first_channel_row = cabi.NUM_OPS + 12
    np.testing.assert_array_equal(got._set.counts[first_channel_row:], want.counts[first_channel_row:])
    for use_pct in (False, True):
        p_got = ops.calculate_gru_quantitative_parameters_from_histograms(got, cfg, use_pct, 99.9)
        box = ol.ParamsBox(H, cfg_c)
        assert ref.ref_gru_params_from_histograms(C.byref(want.c), C.byref(cfg_c), int(use_pct), C.c_float(99.9), C.byref(box.c)) == 0
        for op in cabi.SCALAR_OPS:
            a_, b_ = getattr(p_got, f"scale_{cabi.OP_NAMES[op]}_"), box.c.scale[op]
            assert abs(a_ - b_) <= 0.03 * b_, (cabi.OP_NAMES[op], a_, b_)
        for name in ("W", "R", "bw", "br"):
            np.testing.assert_array_equal(np.array(getattr(p_got, f"scale_{name}_"), np.float32), box.chan[f"scale_{name}"])
    # the encodings drive a quantized forward
    out = ops.forward_quant_int_storage(False, T, B, I, H, dev(W), dev(R), dev(bw), dev(br), dev(x), dev(h0), p_got)
    assert torch.isfinite(out[0]).all()
