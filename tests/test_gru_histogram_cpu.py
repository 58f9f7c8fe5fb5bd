"""QuantGRU histogram calibration: the library's host logic (collector arithmetic, percentile and
SQNR searches, encodings from histograms) against the reference's own headers compiled into
``oracle/_ref/libgru_ref.so``.  No separate C restatement exists for this part; the compiled
reference is the checker."""
from __future__ import annotations

import ctypes as C

import numpy as np
import pytest

import oracle_lib as ol
from rx_met_b200 import _cabi as cabi

needs_ref = pytest.mark.skipif(ol.ref() is None, reason="compiled reference not available")
_f32p = C.POINTER(C.c_float)


def one_hist(bins=2048):
    store = np.zeros(bins, np.float32)
    h = cabi.Histogram()
    h.counts, h.num_bins = store.ctypes.data_as(_f32p), bins
    h.min_val, h.max_val = 3.4028234663852886e38, -3.4028234663852886e38
    h.observed_min, h.observed_max = h.min_val, h.max_val
    return h, store


def state(h, store):
    return (store.copy(), h.min_val, h.max_val, h.observed_min, h.observed_max, h.total_count)


def same(a, b):
    np.testing.assert_array_equal(a[0], b[0])
    assert a[1:] == b[1:], (a[1:], b[1:])


BATCHES = {
    "growing": lambda r: [r.standard_normal(5000).astype(np.float32) * s for s in (1.0, 0.5, 3.0, 3.0, 7.5)],
    "shifted": lambda r: [(r.random(3000).astype(np.float32) + o) for o in (0.0, 2.0, -1.5, 0.25)],
    "constant_then_spread": lambda r: [np.full(100, 0.75, np.float32), np.full(50, 0.75, np.float32),
                                       r.standard_normal(2000).astype(np.float32)],
    "zeros": lambda r: [np.zeros(64, np.float32), np.zeros(64, np.float32)],
    "nonfinite": lambda r: [np.array([1.0, np.nan, -2.0, np.inf, 0.5, -np.inf], np.float32),
                            np.array([np.nan, np.nan], np.float32), r.standard_normal(500).astype(np.float32)],
    "tiny_range": lambda r: [np.float32(1e-9) * r.standard_normal(300).astype(np.float32), r.standard_normal(300).astype(np.float32)],
    "sigmoid_like": lambda r: [(1 / (1 + np.exp(-4 * r.standard_normal(20000)))).astype(np.float32) for _ in range(3)],
}


@needs_ref
@pytest.mark.parametrize("name", sorted(BATCHES))
@pytest.mark.parametrize("bins", [2048, 128])
def test_collect_merge_and_calibrate_match_reference(name, bins):
    lib, ref = cabi.load_library(), ol.ref()
    rng = np.random.default_rng(sum(name.encode()))
    batches = BATCHES[name](rng)
    (a, sa), (b, sb) = one_hist(bins), one_hist(bins)
    for data in batches:
        p = data.ctypes.data_as(_f32p)
        assert lib.rxmet_histogram_collect_host(C.byref(a), p, C.c_uint64(data.size)) == 0, lib.rxmet_last_error()
        assert ref.ref_histogram_collect_host(C.byref(b), p, C.c_uint64(data.size)) == 0
        same(state(a, sa), state(b, sb))
    # merge a second collector built from the batches in reverse order
    (c, sc), (d, sd) = one_hist(bins), one_hist(bins)
    for data in reversed(batches):
        p = data.ctypes.data_as(_f32p)
        lib.rxmet_histogram_collect_host(C.byref(c), p, C.c_uint64(data.size))
        ref.ref_histogram_collect_host(C.byref(d), p, C.c_uint64(data.size))
    assert lib.rxmet_histogram_merge(C.byref(a), C.byref(c)) == 0
    assert ref.ref_histogram_merge(C.byref(b), C.byref(d)) == 0
    same(state(a, sa), state(b, sb))
    if a.total_count == 0:
        return
    for bits, uns, sym in [(8, 0, 1), (8, 0, 0), (8, 1, 1), (8, 1, 0), (16, 0, 0), (4, 0, 1)]:
        for use_pct, pct in [(0, 0.0), (1, 99.99), (1, 99.0)]:
            out1, out2 = (C.c_float * 3)(), (C.c_float * 3)()
            args = (bits, uns, sym, use_pct, C.c_float(pct))
            r1 = lib.rxmet_histogram_calibrate(C.byref(a), *args, C.byref(out1, 0), C.byref(out1, 4), C.byref(out1, 8))
            r2 = ref.ref_histogram_calibrate(C.byref(b), *args, C.byref(out2, 0), C.byref(out2, 4), C.byref(out2, 8))
            assert (r1 == 0) == (r2 == 0)
            if r1 == 0:
                assert list(out1) == list(out2), (bits, uns, sym, use_pct, pct)


@needs_ref
@pytest.mark.parametrize("granularity", [cabi.PER_CHANNEL, cabi.PER_TENSOR, cabi.PER_GATE])
@pytest.mark.parametrize("use_pot2,use_pct", [(False, False), (True, False), (False, True)])
def test_params_from_histograms_match_reference(granularity, use_pot2, use_pct):
    lib, ref = cabi.load_library(), ol.ref()
    T, B, I, H = 9, 5, 6, 8
    W, R, bw, br, x, h0 = ol.gru_problem(4, T, B, I, H, with_h0=True)
    cfg = ol.make_config(bits=8, symmetric=False, use_pot2=use_pot2, granularity=granularity)
    hs = cabi.HistogramSet(H, 256)
    h = np.zeros((T + 1, B, H), np.float32)
    v = np.zeros((T, B, 4 * H), np.float32)
    fp = lambda a_: a_.ctypes.data_as(_f32p)  # noqa: E731
    for scale in (1.0, 1.6):
        xs = np.ascontiguousarray(x * np.float32(scale))
        assert ref.ref_gru_forward_calibrate_hist(T, B, I, H, fp(W), fp(R), fp(bw), fp(br), fp(xs), fp(h0), C.byref(cfg),
                                                  C.byref(hs.c), fp(h), fp(v)) == 0, ref.ref_last_error()
    assert hs.is_valid()
    want, got = ol.ParamsBox(H, cfg), ol.ParamsBox(H, cfg)
    pct = C.c_float(99.9)
    assert ref.ref_gru_params_from_histograms(C.byref(hs.c), C.byref(cfg), int(use_pct), pct, C.byref(want.c)) == 0, ref.ref_last_error()
    assert lib.rxmet_gru_params_from_histograms(C.byref(hs.c), C.byref(cfg), int(use_pct), pct, C.byref(got.c)) == 0, lib.rxmet_last_error()
    for op in range(cabi.NUM_OPS):
        assert got.c.scale[op] == want.c.scale[op] and got.c.zero_point[op] == want.c.zero_point[op], cabi.OP_NAMES[op]
    for name in ("W", "R", "bw", "br"):
        np.testing.assert_array_equal(got.chan[f"scale_{name}"], want.chan[f"scale_{name}"], err_msg=name)


def test_histogram_argument_checks():
    lib = cabi.load_library()
    h = cabi.Histogram()
    assert lib.rxmet_histogram_reset(C.byref(h)) == -1
    a, store = one_hist(16)
    out = (C.c_float * 3)()
    assert lib.rxmet_histogram_calibrate(C.byref(a), 8, 0, 1, 0, C.c_float(0), C.byref(out, 0), C.byref(out, 4), C.byref(out, 8)) == -1
    assert b"invalid" in lib.rxmet_last_error()
    assert lib.rxmet_histogram_workspace_bytes(2048) > 8192


def test_quant_params_conversion_is_kept_until_an_attribute_is_assigned():
    """The binding converts GRUQuantParams to the C struct once and keeps it; assigning any attribute of
    the parameters or of their bit-width configuration makes the next call convert again."""
    import rx_met_b200.gru_interface_binding as binding

    p = binding.GRUQuantParams()
    p.hidden_ = 2
    for name in ("W", "R", "bw", "br"):
        setattr(p, f"scale_{name}_", [0.5] * 6)
    p.scale_x_ = 0.25
    c1, keep1 = p._to_c()
    c2, _ = p._to_c()
    assert c1 is c2 and c1.scale[cabi.X] == 0.25 and keep1[0][5] == 0.5
    p.scale_x_ = 0.125
    c3, _ = p._to_c()
    assert c3 is not c1 and c3.scale[cabi.X] == 0.125
    p.bitwidth_config_.x_ = 16
    c4, _ = p._to_c()
    assert c4 is not c3 and c4.config.bits[cabi.X] == 16
    p.scale_W_ = [0.75] * 6
    c5, keep5 = p._to_c()
    assert c5 is not c4 and keep5[0][0] == 0.75
    cfg = binding.OperatorQuantConfig()
    cfg.h_ = 12
    p.bitwidth_config_ = cfg
    assert p._to_c()[0].config.bits[cabi.H] == 12
