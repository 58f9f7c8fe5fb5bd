"""QuantLSTM histogram calibration: the library's host logic against the reference's own
``histogram.cc`` compiled into ``oracle/_ref/liblstm_ref.so`` (the compiled reference is the
checker for this part; there is no separate C restatement)."""
from __future__ import annotations

import ctypes as C

import numpy as np
import pytest

import lstm_lib as ll
from rx_met_b200 import _cabi_lstm as L
from test_gru_histogram_cpu import BATCHES

needs_ref = pytest.mark.skipif(not ll.have_ref(), reason="compiled reference not available")
_f32p = C.POINTER(C.c_float)


def one_hist(bins=2048):
    store = np.zeros(bins, np.float64)
    h = L.Histogram()
    h.counts, h.num_bins = store.ctypes.data_as(C.POINTER(C.c_double)), bins
    return h, store


def state(h, store):
    return (store.copy(), h.minimum, h.maximum, int(h.total_count))


def same(a, b):
    np.testing.assert_array_equal(a[0], b[0])
    assert a[1:] == b[1:], (a[1:], b[1:])


@needs_ref
@pytest.mark.parametrize("name", sorted(BATCHES))
@pytest.mark.parametrize("bins", [2048, 64])
def test_collect_merge_and_range_match_reference(name, bins):
    from rx_met_b200 import _quant_lstm
    lib, ref = _quant_lstm._library(), ll.lib("ref")
    rng = np.random.default_rng(sum(name.encode()) + 7)
    batches = BATCHES[name](rng)
    (a, sa), (b, sb) = one_hist(bins), one_hist(bins)
    for data in batches:
        p = data.ctypes.data_as(_f32p)
        assert lib.rxmet_lstm_histogram_collect_host(C.byref(a), p, C.c_uint64(data.size)) == 0, lib.rxmet_last_error()
        assert ref.ref_lstm_histogram_collect_host(C.byref(b), p, C.c_uint64(data.size)) == 0
        same(state(a, sa), state(b, sb))
    (c, sc), (d, sd) = one_hist(bins), one_hist(bins)
    for data in reversed(batches):
        p = data.ctypes.data_as(_f32p)
        lib.rxmet_lstm_histogram_collect_host(C.byref(c), p, C.c_uint64(data.size))
        ref.ref_lstm_histogram_collect_host(C.byref(d), p, C.c_uint64(data.size))
    assert lib.rxmet_lstm_histogram_merge(C.byref(a), C.byref(c)) == 0
    assert ref.ref_lstm_histogram_merge(C.byref(b), C.byref(d)) == 0
    same(state(a, sa), state(b, sb))
    if a.total_count == 0:
        return
    for bits, uns, sym in [(8, 0, 1), (8, 0, 0), (8, 1, 1), (8, 1, 0), (16, 0, 0), (4, 0, 1)]:
        for method, pct in [(0, 99.99), (1, 99.99), (1, 95.0), (1, 100.0)]:
            o1, o2 = (C.c_float * 2)(), (C.c_float * 2)()
            r1 = lib.rxmet_lstm_histogram_range(C.byref(a), bits, uns, sym, method, C.c_float(pct), C.byref(o1, 0), C.byref(o1, 4))
            r2 = ref.ref_lstm_histogram_range(C.byref(b), bits, uns, sym, method, C.c_float(pct), C.byref(o2, 0), C.byref(o2, 4))
            assert (r1 == 0) == (r2 == 0), (bits, uns, sym, method, pct)
            if r1 == 0:
                assert list(o1) == list(o2), (bits, uns, sym, method, pct)


@needs_ref
@pytest.mark.parametrize("cfg_kw", [dict(symmetric_activations=True), dict(), dict(parameter_granularity=L.PER_GATE),
                                    dict(parameter_granularity=L.PER_TENSOR, scale_mode=L.SCALE_POT2)])
@pytest.mark.parametrize("method", ["sqnr", "percentile"])
def test_params_from_reference_histograms_match_reference(cfg_kw, method):
    """The session's own collectors (filled by the reference) through the library's finalisation."""
    from rx_met_b200 import _quant_lstm
    lib = _quant_lstm._library()
    cfg = L.default_config(**cfg_kw)
    T, B, I, H = 6, 4, 5, 8
    p = ll.problem(T, B, I, H, seed=17)
    xs = np.stack([p["x"], ll.problem(T, B, I, H, seed=18)["x"] * 1.4])
    hs, want = ll.calibrate_hist(cfg, p, xs, method, 99.9, bins=256)
    ranges, _ = ll.calibrate("orc", cfg, p, xs)  # observed ranges (biases use them)
    got = L.ParamsBox(H)
    rc = lib.rxmet_lstm_params_from_histograms(C.byref(cfg), C.byref(ranges.struct), C.byref(hs.struct),
                                               0 if method == "sqnr" else 1, C.c_float(99.9), I, H, 1, *got.scale_ptrs(),
                                               C.byref(got.struct))
    assert rc == 0, lib.rxmet_last_error()
    for op in range(L.NUM_OPS):
        if op not in L.PARAMETER_OPS:
            assert got.struct.scale[op] == want.struct.scale[op] and got.struct.zero_point[op] == want.struct.zero_point[op], L.OP_NAMES[op]
    for k in range(4):
        np.testing.assert_array_equal(got.channel_scales[k], want.channel_scales[k])
