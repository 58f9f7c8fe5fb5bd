"""CPU tests of the AIMET native restatement: against the reference's own CPU sources (where the
compiled checker is present) and against the known-answer cases of the reference's
tests/integration/test_native_qdq_alignment.py."""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest

import oracle_lib as ol

ROOT = Path(__file__).resolve().parent.parent
AIMET_REF = ROOT / "oracle" / "_ref" / "libaimet_ref.so"


def fp(a):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def ref():
    return C.CDLL(str(AIMET_REF)) if AIMET_REF.exists() else None


def grid(bits, scale, offset=None):
    """Encoding of a `bits`-wide grid: symmetric signed when offset is None."""
    steps = 2 ** bits - 1
    if offset is None:
        offset = -(2 ** (bits - 1))
    return dict(min=scale * offset, max=scale * (offset + steps), delta=scale, offset=offset, bw=bits)


def orc_qdq(x, enc):
    out = np.empty_like(x)
    ol.oracle().orc_aimet_qdq_f32(fp(x), C.c_uint64(x.size), C.c_double(enc["min"]), C.c_double(enc["max"]),
                                  C.c_double(enc["delta"]), fp(out))
    return out


def expected_qdq(x, enc):
    """The contract of the reference's alignment test: clamp, multiply by the float32-rounded
    reciprocal, round half to even, multiply back; all in float32."""
    lo, hi, d = np.float32(enc["min"]), np.float32(enc["max"]), np.float32(enc["delta"])
    inv = np.float32(1.0) / d
    y = np.rint(np.clip(x, lo, hi) * inv).astype(np.float32) * d
    return np.where(np.isnan(x), x, y).astype(np.float32)


def test_ties_to_even_reciprocal_nan_and_infinity():
    codes = np.array([-7.5, -3.5, -2.5, -1.5, -.5, .5, 1.5, 2.5, 3.5, 7.5], np.float32)
    for bits, scale in ((8, 2.0 ** -7), (16, 2.0 ** -15), (32, 2.0 ** -21)):
        for offset in (None, -13):
            enc = grid(bits, scale, offset)
            x = (codes * np.float32(scale)).astype(np.float32)
            got = orc_qdq(x, enc)
            assert np.array_equal(got, expected_qdq(x, enc))
            if offset is None:  # half codes land on the even neighbour
                assert np.array_equal(got / np.float32(scale), np.array([-8, -4, -2, -2, -0., 0, 2, 2, 4, 8], np.float32))
    codes = np.arange(-63, 64, dtype=np.float32) + .5
    for scale in (1. / 32767, .013007, .027019):
        x = codes * np.float32(scale)
        enc = grid(16, scale)
        assert np.array_equal(orc_qdq(x, enc), expected_qdq(x, enc))
    for bits, scale in ((8, 2.0 ** -7), (16, 2.0 ** -15), (32, 2.0 ** -21)):
        enc = grid(bits, scale)
        x = np.array([np.nan, -np.inf, -scale, 0, scale, np.inf], np.float32)
        got = orc_qdq(x, enc)
        want = np.array([np.nan, enc["min"], -scale, 0, scale, enc["max"]], np.float32)
        assert np.array_equal(got, want, equal_nan=True)
    small = np.array([-257, -65, -7, -3, -1, 0, 1, 3, 7, 65, 257], np.float32) * np.float32(2.0 ** -21)
    assert np.array_equal(orc_qdq(small, grid(32, 2.0 ** -21)), small)


@pytest.mark.skipif(ref() is None, reason="compiled reference not present on this machine")
def test_restatement_matches_compiled_reference():
    r, o = ref(), ol.oracle()
    rng = np.random.default_rng(0)
    x = (rng.standard_normal(20011) * 3).astype(np.float32)
    x[::97] = np.nan
    x[5::211] = np.inf
    x[7::311] = -np.inf
    for bits, scale, offset in ((8, 0.0231, None), (8, 0.017, -31), (16, 1.0 / 32767, None), (4, 0.3, -3)):
        enc = grid(bits, scale, offset)
        a, b = np.empty_like(x), np.empty_like(x)
        assert r.ref_aimet_qdq_f32(fp(x), C.c_uint64(x.size), C.c_double(enc["min"]), C.c_double(enc["max"]),
                                   C.c_double(enc["delta"]), fp(a)) == 0
        o.orc_aimet_qdq_f32(fp(x), C.c_uint64(x.size), C.c_double(enc["min"]), C.c_double(enc["max"]),
                            C.c_double(enc["delta"]), fp(b))
        assert np.array_equal(a, b, equal_nan=True)
        finite = np.nan_to_num(x, nan=0.0, posinf=100.0, neginf=-100.0)
        for signed in (0, 1):
            assert r.ref_aimet_to_fxp_f32(fp(finite), C.c_uint64(x.size), C.c_double(enc["min"]), C.c_double(enc["max"]),
                                          C.c_double(enc["delta"]), C.c_double(enc["offset"]), bits, signed, fp(a)) == 0
            o.orc_aimet_to_fxp_f32(fp(finite), C.c_uint64(x.size), C.c_double(enc["min"]), C.c_double(enc["max"]),
                                   C.c_double(enc["delta"]), C.c_double(enc["offset"]), bits, signed, fp(b))
            assert np.array_equal(a, b)
    # double precision
    xd = x.astype(np.float64)
    ad, bd = np.empty_like(xd), np.empty_like(xd)
    enc = grid(16, 0.00731)
    dp = lambda t: t.ctypes.data_as(C.POINTER(C.c_double))  # noqa: E731
    assert r.ref_aimet_qdq_f64(dp(xd), C.c_uint64(xd.size), C.c_double(enc["min"]), C.c_double(enc["max"]),
                               C.c_double(enc["delta"]), dp(ad)) == 0
    o.orc_aimet_qdq_f64(dp(xd), C.c_uint64(xd.size), C.c_double(enc["min"]), C.c_double(enc["max"]),
                        C.c_double(enc["delta"]), dp(bd))
    assert np.array_equal(ad, bd, equal_nan=True)
    # per channel and broadcast
    t = (rng.standard_normal((6, 5, 7)) * 2).astype(np.float32)
    ch = 6
    mn = np.linspace(-3, -1, ch).astype(np.float32)
    dl = np.linspace(0.01, 0.03, ch).astype(np.float32)
    mx = (mn + dl * 255).astype(np.float32)
    off = np.zeros(ch, np.float32)
    a, b = np.empty_like(t), np.empty_like(t)
    assert r.ref_aimet_qdq_per_channel_f32(fp(t), ch, t.size, 35, fp(a), fp(mn), fp(mx), fp(dl), fp(off)) == 0
    o.orc_aimet_qdq_per_channel_f32(fp(t), ch, C.c_int64(t.size), C.c_int64(35), fp(b), fp(mn), fp(mx), fp(dl))
    assert np.array_equal(a, b)
    shape = (C.c_int64 * 3)(6, 5, 7)
    enc_shape = (C.c_int64 * 3)(6, 1, 1)
    d3 = lambda v: (C.c_double * ch)(*[float(q) for q in v])  # noqa: E731
    assert r.ref_aimet_qdq_broadcast_f32(fp(t), fp(a), ch, d3(mn), d3(mx), d3(dl), 3, shape, enc_shape) == 0
    in_str = (C.c_int64 * 3)(35, 7, 1)
    enc_str = (C.c_int64 * 3)(1, 0, 0)
    o.orc_aimet_qdq_broadcast_f32(fp(t), fp(b), C.c_int64(t.size), 3, in_str, enc_str, fp(mn), fp(mx), fp(dl))
    assert np.array_equal(a, b)
    # min/max, whole tensor and per block; NaN never wins, infinities do
    y = (rng.standard_normal(4096) * 5).astype(np.float32)
    y[17] = np.nan
    y[300] = np.inf
    for block in (4096, 256, 7):
        n = y.size // block
        amin, amax, bmin, bmax = (np.empty(n, np.float32) for _ in range(4))
        assert r.ref_aimet_minmax_f32(fp(y), C.c_uint64(y.size), C.c_uint64(block), fp(amin), fp(amax)) == 0
        o.orc_aimet_minmax_f32(fp(y), C.c_uint64(y.size), C.c_uint64(block), fp(bmin), fp(bmax))
        assert np.array_equal(amin, bmin) and np.array_equal(amax, bmax)
    # histogram
    pdf = r.ref_aimet_pdf_size()
    assert pdf == 1536
    z = (rng.standard_normal(50000) * 2).astype(np.float32)
    z[11] = np.nan
    for bucket, offset in ((0.01, -768), (0.0037, -100), (0.5, 0)):
        ha, hb = np.zeros(pdf, np.uint32), np.zeros(pdf, np.uint32)
        u32 = lambda t: t.ctypes.data_as(C.POINTER(C.c_uint32))  # noqa: E731
        assert r.ref_aimet_histogram_f32(fp(z), C.c_uint64(z.size), u32(ha), C.c_double(bucket), offset, 1) == 0
        o.orc_aimet_histogram_f32(fp(z), C.c_uint64(z.size), u32(hb), C.c_double(bucket), offset)
        assert np.array_equal(ha, hb) and ha.sum() > 0


class _Encoding(C.Structure):
    _fields_ = [("min", C.c_double), ("max", C.c_double), ("delta", C.c_double), ("offset", C.c_double), ("bw", C.c_int32)]


@pytest.mark.skipif(ref() is None, reason="compiled reference not available")
def test_library_encodings_match_the_reference():
    """Host logic of the shipped library (range -> encoding, min/max statistics -> encoding)."""
    from rx_met_b200 import _cabi
    lib, r = _cabi.load_library(), ref()
    rng = np.random.default_rng(3)
    ranges = [(-1.0, 1.0), (0.0, 6.0), (-3.5, 0.25), (0.0, 0.0), (-1e-9, 1e-9), (-1e38, 3e38), (0.2, 5.0), (-7.0, -2.0)]
    ranges += [tuple(sorted(rng.standard_normal(2) * 10.0 ** rng.integers(-3, 4))) for _ in range(40)]
    modes = [(0, 0, 0), (1, 0, 0), (1, 1, 0), (1, 0, 1)]
    for lo, hi in ranges:
        for bw in (2, 4, 8, 16, 31):
            for sym, strict, uns in modes:
                e = _Encoding()
                out = (C.c_double * 5)()
                assert lib.rxmet_aimet_compute_encoding(bw, C.c_double(lo), C.c_double(hi), sym, strict, uns, C.byref(e)) == 0
                assert r.ref_aimet_compute_encoding(bw, C.c_double(lo), C.c_double(hi), sym, strict, uns, out) == 0
                got = (e.min, e.max, e.delta, e.offset, float(e.bw))
                assert all(a == b or (a != a and b != b) for a, b in zip(got, out)), (lo, hi, bw, sym, strict, uns, got, list(out))
                lo32, hi32 = np.float32(lo), np.float32(hi)
                assert lib.rxmet_aimet_minmax_encoding(bw, 0, C.c_double(lo32), C.c_double(hi32), sym, strict, uns, C.byref(e)) == 0
                assert r.ref_aimet_minmax_encoding(bw, C.c_float(lo32), C.c_float(hi32), sym, strict, uns, out) == 0
                got = (e.min, e.max, e.delta, e.offset, float(e.bw))
                assert all(a == b or (a != a and b != b) for a, b in zip(got, out)), ("minmax", lo, hi, bw, sym, strict, uns)
    e = _Encoding()
    assert lib.rxmet_aimet_compute_encoding(0, C.c_double(0), C.c_double(1), 0, 0, 0, C.byref(e)) == -1


class _Pdf(C.Structure):
    _fields_ = [("x_left", C.POINTER(C.c_double)), ("pdf", C.POINTER(C.c_double)), ("initialized", C.c_int32),
                ("iterations", C.c_int32), ("updated", C.c_int32)]


def _new_pdf(lib):
    n = lib.rxmet_aimet_pdf_size()
    x_left, pdf = np.zeros(n, np.float64), np.zeros(n, np.float64)
    s = _Pdf(x_left.ctypes.data_as(C.POINTER(C.c_double)), pdf.ctypes.data_as(C.POINTER(C.c_double)), 0, 0, 0)
    assert lib.rxmet_aimet_pdf_reset(C.byref(s)) == 0
    return s, x_left, pdf


def _histogram_cases():
    rng = np.random.default_rng(11)
    cases = {
        "normal": [rng.standard_normal(4000).astype(np.float32) for _ in range(3)],
        "positive": [np.abs(rng.standard_normal(3000)).astype(np.float32) * 4 for _ in range(2)],
        "heavy_tail": [(rng.standard_t(2, 5000) * 0.3).astype(np.float32)],
        "shifted": [(rng.standard_normal(2500) * 0.2 + 5).astype(np.float32), (rng.standard_normal(2500) * 0.2 + 4).astype(np.float32)],
        "zero_then_data": [np.zeros(100, np.float32), rng.standard_normal(1000).astype(np.float32)],
        "constant": [np.full(64, 2.5, np.float32)],
        "outliers_later": [rng.standard_normal(2000).astype(np.float32), (rng.standard_normal(2000) * 30).astype(np.float32)],
        "only_zero": [np.zeros(50, np.float32)],
    }
    return cases


@pytest.mark.skipif(ref() is None, reason="compiled reference not available")
def test_histogram_analyzers_match_the_reference():
    """Running PDF statistics, TF-enhanced and percentile encodings of the shipped library against the
    reference's TfEnhancedEncodingAnalyzer<float> / PercentileEncodingAnalyzer<float> driven in CPU mode."""
    from rx_met_b200 import _cabi
    lib, r = _cabi.load_library(), ref()
    n = lib.rxmet_aimet_pdf_size()
    lib.rxmet_aimet_pdf_update_host.argtypes = [C.POINTER(_Pdf), C.POINTER(C.c_float), C.c_uint64, C.c_int]
    modes = [(0, 0, 0), (1, 0, 0), (1, 1, 0), (1, 0, 1)]
    for name, batches in _histogram_cases().items():
        s, x_left, pdf = _new_pdf(lib)
        for b in batches:
            assert lib.rxmet_aimet_pdf_update_host(C.byref(s), fp(b), b.size, 1) == 0, name
        data = np.concatenate(batches)
        sizes = (C.c_uint64 * len(batches))(*[b.size for b in batches])
        want_pdf = np.zeros(2 * n, np.float64)
        for bw in (4, 8, 16):
            for sym, strict, uns in modes:
                for kind, percentile in ((0, 0.0), (1, 99.9), (1, 100.0), (1, 90.0)):
                    out = (C.c_double * 5)()
                    bins = r.ref_aimet_histogram_encoding(kind, fp(data), sizes, len(batches), bw, sym, strict, uns,
                                                          C.c_float(percentile), out,
                                                          want_pdf.ctypes.data_as(C.POINTER(C.c_double)))
                    assert bins >= 0
                    e = _Encoding()
                    if kind == 0:
                        rc = lib.rxmet_aimet_tf_enhanced_encoding(C.byref(s), bw, sym, strict, uns, C.byref(e))
                    else:
                        rc = lib.rxmet_aimet_percentile_encoding(C.byref(s), bw, sym, strict, uns, C.c_float(percentile), C.byref(e))
                    assert rc == 0
                    got = (e.min, e.max, e.delta, e.offset, float(e.bw))
                    assert all(a == b for a, b in zip(got, out)), (name, bw, sym, strict, uns, kind, percentile, got, list(out))
        if bins:
            np.testing.assert_array_equal(x_left, want_pdf[:n], err_msg=name)
            np.testing.assert_array_equal(pdf, want_pdf[n:], err_msg=name)
        else:
            assert not s.initialized, name


def test_histogram_analyzers_before_any_batch():
    from rx_met_b200 import _cabi
    lib = _cabi.load_library()
    s, _, _ = _new_pdf(lib)
    e = _Encoding()
    assert lib.rxmet_aimet_tf_enhanced_encoding(C.byref(s), 8, 0, 0, 0, C.byref(e)) == 0
    assert (e.min, e.max, e.delta, e.offset, e.bw) == (0.0, 0.0, 0.0, 0.0, 0)  # the failure marker
    assert lib.rxmet_aimet_percentile_encoding(None, 8, 0, 0, 0, C.c_float(99.0), C.byref(e)) == -1


@pytest.mark.skipif(ref() is None, reason="compiled reference not available")
def test_plain_tf_analyzer_is_the_minmax_encoding_of_the_running_range():
    """TfEncodingAnalyzer<float> keeps a running min / max in double that starts at zero; its encoding is the
    library's min/max encoding of that range, so the analyzer binds to rxmet_aimet_minmax (per batch) and
    rxmet_aimet_minmax_encoding (double statistics)."""
    from rx_met_b200 import _cabi
    lib, r = _cabi.load_library(), ref()
    modes = [(0, 0, 0), (1, 0, 0), (1, 1, 0), (1, 0, 1)]
    for name, batches in _histogram_cases().items():
        data = np.concatenate(batches)
        sizes = (C.c_uint64 * len(batches))(*[b.size for b in batches])
        lo = min(0.0, min(float(b.min()) for b in batches))
        hi = max(0.0, max(float(b.max()) for b in batches))
        for bw in (4, 8, 16):
            for sym, strict, uns in modes:
                out = (C.c_double * 5)()
                assert r.ref_aimet_tf_encoding(fp(data), sizes, len(batches), bw, sym, strict, uns, out) == 0
                e = _Encoding()
                assert lib.rxmet_aimet_minmax_encoding(bw, 1, C.c_double(lo), C.c_double(hi), sym, strict, uns, C.byref(e)) == 0
                got = (e.min, e.max, e.delta, e.offset, float(e.bw))
                assert all(a == b for a, b in zip(got, out)), (name, bw, sym, strict, uns, got, list(out))
