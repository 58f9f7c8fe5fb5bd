"""GPU parity tests of the AIMET native kernels (C ABI) against the CPU restatement: bit-exact."""
import ctypes as C

import numpy as np
import pytest

import oracle_lib as ol
from rx_met_b200 import _cabi as cabi
from test_aimet_cpu import expected_qdq, fp, grid, orc_qdq

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("the gpu tests need a CUDA device")
    lib = cabi.load_library()
    lib.rxmet_aimet_minmax_workspace_bytes.restype = C.c_size_t
    return torch, lib


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def ptr(t):
    return C.c_void_p(t.data_ptr())


def stream(torch):
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def gpu_qdq(torch, lib, x, enc, dtype=0, offset_elems=0):
    buf = dev(torch, np.concatenate([np.zeros(offset_elems, x.dtype), x]))
    src = buf[offset_elems:]
    out = torch.empty_like(buf)
    dst = out[offset_elems:]
    rc = lib.rxmet_aimet_qdq(ptr(src), C.c_uint64(x.size), dtype, C.c_double(enc["min"]), C.c_double(enc["max"]),
                             C.c_double(enc["delta"]), 0, C.c_uint64(0), ptr(dst), stream(torch))
    torch.cuda.synchronize()
    assert rc == 0, lib.rxmet_last_error()
    return dst.cpu().numpy()


def test_qdq_known_answers_and_parity(env):
    torch, lib = env
    codes = np.array([-7.5, -3.5, -2.5, -1.5, -.5, .5, 1.5, 2.5, 3.5, 7.5], np.float32)
    for bits, scale in ((8, 2.0 ** -7), (16, 2.0 ** -15), (32, 2.0 ** -21)):
        for offset in (None, -13):
            enc = grid(bits, scale, offset)
            x = (codes * np.float32(scale)).astype(np.float32)
            assert np.array_equal(gpu_qdq(torch, lib, x, enc), expected_qdq(x, enc))
        enc = grid(bits, scale)
        x = np.array([np.nan, -np.inf, -scale, 0, scale, np.inf], np.float32)
        want = np.array([np.nan, enc["min"], -scale, 0, scale, enc["max"]], np.float32)
        assert np.array_equal(gpu_qdq(torch, lib, x, enc), want, equal_nan=True)
    rng = np.random.default_rng(1)
    for n in (1, 3, 4, 1023, 100003):          # empty tail, ragged tail, unaligned start
        x = (rng.standard_normal(n) * 3).astype(np.float32)
        x[::53] = np.nan
        for scale in (0.0231, 1.0 / 32767, .013007):
            enc = grid(8, scale, -31)
            for off in (0, 1, 3):
                assert np.array_equal(gpu_qdq(torch, lib, x, enc, offset_elems=off), orc_qdq(x, enc), equal_nan=True)
    # empty input is a no-op
    assert lib.rxmet_aimet_qdq(None, C.c_uint64(0), 0, C.c_double(0), C.c_double(1), C.c_double(0.1), 0, C.c_uint64(0),
                               None, stream(torch)) == 0
    # float64
    xd = (rng.standard_normal(5001) * 3)
    enc = grid(16, 0.00731)
    want = np.empty_like(xd)
    dp = lambda t: t.ctypes.data_as(C.POINTER(C.c_double))  # noqa: E731
    ol.oracle().orc_aimet_qdq_f64(dp(xd), C.c_uint64(xd.size), C.c_double(enc["min"]), C.c_double(enc["max"]),
                                  C.c_double(enc["delta"]), dp(want))
    assert np.array_equal(gpu_qdq(torch, lib, xd, enc, dtype=1), want)
    # stochastic rounding: every result is one of the two neighbouring grid points, unbiased on average
    x = np.full(200000, 0.3 * 0.01, np.float32)
    enc = grid(8, 0.01)
    src, out = dev(torch, x), dev(torch, np.zeros_like(x))
    assert lib.rxmet_aimet_qdq(ptr(src), C.c_uint64(x.size), 0, C.c_double(enc["min"]), C.c_double(enc["max"]),
                               C.c_double(enc["delta"]), 1, C.c_uint64(7), ptr(out), stream(torch)) == 0
    y = out.cpu().numpy() / np.float32(0.01)
    assert set(np.unique(np.rint(y))) <= {0.0, 1.0} and abs(y.mean() - 0.3) < 0.01


def test_per_channel_broadcast_and_fxp(env):
    torch, lib = env
    rng = np.random.default_rng(2)
    t = (rng.standard_normal((6, 5, 7)) * 2).astype(np.float32)
    ch = 6
    mn = np.linspace(-3, -1, ch).astype(np.float32)
    dl = np.linspace(0.01, 0.03, ch).astype(np.float32)
    mx = (mn + dl * 255).astype(np.float32)
    want = np.empty_like(t)
    ol.oracle().orc_aimet_qdq_per_channel_f32(fp(t), ch, C.c_int64(t.size), C.c_int64(35), fp(want), fp(mn), fp(mx), fp(dl))
    d = {k: dev(torch, v) for k, v in dict(t=t, mn=mn, mx=mx, dl=dl).items()}
    out = torch.empty_like(d["t"])
    assert lib.rxmet_aimet_qdq_per_channel(ptr(d["t"]), ch, C.c_int64(t.size), C.c_int64(35), 0, ptr(d["mn"]),
                                           ptr(d["mx"]), ptr(d["dl"]), ptr(out), stream(torch)) == 0
    assert np.array_equal(out.cpu().numpy(), want)
    # broadcast along the middle axis: encodings of shape (1, 5, 1)
    mn5, dl5 = mn[:5].copy(), dl[:5].copy()
    mx5 = (mn5 + dl5 * 255).astype(np.float32)
    in_str = (C.c_int64 * 3)(35, 7, 1)
    enc_str = (C.c_int64 * 3)(0, 1, 0)
    ol.oracle().orc_aimet_qdq_broadcast_f32(fp(t), fp(want), C.c_int64(t.size), 3, in_str, enc_str, fp(mn5), fp(mx5), fp(dl5))
    e = {k: dev(torch, v) for k, v in dict(mn=mn5, mx=mx5, dl=dl5).items()}
    assert lib.rxmet_aimet_qdq_broadcast(ptr(d["t"]), ptr(out), C.c_int64(t.size), 3, in_str, enc_str, 0, ptr(e["mn"]),
                                         ptr(e["mx"]), ptr(e["dl"]), stream(torch)) == 0
    assert np.array_equal(out.cpu().numpy(), want)
    # fixed-point quantize: half away from zero, optional shift to signed
    x = np.concatenate([(np.arange(-20, 21, dtype=np.float32) + 0.5) * np.float32(0.02), (rng.standard_normal(999) * 3).astype(np.float32)])
    enc = grid(8, 0.02, -31)
    src, dst = dev(torch, x), dev(torch, np.zeros_like(x))
    for signed in (0, 1):
        w = np.empty_like(x)
        ol.oracle().orc_aimet_to_fxp_f32(fp(x), C.c_uint64(x.size), C.c_double(enc["min"]), C.c_double(enc["max"]),
                                         C.c_double(enc["delta"]), C.c_double(enc["offset"]), 8, signed, fp(w))
        assert lib.rxmet_aimet_quantize_to_fxp(ptr(src), C.c_uint64(x.size), 0, C.c_double(enc["min"]), C.c_double(enc["max"]),
                                               C.c_double(enc["delta"]), C.c_double(enc["offset"]), 8, signed, ptr(dst),
                                               stream(torch)) == 0
        assert np.array_equal(dst.cpu().numpy(), w)


def test_minmax_and_histogram(env):
    torch, lib = env
    rng = np.random.default_rng(3)
    ws = torch.empty(lib.rxmet_aimet_minmax_workspace_bytes(), dtype=torch.uint8, device="cuda")
    for n, block in ((1, 1), (4096, 4096), (4096, 256), (4099, 7), (1 << 22, 1 << 22), (1000003, 1000003)):
        y = (rng.standard_normal(n) * 5).astype(np.float32)
        if n > 400:
            y[17] = np.nan
            y[300] = np.inf
        k = n // block
        wmin, wmax = np.empty(k, np.float32), np.empty(k, np.float32)
        ol.oracle().orc_aimet_minmax_f32(fp(y), C.c_uint64(n), C.c_uint64(block), fp(wmin), fp(wmax))
        src = dev(torch, y)
        gmin, gmax = torch.empty(k, device="cuda"), torch.empty(k, device="cuda")
        rc = lib.rxmet_aimet_minmax(ptr(src), C.c_uint64(n), C.c_uint64(block), 0, ptr(gmin), ptr(gmax), ptr(ws),
                                    C.c_size_t(ws.numel()), stream(torch))
        assert rc == 0, lib.rxmet_last_error()
        assert np.array_equal(gmin.cpu().numpy(), wmin) and np.array_equal(gmax.cpu().numpy(), wmax)
    pdf = lib.rxmet_aimet_pdf_size()
    assert pdf == 1536
    z = (rng.standard_normal(300001) * 2).astype(np.float32)
    z[11] = np.nan
    src = dev(torch, z)
    hist = torch.full((pdf,), 12345, dtype=torch.int32, device="cuda")  # must be overwritten
    for bucket, offset in ((0.01, -768), (0.0037, -100), (0.5, 0)):
        want = np.zeros(pdf, np.uint32)
        ol.oracle().orc_aimet_histogram_f32(fp(z), C.c_uint64(z.size), want.ctypes.data_as(C.POINTER(C.c_uint32)),
                                            C.c_double(bucket), offset)
        assert lib.rxmet_aimet_histogram(ptr(src), C.c_uint64(z.size), 0, C.c_double(bucket), offset, ptr(hist),
                                         stream(torch)) == 0
        assert np.array_equal(hist.cpu().numpy().astype(np.uint32), want)
    # total count is conserved when the range covers everything finite
    finite = z[np.isfinite(z)]
    bucket = float((finite.max() - finite.min()) / (pdf - 2))
    offset = int(np.floor(finite.min() / bucket))
    assert lib.rxmet_aimet_histogram(ptr(src), C.c_uint64(z.size), 0, C.c_double(bucket), offset, ptr(hist), stream(torch)) == 0
    assert int(hist.sum().item()) == finite.size


def test_histogram_analyzers_on_device_batches(env):
    """The running PDF statistics fed from device tensors (min/max and bucket counting on the GPU) and the
    TF-enhanced / percentile encodings derived from them, against the reference's analyzers driven on the
    same batches in CPU mode: identical bucket edges, probabilities and encodings."""
    from test_aimet_cpu import AIMET_REF, _Encoding, _histogram_cases, _new_pdf, _Pdf
    torch, lib = env
    if not AIMET_REF.exists():
        pytest.fail("the compiled reference checker (oracle/_ref/libaimet_ref.so) must travel with the tests")
    r = C.CDLL(str(AIMET_REF))
    lib.rxmet_aimet_pdf_workspace_bytes.restype = C.c_size_t
    lib.rxmet_aimet_pdf_update.argtypes = [C.POINTER(_Pdf), C.c_void_p, C.c_uint64, C.c_int, C.c_void_p, C.c_size_t, C.c_void_p]
    n = lib.rxmet_aimet_pdf_size()
    ws = torch.empty(lib.rxmet_aimet_pdf_workspace_bytes(), dtype=torch.uint8, device="cuda")
    rng = np.random.default_rng(5)
    cases = _histogram_cases()
    cases["large"] = [(rng.standard_normal(1 << 20) * (1 + i)).astype(np.float32) for i in range(3)]
    for name, batches in cases.items():
        s, x_left, pdf = _new_pdf(lib)
        for b in batches:
            src = dev(torch, b)
            rc = lib.rxmet_aimet_pdf_update(C.byref(s), ptr(src), b.size, 1, ptr(ws), ws.numel(), stream(torch))
            assert rc == 0, lib.rxmet_last_error()
        data = np.concatenate(batches)
        sizes = (C.c_uint64 * len(batches))(*[b.size for b in batches])
        want_pdf = np.zeros(2 * n, np.float64)
        for bw, sym, strict, uns, kind, percentile in ((8, 0, 0, 0, 0, 0.0), (8, 1, 0, 0, 0, 0.0), (4, 1, 1, 0, 0, 0.0),
                                                       (8, 0, 0, 0, 1, 99.9), (16, 1, 0, 1, 1, 99.0)):
            out = (C.c_double * 5)()
            bins = r.ref_aimet_histogram_encoding(kind, fp(data), sizes, len(batches), bw, sym, strict, uns,
                                                  C.c_float(percentile), out, want_pdf.ctypes.data_as(C.POINTER(C.c_double)))
            e = _Encoding()
            if kind == 0:
                rc = lib.rxmet_aimet_tf_enhanced_encoding(C.byref(s), bw, sym, strict, uns, C.byref(e))
            else:
                rc = lib.rxmet_aimet_percentile_encoding(C.byref(s), bw, sym, strict, uns, C.c_float(percentile), C.byref(e))
            assert rc == 0
            got = (e.min, e.max, e.delta, e.offset, float(e.bw))
            assert all(a == b for a, b in zip(got, out)), (name, bw, sym, strict, uns, kind, got, list(out))
        if bins:
            np.testing.assert_array_equal(x_left, want_pdf[:n], err_msg=name)
            np.testing.assert_array_equal(pdf, want_pdf[n:], err_msg=name)
