"""The allocation-free float forward against the regular entry point.

Some callers of this library run inside a callback that may not allocate (a runtime plugin's
enqueue, a hard-deadline loop, a process with a frozen memory pool), so they cannot hand over a
workspace.  rxmet_gru_forward_fp_static serves them from a scratch array built into the library.
This file checks that it returns exactly what rxmet_gru_forward_fp returns, twice in a row with
different inputs (the scratch keeps the previous call's contents), and that it refuses problems
larger than the built-in scratch.  It is named to be collected last, so that a run stopping at
the first failure has already exercised every other test.
"""
import ctypes as C

import numpy as np
import pytest

import oracle_lib as ol
from rx_met_b200 import _cabi as cabi

pytestmark = pytest.mark.gpu


def _run_static(lib, torch, W, R, bw, br, x, h0):
    T, B, I = x.shape
    H = R.shape[0]
    d = {k: (None if v is None else torch.from_numpy(np.ascontiguousarray(v)).cuda())
         for k, v in dict(W=W, R=R, bw=bw, br=br, x=x, h0=h0).items()}
    h = torch.full((T + 1, B, H), float("nan"), device="cuda")
    v = torch.full((T, B, 4 * H), float("nan"), device="cuda")
    p = lambda t: C.c_void_p(t.data_ptr()) if t is not None else None  # noqa: E731
    rc = lib.rxmet_gru_forward_fp_static(T, B, I, H, p(d["W"]), p(d["R"]), p(d["bw"]), p(d["br"]), p(d["x"]),
                                         p(d["h0"]), p(h), p(v), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return rc, h.cpu().numpy(), v.cpu().numpy()


def test_static_scratch_forward_matches_workspace_forward():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("the gpu tests need a CUDA device")
    import gpu_lib
    lib = cabi.load_library()
    lib.rxmet_static_scratch_bytes.restype = C.c_size_t
    limit = lib.rxmet_static_scratch_bytes()
    assert limit == 8 << 20

    # two calls in a row, different shapes and data: the second must not see the first one's scratch
    for seed, (T, B, I, H), with_h0 in ((41, (9, 6, 40, 128), True), (42, (7, 3, 31, 33), False)):
        W, R, bw, br, x, h0 = ol.gru_problem(seed, T, B, I, H, with_h0=with_h0)
        assert 4 * T * B * 3 * H <= limit
        rc, h_s, v_s = _run_static(lib, torch, W, R, bw, br, x, h0)
        assert rc == 0, lib.rxmet_last_error()
        h_w, v_w = gpu_lib.forward_float(W, R, bw, br, x, h0)
        # same kernels, same inputs: identical results (well inside the 1e-5 the float tests allow)
        assert np.array_equal(h_s, h_w) and np.array_equal(v_s, v_w)
        h_o, v_o = ol.forward_fp(W, R, bw, br, x, h0)
        assert np.abs(h_s - h_o).max() <= 1e-5 * max(np.abs(h_o).max(), 1e-30)
        assert np.abs(v_s - v_o).max() <= 1e-5 * max(np.abs(v_o).max(), 1e-30)

    # beyond the built-in scratch: a clear error and untouched outputs
    T, B, I, H = 100, 64, 8, 128
    assert 4 * T * B * 3 * H > limit
    W, R, bw, br, x, _ = ol.gru_problem(43, T, B, I, H)
    rc, h_s, _ = _run_static(lib, torch, W, R, bw, br, x, None)
    assert rc == -3 and b"built-in scratch" in lib.rxmet_last_error()
    assert np.isnan(h_s).all()
