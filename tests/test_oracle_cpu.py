"""CPU tests: the C restatement against the golden fixtures and (where present) the compiled
reference, known-answer vectors from the reference's own tests, the host-side parameter
derivation of the shipped library against the restatement, and the C-ABI symbol table."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

import oracle_lib as ol
from rx_met_b200 import _cabi as cabi

ROOT = Path(__file__).resolve().parent.parent
GOLDEN = sorted((ROOT / "tests" / "golden").glob("gru_*.npz"))


def load_case(path):
    g = np.load(path)
    seed, T, B, I, H, bits, sym, pot, gran, with_h0 = (int(v) for v in g["meta"])
    cfg = ol.make_config(bits=bits, symmetric=bool(sym), use_pot2=bool(pot), granularity=gran)
    h0 = g["h0"] if with_h0 else None
    return g, cfg, (T, B, I, H), h0


def dict_from(g, prefix):
    return {k[len(prefix):]: g[k] for k in g.files if k.startswith(prefix)}


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: p.stem)
def test_restatement_matches_golden(path):
    """Fixtures were produced by the reference's CPU build; everything must match bit for bit."""
    g, cfg, (T, B, I, H), h0 = load_case(path)
    ranges = ol.RangesBox(H)
    h_fp, v_fp = ol.forward_calibrate_minmax("orc", g["W"], g["R"], g["bw"], g["br"], g["x"], h0, ranges)
    assert np.array_equal(h_fp, g["h_fp"]) and np.array_equal(v_fp, g["v_fp"])
    for k, v in ranges.as_dict().items():
        assert np.array_equal(v, g[f"range_{k}"]), k
    params = ol.params_from_ranges("orc", ranges, cfg)
    for k, v in params.as_dict().items():
        assert np.array_equal(v, g[f"param_{k}"]), k
    assert np.array_equal(ol.build_luts("orc", params), g["luts"])
    fwd = ol.forward_quant("orc", g["W"], g["R"], g["bw"], g["br"], g["x"], h0, params)
    for k, v in dict_from(g, "fwd_").items():
        assert np.array_equal(fwd[k], v), k


@pytest.mark.skipif(ol.ref() is None, reason="compiled reference not present on this machine")
@pytest.mark.parametrize("bits,sym,pot,gran", [(8, False, False, 2), (8, True, True, 0), (16, False, False, 1),
                                               (4, False, True, 2), (12, True, False, 2)])
@pytest.mark.parametrize("shape", [(5, 2, 3, 4), (7, 3, 31, 33), (12, 2, 40, 64)])
def test_restatement_matches_compiled_reference(bits, sym, pot, gran, shape):
    T, B, I, H = shape
    W, R, bw, br, x, h0 = ol.gru_problem(100 + bits + T, T, B, I, H, with_h0=(T % 2 == 1))
    cfg = ol.make_config(bits=bits, symmetric=sym, use_pot2=pot, granularity=gran)
    ro, rr = ol.RangesBox(H), ol.RangesBox(H)
    ho, vo = ol.forward_calibrate_minmax("orc", W, R, bw, br, x, h0, ro)
    hr, vr = ol.forward_calibrate_minmax("ref", W, R, bw, br, x, h0, rr, cfg)
    assert np.array_equal(ho, hr) and np.array_equal(vo, vr)
    for k in ro.as_dict():
        assert np.array_equal(ro.as_dict()[k], rr.as_dict()[k]), k
    po, pr = ol.params_from_ranges("orc", ro, cfg), ol.params_from_ranges("ref", rr, cfg)
    for k in po.as_dict():
        assert np.array_equal(po.as_dict()[k], pr.as_dict()[k]), k
    assert np.array_equal(ol.build_luts("orc", po), ol.build_luts("ref", pr))
    fo, fr = ol.forward_quant("orc", W, R, bw, br, x, h0, po), ol.forward_quant("ref", W, R, bw, br, x, h0, pr)
    for k in fr:
        assert np.array_equal(fo[k], fr[k]), k


def test_rounding_known_answers():
    """Half ties go to even and the zero point is added after rounding, for odd zero points too
    (the cases of the reference's tests/recurrent/test_gru_rounding.py)."""
    lib = ol.oracle()
    lib.orc_rshift_round.restype = C.c_int64
    lib.orc_rshift_round.argtypes = [C.c_int64, C.c_int]
    assert [lib.orc_rshift_round(v, 1) for v in (1, 3, 5, -1, -3, -5, 2, -2)] == [0, 2, 2, 0, -2, -2, 1, -1]
    assert lib.orc_rshift_round(6, 2) == 2 and lib.orc_rshift_round(10, 2) == 2 and lib.orc_rshift_round(-10, 2) == -2
    assert lib.orc_rshift_round(3, -2) == 12 and lib.orc_rshift_round(7, 0) == 7

    class BW(C.Structure):
        _fields_ = [("bits", C.c_int32), ("is_unsigned", C.c_int32)]

    lib.orc_quantize.restype = C.c_int32
    lib.orc_quantize.argtypes = [C.c_float, C.c_float, C.c_int32, BW, C.POINTER(C.c_uint8)]
    keep = C.c_uint8()
    q = lambda v, s, zp, bits=8, uns=0: lib.orc_quantize(v, s, zp, BW(bits, uns), C.byref(keep))  # noqa: E731
    # round(0.5) = 0, round(1.5) = 2, round(2.5) = 2 before the (odd) zero point is added
    assert [q(v, 1.0, 3) for v in (0.5, 1.5, 2.5, -0.5, -1.5)] == [3, 5, 5, 3, 1]
    assert [q(v, 1.0, -7) for v in (0.5, 1.5, 2.5)] == [-7, -5, -5]
    # saturation happens before the integer cast and reports keep = 0
    assert q(1e30, 1.0, 0) == 127 and keep.value == 0
    assert q(-1e30, 1.0, 0) == -128 and keep.value == 0
    assert q(300.0, 1.0, 0, 8, 1) == 255 and keep.value == 0
    assert q(12.0, 1.0, 0) == 12 and keep.value == 1
    if ol.ref() is not None:
        r = ol.ref()
        for v, s, zp in [(0.5, 1.0, 3), (2.5, 1.0, 3), (-1.5, 1.0, -7), (0.37, 0.01, 5), (1e30, 1.0, 0)]:
            assert q(v, s, zp) == r.ref_quantize(v, s, zp, 8, 0)
        for v in (1, 3, 5, -3, 1 << 40, -(1 << 40) + 1):
            for n in (1, 2, 7, 33):
                assert lib.orc_rshift_round(v, n) == r.ref_rshift_round_i64(v, n)


def test_mshift_encoding_known_answers():
    lib = ol.oracle()
    m, s = C.c_int32(), C.c_int32()
    for scale, expect in [(1.0, (32768, 15)), (0.5, (32768, 16)), (0.75, (49152, 16)), (3.0, (49152, 14))]:
        assert lib.orc_encode_mshift(C.c_float(scale), C.byref(m), C.byref(s)) == 0
        assert (m.value, s.value) == expect
        assert m.value * 2.0 ** -s.value == scale
    rng = np.random.default_rng(0)
    for scale in np.exp(rng.uniform(-20, 5, 200)).astype(np.float32):
        assert lib.orc_encode_mshift(C.c_float(scale), C.byref(m), C.byref(s)) == 0
        assert 32768 <= m.value <= 65535
        assert abs(m.value * 2.0 ** -s.value - scale) <= scale * 2.0 ** -16
        if ol.ref() is not None:
            rm, rs = C.c_int32(), C.c_int32()
            ol.ref().ref_encode_mshift(C.c_float(scale), C.byref(rm), C.byref(rs))
            assert (rm.value, rs.value) == (m.value, s.value)
    assert lib.orc_encode_mshift(C.c_float(0.0), C.byref(m), C.byref(s)) != 0


def test_storage_dtypes_agree_and_inference_equals_training_codes():
    """Within the integer carrier, codes do not depend on whether masks are recorded
    (the bit-exactness the reference's tests/test_cpu_ptq.py asserts across its storage modes)."""
    W, R, bw, br, x, h0 = ol.gru_problem(5, 6, 3, 5, 8, with_h0=True)
    cfg = ol.make_config(bits=8, symmetric=False)
    rg = ol.RangesBox(8)
    ol.forward_calibrate_minmax("orc", W, R, bw, br, x, h0, rg)
    p = ol.params_from_ranges("orc", rg, cfg)
    a = ol.forward_quant("orc", W, R, bw, br, x, h0, p, training=True)
    b = ol.forward_quant("orc", W, R, bw, br, x, h0, p, training=False)
    for k in ("h", "v", "h_q", "v_q", "x_q", "W_q", "R_q"):
        assert np.array_equal(a[k], b[k]), k
    # dequantized outputs are the codes on the decoded M*2^-shift grid
    eff = C.c_float()
    assert ol.oracle().orc_gru_decode_effective_scale(C.c_float(p.c.scale[cabi.H]), 0, C.byref(eff)) == 0
    assert np.array_equal(a["h"], (a["h_q"] - p.c.zero_point[cabi.H]).astype(np.float32) * np.float32(eff.value))


def test_backward_oracle_matches_finite_differences_of_float_gru():
    """The float backward restatement is the exact derivative of the float forward."""
    T, B, I, H = 4, 2, 3, 5
    W, R, bw, br, x, h0 = ol.gru_problem(9, T, B, I, H, with_h0=True)
    h, v = ol.forward_fp(W, R, bw, br, x, h0)
    rng = np.random.default_rng(1)
    dh_new = np.zeros((T + 1, B, H), np.float32)
    dh_new[1:] = rng.standard_normal((T, B, H)).astype(np.float32)
    g = ol.backward_fp(W, R, bw, br, x, dh_new, h, v)

    def loss(W_, R_, bw_, br_, x_, h0_):
        hh, _ = ol.forward_fp(W_.astype(np.float32), R_.astype(np.float32), bw_.astype(np.float32),
                              br_.astype(np.float32), x_.astype(np.float32), h0_.astype(np.float32))
        return float((hh[1:].astype(np.float64) * dh_new[1:]).sum())

    args = [W, R, bw, br, x, h0]
    grads = [g["dW"], g["dR"], g["dbw"], g["dbr"], g["dx"], g["dh0"]]
    eps = 1e-2
    for which, (a, ga) in enumerate(zip(args, grads)):
        flat = a.reshape(-1)
        for idx in rng.choice(flat.size, size=min(6, flat.size), replace=False):
            hi = [t.copy() for t in args]
            lo = [t.copy() for t in args]
            hi[which].reshape(-1)[idx] += eps
            lo[which].reshape(-1)[idx] -= eps
            fd = (loss(*hi) - loss(*lo)) / (2 * eps)
            assert abs(fd - ga.reshape(-1)[idx]) < 5e-3 * max(1.0, abs(fd)), (which, idx, fd, ga.reshape(-1)[idx])


def test_backward_masks_zero_the_clamped_paths():
    """STE: a cleared keep-mask removes exactly that element's contribution
    (the identities of the reference's tests/recurrent/test_gru_autograd.py)."""
    T, B, I, H = 3, 2, 4, 6
    W, R, bw, br, x, h0 = ol.gru_problem(21, T, B, I, H, with_h0=True)
    cfg = ol.make_config(bits=8, symmetric=False)
    rg = ol.RangesBox(H)
    ol.forward_calibrate_minmax("orc", W, R, bw, br, x, h0, rg)
    p = ol.params_from_ranges("orc", rg, cfg)
    f = ol.forward_quant("orc", W, R, bw, br, x, h0, p)
    dh_new = np.zeros((T + 1, B, H), np.float32)
    dh_new[1:] = np.random.default_rng(3).standard_normal((T, B, H)).astype(np.float32)
    masks = f["masks"]
    for a in masks.arr.values():
        a[...] = 1
    base = ol.backward_quant(f, dh_new, f["h"], f["v"], p, masks)
    none = ol.backward_quant(f, dh_new, f["h"], f["v"], p, None)
    for k in base:
        assert np.array_equal(base[k], none[k]), k
    masks.arr["x"][1, 0, 2] = 0
    masks.arr["W"][2, 5] = 0
    masks.arr["R"][1, 7] = 0
    masks.arr["bw"][3] = 0
    masks.arr["br"][4] = 0
    masks.arr["h0"][1, 2] = 0
    g = ol.backward_quant(f, dh_new, f["h"], f["v"], p, masks)
    assert g["dx"][1, 0, 2] == 0 and g["dW"][2, 5] == 0 and g["dR"][1, 7] == 0
    assert g["dbw"][3] == 0 and g["dbr"][4] == 0 and g["dh0"][1, 2] == 0
    for k, idx in (("dx", (1, 0, 2)), ("dW", (2, 5)), ("dR", (1, 7)), ("dbw", (3,)), ("dbr", (4,)), ("dh0", (1, 2))):
        rest = np.ones(base[k].shape, bool)
        rest[idx] = False
        assert np.array_equal(g[k][rest], base[k][rest]), k
    # clearing the last step's hidden mask removes all gradient that entered through it
    masks.arr["h"][T - 1] = 0
    only_last = dh_new.copy()
    only_last[1:T] = 0
    g2 = ol.backward_quant(f, only_last, f["h"], f["v"], p, masks)
    assert not np.any(g2["dW"]) and not np.any(g2["dx"]) and not np.any(g2["dh0"])


def test_shipped_host_code_matches_restatement():
    """Encodings, tables and effective scales derived by the library's host code (no GPU needed)."""
    lib = cabi.load_library()
    for seed, (T, B, I, H) in enumerate([(5, 2, 3, 4), (7, 3, 31, 33), (6, 2, 40, 64)]):
        W, R, bw, br, x, h0 = ol.gru_problem(seed, T, B, I, H)
        rg = ol.RangesBox(H)
        ol.forward_calibrate_minmax("orc", W, R, bw, br, x, h0, rg)
        for bits in (8, 16, 4):
            for sym in (True, False):
                for pot in (False, True):
                    for gran in (0, 1, 2):
                        cfg = ol.make_config(bits=bits, symmetric=sym, use_pot2=pot, granularity=gran)
                        po = ol.params_from_ranges("orc", rg, cfg)
                        pp = ol.ParamsBox(H, cfg)
                        assert lib.rxmet_gru_params_from_ranges(C.byref(rg.c), C.byref(cfg), C.byref(pp.c)) == 0
                        for k, v in po.as_dict().items():
                            assert np.array_equal(v, pp.as_dict()[k]), k
                        out = ((cabi.LutSegment * 16) * 3)()
                        assert lib.rxmet_gru_build_luts(C.byref(pp.c), out) == 0
                        got = np.array([[(s.q_b, s.n_bx_total, s.term_c, s.threshold) for s in row] for row in out])
                        assert np.array_equal(got, ol.build_luts("orc", po))
    a, b = C.c_float(), C.c_float()
    for scale in (0.0123, 1.0, 3.7e-4):
        for pot in (0, 1):
            assert lib.rxmet_gru_decode_effective_scale(C.c_float(scale), pot, C.byref(a)) == 0
            assert ol.oracle().orc_gru_decode_effective_scale(C.c_float(scale), pot, C.byref(b)) == 0
            assert a.value == b.value


def test_library_rejects_bad_arguments_without_a_gpu():
    lib = cabi.load_library()
    cfg = ol.make_config()
    cfg.symmetric[cabi.W] = 0
    rg = ol.RangesBox(4)
    pp = ol.ParamsBox(4, cfg)
    assert lib.rxmet_gru_params_from_ranges(C.byref(rg.c), C.byref(cfg), C.byref(pp.c)) == -1
    assert b"symmetric" in lib.rxmet_last_error()
    assert lib.rxmet_gru_workspace_bytes(1, 0, 1, 1, 1) == 0
    assert lib.rxmet_gru_workspace_bytes(1, 10, 4, 8, 16) > 0
    out = C.c_float()
    assert lib.rxmet_gru_decode_effective_scale(C.c_float(-1.0), 0, C.byref(out)) == -1


def test_c_abi_exports_every_declared_symbol():
    header = "".join(f.read_text() for f in sorted((ROOT / "include").glob("*.h")))
    declared = set(re.findall(r"RXMET_API\s+[\w\s\*]+?\b(rxmet_\w+)\s*\(", header))
    assert len(declared) >= 40
    lib = cabi.load_library()
    missing = [name for name in sorted(declared) if not hasattr(lib, name)]
    assert not missing, missing


def test_float_storage_carrier_switch_is_host_state():
    """The module-level switch behind forward_quant_float_storage: default "integer", returns the previous choice,
    rejects anything but the two carriers (no GPU involved)."""
    from rx_met_b200 import gru_interface_binding as ops
    assert ops.float_storage_carrier() == "integer"
    assert ops.set_float_storage_carrier("fp32") == "integer"
    try:
        assert ops.float_storage_carrier() == "fp32"
        with pytest.raises(ValueError):
            ops.set_float_storage_carrier("bf16")
        assert ops.float_storage_carrier() == "fp32"
    finally:
        assert ops.set_float_storage_carrier("integer") == "fp32"
    assert ops.float_storage_carrier() == "integer"
