"""GPU parity tests: the CUDA library, called through its C ABI, against the CPU restatement
and the golden fixtures.  Integer codes, clamp masks and dequantized outputs must be bit-exact;
float paths (calibration forward, backward) must agree within 1e-5 relative."""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest

import oracle_lib as ol
from rx_met_b200 import _cabi as cabi

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
GOLDEN = sorted((ROOT / "tests" / "golden").glob("gru_*.npz"))
REL = 1e-5  # tolerance for float results, relative to the largest magnitude of the tensor


@pytest.fixture(scope="module")
def gl():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("the gpu tests need a CUDA device")
    import gpu_lib
    return gpu_lib


def close(a, b, rel=REL, what=""):
    scale = max(float(np.abs(b).max()), 1e-30)
    err = float(np.abs(a.astype(np.float64) - b.astype(np.float64)).max())
    assert err <= rel * scale, f"{what}: max abs err {err:.3e} vs scale {scale:.3e}"


def calibrated(shape, seed, cfg, with_h0, x_scale=1.0):
    T, B, I, H = shape
    W, R, bw, br, x, h0 = ol.gru_problem(seed, T, B, I, H, x_scale=x_scale, with_h0=with_h0)
    rg = ol.RangesBox(H)
    ol.forward_calibrate_minmax("orc", W, R, bw, br, x, h0, rg)
    return (W, R, bw, br, x, h0), ol.params_from_ranges("orc", rg, cfg)


def assert_forward_equal(got, want, training=True):
    for k in ("W_q", "R_q", "bw_q", "br_q", "x_q", "h_q", "v_q"):
        assert np.array_equal(got[k], want[k]), f"codes {k}: {(got[k] != want[k]).sum()} of {got[k].size} differ"
    for k in ("h", "v"):
        assert np.array_equal(got[k], want[k]), f"dequantized {k} differs"
    if training:
        for k, m in want["masks"].arr.items():
            assert np.array_equal(got["masks"][k], m), f"mask {k}: {(got['masks'][k] != m).sum()} differ"


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: p.stem)
def test_forward_quant_matches_golden(gl, path):
    g = np.load(path)
    seed, T, B, I, H, bits, sym, pot, gran, with_h0 = (int(v) for v in g["meta"])
    cfg = ol.make_config(bits=bits, symmetric=bool(sym), use_pot2=bool(pot), granularity=gran)
    params = ol.ParamsBox(H, cfg).load_dict({k[len("param_"):]: g[k] for k in g.files if k.startswith("param_")})
    h0 = g["h0"] if with_h0 else None
    rc, got = gl.forward_quant(g["W"], g["R"], g["bw"], g["br"], g["x"], h0, params)
    assert rc == 0, got
    for k in ("W_q", "R_q", "bw_q", "br_q", "x_q", "h_q", "v_q", "h", "v"):
        assert np.array_equal(got[k], g[f"fwd_{k}"]), k


CONFIGS = {
    "w8a8": dict(bits=8, symmetric=False),
    "w8a8_sym": dict(bits=8, symmetric=True),
    "w8a8_pot2": dict(bits=8, symmetric=False, use_pot2=True),
    "a16": dict(bits=8, symmetric=False, overrides={n: (16, False, False) for n in (
        "x", "h", "weight_ih_linear", "weight_hh_linear", "update_gate_input", "reset_gate_input",
        "new_gate_input", "new_gate_output", "mul_reset_hidden", "mul_old_contribution", "mul_new_contribution")}),
    "w16a16": dict(bits=16, symmetric=False),
    "w4": dict(bits=8, symmetric=False, granularity=cabi.PER_GATE,
               overrides={"W": (4, False, True), "R": (4, False, True)}),
    "unsigned_x": dict(bits=8, symmetric=False, overrides={"x": (8, True, False)}),
    "b24": dict(bits=24, symmetric=False),
}
SHAPES = [(3, 1, 1, 1), (5, 2, 3, 4), (7, 3, 31, 33), (6, 5, 40, 64), (4, 37, 20, 128), (3, 2, 9, 160)]


@pytest.mark.parametrize("cfg_name", list(CONFIGS))
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_forward_quant_matches_restatement(gl, cfg_name, shape):
    cfg = ol.make_config(**CONFIGS[cfg_name])
    with_h0 = (shape[0] + shape[1]) % 2 == 0
    prob, params = calibrated(shape, seed=sum(shape), cfg=cfg, with_h0=with_h0, x_scale=1.5)
    want = ol.forward_quant("orc", *prob, params, training=True)
    rc, got = gl.forward_quant(*prob, params, training=True)
    assert rc == 0, got
    assert_forward_equal(got, want)
    rc, inf = gl.forward_quant(*prob, params, training=False)
    assert rc == 0, inf
    for k in ("h_q", "v_q", "h", "v"):
        assert np.array_equal(inf[k], want[k]), k
    # integer in / integer out chaining reproduces the same state codes
    h0_q = want["h_q"][0] if with_h0 else None
    assert np.array_equal(gl.forward_int_io(*prob[:4], want["x_q"], h0_q, params), want["h_q"])


def test_forward_quant_saturating_inputs(gl):
    """Inputs far outside the calibrated range exercise every clamp mask."""
    cfg = ol.make_config(bits=8, symmetric=False)
    prob, params = calibrated((6, 4, 12, 32), seed=77, cfg=cfg, with_h0=True)
    W, R, bw, br, x, h0 = prob
    x = (x * 6.0).astype(np.float32)
    h0 = (h0 * 8.0).astype(np.float32)
    want = ol.forward_quant("orc", W, R, bw, br, x, h0, params)
    assert (want["masks"].arr["x"] == 0).any() and (want["masks"].arr["h0"] == 0).any()
    rc, got = gl.forward_quant(W, R, bw, br, x, h0, params)
    assert rc == 0, got
    assert_forward_equal(got, want)


@pytest.mark.parametrize("shape", [(5, 2, 3, 4), (7, 3, 31, 33), (9, 6, 40, 128)], ids=lambda s: "x".join(map(str, s)))
def test_calibration_forward(gl, shape):
    T, B, I, H = shape
    W, R, bw, br, x, h0 = ol.gru_problem(3, T, B, I, H, with_h0=True)
    want_r, got_r = ol.RangesBox(H), ol.RangesBox(H)
    h_w, v_w = ol.forward_calibrate_minmax("orc", W, R, bw, br, x, h0, want_r)
    h_g, v_g = gl.forward_float(W, R, bw, br, x, h0, ranges=got_r)
    close(h_g, h_w, what="h")
    close(v_g, v_w, what="v")
    w, g = want_r.as_dict(), got_r.as_dict()
    for k in ("min_W", "max_W", "min_R", "max_R", "min_bw", "max_bw", "min_br", "max_br"):
        assert np.array_equal(g[k], w[k]), k  # no arithmetic involved: exact
    assert g["min"][cabi.X] == w["min"][cabi.X] and g["max"][cabi.X] == w["max"][cabi.X]
    for op in cabi.SCALAR_OPS:
        for kind in ("min", "max"):
            assert abs(g[kind][op] - w[kind][op]) <= 1e-5 * max(1.0, abs(w[kind][op])), (kind, cabi.OP_NAMES[op])
    # a second batch accumulates into the same ranges, and the float forward alone agrees too
    x2 = (x * 1.7).astype(np.float32)
    ol.forward_calibrate_minmax("orc", W, R, bw, br, x2, None, want_r)
    gl.forward_float(W, R, bw, br, x2, None, ranges=got_r)
    assert got_r.as_dict()["max"][cabi.X] == want_r.as_dict()["max"][cabi.X]
    h_f, v_f = gl.forward_float(W, R, bw, br, x, h0)
    assert np.array_equal(h_f, h_g) and np.array_equal(v_f, v_g)


def test_calibration_ignores_non_finite_values(gl):
    T, B, I, H = 4, 2, 5, 8
    W, R, bw, br, x, _ = ol.gru_problem(8, T, B, I, H)
    x[1, 0, 2] = np.inf
    x[2, 1, 0] = np.nan
    want_r, got_r = ol.RangesBox(H), ol.RangesBox(H)
    ol.forward_calibrate_minmax("orc", W, R, bw, br, x, None, want_r)
    gl.forward_float(W, R, bw, br, x, None, ranges=got_r)
    w, g = want_r.as_dict(), got_r.as_dict()
    assert g["min"][cabi.X] == w["min"][cabi.X] and g["max"][cabi.X] == w["max"][cabi.X]
    assert np.isfinite(g["max"]).all()


@pytest.mark.parametrize("cfg_name", ["w8a8", "a16", "w8a8_pot2"])
@pytest.mark.parametrize("shape", [(5, 2, 3, 4), (7, 3, 31, 33), (8, 9, 40, 128), (6, 20, 72, 64), (6, 20, 72, 96)],
                         ids=lambda s: "x".join(map(str, s)))   # 72 inputs: the streaming dx kernel, 64- and 32-channel chunks
def test_backward_quant(gl, cfg_name, shape):
    T, B, I, H = shape
    cfg = ol.make_config(**CONFIGS[cfg_name])
    prob, params = calibrated(shape, seed=5 + T, cfg=cfg, with_h0=True)
    W, R, bw, br, x, h0 = prob
    x = (x * 2.5).astype(np.float32)  # make some clamps fire
    f = ol.forward_quant("orc", W, R, bw, br, x, h0, params)
    rng = np.random.default_rng(T)
    dh_new = np.zeros((T + 1, B, H), np.float32)
    dh_new[1:] = rng.standard_normal((T, B, H)).astype(np.float32)
    dh_new[-1] += rng.standard_normal((B, H)).astype(np.float32)
    want = ol.backward_quant(f, dh_new, f["h"], f["v"], params, f["masks"])
    got = gl.backward_quant(f, dh_new, f["h"], f["v"], params, f["masks"].arr)
    for k in want:
        close(got[k], want[k], what=k)
    # masked-out positions are exactly zero
    for k, m in (("dx", "x"), ("dW", "W"), ("dR", "R"), ("dbw", "bw"), ("dbr", "br"), ("dh0", "h0")):
        assert not np.any(got[k][f["masks"].arr[m] == 0]), k
    # no masks at all = every mask set
    ones = {k: np.ones_like(v) for k, v in f["masks"].arr.items()}
    a = gl.backward_quant(f, dh_new, f["h"], f["v"], params, ones)
    b = gl.backward_quant(f, dh_new, f["h"], f["v"], params, None)
    for k in a:
        assert np.array_equal(a[k], b[k]), k


@pytest.mark.parametrize("shape", [(80, 256, 40, 128), (80, 256, 72, 64)], ids=lambda s: "x".join(map(str, s)))
def test_backward_quant_row_ranges_of_several_tiles(gl, shape):
    """Enough rows (T*B = 20480) that every CTA of the tcgen05 input-gradient kernel walks two 128-row
    tiles and the split-K weight-gradient kernel runs many chunks per split.  72 inputs: the streaming
    input-gradient kernel over more 128-row tiles than SMs."""
    T, B, I, H = shape
    cfg = ol.make_config(**CONFIGS["w8a8"])
    prob, params = calibrated(shape, seed=91, cfg=cfg, with_h0=True)
    W, R, bw, br, x, h0 = prob
    x = (x * 2.5).astype(np.float32)
    f = ol.forward_quant("orc", W, R, bw, br, x, h0, params)
    rng = np.random.default_rng(17)
    dh_new = np.zeros((T + 1, B, H), np.float32)
    dh_new[1:] = rng.standard_normal((T, B, H)).astype(np.float32)
    want = ol.backward_quant(f, dh_new, f["h"], f["v"], params, f["masks"])
    got = gl.backward_quant(f, dh_new, f["h"], f["v"], params, f["masks"].arr)
    for k in want:
        close(got[k], want[k], what=k)


def test_backward_float(gl):
    T, B, I, H = 6, 5, 12, 48
    W, R, bw, br, x, h0 = ol.gru_problem(31, T, B, I, H, with_h0=True)
    h, v = ol.forward_fp(W, R, bw, br, x, h0)
    dh_new = np.zeros((T + 1, B, H), np.float32)
    dh_new[1:] = np.random.default_rng(2).standard_normal((T, B, H)).astype(np.float32)
    want = ol.backward_fp(W, R, bw, br, x, dh_new, h, v)
    got = gl.backward_fp(W, R, bw, br, x, dh_new, h, v)
    for k in want:
        close(got[k], want[k], what=k)


def test_full_size_properties(gl):
    """QAT-step sized problem (T=100, B=256, I=40, H=128): too slow to check element by element
    on the CPU in a unit test, so it is checked through size-independent properties."""
    shape = (100, 256, 40, 128)
    T, B, I, H = shape
    cfg = ol.make_config(bits=8, symmetric=False)
    small, params = calibrated((20, 8, I, H), seed=1, cfg=cfg, with_h0=False)
    W, R, bw, br = small[:4]
    x = np.random.default_rng(4).standard_normal((T, B, I)).astype(np.float32)
    rc, full = gl.forward_quant(W, R, bw, br, x, None, params)
    assert rc == 0, full
    # (a) sequences are independent: any batch slice run alone gives the same codes
    rc, part = gl.forward_quant(W, R, bw, br, x[:, 100:117], None, params)
    assert rc == 0, part
    assert np.array_equal(part["h_q"], full["h_q"][:, 100:117]) and np.array_equal(part["v_q"], full["v_q"][:, 100:117])
    for k in ("weight_hh_linear", "gate_input", "gate_output", "h", "x", "weight_ih_linear"):
        assert np.array_equal(part["masks"][k], full["masks"][k][:, 100:117]), k
    # (b) the first sequences agree with the CPU restatement element by element
    want = ol.forward_quant("orc", W, R, bw, br, np.ascontiguousarray(x[:, :6]), None, params)
    assert np.array_equal(full["h_q"][:, :6], want["h_q"]) and np.array_equal(full["v_q"][:, :6], want["v_q"])
    # (c) codes stay on their grids and masks are 0/1
    assert full["h_q"].min() >= -128 and full["h_q"].max() <= 127
    assert full["v_q"][..., :2 * H].min() >= 0 and full["v_q"][..., :2 * H].max() <= 255
    for k, m in full["masks"].items():
        assert m.max() <= 1, k
    # (d) repeatable run to run, forward and backward
    rc, again = gl.forward_quant(W, R, bw, br, x, None, params)
    assert np.array_equal(again["h_q"], full["h_q"]) and np.array_equal(again["v"], full["v"])
    dh_new = np.zeros((T + 1, B, H), np.float32)
    dh_new[1:] = np.random.default_rng(6).standard_normal((T, B, H)).astype(np.float32)
    g1 = gl.backward_quant(full, dh_new, full["h"], full["v"], params, full["masks"])
    g2 = gl.backward_quant(full, dh_new, full["h"], full["v"], params, full["masks"])
    for k in g1:
        assert np.array_equal(g1[k], g2[k]), k
    # (e) the backward is linear in the incoming gradient, and zero in gives zero out
    g3 = gl.backward_quant(full, (2.0 * dh_new).astype(np.float32), full["h"], full["v"], params, full["masks"])
    for k in g1:
        close(g3[k], 2.0 * g1[k], what=k)
    g0 = gl.backward_quant(full, np.zeros_like(dh_new), full["h"], full["v"], params, full["masks"])
    assert all(not np.any(v) for v in g0.values())
    # (f) per-sequence gradients: a batch slice of dx equals the slice run alone
    sl = slice(100, 117)
    sub = {k: np.ascontiguousarray(full[k][:, sl]) if full[k].ndim == 3 else full[k]
           for k in ("W_q", "R_q", "bw_q", "br_q", "x_q")}
    sub_masks = {k: (np.ascontiguousarray(m[:, sl]) if m.ndim == 3 else m) for k, m in full["masks"].items()}
    gs = gl.backward_quant(sub, np.ascontiguousarray(dh_new[:, sl]), np.ascontiguousarray(full["h"][:, sl]),
                           np.ascontiguousarray(full["v"][:, sl]), params, sub_masks)
    assert np.array_equal(gs["dx"], g1["dx"][:, sl])


def test_full_size_forward_equals_the_reference_cpu_build(gl):
    """The whole headline workload (T = 100, B = 256, I = 40, H = 128, W8 / A8 asymmetric) against the reference's
    own CPU sources compiled into oracle/_ref: every code and every dequantized value of all 25,600
    sequence-steps, not a slice (the reference's CPU build has no clamp masks; those are checked against its CUDA
    build in test_reference_cuda_gpu.py)."""
    if ol.ref() is None:
        pytest.skip("compiled reference not present")
    T, B, I, H = 100, 256, 40, 128
    cfg = ol.make_config(bits=8, symmetric=False)
    (W, R, bw, br, x, h0), params = calibrated((T, B, I, H), seed=21, cfg=cfg, with_h0=False)
    want = ol.forward_quant("ref", W, R, bw, br, x, None, params, training=True)
    rc, got = gl.forward_quant(W, R, bw, br, x, None, params, training=True)
    assert rc == 0, got
    assert_forward_equal(got, want, training=False)


def test_first_config_calibration_against_the_reference_cpu_calibration(gl):
    """The CPU-runnable configuration (input 40, hidden 64, T = 98, batch 32, W8 symmetric per tensor, A8
    asymmetric, min/max calibration over 16 seeded batches, then a PTQ forward): how many of the finalized
    (scale, zero point) pairs of the GPU calibration differ from the reference's CPU calibration, and that the PTQ
    forward with either parameter set is bit-identical to the reference run with the same set."""
    if ol.ref() is None:
        pytest.skip("compiled reference not present")
    T, B, I, H = 98, 32, 40, 64
    cfg = ol.make_config(bits=8, symmetric=False, granularity=cabi.PER_TENSOR)
    W, R, bw, br, _, _ = ol.gru_problem(100, T, B, I, H)
    ref_ranges, gpu_ranges = ol.RangesBox(H), ol.RangesBox(H)
    batches = [np.random.default_rng(1000 + i).standard_normal((T, B, I)).astype(np.float32) for i in range(16)]
    for x in batches:
        ol.forward_calibrate_minmax("ref", W, R, bw, br, x, None, ref_ranges, cfg)
        gl.forward_float(W, R, bw, br, x, None, ranges=gpu_ranges)
    ref_params = ol.params_from_ranges("ref", ref_ranges, cfg)
    gpu_params = ol.ParamsBox(H, cfg)
    assert cabi.load_library().rxmet_gru_params_from_ranges(C.byref(gpu_ranges.c), C.byref(cfg), C.byref(gpu_params.c)) == 0
    r, g = ref_params.as_dict(), gpu_params.as_dict()
    pairs = len(r["scale"])
    differing = [cabi.OP_NAMES[i] for i in range(pairs) if r["scale"][i] != g["scale"][i] or r["zero_point"][i] != g["zero_point"][i]]
    print(f"configs[0]: {len(differing)} of {pairs} (scale, zero point) pairs differ between GPU and CPU calibration: {differing}")
    # the two float forwards differ in the last ulp (fp32 FMA and CUDA expf / tanhf against sequential sums and glibc),
    # so an observed extreme can move by an ulp; the power-of-two-free affine grids then differ in the last bit of a scale
    for i in range(pairs):
        assert abs(r["scale"][i] - g["scale"][i]) <= 2e-6 * max(abs(r["scale"][i]), 1e-30), cabi.OP_NAMES[i]
        assert abs(int(r["zero_point"][i]) - int(g["zero_point"][i])) <= 1, cabi.OP_NAMES[i]
    assert len(differing) <= pairs // 2
    for key in ("scale_W", "scale_R", "scale_bw", "scale_br"):   # no arithmetic on the way to the weight ranges
        assert np.array_equal(r[key], g[key]), key
    for params in (ref_params, gpu_params):
        want = ol.forward_quant("ref", W, R, bw, br, batches[0], None, params, training=False)
        rc, got = gl.forward_quant(W, R, bw, br, batches[0], None, params, training=False)
        assert rc == 0, got
        assert np.array_equal(got["h_q"], want["h_q"]) and np.array_equal(got["v_q"], want["v_q"])


def test_errors_are_reported_not_fatal(gl):
    cfg = ol.make_config(bits=8, symmetric=False)
    prob, params = calibrated((4, 2, 3, 8), seed=2, cfg=cfg, with_h0=False)
    rc, msg = gl.forward_quant(*prob, params, workspace_bytes=64)
    assert rc == -3 and "workspace" in msg
    wrong = ol.ParamsBox(16, cfg)
    rc, msg = gl.forward_quant(*prob, wrong)
    assert rc == -1 and "hidden" in msg
    rc, ok = gl.forward_quant(*prob, params)  # the context is still usable
    assert rc == 0


def test_python_module_mirrors_reference_binding(gl):
    """The drop-in module returns the reference's 18-tuple and 6-tuple and agrees with the C ABI."""
    import torch
    from rx_met_b200 import gru_interface_binding as ops
    T, B, I, H = 6, 4, 10, 24
    W, R, bw, br, x, h0 = ol.gru_problem(13, T, B, I, H, with_h0=True)
    t = {k: torch.from_numpy(v).cuda() for k, v in dict(W=W, R=R, bw=bw, br=br, x=x, h0=h0).items()}
    cfg = ops.OperatorQuantConfig()
    for name in cabi.OP_NAMES:
        if name not in ("W", "R", "bw", "br"):
            setattr(cfg, f"{name}_symmetric_", False)
    ranges = ops.GRUQuantizationRanges(H)
    h_fp, v_fp = ops.forward_calibrate(False, T, B, I, H, t["W"], t["R"], t["bw"], t["br"], t["x"], t["h0"],
                                       "minmax", cfg, quant_ranges=ranges)
    assert ranges.max_x_ == float(x.max()) and len(ranges.min_W_) == 3 * H
    qp = ops.calculate_gru_quantitative_parameters(ranges, cfg)
    assert qp.hidden_ == H and len(qp.scale_W_) == 3 * H and qp.scale_x_ > 0
    out_i = ops.forward_quant_int_storage(True, T, B, I, H, t["W"], t["R"], t["bw"], t["br"], t["x"], t["h0"], qp)
    out_f = ops.forward_quant_float_storage(True, T, B, I, H, t["W"], t["R"], t["bw"], t["br"], t["x"], t["h0"], qp)
    assert len(out_i) == 18 and len(out_f) == 18
    assert out_i[2].dtype == torch.int32 and out_f[2].dtype == torch.float32 and out_i[7].dtype == torch.uint8
    for a, b in zip(out_i, out_f):
        assert torch.equal(a.float(), b.float())
    inf = ops.forward_quant_int_storage(False, T, B, I, H, t["W"], t["R"], t["bw"], t["br"], t["x"], t["h0"], qp)
    assert torch.equal(inf[0], out_i[0]) and all(m.numel() == 0 for m in inf[7:])
    h, v = out_i[0], out_i[1]
    dh_new = torch.zeros((T + 1, B, H), device="cuda")
    dh_new[1:] = torch.randn((T, B, H), generator=torch.Generator().manual_seed(0)).cuda()
    grads_i = ops.backward_quant_int_storage(T, B, I, H, *out_i[2:7], dh_new, h, v, qp, *out_i[7:])
    grads_f = ops.backward_quant_float_storage(T, B, I, H, *out_f[2:7], dh_new, h, v, qp, *out_f[7:])
    assert len(grads_i) == 6
    for a, b in zip(grads_i, grads_f):
        assert torch.equal(a, b)
    assert tuple(grads_i[0].shape) == (T, B, I) and tuple(grads_i[1].shape) == (I, 3 * H)
    # scale the module reports = scale the kernels dequantize with
    eff = ops.decode_effective_scale(qp.scale_h_, False)
    codes = torch.round(h / eff) + qp.zp_h_
    assert torch.equal((codes - qp.zp_h_) * eff, h)
    with pytest.raises(RuntimeError):
        ops.forward_quant_int_storage(True, T, B, I, H, t["W"].cpu(), t["R"], t["bw"], t["br"], t["x"], t["h0"], qp)
    out_q, hn_q = ops.forward_quantized_int_io(T, B, I, H, t["W"], t["R"], t["bw"], t["br"], out_i[6], None, qp)
    assert out_q.dtype == torch.int32 and tuple(out_q.shape) == (T, B, H) and tuple(hn_q.shape) == (1, B, H)


def test_float_storage_carrier_switch(gl):
    """forward_quant_float_storage with the carrier set to "fp32" returns what the FP32-carrier entry point
    returns (the reference's CUDA float-code arithmetic); the default stays the integer carrier; the backward
    accepts either forward's caches."""
    import types
    import torch
    from rx_met_b200 import gru_interface_binding as ops
    T, B, I, H = 7, 5, 12, 32
    prob = ol.gru_problem(29, T, B, I, H, with_h0=True)
    t = [torch.from_numpy(a).cuda() for a in prob]
    cfg = ops.OperatorQuantConfig()
    for name in cabi.OP_NAMES:
        if name not in ("W", "R", "bw", "br"):
            setattr(cfg, f"{name}_symmetric_", False)
    ranges = ops.GRUQuantizationRanges(H)
    ops.forward_calibrate(False, T, B, I, H, *t, "minmax", cfg, quant_ranges=ranges)
    qp = ops.calculate_gru_quantitative_parameters(ranges, cfg)
    params_c, keep = qp._to_c()
    rc, want = gl.forward_quant(*prob, types.SimpleNamespace(c=params_c), training=True, fp_carrier=True)
    assert rc == 0, want
    assert ops.float_storage_carrier() == "integer"
    previous = ops.set_float_storage_carrier("fp32")
    try:
        out = ops.forward_quant_float_storage(True, T, B, I, H, *t, qp)
    finally:
        ops.set_float_storage_carrier(previous)
    assert ops.float_storage_carrier() == "integer"
    np.testing.assert_array_equal(out[0].cpu().numpy(), want["h"])
    np.testing.assert_array_equal(out[1].cpu().numpy(), want["v"])
    for k, got in zip(("W_q", "R_q", "bw_q", "br_q", "x_q"), out[2:7]):
        assert got.dtype == torch.float32
        np.testing.assert_array_equal(got.cpu().numpy().astype(np.int32), want[k], err_msg=k)
    with pytest.raises(ValueError):
        ops.set_float_storage_carrier("bf16")
    dh_new = torch.zeros((T + 1, B, H), device="cuda")
    dh_new[1:] = torch.randn((T, B, H), generator=torch.Generator().manual_seed(1)).cuda()
    grads = ops.backward_quant_float_storage(T, B, I, H, *out[2:7], dh_new, out[0], out[1], qp, *out[7:])
    assert len(grads) == 6 and all(bool(torch.isfinite(g).all()) for g in grads)
    del keep


@pytest.mark.parametrize("cfg_name", ["a16", "w8a8"])
@pytest.mark.parametrize("shape", [(4, 3, 40, 256), (3, 2, 512, 256)], ids=lambda s: "x".join(map(str, s)))
def test_kws_body_layer_shapes(gl, cfg_name, shape):
    """Layer shapes of the stacked keyword-spotting body (hidden 256, input 40 or 512, W8 per channel,
    A16 or A8): forward codes and masks bit-exact, QAT gradients within 1e-5."""
    T, B, I, H = shape
    cfg = ol.make_config(**CONFIGS[cfg_name])
    prob, params = calibrated(shape, seed=9 + I, cfg=cfg, with_h0=True, x_scale=1.2)
    want = ol.forward_quant("orc", *prob, params, training=True)
    rc, got = gl.forward_quant(*prob, params, training=True)
    assert rc == 0, got
    assert_forward_equal(got, want)
    dh_new = np.zeros((T + 1, B, H), np.float32)
    dh_new[1:] = np.random.default_rng(I).standard_normal((T, B, H)).astype(np.float32)
    wb = ol.backward_quant(want, dh_new, want["h"], want["v"], params, want["masks"])
    gb = gl.backward_quant(want, dh_new, want["h"], want["v"], params, want["masks"].arr)
    for k in wb:
        close(gb[k], wb[k], what=k)


def test_cluster_backward_kernel_agrees(gl, monkeypatch):
    """The opt-in backward recurrence over clusters of eight CTAs (weights in registers, gate gradients exchanged
    through distributed shared memory) gives the gradients of the default kernel; a batch that leaves rows of
    the last cluster empty."""
    T, B, I, H = 5, 19, 40, 256
    cfg = ol.make_config(**CONFIGS["a16"])
    prob, params = calibrated((T, B, I, H), seed=77, cfg=cfg, with_h0=True, x_scale=1.2)
    want = ol.forward_quant("orc", *prob, params, training=True)
    dh_new = np.zeros((T + 1, B, H), np.float32)
    dh_new[1:] = np.random.default_rng(5).standard_normal((T, B, H)).astype(np.float32)
    wb = ol.backward_quant(want, dh_new, want["h"], want["v"], params, want["masks"])
    monkeypatch.setenv("RXMET_GRU_BWD_CLUSTER", "1")
    gb = gl.backward_quant(want, dh_new, want["h"], want["v"], params, want["masks"].arr)
    for k in wb:
        close(gb[k], wb[k], what=k)


def test_bounded_device_wait_gives_up_with_a_status(gl):
    """The poll loop of the tcgen05 kernels on a barrier nothing completes: the kernel returns after its
    limit, the status word is set, the call reports RXMET_ERR_DEVICE_TIMEOUT and the context keeps working."""
    import torch
    lib = cabi.load_library()
    status = torch.zeros(2, dtype=torch.int32, device="cuda")
    polls = C.c_uint(0)
    rc = lib.rxmet_selftest_bounded_wait(C.c_void_p(status.data_ptr()), C.byref(polls),
                                         C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == -5, lib.rxmet_last_error()
    assert b"ran out" in lib.rxmet_last_error()
    assert status.cpu().tolist()[0] == 1 and polls.value == 1 << 20
    # the context is still usable
    assert float((torch.ones(8, device="cuda") * 2).sum().item()) == 16.0


def test_captured_step_replays_the_eager_step():
    """A CUDA-graph replay of the QAT step leaves the same weights and loss as the eager step."""
    import torch
    from rx_met_b200.qat import GruQatStep
    T, B, I, H = 12, 16, 8, 32
    dev = torch.device("cuda")
    gen = torch.Generator(device="cpu").manual_seed(5)
    xs = [torch.randn((T, B, I), generator=gen).to(dev) for _ in range(3)]
    ys = [torch.randn((T, B, H), generator=gen).to(dev) for _ in range(3)]

    def run(graph):
        eng = GruQatStep(T, B, I, H, dev, seed=11)
        eng.calibrate(xs[:2])
        x, y = xs[0].clone(), ys[0].clone()
        losses = []
        if graph:
            replay, loss = eng.capture_step(x, y, 1e-2, warmup=2)
            assert eng.captured_launches >= 6
        else:
            for _ in range(2):
                eng.step(x, y, 1e-2)
        for k in range(3):
            x.copy_(xs[k]); y.copy_(ys[k])
            losses.append(float(replay() if graph else eng.step(x, y, 1e-2)))
        return eng.flat_w.clone(), losses

    w_eager, l_eager = run(False)
    w_graph, l_graph = run(True)
    assert l_eager == l_graph
    assert torch.equal(w_eager, w_graph)


@pytest.mark.parametrize("shape", [(7, 5, 12, 32), (6, 9, 40, 128)], ids=lambda s: "x".join(map(str, s)))
def test_packed_step_flags_equal_the_byte_masks(monkeypatch, shape):
    """The compact save-for-backward of the training engine: the 16-bit word the forward writes per element and
    step holds exactly the 13 byte flags of the reference-shaped masks, and a training step through the packed
    pair leaves the same weights, bit for bit, as the step through the byte masks."""
    import torch
    from rx_met_b200 import gru_interface_binding as ops
    from rx_met_b200.qat import GruQatStep
    T, B, I, H = shape
    dev = torch.device("cuda", 0)
    cfg = ops.OperatorQuantConfig()
    for name in cabi.OP_NAMES:
        if name not in ("W", "R", "bw", "br"):
            setattr(cfg, f"{name}_symmetric_", False)
    gen = torch.Generator().manual_seed(17)
    x = torch.randn((T, B, I), generator=gen).to(dev)
    y = torch.randn((T, B, H), generator=gen).to(dev)
    packed = GruQatStep(T, B, I, H, dev, cfg, seed=5)
    packed.calibrate([x * 0.6])            # narrower calibration input: the step clamps
    assert packed._packed
    monkeypatch.setenv("RXMET_QAT_BYTE_MASKS", "1")
    plain = GruQatStep(T, B, I, H, dev, cfg, seed=5)
    plain.calibrate([x * 0.6])
    assert not plain._packed
    packed.forward(x)
    plain.forward(x)
    m = plain.masks
    C3 = 3 * H
    word = torch.zeros((T, B, H), dtype=torch.int32, device=dev)
    for bit, name in ((0, "gate_output"), (3, "gate_input"), (6, "weight_hh_linear"), (9, "weight_ih_linear")):
        for g in range(3):
            word |= m[name][..., g * H:(g + 1) * H].to(torch.int32) << (bit + g)
    word |= m["h"].to(torch.int32) << 12
    assert torch.equal(packed.step_flags.to(torch.int32) & 0xffff, word)
    assert (word != 0x1fff).any(), "the case should clamp somewhere"
    for _ in range(3):
        lp, lb = packed.step(x, y, 1e-2), plain.step(x, y, 1e-2)
    assert torch.equal(packed.flat_w, plain.flat_w) and torch.equal(lp, lb)


@pytest.mark.parametrize("byte_masks", [False, True], ids=["packed", "bytes"])
def test_time_chunked_step_equals_the_single_launch_step(monkeypatch, byte_masks):
    """The overlapped pipeline cuts the sequence into time chunks (projection / gradient GEMMs of one chunk under the
    recurrence of its neighbour).  Codes, h, v, flags, dx and dh0 are bit-identical to the one-launch path; the
    weight gradients sum the same products in another order (1e-5); a graph of the chunked step replays it."""
    import torch
    from rx_met_b200 import gru_interface_binding as ops
    from rx_met_b200.qat import GruQatStep
    lib = cabi.load_library()
    T, B, I, H = 24, 64, 40, 128
    dev = torch.device("cuda", 0)
    cfg = ops.OperatorQuantConfig()
    for name in cabi.OP_NAMES:
        if name not in ("W", "R", "bw", "br"):
            setattr(cfg, f"{name}_symmetric_", False)
    if byte_masks:
        monkeypatch.setenv("RXMET_QAT_BYTE_MASKS", "1")
    gen = torch.Generator().manual_seed(23)
    x = torch.randn((T, B, I), generator=gen).to(dev)
    y = torch.randn((T, B, H), generator=gen).to(dev)

    def run(chunks):
        monkeypatch.setenv("RXMET_GRU_FWD_CHUNKS", chunks)
        monkeypatch.setenv("RXMET_GRU_BWD_CHUNKS", chunks)
        eng = GruQatStep(T, B, I, H, dev, cfg, seed=9)
        eng.calibrate([x * 0.7])
        before = lib.rxmet_kernel_launch_count()
        eng.forward(x)
        middle = lib.rxmet_kernel_launch_count()
        eng.mse_loss(y)
        eng.backward()
        torch.cuda.synchronize()
        return eng, (middle - before, lib.rxmet_kernel_launch_count() - middle)

    one, launches_one = run("100")
    cut, launches_cut = run("20,30,50")
    assert launches_cut[0] > launches_one[0], "the chunked forward did not run"
    assert launches_cut[1] > launches_one[1], "the chunked backward did not run"
    assert torch.equal(one.h, cut.h) and torch.equal(one.v, cut.v)
    if byte_masks:
        for k in one.masks:
            assert torch.equal(one.masks[k], cut.masks[k]), k
    else:
        assert torch.equal(one.step_flags, cut.step_flags)
    assert torch.equal(one.dx, cut.dx) and torch.equal(one.dh0, cut.dh0)
    scale = float(one.flat_g.abs().max())
    assert float((one.flat_g - cut.flat_g).abs().max()) <= 1e-5 * scale
    # the chunked step inside a captured graph
    eager = [float(cut.step(x, y, 1e-2)) for _ in range(3)]
    graphed = GruQatStep(T, B, I, H, dev, cfg, seed=9)
    graphed.calibrate([x * 0.7])
    replay, loss = graphed.capture_step(x, y, 1e-2, warmup=1)   # one eager step, then the capture
    got = []
    for _ in range(2):
        replay()
        got.append(float(loss))
    assert got == eager[1:]
    assert torch.equal(graphed.flat_w, cut.flat_w)


def test_fused_mse_loss_and_gradient():
    """The step's loss kernel: gradient bit-identical to the eager float32 expressions, loss within 1e-6 relative."""
    import torch
    from rx_met_b200.qat import GruQatStep
    for T, B, I, H in ((12, 16, 8, 32), (5, 3, 4, 33)):   # the second shape is not a multiple of four long
        eng = GruQatStep(T, B, I, H, torch.device("cuda"), seed=3)
        gen = torch.Generator(device="cpu").manual_seed(7)
        eng.h.copy_(torch.randn(eng.h.shape, generator=gen))
        target = torch.randn((T, B, H), generator=gen).cuda()
        loss = eng.mse_loss(target)
        diff = eng.h[1:] - target
        want_grad = torch.mul(diff, 2.0 / diff.numel())
        assert torch.equal(eng.dh_new[1:], want_grad)
        want_loss = diff.double().square().mean()
        assert abs(float(loss) - float(want_loss)) <= 1e-6 * float(want_loss)
        again = float(eng.mse_loss(target))
        assert again == float(loss)
        with pytest.raises(ValueError):
            eng.mse_loss(target[:, :, :-1])


def test_mse_loss_helper():
    import torch
    from rx_met_b200 import losses
    gen = torch.Generator(device="cpu").manual_seed(9)
    h = torch.randn((7, 5, 24), generator=gen).cuda()
    target = torch.randn((6, 5, 24), generator=gen).cuda()
    grad_buffer = torch.zeros_like(h)
    loss, grad = losses.mse_loss_grad(h[1:], target, grad_buffer[1:])
    diff = h[1:] - target
    assert grad.data_ptr() == grad_buffer[1:].data_ptr() and torch.equal(grad, torch.mul(diff, 2.0 / diff.numel()))
    assert not grad_buffer[0].any()
    assert abs(float(loss) - float(diff.double().square().mean())) <= 1e-6 * float(loss)
    loss2, grad2 = losses.mse_loss_grad(h[1:], target)
    assert torch.equal(grad2, grad) and float(loss2) == float(loss)
    with pytest.raises(RuntimeError):
        losses.mse_loss_grad(h[1:], target[:, :, :-1])
    with pytest.raises(RuntimeError):
        losses.mse_loss_grad(h[1:].cpu(), target.cpu())
