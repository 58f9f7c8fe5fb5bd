"""QuantLSTM: the CPU restatement against the reference's golden cases and, where
``oracle/_ref/liblstm_ref.so`` was built, against the reference's own CPU sources."""
from __future__ import annotations

import ctypes as C
import json
from pathlib import Path

import numpy as np
import pytest

import lstm_lib as ll
from rx_met_b200 import _cabi_lstm as L

GOLDEN = json.loads((Path(__file__).parent / "golden" / "lstm_golden.json").read_text())
needs_ref = pytest.mark.skipif(not ll.have_ref(), reason="compiled reference not available")


def arr(t, dtype=None):
    a = np.array(t["data"], dtype=dtype or {"float32": np.float32, "float64": np.float64}.get(t["dtype"], np.int64))
    return a.reshape(t["shape"]) if t["shape"] else a


def golden_params(case):
    """QuantParams of a golden recurrent/cell case (flat scale list with per-operator offsets)."""
    inp = case["inputs"]
    T, B, I, H = inp["shape"]["data"]
    box = L.ParamsBox(H)
    s = box.struct
    s.input_size, s.hidden_size, s.bias_enabled = I, H, int(inp["bias_enabled"]["data"][0])
    s.config.scale_mode = L.SCALE_MODE_NAMES.index(inp["scale_mode"]["data"][0])
    assert tuple(inp["operator_names"]["data"]) == L.OP_NAMES
    scales = np.array(inp["quant_param_scales"]["data"], np.float32)
    zps, offs = inp["quant_param_zero_points"]["data"], inp["quant_param_value_offsets"]["data"]
    for op in range(L.NUM_OPS):
        s.config.bitwidth[op] = inp["operator_bitwidth"]["data"][op]
        s.config.is_unsigned[op] = int(inp["operator_is_unsigned"]["data"][op])
        s.config.is_symmetric[op] = int(inp["operator_is_symmetric"]["data"][op])
        s.config.granularity[op] = L.GRANULARITY_NAMES.index(inp["operator_granularity"]["data"][op])
        lo, hi = offs[op], offs[op + 1]
        if op in L.PARAMETER_OPS:
            box.channel_scales[op - L.WEIGHT_IH][:] = scales[lo:hi]
        else:
            s.scale[op], s.zero_point[op] = scales[lo], zps[lo]
    box.bind()
    return box, (T, B, I, H)


@pytest.mark.parametrize("case_id", ["reference_recurrent_t3_b1_i2_h2_cpu_fp32", "reference_cell_t1_b1_i2_h2_cpu_fp32"])
@pytest.mark.parametrize("prefix", ["orc", pytest.param("ref", marks=needs_ref)])
def test_golden_sequence(case_id, prefix):
    case = GOLDEN[case_id]
    box, (T, B, I, H) = golden_params(case)
    inp, exp = case["inputs"], case["expected"]
    f = lambda n: arr(inp[n], np.float32)
    q = dict(x=f("input"), w_ih=f("weight_ih"), w_hh=f("weight_hh"), b_ih=f("bias_ih"), b_hh=f("bias_hh"),
             h0=f("initial_hidden"), c0=f("initial_cell"))
    out, hn, cn, tr = ll.forward_quantized(prefix, box, T, B, q)
    np.testing.assert_array_equal(out, arr(exp["output"]))
    np.testing.assert_array_equal(hn, arr(exp["h_n"]))
    np.testing.assert_array_equal(cn, arr(exp["c_n"]))
    np.testing.assert_array_equal(tr["cell_states"], arr(exp["cell"]))
    np.testing.assert_array_equal(tr["cell_tanh_outputs"], arr(exp["cell_tanh"]))
    np.testing.assert_array_equal(tr["weight_ih_linear"].reshape(T, B, 4, H), arr(exp["weight_ih_linear"]))
    np.testing.assert_array_equal(tr["weight_hh_linear"].reshape(T, B, 4, H), arr(exp["weight_hh_linear"]))
    for g, name in enumerate(["input", "forget", "cell", "output"]):
        np.testing.assert_array_equal(tr["gate_inputs"].reshape(T, B, 4, H)[:, :, g], arr(exp[f"{name}_gate_input"]))
        np.testing.assert_array_equal(tr["gate_outputs"].reshape(T, B, 4, H)[:, :, g], arr(exp[f"{name}_gate_output"]))


def _one_op_cfg(bits, unsigned, symmetric):
    cfg = L.QuantConfig()
    cfg.bitwidth[0], cfg.is_unsigned[0], cfg.is_symmetric[0] = int(bits), int(unsigned), int(symmetric)
    return cfg


def test_golden_primitives():
    case = GOLDEN["quantize_boundaries"]
    i = case["inputs"]
    for k in range(len(i["value"]["data"])):
        cfg = _one_op_cfg(i["bitwidth"]["data"][k], i["is_unsigned"]["data"][k], i["is_symmetric"]["data"][k])
        got = ll.quantize("orc", np.array([i["value"]["data"][k]], np.float32), [i["scale"]["data"][k]],
                          i["zero_point"]["data"][k], cfg, 0)
        assert got[0] == case["expected"]["quantized"]["data"][k]
    case = GOLDEN["dequantize_boundaries"]
    i = case["inputs"]
    for k in range(len(i["value"]["data"])):
        got = ll.dequantize(np.array([i["value"]["data"][k]], np.float32), [i["scale"]["data"][k]], i["zero_point"]["data"][k])
        assert got[0] == np.float32(case["expected"]["real"]["data"][k])
    case = GOLDEN["real_activation_boundaries_cpu_fp32"]
    i = case["inputs"]
    for k in range(len(i["kind"]["data"])):
        tanh = i["kind"]["data"][k] == "tanh"
        dst = np.zeros(1, np.float32)
        src = np.array([i["quantized"]["data"][k]], np.float32)
        ll._call("orc", "real_activation", ll._fp(src), C.c_longlong(1), C.c_float(i["input_scale"]["data"][k]),
                 i["input_zero_point"]["data"][k], 8, 0, C.c_float(i["output_scale"]["data"][k]),
                 i["output_zero_point"]["data"][k], 8, 0 if tanh else 1, int(tanh), ll._fp(dst))
        assert dst[0] == case["expected"]["quantized"]["data"][k]
    case = GOLDEN["quantized_ranges"]
    i = case["inputs"]
    lo, hi = C.c_int32(), C.c_int32()
    for k in range(len(i["bitwidth"]["data"])):
        cfg = _one_op_cfg(i["bitwidth"]["data"][k], i["is_unsigned"]["data"][k], i["is_symmetric"]["data"][k])
        ll.lib("orc").orc_lstm_type_range(C.byref(cfg), 0, C.byref(lo), C.byref(hi))
        assert (lo.value, hi.value) == (case["expected"]["minimum"]["data"][k], case["expected"]["maximum"]["data"][k])


def test_golden_pot2_cover_range():
    case = GOLDEN["pot2_cover_range"]
    i, e = case["inputs"], case["expected"]
    for k in range(len(i["bitwidth"]["data"])):
        cfg = L.default_config(scale_mode=L.SCALE_POT2)
        op = L.INPUT
        cfg.bitwidth[op] = i["bitwidth"]["data"][k]
        cfg.is_unsigned[op], cfg.is_symmetric[op] = int(i["is_unsigned"]["data"][k]), int(i["is_symmetric"]["data"][k])
        ranges = L.RangesBox(1)
        for o in range(L.NUM_OPS):
            ranges.struct.minimum[o], ranges.struct.maximum[o] = -1.0, 1.0
        for s in range(4):
            ranges.mins[s][:], ranges.maxs[s][:] = -1.0, 1.0
        ranges.struct.minimum[op], ranges.struct.maximum[op] = i["range_minimum"]["data"][k], i["range_maximum"]["data"][k]
        box = ll.params_from_ranges("orc", cfg, ranges, 1, 1, True)
        assert box.struct.scale[op] == np.float32(e["scale"]["data"][k])
        assert box.struct.zero_point[op] == e["zero_point"]["data"][k]


def test_golden_m_shift():
    """encodeMShift vectors, reached through the gate rescale input_scale/output_scale = ratio."""
    case = GOLDEN["m_shift_known_vectors"]
    for ratio, mult, shift in zip(case["inputs"]["ratio"]["data"], case["expected"]["multiplier"]["data"],
                                  case["expected"]["shift"]["data"]):
        box = L.ParamsBox(1)
        s = box.struct
        s.config = L.default_config()
        s.input_size = s.hidden_size = 1
        s.bias_enabled = 0
        for op in range(L.NUM_OPS):
            s.scale[op] = 1.0
        for a in box.channel_scales:
            a[:] = 1.0
        box.bind()
        # ih_to_gate[0] encodes scale[weight_ih_linear] / scale[input_gate_input]
        s.scale[L.WEIGHT_IH_LINEAR] = np.float32(ratio) if np.float32(ratio) == ratio else 1.0
        if np.float32(ratio) != ratio:
            # ratios that are not float32 values: split into an exact float32 quotient
            s.scale[L.WEIGHT_IH_LINEAR] = np.float32(ratio * 65536)
            s.scale[L.INPUT_GATE_INPUT] = 65536.0
            assert float(s.scale[L.WEIGHT_IH_LINEAR]) / 65536.0 == ratio
        ex = ll.derive("orc", box)
        assert ex.struct.ih_to_gate[0].astuple() == (1, mult, shift)


CONFIGS = [dict(), dict(scale_mode=L.SCALE_POT2), dict(symmetric_activations=True),
           dict(parameter_granularity=L.PER_TENSOR), dict(parameter_granularity=L.PER_GATE, scale_mode=L.SCALE_POT2)]


@needs_ref
@pytest.mark.parametrize("bias,state", [(True, True), (False, False), (True, False)])
def test_float_forward_backward_match_reference(bias, state):
    p = ll.problem(6, 3, 5, 7, seed=3, bias=bias, state=state)
    a, b = ll.forward_float("orc", p), ll.forward_float("ref", p)
    for x, y in zip(a[:3], b[:3]):
        np.testing.assert_array_equal(x, y)
    for n in L.TRACE_VALUES:
        np.testing.assert_array_equal(a[3][n], b[3][n])
    rng = np.random.default_rng(5)
    g = [rng.standard_normal(s).astype(np.float32) for s in [(6, 3, 7), (3, 7), (3, 7)]]
    ga, gb = ll.backward_float("orc", p, a[3], *g), ll.backward_float("ref", p, b[3], *g)
    for n in L.MASTER_VALUES:
        np.testing.assert_array_equal(ga[n], gb[n], err_msg=n)


@needs_ref
@pytest.mark.parametrize("cfg_kw", CONFIGS)
@pytest.mark.parametrize("bias,state", [(True, True), (False, False)])
def test_calibration_params_execution_and_forward_match_reference(cfg_kw, bias, state):
    cfg = L.default_config(**cfg_kw)
    T, B, I, H = 7, 4, 6, 9
    p = ll.problem(T, B, I, H, seed=11, bias=bias, state=state)
    xs = np.stack([p["x"], ll.problem(T, B, I, H, seed=12)["x"] * 1.5])
    ra, pa = ll.calibrate("orc", cfg, p, xs)
    rb, pb = ll.calibrate("ref", cfg, p, xs)
    for op in range(L.NUM_OPS):
        if op in L.PARAMETER_OPS:
            continue
        assert ra.struct.minimum[op] == rb.struct.minimum[op] and ra.struct.maximum[op] == rb.struct.maximum[op], op
        assert pa.struct.scale[op] == pb.struct.scale[op] and pa.struct.zero_point[op] == pb.struct.zero_point[op], op
    for k in range(3):
        assert ra.struct.contribution_min[k] == rb.struct.contribution_min[k]
        assert ra.struct.contribution_max[k] == rb.struct.contribution_max[k]
    for k in range(4 if bias else 2):
        np.testing.assert_array_equal(pa.channel_scales[k], pb.channel_scales[k])
    # the same ranges through the stand-alone finalizer
    pc = ll.params_from_ranges("ref", cfg, ra, I, H, bias)
    for k in range(4 if bias else 2):
        np.testing.assert_array_equal(pa.channel_scales[k], pc.channel_scales[k])
    ea, eb = ll.derive("orc", pa), ll.derive("ref", pb)
    assert ea.flat(bias) == eb.flat(bias)
    assert ea.struct.exact_accumulation == eb.struct.exact_accumulation
    qa, qb = ll.quantize_masters("orc", p, pa), ll.quantize_masters("ref", p, pb)
    for n in qa:
        if qa[n] is not None:
            np.testing.assert_array_equal(qa[n], qb[n], err_msg=n)
    fa, fb = ll.forward_quantized("orc", pa, T, B, qa), ll.forward_quantized("ref", pb, T, B, qb)
    for x, y in zip(fa[:3], fb[:3]):
        np.testing.assert_array_equal(x, y)
    for n in L.TRACE_VALUES:
        np.testing.assert_array_equal(fa[3][n], fb[3][n], err_msg=n)
    # the masked variant returns the same values, and each stage replayed on the saved inputs agrees
    out, hn, cn, tr, mk = ll.forward_quantized_masked(pa, T, B, qa)
    for n in L.TRACE_VALUES:
        np.testing.assert_array_equal(tr[n], fa[3][n])
    rows = T * B
    v, m = ll.stage(pa, 2, rows, tr["weight_ih_linear"], tr["weight_hh_linear"], out_shape=(T, B, 4 * H))
    np.testing.assert_array_equal(v, tr["gate_inputs"])
    np.testing.assert_array_equal(m, mk["gate_inputs"])
    v, m = ll.stage(pa, 6, rows, tr["gate_outputs"], tr["cell_tanh_outputs"], out_shape=(T, B, H))
    np.testing.assert_array_equal(v, tr["hidden_outputs"])


def test_backward_masks_zero_the_gradient_paths():
    p = ll.problem(5, 2, 3, 4, seed=2)
    out, hn, cn, tr = ll.forward_float("orc", p)
    rng = np.random.default_rng(1)
    g = [rng.standard_normal(s).astype(np.float32) for s in [(5, 2, 4), (2, 4), (2, 4)]]
    base = ll.backward_float("orc", p, tr, *g)
    none = ll.backward_float("orc", p, tr, *g, masks={})
    for n in L.MASTER_VALUES:
        np.testing.assert_array_equal(base[n], none[n])
    full = {n: np.ones(tr[n].shape, np.uint8) for n in ("gate_inputs",)}
    cut = ll.backward_float("orc", p, tr, *g, masks=full)
    assert not cut["weight_ih"].any() and not cut["input"].any() and not cut["bias_hh"].any()
    assert cut["initial_cell"].any()  # the cell path does not pass through the gate inputs
    wm = (rng.random((16, 3)) < 0.3).astype(np.uint8)
    part = ll.backward_float("orc", p, tr, *g, masks={"weight_ih": wm})
    np.testing.assert_array_equal(part["weight_ih"], np.where(wm, 0, base["weight_ih"]))


# ---- host-side logic of the shipped library (no GPU needed) -------------------

def product():
    from rx_met_b200 import _quant_lstm
    return _quant_lstm


@pytest.mark.parametrize("cfg_kw", CONFIGS)
@pytest.mark.parametrize("bias", [True, False])
def test_library_host_logic_matches_checker(cfg_kw, bias):
    m = product()
    lib = m._library()
    cfg = L.default_config(**cfg_kw)
    T, B, I, H = 6, 3, 5, 8
    p = ll.problem(T, B, I, H, seed=41, bias=bias)
    ranges, want = ll.calibrate("orc", cfg, p, np.stack([p["x"]]))
    got = L.ParamsBox(H)
    assert lib.rxmet_lstm_params_from_ranges(C.byref(cfg), C.byref(ranges.struct), I, H, int(bias), *got.scale_ptrs(),
                                             C.byref(got.struct)) == 0, lib.rxmet_last_error()
    got.bind()
    for op in range(L.NUM_OPS):
        if op not in L.PARAMETER_OPS:
            assert got.struct.scale[op] == want.struct.scale[op] and got.struct.zero_point[op] == want.struct.zero_point[op]
    for k in range(4 if bias else 2):
        np.testing.assert_array_equal(got.channel_scales[k], want.channel_scales[k])
    ex = L.ExecutionBox(H)
    assert lib.rxmet_lstm_derive_execution(C.byref(got.struct), 0, C.byref(ex.struct)) == 0
    ref = ll.derive("orc", want)
    assert ex.flat(bias) == ref.flat(bias)
    assert ex.struct.exact_accumulation == ref.struct.exact_accumulation
    # bundle JSON round trip and audit
    text = m._params_to_bundle(got)
    back = m._bundle_to_params(text)
    assert m._params_to_bundle(back) == text
    audit = m.audit_quant_params_bundle(text)
    assert audit["bundle_json"] == text and audit["bias_enabled"] == bias
    if ex.struct.exact_accumulation == 0:
        assert lib.rxmet_lstm_derive_execution(C.byref(got.struct), 1, C.byref(ex.struct)) == -1
        assert b"require_exact_accumulation" in lib.rxmet_last_error()


def test_library_default_config_and_config_json():
    m = product()
    cfg = L.QuantConfig()
    assert m._library().rxmet_lstm_default_config(C.byref(cfg)) == 0
    want = L.default_config(symmetric_activations=True)
    assert bytes(cfg) == bytes(want)
    text = m._config_to_json(cfg)
    assert m.validate_resolved_quant_config(text) == text
    merged = json.loads(m.resolve_quant_config(text, json.dumps({"scale_mode": "pot2", "operators": {"cell_state": {"bitwidth": 16}}})))
    assert merged["scale_mode"] == "pot2" and merged["operators"]["cell_state"]["bitwidth"] == 16
    with pytest.raises(ValueError):
        m.resolve_quant_config(text, json.dumps({"operators": {"nonsense": {}}}))
    assert m._shortest_float(0.0078125) == "0.0078125" and m._shortest_float(1.1920929e-07) == "1.1920929e-07"
    # the stats layout the fold consumes
    lib = m._library()
    H = 4
    n = lib.rxmet_lstm_stats_floats(H)
    assert n == 2 * (18 + 3 + 16 * H)
    stats = np.concatenate([np.full(n // 2, 3.4028235e38, np.float32), np.full(n // 2, -3.4028235e38, np.float32)])
    stats[L.INPUT], stats[n // 2 + L.INPUT] = -2.0, 5.0
    box = L.RangesBox(H)
    assert lib.rxmet_lstm_ranges_fold_stats(C.byref(box.struct), stats.ctypes.data_as(C.POINTER(C.c_float)), H, 1) == 0
    assert (box.struct.minimum[L.INPUT], box.struct.maximum[L.INPUT]) == (-2.0, 5.0)
    assert box.struct.minimum[L.OUTPUT] == np.inf  # untouched slots stay empty
