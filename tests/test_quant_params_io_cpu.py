"""Operator JSON and AIMET encodings of the QuantGRU parameters against documents written and read by the
reference's own Python code (tests/golden/quant_params_io.json, made by make_quant_params_io_golden.py)."""
import copy
import json
import os

import pytest

import rx_met_b200.gru_interface_binding as gru_ops
from rx_met_b200 import quant_params_io as qio

with open(os.path.join(os.path.dirname(__file__), "golden", "quant_params_io.json"), encoding="utf-8") as _src:
    CASES = json.load(_src)["cases"]
IDS = [case["name"] for case in CASES]


def _config(attrs):
    cfg = gru_ops.OperatorQuantConfig()
    for key, value in attrs.items():
        setattr(cfg, key, value)
    return cfg


def _params(attrs, cfg):
    if attrs is None:
        return None
    params = gru_ops.GRUQuantParams()
    for key, value in attrs.items():
        setattr(params, key, value)
    params.bitwidth_config_ = cfg
    return params


def _config_attrs(cfg):
    return {k: getattr(cfg, k) for k in sorted(dir(cfg)) if not k.startswith("_") and not callable(getattr(cfg, k))}


def _params_attrs(params):
    if params is None:
        return None
    out = {"hidden_": params.hidden_}
    for key in sorted(dir(params)):
        if key.startswith("scale_") or key.startswith("zp_"):
            value = getattr(params, key)
            out[key] = list(value) if hasattr(value, "__iter__") else value
    return out


def _inputs(case):
    cfg = _config(case["config"])
    return cfg, _params(case["params"], cfg), _params(case["params_reverse"], cfg)


def _text(document):
    # key order and every digit of every float
    return json.dumps(document, indent=2, ensure_ascii=False)


@pytest.mark.parametrize("case", CASES, ids=IDS)
def test_operator_json_matches_the_reference(case, tmp_path):
    cfg, params, reverse = _inputs(case)
    fields = dict(input_size=case["input_size"], hidden_size=case["hidden_size"], bias=True, batch_first=False,
                  bidirectional=case["bidirectional"], config=cfg, params=params, params_reverse=reverse)
    assert _text(qio.quant_params_document(**fields)) == _text(case["document"])
    path = tmp_path / "params.json"
    qio.export_quant_params(str(path), **fields)
    assert path.read_text(encoding="utf-8") == _text(case["document"])


@pytest.mark.parametrize("case", CASES, ids=IDS)
def test_operator_json_loads_like_the_reference(case, tmp_path):
    path = tmp_path / "params.json"
    path.write_text(_text(case["document"]), encoding="utf-8")
    loaded = qio.load_quant_params(str(path), input_size=case["input_size"], hidden_size=case["hidden_size"],
                                   bidirectional=case["bidirectional"])
    want = case["loaded_from_document"]
    assert _config_attrs(loaded.config) == want["config"]
    assert _params_attrs(loaded.params) == want["params"]
    assert _params_attrs(loaded.params_reverse) == want["params_reverse"]
    assert loaded.use_pot2_scale == case["document"]["model_info"]["use_pot2_scale"]


@pytest.mark.parametrize("case", CASES, ids=IDS)
def test_aimet_encodings_match_the_reference(case):
    cfg, params, reverse = _inputs(case)
    made = qio.to_aimet_encodings({}, "encoder.gru", config=cfg, params=params, params_reverse=reverse,
                                  bidirectional=case["bidirectional"])
    assert _text(made) == _text(case["aimet"])


@pytest.mark.parametrize("case", CASES, ids=IDS)
def test_aimet_encodings_load_like_the_reference(case):
    loaded = qio.from_aimet_encodings(copy.deepcopy(case["aimet"]), "encoder.gru", hidden_size=case["hidden_size"],
                                      bidirectional=case["bidirectional"])
    assert loaded is not None
    want = case["loaded_from_aimet"]
    assert _config_attrs(loaded.config) == want["config"]
    assert _params_attrs(loaded.params) == want["params"]
    assert _params_attrs(loaded.params_reverse) == want["params_reverse"]


def test_aimet_export_merges_into_an_existing_dictionary():
    case = CASES[0]
    cfg, params, _ = _inputs(case)
    existing = {"schema_version": 3, "activation_encodings": {"conv1": {"output": {"0": {"scale": 0.5}}}},
                "param_encodings": {"conv1.weight": {"scale": [0.25]}}, "tensor_encodings": {"X": {}}}
    made = qio.to_aimet_encodings(existing, "gru", config=cfg, params=params)
    assert made is existing
    assert set(made["activation_encodings"]) == {"conv1", "gru"}
    assert set(made["param_encodings"]) == {"conv1.weight", "gru.weight_ih.weight", "gru.weight_hh.weight", "gru.bias"}
    assert "tensor_encodings" not in made
    assert len(made["param_encodings"]["gru.bias"]["scale"]) == 6 * case["hidden_size"]


def test_load_rejects_a_document_of_another_module():
    case = CASES[0]
    for field, wrong in (("input_size", 99), ("hidden_size", 99), ("bidirectional", True)):
        expect = dict(input_size=case["input_size"], hidden_size=case["hidden_size"], bidirectional=False)
        expect[field] = wrong
        with pytest.raises(ValueError):
            qio.quant_params_from_document(case["document"], **expect)
    with pytest.raises(ValueError):
        qio.quant_params_from_document({"model_info": case["document"]["model_info"]}, input_size=case["input_size"],
                                       hidden_size=case["hidden_size"])


def test_bidirectional_load_wants_both_directions_and_one_input_grid():
    case = next(c for c in CASES if c["bidirectional"])
    expect = dict(input_size=case["input_size"], hidden_size=case["hidden_size"], bidirectional=True)
    document = copy.deepcopy(case["document"])
    del document["operators_reverse"]
    with pytest.raises(ValueError):
        qio.quant_params_from_document(document, **expect)
    document = copy.deepcopy(case["document"])
    document["operators_reverse"]["input"]["zero_point"] += 1
    with pytest.raises(ValueError):
        qio.quant_params_from_document(document, **expect)


def test_older_scale_fields_are_still_read():
    cfg, params = gru_ops.OperatorQuantConfig(), gru_ops.GRUQuantParams()
    m, shift = qio.encode_multiplier_shift(0.0123)
    assert 32768 <= m < 65536
    qio.operators_from_dict({"input": {"dtype": "UINT8", "multiplier": m, "shift": shift, "zero_point": [7]},
                             "output": {"dtype": "INT16", "n": 9},
                             "weight_ih": {"exp2_inv": [3, 4, 5]},
                             "not_an_operator": {"scale": 1.0}}, cfg, params)
    assert params.scale_x_ == qio.decode_multiplier_shift(m, shift) and abs(params.scale_x_ - 0.0123) < 1e-6
    assert params.zp_x_ == 7 and cfg.x_ == 8 and cfg.x_unsigned_ is True
    assert params.scale_h_ == 2.0 ** -9 and cfg.h_ == 16 and cfg.h_unsigned_ is False
    assert list(params.scale_W_) == [0.125, 0.0625, 0.03125]


def test_bad_records_raise():
    cfg, params = gru_ops.OperatorQuantConfig(), gru_ops.GRUQuantParams()
    for record in ({"scale": []}, {"scale": [0.1, 0.0]}, {"dtype": "INT8"}, {"multiplier": [1, 2], "shift": [3]}):
        with pytest.raises(ValueError):
            qio.operators_from_dict({"weight_hh": record}, cfg, params)
    with pytest.raises(ValueError):
        qio.operators_from_dict({"weight_ih": {"scale": [0.1, 0.2], "enc_type": "PER_GATE"}}, cfg, params)
    # the binding keeps per-channel lists only, as the reference's does
    with pytest.raises(AttributeError):
        qio.operators_from_dict({"weight_ih": {"scale": [0.1], "enc_type": "PER_TENSOR"}}, cfg, params)
    with pytest.raises(ValueError):
        qio.operators_from_dict({"input": {"scale": 0.1, "zero_point": []}}, cfg, params)


def test_aimet_load_failures():
    case = CASES[0]
    good = case["aimet"]
    kwargs = dict(hidden_size=case["hidden_size"])
    assert qio.from_aimet_encodings({}, "encoder.gru", **kwargs) is None
    assert qio.from_aimet_encodings(good, "another.gru", **kwargs) is None
    for missing in ("encoder.gru.weight_ih.weight", "encoder.gru.weight_hh.weight", "encoder.gru.bias"):
        broken = copy.deepcopy(good)
        del broken["param_encodings"][missing]
        assert qio.from_aimet_encodings(broken, "encoder.gru", **kwargs) is None
    for missing in ("input", "output"):
        broken = copy.deepcopy(good)
        del broken["activation_encodings"]["encoder.gru"][missing]
        assert qio.from_aimet_encodings(broken, "encoder.gru", **kwargs) is None
    broken = copy.deepcopy(good)
    broken["activation_encodings"]["encoder.gru"]["input"]["0"]["n"] += 1
    with pytest.raises(ValueError):
        qio.from_aimet_encodings(broken, "encoder.gru", **kwargs)
    broken = copy.deepcopy(good)
    broken["activation_encodings"]["encoder.gru"]["internal_ops"]["new_gate_input"]["output"][0]["scale"] = -1.0
    del broken["activation_encodings"]["encoder.gru"]["internal_ops"]["new_gate_input"]["output"][0]["n"]
    assert qio.from_aimet_encodings(broken, "encoder.gru", **kwargs) is None


def test_encoding_exponent_and_code_ranges():
    assert qio.encoding_exponent(0.25) == 2 and qio.encoding_exponent([1.0, 0.1]) == [0, 3]
    for bad in (0.0, -1.0, float("inf"), True, "1"):
        with pytest.raises(ValueError):
            qio.encoding_exponent(bad)
    assert qio.quant_range(8) == (-128, 127) and qio.quant_range(8, True) == (0, 255) and qio.quant_range(4) == (-8, 7)
    with pytest.raises(ValueError):
        qio.quant_range(33)


def test_quantized_weights_section():
    import torch
    case = CASES[0]
    cfg, params, _ = _inputs(case)
    I, H = case["input_size"], case["hidden_size"]
    W_q = torch.arange(I * 3 * H, dtype=torch.int32).reshape(I, 3 * H) - 30
    R_q = torch.arange(H * 3 * H, dtype=torch.int32).reshape(H, 3 * H) - 50
    bw_q, br_q = torch.arange(3 * H, dtype=torch.int32), -torch.arange(3 * H, dtype=torch.int32)
    weights = qio.weight_codes_for_export(W_q, R_q, bw_q, br_q)
    assert weights["W"] == W_q.tolist() and weights["R"] == R_q.tolist()
    assert weights["bw"] == bw_q.tolist() and weights["br"] == br_q.tolist()
    assert set(qio.weight_codes_for_export(W_q, R_q)) == {"W", "R"}
    document = qio.quant_params_document(input_size=I, hidden_size=H, config=cfg, params=params, quantized_weights=weights)
    assert list(document) == ["model_info", "operators", "quantized_weights"]
    json.dumps(document)
    with pytest.raises(RuntimeError):
        qio.quant_params_document(input_size=I, hidden_size=H, config=cfg, params=None)


@pytest.mark.parametrize("case", CASES, ids=IDS)
def test_io_quant_meta_matches_the_reference(case):
    cfg, params, _ = _inputs(case)
    meta = qio.io_quant_meta(cfg, params)
    assert meta == case["io_quant_meta"]
    assert qio.grids_match(meta["output"], meta["hidden"])
    other = dict(meta["input"], zp=meta["input"]["zp"] + 1)
    assert not qio.grids_match(meta["input"], other)
    with pytest.raises(RuntimeError):
        qio.io_quant_meta(cfg, None)
