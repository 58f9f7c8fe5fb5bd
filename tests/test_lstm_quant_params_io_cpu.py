"""Parameter documents and AIMET encodings of QuantLSTM against documents written and read by the
reference's own Python code (tests/golden/lstm_quant_params_io.json, made by
make_lstm_quant_params_io_golden.py)."""
import copy
import json
import os
import warnings

import pytest

import rx_met_b200._quant_lstm as quant_lstm
from rx_met_b200 import lstm_quant_params_io as lio

with open(os.path.join(os.path.dirname(__file__), "golden", "lstm_quant_params_io.json"), encoding="utf-8") as _src:
    CASES = json.load(_src)["cases"]
IDS = [case["name"] for case in CASES]


def _text(document):
    return json.dumps(document, indent=2, ensure_ascii=False)


def _module(case):
    return dict(input_size=case["input_size"], hidden_size=case["hidden_size"], bias=case["bias"], batch_first=False,
                bidirectional=case["bidirectional"])


def _document(case):
    reverse = case["bundles"][1] if case["bidirectional"] else None
    return lio.quant_params_document(case["bundles"][0], reverse_bundle_json=reverse)


def _audited(bundles):
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        return [quant_lstm.audit_quant_params_bundle(text)["bundle_json"] for text in bundles]


@pytest.mark.parametrize("case", CASES, ids=IDS)
def test_document_matches_the_reference(case, tmp_path):
    assert _text(_document(case)) == _text(case["document"])
    path = tmp_path / "lstm.json"
    reverse = case["bundles"][1] if case["bidirectional"] else None
    lio.export_quant_params(str(path), case["bundles"][0], reverse_bundle_json=reverse)
    assert path.read_text(encoding="utf-8") == _text(case["document"]) + "\n"


@pytest.mark.parametrize("case", CASES, ids=IDS)
def test_document_loads_to_the_bundles_of_the_reference(case):
    bundles = lio.bundles_from_document(copy.deepcopy(case["document"]), **_module(case))
    assert _audited(bundles) == case["bundles_from_document"]
    # and the round trip gives back what was exported
    assert _audited(bundles) == case["bundles"]


@pytest.mark.parametrize("case", CASES, ids=IDS)
def test_aimet_encodings_match_the_reference(case):
    made = lio.to_aimet_encodings({}, "encoder.lstm", _document(case))
    assert _text(made) == _text(case["aimet"])


@pytest.mark.parametrize("case", CASES, ids=IDS)
def test_aimet_encodings_load_to_the_bundles_of_the_reference(case):
    document = lio.document_from_aimet_encodings(copy.deepcopy(case["aimet"]), "encoder.lstm", cublas_math_mode="pedantic",
                                                 activation_operators=case["activation_operators"], **_module(case))
    bundles = lio.bundles_from_document(document, **_module(case))
    assert _audited(bundles) == case["bundles_from_aimet"]


def test_parameter_rows_change_gate_order_and_back():
    case = next(c for c in CASES if c["name"] == "unidirectional_defaults")
    H = case["hidden_size"]
    native = case["document"]["operators"]["weight_hh"]["scale"]
    packed = case["aimet"]["param_encodings"]["encoder.lstm.weight_hh.weight"]["scale"]
    gates = [native[g * H:(g + 1) * H] for g in range(4)]  # i, f, g, o
    assert packed == gates[0] + gates[3] + gates[1] + gates[2]  # i, o, f, c
    bias = case["aimet"]["param_encodings"]["encoder.lstm.bias"]["scale"]
    assert len(bias) == 8 * H


def test_missing_module_and_malformed_entries():
    case = CASES[0]
    kwargs = dict(cublas_math_mode="pedantic", activation_operators=case["activation_operators"], **_module(case))
    assert lio.document_from_aimet_encodings({}, "encoder.lstm", **kwargs) is None
    assert lio.document_from_aimet_encodings(case["aimet"], "another", **kwargs) is None

    def broken(edit):
        enc = copy.deepcopy(case["aimet"])
        edit(enc, enc["activation_encodings"]["encoder.lstm"])
        with pytest.raises(ValueError):
            lio.document_from_aimet_encodings(enc, "encoder.lstm", **kwargs)

    broken(lambda enc, entry: entry.update(is_LSTM=False))
    broken(lambda enc, entry: entry.update(internal_ops_reverse={}))
    broken(lambda enc, entry: entry["internal_ops"].pop("cell_state"))
    broken(lambda enc, entry: entry["internal_ops"]["cell_state"]["output"].append({}))
    broken(lambda enc, entry: entry["internal_ops"]["cell_state"]["output"][0].update(is_symmetric=True))
    broken(lambda enc, entry: entry["internal_ops"]["cell_state"]["output"][0].update(bitwidth=4))
    broken(lambda enc, entry: entry["internal_ops"]["cell_state"]["output"][0].update(n=99))
    broken(lambda enc, entry: entry["internal_ops"]["cell_state"]["output"][0].pop("real_min"))
    broken(lambda enc, entry: enc["param_encodings"].pop("encoder.lstm.bias"))
    broken(lambda enc, entry: enc["param_encodings"]["encoder.lstm.weight_ih.weight"]["scale"].pop())
    broken(lambda enc, entry: entry["input"]["0"].update(zero_point=5))
    broken(lambda enc, entry: entry.update(output=[]))


def test_document_validation():
    case = CASES[0]
    module = _module(case)

    def refused(edit, **changed):
        document = copy.deepcopy(case["document"])
        edit(document)
        with pytest.raises(ValueError):
            lio.bundles_from_document(document, **dict(module, **changed))

    refused(lambda d: None, hidden_size=99)
    refused(lambda d: None, bias=not case["bias"])
    refused(lambda d: None, bidirectional=True)
    refused(lambda d: d.update(extra=1))
    refused(lambda d: d.update(schema_version=2))
    refused(lambda d: d.update(schema_version=True))
    refused(lambda d: d["model_info"].pop("bias"))
    refused(lambda d: d["model_info"].update(use_pot2_scale=True))
    refused(lambda d: d["execution_metadata"].update(carrier="other"))
    refused(lambda d: d["execution_metadata"].update(cublas_math_mode="fast"))
    refused(lambda d: d["operators"]["input"].update(real_max=1.0))
    refused(lambda d: d["operators"]["input"].update(dtype="INT0"))
    refused(lambda d: d["operators"]["input"].update(enc_type="PER_ROW"))
    refused(lambda d: d["operators"]["input"].update(zero_point=0.5))
    refused(lambda d: d["operators"]["input"].update(scale=[d["operators"]["input"]["scale"]]))
    refused(lambda d: d["operators"]["input"].pop("symmetric"))
    with pytest.warns(RuntimeWarning):
        lio.bundles_from_document(copy.deepcopy(case["document"]), **dict(module, batch_first=True))


def test_two_directions_must_share_the_input_grid():
    case = next(c for c in CASES if c["bidirectional"])
    document = copy.deepcopy(case["document"])
    record = document["operators_reverse"]["input"]
    record["scale"] = record["scale"] * 2
    record["real_min"], record["real_max"] = record["real_min"] * 2, record["real_max"] * 2
    with pytest.raises(ValueError):
        lio.bundles_from_document(document, **_module(case))


def test_text_helpers():
    assert lio.canonical_float32(0.1) == "0.1" and lio.canonical_float32(2.0 ** -7) == "0.0078125"
    assert lio.canonical_float32(1.0 / 3.0) == "0.33333334"
    for bad in (0.0, -1.0, float("inf"), 1e60):
        with pytest.raises(ValueError):
            lio.canonical_float32(bad)
    assert lio.parse_dtype("UINT4") == (4, True) and lio.parse_dtype("INT32") == (32, False)
    for bad in ("UINT32", "INT33", "int8", 8, "INT08"):
        with pytest.raises(ValueError):
            lio.parse_dtype(bad)
    with pytest.raises(ValueError):
        lio.parse_dtype("INT1", symmetric=True)
    with pytest.raises(ValueError):
        lio.strict_json('{"a": 1, "a": 2}')
    with pytest.raises(ValueError):
        lio.strict_json("[1]")
