"""On-disk forms of the QuantLSTM quantization parameters.

The extension hands quantization parameters around as a *bundle* (compact JSON: per operator bitwidth,
signedness, symmetry, granularity, float32 scales as shortest decimal strings, zero points).  Two public
forms are derived from it:

* the parameter document of ``QuantLSTM.export_quant_params`` / ``load_quant_params``, field-compatible
  with QuantGRU's operator JSON (reference: operators/quant-lstm/pytorch/quant_lstm.py:145-177 bundle ->
  document, :218-292 document -> bundle, :295-380 validation, :778-808 and :1194-1230 export);
* the AIMET encodings dictionary of ``export_quant_params_to_aimet_format`` /
  ``load_quant_params_from_aimet_format`` (operators/quant-lstm/pytorch/lstm_aimet.py:76-176 record
  translation and parameter packing, :293-333 export, :335-410 load).  Parameter encodings are per
  channel in the ONNX gate order i, o, f, c; the bundle's order is i, f, g(c), o.

Everything here is host-side text work; the bundles it returns go to
`rx_met_b200._quant_lstm.audit_quant_params_bundle`, which re-derives the execution encodings.
"""
from __future__ import annotations

import json
import math
import struct
import warnings
from copy import deepcopy
from typing import Any, Dict, Iterable, List, Optional, Tuple

PARAMETER_OPERATORS = ("weight_ih", "weight_hh", "bias_ih", "bias_hh")
_RECORD_FIELDS = ("dtype", "symmetric", "scale", "zero_point", "enc_type", "real_min", "real_max")
_VALUE_FIELDS = ("scale", "zero_point", "real_min", "real_max")
_ENC_TYPE = {"per_tensor": "PER_TENSOR", "per_gate": "PER_GATE", "per_channel": "PER_CHANNEL"}
_GRANULARITY = {v: k for k, v in _ENC_TYPE.items()}
_MATH_MODES = ("pedantic", "tf32")
_CARRIER = "cuda_fp32_qcarrier"
_ACTIVATIONS = "real_sigmoid_tanh"
# bundle rows run i, f, g, o; ONNX rows run i, o, f, c(=g)
_TO_ONNX = (0, 3, 1, 2)
_FROM_ONNX = (0, 2, 3, 1)


def strict_json(text: str) -> Dict[str, Any]:
    """json.loads that refuses duplicate keys and a non-object root (quant_lstm.py:80-92)."""
    def unique(pairs):
        out: Dict[str, Any] = {}
        for key, value in pairs:
            if key in out:
                raise ValueError(f"JSON has a duplicate key: {key}")
            out[key] = value
        return out

    value = json.loads(text, object_pairs_hook=unique)
    if not isinstance(value, dict):
        raise ValueError("JSON root must be an object")
    return value


def _float32(value: float) -> float:
    try:
        return struct.unpack("!f", struct.pack("!f", value))[0]
    except (OverflowError, struct.error) as error:
        raise ValueError("scale is outside the float32 range") from error


def canonical_float32(value: float) -> str:
    """Shortest `%g` decimal (1-9 digits) that reads back as the same float32 (quant_lstm.py:206-215)."""
    rounded = _float32(value)
    if not math.isfinite(rounded) or rounded <= 0.0:
        raise ValueError("scale must be a finite positive float32")
    bits = struct.pack("!f", rounded)
    for digits in range(1, 10):
        text = format(rounded, f".{digits}g")
        if struct.pack("!f", float(text)) == bits:
            return text
    raise ValueError("scale has no float32 decimal form")


def _code_range(bitwidth: int, unsigned: bool) -> Tuple[int, int]:
    if unsigned:
        return 0, (1 << bitwidth) - 1
    return -(1 << (bitwidth - 1)), (1 << (bitwidth - 1)) - 1


def _one_or_all(values: List[Any]) -> Any:
    return values[0] if len(values) == 1 else values


_DTYPE_ERROR = "Encoding dtype must be an INTn or UINTn string"
_MAX_BITS = {"INT": 32, "UINT": 31}


def parse_dtype(dtype: Any, *, symmetric: Optional[bool] = None) -> Tuple[int, bool]:
    """"INT8" -> (8, False), "UINT4" -> (4, True).  Same acceptance rules and messages as the reference's
    parser (lstm_aimet.py:51-63): widths 1..32 signed, 1..31 unsigned, no leading zeros, and no signed symmetric
    one-bit grid (its largest code would be 0)."""
    if not isinstance(dtype, str):
        raise ValueError(_DTYPE_ERROR)
    for family in ("UINT", "INT"):
        digits = dtype[len(family):]
        if dtype.startswith(family) and digits.isascii() and digits.isdigit() and digits[0] != "0":
            break
    else:
        raise ValueError(_DTYPE_ERROR)
    bitwidth = int(digits)
    if bitwidth < 1 or bitwidth > _MAX_BITS[family]:
        raise ValueError("Encoding bitwidth must be INT1..INT32 or UINT1..UINT31")
    if family == "INT" and bitwidth == 1 and symmetric is True:
        raise ValueError("signed symmetric INT1 has qmax=0 and is unsupported")
    return bitwidth, family == "UINT"


def encoding_exponent(scale: Any) -> Any:
    """n with scale ~ 2^-n for one scale or, element by element, for a non-empty list of them
    (lstm_aimet.py:66-73); anything but a positive finite number is rejected."""
    if isinstance(scale, list):
        if len(scale) == 0:
            raise ValueError("Encoding scale cannot be empty")
        return list(map(encoding_exponent, scale))
    is_number = isinstance(scale, (int, float)) and not isinstance(scale, bool)
    if not (is_number and math.isfinite(scale) and scale > 0):
        raise ValueError("Encoding scale must be positive and finite")
    return int(round(-math.log2(scale)))


# ---------------------------------------------------------------------------------------------
# bundle <-> parameter document
# ---------------------------------------------------------------------------------------------

def operator_record(operator: Dict[str, Any]) -> Dict[str, Any]:
    """One bundle operator as a public record (quant_lstm.py:145-170)."""
    scales = [_float32(float(v)) for v in operator["scales"]]
    zeros = [int(v) for v in operator["zero_points"]]
    low, high = _code_range(operator["bitwidth"], operator["is_unsigned"])
    return {
        "dtype": f"{'U' if operator['is_unsigned'] else ''}INT{operator['bitwidth']}",
        "symmetric": operator["is_symmetric"],
        "scale": _one_or_all(scales),
        "zero_point": _one_or_all(zeros),
        "enc_type": _ENC_TYPE[operator["granularity"]],
        "real_min": _one_or_all([s * (low - z) for s, z in zip(scales, zeros)]),
        "real_max": _one_or_all([s * (high - z) for s, z in zip(scales, zeros)]),
    }


def quant_params_document(bundle_json: str, *, batch_first: bool = False, cublas_math_mode: str = "pedantic",
                          reverse_bundle_json: Optional[str] = None) -> Dict[str, Any]:
    """The document ``export_quant_params`` returns for a calibrated module; `reverse_bundle_json` makes it
    the bidirectional form (quant_lstm.py:778-808, :1194-1230)."""
    if bundle_json is None:
        raise RuntimeError("the module is not calibrated: there are no quantization parameters to export")
    bundle = strict_json(bundle_json)
    pot2 = bundle["scale_mode"] == "pot2"
    document: Dict[str, Any] = {
        "schema_version": 1,
        "model_info": {
            "input_size": bundle["input_size"],
            "hidden_size": bundle["hidden_size"],
            "bias": bundle["bias_enabled"],
            "batch_first": batch_first,
            "bidirectional": reverse_bundle_json is not None,
            "use_pot2_scale": pot2,
        },
        "execution_metadata": {
            "carrier": _CARRIER,
            "activation_mode": _ACTIVATIONS,
            "cublas_math_mode": cublas_math_mode,
            "standard_scale_mode": bundle["scale_mode"],
        },
        "operators": {name: operator_record(op) for name, op in bundle["operators"].items()},
    }
    if reverse_bundle_json is not None:
        reverse = strict_json(reverse_bundle_json)
        document["operators_reverse"] = {name: operator_record(op) for name, op in reverse["operators"].items()}
    return document


def export_quant_params(destination: str, bundle_json: str, **fields) -> Dict[str, Any]:
    document = quant_params_document(bundle_json, **fields)
    with open(destination, "w", encoding="utf-8") as out:
        out.write(json.dumps(document, indent=2, ensure_ascii=False) + "\n")
    return document


def _numbers(value: Any, field: str) -> Tuple[List[float], bool]:
    listed = isinstance(value, list)
    values = value if listed else [value]
    if not values:
        raise ValueError(f"{field} must not be empty")
    out = []
    for item in values:
        if isinstance(item, bool) or not isinstance(item, (int, float)):
            raise ValueError(f"{field} must be a JSON number or an array of numbers")
        if not math.isfinite(float(item)):
            raise ValueError(f"{field} must be finite")
        out.append(float(item))
    return out, listed


def _integers(value: Any, field: str) -> Tuple[List[int], bool]:
    listed = isinstance(value, list)
    values = value if listed else [value]
    if not values:
        raise ValueError(f"{field} must not be empty")
    if any(isinstance(item, bool) or not isinstance(item, int) for item in values):
        raise ValueError(f"{field} must be a JSON integer or an array of integers")
    return [int(item) for item in values], listed


def bundle_operator(name: str, record: Any) -> Dict[str, Any]:
    """A public record back as a bundle operator; real_min / real_max must agree with scale and zero
    point to 1e-12 relative (quant_lstm.py:218-275)."""
    if not isinstance(record, dict) or set(record) != set(_RECORD_FIELDS):
        raise ValueError(f"operator {name}: fields are missing or unknown")
    if not isinstance(record["symmetric"], bool):
        raise ValueError(f"operator {name}: symmetric must be a boolean")
    try:
        bitwidth, unsigned = parse_dtype(record["dtype"], symmetric=record["symmetric"])
    except ValueError as error:
        raise ValueError(f"operator {name}: bad dtype: {error}") from error
    if record["enc_type"] not in _GRANULARITY:
        raise ValueError(f"operator {name}: bad enc_type")
    scales, a = _numbers(record["scale"], f"{name}.scale")
    zeros, b = _integers(record["zero_point"], f"{name}.zero_point")
    lows, c = _numbers(record["real_min"], f"{name}.real_min")
    highs, d = _numbers(record["real_max"], f"{name}.real_max")
    if not a == b == c == d:
        raise ValueError(f"operator {name}: scalar and array fields are mixed")
    if not len(scales) == len(zeros) == len(lows) == len(highs):
        raise ValueError(f"operator {name}: field lengths differ")
    low, high = _code_range(bitwidth, unsigned)
    for index, (scale, zero, real_low, real_high) in enumerate(zip(scales, zeros, lows, highs)):
        if not math.isclose(real_low, scale * (low - zero), rel_tol=1.0e-12):
            raise ValueError(f"operator {name}: real_min[{index}] disagrees with scale and zero point")
        if not math.isclose(real_high, scale * (high - zero), rel_tol=1.0e-12):
            raise ValueError(f"operator {name}: real_max[{index}] disagrees with scale and zero point")
    return {"bitwidth": bitwidth, "is_unsigned": unsigned, "is_symmetric": record["symmetric"],
            "granularity": _GRANULARITY[record["enc_type"]],
            "scales": [canonical_float32(v) for v in scales], "zero_points": zeros}


def validate_document(document: Any, *, input_size: int, hidden_size: int, bias: bool, batch_first: bool,
                      bidirectional: bool) -> None:
    """Shape of a parameter document and its fit to the module it is loaded into (quant_lstm.py:295-380).
    A different batch_first only warns: the parameters do not depend on the layout."""
    fields = {"schema_version", "model_info", "execution_metadata", "operators"}
    if bidirectional:
        fields.add("operators_reverse")
    if not isinstance(document, dict) or set(document) != fields:
        raise ValueError("parameter document: fields are missing or unknown")
    version = document["schema_version"]
    if isinstance(version, bool) or not isinstance(version, int) or version != 1:
        raise ValueError("parameter document: only schema_version=1 is supported")

    info = document["model_info"]
    if not isinstance(info, dict) or set(info) != {"input_size", "hidden_size", "bias", "batch_first",
                                                   "bidirectional", "use_pot2_scale"}:
        raise ValueError("model_info: fields are missing or unknown")
    for field in ("bias", "batch_first", "bidirectional", "use_pot2_scale"):
        if not isinstance(info[field], bool):
            raise ValueError(f"model_info.{field} must be a boolean")
    for field in ("input_size", "hidden_size"):
        if isinstance(info[field], bool) or not isinstance(info[field], int):
            raise ValueError(f"model_info.{field} must be an integer")
    if (info["input_size"], info["hidden_size"], info["bias"], info["bidirectional"]) != (
            input_size, hidden_size, bias, bidirectional):
        raise ValueError("model_info: shape, bias or bidirectional does not match the module")
    if info["batch_first"] != batch_first:
        warnings.warn("the document's batch_first differs from the module's; quantization parameters do not "
                      "depend on the layout", RuntimeWarning, stacklevel=3)

    meta = document["execution_metadata"]
    if not isinstance(meta, dict) or set(meta) != {"carrier", "activation_mode", "cublas_math_mode",
                                                   "standard_scale_mode"}:
        raise ValueError("execution_metadata: fields are missing or unknown")
    if meta["carrier"] != _CARRIER:
        raise ValueError(f"only the {_CARRIER} carrier is supported")
    if meta["activation_mode"] != _ACTIVATIONS:
        raise ValueError(f"only the {_ACTIVATIONS} activation mode is supported")
    if meta["cublas_math_mode"] not in _MATH_MODES:
        raise ValueError("cublas_math_mode is not one of pedantic, tf32")
    if meta["standard_scale_mode"] not in ("affine", "pot2"):
        raise ValueError("standard_scale_mode is not one of affine, pot2")
    if info["use_pot2_scale"] != (meta["standard_scale_mode"] == "pot2"):
        raise ValueError("use_pot2_scale contradicts standard_scale_mode")
    for field in ("operators", "operators_reverse"):
        if field in document and not isinstance(document[field], dict):
            raise ValueError(f"{field} must be an object")


def bundle_from_document(document: Dict[str, Any], operators_field: str = "operators") -> str:
    """Compact bundle JSON of one direction of a validated document (quant_lstm.py:278-292, :826-830)."""
    info = document["model_info"]
    bundle = {
        "schema_version": 1,
        "input_size": info["input_size"],
        "hidden_size": info["hidden_size"],
        "bias_enabled": info["bias"],
        "scale_mode": document["execution_metadata"]["standard_scale_mode"],
        "operators": {name: bundle_operator(name, record) for name, record in document[operators_field].items()},
    }
    return json.dumps(bundle, separators=(",", ":"), ensure_ascii=False)


def bundles_from_document(document: Any, **module) -> List[str]:
    """Validates `document` against the module (`input_size`, `hidden_size`, `bias`, `batch_first`,
    `bidirectional`) and returns one bundle per direction.  A bidirectional document must share the input
    grid between its directions (quant_lstm.py:1232-1280)."""
    validate_document(document, **module)
    bundles = [bundle_from_document(document, "operators")]
    if module["bidirectional"]:
        bundles.append(bundle_from_document(document, "operators_reverse"))
        if document["operators"]["input"] != document["operators_reverse"]["input"]:
            raise ValueError("the two directions do not share the input quantization grid")
    return bundles


# ---------------------------------------------------------------------------------------------
# AIMET encodings
# ---------------------------------------------------------------------------------------------

def _as_encoding(record: Dict[str, Any]) -> Dict[str, Any]:
    """lstm_aimet.py:76-83."""
    encoding = deepcopy(record)
    encoding["bitwidth"], _ = parse_dtype(encoding["dtype"], symmetric=encoding["symmetric"])
    encoding["is_symmetric"] = "True" if encoding.pop("symmetric") else "False"
    encoding["n"] = encoding_exponent(encoding["scale"])
    return encoding


def _internal_ops(operators: Dict[str, Dict[str, Any]]) -> Dict[str, Dict[str, list]]:
    return {name: {"output": [_as_encoding(record)]} for name, record in operators.items()
            if name not in PARAMETER_OPERATORS}


def _packed_parameter(document: Dict[str, Any], names: Iterable[str]) -> Dict[str, Any]:
    """One per-channel encoding over every direction and every operator of `names`, rows reordered to the
    ONNX gate order; scalar (per-tensor) fields are repeated per row (lstm_aimet.py:93-121)."""
    names = tuple(names)
    hidden = document["model_info"]["hidden_size"]
    directions = [document["operators"]] + ([document["operators_reverse"]] if "operators_reverse" in document else [])
    first = directions[0][names[0]]
    for operators in directions:
        for name in names:
            if any(operators[name][key] != first[key] for key in ("dtype", "symmetric")):
                raise ValueError(f"ONNX packed parameter has incompatible encodings: {names}")
    packed: Dict[str, Any] = {"dtype": first["dtype"], "symmetric": first["symmetric"], "enc_type": "PER_CHANNEL"}
    for field in _VALUE_FIELDS:
        rows: List[Any] = []
        for operators in directions:
            for name in names:
                values = operators[name][field]
                if not isinstance(values, list):
                    values = [values] * (4 * hidden)
                if len(values) != 4 * hidden:
                    raise ValueError(f"Invalid native LSTM parameter row count: {name}.{field}")
                rows.extend(values[gate * hidden + j] for gate in _TO_ONNX for j in range(hidden))
        packed[field] = rows
    return _as_encoding(packed)


def to_aimet_encodings(encodings: Dict[str, Any], module_name: Optional[str], document: Dict[str, Any]) -> Dict[str, Any]:
    """Merges a module's parameter document into an AIMET encodings dictionary (lstm_aimet.py:293-333).
    The caller's dictionary is only touched after every parameter has packed."""
    name = module_name if module_name is not None else "lstm"
    operators = document["operators"]
    entry: Dict[str, Any] = {
        "is_LSTM": True,
        "input": {"0": _as_encoding(operators["input"])},
        "output": {"0": _as_encoding(operators["output"])},
        "internal_ops": _internal_ops(operators),
    }
    if "operators_reverse" in document:
        entry["internal_ops_reverse"] = _internal_ops(document["operators_reverse"])
    parameters = {}
    for suffix, names in (("weight_ih.weight", ("weight_ih",)), ("weight_hh.weight", ("weight_hh",)),
                          ("bias", ("bias_ih", "bias_hh"))):
        if suffix == "bias" and not document["model_info"]["bias"]:
            continue
        parameters[f"{name}.{suffix}"] = _packed_parameter(document, names)
    encodings.setdefault("schema_version", 3)
    encodings.setdefault("activation_encodings", {})[name] = entry
    encodings.setdefault("param_encodings", {}).update(parameters)
    return encodings


def _record_of_encoding(encoding: Any, label: str) -> Dict[str, Any]:
    """An AIMET encoding back as a public record, checked for consistency (lstm_aimet.py:124-152)."""
    if not isinstance(encoding, dict):
        raise ValueError(f"Invalid encoding record: {label}")
    symmetric = encoding.get("is_symmetric")
    if symmetric not in ("True", "False"):
        raise ValueError(f"Invalid encoding symmetry: {label}")
    try:
        bitwidth, _ = parse_dtype(encoding.get("dtype"), symmetric=symmetric == "True")
    except ValueError as error:
        raise ValueError(f"Invalid encoding dtype for {label}: {error}") from error
    stored = encoding.get("bitwidth")
    if not isinstance(stored, int) or isinstance(stored, bool) or stored != bitwidth:
        raise ValueError(f"Inconsistent encoding bitwidth: {label}")

    def same(actual, expected):
        if isinstance(expected, list):
            return (isinstance(actual, list) and len(actual) == len(expected)
                    and all(same(a, b) for a, b in zip(actual, expected)))
        return isinstance(actual, int) and not isinstance(actual, bool) and actual == expected

    try:
        if "n" in encoding and not same(encoding["n"], encoding_exponent(encoding["scale"])):
            raise ValueError(f"Encoding n does not match scale: {label}")
        return {"dtype": encoding["dtype"], "symmetric": symmetric == "True", "enc_type": encoding["enc_type"],
                **{field: deepcopy(encoding[field]) for field in _VALUE_FIELDS}}
    except KeyError as error:
        raise ValueError(f"Missing encoding field for {label}: {error.args[0]}") from error


def _unpacked_parameter(encoding: Any, names: Tuple[str, ...], hidden: int, directions: int,
                        label: str) -> List[Dict[str, Dict[str, Any]]]:
    """Inverse of `_packed_parameter`: per direction, per operator, rows back in the bundle's gate order
    (lstm_aimet.py:155-176)."""
    record = _record_of_encoding(encoding, label)
    rows = 4 * hidden
    for field in _VALUE_FIELDS:
        if not isinstance(record[field], list) or len(record[field]) != directions * len(names) * rows:
            raise ValueError(f"Invalid ONNX parameter encoding length: {label}.{field}")
    out: List[Dict[str, Dict[str, Any]]] = [dict() for _ in range(directions)]
    for direction in range(directions):
        for index, name in enumerate(names):
            start = (direction * len(names) + index) * rows
            piece: Dict[str, Any] = {"dtype": record["dtype"], "symmetric": record["symmetric"], "enc_type": "PER_CHANNEL"}
            for field in _VALUE_FIELDS:
                piece[field] = [record[field][start + gate * hidden + j] for gate in _FROM_ONNX for j in range(hidden)]
            out[direction][name] = piece
    return out


def document_from_aimet_encodings(encodings: Dict[str, Any], module_name: Optional[str], *, input_size: int,
                                  hidden_size: int, bias: bool, batch_first: bool, bidirectional: bool,
                                  cublas_math_mode: str, activation_operators: Iterable[str]) -> Optional[Dict[str, Any]]:
    """Rebuilds the in-memory parameter document of a module from an AIMET encodings dictionary; the
    caller loads it like any other document (lstm_aimet.py:335-410).  `activation_operators` names the
    module's non-parameter operators: internal_ops must hold exactly those.  Returns None when the module
    has no entry; raises ValueError on a malformed one."""
    name = module_name if module_name is not None else "lstm"
    entry = encodings.get("activation_encodings", {}).get(name)
    if entry is None:
        return None
    if not isinstance(entry, dict) or entry.get("is_LSTM") is not True:
        raise ValueError(f"Expected LSTM activation encodings: {name}")
    directions = 2 if bidirectional else 1
    if not bidirectional and "internal_ops_reverse" in entry:
        raise ValueError(f"Unexpected reverse LSTM encodings: {name}")
    required = set(activation_operators) - set(PARAMETER_OPERATORS)
    operators: List[Dict[str, Dict[str, Any]]] = []
    for field in ("internal_ops", "internal_ops_reverse")[:directions]:
        internal = entry.get(field)
        if not isinstance(internal, dict) or set(internal) != required:
            raise ValueError(f"Missing or unexpected LSTM internal encodings: {name}.{field}")
        records = {}
        for operator, slot in internal.items():
            inner = slot.get("output") if isinstance(slot, dict) else None
            if not isinstance(inner, list) or len(inner) != 1:
                raise ValueError(f"Expected one internal encoding: {name}.{field}.{operator}")
            records[operator] = _record_of_encoding(inner[0], f"{name}.{field}.{operator}")
        operators.append(records)
    parameters = encodings.get("param_encodings", {})
    for suffix, names in (("weight_ih.weight", ("weight_ih",)), ("weight_hh.weight", ("weight_hh",)),
                          ("bias", ("bias_ih", "bias_hh"))):
        if suffix == "bias" and not bias:
            continue
        key = f"{name}.{suffix}"
        if key not in parameters:
            raise ValueError(f"Missing LSTM parameter encoding: {key}")
        for records, unpacked in zip(operators, _unpacked_parameter(parameters[key], names, hidden_size, directions, key)):
            records.update(unpacked)
    scales = [s for records in operators for record in records.values()
              for s in (record["scale"] if isinstance(record["scale"], list) else [record["scale"]])]
    pot2 = all(isinstance(s, (int, float)) and s > 0 and math.isfinite(s) and math.frexp(s)[0] == 0.5 for s in scales)
    document: Dict[str, Any] = {
        "schema_version": 1,
        "model_info": {"input_size": input_size, "hidden_size": hidden_size, "bias": bias, "batch_first": batch_first,
                       "bidirectional": bidirectional, "use_pot2_scale": pot2},
        "execution_metadata": {"carrier": _CARRIER, "activation_mode": _ACTIVATIONS,
                               "cublas_math_mode": cublas_math_mode,
                               "standard_scale_mode": "pot2" if pot2 else "affine"},
        "operators": operators[0],
    }
    if bidirectional:
        document["operators_reverse"] = operators[1]
    for side in ("input", "output"):
        port = entry.get(side)
        if isinstance(port, dict) and set(port) == {"0"}:
            encoding = port["0"]
        elif isinstance(port, list) and len(port) == 1:
            encoding = port[0]
        else:
            raise ValueError(f"Expected one LSTM {side} encoding: {name}")
        if _record_of_encoding(encoding, f"{name}.{side}") != operators[0][side]:
            raise ValueError(f"LSTM input/output encodings disagree with internal grids: {name}")
    return document
