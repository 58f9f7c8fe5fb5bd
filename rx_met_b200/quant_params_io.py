"""On-disk forms of the QuantGRU quantization parameters.

Two formats carry an `OperatorQuantConfig` + `GRUQuantParams` pair (one pair per direction) between
calibration and deployment:

* the operator JSON written by ``QuantGRU.export_quant_params`` / read by ``load_quant_params``
  (reference: operators/quant-gru/pytorch/quant_gru.py:4111-4216 build, :4231-4434 parse,
  :4475-4527 export, :4581-4667 load);
* the AIMET encodings dictionary filled by ``export_quant_params_to_aimet_format`` and read back by
  ``load_quant_params_from_aimet_format`` (quant_gru.py:2593-3163 and :3165-3590).

The functions here take and return the binding objects of `rx_met_b200.gru_interface_binding`, so the
module methods of the reference delegate to them one to one.  Nothing here touches a device: the
parameters are host scalars and per-channel lists.
"""
from __future__ import annotations

import copy
import json
import math
import re
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from . import gru_interface_binding as gru_ops

# JSON name -> attribute stem of the binding objects, in the order of the exported file
# (quant_gru.py:210-235).  The four weight operators are per channel and have no zero point.
_WEIGHT_OPS = ("weight_ih", "weight_hh", "bias_ih", "bias_hh")
_STEMS: Dict[str, str] = {
    "input": "x_",
    "output": "h_",
    "weight_ih": "W_",
    "weight_hh": "R_",
    "bias_ih": "bw_",
    "bias_hh": "br_",
    "weight_ih_linear": "weight_ih_linear_",
    "weight_hh_linear": "weight_hh_linear_",
    "update_gate_input": "update_gate_input_",
    "update_gate_output": "update_gate_output_",
    "reset_gate_input": "reset_gate_input_",
    "reset_gate_output": "reset_gate_output_",
    "new_gate_input": "new_gate_input_",
    "new_gate_output": "new_gate_output_",
    "mul_reset_hidden": "mul_reset_hidden_",
    "mul_old_contribution": "mul_old_contribution_",
    "mul_new_contribution": "mul_new_contribution_",
}
# operators that live under internal_ops of an AIMET module entry, in reading order
_INTERNAL_OPS = (
    "weight_ih_linear", "weight_hh_linear", "update_gate_input", "update_gate_output", "reset_gate_input",
    "reset_gate_output", "new_gate_input", "new_gate_output", "mul_reset_hidden", "mul_old_contribution",
    "mul_new_contribution",
)
# two more entries repeat another operator's encoding: the final add has the grid of the output, 1 - u the
# grid of the update gate
_ALIASED_INTERNAL_OPS = (("add_final_hidden", "output"), ("sub_one_minus_update", "update_gate_output"))
_LIST_FIELDS = ("scale", "zero_point", "real_min", "real_max")
_GRANULARITY = {0: "PER_TENSOR", 1: "PER_GATE", 2: "PER_CHANNEL"}


@dataclass
class LoadedQuantParams:
    """What a load returns: the configuration shared by both directions and one parameter set each."""
    config: "gru_ops.OperatorQuantConfig"
    params: "gru_ops.GRUQuantParams"
    params_reverse: Optional["gru_ops.GRUQuantParams"]
    use_pot2_scale: bool
    model_info: Dict[str, Any]


def quant_range(bitwidth: int, is_unsigned: bool = False) -> Tuple[int, int]:
    """Code range of a grid (quant_gru.py:766-796)."""
    if not 1 <= bitwidth <= 32:
        raise ValueError(f"bitwidth must be in range [1, 32], got {bitwidth}")
    if is_unsigned:
        return 0, (1 << bitwidth) - 1
    return -(1 << (bitwidth - 1)), (1 << (bitwidth - 1)) - 1


def _one_or_all(values: List[Any]) -> Any:
    return values[0] if len(values) == 1 else values


def _as_floats(value: Any) -> List[float]:
    if hasattr(value, "__iter__") and not isinstance(value, str):
        return [float(v) for v in value]
    return [float(value)]


def encoding_exponent(scale: Any) -> Any:
    """The descriptive ``n`` of an encoding: the nearest power-of-two exponent of its scale
    (quant_gru.py:4039-4046)."""
    if isinstance(scale, list):
        if not scale:
            raise ValueError("Encoding scale cannot be empty")
        return [encoding_exponent(v) for v in scale]
    if isinstance(scale, bool) or not isinstance(scale, (int, float)) or not math.isfinite(scale) or scale <= 0:
        raise ValueError("Encoding scale must be positive and finite")
    return int(round(-math.log2(scale)))


def validate_encoding_exponents(value: Any) -> None:
    """Raises ValueError where a stored ``n`` disagrees with its ``scale`` (quant_gru.py:4049-4065)."""
    def same(actual: Any, expected: Any) -> bool:
        if isinstance(expected, list):
            return (isinstance(actual, list) and len(actual) == len(expected)
                    and all(same(a, b) for a, b in zip(actual, expected)))
        return isinstance(actual, int) and not isinstance(actual, bool) and actual == expected

    if isinstance(value, dict):
        if "scale" in value:
            if "n" in value and not same(value["n"], encoding_exponent(value["scale"])):
                raise ValueError("Encoding n does not match scale")
        else:
            for child in value.values():
                validate_encoding_exponents(child)
    elif isinstance(value, list):
        for child in value:
            validate_encoding_exponents(child)


def encode_multiplier_shift(scale: float) -> Tuple[int, int]:
    """16-bit multiplier and shift of a real scale, scale ~= m * 2**-shift with m in [2**15, 2**16)
    (quant_gru.py:4068-4081)."""
    if not scale > 0.0:
        raise ValueError(f"scale must be > 0, got {scale}")
    mantissa, exponent = math.frexp(float(scale))
    m = int(round(mantissa * 65536.0))
    if m == 65536:
        m, exponent = 32768, exponent + 1
    m = max(m, 32768)
    shift = 16 - exponent
    if not -128 <= shift <= 127:
        raise ValueError(f"shift {shift} of scale {scale} is out of range")
    return m, shift


def decode_multiplier_shift(multiplier: int, shift: int) -> float:
    """quant_gru.py:4084-4085."""
    return float(multiplier) * math.ldexp(1.0, -int(shift))


# ---------------------------------------------------------------------------------------------
# operator dictionaries
# ---------------------------------------------------------------------------------------------

def _operator_record(config, params, name: str) -> Optional[Dict[str, Any]]:
    stem = _STEMS[name]
    weight = name in _WEIGHT_OPS
    bitwidth = getattr(config, stem)
    symmetric = getattr(config, stem + "symmetric_")
    unsigned = getattr(config, stem + "unsigned_", False)
    qmin, qmax = quant_range(bitwidth, unsigned)
    if not hasattr(params, "scale_" + stem):
        return None
    raw = getattr(params, "scale_" + stem)
    if weight:
        scales = _as_floats(raw)
        # The reference looks the granularity up under the JSON name ("weight_ih_granularity_"), an
        # attribute the configuration does not have, and then writes PER_CHANNEL (quant_gru.py:3971-4010).
        # The same lookup is kept so that both sides write the same file.
        enc_type = _GRANULARITY.get(getattr(config, name + "_granularity_", None), "PER_CHANNEL")
        zero = 0
    else:
        scales = _as_floats(raw)
        if hasattr(raw, "__iter__") and not scales:
            scales = [1.0]
        enc_type = "PER_TENSOR"
        zero = int(getattr(params, "zp_" + stem)) if hasattr(params, "zp_" + stem) else 0
    zeros = [zero] * len(scales)
    return {
        "dtype": ("UINT" if unsigned else "INT") + str(bitwidth),
        "symmetric": symmetric,
        "scale": _one_or_all(scales),
        "zero_point": _one_or_all(zeros),
        "enc_type": enc_type,
        "real_min": _one_or_all([s * (qmin - z) for s, z in zip(scales, zeros)]),
        "real_max": _one_or_all([s * (qmax - z) for s, z in zip(scales, zeros)]),
    }


def operators_to_dict(config, params) -> Dict[str, Dict[str, Any]]:
    """One record per operator; the per-tensor operators first, the per-channel ones last
    (quant_gru.py:4172-4214)."""
    scalars: Dict[str, Dict[str, Any]] = {}
    vectors: Dict[str, Dict[str, Any]] = {}
    for name in _STEMS:
        record = _operator_record(config, params, name)
        if record is None:
            continue
        (vectors if record["enc_type"] in ("PER_CHANNEL", "PER_GATE") else scalars)[name] = record
    scalars.update(vectors)
    return scalars


def _record_scales(name: str, record: Dict[str, Any]) -> List[float]:
    """Scales of a record: ``scale`` first, then the older multiplier/shift pair, then a bare
    power-of-two exponent (quant_gru.py:4231-4267)."""
    if "scale" in record:
        scales = _as_floats(record["scale"]) if isinstance(record["scale"], list) else [float(record["scale"])]
        if not scales:
            raise ValueError(f"operator '{name}': scale is empty")
        if any(v <= 0 for v in scales):
            raise ValueError(f"operator '{name}': every scale must be > 0")
        return scales
    if "multiplier" in record and "shift" in record:
        multipliers, shifts = record["multiplier"], record["shift"]
        multipliers = multipliers if isinstance(multipliers, list) else [multipliers]
        shifts = shifts if isinstance(shifts, list) else [shifts]
        if len(multipliers) != len(shifts):
            raise ValueError(f"operator '{name}': multiplier and shift differ in length")
        return [decode_multiplier_shift(int(m), int(s)) for m, s in zip(multipliers, shifts)]
    if "n" in record or "exp2_inv" in record or "shift" in record:
        exponents = record.get("n", record.get("exp2_inv", record.get("shift")))
        exponents = exponents if isinstance(exponents, list) else [exponents]
        return [math.ldexp(1.0, -int(e)) for e in exponents]
    raise ValueError(f"operator '{name}': no scale, multiplier/shift or exponent field")


def _apply_record(config, params, name: str, record: Dict[str, Any]) -> None:
    stem = _STEMS[name]
    if "dtype" in record:
        digits = re.search(r"(\d+)", record["dtype"])
        setattr(config, stem, int(digits.group(1)) if digits else 8)
        setattr(config, stem + "unsigned_", record["dtype"].upper().startswith("UINT"))
    if "symmetric" in record:
        setattr(config, stem + "symmetric_", record["symmetric"])
    if name in _WEIGHT_OPS:
        enc_type = record.get("enc_type") or "PER_CHANNEL"
        scales = _record_scales(name, record)
        if enc_type == "PER_TENSOR":
            # the binding keeps per-channel lists only; the reference fails the same way (quant_gru.py:4297-4304)
            setattr(config, stem + "granularity_", 0)
            if not hasattr(params, f"scale_{stem}tensor_"):
                raise AttributeError(f"GRUQuantParams has no attribute 'scale_{stem}tensor_'")
            setattr(params, f"scale_{stem}tensor_", float(scales[0]))
        elif enc_type == "PER_GATE":
            setattr(config, stem + "granularity_", 1)
            if len(scales) != 3:
                raise ValueError(f"operator '{name}': PER_GATE needs 3 scales, got {len(scales)}")
            if not hasattr(params, f"scale_{stem}gate_"):
                raise AttributeError(f"GRUQuantParams has no attribute 'scale_{stem}gate_'")
            setattr(params, f"scale_{stem}gate_", [float(v) for v in scales])
        else:
            setattr(config, stem + "granularity_", 2)
            setattr(params, "scale_" + stem, [float(v) for v in scales])
        return
    if not hasattr(params, "scale_" + stem):
        raise AttributeError(f"'gru_interface_binding.GRUQuantParams' object has no attribute 'scale_{stem}'")
    scales = _record_scales(stem.rstrip("_"), record)
    setattr(params, "scale_" + stem, float(scales[0]))
    if "zero_point" in record:
        zero = record["zero_point"]
        if isinstance(zero, list):
            if not zero:
                raise ValueError("zero_point list is empty")
            zero = zero[0]
        setattr(params, "zp_" + stem, int(zero))


def operators_from_dict(operators: Dict[str, Dict[str, Any]], config, params) -> None:
    """Writes every known record into the configuration and the parameter set; unknown names are skipped
    (quant_gru.py:4353-4432)."""
    for name, record in operators.items():
        if name in _STEMS:
            _apply_record(config, params, name, record)


# ---------------------------------------------------------------------------------------------
# grids at the module boundary (integer-in / integer-out chaining of stacked layers)
# ---------------------------------------------------------------------------------------------

def io_quant_meta(config, params, use_pot2_scale: Optional[bool] = None) -> Dict[str, Dict[str, Any]]:
    """Grids of the input, the output sequence and the hidden state of a module, with the scale the integer
    kernels really use (after the power-of-two or 16-bit multiplier encoding), so that codes handed from one
    layer to the next mean the same on both sides (``QuantGRU.get_io_quant_meta``, quant_gru.py:2378-2425)."""
    if params is None:
        raise RuntimeError("QuantGRU not calibrated")
    pot2 = bool(getattr(config, "usePOT2_", False)) if use_pot2_scale is None else bool(use_pot2_scale)

    def entry(stem: str) -> Dict[str, Any]:
        symmetric = bool(getattr(config, stem + "symmetric_"))
        unsigned = bool(getattr(config, stem + "unsigned_", False))
        return {
            "scale": float(gru_ops.decode_effective_scale(float(getattr(params, "scale_" + stem)), pot2)),
            "zp": int(getattr(params, "zp_" + stem)),
            "bitwidth": int(getattr(config, stem)),
            "is_symmetric": symmetric and not unsigned,
            "is_unsigned": unsigned,
        }

    return {"input": entry("x_"), "output": entry("h_"), "hidden": entry("h_")}


def grids_match(producer: Dict[str, Any], consumer: Dict[str, Any]) -> bool:
    """True when codes on `producer`'s grid (a layer's "output") can be fed to `consumer`'s (the next layer's
    "input") as they are: same effective scale, zero point, width and signedness."""
    return all(producer[key] == consumer[key] for key in ("scale", "zp", "bitwidth", "is_unsigned"))


# ---------------------------------------------------------------------------------------------
# operator JSON
# ---------------------------------------------------------------------------------------------

def quant_params_document(*, input_size: int, hidden_size: int, bias: bool = True, batch_first: bool = False,
                          bidirectional: bool = False, config, params, params_reverse=None,
                          quantized_weights: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
    """The document ``export_quant_params`` writes (quant_gru.py:4493-4515).  `quantized_weights`, when
    given, holds the integer codes the quantized forward returned (W_q, R_q, bw_q, br_q) as nested lists."""
    if params is None:
        raise RuntimeError("calibrate first: there are no quantization parameters to export")
    document: Dict[str, Any] = {
        "model_info": {
            "input_size": input_size,
            "hidden_size": hidden_size,
            "bias": bias,
            "batch_first": batch_first,
            "bidirectional": bidirectional,
            "use_pot2_scale": bool(getattr(config, "usePOT2_", False)),
        },
        "operators": operators_to_dict(config, params),
    }
    if bidirectional and params_reverse is not None:
        document["operators_reverse"] = operators_to_dict(config, params_reverse)
    if quantized_weights is not None:
        document["quantized_weights"] = quantized_weights
    return document


def export_quant_params(export_path: str, **fields) -> None:
    """Writes `quant_params_document(**fields)` the way the reference does: UTF-8, two-space indent."""
    with open(export_path, "w", encoding="utf-8") as out:
        json.dump(quant_params_document(**fields), out, indent=2, ensure_ascii=False)


def weight_codes_for_export(W_q, R_q, bw_q=None, br_q=None) -> Dict[str, Any]:
    """``quantized_weights`` of the document from the code tensors of a quantized forward
    (layout of quant_gru.py:4529-4578: W [I][3H], R [H][3H], biases [3H])."""
    weights = {"W": W_q.cpu().int().tolist(), "R": R_q.cpu().int().tolist()}
    if bw_q is not None and br_q is not None:
        weights["bw"] = bw_q.cpu().int().reshape(-1).tolist()
        weights["br"] = br_q.cpu().int().reshape(-1).tolist()
    return weights


def _new_direction(hidden_size: int):
    params = gru_ops.GRUQuantParams()
    params.hidden_ = hidden_size
    return params


def quant_params_from_document(document: Dict[str, Any], *, input_size: int, hidden_size: int,
                               bidirectional: bool = False) -> LoadedQuantParams:
    """Checks the document against the module it is loaded into and rebuilds the binding objects
    (quant_gru.py:4590-4655).  Raises ValueError on a mismatch, like the reference."""
    info = document.get("model_info", {})
    if info.get("input_size") != input_size:
        raise ValueError(f"input_size mismatch: file has {info.get('input_size')}, module has {input_size}")
    if info.get("hidden_size") != hidden_size:
        raise ValueError(f"hidden_size mismatch: file has {info.get('hidden_size')}, module has {hidden_size}")
    if info.get("bidirectional", False) != bidirectional:
        raise ValueError(f"bidirectional mismatch: file has {info.get('bidirectional')}, module has {bidirectional}")
    if "operators" not in document:
        raise ValueError(f"unsupported format: no 'operators' field (fields: {list(document.keys())})")

    config = gru_ops.OperatorQuantConfig()
    use_pot2 = bool(info.get("use_pot2_scale", False))
    config.usePOT2_ = use_pot2
    params = _new_direction(hidden_size)
    operators_from_dict(document["operators"], config, params)
    params.bitwidth_config_ = config

    reverse = None
    if bidirectional:
        if "operators_reverse" not in document:
            raise ValueError("bidirectional=True needs operators_reverse in the file")
        reverse = _new_direction(hidden_size)
        operators_from_dict(document["operators_reverse"], config, reverse)
        reverse.bitwidth_config_ = config
        # both directions read the same input tensor
        forward_input = document["operators"].get("input", {})
        reverse_input = document["operators_reverse"].get("input", {})
        for field in ("multiplier", "shift", "zero_point"):
            if (field in forward_input or field in reverse_input) and forward_input.get(field) != reverse_input.get(field):
                raise ValueError(f"operators.input and operators_reverse.input differ in {field}")
    return LoadedQuantParams(config, params, reverse, use_pot2, info)


def load_quant_params(import_path: str, **expect) -> LoadedQuantParams:
    with open(import_path, "r", encoding="utf-8") as src:
        return quant_params_from_document(json.load(src), **expect)


# ---------------------------------------------------------------------------------------------
# AIMET encodings
# ---------------------------------------------------------------------------------------------

def _zero_points_like_scales(record: Dict[str, Any]) -> Dict[str, Any]:
    """A list of scales wants a list of zero points of the same length (quant_gru.py:2593-2626).
    Works in place, like the reference."""
    if isinstance(record, dict) and isinstance(record.get("scale"), list):
        scales = record["scale"]
        zero = record.get("zero_point", 0)
        if not isinstance(zero, list):
            record["zero_point"] = [zero] * len(scales)
        elif len(zero) == 1:
            record["zero_point"] = zero * len(scales)
        elif len(zero) == 0:
            record["zero_point"] = [0] * len(scales)
        elif len(zero) != len(scales):
            raise ValueError(f"zero_point has {len(zero)} entries for {len(scales)} scales")
    return record


def _as_encoding(record: Any) -> Any:
    """Operator record -> AIMET encoding: adds bitwidth, turns `symmetric` into the string `is_symmetric`,
    drops execution fields and derives `n` from the scale (quant_gru.py:2628-2671)."""
    if not isinstance(record, dict):
        return record
    encoding = copy.deepcopy(record)
    if "dtype" in encoding:
        match = re.fullmatch(r"U?INT([1-9][0-9]*)", encoding["dtype"])
        if match:
            encoding["bitwidth"] = int(match.group(1))
    if "symmetric" in encoding:
        encoding["is_symmetric"] = "True" if encoding.pop("symmetric") else "False"
    if isinstance(encoding.get("is_symmetric"), bool):
        encoding["is_symmetric"] = "True" if encoding["is_symmetric"] else "False"
    for stale in ("multiplier", "shift", "scale_encoding", "n", "exp2_inv"):
        encoding.pop(stale, None)
    if "scale" in encoding:
        encoding["n"] = encoding_exponent(encoding["scale"])
    return encoding


def _append_fields(first: Optional[Dict[str, Any]], second: Optional[Dict[str, Any]]) -> Optional[Dict[str, Any]]:
    """Appends the list fields of `second` to those of `first` (forward before reverse, bias_ih before
    bias_hh); every other field keeps the value of `first` (quant_gru.py:2698-2733)."""
    if first is None:
        return copy.deepcopy(second)
    if second is None:
        return first
    for field in _LIST_FIELDS:
        if field not in second:
            continue
        if field not in first:
            first[field] = copy.deepcopy(second[field])
            continue
        a, b = first[field], second[field]
        if isinstance(a, list):
            a.extend(b) if isinstance(b, list) else a.append(b)
        else:
            first[field] = [a] + b if isinstance(b, list) else [a, b]
    return first


def _internal_ops_skeleton() -> Dict[str, Dict[str, list]]:
    # key order of a fresh module entry (quant_gru.py:2783-2797)
    names = ("add_final_hidden", "mul_new_contribution", "mul_old_contribution", "mul_reset_hidden", "new_gate_input",
             "new_gate_output", "reset_gate_input", "reset_gate_output", "sub_one_minus_update", "update_gate_input",
             "update_gate_output", "weight_ih_linear", "weight_hh_linear")
    return {name: {"output": []} for name in names}


def _fill_internal_ops(slots: Dict[str, Any], operators: Dict[str, Dict[str, Any]]) -> None:
    sources = [(name, name) for name in _INTERNAL_OPS] + list(_ALIASED_INTERNAL_OPS)
    for slot, source in sources:
        if source not in operators or (slot != source and slot not in slots):
            continue
        encoding = _as_encoding(_zero_points_like_scales(operators[source]))
        if "output" in slots[slot]:
            slots[slot]["output"] = [encoding]
        else:
            slots[slot] = encoding


def to_aimet_encodings(encodings: Dict[str, Any], module_name: str, *, config, params, params_reverse=None,
                       bidirectional: bool = False) -> Dict[str, Any]:
    """Merges one QuantGRU module into an AIMET encodings dictionary (schema 3) and returns it
    (quant_gru.py:2674-3162).  Activations go under activation_encodings[module_name] (input, output,
    internal_ops and, for a bidirectional module, internal_ops_reverse); weights under param_encodings as
    `<module>.weight_ih.weight`, `<module>.weight_hh.weight` and one merged `<module>.bias` whose lists run
    bias_ih, bias_hh, then the same of the reverse direction."""
    if params is None:
        return encodings
    module_name = module_name or "gru"
    operators = operators_to_dict(config, params)
    if not operators:
        return encodings
    reverse = operators_to_dict(config, params_reverse) if bidirectional and params_reverse is not None else None

    encodings.setdefault("schema_version", 3)
    activations = encodings.setdefault("activation_encodings", {})
    if module_name not in activations:
        activations[module_name] = {"is_GRU": True, "input": {}, "output": {}, "internal_ops": _internal_ops_skeleton()}
    entry = activations[module_name]
    if bidirectional and "internal_ops_reverse" not in entry:
        entry["internal_ops_reverse"] = _internal_ops_skeleton()
    parameters = encodings.setdefault("param_encodings", {})

    for side in ("input", "output"):
        if side in operators:
            encoding = _as_encoding(_zero_points_like_scales(operators[side]))
            entry[side] = {"0": encoding} if isinstance(encoding, dict) else encoding

    for name in ("weight_ih", "weight_hh"):
        if name not in operators:
            continue
        record = _zero_points_like_scales(operators[name])
        if reverse is not None and name in reverse:
            record = _append_fields(record, _zero_points_like_scales(reverse[name]))
        parameters[f"{module_name}.{name}.weight"] = _as_encoding(record)

    for name in ("bias_ih", "bias_hh"):
        if name not in operators:
            raise ValueError(f"module {module_name}: no '{name}' (the merged bias needs bias_ih and bias_hh)")
    merged = copy.deepcopy(_zero_points_like_scales(operators["bias_ih"]))
    second = _zero_points_like_scales(operators["bias_hh"])
    merged = _append_fields(merged, {f: second[f] for f in _LIST_FIELDS if f in second and f in merged})
    if reverse is not None and "bias_ih" in reverse and "bias_hh" in reverse:
        merged = _append_fields(merged, _zero_points_like_scales(reverse["bias_ih"]))
        merged = _append_fields(merged, _zero_points_like_scales(reverse["bias_hh"]))
    parameters[f"{module_name}.bias"] = _as_encoding(merged)

    _fill_internal_ops(entry["internal_ops"], operators)
    if bidirectional and reverse is not None and "internal_ops_reverse" in entry:
        _fill_internal_ops(entry["internal_ops_reverse"], reverse)
    # the reference builds tensor_encodings on the way and removes the key before it returns
    encodings.pop("tensor_encodings", None)
    return encodings


def _first_encoding(slot: Any) -> Optional[Dict[str, Any]]:
    """An activation slot holds its encoding as {"0": e}, [e] or e itself."""
    if isinstance(slot, dict) and "0" in slot:
        return slot["0"]
    if isinstance(slot, list) and slot:
        return slot[0]
    if isinstance(slot, dict):
        return slot
    return None


def _internal_encoding(slot: Any) -> Optional[Dict[str, Any]]:
    if isinstance(slot, dict) and "output" in slot:
        inner = slot["output"]
        if isinstance(inner, list) and inner:
            return inner[0]
        return inner if isinstance(inner, dict) else None
    return slot if isinstance(slot, dict) else None


def _slices(record: Dict[str, Any], fields: Tuple[str, ...], bounds: List[Tuple[int, int]]) -> List[Dict[str, Any]]:
    """Copies of `record`, one per (begin, end) pair, whose list fields hold that slice."""
    pieces = [copy.deepcopy(record) for _ in bounds]
    for field in fields:
        if isinstance(record.get(field), list):
            for piece, (begin, end) in zip(pieces, bounds):
                piece[field] = record[field][begin:end]
    return pieces


def from_aimet_encodings(encodings: Dict[str, Any], module_name: str, *, hidden_size: int,
                         bidirectional: bool = False) -> Optional[LoadedQuantParams]:
    """Reads one QuantGRU module back out of an AIMET encodings dictionary (quant_gru.py:3165-3590).
    Returns None where the reference returns False: the module, its input / output or one of its three
    parameter entries is missing, the merged bias does not split evenly, or a record does not parse.
    A stored `n` that contradicts its scale raises ValueError, as there."""
    module_name = module_name or "gru"
    entry = encodings.get("activation_encodings", {}).get(module_name) if "activation_encodings" in encodings else None
    if entry is None:
        return None
    validate_encoding_exponents(entry)
    for suffix in ("weight_ih.weight", "weight_hh.weight", "bias"):
        validate_encoding_exponents(encodings.get("param_encodings", {}).get(f"{module_name}.{suffix}"))

    operators: Dict[str, Any] = {}
    reverse: Optional[Dict[str, Any]] = {} if bidirectional else None
    for side in ("input", "output"):
        if side not in entry:
            return None
        found = _first_encoding(entry[side])
        if found is not None:
            operators[side] = found
    if bidirectional and "input" in operators:
        reverse["input"] = copy.deepcopy(operators["input"])

    if "param_encodings" in encodings:
        parameters = encodings["param_encodings"]
        weight_fields = ("scale", "multiplier", "shift", "real_min", "real_max", "zero_point")
        for name in ("weight_ih", "weight_hh"):
            key = f"{module_name}.{name}.weight"
            if key not in parameters:
                return None
            record = parameters[key]
            if bidirectional and isinstance(record, dict):
                # every list is cut at its own midpoint: forward half, reverse half
                forward, backward = copy.deepcopy(record), copy.deepcopy(record)
                for field in weight_fields:
                    if isinstance(record.get(field), list):
                        mid = len(record[field]) // 2
                        forward[field], backward[field] = record[field][:mid], record[field][mid:]
                operators[name], reverse[name] = forward, backward
            else:
                operators[name] = record
        key = f"{module_name}.bias"
        if key not in parameters:
            return None
        merged = parameters[key]
        length = next((len(merged[f]) for f in _LIST_FIELDS if isinstance(merged.get(f), list)), None)
        if not bidirectional:
            if length is None:
                operators["bias_ih"], operators["bias_hh"] = copy.deepcopy(merged), copy.deepcopy(merged)
            else:
                half = length // 2
                operators["bias_ih"], operators["bias_hh"] = _slices(
                    merged, _LIST_FIELDS, [(0, half), (half, None)])
        else:
            per_direction = None if length is None else length // 2
            if per_direction is None or per_direction % 2 != 0:
                return None
            quarter = per_direction // 2
            pieces = _slices(merged, _LIST_FIELDS, [(0, quarter), (quarter, per_direction),
                                                    (per_direction, per_direction + quarter),
                                                    (per_direction + quarter, 2 * per_direction)])
            for piece in pieces:
                for field in _LIST_FIELDS:
                    if not isinstance(merged.get(field), list):
                        piece[field] = merged.get(field)
            operators["bias_ih"], operators["bias_hh"], reverse["bias_ih"], reverse["bias_hh"] = pieces

    for slots, target in ((entry.get("internal_ops"), operators),
                          (entry.get("internal_ops_reverse") if bidirectional else None, reverse)):
        if slots is None or target is None:
            continue
        for name in _INTERNAL_OPS:
            if name in slots:
                found = _internal_encoding(slots[name])
                if found is not None:
                    target[name] = found
    if bidirectional and "internal_ops_reverse" in entry and "add_final_hidden" in entry["internal_ops_reverse"]:
        found = _internal_encoding(entry["internal_ops_reverse"]["add_final_hidden"])
        if found is not None:
            reverse["output"] = found

    # only the forward records get `symmetric` back; both directions share one configuration
    for record in operators.values():
        if isinstance(record, dict) and isinstance(record.get("is_symmetric"), (str, bool)):
            flag = record.pop("is_symmetric")
            record["symmetric"] = flag.lower() == "true" if isinstance(flag, str) else flag

    try:
        scales: List[Any] = []
        for direction in (operators, reverse):
            for record in (direction or {}).values():
                scale = record.get("scale", [])
                scales.extend(scale if isinstance(scale, list) else [scale])
        # power-of-two mode is recognised by the scales themselves: every mantissa is exactly one half
        use_pot2 = bool(scales) and all(isinstance(s, (int, float)) and s > 0 and math.isfinite(s)
                                        and math.frexp(s)[0] == 0.5 for s in scales)
        config = gru_ops.OperatorQuantConfig()
        config.usePOT2_ = use_pot2
        params = _new_direction(hidden_size)
        operators_from_dict(operators, config, params)
        params.bitwidth_config_ = config
        params_reverse = None
        if bidirectional and reverse:
            params_reverse = _new_direction(hidden_size)
            operators_from_dict(reverse, config, params_reverse)
            params_reverse.bitwidth_config_ = config
        return LoadedQuantParams(config, params, params_reverse, use_pot2, {})
    except Exception:
        return None
