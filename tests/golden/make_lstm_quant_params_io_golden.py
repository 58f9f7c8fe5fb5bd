"""Writes tests/golden/lstm_quant_params_io.json from the reference's own Python code.

Run where the reference checkout is present:

    PYTHONPATH=. python tests/golden/make_lstm_quant_params_io_golden.py /path/to/reference

operators/quant-lstm/pytorch/quant_lstm.py and lstm_aimet.py are imported with this package's
`_quant_lstm` standing in for the compiled extension (used here only to resolve configurations and to
audit bundles, both host-side).  A reference `QuantLSTM` is given seeded parameter bundles, and its
export_quant_params / load_quant_params / export_quant_params_to_aimet_format /
load_quant_params_from_aimet_format are run.  The fixture holds, per case, the bundles that went in, the
documents that came out and the bundles the reference's loaders ended up with.
"""
import json
import os
import random
import sys

import numpy as np

import rx_met_b200._quant_lstm as mirror
from rx_met_b200 import _cabi_lstm as L


def seeded_bundle(rng, resolved, input_size, hidden, bias, pot2):
    operators = {}
    for name, cfg in resolved["operators"].items():
        if not bias and name in ("bias_ih", "bias_hh"):
            continue
        count = 4 * hidden if name in ("weight_ih", "weight_hh", "bias_ih", "bias_hh") else 1

        def scale():
            value = 2.0 ** -rng.randint(2, 10) if pot2 else rng.uniform(1e-3, 1e-1)
            return mirror._shortest_float(np.float32(value))

        if cfg["granularity"] == "per_tensor" and count > 1:
            scales = [scale()] * count
        elif cfg["granularity"] == "per_gate" and count > 1:
            scales = [s for s in (scale() for _ in range(4)) for _ in range(hidden)]
        else:
            scales = [scale() for _ in range(count)]
        if cfg["is_symmetric"] or count > 1:
            zeros = [0] * count
        else:
            low = 0 if cfg["is_unsigned"] else -(1 << (cfg["bitwidth"] - 1))
            zeros = [rng.randint(low + 1, low + (1 << cfg["bitwidth"]) - 2)]
        operators[name] = dict(cfg, scales=scales, zero_points=zeros)
    return json.dumps({"schema_version": 1, "input_size": input_size, "hidden_size": hidden, "bias_enabled": bias,
                       "scale_mode": "pot2" if pot2 else "affine", "operators": operators}, separators=(",", ":"))


def main(reference_root):
    sys.path.insert(0, os.path.join(reference_root, "operators", "quant-lstm", "pytorch"))
    sys.modules["_quant_lstm"] = mirror
    import quant_lstm as ref

    specs = [("unidirectional_defaults", 3, 2, True, False, None, False),
             ("bidirectional_defaults", 4, 3, True, True, None, False),
             ("unidirectional_no_bias_power_of_two", 3, 2, False, False, None, True),
             ("bidirectional_varied_grids", 2, 2, True, True, {
                 "input": {"is_symmetric": False, "bitwidth": 16},
                 "output": {"is_symmetric": False, "is_unsigned": True},
                 "cell_state": {"bitwidth": 16},
                 "weight_ih": {"granularity": "per_tensor"},
                 "weight_hh": {"granularity": "per_gate", "bitwidth": 4},
                 "input_gate_input": {"is_symmetric": False, "bitwidth": 12}}, False)]
    cases = []
    for index, (name, input_size, hidden, bias, bidirectional, override, pot2) in enumerate(specs):
        rng = random.Random(2000 + index)
        config = {"schema_version": 1, "operators": override or {}}
        if pot2:
            config["scale_mode"] = "pot2"
        module = ref.QuantLSTM(input_size, hidden, bias=bias, bidirectional=bidirectional, quant_config=config)
        resolved = module.get_quant_config()
        bundles = []
        for _ in range(2 if bidirectional else 1):
            audited = mirror.audit_quant_params_bundle(seeded_bundle(rng, resolved, input_size, hidden, bias, pot2))
            bundles.append(audited["bundle_json"])
        if bidirectional:  # both directions read the same input tensor
            forward, reverse = json.loads(bundles[0]), json.loads(bundles[1])
            reverse["operators"]["input"] = forward["operators"]["input"]
            bundles[1] = mirror.audit_quant_params_bundle(json.dumps(reverse, separators=(",", ":")))["bundle_json"]
        module._quant_params_bundle_json = bundles[0]
        if bidirectional:
            module._reverse_quant_params_bundle_json = bundles[1]
        module._resolved_config_json = audited["resolved_config_json"]

        document = module.export_quant_params()
        encodings = module.export_quant_params_to_aimet_format({}, "encoder.lstm")
        case = {"name": name, "input_size": input_size, "hidden_size": hidden, "bias": bias,
                "bidirectional": bidirectional, "bundles": bundles, "document": json.loads(json.dumps(document)),
                "aimet": json.loads(json.dumps(encodings)),
                "activation_operators": sorted(set(resolved["operators"]) - {"weight_ih", "weight_hh", "bias_ih", "bias_hh"})}

        loaded = ref.QuantLSTM(input_size, hidden, bias=bias, bidirectional=bidirectional)
        loaded.load_quant_params(json.loads(json.dumps(document)))
        case["bundles_from_document"] = [loaded._quant_params_bundle_json] + (
            [loaded._reverse_quant_params_bundle_json] if bidirectional else [])
        loaded = ref.QuantLSTM(input_size, hidden, bias=bias, bidirectional=bidirectional)
        assert loaded.load_quant_params_from_aimet_format(json.loads(json.dumps(encodings)), "encoder.lstm") is True
        case["bundles_from_aimet"] = [loaded._quant_params_bundle_json] + (
            [loaded._reverse_quant_params_bundle_json] if bidirectional else [])
        cases.append(case)

    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lstm_quant_params_io.json")
    with open(out, "w", encoding="utf-8") as dst:
        json.dump({"source": "operators/quant-lstm/pytorch/quant_lstm.py and lstm_aimet.py (export/load of QuantLSTM)",
                   "cases": cases}, dst, separators=(",", ":"))
    print("wrote", out, len(cases), "cases")


if __name__ == "__main__":
    main(sys.argv[1])
