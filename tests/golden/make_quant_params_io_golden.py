"""Writes tests/golden/quant_params_io.json from the reference's own Python code.

Run where the reference checkout is present:

    PYTHONPATH=. python tests/golden/make_quant_params_io_golden.py /path/to/reference

The reference's operators/quant-gru/pytorch/quant_gru.py is imported with this package's
`gru_interface_binding` standing in for its compiled binding (the module only stores attributes on the
binding objects on this path), a reference `QuantGRU` module is given seeded quantization parameters, and
its export_quant_params / load_quant_params / export_quant_params_to_aimet_format /
load_quant_params_from_aimet_format are run.  The fixture holds, per case, the inputs, both exported
documents and the attributes the reference's loaders produced from them.
"""
import json
import os
import random
import sys
import tempfile

import rx_met_b200.gru_interface_binding as mirror

SCALAR_OPS = ["x", "h", "weight_ih_linear", "weight_hh_linear", "update_gate_input", "update_gate_output",
              "reset_gate_input", "reset_gate_output", "new_gate_input", "new_gate_output", "mul_reset_hidden",
              "mul_old_contribution", "mul_new_contribution"]
WEIGHT_OPS = ["W", "R", "bw", "br"]


def config_attrs(cfg):
    return {k: getattr(cfg, k) for k in sorted(dir(cfg))
            if not k.startswith("_") and not callable(getattr(cfg, k))}


def params_attrs(p):
    out = {"hidden_": p.hidden_}
    for k in sorted(dir(p)):
        if k.startswith("scale_") or k.startswith("zp_"):
            v = getattr(p, k)
            out[k] = list(v) if hasattr(v, "__iter__") else v
    return out


def seeded_params(rng, hidden, pot2):
    p = mirror.GRUQuantParams()
    p.hidden_ = hidden

    def scale():
        return 2.0 ** -rng.randint(2, 12) if pot2 else rng.uniform(1e-4, 2e-1)

    for op in WEIGHT_OPS:
        setattr(p, f"scale_{op}_", [scale() for _ in range(3 * hidden)])
    for op in SCALAR_OPS:
        setattr(p, f"scale_{op}_", scale())
        setattr(p, f"zp_{op}_", rng.randint(-40, 40))
    return p


def seeded_config(rng, varied):
    cfg = mirror.OperatorQuantConfig()
    if varied:
        for op in SCALAR_OPS + WEIGHT_OPS:
            setattr(cfg, f"{op}_", rng.choice([4, 8, 12, 16]))
        for op in SCALAR_OPS:
            setattr(cfg, f"{op}_symmetric_", rng.random() < 0.5)
            setattr(cfg, f"{op}_unsigned_", rng.random() < 0.3)
    return cfg


def main(reference_root):
    sys.path.insert(0, os.path.join(reference_root, "operators", "quant-gru", "pytorch"))
    sys.modules["gru_interface_binding"] = mirror
    import quant_gru as ref

    cases = []
    specs = [("unidirectional_defaults", 5, 4, False, False, False),
             ("bidirectional_defaults", 6, 3, True, False, False),
             ("unidirectional_varied_grids", 7, 5, False, True, False),
             ("bidirectional_varied_grids", 4, 2, True, True, False),
             ("unidirectional_power_of_two", 3, 2, False, False, True)]
    for index, (name, input_size, hidden, bidirectional, varied, pot2) in enumerate(specs):
        rng = random.Random(1000 + index)
        module = ref.QuantGRU(input_size, hidden, bidirectional=bidirectional)
        cfg = seeded_config(rng, varied)
        cfg.usePOT2_ = pot2
        module._bitwidth_config = cfg
        module.use_pot2_scale = pot2
        module.quant_params = seeded_params(rng, hidden, pot2)
        module.quant_params_reverse = seeded_params(rng, hidden, pot2) if bidirectional else None
        if bidirectional:  # both directions read the same input tensor
            module.quant_params_reverse.scale_x_ = module.quant_params.scale_x_
            module.quant_params_reverse.zp_x_ = module.quant_params.zp_x_
        module._quant_params_dirty = False
        case = {"name": name, "input_size": input_size, "hidden_size": hidden, "bidirectional": bidirectional,
                "config": config_attrs(cfg), "params": params_attrs(module.quant_params),
                "params_reverse": params_attrs(module.quant_params_reverse) if bidirectional else None}

        case["io_quant_meta"] = module.get_io_quant_meta()
        with tempfile.TemporaryDirectory() as folder:
            path = os.path.join(folder, "params.json")
            module.export_quant_params(path)
            with open(path, encoding="utf-8") as src:
                case["document"] = json.load(src)
            loaded = ref.QuantGRU(input_size, hidden, bidirectional=bidirectional)
            loaded.load_quant_params(path)
        case["loaded_from_document"] = {
            "config": config_attrs(loaded._bitwidth_config), "params": params_attrs(loaded.quant_params),
            "params_reverse": params_attrs(loaded.quant_params_reverse) if bidirectional else None}

        encodings = module.export_quant_params_to_aimet_format({}, "encoder.gru")
        case["aimet"] = json.loads(json.dumps(encodings))
        loaded = ref.QuantGRU(input_size, hidden, bidirectional=bidirectional)
        ok = loaded.load_quant_params_from_aimet_format(json.loads(json.dumps(encodings)), "encoder.gru")
        assert ok is True, name
        case["loaded_from_aimet"] = {
            "config": config_attrs(loaded._bitwidth_config), "params": params_attrs(loaded.quant_params),
            "params_reverse": params_attrs(loaded.quant_params_reverse) if bidirectional else None}
        cases.append(case)

    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "quant_params_io.json")
    with open(out, "w", encoding="utf-8") as dst:
        json.dump({"source": "operators/quant-gru/pytorch/quant_gru.py (export/load functions of QuantGRU)",
                   "cases": cases}, dst, separators=(",", ":"))
    print("wrote", out, len(cases), "cases")


if __name__ == "__main__":
    main(sys.argv[1])
