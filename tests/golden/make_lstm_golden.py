"""Converts the golden cases of the reference's QuantLSTM test suite
(operators/quant-lstm/tests/golden/spec) into ``tests/golden/lstm_golden.json``.

Run once where the reference checkout is present:
    python tests/golden/make_lstm_golden.py <path-to-reference-checkout>
Only numbers are carried over (tensor name -> dtype, shape, flat data); decimal strings of
float tensors are parsed to Python floats, which round-trip float32 exactly.
"""
import json
import sys
from pathlib import Path

CASES = ["recurrent/reference_recurrent_t3_b1_i2_h2_cpu_fp32", "cell/reference_cell_t1_b1_i2_h2_cpu_fp32",
         "primitive/real_activation_boundaries_cpu_fp32", "primitive/quant_dequant_boundaries",
         "primitive/dequantize_boundaries", "primitive/pot2_cover_range", "primitive/m_shift_known_vectors",
         "primitive/round_half_ties", "primitive/quantized_ranges"]


def tensor(t):
    data = t["data"]
    if t["dtype"].startswith("float"):
        data = [float(v) for v in data]
    return {"dtype": t["dtype"], "shape": t["shape"], "data": data}


def main(ref_root):
    spec = Path(ref_root) / "operators" / "quant-lstm" / "tests" / "golden" / "spec"
    out = {}
    for rel in CASES:
        case = json.loads((spec / (rel + ".json")).read_text())
        out[case["case_id"]] = {
            "kind": case["kind"], "primitive": case.get("primitive"), "attributes": case.get("attributes", {}),
            "inputs": {k: tensor(v) for k, v in case["inputs"].items()},
            "expected": {k: tensor(v) for k, v in case["expected"]["checkpoints"].items()},
            "diagnostics": {k: tensor(v) for k, v in case["expected"].get("diagnostics", {}).items()},
        }
    target = Path(__file__).resolve().parent / "lstm_golden.json"
    target.write_text(json.dumps(out, indent=None, separators=(",", ":")) + "\n")
    print(f"wrote {target} ({target.stat().st_size} bytes, {len(out)} cases)")


if __name__ == "__main__":
    main(sys.argv[1])
