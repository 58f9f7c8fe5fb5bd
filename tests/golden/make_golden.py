"""Generates the golden fixtures in this folder from the reference's own CPU build.

Run where the reference checkout is available:

    make -f oracle/Makefile ref && python tests/golden/make_golden.py

Each ``gru_*.npz`` holds one seeded QuantGRU problem (weights, inputs), the
ranges the reference's calibration forward observed, the encodings and the three
activation tables it derived and the integer codes / dequantized outputs of its
quantized CPU forward.  The files are small on purpose; tests replay them
against the C restatement and against the CUDA library.
"""
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
sys.path.insert(0, str(HERE.parent))

import oracle_lib as ol  # noqa: E402

CASES = {
    # name: (seed, T, B, I, H, bits, symmetric activations, pot2, granularity, h0, x_scale)
    "gru_w8a8_affine": (11, 6, 3, 5, 8, 8, False, False, 2, False, 1.0),
    "gru_w8a8_pot2_h0": (12, 5, 2, 7, 12, 8, True, True, 2, True, 1.0),
    "gru_a16_per_tensor": (13, 4, 2, 6, 10, 16, False, False, 0, True, 0.5),
    "gru_w4_per_gate": (14, 5, 3, 4, 6, 4, False, False, 1, False, 1.0),
    "gru_odd_shapes": (15, 7, 3, 31, 33, 8, False, False, 2, True, 2.0),
}


def main():
    assert ol.ref() is not None, "build oracle/_ref first (make -f oracle/Makefile ref)"
    for name, (seed, T, B, I, H, bits, sym, pot, gran, with_h0, xs) in CASES.items():
        W, R, bw, br, x, h0 = ol.gru_problem(seed, T, B, I, H, x_scale=xs, with_h0=with_h0)
        cfg = ol.make_config(bits=bits, symmetric=sym, use_pot2=pot, granularity=gran)
        ranges = ol.RangesBox(H)
        h_fp, v_fp = ol.forward_calibrate_minmax("ref", W, R, bw, br, x, h0, ranges, cfg)
        params = ol.params_from_ranges("ref", ranges, cfg)
        luts = ol.build_luts("ref", params)
        fwd = ol.forward_quant("ref", W, R, bw, br, x, h0, params)
        out = {"meta": np.array([seed, T, B, I, H, bits, int(sym), int(pot), gran, int(with_h0)], np.int64),
               "W": W, "R": R, "bw": bw, "br": br, "x": x, "h_fp": h_fp, "v_fp": v_fp, "luts": luts}
        if h0 is not None:
            out["h0"] = h0
        out.update({f"range_{k}": v for k, v in ranges.as_dict().items()})
        out.update({f"param_{k}": v for k, v in params.as_dict().items()})
        out.update({f"fwd_{k}": v for k, v in fwd.items()})
        np.savez_compressed(HERE / f"{name}.npz", **out)
        print(name, "written")


if __name__ == "__main__":
    main()
