"""Loader and numpy wrappers for the parity checkers (test infrastructure).

``oracle/librxmet_oracle.so``  - plain-C restatement of the path (always built)
``oracle/_ref/libgru_ref.so``  - the reference's own CPU sources (present only
                                  where the reference checkout was available
                                  when it was built)
Both export the same entry points with the prefixes ``orc_`` and ``ref_``.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

from rx_met_b200 import _cabi as cabi

ROOT = Path(__file__).resolve().parent.parent
ORACLE_SO = ROOT / "oracle" / "librxmet_oracle.so"
REF_SO = ROOT / "oracle" / "_ref" / "libgru_ref.so"

_f32p = C.POINTER(C.c_float)
_i32p = C.POINTER(C.c_int32)


def _fp(a):
    return None if a is None else a.ctypes.data_as(_f32p)


def _ip(a):
    return None if a is None else a.ctypes.data_as(_i32p)


def build_oracle():
    subprocess.run(["make", "-s", "-f", str(ROOT / "oracle" / "Makefile"), "oracle"], check=True)


_oracle = None
_ref = None


def oracle() -> C.CDLL:
    global _oracle
    if _oracle is None:
        if not ORACLE_SO.exists():
            build_oracle()
        _oracle = C.CDLL(str(ORACLE_SO))
    return _oracle


def ref():
    """The compiled reference, or None when it is not available."""
    global _ref
    if _ref is None and REF_SO.exists():
        _ref = C.CDLL(str(REF_SO))
        _ref.ref_last_error.restype = C.c_char_p
        _ref.ref_rshift_round_i64.restype = C.c_int64
        _ref.ref_rshift_round_i64.argtypes = [C.c_int64, C.c_int]
        _ref.ref_quantize.restype = C.c_int32
        _ref.ref_quantize.argtypes = [C.c_float, C.c_float, C.c_int32, C.c_int, C.c_int]
    return _ref


# --------------------------------------------------------------------------
# struct builders that keep their numpy storage alive
# --------------------------------------------------------------------------

def make_config(bits=8, symmetric=True, use_pot2=False, granularity=cabi.PER_CHANNEL,
                pot_method=cabi.POT_COVER_RANGE, overrides=None) -> cabi.QuantConfig:
    """Reference defaults (all `bits` wide, gate outputs z/r unsigned); activations get
    ``symmetric``; W/R/bw/br stay symmetric as the reference requires."""
    cfg = cabi.QuantConfig()
    for i in range(cabi.NUM_OPS):
        cfg.bits[i] = bits
        cfg.is_unsigned[i] = 1 if i in (cabi.UPDATE_GATE_OUTPUT, cabi.RESET_GATE_OUTPUT) else 0
        cfg.symmetric[i] = 1 if (symmetric or i in (cabi.W, cabi.R, cabi.BW, cabi.BR)) else 0
    cfg.W_granularity = cfg.R_granularity = cfg.bw_granularity = cfg.br_granularity = granularity
    cfg.use_pot2 = 1 if use_pot2 else 0
    cfg.pot_scale_method = pot_method
    cfg.pot_scale_tolerance = 0.02
    for name, (b, uns, sym) in (overrides or {}).items():
        i = cabi.OP_NAMES.index(name)
        cfg.bits[i], cfg.is_unsigned[i], cfg.symmetric[i] = b, int(uns), int(sym)
    return cfg


class RangesBox:
    """rxmet_gru_ranges plus the arrays its pointers refer to."""

    def __init__(self, hidden: int):
        self.hidden = hidden
        self.chan = {k: np.empty(3 * hidden, np.float32) for k in
                     ("min_W", "max_W", "min_R", "max_R", "min_bw", "max_bw", "min_br", "max_br")}
        self.c = cabi.Ranges()
        self.c.hidden = hidden
        for k, a in self.chan.items():
            setattr(self.c, k, _fp(a))
        self.reset()

    def reset(self):
        fmax = np.finfo(np.float32).max
        for i in range(cabi.NUM_OPS):
            self.c.min[i] = fmax
            self.c.max[i] = -fmax
        for k, a in self.chan.items():
            a[:] = fmax if k.startswith("min") else -fmax

    def scalars(self):
        return (np.array(list(self.c.min), np.float32), np.array(list(self.c.max), np.float32))

    def as_dict(self):
        mn, mx = self.scalars()
        d = {"min": mn, "max": mx}
        d.update({k: v.copy() for k, v in self.chan.items()})
        return d

    @classmethod
    def from_dict(cls, d):
        box = cls(len(d["min_W"]) // 3)
        for i in range(cabi.NUM_OPS):
            box.c.min[i] = float(d["min"][i])
            box.c.max[i] = float(d["max"][i])
        for k in box.chan:
            box.chan[k][:] = d[k]
        return box


class ParamsBox:
    """rxmet_gru_quant_params plus the four per-channel scale arrays."""

    def __init__(self, hidden: int, cfg: cabi.QuantConfig | None = None):
        self.hidden = hidden
        self.chan = {k: np.zeros(3 * hidden, np.float32) for k in
                     ("scale_W", "scale_R", "scale_bw", "scale_br")}
        self.c = cabi.QuantParams()
        self.c.hidden = hidden
        for k, a in self.chan.items():
            setattr(self.c, k, _fp(a))
        if cfg is not None:
            self.c.config = cfg

    def as_dict(self):
        d = {"scale": np.array(list(self.c.scale), np.float32),
             "zero_point": np.array(list(self.c.zero_point), np.int32)}
        d.update({k: v.copy() for k, v in self.chan.items()})
        return d

    def load_dict(self, d):
        for i in range(cabi.NUM_OPS):
            self.c.scale[i] = float(d["scale"][i])
            self.c.zero_point[i] = int(d["zero_point"][i])
        for k in self.chan:
            self.chan[k][:] = d[k]
        return self


class MasksBox:
    """Host uint8 mask arrays with the rxmet_gru_masks struct pointing at them."""

    def __init__(self, T, B, I, H, with_h0=True):
        shapes = {"x": (T, B, I), "h0": (B, H), "W": (I, 3 * H), "R": (H, 3 * H), "bw": (3 * H,),
                  "br": (3 * H,), "weight_ih_linear": (T, B, 3 * H), "weight_hh_linear": (T, B, 3 * H),
                  "gate_input": (T, B, 3 * H), "gate_output": (T, B, 3 * H), "h": (T, B, H)}
        self.arr = {k: np.full(s, 255, np.uint8) for k, s in shapes.items()}
        if not with_h0:
            del self.arr["h0"]
        self.c = cabi.Masks()
        for k, a in self.arr.items():
            setattr(self.c, k, a.ctypes.data)


# --------------------------------------------------------------------------
# calls (prefix "orc" = restatement, "ref" = compiled reference)
# --------------------------------------------------------------------------

def _lib(prefix):
    lib = oracle() if prefix == "orc" else ref()
    if lib is None:
        raise RuntimeError("compiled reference not available")
    return lib


def params_from_ranges(prefix, ranges: RangesBox, cfg) -> ParamsBox:
    out = ParamsBox(ranges.hidden, cfg)
    rc = getattr(_lib(prefix), f"{prefix}_gru_params_from_ranges")(C.byref(ranges.c), C.byref(cfg), C.byref(out.c))
    if rc != 0:
        raise ValueError(f"{prefix}_gru_params_from_ranges failed")
    return out


def build_luts(prefix, params: ParamsBox) -> np.ndarray:
    out = ((cabi.LutSegment * 16) * 3)()
    rc = getattr(_lib(prefix), f"{prefix}_gru_build_luts")(C.byref(params.c), out)
    assert rc == 0
    return np.array([[(s.q_b, s.n_bx_total, s.term_c, s.threshold) for s in row] for row in out], np.int64)


def forward_calibrate_minmax(prefix, W, R, bw, br, x, h0, ranges: RangesBox, cfg=None):
    T, B, I = x.shape
    H = R.shape[0]
    h = np.empty((T + 1, B, H), np.float32)
    v = np.empty((T, B, 4 * H), np.float32)
    lib = _lib(prefix)
    if prefix == "ref":
        rc = lib.ref_gru_forward_calibrate_minmax(T, B, I, H, _fp(W), _fp(R), _fp(bw), _fp(br), _fp(x), _fp(h0),
                                                  C.byref(cfg), C.byref(ranges.c), _fp(h), _fp(v))
    else:
        rc = lib.orc_gru_forward_calibrate_minmax(T, B, I, H, _fp(W), _fp(R), _fp(bw), _fp(br), _fp(x), _fp(h0),
                                                  C.byref(ranges.c), _fp(h), _fp(v))
    assert rc == 0
    return h, v


def forward_quant(prefix, W, R, bw, br, x, h0, params: ParamsBox, training=True, want_float=True):
    """Returns a dict with h, v (float) and the codes; the restatement also returns masks.
    want_float=False skips the dequantized outputs (the compiled reference needs a second pass
    over the sequence to produce them)."""
    T, B, I = x.shape
    H = R.shape[0]
    out = {"h": np.empty((T + 1, B, H), np.float32), "v": np.empty((T, B, 4 * H), np.float32),
           "x_q": np.empty((T, B, I), np.int32), "h_q": np.empty((T + 1, B, H), np.int32),
           "v_q": np.empty((T, B, 4 * H), np.int32)}
    lib = _lib(prefix)
    if prefix == "ref":
        rc = lib.ref_gru_forward_quant(T, B, I, H, _fp(W), _fp(R), _fp(bw), _fp(br), _fp(x), _fp(h0),
                                       C.byref(params.c), _ip(out["x_q"]), _ip(out["h_q"]), _ip(out["v_q"]),
                                       _fp(out["h"]) if want_float else None, _fp(out["v"]) if want_float else None)
        assert rc == 0, lib.ref_last_error()
        if not want_float:
            return out
        wq = {k: np.empty(s, np.int32) for k, s in
              (("W_q", (I, 3 * H)), ("R_q", (H, 3 * H)), ("bw_q", (3 * H,)), ("br_q", (3 * H,)))}
        rc = lib.ref_gru_quantize_weights(I, H, _fp(W), _fp(R), _fp(bw), _fp(br), C.byref(params.c),
                                          _ip(wq["W_q"]), _ip(wq["R_q"]), _ip(wq["bw_q"]), _ip(wq["br_q"]))
        assert rc == 0
        out.update(wq)
        return out
    out.update({"W_q": np.empty((I, 3 * H), np.int32), "R_q": np.empty((H, 3 * H), np.int32),
                "bw_q": np.empty(3 * H, np.int32), "br_q": np.empty(3 * H, np.int32)})
    masks = MasksBox(T, B, I, H, with_h0=h0 is not None) if training else None
    rc = lib.orc_gru_forward_quant(int(training), T, B, I, H, _fp(W), _fp(R), _fp(bw), _fp(br), _fp(x), _fp(h0),
                                   C.byref(params.c), _fp(out["h"]), _fp(out["v"]),
                                   _ip(out["W_q"]), _ip(out["R_q"]), _ip(out["bw_q"]), _ip(out["br_q"]),
                                   _ip(out["x_q"]), _ip(out["h_q"]), _ip(out["v_q"]),
                                   C.byref(masks.c) if masks else None)
    assert rc == 0
    if masks:
        out["masks"] = masks
    return out


def forward_fp(W, R, bw, br, x, h0):
    T, B, I = x.shape
    H = R.shape[0]
    h = np.empty((T + 1, B, H), np.float32)
    v = np.empty((T, B, 4 * H), np.float32)
    rc = oracle().orc_gru_forward_fp(T, B, I, H, _fp(W), _fp(R), _fp(bw), _fp(br), _fp(x), _fp(h0), _fp(h), _fp(v))
    assert rc == 0
    return h, v


def backward_quant(codes, dh_new, h, v, params: ParamsBox, masks: MasksBox | None):
    T, B, I = codes["x_q"].shape
    H = codes["R_q"].shape[0]
    g = {"dx": np.empty((T, B, I), np.float32), "dW": np.empty((I, 3 * H), np.float32),
         "dR": np.empty((H, 3 * H), np.float32), "dbw": np.empty(3 * H, np.float32),
         "dbr": np.empty(3 * H, np.float32), "dh0": np.empty((B, H), np.float32)}
    rc = oracle().orc_gru_backward_quant(
        T, B, I, H, _ip(codes["W_q"]), _ip(codes["R_q"]), _ip(codes["bw_q"]), _ip(codes["br_q"]),
        _ip(codes["x_q"]), _fp(dh_new), _fp(h), _fp(v), C.byref(params.c),
        C.byref(masks.c) if masks else None,
        _fp(g["dx"]), _fp(g["dW"]), _fp(g["dR"]), _fp(g["dbw"]), _fp(g["dbr"]), _fp(g["dh0"]))
    assert rc == 0
    return g


def backward_fp(W, R, bw, br, x, dh_new, h, v):
    T, B, I = x.shape
    H = R.shape[0]
    g = {"dx": np.empty((T, B, I), np.float32), "dW": np.empty((I, 3 * H), np.float32),
         "dR": np.empty((H, 3 * H), np.float32), "dbw": np.empty(3 * H, np.float32),
         "dbr": np.empty(3 * H, np.float32), "dh0": np.empty((B, H), np.float32)}
    rc = oracle().orc_gru_backward_fp(T, B, I, H, _fp(W), _fp(R), _fp(bw), _fp(br), _fp(x), _fp(dh_new),
                                      _fp(h), _fp(v), _fp(g["dx"]), _fp(g["dW"]), _fp(g["dR"]),
                                      _fp(g["dbw"]), _fp(g["dbr"]), _fp(g["dh0"]))
    assert rc == 0
    return g


# --------------------------------------------------------------------------
# seeded synthetic problems shared by the tests and the fixture generator
# --------------------------------------------------------------------------

def gru_problem(seed, T, B, I, H, x_scale=1.0, with_h0=False):
    """Weights U(-1/sqrt(H), 1/sqrt(H)) like torch.nn.GRU, inputs N(0,1)*x_scale,
    already in the operator's layout (gate order z,r,n; W [I,3H], R [H,3H])."""
    rng = np.random.default_rng(seed)
    k = 1.0 / np.sqrt(H)
    W = rng.uniform(-k, k, (I, 3 * H)).astype(np.float32)
    R = rng.uniform(-k, k, (H, 3 * H)).astype(np.float32)
    bw = rng.uniform(-k, k, 3 * H).astype(np.float32)
    br = rng.uniform(-k, k, 3 * H).astype(np.float32)
    x = (rng.standard_normal((T, B, I)) * x_scale).astype(np.float32)
    h0 = (rng.standard_normal((B, H)) * 0.3).astype(np.float32) if with_h0 else None
    return W, R, bw, br, x, h0
