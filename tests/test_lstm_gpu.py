"""QuantLSTM on the GPU (through the drop-in module, i.e. through the C ABI) against the CPU checker."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import lstm_lib as ll
from rx_met_b200 import _cabi_lstm as L

pytestmark = pytest.mark.gpu


def mod():
    from rx_met_b200 import _quant_lstm
    return _quant_lstm


def dev(a):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda()


def state3(a):
    return None if a is None else dev(a).unsqueeze(0)


def close(got, want, tol=1e-5, name=""):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    scale = max(np.abs(want).max(), 1e-30)
    err = np.abs(got - want).max() / scale
    assert err <= tol, f"{name}: max error {err:.3e} of the largest magnitude"


def torch_args(p):
    return (dev(p["x"]), dev(p["w_ih"]), dev(p["w_hh"]), dev(p["b_ih"]), dev(p["b_hh"]), state3(p["h0"]), state3(p["c0"]))


SHAPES = [(5, 3, 6, 9, True, True), (7, 5, 40, 128, True, False), (4, 300, 12, 64, False, True), (3, 2, 1, 1, True, True)]


@pytest.mark.parametrize("T,B,I,H,bias,state", SHAPES)
def test_float_forward_and_backward(T, B, I, H, bias, state):
    p = ll.problem(T, B, I, H, seed=T + H, bias=bias, state=state)
    want = ll.forward_float("orc", p)
    m = mod()
    out = m.lstm_forward_training(*torch_args(p), False)
    names = ["output", "h_n", "c_n", "gate_outputs", "cell_states", "cell_tanh_outputs", "hidden_outputs"]
    refs = [want[0], want[1][None], want[2][None], want[3]["gate_outputs"], want[3]["cell_states"],
            want[3]["cell_tanh_outputs"], want[3]["hidden_outputs"]]
    for n, g, w in zip(names, out, refs):
        close(g.cpu().numpy(), w, 2e-5, n)
    plain = m.lstm_forward(*torch_args(p), False)
    assert torch.equal(plain[0], out[0]) and torch.equal(plain[1], out[1]) and torch.equal(plain[2], out[2])
    rng = np.random.default_rng(9)
    g = [rng.standard_normal(s).astype(np.float32) for s in [(T, B, H), (B, H), (B, H)]]
    tr = want[3]
    wg = ll.backward_float("orc", p, tr, *g)
    got = m.lstm_backward_float(*torch_args(p), False, dev(tr["gate_outputs"]), dev(tr["cell_states"]),
                                dev(tr["cell_tanh_outputs"]), dev(tr["hidden_outputs"]), dev(g[0]), dev(g[1]), dev(g[2]))
    for n, t in zip(L.MASTER_VALUES, got):
        close(t.cpu().numpy().reshape(wg[n].shape), wg[n], 2e-5, n)


def test_float_backward_with_masks_and_batch_first():
    T, B, I, H = 6, 4, 5, 8
    p = ll.problem(T, B, I, H, seed=21)
    out, hn, cn, tr = ll.forward_float("orc", p)
    rng = np.random.default_rng(2)
    g = [rng.standard_normal(s).astype(np.float32) for s in [(T, B, H), (B, H), (B, H)]]
    shapes = dict(input=(T, B, I), weight_ih=(4 * H, I), weight_hh=(4 * H, H), bias_ih=(4 * H,), bias_hh=(4 * H,),
                  initial_hidden=(B, H), initial_cell=(B, H))
    shapes.update({n: tr[n].shape for n in L.TRACE_VALUES})
    masks = {n: (rng.random(s) < 0.15).astype(np.uint8) for n, s in shapes.items()}
    want = ll.backward_float("orc", p, tr, *g, masks=masks)
    m = mod()
    master = [dev(masks["input"]).transpose(0, 1).contiguous().bool(), dev(masks["weight_ih"]), dev(masks["weight_hh"]),
              dev(masks["bias_ih"]), dev(masks["bias_hh"]), dev(masks["initial_hidden"])[None].bool(),
              dev(masks["initial_cell"])[None]]
    ckpt = [dev(masks[n]) for n in L.TRACE_VALUES]
    a = list(torch_args(p))
    a[0] = a[0].transpose(0, 1).contiguous()  # batch first
    got = m.lstm_backward_float(*a, True, dev(tr["gate_outputs"]), dev(tr["cell_states"]), dev(tr["cell_tanh_outputs"]),
                                dev(tr["hidden_outputs"]), dev(g[0]), dev(g[1]), dev(g[2]), master, ckpt)
    close(got[0].transpose(0, 1).cpu().numpy(), want["input"], 2e-5, "input")
    for n, t in list(zip(L.MASTER_VALUES, got))[1:]:
        close(t.cpu().numpy().reshape(want[n].shape), want[n], 2e-5, n)
        assert (t.cpu().numpy().reshape(want[n].shape)[masks[n] != 0] == 0).all()


CONFIGS = [dict(symmetric_activations=True), dict(), dict(scale_mode=L.SCALE_POT2, symmetric_activations=True),
           dict(parameter_granularity=L.PER_TENSOR), dict(parameter_granularity=L.PER_GATE, scale_mode=L.SCALE_POT2)]


def calibrated_bundle(cfg, p, scale_x=1.0):
    m = mod()
    xs = np.stack([p["x"] * scale_x])
    ranges, box = ll.calibrate("orc", cfg, p, xs)
    return box, m._params_to_bundle(box)


@pytest.mark.parametrize("cfg_kw", CONFIGS)
@pytest.mark.parametrize("T,B,I,H,bias,state", SHAPES[:3])
def test_quantized_forward_is_bit_exact(cfg_kw, T, B, I, H, bias, state):
    cfg = L.default_config(**cfg_kw)
    p = ll.problem(T, B, I, H, seed=3 * T + H, bias=bias, state=state)
    # calibrate on a narrower input so that clamping really happens in the measured pass
    box, bundle = calibrated_bundle(cfg, p, scale_x=0.6)
    q, qmask = ll.quantize_masters("orc", p, box, with_masks=True)
    w_out, w_hn, w_cn, w_tr, w_mk = ll.forward_quantized_masked(box, T, B, q)
    s = box.struct
    m = mod()
    out, hn, cn, ck, safety = m.lstm_forward_quantized(*torch_args(p), False, bundle, "pedantic", False, True)
    for n in L.TRACE_VALUES:
        np.testing.assert_array_equal(ck["values"][n].cpu().numpy(), w_tr[n], err_msg=n)
        np.testing.assert_array_equal(ck["clamp_masks"][n].cpu().numpy(), w_mk[n], err_msg=n + " mask")
    np.testing.assert_array_equal(out.cpu().numpy(), ll.dequantize(w_out, [s.scale[L.OUTPUT]], s.zero_point[L.OUTPUT]))
    np.testing.assert_array_equal(hn.cpu().numpy()[0], ll.dequantize(w_hn, [s.scale[L.OUTPUT]], s.zero_point[L.OUTPUT]))
    np.testing.assert_array_equal(cn.cpu().numpy()[0], ll.dequantize(w_cn, [s.scale[L.CELL_STATE]], s.zero_point[L.CELL_STATE]))
    pairs = [("input", "x"), ("weight_ih", "w_ih"), ("weight_hh", "w_hh"), ("bias_ih", "b_ih"), ("bias_hh", "b_hh"),
             ("h_0", "h0"), ("c_0", "c0")]
    for name, key in pairs:
        if q[key] is None:
            continue
        np.testing.assert_array_equal(ck["quantized_master"][name].cpu().numpy().reshape(q[key].shape), q[key], err_msg=name)
        np.testing.assert_array_equal(ck["master_clamp_masks"][name].cpu().numpy().reshape(q[key].shape).astype(np.uint8),
                                      qmask[key], err_msg=name + " mask")
    assert sum(int(w_mk[n].sum()) for n in L.TRACE_VALUES) > 0 or T * B < 50  # the case exercises clamping
    # inference call (no checkpoints) returns the same outputs
    out2, hn2, cn2, empty, _ = m.lstm_forward_quantized(*torch_args(p), False, bundle)
    assert torch.equal(out, out2) and torch.equal(hn, hn2) and torch.equal(cn, cn2) and empty == {}


def qat_round_trip(T, B, I, H, seed, cfg, batch_first):
    """Quantized training forward (bit-exact against the checker), then the QAT backward on the saved
    tensors against the masked float backward of the checker on the dequantized tensors."""
    p = ll.problem(T, B, I, H, seed=seed, wscale=0.15)
    box, bundle = calibrated_bundle(cfg, p, scale_x=0.8)
    q, qmask = ll.quantize_masters("orc", p, box, with_masks=True)
    w_out, w_hn, w_cn, w_tr, w_mk = ll.forward_quantized_masked(box, T, B, q)
    m = mod()
    a = list(torch_args(p))
    if batch_first:
        a[0] = a[0].transpose(0, 1).contiguous()
    out, hn, cn, ck, _ = m.lstm_forward_quantized(*a, batch_first, bundle, "pedantic", False, True)
    for n in L.TRACE_VALUES:
        np.testing.assert_array_equal(ck["values"][n].cpu().numpy(), w_tr[n], err_msg=n)
        np.testing.assert_array_equal(ck["clamp_masks"][n].cpu().numpy(), w_mk[n], err_msg=n + " mask")
    assert out.shape == ((B, T, H) if batch_first else (T, B, H))
    s = box.struct
    deq = lambda v, op: ll.dequantize(v, [s.scale[op]], s.zero_point[op])  # noqa: E731
    real = dict(p)
    real.update(x=deq(q["x"], L.INPUT), h0=deq(q["h0"], L.OUTPUT), c0=deq(q["c0"], L.CELL_STATE),
                w_ih=ll.dequantize(q["w_ih"], box.channel_scales[0], 0, I), w_hh=ll.dequantize(q["w_hh"], box.channel_scales[1], 0, H))
    go = np.concatenate([deq(w_tr["gate_outputs"][..., g * H:(g + 1) * H], L.INPUT_GATE_OUTPUT + g) for g in range(4)], -1)
    rtr = dict(gate_outputs=go, cell_states=deq(w_tr["cell_states"], L.CELL_STATE),
               cell_tanh_outputs=deq(w_tr["cell_tanh_outputs"], L.CELL_TANH_OUTPUT),
               hidden_outputs=deq(w_tr["hidden_outputs"], L.OUTPUT))
    rng = np.random.default_rng(4)
    g = [rng.standard_normal(sh).astype(np.float32) for sh in [(T, B, H), (B, H), (B, H)]]
    masks = dict(input=qmask["x"], weight_ih=qmask["w_ih"], weight_hh=qmask["w_hh"], bias_ih=qmask["b_ih"],
                 bias_hh=qmask["b_hh"], initial_hidden=qmask["h0"], initial_cell=qmask["c0"])
    masks.update(w_mk)
    want = ll.backward_float("orc", real, rtr, *g, masks=masks)
    qm, qk = ck["quantized_master"], ck["master_clamp_masks"]
    order = ("input", "weight_ih", "weight_hh", "bias_ih", "bias_hh", "h_0", "c_0")
    values = [ck["values"][n] for n in ("gate_outputs", "cell_states", "cell_tanh_outputs", "hidden_outputs")]
    got = m.lstm_backward_qat([qm[n] for n in order], batch_first, bundle, values, dev(g[0]), dev(g[1]), dev(g[2]),
                              [qk[n] for n in order], [ck["clamp_masks"][n] for n in L.TRACE_VALUES])
    dx = got[0].transpose(0, 1) if batch_first else got[0]
    close(dx.cpu().numpy(), want["input"], 2e-5, "input")
    for n, t in list(zip(L.MASTER_VALUES, got))[1:]:
        close(t.cpu().numpy().reshape(want[n].shape), want[n], 2e-5, n)


def test_quantized_forward_bench_shape_round_trip_and_qat_backward():
    """I=40, H=128, B=256: the shape of the QAT throughput measurement (tensor-core backward, two batch rows per CTA)."""
    qat_round_trip(20, 256, 40, 128, 77, L.default_config(symmetric_activations=True), batch_first=True)


def test_qat_backward_row_ranges_of_several_tiles():
    """T*B = 20480 rows: every CTA of the tcgen05 input-gradient kernel walks two 128-row tiles."""
    qat_round_trip(80, 256, 40, 128, 78, L.default_config(symmetric_activations=True), batch_first=False)


@pytest.mark.parametrize("T,B,I,H", [(6, 3, 8, 32), (5, 5, 12, 64), (4, 2, 40, 96), (5, 700, 16, 32), (6, 4, 9, 20)])
def test_qat_backward_other_tile_shapes(T, B, I, H):
    """Every hidden size the tensor-core backward is built for, one / two / four rows per CTA, an
    asymmetric grid, and a hidden size that takes the SIMT kernel (H = 20)."""
    qat_round_trip(T, B, I, H, 7 + H, L.default_config(), batch_first=False)


def test_calibration_session_matches_checker():
    T, B, I, H = 9, 6, 10, 16
    cfg = L.default_config()
    p = ll.problem(T, B, I, H, seed=31)
    p2 = ll.problem(T, B, I, H, seed=32)
    m = mod()
    session = m.CalibrationSession(m._config_to_json(cfg), I, H, True)
    assert session.state == "empty"
    for x in (p["x"], p2["x"] * 1.7):
        session.collect(dev(x), dev(p["w_ih"]), dev(p["w_hh"]), dev(p["b_ih"]), dev(p["b_hh"]), state3(p["h0"]), state3(p["c0"]))
    assert session.state == "dirty" and session.batch_count == 2
    ranges, box = ll.calibrate("orc", cfg, p, np.stack([p["x"], p2["x"] * 1.7]))
    r = session._ranges.struct
    for op in range(L.NUM_OPS):
        if op in L.PARAMETER_OPS:
            continue
        close([r.minimum[op], r.maximum[op]], [ranges.struct.minimum[op], ranges.struct.maximum[op]], 1e-5, L.OP_NAMES[op])
    for k in range(3):
        close([r.contribution_min[k], r.contribution_max[k]],
              [ranges.struct.contribution_min[k], ranges.struct.contribution_max[k]], 1e-5, f"contribution {k}")
    for k in range(4):
        np.testing.assert_array_equal(session._ranges.mins[k], ranges.mins[k])
        np.testing.assert_array_equal(session._ranges.maxs[k], ranges.maxs[k])
    final = session.finalize()
    assert session.state == "locked" and final["batch_count"] == 2
    got = m._bundle_to_params(final["bundle_json"])
    for k in range(4):  # parameter scales depend on the weights only: exact
        np.testing.assert_array_equal(got.channel_scales[k], box.channel_scales[k])
    for op in range(L.NUM_OPS):
        if op not in L.PARAMETER_OPS:
            close([got.struct.scale[op]], [box.struct.scale[op]], 1e-5, L.OP_NAMES[op])
    with pytest.raises(RuntimeError):
        session.collect(dev(p["x"]), dev(p["w_ih"]), dev(p["w_hh"]), dev(p["b_ih"]), dev(p["b_hh"]))
    audit = m.audit_quant_params_bundle(final["bundle_json"])
    assert audit["bundle_json"] == final["bundle_json"] and audit["hidden_size"] == H


def test_errors_are_reported_not_faulted():
    m = mod()
    p = ll.problem(3, 2, 4, 8, seed=1)
    cfg = L.default_config()
    box, bundle = calibrated_bundle(cfg, p)
    with pytest.raises(RuntimeError):
        m.lstm_forward(torch.zeros(3, 2, 4), dev(p["w_ih"]), dev(p["w_hh"]))  # CPU tensor
    with pytest.raises(RuntimeError):
        m.lstm_forward_quantized(dev(p["x"]), dev(p["w_ih"]), dev(p["w_hh"]), None, None, None, None, False, bundle)  # bias mismatch
    with pytest.raises(ValueError):
        m.lstm_forward_quantized(*torch_args(p), False, "{not json")
    wide = L.default_config()
    wide.bitwidth[L.CELL_STATE] = 20  # activation grids of up to 16 bits are built
    wbox, wbundle = calibrated_bundle(wide, p)
    with pytest.raises(RuntimeError, match="16 bits"):
        m.lstm_forward_quantized(*torch_args(p), False, wbundle)
    wide = L.default_config()
    wide.bitwidth[L.WEIGHT_HH] = 12  # weight grids of up to 8 bits are built
    wbox, wbundle = calibrated_bundle(wide, p)
    with pytest.raises(RuntimeError, match="8 bits"):
        m.lstm_forward_quantized(*torch_args(p), False, wbundle)


@pytest.mark.skipif(not ll.have_ref(), reason="compiled reference not available")
@pytest.mark.parametrize("method", ["sqnr", "percentile"])
@pytest.mark.parametrize("state", [True, False])
def test_histogram_calibration_session_matches_reference(method, state):
    T, B, I, H = 12, 8, 10, 16
    cfg = L.default_config()
    p = ll.problem(T, B, I, H, seed=51, state=state)
    xs = np.stack([p["x"], ll.problem(T, B, I, H, seed=52)["x"] * 1.5])
    want_h, want_p = ll.calibrate_hist(cfg, p, xs, method, 99.9)
    m = mod()
    session = m.CalibrationSession(m._config_to_json(cfg), I, H, True, method, 99.9)
    for x in xs:
        session.collect(dev(x), dev(p["w_ih"]), dev(p["w_hh"]), dev(p["b_ih"]), dev(p["b_hh"]), state3(p["h0"]), state3(p["c0"]))
    got_h = session._hists
    for (glo, ghi, gn), (wlo, whi, wn) in zip(got_h.states(), want_h.states()):
        assert gn == wn
        if wn:
            span = max(whi - wlo, 1e-6)
            assert abs(glo - wlo) <= 1e-5 * span + 1e-7 and abs(ghi - whi) <= 1e-5 * span + 1e-7
    for op in range(L.NUM_OPS):
        total = want_h.struct.point[op].total_count
        if total:
            moved = np.abs(got_h.counts[op] - want_h.counts[op]).sum()
            assert moved <= 0.02 * total, (L.OP_NAMES[op], moved, total)
    # x and the parameters involve no arithmetic: exact
    np.testing.assert_array_equal(got_h.counts[L.INPUT], want_h.counts[L.INPUT])
    np.testing.assert_array_equal(got_h.counts[L.NUM_OPS:], want_h.counts[L.NUM_OPS:])
    final = session.finalize()
    got_p = m._bundle_to_params(final["bundle_json"])
    for k in range(4):
        np.testing.assert_array_equal(got_p.channel_scales[k], want_p.channel_scales[k])
    for op in range(L.NUM_OPS):
        if op not in L.PARAMETER_OPS:
            close([got_p.struct.scale[op]], [want_p.struct.scale[op]], 0.03, L.OP_NAMES[op])
    out = m.lstm_forward_quantized(*torch_args(p), False, final["bundle_json"])
    assert torch.isfinite(out[0]).all()
