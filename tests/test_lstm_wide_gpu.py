"""QuantLSTM with 16-bit activation grids, W4 / W8 weights and hidden sizes up to 512 on the GPU, through the
drop-in module (C ABI), against the CPU checkers: bit-exact against the restatement with exactly accumulated
linear stages, and against the reference's own float-carrier CPU forward."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import lstm_lib as ll
from rx_met_b200 import _cabi_lstm as L
from test_lstm_gpu import close, dev, mod, torch_args

pytestmark = pytest.mark.gpu

CASES = [
    # T, B, I, H, weight bits, activation bits, granularity, bias, state
    (4, 4, 20, 24, 8, 16, L.PER_CHANNEL, True, True),
    (6, 9, 80, 128, 8, 16, L.PER_CHANNEL, True, False),    # bidirectional QuantLSTM H128 I80, W8 per channel / A16
    (3, 5, 256, 512, 4, 16, L.PER_CHANNEL, True, True),    # QuantLSTM I256 H512, W4 per channel / A16
    (4, 300, 40, 200, 8, 8, L.PER_TENSOR, False, True),    # 8-bit grids beyond H = 128; several rows per thread
    (5, 3, 17, 33, 4, 12, L.PER_GATE, True, True),
    (3, 700, 12, 64, 8, 16, L.PER_CHANNEL, True, True),    # many rows per CTA
]


def setup(T, B, I, H, wb, ab, gran, bias, state, seed=1, scale_x=0.8):
    cfg = L.mixed_config(wb, ab, parameter_granularity=gran)
    p = ll.problem(T, B, I, H, seed=seed, bias=bias, state=state, wscale=float(1.0 / np.sqrt(H)))
    _, box = ll.calibrate("orc", cfg, p, np.stack([p["x"] * scale_x]))
    return p, box, mod()._params_to_bundle(box)


@pytest.mark.parametrize("T,B,I,H,wb,ab,gran,bias,state", CASES)
def test_wide_forward_is_bit_exact(T, B, I, H, wb, ab, gran, bias, state):
    p, box, bundle = setup(T, B, I, H, wb, ab, gran, bias, state)
    q, qmask = ll.quantize_masters("orc", p, box, with_masks=True)
    w_out, w_hn, w_cn, w_tr, w_mk = ll.forward_quantized_masked(box, T, B, q, exact_sums=True)
    m = mod()
    out, hn, cn, ck, _ = m.lstm_forward_quantized(*torch_args(p), False, bundle, "pedantic", False, True)
    for n in L.TRACE_VALUES:
        np.testing.assert_array_equal(ck["values"][n].cpu().numpy(), w_tr[n], err_msg=n)
        np.testing.assert_array_equal(ck["clamp_masks"][n].cpu().numpy(), w_mk[n], err_msg=n + " mask")
    s = box.struct
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
    # the inference call (no checkpoints) returns the same outputs
    out2, hn2, cn2, empty, _ = m.lstm_forward_quantized(*torch_args(p), False, bundle)
    assert torch.equal(out, out2) and torch.equal(hn, hn2) and torch.equal(cn, cn2) and empty == {}
    # the reference's own CPU forward on the float carrier (sequential float sums)
    if ll.have_ref():
        r_out, r_hn, r_cn, r_tr = ll.forward_quantized("ref", box, T, B, q)
        for n in L.TRACE_VALUES:
            np.testing.assert_array_equal(ck["values"][n].cpu().numpy(), r_tr[n], err_msg=n + " (reference CPU)")


@pytest.mark.parametrize("T,B,I,H", [(5, 6, 30, 160), (3, 150, 256, 512), (4, 3, 7, 130)])
def test_float_forward_and_backward_beyond_128(T, B, I, H):
    p = ll.problem(T, B, I, H, seed=T + H, wscale=float(1.0 / np.sqrt(H)))
    want = ll.forward_float("orc", p)
    m = mod()
    out = m.lstm_forward_training(*torch_args(p), False)
    names = ["output", "h_n", "c_n", "gate_outputs", "cell_states", "cell_tanh_outputs", "hidden_outputs"]
    refs = [want[0], want[1][None], want[2][None], want[3]["gate_outputs"], want[3]["cell_states"],
            want[3]["cell_tanh_outputs"], want[3]["hidden_outputs"]]
    for n, g, w in zip(names, out, refs):
        close(g.cpu().numpy(), w, 2e-5, n)
    rng = np.random.default_rng(9)
    g = [rng.standard_normal(s).astype(np.float32) for s in [(T, B, H), (B, H), (B, H)]]
    tr = want[3]
    shapes = dict(input=(T, B, I), weight_ih=(4 * H, I), weight_hh=(4 * H, H), bias_ih=(4 * H,), bias_hh=(4 * H,),
                  initial_hidden=(B, H), initial_cell=(B, H))
    shapes.update({n: tr[n].shape for n in L.TRACE_VALUES})
    masks = {n: (rng.random(s) < 0.1).astype(np.uint8) for n, s in shapes.items()}
    wg = ll.backward_float("orc", p, tr, *g, masks=masks)
    master = [dev(masks["input"]).bool(), dev(masks["weight_ih"]), dev(masks["weight_hh"]), dev(masks["bias_ih"]),
              dev(masks["bias_hh"]), dev(masks["initial_hidden"])[None].bool(), dev(masks["initial_cell"])[None]]
    ckpt = [dev(masks[n]) for n in L.TRACE_VALUES]
    got = m.lstm_backward_float(*torch_args(p), False, dev(tr["gate_outputs"]), dev(tr["cell_states"]),
                                dev(tr["cell_tanh_outputs"]), dev(tr["hidden_outputs"]), dev(g[0]), dev(g[1]), dev(g[2]),
                                master, ckpt)
    for n, t in zip(L.MASTER_VALUES, got):
        close(t.cpu().numpy().reshape(wg[n].shape), wg[n], 2e-5, n)


@pytest.mark.parametrize("T,B,I,H,wb,ab", [(4, 6, 80, 128, 8, 16), (3, 5, 256, 512, 4, 16), (5, 130, 32, 256, 4, 16), (3, 40, 32, 384, 8, 16), (2, 2400, 16, 256, 4, 16)])
def test_wide_qat_backward(T, B, I, H, wb, ab):
    """Quantized training forward on 16-bit grids, then the QAT backward on the saved tensors against the
    masked float backward of the checker on the dequantized tensors."""
    p, box, bundle = setup(T, B, I, H, wb, ab, L.PER_CHANNEL, True, True, seed=5)
    q, qmask = ll.quantize_masters("orc", p, box, with_masks=True)
    w_out, w_hn, w_cn, w_tr, w_mk = ll.forward_quantized_masked(box, T, B, q, exact_sums=True)
    m = mod()
    out, hn, cn, ck, _ = m.lstm_forward_quantized(*torch_args(p), False, bundle, "pedantic", False, True)
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
    got = m.lstm_backward_qat([qm[n] for n in order], False, bundle, values, dev(g[0]), dev(g[1]), dev(g[2]),
                              [qk[n] for n in order], [ck["clamp_masks"][n] for n in L.TRACE_VALUES])
    for n, t in zip(L.MASTER_VALUES, got):
        close(t.cpu().numpy().reshape(want[n].shape), want[n], 2e-5, n)


def test_wide_calibration_session_matches_the_reference():
    """Min/max calibration of the 16-bit W8 configuration at H = 160 (float forward of the wide kernels): the
    finalized bundle of a GPU session against a reference session on the same batches."""
    if not ll.have_ref():
        pytest.skip("reference CPU sources not built")
    T, B, I, H = 5, 12, 24, 160
    cfg = L.mixed_config(8, 16)
    p = ll.problem(T, B, I, H, seed=11, wscale=float(1.0 / np.sqrt(H)))
    xs = np.stack([p["x"], p["x"][::-1] * 0.7])
    m = mod()
    session = m.CalibrationSession(m._config_to_json(cfg), I, H, True, "minmax")
    for x in xs:
        session.collect(dev(x), dev(p["w_ih"]), dev(p["w_hh"]), dev(p["b_ih"]), dev(p["b_hh"]), dev(p["h0"])[None],
                        dev(p["c0"])[None], False)
    got = m._bundle_to_params(session.finalize(False)["bundle_json"])
    _, want = ll.calibrate("ref", cfg, p, xs)
    a, b = got.struct, want.struct
    differing = 0
    for op in range(L.NUM_OPS):
        if op in L.PARAMETER_OPS:
            continue
        # the float forwards differ in the last place, so a range end may move by one ulp
        assert abs(a.scale[op] - b.scale[op]) <= 1e-5 * b.scale[op], op
        assert abs(a.zero_point[op] - b.zero_point[op]) <= 1, op
        differing += (a.scale[op] != b.scale[op]) or (a.zero_point[op] != b.zero_point[op])
    for k in range(4):
        np.testing.assert_array_equal(got.channel_scales[k], want.channel_scales[k])
    print(f"activation points whose (scale, zero point) differ from the reference CPU session: {differing} of 14")
