"""Stack of bidirectional QuantGRU layers under a classification head (`rx_met_b200.stacked_qat`): every layer's
outputs and the gradients of one QAT step against the CPU checker run layer by layer."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import oracle_lib as ol

pytestmark = pytest.mark.gpu


class _Params:
    """The C parameter struct of one direction, in the shape the checker's wrappers expect."""

    def __init__(self, direction):
        self.c = direction._c_params
        self.hidden = direction.H


def _np(t):
    return t.detach().cpu().numpy().copy()


def _close(got, want, tol, name):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    err = np.abs(got - want).max() / max(np.abs(want).max(), 1e-30)
    assert err <= tol, f"{name}: max error {err:.3e} of the largest magnitude"


_FLAG_BITS = {"gate_output": 0, "gate_input": 3, "weight_hh_linear": 6, "h": 12}   # weight_ih_linear stays a byte mask


@pytest.mark.parametrize("T,B,I,H,layers,bits", [(5, 6, 10, 32, 2, 16), (4, 5, 40, 256, 3, 16), (6, 4, 12, 64, 2, 8)])
def test_stacked_step_matches_the_checker(T, B, I, H, layers, bits):
    from rx_met_b200.stacked_qat import StackedGruQat, a16_config
    dev = torch.device("cuda:0")
    classes = 12
    model = StackedGruQat(T, B, I, H, layers, classes, dev, a16_config(8, bits), seed=3)
    gen = torch.Generator().manual_seed(7)
    batches = [torch.randn(T, B, I, generator=gen).clamp_(-4, 4).to(dev) for _ in range(2)]
    labels = torch.randint(0, classes, (B,), generator=gen).to(dev)
    model.calibrate(batches)
    x = batches[0]
    loss = model.step(x, labels, lr=0.0)  # lr = 0: the weights stay what the checker sees
    torch.cuda.synchronize()

    # ---- forward, layer by layer -------------------------------------------------
    xin = _np(x)
    saved = []
    for li, (fw, bw) in enumerate(model.dirs):
        outs = []
        for d, flip in ((fw, False), (bw, True)):
            xi = np.ascontiguousarray(xin[::-1]) if flip else xin
            want = ol.forward_quant("orc", _np(d.W), _np(d.R), _np(d.bw), _np(d.br), xi, None, _Params(d), training=True)
            np.testing.assert_array_equal(_np(d.x_q), want["x_q"], err_msg=f"layer {li} x codes")
            np.testing.assert_array_equal(_np(d.h), want["h"], err_msg=f"layer {li} h")
            np.testing.assert_array_equal(_np(d.v), want["v"], err_msg=f"layer {li} v")
            flags = _np(d.step_flags).astype(np.int32) & 0xffff if d._packed else None
            for k, m in want["masks"].arr.items():
                if flags is not None and k in _FLAG_BITS:   # the engine kept these as one 16-bit word per element and step
                    first = _FLAG_BITS[k]
                    got = (flags >> first) & 1 if k == "h" else np.concatenate([(flags >> (first + g)) & 1 for g in range(3)], -1)
                    np.testing.assert_array_equal(got.astype(np.uint8), m, err_msg=f"layer {li} packed flags {k}")
                    continue
                np.testing.assert_array_equal(_np(d.masks[k]), m, err_msg=f"layer {li} mask {k}")
            saved.append((d, want, flip))
            outs.append(want["h"][1:][::-1] if flip else want["h"][1:])
        xin = np.ascontiguousarray(np.concatenate(outs, -1))
        np.testing.assert_array_equal(_np(model.y[li]), xin, err_msg=f"layer {li} output")

    # ---- head ------------------------------------------------------------------------
    feat = xin.astype(np.float64).mean(0)
    logits = feat @ _np(model.head_w).astype(np.float64).T + _np(model.head_b)
    logits -= logits.max(1, keepdims=True)
    p = np.exp(logits) / np.exp(logits).sum(1, keepdims=True)
    lab = _np(labels)
    want_loss = -np.log(p[np.arange(B), lab]).mean()
    assert abs(float(loss) - want_loss) <= 1e-5 * max(1.0, abs(want_loss))
    dlogits = p.copy()
    dlogits[np.arange(B), lab] -= 1.0
    dlogits /= B
    _close(_np(model.head_dw), dlogits.T @ feat, 1e-5, "head weight gradient")
    _close(_np(model.head_db), dlogits.sum(0), 1e-5, "head bias gradient")
    dy = np.broadcast_to((dlogits @ _np(model.head_w).astype(np.float64) / T)[None], (T, B, 2 * H)).astype(np.float32)

    # ---- backward, top layer first -----------------------------------------------------
    for li in range(layers - 1, -1, -1):
        dx_sum = None
        for idx in (0, 1):
            d, fwd, flip = saved[2 * li + idx]
            part = dy[..., idx * H:(idx + 1) * H]
            dh_new = np.zeros((T + 1, B, H), np.float32)
            dh_new[1:] = part[::-1] if flip else part
            want = ol.backward_quant(fwd, dh_new, fwd["h"], fwd["v"], _Params(d), fwd["masks"])
            for name, got in (("dW", d.dW), ("dR", d.dR), ("dbw", d.dbw), ("dbr", d.dbr)):
                _close(_np(got), want[name], 2e-5, f"layer {li} direction {idx} {name}")
            dx = want["dx"][::-1] if flip else want["dx"]
            dx_sum = dx if dx_sum is None else dx_sum + dx
        dy = np.ascontiguousarray(dx_sum)
        if li > 0:
            _close(_np(model.dx[li]), dy, 2e-5, f"layer {li} input gradient")


def test_step_trains():
    """A few steps with a real learning rate lower the loss on a fixed batch."""
    from rx_met_b200.stacked_qat import StackedGruQat, a16_config
    dev = torch.device("cuda:0")
    T, B, I, H = 8, 16, 12, 32
    model = StackedGruQat(T, B, I, H, 2, 4, dev, a16_config(8, 16), seed=1)
    gen = torch.Generator().manual_seed(2)
    x = torch.randn(T, B, I, generator=gen).to(dev)
    labels = torch.randint(0, 4, (B,), generator=gen).to(dev)
    model.calibrate([x])
    losses = [float(model.step(x, labels, lr=0.5)) for _ in range(12)]
    assert losses[-1] < losses[0]


def test_captured_step_replays_the_eager_step():
    """One CUDA graph for the whole stacked step: after the same number of steps on the same inputs the weights
    and the loss equal those of the eager engine bit for bit."""
    from rx_met_b200.stacked_qat import StackedGruQat, a16_config
    T, B, I, H, layers, classes = 6, 8, 12, 64, 2, 5
    dev = torch.device("cuda", 0)
    gen = torch.Generator().manual_seed(3)
    x = torch.randn((T, B, I), generator=gen).to(dev)
    labels = torch.randint(0, classes, (B,), generator=gen).to(dev)
    engines = [StackedGruQat(T, B, I, H, layers, classes, dev, a16_config(8, 16), seed=11) for _ in range(2)]
    for e in engines:
        e.calibrate([x])
    eager, captured = engines
    replay, loss_c = captured.capture_step(x, labels, 1e-2, warmup=2)
    for _ in range(2):
        eager.step(x, labels, 1e-2)
    for _ in range(3):
        loss_e = eager.step(x, labels, 1e-2)
        loss_c = replay()
    torch.cuda.synchronize()
    assert captured.captured_launches > 50
    assert torch.equal(eager.flat_w, captured.flat_w)
    assert torch.equal(loss_e, loss_c)
