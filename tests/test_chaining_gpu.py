"""Integer-in / integer-out module glue: bidirectional flip / concatenate in the integer domain and a stack of
layers chained on codes, against the same layers run one by one through the binding."""
import numpy as np
import pytest
import torch

import oracle_lib as ol
from rx_met_b200 import _cabi as cabi

pytestmark = pytest.mark.gpu


def make_direction(seed, T, B, I, H, x):
    from rx_met_b200 import gru_interface_binding as ops
    from rx_met_b200.chaining import Direction
    W, R, bw, br, _, _ = ol.gru_problem(seed, T, B, I, H, with_h0=False)
    t = [torch.from_numpy(v).cuda() for v in (W, R, bw, br)]
    cfg = ops.OperatorQuantConfig()
    for name in cabi.OP_NAMES:
        if name not in ("W", "R", "bw", "br"):
            setattr(cfg, f"{name}_symmetric_", False)
    ranges = ops.GRUQuantizationRanges(H)
    ops.forward_calibrate(False, T, B, I, H, *t, x, None, "minmax", cfg, quant_ranges=ranges)
    qp = ops.calculate_gru_quantitative_parameters(ranges, cfg)
    return Direction(*t, qp), cfg


def quantize(x, scale, zp, bitwidth=8, unsigned=False):
    lo, hi = (0, (1 << bitwidth) - 1) if unsigned else (-(1 << (bitwidth - 1)), (1 << (bitwidth - 1)) - 1)
    return torch.clamp(torch.round(x / scale) + zp, lo, hi).to(torch.int32)


def test_bidirectional_module_on_codes():
    from rx_met_b200 import chaining, gru_interface_binding as ops, quant_params_io as qio
    T, B, I, H = 7, 5, 12, 32
    x = torch.randn((T, B, I), generator=torch.Generator().manual_seed(1)).cuda()
    fwd, cfg = make_direction(21, T, B, I, H, x)
    rev, _ = make_direction(22, T, B, I, H, x.flip(0).contiguous())
    rev.params.scale_x_, rev.params.zp_x_ = fwd.params.scale_x_, fwd.params.zp_x_   # one input tensor, one grid
    meta = qio.io_quant_meta(cfg, fwd.params)
    x_q = quantize(x, meta["input"]["scale"], meta["input"]["zp"])
    hx_q = torch.randint(-20, 20, (2, B, H), dtype=torch.int32, device="cuda")
    out, last = chaining.forward_quantized(chaining.Layer(fwd, rev), x_q, hx_q)
    assert out.dtype == torch.int32 and tuple(out.shape) == (T, B, 2 * H) and tuple(last.shape) == (2, B, H)
    want_f, last_f = ops.forward_quantized_int_io(T, B, I, H, fwd.W, fwd.R, fwd.bw, fwd.br, x_q, hx_q[0], fwd.params)
    want_r, last_r = ops.forward_quantized_int_io(T, B, I, H, rev.W, rev.R, rev.bw, rev.br, x_q.flip(0).contiguous(),
                                                  hx_q[1], rev.params)
    assert torch.equal(out[..., :H], want_f) and torch.equal(out[..., H:], want_r.flip(0))
    assert torch.equal(last[0], last_f[0]) and torch.equal(last[1], last_r[0])
    assert torch.equal(last[0], out[-1, :, :H]) and torch.equal(last[1], out[0, :, H:])
    # batch-first layout in and out
    out_bf, last_bf = chaining.forward_quantized(chaining.Layer(fwd, rev), x_q.transpose(0, 1).contiguous(), hx_q,
                                                 batch_first=True)
    assert torch.equal(out_bf.transpose(0, 1), out) and torch.equal(last_bf, last)
    with pytest.raises(TypeError):
        chaining.forward_quantized(chaining.Layer(fwd, rev), x)
    with pytest.raises(ValueError):
        chaining.forward_quantized(chaining.Layer(fwd, rev), x_q, hx_q[:1])


def test_stack_chains_codes_when_the_grids_agree():
    from rx_met_b200 import chaining, gru_interface_binding as ops, quant_params_io as qio
    T, B, I, H = 9, 4, 16, 32
    x = torch.randn((T, B, I), generator=torch.Generator().manual_seed(2)).cuda()
    first, cfg1 = make_direction(31, T, B, I, H, x)
    meta1 = qio.io_quant_meta(cfg1, first.params)
    x_q = quantize(x, meta1["input"]["scale"], meta1["input"]["zp"])
    h1_q, _ = ops.forward_quantized_int_io(T, B, I, H, first.W, first.R, first.bw, first.br, x_q, None, first.params)
    h1 = (h1_q - meta1["output"]["zp"]).float() * meta1["output"]["scale"]
    second, cfg2 = make_direction(32, T, B, H, H, h1)
    # the second layer is calibrated on the first one's output; its input grid is then set to that output grid
    second.params.scale_x_, second.params.zp_x_ = first.params.scale_h_, first.params.zp_h_
    layers = [chaining.Layer(first), chaining.Layer(second)]
    out, finals = chaining.forward_quantized_stack(layers, [cfg1, cfg2], x_q)
    want, last = ops.forward_quantized_int_io(T, B, H, H, second.W, second.R, second.bw, second.br, h1_q, None,
                                              second.params)
    assert torch.equal(out, want) and torch.equal(finals[1], last) and len(finals) == 2
    # the fp32 round trip between the layers gives the same codes: that is what chaining saves
    meta2 = qio.io_quant_meta(cfg2, second.params)
    again = quantize(h1, meta2["input"]["scale"], meta2["input"]["zp"])
    assert torch.equal(again, h1_q)
    second.params.zp_x_ = first.params.zp_h_ + 1
    with pytest.raises(ValueError):
        chaining.forward_quantized_stack(layers, [cfg1, cfg2], x_q)
    with pytest.raises(ValueError):
        chaining.forward_quantized_stack([chaining.Layer(first, first)], [cfg1], x_q)
