"""Integer-in / integer-out inference of a QuantGRU module and of a stack of them.

``QuantGRU.forward_quantized`` (operators/quant-gru/pytorch/quant_gru.py:2447-2543) runs one module on codes:
the input arrives as int32 codes on the module's input grid, the output leaves as int32 codes on its hidden
grid, the reverse direction of a bidirectional module reads the sequence flipped in time and its output is
flipped back and concatenated to the forward one, all in the integer domain.  Stacked layers chain their codes
directly when the producer's output grid is the consumer's input grid (`quant_params_io.grids_match`), which
removes the dequantize -> requantize round trip through fp32 tensors between layers.

The arithmetic is `gru_interface_binding.forward_quantized_int_io` (C ABI `rxmet_gru_forward_quant_int_io`);
this file only holds the module-level glue.  Weights are in the binding's layout: W [I, 3H], R [H, 3H],
bw / br [3H], gate order z, r, n.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch

from . import gru_interface_binding as gru_ops
from . import quant_params_io


@dataclass
class Direction:
    """Weights and quantization parameters of one direction of one layer."""
    W: torch.Tensor
    R: torch.Tensor
    bw: torch.Tensor
    br: torch.Tensor
    params: "gru_ops.GRUQuantParams"


@dataclass
class Layer:
    forward: Direction
    reverse: Optional[Direction] = None

    @property
    def hidden_size(self) -> int:
        return self.forward.R.shape[0]


def _run(direction: Direction, x_q: torch.Tensor, h0_q: Optional[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
    T, B, I = x_q.shape
    return gru_ops.forward_quantized_int_io(T, B, I, direction.R.shape[0], direction.W, direction.R, direction.bw,
                                            direction.br, x_q, h0_q, direction.params)


def forward_quantized(layer: Layer, x_q: torch.Tensor, hx_q: Optional[torch.Tensor] = None,
                      batch_first: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """One module on codes.  x_q: int32 [T, B, I] (or [B, T, I] with batch_first) on the layer's input grid;
    hx_q: int32 [directions, B, H] on its hidden grid, or None.  Returns (output_q [T, B, directions * H],
    h_n_q [directions, B, H]), the output in the caller's layout."""
    if x_q.is_floating_point():
        raise TypeError(f"forward_quantized takes integer codes (int in, int out); got dtype={x_q.dtype}")
    if batch_first:
        x_q = x_q.transpose(0, 1)
    x_q = x_q.to(dtype=torch.int32).contiguous()
    directions = 2 if layer.reverse is not None else 1
    if hx_q is not None:
        expected = (directions, x_q.shape[1], layer.hidden_size)
        if tuple(hx_q.shape) != expected:
            raise ValueError(f"hx shape should be {expected}, got {tuple(hx_q.shape)}")
        hx_q = hx_q.to(device=x_q.device, dtype=torch.int32).contiguous()
    out, last = _run(layer.forward, x_q, hx_q[0] if hx_q is not None else None)
    if layer.reverse is not None:
        out_r, last_r = _run(layer.reverse, x_q.flip(0).contiguous(), hx_q[1] if hx_q is not None else None)
        out = torch.cat([out, out_r.flip(0)], dim=-1)
        last = torch.cat([last, last_r], dim=0)
    if batch_first:
        out = out.transpose(0, 1).contiguous()
    return out, last


def forward_quantized_stack(layers: Sequence[Layer], configs: Sequence["gru_ops.OperatorQuantConfig"], x_q: torch.Tensor,
                            batch_first: bool = False) -> Tuple[torch.Tensor, List[torch.Tensor]]:
    """A stack of unidirectional layers on codes.  Layer k's output codes feed layer k+1 as they are; the grids
    must agree (effective scale, zero point, width, signedness), otherwise ValueError names the pair: such a
    stack has to requantize between those two layers and is not a pure integer chain."""
    metas = []
    for layer, config in zip(layers, configs):
        if layer.reverse is not None:
            raise ValueError("a bidirectional layer's two output grids cannot feed one input grid; chain unidirectional layers")
        metas.append(quant_params_io.io_quant_meta(config, layer.forward.params))
    for k in range(len(metas) - 1):
        if not quant_params_io.grids_match(metas[k]["output"], metas[k + 1]["input"]):
            raise ValueError(f"output grid of layer {k} {metas[k]['output']} is not the input grid of layer {k + 1} "
                             f"{metas[k + 1]['input']}")
    finals = []
    codes = x_q
    for layer in layers:
        codes, last = forward_quantized(layer, codes, None, batch_first)
        finals.append(last)
    return codes, finals
