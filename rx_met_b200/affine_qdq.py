"""Fused quantize-dequantize of the affine quantizers with a learned grid.

Mirror of ``quantize_dequantize`` and ``QuantDequantFunc`` of the reference's default backend
(src/aimet_torch/v2/quantization/affine/backends/torch_builtins.py:199-285 and :618-691): same arguments,
same choice between the fake-quantize fast path (grid not trained) and the differentiable form, same
gradients for tensor, scale and offset.  The arithmetic runs in two CUDA kernels of this package's library
(one pass forward, one pass backward) instead of a chain of eager tensor expressions; torch is used for
memory, the current stream and the autograd graph only.  float32 CUDA tensors; per-tensor grids, grids along one
axis or a run of adjacent axes, and blockwise grids (`block_size`); anything else raises (there is no eager path
here).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from . import _cabi as cabi

_BOUND = False


def _library():
    global _BOUND
    lib = cabi.load_library()
    if not _BOUND:
        u64 = C.c_uint64
        lib.rxmet_affine_qdq_forward.restype = C.c_int
        lib.rxmet_affine_qdq_forward.argtypes = [C.c_void_p, u64, u64, u64, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                                 C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
        lib.rxmet_affine_qdq_backward_workspace_bytes.restype = C.c_size_t
        lib.rxmet_affine_qdq_backward_workspace_bytes.argtypes = [u64, u64, u64]
        lib.rxmet_affine_qdq_backward.restype = C.c_int
        lib.rxmet_affine_qdq_backward.argtypes = [C.c_void_p, C.c_void_p, u64, u64, u64, C.c_void_p, C.c_void_p, C.c_int,
                                                  C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                                  C.c_size_t, C.c_void_p]
        _BOUND = True
    return lib


def _ptr(t: Optional[torch.Tensor]):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def _stream(device) -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def grid_layout(tensor_shape, scale_shape) -> Tuple[int, int, int]:
    """(outer, channels, inner) of a tensor whose grid has `scale_shape` (right-aligned, as broadcasting does):
    one element, or the tensor's extents along one run of adjacent axes and 1 elsewhere.  The run makes the grid
    entries contiguous blocks of `inner` elements, which is the layout the kernels take."""
    tensor_shape, scale_shape = tuple(tensor_shape), tuple(scale_shape)
    count = 1
    for n in scale_shape:
        count *= n
    total = 1
    for n in tensor_shape:
        total *= n
    if count == 1:
        return 1, 1, total
    if len(scale_shape) > len(tensor_shape):
        raise RuntimeError(f"grid of shape {scale_shape} does not fit a tensor of shape {tensor_shape}")
    padded = (1,) * (len(tensor_shape) - len(scale_shape)) + scale_shape
    axes = [a for a, n in enumerate(padded) if n != 1]
    first, last = axes[0], axes[-1]
    if any(padded[a] != tensor_shape[a] for a in range(first, last + 1)):
        raise RuntimeError(f"only per-tensor grids and grids along adjacent axes are built (grid {scale_shape}, "
                           f"tensor {tensor_shape})")
    outer = 1
    for n in tensor_shape[:first]:
        outer *= n
    inner = 1
    for n in tensor_shape[last + 1:]:
        inner *= n
    return outer, count, inner


def blocked_shapes(tensor_shape, scale_shape, block_size) -> Tuple[Tuple[int, ...], Tuple[int, ...]]:
    """Shapes the reference views tensor and grid in for blockwise grids (torch_builtins.py:694-754): every
    blocked dimension d becomes (blocks, block length), the grid gets a 1 after each of its dimensions.  A block
    size of -1 takes the whole extent per grid entry."""
    tensor_shape, scale_shape, block_size = tuple(tensor_shape), tuple(scale_shape), tuple(block_size)
    if len(scale_shape) != len(block_size) or len(block_size) > len(tensor_shape):
        raise RuntimeError(f"block_size {block_size} does not fit grid {scale_shape} and tensor {tensor_shape}")
    view = []
    for k in range(1, len(block_size) + 1):
        blocks, extent = scale_shape[-k], tensor_shape[-k]
        length = extent // blocks if block_size[-k] == -1 else block_size[-k]
        if blocks * length != extent:
            raise RuntimeError(f"dimension {-k} of size {extent} is not {blocks} blocks of {length}")
        view = [blocks, length] + view
    grid = []
    for n in scale_shape:
        grid += [n, 1]
    return tensor_shape[:-len(block_size)] + tuple(view), tuple(grid)


def _checked(tensor, scale, offset):
    if not (tensor.is_cuda and scale.is_cuda and offset.is_cuda):
        raise RuntimeError("affine_qdq runs on CUDA tensors only")
    if tensor.dtype != torch.float32:
        raise RuntimeError("affine_qdq: float32 tensors only")
    if scale.numel() != offset.numel():
        raise RuntimeError("affine_qdq: scale and offset differ in size")
    return (tensor.contiguous(), scale.detach().to(torch.float32).contiguous(),
            offset.detach().to(torch.float32).contiguous())


def _layout(x, scale, block_size):
    if block_size is None:
        return grid_layout(x.shape, scale.shape)
    return grid_layout(*blocked_shapes(x.shape, scale.shape, block_size))


def forward(tensor, scale, offset, qmin: int, qmax: int, *, reciprocal: bool, want_keep: bool = False, block_size=None):
    """y (and the in-grid flags as a bool tensor when `want_keep`) of one fused pass."""
    x, s, o = _checked(tensor, scale, offset)
    outer, channels, inner = _layout(x, scale, block_size)
    y = torch.empty_like(x)
    keep = torch.empty(x.shape, dtype=torch.bool, device=x.device) if want_keep else None
    with torch.cuda.device(x.device):  # launch on the tensor's device, whatever device is current
        cabi.check(_library().rxmet_affine_qdq_forward(_ptr(x), outer, channels, inner, _ptr(s), _ptr(o), int(qmin),
                                                      int(qmax), int(reciprocal), _ptr(y), _ptr(keep), _stream(x.device)),
                   "affine_qdq.forward")
    return y, keep


def backward(grad, tensor, scale, offset, qmin: int, qmax: int, *, reciprocal: bool, want_tensor_grad: bool = True,
             want_scale_grad: bool = False, want_offset_grad: bool = False, block_size=None):
    """(dx, dscale, doffset); the grid gradients have the shape of `scale` / `offset`."""
    x, s, o = _checked(tensor, scale, offset)
    g = grad.to(torch.float32).contiguous()
    outer, channels, inner = _layout(x, scale, block_size)
    lib = _library()
    dx = torch.empty_like(x) if want_tensor_grad else None
    ds = torch.empty(channels, dtype=torch.float32, device=x.device) if want_scale_grad else None
    do = torch.empty(channels, dtype=torch.float32, device=x.device) if want_offset_grad else None
    ws = None
    ws_bytes = 0
    if ds is not None or do is not None:
        ws_bytes = lib.rxmet_affine_qdq_backward_workspace_bytes(outer, channels, inner)
        ws = torch.empty(max(ws_bytes, 4), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        cabi.check(lib.rxmet_affine_qdq_backward(_ptr(g), _ptr(x), outer, channels, inner, _ptr(s), _ptr(o), int(qmin),
                                                 int(qmax), int(reciprocal), _ptr(dx), _ptr(ds), _ptr(do), _ptr(ws), ws_bytes,
                                                 _stream(x.device)), "affine_qdq.backward")
    return (dx, ds.view(scale.shape) if ds is not None else None, do.view(offset.shape) if do is not None else None)


class QuantDequantFunc(torch.autograd.Function):
    """Differentiable quantize-dequantize; saves the input itself instead of a mask (the backward
    recomputes the flags in the same pass that reads the input for the scale gradient)."""

    @staticmethod
    def forward(ctx, tensor, scale, offset, qmin: int, qmax: int, reciprocal: bool = False, block_size=None):
        y, _ = forward(tensor, scale, offset, qmin, qmax, reciprocal=reciprocal, block_size=block_size)
        ctx.qmin, ctx.qmax, ctx.reciprocal, ctx.block_size = qmin, qmax, reciprocal, block_size
        ctx.save_for_backward(tensor, scale, offset)
        return y

    @staticmethod
    def backward(ctx, grad):
        tensor, scale, offset = ctx.saved_tensors
        need = ctx.needs_input_grad
        dx, ds, do = backward(grad, tensor, scale, offset, ctx.qmin, ctx.qmax, reciprocal=ctx.reciprocal,
                              want_tensor_grad=need[0], want_scale_grad=need[1], want_offset_grad=need[2],
                              block_size=ctx.block_size)
        return dx, ds, do, None, None, None, None


def quantize_dequantize(tensor: torch.Tensor, scale: torch.Tensor, offset: torch.Tensor, qmin: int, qmax: int,
                        block_size=None, zero_point_shift: float = 0.0) -> torch.Tensor:
    """Drop-in for the reference's ``quantize_dequantize`` (torch_builtins.py:199).  The fast form is taken under
    the reference's own conditions: no blocks and a grid that is not being trained."""
    if zero_point_shift != 0.0:
        raise RuntimeError("affine_qdq: zero_point_shift is not built")
    trained = (scale.requires_grad or offset.requires_grad) and torch.is_grad_enabled()
    # blockwise grids always take the divide form: the reference's fast path does not handle them
    reciprocal = not trained and block_size is None
    return QuantDequantFunc.apply(tensor, scale, offset, qmin, qmax, reciprocal,
                                  None if block_size is None else tuple(block_size))
