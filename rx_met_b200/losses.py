"""Loss of a training step on the device: mean-squared error and its gradient in one pass (C ABI
`rxmet_mse_loss_grad`).  Torch supplies memory and the current stream only."""
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
        lib.rxmet_mse_loss_workspace_bytes.restype = C.c_size_t
        lib.rxmet_mse_loss_grad.restype = C.c_int
        lib.rxmet_mse_loss_grad.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p, C.c_void_p,
                                            C.c_size_t, C.c_void_p]
        _BOUND = True
    return lib


def workspace(device) -> torch.Tensor:
    """Scratch for `mse_loss_grad`; allocate once and pass it to every call of a loop."""
    return torch.empty(_library().rxmet_mse_loss_workspace_bytes(), dtype=torch.uint8, device=device)


def mse_loss_grad(out: torch.Tensor, target: torch.Tensor, grad: Optional[torch.Tensor] = None,
                  loss: Optional[torch.Tensor] = None, scratch: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """(loss, grad) with loss = mean((out - target)^2) as a device scalar and grad = (out - target) * (2 / n), the
    gradient of that loss with respect to `out`, bit-identical to the eager float32 expressions.  `grad`, `loss` and
    `scratch` may be preallocated (grad contiguous, same shape as out; views are fine)."""
    if not (out.is_cuda and target.is_cuda) or out.dtype != torch.float32 or target.dtype != torch.float32:
        raise RuntimeError("mse_loss_grad takes float32 CUDA tensors")
    if out.shape != target.shape or not out.is_contiguous() or not target.is_contiguous():
        raise RuntimeError("mse_loss_grad: out and target must be contiguous and of one shape")
    grad = torch.empty_like(out) if grad is None else grad
    if grad.shape != out.shape or not grad.is_contiguous() or grad.dtype != torch.float32:
        raise RuntimeError("mse_loss_grad: grad must be a contiguous float32 tensor of the shape of out")
    loss = torch.empty((), dtype=torch.float32, device=out.device) if loss is None else loss
    scratch = workspace(out.device) if scratch is None else scratch
    ptr = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
    with torch.cuda.device(out.device):  # the launch goes to the tensors' device, whatever device is current
        cabi.check(_library().rxmet_mse_loss_grad(ptr(out), ptr(target), out.numel(), ptr(grad), ptr(loss), ptr(scratch),
                                                  scratch.numel(),
                                                  C.c_void_p(torch.cuda.current_stream(out.device).cuda_stream)),
                   "mse_loss_grad")
    return loss, grad
