"""Host -> device staging of a step's inputs next to a running training step.

``stage_from_pinned_host`` copies a page-locked host tensor into a device tensor with a narrow
kernel that reads the host memory over PCIe (``rxmet_stage_from_pinned_host``) instead of a
copy-engine transfer: on a side stream it disturbs the latency-bound recurrent kernels of the
step less than the same bytes moved by the copy engine.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _cabi as cabi

_configured = False


def stage_from_pinned_host(dst: torch.Tensor, src: torch.Tensor, ctas: int = 4, stream=None) -> None:
    """dst (CUDA, contiguous) <- src (pinned host, contiguous, same dtype and number of elements),
    enqueued on ``stream`` (default: the current stream); returns without waiting."""
    global _configured
    if not (dst.is_cuda and dst.is_contiguous()):
        raise RuntimeError("dst must be a contiguous CUDA tensor")
    if src.is_cuda or not src.is_pinned() or not src.is_contiguous():
        raise RuntimeError("src must be a contiguous tensor in page-locked host memory")
    if dst.dtype != src.dtype or dst.numel() != src.numel():
        raise RuntimeError("dst and src must agree in dtype and number of elements")
    lib = cabi.load_library()
    if not _configured:
        lib.rxmet_stage_from_pinned_host.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p]
        _configured = True
    stream = stream if stream is not None else torch.cuda.current_stream(dst.device)
    with torch.cuda.device(dst.device):
        rc = lib.rxmet_stage_from_pinned_host(dst.data_ptr(), src.data_ptr(), dst.numel() * dst.element_size(), int(ctas),
                                              stream.cuda_stream)
    if rc != 0:
        raise RuntimeError(lib.rxmet_last_error().decode())
