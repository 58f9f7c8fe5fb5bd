"""Exchange hook for data-parallel calibration (`rxmet_exchange`, include/rxmet_b200.h).

With the batch sharded over ranks, a histogram calibration batch needs two exchanges between its
kernels: the finite extremes (MIN / MAX) before anything is binned, and the bin counts (SUM) before
the host merges them.  The library calls a C function pointer for each; this module supplies one
that runs `torch.distributed.all_reduce` (NCCL over NVLink on CUDA tensors) in place on the device
buffer the library hands over, ordered on the library's stream.
"""
from __future__ import annotations

import ctypes as C

import torch

REDUCE_MIN_F32, REDUCE_MAX_F32, REDUCE_SUM_U32, REDUCE_SUM_U64 = 0, 1, 2, 3

ReduceFn = C.CFUNCTYPE(C.c_int, C.c_int, C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p)


class Exchange(C.Structure):
    _fields_ = [("reduce", ReduceFn), ("user", C.c_void_p), ("world_size", C.c_int32)]


class _DeviceArray:
    """Device memory owned by the library, seen through the CUDA array interface."""

    def __init__(self, ptr: int, count: int, typestr: str):
        self.__cuda_array_interface__ = {"shape": (count,), "typestr": typestr, "data": (ptr, False), "version": 3}


# unsigned sums travel as signed integers of the same width: the totals stay far below 2^31 / 2^63
_KINDS = {REDUCE_MIN_F32: ("<f4", "MIN"), REDUCE_MAX_F32: ("<f4", "MAX"), REDUCE_SUM_U32: ("<i4", "SUM"),
          REDUCE_SUM_U64: ("<i8", "SUM")}


def make_exchange(group, device) -> Exchange:
    """The struct to pass as `exchange`; keep the returned object alive for as long as the library may call it."""
    import torch.distributed as dist
    device = torch.device(device)
    ops = {"MIN": dist.ReduceOp.MIN, "MAX": dist.ReduceOp.MAX, "SUM": dist.ReduceOp.SUM}

    def reduce(kind, ptr, count, stream, _user):
        try:
            typestr, op = _KINDS[kind]
            if count == 0:
                return 0
            with torch.cuda.device(device):
                t = torch.as_tensor(_DeviceArray(ptr, int(count), typestr), device=device)
                if t.data_ptr() != ptr:
                    raise RuntimeError("the exchange buffer was copied instead of aliased")
                # Calibration is not a hot path: the exchange is fenced by device-wide synchronisation on both
                # sides, so it does not rely on how the process group orders its kernels against foreign streams.
                torch.cuda.synchronize(device)
                dist.all_reduce(t, op=ops[op], group=group)
                torch.cuda.synchronize(device)
            return 0
        except Exception:  # the C caller turns a non-zero return into an error status
            import traceback
            traceback.print_exc()
            return 1

    ex = Exchange()
    ex._callback = ReduceFn(reduce)  # referenced by the struct only as a raw pointer: hold it here
    ex.reduce = ex._callback
    ex.user = None
    ex.world_size = dist.get_world_size(group)
    return ex
