"""ctypes access to the reference's own CUDA build of the QuantGRU path (oracle/_ref/libgru_ref_cuda.so, built by
`make -f oracle/Makefile refcuda`).  Test infrastructure: a same-device checker, never part of the product."""
from __future__ import annotations

import ctypes as C

import oracle_lib

SO = oracle_lib.ROOT / "oracle" / "_ref" / "libgru_ref_cuda.so"
_lib = None


def lib():
    global _lib
    if _lib is None and SO.exists():
        try:
            _lib = C.CDLL(str(SO))
            _lib.refcuda_last_error.restype = C.c_char_p
        except OSError:
            _lib = None
    return _lib


def call(name, *args):
    fn = getattr(lib(), name)
    fn.restype = C.c_int
    if fn(*args) != 0:
        raise RuntimeError(f"{name}: {lib().refcuda_last_error().decode(errors='replace')}")
