"""Builder and ctypes loader of the allocation-free column-sum library (``libwallx_noalloc.so``).

The library is plain CUDA C (no torch dependency) and exports ``wx_column_sum_bf16_noalloc``; see
``csrc/no_alloc.h`` for the contract. It is meant for callers that cannot allocate device memory;
Python users normally want :func:`wallx_b200.ops.functional.column_sum` instead.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

from . import _ext

LIB_NAME = "libwallx_noalloc.so"
MAX_COLS = 65536


def lib_path() -> str:
    return os.path.join(_ext.BUILD_DIR, LIB_NAME)


def build(verbose: bool = False) -> str:
    os.makedirs(_ext.BUILD_DIR, exist_ok=True)
    src = os.path.join(_ext.CSRC, "no_alloc.cu")
    out = lib_path()
    if os.path.exists(out) and os.path.getmtime(out) >= max(os.path.getmtime(src), os.path.getmtime(src[:-3] + ".h")):
        return out
    cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-shared",
           "-Xcompiler", "-fPIC", "-I", _ext.CSRC, "-o", out, src]
    subprocess.run(cmd, check=True, capture_output=not verbose)
    return out


_lib = None


def load():
    """ctypes handle with argument types set; raises if the library has not been built."""
    global _lib
    if _lib is None:
        path = lib_path()
        if not os.path.exists(path):
            raise RuntimeError(f"{path} is missing: run __graft_entry__.build()")
        lib = ctypes.CDLL(path)
        lib.wx_column_sum_bf16_noalloc.argtypes = [ctypes.c_void_p, ctypes.c_long, ctypes.c_void_p, ctypes.c_int,
                                                   ctypes.c_int, ctypes.c_void_p]
        lib.wx_column_sum_bf16_noalloc.restype = ctypes.c_int
        lib.wx_noalloc_strerror.argtypes = [ctypes.c_int]
        lib.wx_noalloc_strerror.restype = ctypes.c_char_p
        _lib = lib
    return _lib
