"""Loader for the host-side C++ helper library (``csrc/host/hostops.cpp``).

The library has a C ABI and no CUDA dependency. ``get()`` returns the ``ctypes`` handle or
``None`` when it has not been built; callers on the CPU control plane then use their
pure-Python equivalents, which produce identical results.
"""

from __future__ import annotations

import ctypes
import os
import subprocess
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(os.path.dirname(_HERE), "csrc", "host", "hostops.cpp")
_LIB = os.path.join(_HERE, "_xv_host.so")

_lock = threading.Lock()
_handle = None
_tried = False


def build(force: bool = False) -> str:
    """Compile the library in-tree with g++ (about a second)."""
    if force or not os.path.isfile(_LIB) or os.path.getmtime(_LIB) < os.path.getmtime(_SRC):
        tmp = _LIB + f".tmp{os.getpid()}"
        subprocess.run(["g++", "-O3", "-std=c++17", "-shared", "-fPIC", "-o", tmp, _SRC], check=True)
        os.replace(tmp, _LIB)
    return _LIB


def _declare(lib: ctypes.CDLL) -> None:
    vp, i32, u64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint64
    lib.xv_hash_chain.argtypes = [vp, i32, i32, u64, i32, vp]
    lib.xv_hash_chain.restype = None
    lib.xv_xxh64.argtypes = [vp, u64]
    lib.xv_xxh64.restype = u64
    lib.xv_fill_slots.argtypes = [vp, i32, i32, i32, vp]
    lib.xv_fill_slots.restype = None
    lib.xv_fill_decode.argtypes = [i32, vp, vp, vp, i32, i32, vp, vp, vp, vp, i32]
    lib.xv_fill_decode.restype = None
    lib.xv_st_open.argtypes = [ctypes.c_char_p]
    lib.xv_st_open.restype = vp
    lib.xv_st_header_len.argtypes = [vp]
    lib.xv_st_header_len.restype = u64
    lib.xv_st_file_size.argtypes = [vp]
    lib.xv_st_file_size.restype = u64
    lib.xv_st_header.argtypes = [vp, ctypes.c_char_p, u64]
    lib.xv_st_header.restype = u64
    lib.xv_st_read_block.argtypes = [vp, u64, u64, u64, u64, u64, u64, vp]
    lib.xv_st_read_block.restype = i32
    lib.xv_st_close.argtypes = [vp]
    lib.xv_st_close.restype = None


def get():
    """ctypes handle, building on first use if a compiler is present; None if unavailable."""
    global _handle, _tried
    if _handle is not None or _tried:
        return _handle
    with _lock:
        if _handle is not None or _tried:
            return _handle
        _tried = True
        if os.environ.get("XV_NO_HOSTLIB") == "1":
            return None
        try:
            path = build()
            lib = ctypes.CDLL(path)
            _declare(lib)
            _handle = lib
        except (OSError, subprocess.CalledProcessError, FileNotFoundError):
            _handle = None
    return _handle
