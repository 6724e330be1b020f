"""Loader of the native IO library (``csrc/hdf5_lite.cpp`` -> ``_ext/libclt_io.so``).

Pure C ABI through ctypes: no torch or CUDA dependency, compiles with g++ in a few seconds.  The library is
built in-tree on first use when it is missing or older than its source.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
import threading
from pathlib import Path

_PKG = Path(__file__).resolve().parent.parent
SRC = _PKG / "csrc" / "hdf5_lite.cpp"
LIB = _PKG / "_ext" / "libclt_io.so"
_lock = threading.Lock()
_lib = None


def build() -> Path:
    LIB.parent.mkdir(parents=True, exist_ok=True)
    tmp = LIB.with_suffix(f".so.{os.getpid()}.tmp")
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-pthread", "-o", str(tmp), str(SRC), "-lz"]
    subprocess.run(cmd, check=True, capture_output=True)
    os.replace(tmp, LIB)
    return LIB


def load() -> ctypes.CDLL:
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not LIB.exists() or (SRC.exists() and SRC.stat().st_mtime > LIB.stat().st_mtime):
            build()
        lib = ctypes.CDLL(str(LIB))
        c = ctypes
        lib.clt_h5_last_error.restype = c.c_char_p
        lib.clt_h5w_open.restype = c.c_void_p
        lib.clt_h5w_open.argtypes = [c.c_char_p]
        lib.clt_h5w_add_dataset.restype = c.c_int
        lib.clt_h5w_add_dataset.argtypes = [c.c_void_p, c.c_char_p, c.c_char_p, c.c_void_p, c.c_uint64, c.c_uint64,
                                            c.c_int, c.c_uint64, c.c_int]
        lib.clt_h5w_close.restype = c.c_int
        lib.clt_h5w_close.argtypes = [c.c_void_p]
        lib.clt_h5r_open.restype = c.c_void_p
        lib.clt_h5r_open.argtypes = [c.c_char_p]
        lib.clt_h5r_close.restype = None
        lib.clt_h5r_close.argtypes = [c.c_void_p]
        lib.clt_h5r_list.restype = c.c_longlong
        lib.clt_h5r_list.argtypes = [c.c_void_p, c.c_char_p, c.c_char_p, c.c_longlong]
        lib.clt_h5r_dataset_info.restype = c.c_int
        lib.clt_h5r_dataset_info.argtypes = [c.c_void_p, c.c_char_p, c.POINTER(c.c_uint64)]
        lib.clt_h5r_read_rows.restype = c.c_int
        lib.clt_h5r_read_rows.argtypes = [c.c_void_p, c.c_char_p, c.c_void_p, c.c_uint64, c.c_void_p]
        lib.clt_h5r_scatter_rows.restype = c.c_int
        lib.clt_h5r_scatter_rows.argtypes = [c.c_void_p, c.c_char_p, c.c_int, c.c_void_p, c.c_void_p, c.c_uint64,
                                             c.c_void_p, c.c_uint64, c.c_int]
        lib.clt_h5r_read_all.restype = c.c_int
        lib.clt_h5r_read_all.argtypes = [c.c_void_p, c.c_char_p, c.c_void_p]
        _lib = lib
        return lib


def last_error() -> str:
    msg = load().clt_h5_last_error()
    return msg.decode("utf-8", "replace") if msg else "unknown error"
