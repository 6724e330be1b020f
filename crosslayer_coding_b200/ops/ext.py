"""Build and load the sm_100a extension (``csrc/*.cu`` + ``csrc/bindings.cpp``).

The shared object is built in-tree (``crosslayer_coding_b200/_ext``) so that it travels with
the source tree; loading prefers the prebuilt file and only compiles when it is missing or
older than its sources.  There is no silent fallback: on a CUDA machine a missing extension
raises, so a "passing" GPU run always ran the native kernels.
"""
from __future__ import annotations

import importlib.util
import os
import sys
import threading
from pathlib import Path
from typing import Optional

_PKG = Path(__file__).resolve().parent.parent
CSRC = _PKG / "csrc"
BUILD_DIR = _PKG / "_ext"
EXT_NAME = "clt_b200_ext"
# every kernel file is compiled for bf16 and, through a one-line wrapper that defines CLT_HALF, for fp16
KERNEL_FILES = ["encoder_gemm.cu", "theta_grad_gemm.cu", "select.cu", "decode.cu", "adam.cu", "comm.cu", "step.cu", "dense_gemm.cu", "aux.cu"]
SOURCES = ["bindings.cpp"] + KERNEL_FILES + [f"half/{name[:-3]}_h.cu" for name in KERNEL_FILES]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
]

_lock = threading.Lock()
_module = None
_debug_module = None
# CLT_DEBUG_BOUNDS=1 in the environment makes load() return the debug build: the same sources compiled with
# -DCLT_DEBUG_BOUNDS, where indices that come from data are checked before use and reported through the status word
DEBUG_ENV = "CLT_DEBUG_BOUNDS"
DEBUG_NAME = EXT_NAME + "_dbg"


def _so_path() -> Path:
    return BUILD_DIR / f"{EXT_NAME}.so"


def _sources() -> list:
    return [str(CSRC / s) for s in SOURCES if (CSRC / s).exists()]


def _stale() -> bool:
    so = _so_path()
    if not so.exists():
        return True
    newest = max(os.path.getmtime(p) for p in _sources() + [str(CSRC / "common.cuh"), str(CSRC / "clt_api.inc"), str(CSRC / "csr_static.h")])
    return newest > os.path.getmtime(so)


def build(verbose: bool = False, debug: bool = False):
    """Compile every CUDA source for sm_100a and import the result (``debug``: the index-checking build)."""
    from torch.utils import cpp_extension

    out_dir = BUILD_DIR / "dbg" if debug else BUILD_DIR
    out_dir.mkdir(parents=True, exist_ok=True)
    os.environ.setdefault("MAX_JOBS", "8")
    return cpp_extension.load(
        name=DEBUG_NAME if debug else EXT_NAME,
        sources=_sources(),
        extra_cflags=["-O3", "-std=c++17"],
        extra_cuda_cflags=NVCC_FLAGS + (["-DCLT_DEBUG_BOUNDS"] if debug else []),
        extra_include_paths=[str(CSRC)],
        build_directory=str(out_dir),
        with_cuda=True,
        verbose=verbose,
    )


def load_debug(allow_build: bool = True):
    """The index-checking build (``-DCLT_DEBUG_BOUNDS``), compiled on first use into ``_ext/dbg``."""
    global _debug_module
    with _lock:
        if _debug_module is not None:
            return _debug_module
        so = BUILD_DIR / "dbg" / f"{DEBUG_NAME}.so"
        newest = max(os.path.getmtime(p) for p in _sources() + [str(CSRC / "common.cuh"), str(CSRC / "clt_api.inc")])
        if so.exists() and os.path.getmtime(so) >= newest:
            import torch  # noqa: F401

            spec = importlib.util.spec_from_file_location(DEBUG_NAME, str(so))
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            sys.modules[DEBUG_NAME] = mod
            _debug_module = mod
            return mod
        if not allow_build:
            raise RuntimeError(f"{so} is missing or out of date; run __graft_entry__.build()")
        _debug_module = build(debug=True)
        return _debug_module


def _import_prebuilt():
    import torch  # noqa: F401  (libtorch symbols must be loaded first)

    spec = importlib.util.spec_from_file_location(EXT_NAME, str(_so_path()))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules[EXT_NAME] = mod
    return mod


def load(allow_build: bool = True):
    """Return the extension module, importing the prebuilt ``.so`` or compiling it."""
    global _module
    if os.environ.get(DEBUG_ENV, "") not in ("", "0"):
        return load_debug(allow_build)
    with _lock:
        if _module is not None:
            return _module
        if not _stale():
            try:
                _module = _import_prebuilt()
                return _module
            except Exception:
                if not allow_build:
                    raise
        if not allow_build:
            raise RuntimeError(f"{_so_path()} is missing or out of date; run __graft_entry__.build()")
        _module = build()
        return _module


def available() -> bool:
    """True when CUDA is usable; the extension is then mandatory for the fused ops."""
    import torch

    return torch.cuda.is_available()


def so_file() -> Optional[str]:
    return str(_so_path()) if _so_path().exists() else None
