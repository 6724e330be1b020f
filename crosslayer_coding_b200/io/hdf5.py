"""HDF5 chunk files without h5py: thin Python face of the native reader / writer.

The activation manifest format stores each chunk as ``chunk_{i}.hdf5`` (or ``.h5``) with groups
``layer_{id}`` holding 2-D datasets ``inputs`` and ``targets`` of shape ``(rows, d_model)`` and dtype
float32 / float16 / uint16, where uint16 carries bfloat16 *bit patterns*
(reference writer: clt/activation_generation/generator.py:768-799; readers:
clt/training/data/local_activation_store.py:212-236, clt_server/core/storage.py:101-173).

bfloat16 is written and read by reinterpretation.  (The reference hands a signed int16 view to a uint16
dataset, which HDF5 converts by value and clamps every negative bf16 number to zero, and its reader converts
the stored integers numerically; this implementation keeps the bits.)
"""
from __future__ import annotations

import ctypes
import os
import re
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import native

DT_CODES = {"float32": 0, "float16": 1, "uint16": 2, "int16": 3, "float64": 4, "uint8": 5, "int32": 6}
STORAGE_DTYPE = {"float32": np.float32, "float16": np.float16, "bfloat16": np.uint16}
TORCH_DTYPE = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}


def to_storage_array(t: torch.Tensor, activation_dtype: str) -> np.ndarray:
    """Tensor -> numpy array in the on-disk dtype (bf16 as uint16 bit patterns)."""
    t = t.detach().to("cpu")
    if activation_dtype == "bfloat16":
        return t.to(torch.bfloat16).contiguous().view(torch.int16).numpy().view(np.uint16)
    if activation_dtype == "float16":
        return t.to(torch.float16).contiguous().numpy()
    if activation_dtype == "float32":
        return t.to(torch.float32).contiguous().numpy()
    raise ValueError(f"unsupported activation dtype {activation_dtype!r}")


def from_storage_array(a: np.ndarray, activation_dtype: Optional[str] = None) -> torch.Tensor:
    """Inverse of :func:`to_storage_array`; uint16 data is bf16 bit patterns."""
    if a.dtype == np.uint16 or activation_dtype == "bfloat16":
        return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(torch.bfloat16)
    return torch.from_numpy(np.ascontiguousarray(a))


def _natural_key(name: str):
    m = re.search(r"(\d+)$", name)
    return (int(m.group(1)) if m else 1 << 60, name)


class H5Writer:
    def __init__(self, path: str):
        self._lib = native.load()
        self._h = self._lib.clt_h5w_open(os.fsencode(path))
        if not self._h:
            raise OSError(native.last_error())

    def add(self, group: str, name: str, array: np.ndarray, chunk_rows: int = 0, gzip_level: int = 0) -> None:
        a = np.ascontiguousarray(array)
        if a.ndim != 2:
            raise ValueError("datasets are 2-D (rows, d_model)")
        code = DT_CODES.get(a.dtype.name)
        if code is None:
            raise ValueError(f"unsupported numpy dtype {a.dtype}")
        rc = self._lib.clt_h5w_add_dataset(self._h, group.encode(), name.encode(), a.ctypes.data_as(ctypes.c_void_p),
                                           a.shape[0], a.shape[1], code, int(chunk_rows), int(gzip_level))
        if rc != 0:
            raise OSError(native.last_error())

    def close(self) -> None:
        if self._h:
            h, self._h = self._h, None
            if self._lib.clt_h5w_close(h) != 0:
                raise OSError(native.last_error())

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class H5Dataset:
    def __init__(self, file: "H5File", path: str):
        self.file, self.path = file, path
        info = (ctypes.c_uint64 * 8)()
        if file._lib.clt_h5r_dataset_info(file._h, path.encode(), info) != 0:
            raise KeyError(f"{path}: {native.last_error()}")
        self.rows, self.cols, self.elem_size = int(info[0]), int(info[1]), int(info[2])
        self.type_class, self.signed = int(info[3]), bool(info[4])
        self.layout, self.chunk_rows, self.compressed = int(info[5]), int(info[6]), bool(info[7])
        self.shape = (self.rows, self.cols)
        if self.type_class == 1:
            self.dtype = np.dtype({2: np.float16, 4: np.float32, 8: np.float64}[self.elem_size])
        else:
            base = {1: "u1", 2: "u2", 4: "u4", 8: "u8"}[self.elem_size]
            self.dtype = np.dtype(base.replace("u", "i") if self.signed else base)

    def read_rows(self, rows: Sequence[int]) -> np.ndarray:
        idx = np.ascontiguousarray(np.asarray(rows, dtype=np.uint64))
        out = np.empty((len(idx), self.cols), dtype=self.dtype)
        rc = self.file._lib.clt_h5r_read_rows(self.file._h, self.path.encode(), idx.ctypes.data_as(ctypes.c_void_p),
                                              len(idx), out.ctypes.data_as(ctypes.c_void_p))
        if rc != 0:
            raise OSError(native.last_error())
        return out

    def read_all(self) -> np.ndarray:
        out = np.empty(self.shape, dtype=self.dtype)
        if self.file._lib.clt_h5r_read_all(self.file._h, self.path.encode(), out.ctypes.data_as(ctypes.c_void_p)) != 0:
            raise OSError(native.last_error())
        return out

    def __getitem__(self, key) -> np.ndarray:
        if isinstance(key, slice):
            return self.read_rows(range(*key.indices(self.rows)))
        if isinstance(key, (list, np.ndarray, tuple)):
            return self.read_rows(key)
        if key is Ellipsis:
            return self.read_all()
        return self.read_rows([int(key)])[0]

    def __len__(self) -> int:
        return self.rows


class H5File:
    """Read-only view of an HDF5 file (memory mapped)."""

    def __init__(self, path: str):
        self._lib = native.load()
        self.path = path
        self._h = self._lib.clt_h5r_open(os.fsencode(path))
        if not self._h:
            raise OSError(f"{path}: {native.last_error()}")
        self._ds: Dict[str, H5Dataset] = {}

    def keys(self, group: str = "/") -> List[str]:
        need = self._lib.clt_h5r_list(self._h, group.encode(), None, 0)
        if need < 0:
            raise KeyError(f"{group}: {native.last_error()}")
        buf = ctypes.create_string_buffer(int(need))
        self._lib.clt_h5r_list(self._h, group.encode(), buf, need)
        return [n for n in buf.value.decode().split("\n") if n]

    def layer_groups(self) -> List[str]:
        """``layer_N`` groups in numeric order (layer_10 after layer_2)."""
        return sorted((k for k in self.keys() if k.startswith("layer_")), key=_natural_key)

    def dataset(self, path: str) -> H5Dataset:
        ds = self._ds.get(path)
        if ds is None:
            ds = self._ds[path] = H5Dataset(self, path)
        return ds

    def scatter_rows(self, paths: Sequence[str], rows: np.ndarray, dst_pos: np.ndarray, dst_ptrs: Sequence[int],
                     dst_row_stride: int, threads: int = 8) -> None:
        """Copy rows ``rows[i]`` of every dataset in ``paths`` to ``dst_ptrs[p] + dst_pos[i] * dst_row_stride``
        (raw addresses, e.g. into a pinned batch buffer) with ``threads`` native threads."""
        rows = np.ascontiguousarray(np.asarray(rows, dtype=np.uint64))
        pos = np.ascontiguousarray(np.asarray(dst_pos, dtype=np.int64))
        assert len(rows) == len(pos) and len(paths) == len(dst_ptrs)
        bases = (ctypes.c_void_p * len(dst_ptrs))(*[int(p) for p in dst_ptrs])
        rc = self._lib.clt_h5r_scatter_rows(self._h, "\n".join(paths).encode(), len(paths), rows.ctypes.data_as(ctypes.c_void_p),
                                            pos.ctypes.data_as(ctypes.c_void_p), len(rows), bases, int(dst_row_stride), int(threads))
        if rc != 0:
            raise OSError(native.last_error())

    def __getitem__(self, path: str) -> H5Dataset:
        return self.dataset(path)

    def __contains__(self, path: str) -> bool:
        try:
            self.dataset(path)
            return True
        except (KeyError, OSError):
            parts = [p for p in path.split("/") if p]
            try:
                return len(parts) == 1 and parts[0] in self.keys()
            except KeyError:
                return False

    def close(self) -> None:
        if self._h:
            h, self._h = self._h, None
            self._lib.clt_h5r_close(h)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def write_chunk_file(
    path: str,
    layers: Dict[int, Tuple[np.ndarray, np.ndarray]],
    compression: Optional[str] = None,
    chunk_rows: Optional[int] = None,
) -> None:
    """Write one activation chunk: ``layers[l] = (inputs, targets)`` arrays of shape ``(rows, d)`` in the
    on-disk dtype.  Datasets are row-chunked ``(min(rows, 16384), d)`` like the reference writer; ``gzip``
    compresses every chunk (``lz4`` is not an HDF5 core filter and is stored uncompressed)."""
    gz = 4 if compression == "gzip" else 0
    with H5Writer(path) as w:
        for l in sorted(layers):
            x, y = layers[l]
            rows = x.shape[0]
            cr = chunk_rows if chunk_rows is not None else min(max(rows, 1), 16384)
            w.add(f"layer_{l}", "inputs", x, chunk_rows=cr, gzip_level=gz)
            w.add(f"layer_{l}", "targets", y, chunk_rows=cr, gzip_level=gz)


def open_chunk(dataset_dir: str, chunk_id: int) -> H5File:
    """Open ``chunk_{id}.h5`` or ``chunk_{id}.hdf5`` (both spellings exist in the wild)."""
    for ext in (".h5", ".hdf5"):
        p = os.path.join(dataset_dir, f"chunk_{chunk_id}{ext}")
        if os.path.exists(p):
            return H5File(p)
    raise FileNotFoundError(f"chunk {chunk_id} not found in {dataset_dir}")
