"""Activation store over a local manifest dataset (reference: clt/training/data/local_activation_store.py:26-279).

Reads ``metadata.json``, ``index.bin`` (both layouts), ``norm_stats.json`` and ``chunk_{id}.hdf5|.h5`` from a
directory.  Rows are gathered straight from the memory-mapped chunk file by the native HDF5 reader (the
reference loads whole datasets into an LRU RAM cache and fancy-indexes them); open files are kept in a small
LRU.
"""
from __future__ import annotations

import logging
import os
from collections import OrderedDict
from typing import Any, Dict, Optional

import numpy as np

from ...io import hdf5, manifest
from .manifest_activation_store import ManifestActivationStore

logger = logging.getLogger(__name__)


class LocalActivationStore(ManifestActivationStore):
    def __init__(
        self,
        dataset_path: str,
        train_batch_size_tokens: int = 4096,
        device: Optional[Any] = None,
        dtype: Any = "bfloat16",
        rank: int = 0,
        world: int = 1,
        seed: int = 42,
        sampling_strategy: str = "sequential",
        normalization_method: str = "none",
        shard_data: bool = True,
        prefetch_batches: int = 2,
        auto_advance_epoch: bool = False,
        max_open_files: int = 128,
        shard_group=None,
    ):
        self.dataset_path = str(dataset_path)
        if not os.path.isdir(self.dataset_path):
            raise FileNotFoundError(f"activation dataset directory not found: {self.dataset_path}")
        self._files: "OrderedDict[int, hdf5.H5File]" = OrderedDict()
        self._max_open = max_open_files
        self._layer_names: Dict[int, list] = {}
        self._gather_threads = max(1, min(16, (os.cpu_count() or 4)))
        super().__init__(
            train_batch_size_tokens=train_batch_size_tokens, device=device, dtype=dtype, rank=rank, world=world,
            seed=seed, sampling_strategy=sampling_strategy, normalization_method=normalization_method,
            shard_data=shard_data, prefetch_batches=prefetch_batches, auto_advance_epoch=auto_advance_epoch,
            shard_group=shard_group,
        )

    def _load_metadata(self) -> Optional[Dict[str, Any]]:
        return manifest.load_metadata(self.dataset_path)

    def _load_manifest(self) -> Dict[int, int]:
        return manifest.read_index(os.path.join(self.dataset_path, "index.bin"), self.total_tokens)

    def _load_norm_stats(self) -> Optional[Dict[str, Any]]:
        return manifest.load_norm_stats(self.dataset_path)

    def _open(self, chunk_id: int) -> hdf5.H5File:
        f = self._files.get(chunk_id)
        if f is not None:
            self._files.move_to_end(chunk_id)
            return f
        f = hdf5.open_chunk(self.dataset_path, chunk_id)
        self._files[chunk_id] = f
        names = f.layer_groups()  # numeric order: layer_2 before layer_10
        if len(names) != self.num_layers:
            raise ValueError(f"chunk {chunk_id} holds {len(names)} layer groups, metadata says {self.num_layers}")
        self._layer_names[chunk_id] = names
        while len(self._files) > self._max_open:
            old_id, old = self._files.popitem(last=False)
            self._layer_names.pop(old_id, None)
            old.close()
        return f

    def _fetch_slice(self, chunk_id: int, row_indices: np.ndarray) -> bytes:
        f = self._open(chunk_id)
        parts = []
        for name in self._layer_names[chunk_id]:
            parts.append(f[f"{name}/inputs"].read_rows(row_indices).tobytes())
            parts.append(f[f"{name}/targets"].read_rows(row_indices).tobytes())
        return b"".join(parts)

    def _assemble(self, idx: np.ndarray, host) -> None:
        """Native batch assembly: every (layer, side) dataset's rows go straight from the mapped chunk file to their
        batch positions in the pinned ``[2, L, B, d]`` buffer, copied by a pool of native threads.  (The generic path
        of the base class builds the server's wire format first and re-orders it with numpy.)"""
        import random
        import time

        L, d = self.num_layers, self.d_model
        row_bytes = d * self.bytes_per_element
        side_stride = host.stride(0) * host.element_size()
        layer_stride = host.stride(1) * host.element_size()
        base = host.data_ptr()
        chunk_ids = idx[:, 0]
        for cid in np.unique(chunk_ids):
            pos = np.nonzero(chunk_ids == cid)[0].astype(np.int64)
            if self.row_shard is not None:  # tensor-parallel staging: this rank's token rows only
                pos = pos[(pos >= self.row_shard[0]) & (pos < self.row_shard[0] + self.row_shard[1])]
                if pos.size == 0:
                    continue
            rows = idx[pos, 1].astype(np.uint64)
            order = np.argsort(rows, kind="stable")  # ascending file order
            rows, pos = rows[order], pos[order]
            delay, last = 0.2, None
            for attempt in range(3):
                try:
                    f = self._open(int(cid))
                    names = self._layer_names[int(cid)]
                    paths, ptrs = [], []
                    for l, name in enumerate(names):
                        for side, key in enumerate(("inputs", "targets")):
                            ds = f[f"{name}/{key}"]
                            if ds.cols != d or ds.elem_size != self.bytes_per_element:
                                raise ValueError(f"chunk {cid}: {name}/{key} has rows of {ds.cols} x {ds.elem_size} bytes")
                            paths.append(f"{name}/{key}")
                            ptrs.append(base + side * side_stride + l * layer_stride)
                    f.scatter_rows(paths, rows, pos, ptrs, row_bytes, threads=self._gather_threads)
                    last = None
                    break
                except Exception as exc:  # noqa: BLE001 - every failure is retried, the last one is raised
                    last = exc
                    bad = self._files.pop(int(cid), None)
                    if bad is not None:
                        bad.close()
                    if attempt < 2:
                        time.sleep(delay + random.random() * 0.1 * delay)
                        delay *= 2
            if last is not None:
                raise RuntimeError(f"Rank {self.rank}: fetching chunk {cid} failed after 3 attempts: {last}") from last

    def close(self) -> None:
        super().close()
        for f in self._files.values():
            f.close()
        self._files.clear()
