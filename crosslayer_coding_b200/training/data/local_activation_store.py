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
    ):
        self.dataset_path = str(dataset_path)
        if not os.path.isdir(self.dataset_path):
            raise FileNotFoundError(f"activation dataset directory not found: {self.dataset_path}")
        self._files: "OrderedDict[int, hdf5.H5File]" = OrderedDict()
        self._max_open = max_open_files
        self._layer_names: Dict[int, list] = {}
        super().__init__(
            train_batch_size_tokens=train_batch_size_tokens, device=device, dtype=dtype, rank=rank, world=world,
            seed=seed, sampling_strategy=sampling_strategy, normalization_method=normalization_method,
            shard_data=shard_data, prefetch_batches=prefetch_batches, auto_advance_epoch=auto_advance_epoch,
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

    def close(self) -> None:
        super().close()
        for f in self._files.values():
            f.close()
        self._files.clear()
