"""Activation store backed by the HTTP slice server (reference: clt/training/data/remote_activation_store.py:36-173).

Protocol (see ``crosslayer_coding_b200.server``): ``GET datasets/{id}/info`` (metadata), ``GET .../manifest``
(raw ``index.bin``), ``GET .../norm_stats`` (404 tolerated), ``POST .../slice?chunk=N`` with ``{"rows": [...]}``
returning the raw slice bytes.  The dataset id is URL-quoted with no safe characters.  Unlike the reference
client, both manifest layouts are understood (the reference's generator uploads the 3-field layout its own
client cannot parse).
"""
from __future__ import annotations

import json
import logging
import time
from typing import Any, Dict, Optional
from urllib.parse import quote, urljoin

import numpy as np
import requests

from ...io import manifest
from .manifest_activation_store import ManifestActivationStore

logger = logging.getLogger(__name__)


class RemoteActivationStore(ManifestActivationStore):
    def __init__(
        self,
        server_url: str,
        dataset_id: str,
        train_batch_size_tokens: int = 4096,
        device: Optional[Any] = None,
        dtype: Any = "bfloat16",
        rank: int = 0,
        world: int = 1,
        seed: int = 42,
        timeout: int = 60,
        sampling_strategy: str = "sequential",
        normalization_method: str = "none",
        shard_data: bool = True,
        prefetch_batches: int = 2,
        auto_advance_epoch: bool = False,
        max_retries: int = 3,
    ):
        self.server = server_url.rstrip("/") + "/"
        self.did_raw = dataset_id
        self.did_enc = quote(dataset_id, safe="")
        self.timeout = timeout
        self.max_retries = max(1, max_retries)
        self._session = requests.Session()
        super().__init__(
            train_batch_size_tokens=train_batch_size_tokens, device=device, dtype=dtype, rank=rank, world=world,
            seed=seed, sampling_strategy=sampling_strategy, normalization_method=normalization_method,
            shard_data=shard_data, prefetch_batches=prefetch_batches, auto_advance_epoch=auto_advance_epoch,
        )

    def _url(self, tail: str) -> str:
        return urljoin(self.server, f"datasets/{self.did_enc}/{tail}")

    def _get(self, tail: str, tolerate_404: bool = False) -> Optional[requests.Response]:
        last: Optional[Exception] = None
        for attempt in range(self.max_retries):
            try:
                resp = requests.get(self._url(tail), timeout=self.timeout)
                if tolerate_404 and resp.status_code == 404:
                    return None
                resp.raise_for_status()
                return resp
            except requests.RequestException as exc:
                last = exc
                if attempt + 1 < self.max_retries:
                    time.sleep(2 * (2 ** attempt))
        raise RuntimeError(f"GET {self._url(tail)} failed after {self.max_retries} attempts: {last}") from last

    def _load_metadata(self) -> Optional[Dict[str, Any]]:
        resp = self._get("info")
        return resp.json() if resp is not None else None

    def _load_manifest(self) -> Dict[int, int]:
        resp = self._get("manifest")
        return manifest.parse_index_bytes(resp.content, self.total_tokens)

    def _load_norm_stats(self) -> Optional[Dict[str, Any]]:
        resp = self._get("norm_stats", tolerate_404=True)
        return resp.json() if resp is not None else None

    def _fetch_slice(self, chunk_id: int, row_indices: np.ndarray) -> bytes:
        url = self._url("slice") + f"?chunk={int(chunk_id)}"
        resp = requests.post(url, json={"rows": [int(r) for r in row_indices]}, timeout=self.timeout)
        resp.raise_for_status()
        return resp.content
