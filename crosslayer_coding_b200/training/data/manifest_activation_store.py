"""Manifest-driven activation store with a pinned, prefetching host->device pipeline.

Contract and semantics follow the reference ``ManifestActivationStore``
(clt/training/data/manifest_activation_store.py:328-1088): the sampler yields ``(chunk_id, row_id)`` pairs,
rows are fetched per chunk in ascending row order (3 attempts with exponential backoff and jitter), a slice
is the raw bytes ``L0_in | L0_tg | L1_in | L1_tg ...`` in the stored dtype and is length-checked, rows go
back to sampler order, inputs and targets are normalised in fp32 (``mean_std``: ``(x - mean) / (std + 1e-6)``,
``sqrt_d_model``: ``x * sqrt(d)``) and cast to the store dtype; ``state_dict`` carries the sampler state.

What is different:

* a batch is assembled directly in one pinned ``[2, L, B, d]`` buffer and moved with one async copy on a
  side stream (the reference issues a synchronous pageable ``.to(device)`` per layer and chunk,
  manifest_activation_store.py:894-895); a background thread keeps ``prefetch_batches`` batches in flight
  (the reference has such a thread but no caller enables it);
* bf16 data is carried as bit patterns end to end;
* when the sampler is exhausted the store can start the next epoch (``advance_epoch``) instead of ending
  training after one pass.
"""
from __future__ import annotations

import logging
import queue
import random
import threading
import time
from abc import abstractmethod
from typing import Any, Dict, List, Optional, Tuple

import numpy as np
import torch

from .base_store import ActivationBatch, BaseActivationStore, LayerBatch
from .sampler import ChunkRowSampler
from .staging import DeviceStager

logger = logging.getLogger(__name__)

_NP_STORAGE = {"float32": np.float32, "float16": np.float16, "bfloat16": np.uint16}
_TORCH_VIEW = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}
_TORCH_OUT = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}


class ManifestActivationStore(BaseActivationStore):
    def __init__(
        self,
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
        shard_group=None,
    ):
        """``shard_group`` (tensor-parallel group, CUDA only): every rank assembles and copies only its ``1/W`` of
        each batch's token rows and the slices are all-gathered over NVLink (``DeviceStager``); the ranks must
        draw identical batches, i.e. ``shard_data=False``."""
        self.train_batch_size_tokens = int(train_batch_size_tokens)
        self.device = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
        dtype_name = str(dtype).replace("torch.", "")
        self.dtype = _TORCH_OUT.get(dtype_name, torch.float32) if not isinstance(dtype, torch.dtype) else dtype
        self.rank, self.world, self.seed = rank, world, seed
        self.sampling_strategy = sampling_strategy
        from ...config import canonical_normalization

        self.normalization_method = canonical_normalization(normalization_method)
        if self.normalization_method not in ("none", "mean_std", "sqrt_d_model"):
            raise ValueError(f"Invalid normalization_method: {normalization_method}")
        self.shard_data = shard_data
        self.prefetch_batches = max(1, int(prefetch_batches))
        self.auto_advance_epoch = auto_advance_epoch
        self.epoch = 0

        meta = self._load_metadata()
        if not meta:
            raise RuntimeError("could not load dataset metadata")
        self.metadata = meta
        self.num_layers = int(meta["num_layers"])
        self.d_model = int(meta["d_model"])
        self.total_tokens = int(meta["total_tokens"])
        self.chunk_tokens = int(meta.get("chunk_tokens", -1))
        self.stored_dtype = str(meta.get("dtype", "bfloat16")).replace("torch.", "")
        if self.stored_dtype not in _NP_STORAGE:
            raise ValueError(f"unsupported stored dtype {self.stored_dtype!r}")
        self.bytes_per_element = np.dtype(_NP_STORAGE[self.stored_dtype]).itemsize
        self.layer_indices = list(range(self.num_layers))
        self.chunk_sizes = self._load_manifest()
        if not self.chunk_sizes:
            raise RuntimeError("manifest is empty")
        self.num_chunks = max(self.chunk_sizes) + 1

        self.apply_normalization = self.normalization_method != "none"
        self.mean_in: Dict[int, torch.Tensor] = {}
        self.std_in: Dict[int, torch.Tensor] = {}
        self.mean_tg: Dict[int, torch.Tensor] = {}
        self.std_tg: Dict[int, torch.Tensor] = {}
        self._norm_pack: Optional[Tuple[torch.Tensor, torch.Tensor]] = None
        if self.normalization_method == "mean_std":
            self._prep_norm(self._load_norm_stats())

        self.sampler = ChunkRowSampler(
            self.chunk_sizes, self.num_chunks, self.train_batch_size_tokens, seed, self.epoch, rank, world,
            sampling_strategy, shard_data,
        )
        shape = (2, self.num_layers, self.train_batch_size_tokens, self.d_model)
        self._storage_torch = _TORCH_VIEW[self.stored_dtype]
        # slots: prefetch in the queue + one being assembled + one held by the consumer
        use_shard = shard_group if (not shard_data or world == 1) else None
        # sharded staging keeps two batches' copy + gather queued ahead of the consumer: more slots in flight
        self.stager = DeviceStager(shape, self._storage_torch, self.device, depth=self.prefetch_batches + (4 if use_shard is not None else 2),
                                   shard_group=use_shard, row_dim=2)
        self.row_shard = None  # (first row, row count) of the batch positions this rank assembles
        if getattr(self.stager, "shard_world", 1) > 1:
            self.row_shard = (self.stager.shard_rank * self.stager.rows_per_rank, self.stager.rows_per_rank)
        self._submitted: list = []  # sharded staging: slots whose copy + gather the consumer thread has queued
        self.h2d_bytes_per_batch = self.stager.bytes_per_batch
        self._queue: "queue.Queue" = queue.Queue(maxsize=self.prefetch_batches)
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._last_slot: Optional[int] = None
        self._consumed_state: Optional[Dict[str, Any]] = None
        self._failed_once = False

    # ------------------------------------------------------------------ abstract hooks
    @abstractmethod
    def _load_metadata(self) -> Optional[Dict[str, Any]]: ...

    @abstractmethod
    def _load_manifest(self) -> Dict[int, int]: ...

    @abstractmethod
    def _load_norm_stats(self) -> Optional[Dict[str, Any]]: ...

    @abstractmethod
    def _fetch_slice(self, chunk_id: int, row_indices: np.ndarray) -> bytes: ...

    # ------------------------------------------------------------------ normalisation
    def _prep_norm(self, stats: Optional[Dict[str, Any]]) -> None:
        if not stats:
            logger.warning("Rank %d: normalization 'mean_std' requested but no norm_stats found; disabling", self.rank)
            self.apply_normalization = False
            return
        L, d = self.num_layers, self.d_model
        mean = torch.zeros(2, L, 1, d)
        std = torch.ones(2, L, 1, d)
        for l in range(L):
            entry = stats.get(str(l)) or stats.get(l)
            if entry is None:
                logger.warning("norm stats miss layer %d; disabling normalization", l)
                self.apply_normalization = False
                return
            for side, key in enumerate(("inputs", "targets")):
                mean[side, l, 0] = torch.tensor(entry[key]["mean"], dtype=torch.float32)
                std[side, l, 0] = torch.tensor(entry[key]["std"], dtype=torch.float32) + 1e-6
        mean, std = mean.to(self.device), std.to(self.device)
        self._norm_pack = (mean, std)
        for l in range(L):
            self.mean_in[l], self.std_in[l] = mean[0, l], std[0, l]
            self.mean_tg[l], self.std_tg[l] = mean[1, l], std[1, l]

    def _normalise(self, raw: torch.Tensor) -> torch.Tensor:
        """``raw``: ``[2, L, B, d]`` in the stored dtype on the device -> normalised, store dtype."""
        if not self.apply_normalization:
            return raw if raw.dtype == self.dtype else raw.to(self.dtype)
        if raw.is_cuda and self.dtype in (torch.bfloat16, torch.float16) and self.d_model % 8 == 0:
            # one pass on the device: (x - mean) / std (or x * sqrt(d)) and the cast to the training type
            from ...ops import ext

            out = torch.empty(raw.shape, dtype=self.dtype, device=raw.device)
            raw_c = raw.contiguous()
            if self.normalization_method == "mean_std" and self._norm_pack is not None:
                if getattr(self, "_norm_flat", None) is None:
                    mean, std = self._norm_pack
                    self._norm_flat = (mean.reshape(-1, self.d_model).contiguous(), (1.0 / std).reshape(-1, self.d_model).contiguous())
                ext.load().normalize_cast(raw_c, out, self._norm_flat[0], self._norm_flat[1], raw_c.shape[-2], 1.0)
            elif self.normalization_method == "sqrt_d_model":
                ext.load().normalize_cast(raw_c, out, None, None, 0, float(self.d_model ** 0.5))
            else:
                return raw if raw.dtype == self.dtype else raw.to(self.dtype)
            return out
        x = raw.float()
        if self.normalization_method == "mean_std" and self._norm_pack is not None:
            mean, std = self._norm_pack
            x = (x - mean) / std
        elif self.normalization_method == "sqrt_d_model":
            x = x * (self.d_model ** 0.5)
        return x.to(self.dtype)

    # ------------------------------------------------------------------ fetching
    def _fetch_with_retry(self, chunk_id: int, rows_sorted: np.ndarray) -> bytes:
        expected = len(rows_sorted) * self.d_model * self.bytes_per_element * 2 * self.num_layers
        delay = 0.2
        last: Optional[Exception] = None
        for attempt in range(3):
            try:
                raw = self._fetch_slice(chunk_id, rows_sorted)
                if len(raw) != expected:
                    raise ValueError(f"chunk {chunk_id}: got {len(raw)} bytes, expected {expected}")
                return raw
            except Exception as exc:  # noqa: BLE001 - every failure is retried, the last one is raised
                last = exc
                if attempt < 2:
                    time.sleep(delay + random.random() * 0.1 * delay)
                    delay *= 2
        raise RuntimeError(f"Rank {self.rank}: fetching chunk {chunk_id} failed after 3 attempts: {last}") from last

    def _assemble(self, idx: np.ndarray, host: torch.Tensor) -> None:
        """Fill the pinned ``[2, L, B, d]`` buffer ``host`` with the rows ``idx`` (``[B, 2]``) in sampler order."""
        L, d = self.num_layers, self.d_model
        view = host.view(torch.int16) if self.stored_dtype == "bfloat16" else host
        dst = view.numpy()  # shares memory with the pinned tensor
        if self.stored_dtype == "bfloat16":
            dst = dst.view(np.uint16)
        np_dt = _NP_STORAGE[self.stored_dtype]
        chunk_ids = idx[:, 0]
        for cid in np.unique(chunk_ids):
            pos = np.nonzero(chunk_ids == cid)[0]
            if self.row_shard is not None:
                pos = pos[(pos >= self.row_shard[0]) & (pos < self.row_shard[0] + self.row_shard[1])]
                if pos.size == 0:
                    continue
            rows = idx[pos, 1].astype(np.int64)
            order = np.argsort(rows, kind="stable")
            rows_sorted = rows[order]
            raw = self._fetch_with_retry(int(cid), rows_sorted)
            block = np.frombuffer(raw, dtype=np_dt).reshape(L, 2, len(rows_sorted), d)
            target_pos = pos[order]  # slice row j belongs to batch position target_pos[j]
            dst[0][:, target_pos, :] = block[:, 0]
            dst[1][:, target_pos, :] = block[:, 1]

    # ------------------------------------------------------------------ pipeline
    def _producer(self) -> None:
        try:
            while not self._stop.is_set():
                try:
                    idx = next(self.sampler)
                except StopIteration:
                    if self.auto_advance_epoch:
                        self.epoch += 1
                        self.sampler.set_epoch(self.epoch)
                        continue
                    self._producer_done = True
                    self._queue.put(("end", None, None))
                    return
                state_after = {"epoch": self.epoch, "sampler_state": self.sampler.state_dict()}
                try:
                    slot, host = self.stager.host_slot()
                    self._assemble(idx, host)
                except Exception as exc:  # noqa: BLE001
                    if not self._failed_once:  # skip one failed batch, stop at the second (reference policy)
                        self._failed_once = True
                        logger.warning("Rank %d: skipping a batch that could not be fetched: %s", self.rank, exc)
                        continue
                    self._producer_done = True
                    self._queue.put(("error", exc, None))
                    return
                if self.row_shard is None:
                    self.stager.submit(slot)  # sharded staging queues its copy + all-gather on the consumer's thread
                while not self._stop.is_set():
                    try:
                        self._queue.put(("batch", slot, state_after), timeout=0.1)
                        break
                    except queue.Full:
                        continue
        except Exception as exc:  # noqa: BLE001
            self._producer_done = True
            self._queue.put(("error", exc, None))

    def _ensure_thread(self) -> None:
        # a producer that ran to the end of the epoch (or failed) has left its final message in the queue: starting another
        # one before the consumer has read it would queue a second, stale one
        if getattr(self, "_producer_done", False):
            return
        if self._thread is None or not self._thread.is_alive():
            self._stop.clear()
            self._thread = threading.Thread(target=self._producer, name="clt-activation-prefetch", daemon=True)
            self._thread.start()

    def get_batch(self) -> ActivationBatch:
        if self._last_slot is not None:
            self.stager.release(self._last_slot)
            self._last_slot = None
        if getattr(self, "_epoch_ended", False):
            raise StopIteration  # until advance_epoch() / load_state_dict()
        self._ensure_thread()
        if self.row_shard is not None:
            # collectives are issued from this thread only, in the same order on every rank: queue the copy + gather
            # of this batch (if not done by the look-ahead of the previous call) and of the next one if it is ready
            if not self._submitted:
                self._submitted.append(self._queue.get())
                if self._submitted[-1][0] == "batch":
                    self.stager.submit(self._submitted[-1][1])
            kind, payload, state = self._submitted.pop(0)
        else:
            kind, payload, state = self._queue.get()
        if kind == "end":
            self._thread = None
            self._epoch_ended = True
            raise StopIteration
        if kind == "error":
            self._thread = None
            self._producer_done = False  # the next call starts a new producer at the sampler's position
            raise payload
        slot = payload
        # two batches ahead: the gather of a batch queued only one step ahead tends to sit behind the step's long
        # kernels and to finish after the step does
        while self.row_shard is not None and len(self._submitted) < 2 and (not self._submitted or self._submitted[-1][0] == "batch"):
            nxt = self._queue.get()
            self._submitted.append(nxt)
            if nxt[0] == "batch":
                self.stager.submit(nxt[1])
        raw = self.stager.acquire(slot)
        self._last_slot = slot
        self._consumed_state = state
        batch = self._normalise(raw)
        inputs = LayerBatch.from_stacked(batch[0], self.layer_indices)
        targets = LayerBatch.from_stacked(batch[1], self.layer_indices)
        return inputs, targets

    def advance_epoch(self) -> None:
        self._shutdown_thread()
        self.epoch += 1
        self.sampler.set_epoch(self.epoch)

    def _shutdown_thread(self) -> None:
        self._stop.set()
        if self._thread is not None:
            while self._thread.is_alive():
                try:
                    self._queue.get_nowait()
                except queue.Empty:
                    pass
                self._thread.join(timeout=0.05)
        self._thread = None
        while True:
            try:
                self._queue.get_nowait()
            except queue.Empty:
                break
        self._stop.clear()
        self._producer_done = False
        self._epoch_ended = False
        self._submitted = []

    # ------------------------------------------------------------------ state
    def state_dict(self) -> Dict[str, Any]:
        # the sampler runs ahead of the consumer by the prefetch depth: report the state as of the last
        # batch that was handed out, so a resumed run continues with the next unseen batch
        if self._consumed_state is not None:
            sampler_state, epoch = self._consumed_state["sampler_state"], self._consumed_state["epoch"]
        else:
            sampler_state, epoch = self.sampler.state_dict(), self.epoch
        return {
            "store_type": type(self).__name__,
            "epoch": epoch,
            "seed": self.seed,
            "sampling_strategy": self.sampling_strategy,
            "shard_data": self.shard_data,
            "sampler_state": sampler_state,
        }

    def load_state_dict(self, state_dict: Dict[str, Any]) -> None:
        self._shutdown_thread()
        self.seed = int(state_dict.get("seed", self.seed))
        self.epoch = int(state_dict.get("epoch", 0))
        self.sampler.seed = self.seed
        self.sampler.set_epoch(self.epoch)
        if state_dict.get("sampler_state"):
            self.sampler.load_state_dict(state_dict["sampler_state"])
        self._consumed_state = None

    def close(self) -> None:
        self._shutdown_thread()

    def __len__(self) -> int:
        return len(self.sampler)
