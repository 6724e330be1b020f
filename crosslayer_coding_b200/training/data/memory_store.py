"""In-memory activation store: a pool of batches in pinned host memory, streamed to the device.

Used for synthetic benchmarks and tests, and as the simplest example of the store contract: every
``get_batch`` copies one ``[2, L, B, d]`` batch host->device on the staging stream (prefetching the
next one) and returns per-layer views of the stacked device tensor.
"""
from __future__ import annotations

from typing import Any, Dict, Optional

import torch

from .base_store import ActivationBatch, BaseActivationStore, LayerBatch
from .staging import DeviceStager


class InMemoryActivationStore(BaseActivationStore):
    def __init__(
        self,
        pool: torch.Tensor,
        device,
        loop: bool = True,
        prefetch: int = 2,
        shard_group=None,
    ):
        """``pool``: ``[N, 2, L, B, d]`` host tensor (inputs at index 0, targets at 1), already normalised.
        ``shard_group``: tensor-parallel group; each rank then copies ``1/W`` of every batch host->device and
        the rest arrives over NVLink (see ``DeviceStager``)."""
        assert pool.dim() == 5 and pool.shape[1] == 2, "pool must be [N, 2, L, B, d]"
        self.device = torch.device(device)
        self.pool = pool.pin_memory() if (self.device.type == "cuda" and not pool.is_pinned()) else pool
        self.num_batches, _, self.num_layers, self.train_batch_size_tokens, self.d_model = pool.shape
        self.layer_indices = list(range(self.num_layers))
        self.dtype = pool.dtype
        self.total_tokens = self.num_batches * self.train_batch_size_tokens
        self.loop = loop
        self.apply_normalization = False
        self.mean_tg: Dict[int, torch.Tensor] = {}
        self.std_tg: Dict[int, torch.Tensor] = {}
        self.stager = DeviceStager(tuple(pool.shape[1:]), pool.dtype, self.device, depth=max(2, prefetch + 2),  # one spare slot: a refill never has to wait for the slot the consumer released last
                                  
                                   shard_group=shard_group, row_dim=2)
        self.cursor = 0
        self.epoch = 0
        self._inflight = []  # (slot, pool index)
        self._last_slot: Optional[int] = None
        self.prefetch = max(1, prefetch) if self.device.type == "cuda" else 1
        self.h2d_bytes_per_batch = self.stager.bytes_per_batch          # whole job (sum over ranks)
        self.h2d_bytes_per_rank = self.stager.h2d_bytes_per_rank

    def _submit_next(self) -> bool:
        if self.cursor >= self.num_batches:
            if not self.loop:
                return False
            self.cursor = 0
            self.epoch += 1
        idx = self.cursor
        self.cursor += 1
        slot = self.stager._next
        self.stager._next = (slot + 1) % self.stager.depth
        self.stager.submit(slot, src=self.pool[idx])
        self._inflight.append((slot, idx))
        return True

    def get_batch(self) -> ActivationBatch:
        if self._last_slot is not None:
            self.stager.release(self._last_slot)
            self._last_slot = None
        while len(self._inflight) < self.prefetch and self._submit_next():
            pass
        if not self._inflight:
            raise StopIteration
        slot, _ = self._inflight.pop(0)
        dev = self.stager.acquire(slot)
        self._last_slot = slot
        # keep the pipeline full: queue the copy of the batch after this one now
        while len(self._inflight) < self.prefetch and self.stager.cuda and len(self._inflight) < self.stager.depth - 1:
            if not self._submit_next():
                break
        inputs = LayerBatch.from_stacked(dev[0], self.layer_indices)
        targets = LayerBatch.from_stacked(dev[1], self.layer_indices)
        return inputs, targets

    def state_dict(self) -> Dict[str, Any]:
        return {"store_type": type(self).__name__, "cursor": self.cursor - len(self._inflight), "epoch": self.epoch}

    def load_state_dict(self, state_dict: Dict[str, Any]) -> None:
        self._inflight.clear()
        self.cursor = int(state_dict.get("cursor", 0)) % max(1, self.num_batches)
        self.epoch = int(state_dict.get("epoch", 0))
