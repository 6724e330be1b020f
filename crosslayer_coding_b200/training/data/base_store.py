"""Activation-store interface (reference: clt/training/data/base_store.py:12-56).

A store is an iterator of ``(inputs, targets)`` where each is a mapping ``layer -> [B, d]`` tensor on the
training device.  Stores of this framework return :class:`LayerBatch` mappings whose per-layer tensors are
views of one stacked ``[L, B, d]`` tensor (``.stacked``), which is what the fused step consumes without
any re-packing.
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any, Dict, Iterator, Optional, Tuple

import torch


class LayerBatch(dict):
    """``{layer: [B, d] view}`` plus the stacked ``[L, B, d]`` tensor the views come from."""

    stacked: Optional[torch.Tensor] = None

    @classmethod
    def from_stacked(cls, stacked: torch.Tensor, layers) -> "LayerBatch":
        out = cls({l: stacked[i] for i, l in enumerate(layers)})
        out.stacked = stacked
        return out


ActivationBatch = Tuple[Dict[int, torch.Tensor], Dict[int, torch.Tensor]]


class BaseActivationStore(ABC):
    layer_indices: list
    d_model: int
    dtype: torch.dtype
    device: torch.device
    train_batch_size_tokens: int
    total_tokens: int

    @abstractmethod
    def get_batch(self) -> ActivationBatch: ...

    @abstractmethod
    def state_dict(self) -> Dict[str, Any]: ...

    @abstractmethod
    def load_state_dict(self, state_dict: Dict[str, Any]) -> None: ...

    def close(self) -> None:
        pass

    def __iter__(self) -> Iterator[ActivationBatch]:
        return self

    def __next__(self) -> ActivationBatch:
        return self.get_batch()

    def __len__(self) -> int:
        total = getattr(self, "total_tokens", 0)
        batch = getattr(self, "train_batch_size_tokens", 0)
        if not total or not batch:
            return 0
        return (total + batch - 1) // batch
