"""Abstract transcoder interface (reference: clt/models/base.py:13-101)."""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Dict, Optional

import torch
import torch.nn as nn

from ..config import CLTConfig


def mark_replicated(param: torch.nn.Parameter) -> torch.nn.Parameter:
    """Tag a parameter whose value is identical on every tensor-parallel rank
    (reference: clt/models/__init__.py:4-12)."""
    setattr(param, "_is_replicated", True)
    return param


def is_replicated(param: torch.nn.Parameter) -> bool:
    return getattr(param, "_is_replicated", False)


def shard_width(num_features: int, world_size: int) -> int:
    """Padded number of features per tensor-parallel rank: ``ceil(F / W)`` like the reference
    (clt/models/parallel.py:53-77), rounded up to a multiple of 8 when sharded so that every shard satisfies
    the 16-byte alignment of the fused kernels' vector loads and TMA boxes; the padding columns hold zeros and
    sit behind the last valid feature of the rank."""
    local = -(-num_features // max(1, world_size))
    if world_size > 1:
        local = (local + 7) // 8 * 8
    return local


class BaseTranscoder(nn.Module, ABC):
    def __init__(self, config: CLTConfig):
        super().__init__()
        self.config = config

    @abstractmethod
    def encode(self, x: torch.Tensor, layer_idx: int) -> torch.Tensor: ...

    @abstractmethod
    def decode(self, a: Dict[int, torch.Tensor], layer_idx: int) -> torch.Tensor: ...

    @abstractmethod
    def forward(self, inputs: Dict[int, torch.Tensor]) -> Dict[int, torch.Tensor]: ...

    def save(self, path: str) -> None:
        """``torch.save`` of ``{"config", "state_dict"}`` like the reference (base.py:65-78)."""
        torch.save({"config": self.config.to_dict(), "state_dict": self.state_dict()}, path)

    @classmethod
    def load(cls, path: str, device: Optional[torch.device] = None):
        """Load a single-process checkpoint written by :meth:`save`.  (The reference's
        classmethod cannot construct a CLT because it omits the process group,
        base.py:81-101; this one builds a single-rank model.)"""
        blob = torch.load(path, map_location=device or "cpu", weights_only=False)
        config = CLTConfig.from_dict(blob["config"])
        model = cls(config, process_group=None, device=device)  # type: ignore[call-arg]
        model.load_state_dict(blob["state_dict"])
        return model
