"""Stand-alone tensor-parallel linear layers (reference: clt/models/parallel.py:13-397).

``CrossLayerTranscoder`` keeps its encoders and decoders in packed, feature-major tensors and shards those
directly; these two modules offer the reference's layer-level API for code that builds its own models on the
same sharding rules:

* :class:`ColumnParallelLinear` — the output features are split over the ranks (weight ``[F_local, d_in]``,
  bias ``[F_local]``); ``forward`` returns the full ``[B, F]`` width on every rank by an all-gather whose
  backward is a local slice (no communication), or the local shard with ``gather_output=False``.
* :class:`RowParallelLinear` — the input features are split (weight ``[d_out, F_local]``), the partial
  products are summed across ranks (backward: identity) and the replicated bias is added after the reduce.

Both pad every shard to :func:`crosslayer_coding_b200.models.base.shard_width` features; padding columns hold
zeros and never reach the caller.  Initialisation follows the reference: column weights ``U(+-1/sqrt(F))``, row
weights ``U(+-1/sqrt(num_layers * d_model))`` when those are given, zero biases.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..models.base import mark_replicated, shard_width
from . import ops as pops


class _ParallelLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool, process_group, partition_dim: int,
                 device=None, dtype=None, init_bound: Optional[float] = None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.process_group = process_group
        self.world_size = pops.get_world_size(process_group) if process_group is not None else 1
        self.rank = pops.get_rank(process_group) if process_group is not None else 0
        self.partition_dim = partition_dim
        kw = dict(device=device, dtype=dtype)
        self.full_features = out_features if partition_dim == 0 else in_features
        self.local_features = shard_width(self.full_features, self.world_size)
        self.feature_start = self.rank * self.local_features
        self.valid_features = max(0, min(self.full_features, self.feature_start + self.local_features) - self.feature_start)
        if partition_dim == 0:  # column parallel: rows of the weight are output features
            bound = init_bound if init_bound is not None else 1.0 / math.sqrt(out_features)
            self.weight = nn.Parameter(torch.empty(self.local_features, in_features, **kw).uniform_(-bound, bound))
            self.bias_param = nn.Parameter(torch.zeros(self.local_features, **kw)) if bias else None
            pad_rows = slice(self.valid_features, None)
            with torch.no_grad():
                self.weight[pad_rows].zero_()
        else:  # row parallel: columns of the weight are input features
            bound = init_bound if init_bound is not None else 1.0 / math.sqrt(in_features)
            self.weight = nn.Parameter(torch.empty(out_features, self.local_features, **kw).uniform_(-bound, bound))
            self.bias_param = mark_replicated(nn.Parameter(torch.zeros(out_features, **kw))) if bias else None
            with torch.no_grad():
                self.weight[:, self.valid_features:].zero_()


class ColumnParallelLinear(_ParallelLinear):
    """``y = x W^T + b`` with the output features sharded over the ranks."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, process_group=None, gather_output: bool = True,
                 device=None, dtype=None, init_bound: Optional[float] = None):
        super().__init__(in_features, out_features, bias, process_group, 0, device, dtype, init_bound)
        self.gather_output = gather_output

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        local = F.linear(x, self.weight, self.bias_param)
        if not self.gather_output:
            return local[..., : self.valid_features]
        if self.world_size == 1:
            return local[..., : self.full_features]
        return pops.gather_cols(local, self.full_features, self.process_group)


class RowParallelLinear(_ParallelLinear):
    """``y = sum_ranks x_shard W_shard^T + b`` with the input features sharded over the ranks."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, process_group=None, input_is_parallel: bool = False,
                 device=None, dtype=None, init_bound: Optional[float] = None):
        super().__init__(in_features, out_features, bias, process_group, 1, device, dtype, init_bound)
        self.input_is_parallel = input_is_parallel

    def _split(self, x: torch.Tensor) -> torch.Tensor:
        """This rank's slice of a full-width input, zero-padded to the shard width."""
        piece = x[..., self.feature_start : self.feature_start + self.valid_features]
        pad = self.local_features - piece.shape[-1]
        return F.pad(piece, (0, pad)) if pad else piece

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not self.input_is_parallel and x.shape[-1] == self.full_features:
            x = self._split(x)
        elif x.shape[-1] != self.local_features:  # the valid width of a parallel input
            x = F.pad(x, (0, self.local_features - x.shape[-1]))
        partial = F.linear(x, self.weight)
        out = pops.reduce_sum(partial, self.process_group) if self.world_size > 1 else partial
        return out + self.bias_param if self.bias_param is not None else out
