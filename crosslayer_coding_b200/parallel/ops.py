"""Thin control-plane wrappers over ``torch.distributed`` (NCCL on GPUs, Gloo on CPU).

Same call surface as the reference wrapper (clt/parallel/ops.py:18-117): every
function degrades to a single-process no-op when no process group exists.  The
data plane of the fused step (candidate exchange, reconstruction reduce) does
not go through here; it lives in ``parallel/symm.py`` and the CUDA kernels.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist
from torch.distributed import ProcessGroup, ReduceOp

SUM = ReduceOp.SUM
AVG = ReduceOp.AVG if hasattr(ReduceOp, "AVG") else None
PRODUCT = ReduceOp.PRODUCT
MIN = ReduceOp.MIN
MAX = ReduceOp.MAX


def is_dist_initialized_and_available() -> bool:
    return dist.is_available() and dist.is_initialized()


def get_rank(group: Optional[ProcessGroup] = None) -> int:
    return dist.get_rank(group=group) if is_dist_initialized_and_available() else 0


def get_world_size(group: Optional[ProcessGroup] = None) -> int:
    return dist.get_world_size(group=group) if is_dist_initialized_and_available() else 1


def is_main_process(group: Optional[ProcessGroup] = None) -> bool:
    return get_rank(group) == 0


def _single(group: Optional[ProcessGroup]) -> bool:
    return (not is_dist_initialized_and_available()) or get_world_size(group) == 1


def all_reduce(tensor: torch.Tensor, op=SUM, group: Optional[ProcessGroup] = None, async_op: bool = False):
    if _single(group):
        return None
    return dist.all_reduce(tensor, op=op, group=group, async_op=async_op)


def broadcast(tensor: torch.Tensor, src: int, group: Optional[ProcessGroup] = None, async_op: bool = False):
    if _single(group):
        return None
    return dist.broadcast(tensor, src=src, group=group, async_op=async_op)


def all_gather(
    tensor_list: List[torch.Tensor],
    tensor: torch.Tensor,
    group: Optional[ProcessGroup] = None,
    async_op: bool = False,
):
    if not is_dist_initialized_and_available():
        tensor_list[get_rank(group)] = tensor
        return None
    return dist.all_gather(tensor_list, tensor, group=group, async_op=async_op)


def barrier(group: Optional[ProcessGroup] = None) -> None:
    if not _single(group):
        dist.barrier(group=group)


def all_gather_cat(tensor: torch.Tensor, dim: int = 0, group: Optional[ProcessGroup] = None) -> torch.Tensor:
    """All-gather equally shaped tensors and concatenate along ``dim`` (no autograd)."""
    if _single(group):
        return tensor
    parts = [torch.empty_like(tensor) for _ in range(get_world_size(group))]
    dist.all_gather(parts, tensor.contiguous(), group=group)
    return torch.cat(parts, dim=dim)


class _ReduceSum(torch.autograd.Function):
    """Forward: all-reduce(SUM); backward: identity (row-parallel output reduce,
    reference clt/models/parallel.py:184-203)."""

    @staticmethod
    def forward(ctx, x: torch.Tensor, group):
        if _single(group):
            return x
        y = x.contiguous().clone()
        dist.all_reduce(y, op=SUM, group=group)
        return y

    @staticmethod
    def backward(ctx, g):
        return g, None


class _GatherCols(torch.autograd.Function):
    """Forward: all-gather along the last dim and drop padding; backward: take the
    local slice without communication (reference clt/models/parallel.py:99-181)."""

    @staticmethod
    def forward(ctx, x: torch.Tensor, group, full_dim: int):
        if _single(group):
            ctx.slice = None
            return x[..., :full_dim]
        w, r = get_world_size(group), get_rank(group)
        local = x.shape[-1]
        parts = [torch.empty_like(x) for _ in range(w)]
        dist.all_gather(parts, x.contiguous(), group=group)
        ctx.slice = (r * local, local, full_dim)
        return torch.cat(parts, dim=-1)[..., :full_dim]

    @staticmethod
    def backward(ctx, g):
        if ctx.slice is None:
            return g, None, None
        start, local, full_dim = ctx.slice
        end = min(start + local, full_dim)
        out = g.new_zeros(*g.shape[:-1], local)
        if end > start:
            out[..., : end - start] = g[..., start:end]
        return out, None, None


def reduce_sum(x: torch.Tensor, group: Optional[ProcessGroup] = None) -> torch.Tensor:
    return _ReduceSum.apply(x, group)


def gather_cols(x: torch.Tensor, full_dim: int, group: Optional[ProcessGroup] = None) -> torch.Tensor:
    return _GatherCols.apply(x, group, full_dim)
