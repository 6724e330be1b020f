"""Activation functions of the transcoder as plain PyTorch (the CPU oracle and the
autograd path).  The fused sm_100a step computes the same quantities without ever
materialising ``[B, L*F]`` tensors; its tests compare against this file.

Semantics follow the single-GPU reference path:

* BatchTopK keeps the top ``min(k*B, numel)`` entries of the flattened ranking
  tensor and passes the *original* values through (clt/models/activations.py:11-96).
* TokenTopK keeps ``k`` entries per row; ``k < 1`` is a fraction of the row
  (clt/models/activations.py:101-172).
* JumpReLU gates at ``x >= theta`` with a rectangle-kernel straight-through
  gradient for ``theta`` (clt/models/activations.py:175-220).
* The global variants rank on per-layer batch z-scores
  ``(x - mean_B) / (std_B + 1e-6)`` (clt/models/activations.py:281-357).

Deliberate difference: ties are broken by the lowest flat index
``b*(L*F) + l*F + f`` so that the selection is identical for every tensor-parallel
world size (``torch.topk`` leaves the tie order unspecified), and the
tensor-parallel path selects exactly ``k*B`` entries (the reference's
"local-global" variant keeps about ``k*B/W``, clt/models/activations_local_global.py:84-146).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..parallel import ops as pops

ZSCORE_EPS = 1e-6


# ---------------------------------------------------------------------------
# mask construction
# ---------------------------------------------------------------------------
def _topk_flat_mask(rank: torch.Tensor, k_total: int) -> torch.Tensor:
    """Boolean mask of the ``k_total`` largest entries of ``rank`` (any shape), ties
    resolved towards the lower flat index."""
    n = rank.numel()
    mask = torch.zeros(n, dtype=torch.bool, device=rank.device)
    if k_total <= 0 or n == 0:
        return mask.view_as(rank)
    if k_total >= n:
        return torch.ones_like(mask).view_as(rank)
    flat = rank.reshape(-1)
    # k-th largest value by partial selection, then the ties at that value in index order: the same set as a
    # stable descending sort, without sorting the (mostly discarded) rest
    kth = torch.topk(flat, k_total, sorted=False).values.min()
    if torch.isnan(kth):
        _, order = torch.sort(flat, descending=True, stable=True)
        mask[order[:k_total]] = True
        return mask.view_as(rank)
    torch.gt(flat, kth, out=mask)
    need = k_total - int(mask.sum())
    if need > 0:
        mask[(flat == kth).nonzero(as_tuple=True)[0][:need]] = True
    return mask.view_as(rank)


class BatchTopK(torch.autograd.Function):
    @staticmethod
    def _compute_mask(x: torch.Tensor, k_per_token: int, x_for_ranking: Optional[torch.Tensor] = None) -> torch.Tensor:
        if x.numel() == 0:
            return torch.zeros_like(x, dtype=torch.bool)
        batch = x.size(0)
        k_total = min(int(k_per_token) * batch, x.numel())
        rank = x if x_for_ranking is None else x_for_ranking
        return _topk_flat_mask(rank, k_total).view_as(x)

    @staticmethod
    def forward(ctx, x, k, straight_through: bool = True, x_for_ranking: Optional[torch.Tensor] = None):
        mask = BatchTopK._compute_mask(x, int(k), x_for_ranking)
        ctx.save_for_backward(mask)
        return x * mask.to(x.dtype)

    @staticmethod
    def backward(ctx, grad_output):
        (mask,) = ctx.saved_tensors
        # Both the straight-through and the "plain" variants of the reference
        # pass the gradient at the kept positions only.
        return grad_output * mask.to(grad_output.dtype), None, None, None


def resolve_token_k(k_float: float, row_width: int) -> int:
    if k_float <= 0:
        return 0
    if k_float < 1:
        k = int(math.ceil(k_float * row_width))
    else:
        k = int(k_float)
    return max(0, min(k, row_width))


class TokenTopK(torch.autograd.Function):
    @staticmethod
    def _compute_mask(x: torch.Tensor, k_float: float, x_for_ranking: Optional[torch.Tensor] = None) -> torch.Tensor:
        if x.numel() == 0:
            return torch.zeros_like(x, dtype=torch.bool)
        width = x.size(-1)
        k = resolve_token_k(float(k_float), width)
        if k == 0:
            return torch.zeros_like(x, dtype=torch.bool)
        if k >= width:
            return torch.ones_like(x, dtype=torch.bool)
        rank = x if x_for_ranking is None else x_for_ranking
        kth = torch.topk(rank, k, dim=-1, sorted=False).values.amin(dim=-1, keepdim=True)
        if bool(torch.isnan(kth).any()):
            _, order = torch.sort(rank, dim=-1, descending=True, stable=True)
            mask = torch.zeros_like(x, dtype=torch.bool)
            mask.scatter_(-1, order[..., :k], True)
            return mask
        # strictly larger entries, then the ties at the k-th value in index order (what a stable sort keeps)
        mask = rank > kth
        tie = rank == kth
        need = k - mask.sum(dim=-1, keepdim=True)
        mask |= tie & (tie.cumsum(dim=-1) <= need)
        return mask

    @staticmethod
    def forward(ctx, x, k, straight_through: bool = True, x_for_ranking: Optional[torch.Tensor] = None):
        mask = TokenTopK._compute_mask(x, float(k), x_for_ranking)
        ctx.save_for_backward(mask)
        return x * mask.to(x.dtype)

    @staticmethod
    def backward(ctx, grad_output):
        (mask,) = ctx.saved_tensors
        return grad_output * mask.to(grad_output.dtype), None, None, None


class _MaskSTE(torch.autograd.Function):
    """``x * mask`` with the gradient passed at kept positions (mask given)."""

    @staticmethod
    def forward(ctx, x, mask):
        ctx.save_for_backward(mask)
        return x * mask.to(x.dtype)

    @staticmethod
    def backward(ctx, g):
        (mask,) = ctx.saved_tensors
        return g * mask.to(g.dtype), None


class JumpReLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input: torch.Tensor, threshold: torch.Tensor, bandwidth: float):
        ctx.save_for_backward(input, threshold)
        ctx.bandwidth = float(bandwidth)
        # The gate is promoted to fp32 like the reference does (activations.py:177-180).
        return (input >= threshold).float() * input

    @staticmethod
    def backward(ctx, grad_output):
        input, threshold = ctx.saved_tensors
        bw = ctx.bandwidth
        grad_input = grad_threshold = None
        if ctx.needs_input_grad[0]:
            grad_input = grad_output * (input >= threshold).to(grad_output.dtype)
        if ctx.needs_input_grad[1]:
            window = ((input - threshold).abs() <= bw / 2).to(grad_output.dtype)
            per_elem = grad_output * (-(input.to(grad_output.dtype)) / bw) * window
            if threshold.dim() == 0 or threshold.numel() == 1:
                grad_threshold = per_elem.sum().reshape(threshold.shape)
            else:
                # threshold is per feature (last dim); sum over the leading dims.
                lead = tuple(range(per_elem.dim() - threshold.dim()))
                grad_threshold = per_elem.sum(dim=lead) if lead else per_elem
                grad_threshold = grad_threshold.reshape(threshold.shape)
            grad_threshold = grad_threshold.to(threshold.dtype)
        return grad_input, grad_threshold, None


# ---------------------------------------------------------------------------
# batch z-score and global selection over all layers
# ---------------------------------------------------------------------------
def batch_zscore(x: torch.Tensor) -> torch.Tensor:
    """Per-feature z-score over the token dimension with the unbiased std."""
    xf = x.float()
    if xf.size(0) < 2:
        return xf - xf.mean(dim=0, keepdim=True)
    mean = xf.mean(dim=0, keepdim=True)
    std = xf.std(dim=0, keepdim=True)
    return (xf - mean) / (std + ZSCORE_EPS)


def _concat_layers(preacts: Dict[int, torch.Tensor]) -> Tuple[List[int], torch.Tensor, torch.Tensor, List[int]]:
    layers = sorted(preacts.keys())
    widths = [preacts[l].shape[-1] for l in layers]
    orig = torch.cat([preacts[l] for l in layers], dim=-1)
    ranks = torch.cat([batch_zscore(preacts[l]) for l in layers], dim=-1)
    return layers, orig, ranks, widths


def _global_flat_index(
    batch: int, widths: List[int], full_width: int, shard_offset: int, device
) -> torch.Tensor:
    """Flat index ``b*(L*F) + l*F + f_global`` of every element of a ``[B, sum(widths)]``
    shard whose layer ``l`` occupies global columns ``[l*F + shard_offset, ...)``."""
    cols = []
    for li, w in enumerate(widths):
        cols.append(li * full_width + shard_offset + torch.arange(w, device=device, dtype=torch.int64))
    col = torch.cat(cols)
    total = len(widths) * full_width
    return torch.arange(batch, device=device, dtype=torch.int64)[:, None] * total + col[None, :]


def sharded_flat_topk_mask(
    rank: torch.Tensor,
    gidx: torch.Tensor,
    k_total: int,
    group=None,
) -> torch.Tensor:
    """Exact global top-``k_total`` mask over the union of all ranks' ``rank`` tensors.

    Each rank contributes its best ``min(k_total, numel)`` candidates (value, global
    flat index); all ranks merge the same candidate set and derive one cut
    ``(v*, idx*)``; an element is kept iff ``v > v*`` or ``v == v*`` and ``idx <= idx*``.
    """
    world = pops.get_world_size(group)
    flat = rank.reshape(-1)
    fidx = gidx.reshape(-1)
    if world == 1:
        return _topk_flat_mask(rank, min(k_total, rank.numel()))
    n_local = flat.numel()
    counts = [torch.zeros(1, dtype=torch.int64, device=flat.device) for _ in range(world)]
    dist.all_gather(counts, torch.tensor([n_local], dtype=torch.int64, device=flat.device), group=group)
    n_global = int(sum(int(c.item()) for c in counts))
    if k_total >= n_global:
        return torch.ones_like(rank, dtype=torch.bool)
    if k_total <= 0:
        return torch.zeros_like(rank, dtype=torch.bool)
    # local candidates, ordered by (value desc, global index asc)
    by_idx = torch.argsort(fidx, stable=True)
    v_sorted, order = torch.sort(flat[by_idx], descending=True, stable=True)
    take = min(k_total, n_local)
    cand_v = torch.full((k_total,), float("-inf"), dtype=flat.dtype, device=flat.device)
    cand_i = torch.full((k_total,), torch.iinfo(torch.int64).max, dtype=torch.int64, device=flat.device)
    cand_v[:take] = v_sorted[:take]
    cand_i[:take] = fidx[by_idx][order[:take]]
    all_v = [torch.empty_like(cand_v) for _ in range(world)]
    all_i = [torch.empty_like(cand_i) for _ in range(world)]
    dist.all_gather(all_v, cand_v, group=group)
    dist.all_gather(all_i, cand_i, group=group)
    mv, mi = torch.cat(all_v), torch.cat(all_i)
    o1 = torch.argsort(mi, stable=True)
    mv2, o2 = torch.sort(mv[o1], descending=True, stable=True)
    cut_v = mv2[k_total - 1]
    cut_i = mi[o1][o2[k_total - 1]]
    keep = (flat > cut_v) | ((flat == cut_v) & (fidx <= cut_i))
    return keep.view_as(rank)


def apply_global_batchtopk(
    preacts: Dict[int, torch.Tensor],
    k: Optional[int],
    *,
    full_width: Optional[int] = None,
    shard_offset: int = 0,
    group=None,
    return_mask: bool = False,
) -> Dict[int, torch.Tensor]:
    """Global BatchTopK over all layers (and all feature shards when ``group`` has
    more than one rank).  ``preacts[l]`` is ``[B, F_local]``; ``full_width`` is the
    un-sharded per-layer feature count."""
    if not preacts:
        return {}
    layers, orig, ranks, widths = _concat_layers(preacts)
    batch = orig.size(0)
    if k is None:
        mask = torch.ones_like(orig, dtype=torch.bool)
    else:
        world = pops.get_world_size(group)
        fw = full_width if full_width is not None else widths[0]
        if world == 1:
            k_total = min(int(k) * batch, orig.numel())
            mask = _topk_flat_mask(ranks, k_total)
        else:
            gidx = _global_flat_index(batch, widths, fw, shard_offset, orig.device)
            mask = sharded_flat_topk_mask(ranks, gidx, int(k) * batch, group)
    out = _MaskSTE.apply(orig, mask)
    parts = torch.split(out, widths, dim=-1)
    result = {l: p for l, p in zip(layers, parts)}
    if return_mask:
        return result, {l: m for l, m in zip(layers, torch.split(mask, widths, dim=-1))}
    return result


def sharded_row_topk_mask(ranks: torch.Tensor, gidx: torch.Tensor, k: int, group=None) -> torch.Tensor:
    """Per-row top-``k`` mask over rows that are column-sharded across ``group``.
    ``gidx`` holds a globally consistent column order used to break ties."""
    world = pops.get_world_size(group)
    batch, width = ranks.shape
    if k <= 0:
        return torch.zeros_like(ranks, dtype=torch.bool)
    if world == 1:
        if k >= width:
            return torch.ones_like(ranks, dtype=torch.bool)
        _, order = torch.sort(ranks, dim=-1, descending=True, stable=True)
        mask = torch.zeros_like(ranks, dtype=torch.bool)
        mask.scatter_(-1, order[:, :k], True)
        return mask
    take = min(k, width)
    v_sorted, order = torch.sort(ranks, dim=-1, descending=True, stable=True)
    cand_v = torch.full((batch, k), float("-inf"), dtype=ranks.dtype, device=ranks.device)
    cand_i = torch.full((batch, k), torch.iinfo(torch.int64).max, dtype=torch.int64, device=ranks.device)
    cand_v[:, :take] = v_sorted[:, :take]
    cand_i[:, :take] = torch.gather(gidx, 1, order[:, :take])
    av = [torch.empty_like(cand_v) for _ in range(world)]
    ai = [torch.empty_like(cand_i) for _ in range(world)]
    dist.all_gather(av, cand_v, group=group)
    dist.all_gather(ai, cand_i, group=group)
    mv, mi = torch.cat(av, dim=1), torch.cat(ai, dim=1)
    o1 = torch.argsort(mi, dim=1, stable=True)
    mv1 = torch.gather(mv, 1, o1)
    mi1 = torch.gather(mi, 1, o1)
    mv2, o2 = torch.sort(mv1, dim=1, descending=True, stable=True)
    mi2 = torch.gather(mi1, 1, o2)
    cut_v = mv2[:, k - 1 : k]
    cut_i = mi2[:, k - 1 : k]
    # rows with fewer than k real candidates have a -inf cut: keep every finite entry
    return ((ranks > cut_v) | ((ranks == cut_v) & (gidx <= cut_i))) & (ranks > float("-inf"))


def apply_global_tokentopk(
    preacts: Dict[int, torch.Tensor],
    k_float: Optional[float],
    *,
    full_width: Optional[int] = None,
    shard_offset: int = 0,
    group=None,
) -> Dict[int, torch.Tensor]:
    """Per-token top-k over the concatenation of all layers' features.  Under tensor
    parallelism each rank contributes its per-row candidates and all ranks apply the
    same per-row cut."""
    if not preacts:
        return {}
    layers, orig, ranks, widths = _concat_layers(preacts)
    world = pops.get_world_size(group)
    if k_float is None:
        mask = torch.ones_like(orig, dtype=torch.bool)
    elif world == 1:
        mask = TokenTopK._compute_mask(orig, float(k_float), ranks)
    else:
        fw = full_width if full_width is not None else widths[0]
        k = resolve_token_k(float(k_float), len(widths) * fw)
        gidx = _global_flat_index(orig.size(0), widths, fw, shard_offset, orig.device)
        mask = sharded_row_topk_mask(ranks, gidx, k, group)
    out = _MaskSTE.apply(orig, mask)
    parts = torch.split(out, widths, dim=-1)
    return {l: p for l, p in zip(layers, parts)}


# Names kept for users of the reference helpers (clt/models/activations.py:229,360).
def _apply_batch_topk_helper(preactivations_dict, config, device=None, dtype=None, rank=0, process_group=None, profiler=None):
    return apply_global_batchtopk(preactivations_dict, config.batchtopk_k, full_width=config.num_features, group=process_group)


def _apply_token_topk_helper(preactivations_dict, config, device=None, dtype=None, rank=0, process_group=None, profiler=None):
    return apply_global_tokentopk(preactivations_dict, config.topk_k, full_width=config.num_features, group=process_group)
