"""BatchTopK/TopK -> JumpReLU threshold estimation.

Behaviour follows the reference ThetaManager (clt/models/theta.py:81-173 for the
per-batch statistic, :175-432 for the accumulation loop, :434-636 for the
conversion):

1. per batch and layer, z-score the pre-activations over the tokens (unbiased std,
   eps 1e-6) and accumulate the batch mean / std of every feature;
2. run the model's (Batch)TopK selection ranked on the z-scores;
3. per feature, take the minimum *z-scored* pre-activation among the selected
   entries whose original value is positive, and accumulate it (sum and count);
4. conversion: one scalar per layer ``theta_norm`` = mean over features of
   ``sum / count`` restricted to finite positive values (fallback 1e-5), then
   ``theta_f = theta_norm * std_f + mean_f`` clamped at 1e-7, stored as
   ``log_threshold``; the config switches to ``activation_fn="jumprelu"``.

All statistics live with the feature shard that owns them; the only cross-rank
quantity is the per-layer scalar of step 4 (one ``[L, 2]`` all-reduce).  The
reference all-reduces four ``[L, F]`` tensors instead (theta.py:473-480).
``default_theta_value`` is accepted for signature compatibility and, as in the
reference, does not enter the arithmetic.
"""
from __future__ import annotations

import logging
from typing import Dict, Iterable, Optional

import torch
import torch.nn as nn

from ..parallel import ops as pops
from . import activations as act

logger = logging.getLogger(__name__)


def _new_stats(model) -> Dict[str, torch.Tensor]:
    L, w = model.config.num_layers, model.valid_features
    dev = model.enc_weight.device
    z = lambda: torch.zeros(L, w, device=dev, dtype=torch.float32)  # noqa: E731
    return {"sum_min": z(), "cnt_min": z(), "mean": z(), "std": z(), "batches": torch.zeros(L, device=dev)}


@torch.no_grad()
def accumulate_theta_batch(model, inputs: Dict[int, torch.Tensor], stats: Dict[str, torch.Tensor]) -> None:
    """Steps 1-3 of the module docstring for one batch."""
    cfg = model.config
    pre, _ = model._encode_all_layers(inputs, gather=False)
    if not pre:
        return
    zs = {}
    for l, x in pre.items():
        xf = x.float()
        if xf.numel() == 0:
            continue
        mean = xf.mean(dim=0)
        std = xf.std(dim=0) if xf.size(0) > 1 else torch.zeros_like(mean)
        stats["mean"][l] += mean
        stats["std"][l] += std
        stats["batches"][l] += 1
        zs[l] = (xf - mean) / (std + act.ZSCORE_EPS)
    group = model.process_group if model.world_size > 1 else None
    kwargs = dict(full_width=cfg.num_features, shard_offset=model.feature_start, group=group)
    if cfg.activation_fn == "batchtopk":
        _, masks = act.apply_global_batchtopk(pre, cfg.batchtopk_k, return_mask=True, **kwargs)
        gated = {l: pre[l].float() * masks[l] for l in pre}
    elif cfg.activation_fn == "topk":
        gated_t = act.apply_global_tokentopk(pre, cfg.topk_k, **kwargs)
        gated = {l: gated_t[l].float() for l in pre}
    else:
        raise ValueError(f"theta estimation needs a batchtopk/topk model, got {cfg.activation_fn!r}")
    for l, z in zs.items():
        active = gated[l] > 0
        masked = torch.where(active, z, torch.full_like(z, float("inf")))
        mins = masked.amin(dim=0)
        ok = torch.isfinite(mins)
        stats["sum_min"][l] += torch.where(ok, mins, torch.zeros_like(mins))
        stats["cnt_min"][l] += ok.float()


@torch.no_grad()
def accumulate_theta_batch_sparse(sf, X: torch.Tensor, stats: Dict[str, torch.Tensor]) -> None:
    """The same statistic from the sparse forward (``models.sparse_forward.SparseForward``): the batch mean / std of
    every feature come from the column-statistics kernel, the per-feature minimum of the selected z-scores from the
    entry list - no dense ``[B, L*F]`` selection, which is what the dense path spends its time on."""
    sf.encode(X)
    L, Fl = sf.L, sf.Fl
    std = 1.0 / sf.rstd - act.ZSCORE_EPS
    stats["mean"] += sf.mean[:, : stats["mean"].shape[1]]
    stats["std"] += std[:, : stats["std"].shape[1]]
    stats["batches"] += 1
    cap = sf.ent_val.numel()
    n = torch.clamp(sf.ctl[3], max=cap)
    live = (torch.arange(cap, device=X.device) < n) & (sf.ent_val > 0)
    col = torch.where(live, sf.ent_col, torch.zeros_like(sf.ent_col)).long()
    z = (sf.ent_val - sf.mean.reshape(-1)[col]) * sf.rstd.reshape(-1)[col]
    z = torch.where(live, z, torch.full_like(z, float("inf")))
    mins = torch.full((L * Fl,), float("inf"), device=X.device)
    mins.scatter_reduce_(0, col, z, reduce="amin", include_self=True)
    mins = mins.view(L, Fl)[:, : stats["sum_min"].shape[1]]
    ok = torch.isfinite(mins)
    stats["sum_min"] += torch.where(ok, mins, torch.zeros_like(mins))
    stats["cnt_min"] += ok.float()


@torch.no_grad()
def estimate_theta_posthoc(
    model,
    data_iter: Iterable,
    num_batches: Optional[int] = None,
    default_theta_value: float = 1e6,
    device: Optional[torch.device] = None,
) -> torch.Tensor:
    """Accumulate statistics over ``num_batches`` batches of ``data_iter`` (yielding
    ``(inputs, targets)``), convert the model in place and return ``theta [L, F_local]``."""
    was_training = model.training
    model.eval()
    stats = _new_stats(model)
    done = 0
    sparse = None  # sm_100a sparse forward, built for the first batch's size when the model is covered by it
    for batch in data_iter:
        if num_batches is not None and done >= num_batches:
            break
        inputs = batch[0] if isinstance(batch, (tuple, list)) else batch
        dev = model.enc_weight.device
        inputs = {l: x.to(dev) for l, x in inputs.items()}
        layers = sorted(inputs)
        rows = inputs[layers[0]].reshape(-1, model.config.d_model).shape[0] if layers else 0
        if sparse is None and dev.type == "cuda" and layers == list(range(model.config.num_layers)):
            from . import sparse_forward

            if sparse_forward.supports(model) is None:
                sparse = sparse_forward.SparseForward(model, rows)
        if sparse is not None and rows == sparse.B:
            X = torch.stack([inputs[l].reshape(-1, model.config.d_model) for l in layers]).to(torch.bfloat16)
            accumulate_theta_batch_sparse(sparse, X, stats)
            sparse.check_status()
        else:
            accumulate_theta_batch(model, inputs, stats)
        done += 1
    if done == 0:
        logger.warning("Rank %d: no batches were processed for theta estimation", model.rank)
    nb = stats["batches"].clamp_min(1.0).unsqueeze(-1)
    stats["mean"] /= nb
    stats["std"] /= nb
    model._theta_stats = stats
    convert_to_jumprelu_inplace(model, default_theta_value)
    model.train(was_training)
    return model.log_threshold.detach().exp()


@torch.no_grad()
def convert_to_jumprelu_inplace(model, default_theta_value: float = 1e6) -> None:
    cfg = model.config
    if cfg.activation_fn not in ("batchtopk", "topk"):
        logger.warning("Model activation is %r; conversion expects batchtopk/topk.", cfg.activation_fn)
    stats = model._theta_stats
    if stats is None:
        raise RuntimeError("run estimate_theta_posthoc (or accumulate_theta_batch) before converting")
    L = cfg.num_layers
    ratio = stats["sum_min"] / stats["cnt_min"].clamp_min(1.0)
    good = (stats["cnt_min"] > 0) & torch.isfinite(ratio) & (ratio > 0)
    agg = torch.stack([torch.where(good, ratio, torch.zeros_like(ratio)).sum(dim=1), good.float().sum(dim=1)], dim=1)
    if model.world_size > 1:
        pops.all_reduce(agg, group=model.process_group)
    theta_norm = torch.where(agg[:, 1] > 0, agg[:, 0] / agg[:, 1].clamp_min(1.0), torch.full_like(agg[:, 0], 1e-5))
    theta_raw = theta_norm.unsqueeze(-1) * stats["std"] + stats["mean"]
    log_theta = theta_raw.clamp_min(1e-7).log()
    pad = model.local_features - model.valid_features
    if pad:
        log_theta = torch.nn.functional.pad(log_theta, (0, pad), value=float(torch.tensor(default_theta_value).log()))
    log_theta = log_theta.to(device=model.enc_weight.device, dtype=torch.float32)  # fp32 whatever the weight type is

    # config mutation mirrors the reference (theta.py:584-595)
    cfg.activation_fn = "jumprelu"
    cfg.jumprelu_threshold = 0.0
    cfg.batchtopk_k = None
    cfg.batchtopk_straight_through = False
    cfg.topk_k = None
    if model.log_threshold is None:
        model.log_threshold = nn.Parameter(log_theta)
    else:
        model.log_threshold.data = log_theta
    model._theta_stats = None
    logger.info(
        "Rank %d: converted to JumpReLU; per-layer normalised theta: %s",
        model.rank, [round(float(v), 4) for v in theta_norm.tolist()],
    )
    assert model.log_threshold.shape == (L, model.local_features)
