"""Sparsity-penalty diagnostics (reference: clt/training/diagnostics.py:9-124).

For the active entries of every layer, statistics of ``z = c * ||W_dec,f|| * a``: median, 90th percentile,
mean ``tanh(z)``, fraction saturated (``tanh > 0.99``), mean ``|a|`` and the mean decoder norm, plus
aggregates over layers.  ``get_decoder_norms`` is a collective under tensor parallelism, so every rank
must call this function.
"""
from __future__ import annotations

from typing import Any, Dict

import torch


@torch.no_grad()
def compute_sparsity_diagnostics(model, training_config, feature_activations: Dict[int, torch.Tensor]) -> Dict[str, Any]:
    out: Dict[str, Any] = {}
    if not feature_activations:
        return out
    widths = {a.shape[-1] for a in feature_activations.values()}
    local = model.world_size > 1 and model.config.num_features not in widths
    norms = model.get_decoder_norms(gather=not local)
    c = training_config.sparsity_c
    agg = {"z_median": [], "z_p90": [], "mean_tanh": [], "sat_frac": [], "abs_act_mean": [], "dec_norm_mean": []}
    for l, a in sorted(feature_activations.items()):
        if a.numel() == 0:
            continue
        a2 = a.reshape(-1, a.shape[-1]).float()
        w = norms[l][: a2.shape[-1]].float().to(a2.device)
        active = a2 != 0
        if not bool(active.any()):
            continue
        z = (c * a2 * w.unsqueeze(0))[active]
        th = torch.tanh(z)
        zs = z.abs()
        if zs.numel() > 1_000_000:  # quantiles on a sample keep this cheap
            zs = zs[torch.randint(0, zs.numel(), (1_000_000,), device=zs.device)]
        vals = {
            "z_median": torch.quantile(zs, 0.5).item(),
            "z_p90": torch.quantile(zs, 0.9).item(),
            "mean_tanh": th.mean().item(),
            "sat_frac": (th.abs() > 0.99).float().mean().item(),
            "abs_act_mean": a2[active].abs().mean().item(),
            "dec_norm_mean": w.mean().item(),
        }
        for k, v in vals.items():
            out[f"diag/layer_{l}/{k}"] = v
            agg[k].append(v)
    for k, vs in agg.items():
        if vs:
            out[f"diag/agg/{k}"] = float(sum(vs) / len(vs))
    return out
