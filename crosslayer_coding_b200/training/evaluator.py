"""Evaluation metrics (reference: clt/training/evaluator.py:28-522).

Metric definitions and key names are the reference's logging contract:

* ``sparsity/total_l0 | avg_l0 | sparsity_fraction`` and ``layerwise/l0/layer_i`` — mean number of
  non-zero features per token per layer;
* ``reconstruction/explained_variance`` and ``reconstruction/normalized_mean_reconstruction_error`` —
  per layer ``NMSE = MSE / mean_d(var_tokens(target))`` and ``EV = 1 - mean_d var(err) / mean_d var(target)``
  in de-normalised units, averaged over layers (EV clamped to [0, 1]);
* ``layerwise/log_feature_density`` (log10 of the firing frequency, ``a > 1e-6``) and the
  "consistent activation heuristic" per layer, plus their aggregates under ``sparsity/``;
* ``layerwise/dead_features`` and ``dead_features/total_eval`` from the trainer's dead mask.

Differences: one forward pass instead of two (the reference runs ``model(inputs)`` and
``get_feature_activations`` separately, evaluator.py:124-125), every scalar is accumulated on the device
and read back in a single transfer, and under tensor parallelism per-feature statistics are computed on
the local shard and gathered once.
"""
from __future__ import annotations

import logging
import time
from typing import Any, Dict, List, Optional

import numpy as np
import torch

from ..parallel import ops as pops

logger = logging.getLogger(__name__)


class CLTEvaluator:
    def __init__(
        self,
        model,
        device: torch.device,
        start_time: Optional[float] = None,
        mean_tg: Optional[Dict[int, torch.Tensor]] = None,
        std_tg: Optional[Dict[int, torch.Tensor]] = None,
        normalization_method: str = "none",
        d_model: Optional[int] = None,
    ):
        self.model = model
        self.device = torch.device(device)
        self.start_time = start_time or time.time()
        self.mean_tg = mean_tg or {}
        self.std_tg = std_tg or {}
        self.normalization_method = normalization_method
        self.d_model = d_model

    @staticmethod
    def _log_density(density: torch.Tensor, eps: float = 1e-10) -> torch.Tensor:
        return torch.log10(density + eps)

    def _denorm(self, l: int, t: torch.Tensor) -> torch.Tensor:
        if self.normalization_method == "mean_std" and l in self.mean_tg and l in self.std_tg:
            return t * self.std_tg[l].to(t.device, t.dtype) + self.mean_tg[l].to(t.device, t.dtype)
        if self.normalization_method == "sqrt_d_model" and self.d_model is not None:
            return t / (self.d_model ** 0.5)
        return t

    @torch.no_grad()
    def compute_metrics(
        self,
        inputs: Dict[int, torch.Tensor],
        targets: Dict[int, torch.Tensor],
        dead_neuron_mask: Optional[torch.Tensor] = None,
    ) -> Dict[str, Any]:
        model = self.model
        inputs = {k: v.to(self.device) for k, v in inputs.items()}
        targets = {k: v.to(self.device) for k, v in targets.items()}
        acts = model.get_feature_activations(inputs, gather=False)
        recons = model.decode_all(acts, inputs)
        metrics: Dict[str, Any] = {}
        metrics.update(self._compute_sparsity(acts))
        metrics.update(self._compute_reconstruction_metrics(targets, recons))
        density = self._compute_feature_density(acts)
        metrics.update(density)
        dens = density.get("layerwise/log_feature_density", {})
        heur = density.get("layerwise/consistent_activation_heuristic", {})
        flat_d = [v for vals in dens.values() for v in vals]
        flat_h = [v for vals in heur.values() for v in vals]
        if flat_d:
            metrics["sparsity/feature_density_mean"] = float(np.mean(flat_d))
            metrics["sparsity/log_feature_density_agg_hist"] = flat_d
        if flat_h:
            metrics["sparsity/consistent_activation_heuristic_mean"] = float(np.mean(flat_h))
            metrics["sparsity/consistent_activation_heuristic_agg_hist"] = flat_h
        dead = self._compute_dead_neuron_metrics(dead_neuron_mask)
        dead["dead_features/total_eval"] = sum(dead.get("layerwise/dead_features", {}).values())
        metrics.update(dead)
        return metrics

    @torch.no_grad()
    def compute_metrics_from_engine(self, engine, X: torch.Tensor, Y: torch.Tensor,
                                    dead_neuron_mask: Optional[torch.Tensor] = None) -> Dict[str, Any]:
        """The same metrics from the fused step's sparse forward: reconstructions from the sparse decode, L0 and
        feature densities from the entry list (no dense ``[B, F]`` activation tensor is formed).  ``X`` / ``Y``:
        ``[L, B, d]`` bf16, already normalised."""
        model = self.model
        L, B, Fl = engine.L, engine.B, engine.Fl
        fired_before = engine.fired.clone()  # an evaluation forward must not count as "fired" for the dead-feature window
        yhat = engine.forward(X, Y)  # [L, B, d] fp32, summed over ranks
        engine.fired.copy_(fired_before)
        cap = engine.ent_val.numel()
        n = torch.clamp(engine.ctl[3], max=cap)
        live = torch.arange(cap, device=X.device) < n
        col = torch.where(live, engine.ent_col, (torch.arange(cap, device=X.device, dtype=torch.int32) % engine.ncols)).long()
        nonzero = torch.zeros(engine.ncols, dtype=torch.float32, device=X.device)
        fired = torch.zeros(engine.ncols, dtype=torch.float32, device=X.device)
        nonzero.index_add_(0, col, (live & (engine.ent_val != 0)).float())
        fired.index_add_(0, col, (live & (engine.ent_val > 1e-6)).float())
        nonzero, fired = nonzero.view(L, Fl), fired.view(L, Fl)
        per_layer = nonzero.sum(dim=1) / B
        if model.world_size > 1:
            pops.all_reduce(per_layer, group=model.process_group)
            fired = pops.all_gather_cat(fired, dim=1, group=model.process_group)
        fired = fired[:, : model.config.num_features]
        host = per_layer.tolist()
        total = float(sum(host))
        avg = total / L
        metrics: Dict[str, Any] = {
            "sparsity/total_l0": total, "sparsity/avg_l0": avg,
            "sparsity/sparsity_fraction": max(0.0, min(1.0, 1.0 - avg / model.config.num_features)),
            "layerwise/l0": {f"layer_{l}": v for l, v in enumerate(host)},
        }
        metrics.update(self._compute_reconstruction_metrics({l: Y[l] for l in range(L)}, {l: yhat[l] for l in range(L)}))
        dens = {f"layer_{l}": self._log_density(fired[l] / B).tolist() for l in range(L)}
        heur = {f"layer_{l}": (fired[l] / ((fired[l] > 0).float() + 1e-9)).tolist() for l in range(L)}
        metrics["layerwise/log_feature_density"] = dens
        metrics["layerwise/consistent_activation_heuristic"] = heur
        flat_d = [v for vals in dens.values() for v in vals]
        flat_h = [v for vals in heur.values() for v in vals]
        metrics["sparsity/feature_density_mean"] = float(np.mean(flat_d))
        metrics["sparsity/log_feature_density_agg_hist"] = flat_d
        metrics["sparsity/consistent_activation_heuristic_mean"] = float(np.mean(flat_h))
        metrics["sparsity/consistent_activation_heuristic_agg_hist"] = flat_h
        dead = self._compute_dead_neuron_metrics(dead_neuron_mask)
        dead["dead_features/total_eval"] = sum(dead.get("layerwise/dead_features", {}).values())
        metrics.update(dead)
        # per-layer spread of the pre-activations of this forward (reference trainer.py:884-897)
        stds = engine.preact[:, :, : engine.Fv].float().std(dim=(1, 2)) if engine.Fv > 0 else torch.zeros(L, device=X.device)
        metrics["layerwise/preactivation_std_dev"] = {f"layer_{l}": v for l, v in enumerate(stds.tolist())}
        return metrics

    # ------------------------------------------------------------------ pieces
    def _compute_sparsity(self, activations: Dict[int, torch.Tensor]) -> Dict[str, Any]:
        L = self.model.config.num_layers
        if not activations or not any(v.numel() > 0 for v in activations.values()):
            return {"sparsity/total_l0": 0.0, "sparsity/avg_l0": 0.0, "sparsity/sparsity_fraction": 1.0,
                    "layerwise/l0": {f"layer_{i}": 0.0 for i in range(L)}}
        layers = sorted(activations.keys())
        vals = []
        for l in layers:
            a = activations[l]
            vals.append((a != 0).float().sum() / max(1, a.shape[0]) if a.numel() else torch.zeros((), device=self.device))
        per_layer = torch.stack(vals)
        if self.model.world_size > 1 and all(a.shape[-1] != self.model.config.num_features for a in activations.values()):
            pops.all_reduce(per_layer, group=self.model.process_group)
        host = per_layer.tolist()
        total = float(sum(host))
        n_valid = sum(1 for l in layers if activations[l].numel() > 0)
        avg = total / n_valid if n_valid else 0.0
        frac = max(0.0, min(1.0, 1.0 - avg / self.model.config.num_features))
        return {"sparsity/total_l0": total, "sparsity/avg_l0": avg, "sparsity/sparsity_fraction": frac,
                "layerwise/l0": {f"layer_{l}": v for l, v in zip(layers, host)}}

    def _compute_reconstruction_metrics(self, targets: Dict[int, torch.Tensor], reconstructions: Dict[int, torch.Tensor]) -> Dict[str, Any]:
        rows = []
        layers = []
        for l, tgt in targets.items():
            if l not in reconstructions:
                continue
            rec = reconstructions[l].float()
            t = self._denorm(l, tgt.to(rec.device).float()).reshape(-1, rec.shape[-1])
            r = self._denorm(l, rec).reshape(-1, rec.shape[-1])
            if t.shape != r.shape or t.numel() == 0:
                continue
            err = t - r
            rows.append(torch.stack([(err ** 2).mean(), t.var(dim=0, unbiased=False).mean(), err.var(dim=0, unbiased=False).mean()]))
            layers.append(l)
        if not rows:
            return {"reconstruction/explained_variance": 0.0, "reconstruction/normalized_mean_reconstruction_error": 0.0,
                    "layerwise/normalized_mse": {}, "layerwise/explained_variance": {}}
        host = torch.stack(rows).double().tolist()
        nmse, ev = {}, {}
        for l, (mse, tvar, evar) in zip(layers, host):
            if tvar > 1e-9:
                ev[f"layer_{l}"] = 1.0 - evar / tvar
                nmse[f"layer_{l}"] = mse / tvar
            else:
                ev[f"layer_{l}"] = 1.0 if evar < 1e-9 else 0.0
                nmse[f"layer_{l}"] = 0.0 if mse < 1e-9 else float("inf")
        n = len(layers)
        return {
            "reconstruction/explained_variance": max(0.0, min(1.0, sum(ev.values()) / n)),
            "reconstruction/normalized_mean_reconstruction_error": sum(nmse.values()) / n,
            "layerwise/normalized_mse": nmse,
            "layerwise/explained_variance": ev,
        }

    def _compute_feature_density(self, activations: Dict[int, torch.Tensor]) -> Dict[str, Any]:
        if not activations or not any(v.numel() > 0 for v in activations.values()):
            return {"layerwise/log_feature_density": {}, "layerwise/consistent_activation_heuristic": {}}
        dens: Dict[str, List[float]] = {}
        heur: Dict[str, List[float]] = {}
        model = self.model
        for l in sorted(activations.keys()):
            a = activations[l]
            if a.numel() == 0 or a.shape[0] == 0:
                continue
            fired = (a > 1e-6).float()
            count = fired.sum(dim=0)
            if model.world_size > 1 and a.shape[-1] != model.config.num_features:
                pad = model.local_features - count.shape[0]
                if pad:
                    count = torch.nn.functional.pad(count, (0, pad))
                count = pops.all_gather_cat(count, dim=0, group=model.process_group)[: model.config.num_features]
            density = count / a.shape[0]
            dens[f"layer_{l}"] = self._log_density(density).tolist()
            heur[f"layer_{l}"] = (count / ((count > 0).float() + 1e-9)).tolist()
        return {"layerwise/log_feature_density": dens, "layerwise/consistent_activation_heuristic": heur}

    def _compute_dead_neuron_metrics(self, dead_neuron_mask: Optional[torch.Tensor]) -> Dict[str, Any]:
        out: Dict[str, Any] = {"layerwise/dead_features": {}}
        if dead_neuron_mask is None:
            return out
        m = dead_neuron_mask.to(self.device)
        L = self.model.config.num_layers
        if m.dim() != 2 or m.shape[0] != L:
            logger.warning("dead_neuron_mask has unexpected shape %s; skipping dead-feature metrics", tuple(m.shape))
            return out
        per_layer = m.sum(dim=1).float()
        if self.model.world_size > 1 and m.shape[1] != self.model.config.num_features:
            pops.all_reduce(per_layer, group=self.model.process_group)
        out["layerwise/dead_features"] = {f"layer_{i}": int(v) for i, v in enumerate(per_layer.tolist())}
        return out

    def print_evaluation_report(self, metrics: Dict[str, Any], step: Optional[int] = None) -> None:
        head = f"Evaluation report (step {step})" if step is not None else "Evaluation report"
        lines = [head]
        for key in ("reconstruction/explained_variance", "reconstruction/normalized_mean_reconstruction_error",
                    "sparsity/avg_l0", "sparsity/total_l0", "sparsity/sparsity_fraction", "dead_features/total_eval"):
            if key in metrics:
                lines.append(f"  {key:<58s} {metrics[key]:.6g}")
        for key in ("layerwise/normalized_mse", "layerwise/l0", "layerwise/dead_features"):
            if metrics.get(key):
                lines.append(f"  {key}: " + ", ".join(f"{k}={v:.4g}" for k, v in metrics[key].items()))
        logger.info("\n".join(lines))
