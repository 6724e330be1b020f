"""Loss terms of CLT training (autograd path and CPU oracle).

Definitions follow the reference LossManager (clt/training/losses.py:45-407):

* reconstruction: sum over layers of ``mean_{B,d}((y_hat - y)^2)`` after undoing the
  store's normalisation (``x*std + mean`` for ``mean_std``, ``/sqrt(d)`` for ``sqrt_d_model``);
* sparsity: ``lambda(t) * sum_{layers,tokens,features} tanh(c * ||W_dec,f|| * a)`` with the
  linear / delayed-linear warm-up of ``lambda`` — a sum, not a mean, over tokens;
* pre-activation: ``coef * mean(relu(-preact))`` over all layers;
* auxiliary (AuxK): per layer, the top ``min(512, n_dead)`` dead-feature
  pre-activations of every token decode to the same layer and are matched to the
  de-normalised residual, scaled by ``min(n_dead/k_aux, 1) * aux_loss_factor``.

Differences that are deliberate: one encoder pass feeds every term (the reference
runs the encoder two to four times per step, losses.py:357,248,285); all terms work
on this rank's feature shard and only scalars are all-reduced for reporting.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
import torch.nn.functional as F

from ..config import CLTConfig, TrainingConfig
from ..models import activations as act
from ..parallel import ops as pops


def sparsity_lambda_at(cfg: TrainingConfig, current_step: int, total_steps: int) -> float:
    """Warm-up schedule of the sparsity coefficient (losses.py:117-137)."""
    progress = min(1.0, current_step / total_steps) if total_steps > 0 else 1.0
    if cfg.sparsity_lambda_schedule == "linear":
        return cfg.sparsity_lambda * progress
    start = cfg.sparsity_lambda_delay_frac * total_steps
    if current_step < start:
        return 0.0
    if total_steps > start:
        return cfg.sparsity_lambda * min(1.0, (current_step - start) / (total_steps - start))
    return cfg.sparsity_lambda


class LossManager:
    def __init__(
        self,
        config: TrainingConfig,
        mean_tg: Optional[Dict[int, torch.Tensor]] = None,
        std_tg: Optional[Dict[int, torch.Tensor]] = None,
        clt_config: Optional[CLTConfig] = None,
    ):
        self.config = config
        self.mean_tg = mean_tg or {}
        self.std_tg = std_tg or {}
        self.clt_config = clt_config
        self.aux_loss_factor = config.aux_loss_factor
        self.apply_sparsity_penalty_to_batchtopk = config.apply_sparsity_penalty_to_batchtopk
        self.current_sparsity_lambda = 0.0

    # ----------------------------------------------------------- helpers
    def _denorm(self, layer_idx: int, pred: torch.Tensor, tgt: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        m = self.config.normalization_method
        if m == "mean_std" and layer_idx in self.mean_tg and layer_idx in self.std_tg:
            mean = self.mean_tg[layer_idx].to(pred.device, pred.dtype)
            std = self.std_tg[layer_idx].to(pred.device, pred.dtype)
            return pred * std + mean, tgt.to(pred.dtype) * std + mean
        if m == "sqrt_d_model" and self.clt_config is not None:
            s = self.clt_config.d_model ** 0.5
            return pred / s, tgt.to(pred.dtype) / s
        return pred, tgt.to(pred.dtype)

    def compute_reconstruction_loss(self, predicted: Dict[int, torch.Tensor], target: Dict[int, torch.Tensor]) -> torch.Tensor:
        dev = next(iter(predicted.values())).device if predicted else torch.device("cpu")
        total = torch.zeros((), device=dev)
        for l, pred in predicted.items():
            if l not in target:
                continue
            p, t = self._denorm(l, pred, target[l].to(pred.device))
            total = total + F.mse_loss(p, t)
        return total

    def compute_sparsity_penalty(self, model, activations: Dict[int, torch.Tensor], current_step: int, total_steps: int):
        """Penalty over the activations given (full ``[B,F]`` or this rank's shard)."""
        dev = next(model.parameters()).device
        lam = sparsity_lambda_at(self.config, current_step, total_steps)
        if not activations or lam < 1e-9:
            return torch.zeros((), device=dev), 0.0
        if model.config.activation_fn == "batchtopk" and not self.apply_sparsity_penalty_to_batchtopk:
            return torch.zeros((), device=dev), 0.0
        widths = {a.shape[-1] for a in activations.values()}
        local = model.world_size > 1 and widths <= {model.valid_features, model.local_features} \
            and model.config.num_features not in widths
        norms = model.get_decoder_norms(gather=not local)
        total = torch.zeros((), device=dev)
        for l, a in activations.items():
            if a.numel() == 0:
                continue
            a2 = a.reshape(-1, a.shape[-1])
            w = norms[l][: a2.shape[-1]].to(a2.device)
            total = total + torch.tanh(self.config.sparsity_c * a2 * w.unsqueeze(0)).sum()
        return lam * total, lam

    def compute_preactivation_loss(self, model, inputs: Dict[int, torch.Tensor], preacts: Optional[Dict[int, torch.Tensor]] = None) -> torch.Tensor:
        coef = self.config.preactivation_coef
        dev = next(iter(inputs.values())).device if inputs else torch.device("cpu")
        if coef is None or abs(coef) < 1e-9 or not inputs:
            return torch.zeros((), device=dev)
        if preacts is None:
            preacts, _ = model._encode_all_layers(inputs, gather=False)
        total = torch.zeros((), device=dev)
        numel = 0
        for l, p in preacts.items():
            if p.numel() == 0:
                continue
            total = total + F.relu(-p).sum()
            numel += p.shape[0] * model.config.num_features
        if numel == 0:
            return torch.zeros((), device=dev)
        # local share; summing the ranks' values gives the reference's mean over [B, F]
        return coef * total / numel

    def compute_auxiliary_loss(
        self,
        model,
        inputs: Dict[int, torch.Tensor],
        residuals: Dict[int, torch.Tensor],
        dead_mask: Optional[torch.Tensor] = None,
        k_aux_default: int = 512,
        preacts: Optional[Dict[int, torch.Tensor]] = None,
    ) -> torch.Tensor:
        """``dead_mask`` is ``[L, F]`` (full) or ``[L, valid_features]`` (this rank's shard)."""
        dev = next(model.parameters()).device
        if not self.aux_loss_factor or dead_mask is None:
            return torch.zeros((), device=dev)
        if preacts is None:
            preacts, _ = model._encode_all_layers(inputs, gather=False)
        if dead_mask.shape[-1] != model.valid_features:
            dead_mask = dead_mask[:, model.feature_start : model.feature_start + model.valid_features]
        group = model.process_group if model.world_size > 1 else None
        n_dead_all = dead_mask.sum(dim=1).to(torch.float32)
        if group is not None:
            pops.all_reduce(n_dead_all, group=group)
        n_dead_host = n_dead_all.tolist()  # one host read for all layers
        total = torch.zeros((), device=dev)
        for l, pre in preacts.items():
            if pre.numel() == 0 or l >= dead_mask.shape[0] or l not in residuals:
                continue
            n_dead = int(n_dead_host[l])
            if n_dead == 0:
                continue
            k_aux = max(1, min(k_aux_default, n_dead))
            ranks = torch.where(dead_mask[l].unsqueeze(0), pre.float(), torch.full_like(pre, float("-inf"), dtype=torch.float32))
            gidx = (model.feature_start + torch.arange(pre.shape[-1], device=pre.device, dtype=torch.int64)).unsqueeze(0).expand_as(ranks)
            mask = act.sharded_row_topk_mask(ranks.detach(), gidx, k_aux, group)
            aux_acts = act._MaskSTE.apply(pre, mask)
            recon = model.decode({l: aux_acts}, l)
            layer = F.mse_loss(recon, residuals[l].to(recon.device, recon.dtype))
            total = total + min(n_dead / k_aux, 1.0) * layer
        return self.aux_loss_factor * total

    # -------------------------------------------------------------- total
    def compute_total_loss_tensors(
        self,
        model,
        inputs: Dict[int, torch.Tensor],
        targets: Dict[int, torch.Tensor],
        current_step: int,
        total_steps: int,
        precomputed_activations: Optional[Dict[int, torch.Tensor]] = None,
        dead_neuron_mask: Optional[torch.Tensor] = None,
    ):
        """Returns ``(loss_for_backward, {name: 0-dim tensor}, activations)`` with one
        encoder pass.  Under tensor parallelism ``loss_for_backward`` holds this rank's
        share of the feature-summed terms; the reported values are all-reduced."""
        cfg = model.config
        need_pre = (self.config.preactivation_coef or 0) != 0 or bool(self.aux_loss_factor)
        preacts = None
        if precomputed_activations is None:
            if cfg.activation_fn in ("batchtopk", "topk") and cfg.topk_mode == "global":
                preacts, _ = model._encode_all_layers(inputs, gather=False)
                acts = model._select(preacts, batch=(cfg.activation_fn == "batchtopk"))
            else:
                if need_pre:
                    preacts, _ = model._encode_all_layers(inputs, gather=False)
                    acts = {l: model._activate_layer_local(p, l) for l, p in preacts.items()}
                else:
                    acts = model.get_feature_activations(inputs, gather=False)
        else:
            acts = precomputed_activations
        predictions = model.decode_all(acts, inputs)
        recon = self.compute_reconstruction_loss(predictions, targets)
        sparsity, lam = self.compute_sparsity_penalty(model, acts, current_step, total_steps)
        self.current_sparsity_lambda = lam
        preact = self.compute_preactivation_loss(model, inputs, preacts)
        aux = torch.zeros((), device=recon.device)
        if cfg.activation_fn in ("batchtopk", "topk") and self.aux_loss_factor and dead_neuron_mask is not None:
            residuals = {}
            for l, pred in predictions.items():
                if l in targets:
                    p, t = self._denorm(l, pred, targets[l].to(pred.device))
                    residuals[l] = t - p
            aux = self.compute_auxiliary_loss(model, inputs, residuals, dead_neuron_mask, preacts=preacts)
        loss = recon + sparsity + preact + aux
        sp_rep, pre_rep = sparsity.detach().clone(), preact.detach().clone()
        local_terms = model.world_size > 1 and all(a.shape[-1] != cfg.num_features for a in acts.values())
        if local_terms:
            both = torch.stack([sp_rep, pre_rep])
            pops.all_reduce(both, group=model.process_group)
            sp_rep, pre_rep = both[0], both[1]
        elif model.world_size > 1:
            pre_both = pre_rep.clone()
            pops.all_reduce(pre_both, group=model.process_group)
            pre_rep = pre_both
        parts = {
            "total": recon.detach() + sp_rep + pre_rep + aux.detach(),
            "reconstruction": recon.detach(),
            "sparsity": sp_rep,
            "preactivation": pre_rep,
            "auxiliary": aux.detach(),
        }
        return loss, parts, acts

    def compute_total_loss(
        self,
        model,
        inputs: Dict[int, torch.Tensor],
        targets: Dict[int, torch.Tensor],
        current_step: int,
        total_steps: int,
        precomputed_activations: Optional[Dict[int, torch.Tensor]] = None,
        dead_neuron_mask: Optional[torch.Tensor] = None,
    ) -> Tuple[torch.Tensor, Dict[str, float]]:
        loss, parts, _ = self.compute_total_loss_tensors(
            model, inputs, targets, current_step, total_steps, precomputed_activations, dead_neuron_mask
        )
        host = torch.stack([parts[k].float() for k in ("total", "reconstruction", "sparsity", "preactivation", "auxiliary")]).tolist()
        keys = ("total", "reconstruction", "sparsity", "preactivation", "auxiliary")
        return loss, dict(zip(keys, host))

    def get_current_sparsity_lambda(self) -> float:
        return self.current_sparsity_lambda
