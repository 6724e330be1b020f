"""BatchTopK/TopK -> JumpReLU conversion with layer-wise L0 calibration.

Workflow of the reference conversion script (scripts/convert_batchtopk_to_jumprelu.py:90-1053):
estimate per-feature thresholds over N batches (``model.estimate_theta_posthoc``), compare L0 / NMSE of the
converted model with the original, and optionally calibrate every layer: one scale ``s`` in ``[0.1, 10]``
multiplies that layer's threshold vector so that the layer's L0 matches the original model's L0.

The reference finds ``s`` by a 15-step binary search that re-encodes a fresh sample of <= 1024 tokens per probe
(:649-870).  Here the pre-activations of the calibration tokens are computed once per layer and the L0 of
*every* candidate scale comes from one histogram of ``x / theta`` (``l0_for_scales``), followed by a short exact
bisection between the two best grid points.
"""
from __future__ import annotations

import copy
import logging
import math
from typing import Dict, Iterable, List, Optional, Tuple

import torch

logger = logging.getLogger(__name__)


@torch.no_grad()
def layer_l0(model, inputs: Dict[int, torch.Tensor]) -> Dict[int, float]:
    """Mean number of active features per token and layer (summed over tensor-parallel shards)."""
    from .parallel import ops as pops

    acts = model.get_feature_activations(inputs, gather=False)
    layers = sorted(acts)
    vals = torch.stack([(acts[l] != 0).float().sum() / max(1, acts[l].shape[0]) for l in layers])
    if model.world_size > 1:
        pops.all_reduce(vals, group=model.process_group)
    return {l: float(v) for l, v in zip(layers, vals.tolist())}


@torch.no_grad()
def quick_l0_check(model, inputs: Dict[int, torch.Tensor], num_tokens: int = 1024, seed: Optional[int] = None) -> Dict[int, float]:
    """Empirical L0 per layer on ``inputs`` (reference: ``run_quick_l0_checks_script``,
    scripts/convert_batchtopk_to_jumprelu.py:766-870).  (Batch)TopK models are measured on the whole batch
    through ``get_feature_activations`` (the selection is global), per-layer activations (JumpReLU, ReLU) on a
    random sample of at most ``num_tokens`` tokens through ``encode``.  Entries count as active when
    ``|a| > 1e-8``; a layer without tokens reports NaN."""
    from .parallel import ops as pops

    L = model.config.num_layers
    out: Dict[int, float] = {l: float("nan") for l in range(L)}
    dev, dt = model.enc_weight.device, model.enc_weight.dtype
    live = {l: (x.reshape(-1, x.shape[-1]) if x.dim() == 3 else x).to(device=dev, dtype=dt) for l, x in inputs.items() if x.numel() > 0}
    if not live:
        return out
    if model.config.activation_fn in ("batchtopk", "topk"):
        acts = model.get_feature_activations(live, gather=False)
        vals = {l: (a.abs() > 1e-8).sum(dim=1).float().mean() for l, a in acts.items() if a.shape[0] > 0}
    else:
        gen = torch.Generator(device="cpu")
        if seed is not None:
            gen.manual_seed(int(seed))
        else:
            gen.seed()
        vals = {}
        for l, x in live.items():
            n = min(int(num_tokens), x.shape[0])
            idx = torch.randperm(x.shape[0], generator=gen)[:n].to(dev)
            a = model.encode(x[idx], l, gather=False)
            vals[l] = (a.abs() > 1e-8).sum(dim=1).float().mean()
    if vals:
        layers = sorted(vals)
        t = torch.stack([vals[l] for l in layers])
        if model.world_size > 1:
            pops.all_reduce(t, group=model.process_group)
        for l, v in zip(layers, t.tolist()):
            out[l] = float(v)
    return out


@torch.no_grad()
def l0_for_scales(preact: torch.Tensor, theta: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """``L0(s) = mean_tokens #{f : x_f >= s * theta_f}`` for every ``s`` in the ascending vector ``scales``,
    from a single pass over ``preact [B, F]``."""
    if preact.is_cuda and preact.dtype in (torch.bfloat16, torch.float16) and preact.dim() == 2 and scales.numel() <= 1024:
        # one kernel pass over the 16-bit pre-activations (csrc/step.cu: scale_histogram_kernel)
        from .ops import ext

        hist = torch.empty(scales.numel() + 1, dtype=torch.int64, device=preact.device)
        ext.load().scale_histogram(preact.contiguous(), theta.float().contiguous(), scales.float().contiguous(), hist)
        active = torch.flip(torch.cumsum(torch.flip(hist.double(), dims=[0]), dim=0), dims=[0])[1:]
        return (active / preact.shape[0]).float()
    ratio = (preact.float() / theta.float().clamp_min(1e-30)).reshape(-1)
    ratio = ratio[ratio >= scales[0]]
    # number of scales that an element satisfies = index of the first scale above its ratio
    k = torch.bucketize(ratio, scales, right=True)  # in 1..len(scales)
    hist = torch.bincount(k, minlength=scales.numel() + 1).double()
    # elements with k >= j+1 are active at scale j
    active = torch.flip(torch.cumsum(torch.flip(hist, dims=[0]), dim=0), dims=[0])[1:]
    return (active / preact.shape[0]).float()


@torch.no_grad()
def calibrate_layerwise_theta(
    model,
    inputs: Dict[int, torch.Tensor],
    target_l0: Dict[int, float],
    tolerance: float = 0.5,
    scale_range: Tuple[float, float] = (0.1, 10.0),
    grid: int = 257,
    refine_steps: int = 12,
    max_tokens: Optional[int] = None,
    seed: Optional[int] = None,
) -> Dict[int, float]:
    """Scale every layer's threshold vector in place so that its L0 on ``inputs`` matches ``target_l0``.
    Returns the scale applied per layer.  ``scale_range`` and ``refine_steps`` are the reference's search
    range and iteration limit (``--l0-calibration-search-min/max-scale``, ``--l0-calibration-max-iters``);
    ``max_tokens`` draws one random sample of the calibration tokens (the reference re-samples <= 1024 tokens
    per probe; one fixed sample makes L0(s) monotone, so the search cannot oscillate)."""
    from .parallel import ops as pops

    if model.log_threshold is None:
        raise ValueError("calibration needs a JumpReLU model (log_threshold missing)")
    dev = model.log_threshold.device
    lo, hi = scale_range
    scales = torch.logspace(math.log10(lo), math.log10(hi), grid, device=dev)
    applied: Dict[int, float] = {}

    def count(pre, theta, s) -> float:
        c = (pre >= s * theta).float().sum() / pre.shape[0]
        if model.world_size > 1:
            pops.all_reduce(c, group=model.process_group)
        return float(c)

    for l in sorted(inputs):
        if l not in target_l0:
            continue
        x_l = inputs[l]
        if max_tokens is not None and x_l.shape[0] > max_tokens:
            gen = torch.Generator(device="cpu")
            gen.manual_seed(int(seed if seed is not None else 0) + l)
            x_l = x_l[torch.randperm(x_l.shape[0], generator=gen)[: int(max_tokens)].to(x_l.device)]
        pre16 = model.get_preactivations(x_l.to(dev), l, gather=False)
        pre = pre16.float()
        theta = model.log_threshold[l][: pre.shape[-1]].float().exp()
        l0s = l0_for_scales(pre16 if pre16.dtype in (torch.bfloat16, torch.float16) else pre, theta, scales)
        if model.world_size > 1:
            pops.all_reduce(l0s, group=model.process_group)
        tgt = float(target_l0[l])
        err = (l0s - tgt).abs()
        j = int(torch.argmin(err))
        best_s, best_err = float(scales[j]), float(err[j])
        if best_err > tolerance:
            # L0 falls with s: bisect exactly between the neighbours that bracket the target
            a = float(scales[max(j - 1, 0)])
            b = float(scales[min(j + 1, grid - 1)])
            for _ in range(refine_steps):
                mid = math.sqrt(a * b)
                v = count(pre, theta, mid)
                if abs(v - tgt) < best_err:
                    best_s, best_err = mid, abs(v - tgt)
                if best_err <= tolerance:
                    break
                if v > tgt:
                    a = mid
                else:
                    b = mid
        model.log_threshold.data[l] += math.log(best_s)
        applied[l] = best_s
        logger.info("layer %d: scale %.4f, |L0 - target| = %.3f (target %.2f)", l, best_s, best_err, tgt)
    return applied


@torch.no_grad()
def convert_model_to_jumprelu(
    model,
    data_iter: Iterable,
    num_batches: int,
    calibration_inputs: Optional[Dict[int, torch.Tensor]] = None,
    l0_tolerance: float = 0.5,
    default_theta_value: float = 1e6,
):
    """Estimate thresholds, convert ``model`` in place and (when calibration tokens are given) match the
    original model's layer-wise L0.  Returns ``(report, scales)``."""
    report: Dict[str, Dict[int, float]] = {}
    original = None
    if calibration_inputs is not None:
        report["l0_original"] = layer_l0(model, calibration_inputs)
    model.estimate_theta_posthoc(data_iter, num_batches=num_batches, default_theta_value=default_theta_value)
    scales: Dict[int, float] = {}
    if calibration_inputs is not None:
        report["l0_converted"] = layer_l0(model, calibration_inputs)
        scales = calibrate_layerwise_theta(model, calibration_inputs, report["l0_original"], tolerance=l0_tolerance)
        report["l0_calibrated"] = layer_l0(model, calibration_inputs)
    return report, scales
