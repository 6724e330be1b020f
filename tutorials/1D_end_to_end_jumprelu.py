#!/usr/bin/env python
"""Tutorial 1D - JumpReLU with learned thresholds, trained with the tanh sparsity penalty and the pre-activation
loss (reference walk-through: tutorials/1D-end-to-end-training-pythia-jumprelu.py).

The thresholds ``exp(log_threshold[l, f])`` get their gradient through the rectangle window of width ``bandwidth``
around the threshold (clt/models/activations.py:183-220); the sparsity weight ramps up linearly over the run
(clt/training/losses.py:117-137).  On a B200 pass ``engine="fused"`` to ``CLTTrainer`` for the fused step with the
threshold-gradient GEMM (bf16 weights).

    python tutorials/1D_end_to_end_jumprelu.py
"""
import os

import torch

from _common import clt_config, dataset, device, training_config, workdir

from crosslayer_coding_b200 import CrossLayerTranscoder
from crosslayer_coding_b200.training.trainer import CLTTrainer


def l0(model, inputs) -> float:
    with torch.no_grad():
        acts = model.get_feature_activations(inputs)
    return float(sum((a != 0).float().sum(-1).mean() for a in acts.values()))


def main() -> None:
    root = workdir("1D")
    data = dataset(os.path.join(root, "activations"))
    cfg = clt_config(activation_fn="jumprelu", jumprelu_threshold=0.03, batchtopk_k=None)
    tc = training_config(data, steps=80, sparsity_lambda=1e-4, sparsity_lambda_schedule="linear", sparsity_c=1.0,
                         preactivation_coef=3e-6, compute_sparsity_diagnostics=True)
    trainer = CLTTrainer(cfg, tc, log_dir=os.path.join(root, "run"), device=device())
    inputs, _ = next(iter(trainer.activation_store))
    before = l0(trainer.model, inputs)
    theta0 = trainer.model.log_threshold.detach().exp().mean().item()
    model = trainer.train()
    print(f"active features per token: {before:.1f} -> {l0(model, inputs):.1f}")
    print(f"mean threshold: {theta0:.4f} -> {model.log_threshold.detach().exp().mean().item():.4f}")
    path = os.path.join(root, "jumprelu.safetensors")
    model.save(path)
    again = CrossLayerTranscoder.load(path, device=torch.device(device()))
    assert torch.equal(again.log_threshold.detach().cpu(), model.log_threshold.detach().cpu())
    print("reloaded model with trained thresholds")


if __name__ == "__main__":
    main()
