#!/usr/bin/env python
"""JumpReLU hyper-parameter grid: sparsity coefficient c, lambda, initial threshold and seed
(reference: tutorials/jumprelu_sparsity_sweep.py).  Prints one line per run: final L0 and normalised MSE.

    python tutorials/jumprelu_sparsity_sweep.py
"""
import itertools
import os

import torch

from _common import clt_config, dataset, device, training_config, workdir

from crosslayer_coding_b200.training.trainer import CLTTrainer


def main() -> None:
    root = workdir("sweep")
    data = dataset(os.path.join(root, "activations"))
    grid = itertools.product([1.0, 3.0], [1e-3, 1e-2], [0.03, 0.1], [0])
    for c, lam, theta, seed in grid:
        name = f"c{c}_lam{lam}_th{theta}_s{seed}"
        cfg = clt_config(activation_fn="jumprelu", jumprelu_threshold=theta)
        tc = training_config(data, steps=40, sparsity_lambda=lam, sparsity_c=c, seed=seed, eval_interval=10 ** 9,
                             checkpoint_interval=10 ** 9)
        trainer = CLTTrainer(cfg, tc, log_dir=os.path.join(root, name), device=device())
        model = trainer.train()
        inputs, targets = next(iter(trainer.activation_store))
        with torch.no_grad():
            acts = model.get_feature_activations(inputs)
            out = model(inputs)
        l0 = sum(float((a != 0).float().sum(-1).mean()) for a in acts.values())
        num = sum(((out[l].float() - targets[l].float()) ** 2).sum() for l in out)
        den = sum((targets[l].float() ** 2).sum() for l in out)
        print(f"{name}: total L0 {l0:.1f}, normalised MSE {float(num / den):.4f}")


if __name__ == "__main__":
    main()
