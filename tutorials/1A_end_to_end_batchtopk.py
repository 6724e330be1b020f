#!/usr/bin/env python
"""Tutorial 1A - generate activations, train a BatchTopK CLT, save, reload, evaluate
(reference walk-through: tutorials/1A-end-to-end-training-gpt2-relu.py and its BatchTopK sibling).

    python tutorials/1A_end_to_end_batchtopk.py
"""
import os

import torch

from _common import clt_config, dataset, device, training_config, workdir

from crosslayer_coding_b200 import CrossLayerTranscoder
from crosslayer_coding_b200.training.trainer import CLTTrainer


def main() -> None:
    root = workdir("1A")
    data = dataset(os.path.join(root, "activations"))
    trainer = CLTTrainer(clt_config(), training_config(data), log_dir=os.path.join(root, "run"), device=device())
    model = trainer.train()

    # save / reload: safetensors weights + cfg.json, reference key names
    path = os.path.join(root, "model.safetensors")
    model.save(path)
    again = CrossLayerTranscoder.load(path, device=torch.device(device()))
    batch = next(iter(trainer.activation_store))
    inputs, targets = batch
    with torch.no_grad():
        out = again(inputs)
    num = sum(((out[l].float() - targets[l].float()) ** 2).sum() for l in out)
    den = sum((targets[l].float() ** 2).sum() for l in out)
    print(f"reloaded model, normalised MSE on one batch: {float(num / den):.4f}")
    acts = again.get_feature_activations(inputs)
    print("active features per token and layer:", [round(float((a != 0).float().sum(-1).mean()), 1) for a in acts.values()])


if __name__ == "__main__":
    main()
