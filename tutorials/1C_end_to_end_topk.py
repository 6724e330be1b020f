#!/usr/bin/env python
"""Tutorial 1C - per-token TopK: every token keeps its ``topk_k`` highest-ranked features across all layers
(reference walk-through: tutorials/1C-end-to-end-training-pythia-topk.py).

``topk_k >= 1`` is a count, ``topk_k < 1`` a fraction of the ``num_layers * num_features`` features of a token
(clt/models/activations.py:101-128).  Ranking uses the per-feature batch z-scores, the kept values are the raw
pre-activations.  On a B200 with bf16 weights the step is the fused one with the exact per-token radix selection.

    python tutorials/1C_end_to_end_topk.py
"""
import os

import torch

from _common import clt_config, dataset, device, training_config, workdir

from crosslayer_coding_b200 import CrossLayerTranscoder
from crosslayer_coding_b200.training.trainer import CLTTrainer


def main() -> None:
    root = workdir("1C")
    data = dataset(os.path.join(root, "activations"))
    for name, k in (("count", 16.0), ("fraction", 0.01)):
        cfg = clt_config(activation_fn="topk", topk_k=k, batchtopk_k=None)
        trainer = CLTTrainer(cfg, training_config(data, steps=40), log_dir=os.path.join(root, name), device=device())
        model = trainer.train()
        inputs, _ = next(iter(trainer.activation_store))
        with torch.no_grad():
            acts = model.get_feature_activations(inputs)
        per_token = sum((a != 0).sum(-1) for a in acts.values())
        print(f"topk_k={k}: active features per token min/max = {int(per_token.min())}/{int(per_token.max())}")
    path = os.path.join(root, "topk.safetensors")
    model.save(path)
    again = CrossLayerTranscoder.load(path, device=torch.device(device()))
    print("reloaded:", again.config.activation_fn, "topk_k =", again.config.topk_k)


if __name__ == "__main__":
    main()
