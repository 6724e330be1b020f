#!/usr/bin/env python
"""Tutorial 1B - train with BatchTopK, convert to JumpReLU thresholds, calibrate the layer-wise L0
(reference: tutorials/1B-end-to-end-training-gpt2-batchtopk.py:300-470 and scripts/convert_batchtopk_to_jumprelu.py).

    python tutorials/1B_theta_conversion.py
"""
import os

import torch

from _common import clt_config, dataset, device, training_config, workdir

from crosslayer_coding_b200.conversion import convert_model_to_jumprelu, layer_l0
from crosslayer_coding_b200.training.trainer import CLTTrainer


def main() -> None:
    root = workdir("1B")
    data = dataset(os.path.join(root, "activations"))
    trainer = CLTTrainer(clt_config(), training_config(data), log_dir=os.path.join(root, "run"), device=device())
    model = trainer.train()
    store = trainer.activation_store
    calib_inputs, _ = next(iter(store))
    before = layer_l0(model, calib_inputs)
    report, scales = convert_model_to_jumprelu(model, iter(store), num_batches=8, calibration_inputs=calib_inputs, l0_tolerance=0.5)
    after = layer_l0(model, calib_inputs)
    print("activation function is now:", model.config.activation_fn)
    for l in sorted(before):
        print(f"layer {l}: L0 batchtopk {before[l]:.2f} -> jumprelu {after[l]:.2f} (scale {scales.get(l, 1.0):.3f})")
    model.save(os.path.join(root, "jumprelu.safetensors"))
    # on a B200 the converted model runs through the sparse inference path
    if torch.cuda.is_available():
        from crosslayer_coding_b200.models.sparse_forward import SparseForward, supports

        print("sparse forward available:", supports(model) is None or supports(model))


if __name__ == "__main__":
    main()
