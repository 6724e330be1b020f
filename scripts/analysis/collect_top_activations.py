#!/usr/bin/env python
"""Top-activating tokens per feature of one layer (reference: scripts/analysis/collect_top_activations.py:100-586).

Streams ``(inputs, targets)`` batches from an activation dataset, runs ``model.encode`` for ``--layer`` and keeps,
for every feature, the ``--top-k`` largest activations with their global token positions (a vectorised running
top-k on the device instead of one Python min-heap per feature).  Output: JSON shards
``{feature: [[activation, token_index], ...]}``.  With a Hugging Face model and tokenizer available the same loop
can be fed by ``ActivationExtractorCLT.stream_activations`` to attach token text.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent.parent))

from crosslayer_coding_b200 import CLTConfig, CrossLayerTranscoder  # noqa: E402
from crosslayer_coding_b200.training.data import LocalActivationStore  # noqa: E402


@torch.no_grad()
def collect(model, store, layer: int, top_k: int, max_batches: int):
    F = model.config.num_features
    dev = model.enc_weight.device
    best_v = torch.full((top_k, F), float("-inf"), device=dev)
    best_i = torch.full((top_k, F), -1, dtype=torch.long, device=dev)
    seen = 0
    for b, (x, _) in enumerate(store):
        if b >= max_batches:
            break
        a = model.encode(x[layer], layer).float()  # [B, F]
        idx = torch.arange(seen, seen + a.shape[0], device=dev).unsqueeze(1).expand_as(a)
        v = torch.cat([best_v, a])
        i = torch.cat([best_i, idx])
        top = torch.topk(v, top_k, dim=0)
        best_v, best_i = top.values, torch.gather(i, 0, top.indices)
        seen += a.shape[0]
    return best_v.cpu(), best_i.cpu(), seen


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--checkpoint", required=True)
    ap.add_argument("--config", required=True)
    ap.add_argument("--activation-path", required=True)
    ap.add_argument("--layer", type=int, required=True)
    ap.add_argument("--top-k", type=int, default=20)
    ap.add_argument("--max-batches", type=int, default=100)
    ap.add_argument("--batch-size-tokens", type=int, default=4096)
    ap.add_argument("--output-dir", required=True)
    ap.add_argument("--features-per-shard", type=int, default=4096)
    ap.add_argument("--device", default=None)
    args = ap.parse_args(argv)
    dev = torch.device(args.device or ("cuda" if torch.cuda.is_available() else "cpu"))
    cfg = CLTConfig.from_json(args.config)
    model = CrossLayerTranscoder(cfg, device=dev)
    from safetensors.torch import load_file

    model.load_state_dict(load_file(args.checkpoint))
    if cfg.activation_fn in ("batchtopk", "topk"):
        cfg.topk_mode = "per_layer"  # encode() of a single layer ranks within that layer
    store = LocalActivationStore(args.activation_path, train_batch_size_tokens=args.batch_size_tokens, device=dev, dtype="float32",
                                 normalization_method="auto", shard_data=False)
    vals, idx, seen = collect(model, store, args.layer, args.top_k, args.max_batches)
    store.close()
    os.makedirs(args.output_dir, exist_ok=True)
    F = cfg.num_features
    for s in range(0, F, args.features_per_shard):
        shard = {}
        for f in range(s, min(F, s + args.features_per_shard)):
            keep = vals[:, f] > 0
            if keep.any():
                shard[str(f)] = [[float(v), int(i)] for v, i in zip(vals[keep, f], idx[keep, f])]
        with open(os.path.join(args.output_dir, f"layer{args.layer}_features_{s}.json"), "w") as fh:
            json.dump({"layer": args.layer, "tokens_seen": seen, "features": shard}, fh)
    print(args.output_dir)
    return 0


if __name__ == "__main__":
    sys.exit(main())
