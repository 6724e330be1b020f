#!/usr/bin/env python
"""Top-activating examples per feature of one layer (reference: scripts/analysis/collect_top_activations.py:100-586).

Two sources of activations:

* **base model in the loop** (the reference's mode): ``--model-name`` + ``--dataset`` stream text through the Hugging
  Face model (``ActivationExtractorCLT`` hooks on the MLP input of ``--layer``), the activations are normalised with
  the ``norm_stats.json`` that lies next to the CLT config (when the config asks for it), ``clt.encode`` gives the
  feature activations per token, and every feature keeps its ``--topk-per-feature`` sequences ranked by the
  sequence's largest activation.  Output, as in the reference, one or several JSON files::

      {"<feature>": {"activations": {"<rank>": {"text": [decoded tokens], "values": [activation per token], "score": max}}}}

  ``--dataset`` may also be a local ``.txt`` (one document per line) or ``.jsonl`` file (no network needed).
* **stored activation dataset** (``--activation-path``): no base model; features keep their largest activations with
  the global token index, and ``--context-window`` neighbouring token indices around each hit.

The reference pushes every (sequence, feature) pair through a Python heap; here the candidates of a batch are
ranked on the device (per-sequence maxima ``[b, F]``, running top-k ``[k, F]``) and only sequences that enter some
feature's top-k are brought to the host.
"""
from __future__ import annotations

import argparse
import json
import logging
import os
import sys
from pathlib import Path
from typing import Dict, Iterable, List, Optional

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent.parent))

from crosslayer_coding_b200 import CLTConfig, CrossLayerTranscoder  # noqa: E402

logger = logging.getLogger("collect_top_activations")


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description="Collect top activating examples for CLT features.")
    ap.add_argument("--clt-checkpoint", "--checkpoint", dest="clt_checkpoint", required=True, help="CLT checkpoint (.safetensors or .pt)")
    ap.add_argument("--clt-config", "--config", dest="clt_config", required=True, help="cfg.json of the CLT")
    ap.add_argument("--model-name", default=None, help="base Hugging Face model (e.g. gpt2)")
    ap.add_argument("--dataset", default=None, help="Hugging Face dataset name, or a local .txt / .jsonl file")
    ap.add_argument("--dataset-split", default="validation")
    ap.add_argument("--dataset-text-column", default="text")
    ap.add_argument("--layer", type=int, default=0)
    ap.add_argument("--topk-per-feature", "--top-k", dest="topk_per_feature", type=int, default=10)
    ap.add_argument("--batch-size", type=int, default=32, help="texts per forward pass of the base model")
    ap.add_argument("--context-size", type=int, default=128)
    ap.add_argument("--device", default=None)
    ap.add_argument("--output-json", default="./top_activating_examples.json")
    ap.add_argument("--max-dataset-samples", type=int, default=None)
    ap.add_argument("--mlp-input-template", default="transformer.h.{}.mlp.c_fc")
    ap.add_argument("--mlp-output-template", default="transformer.h.{}.mlp.c_proj")
    ap.add_argument("--features-per-file", "--features-per-shard", dest="features_per_file", type=int, default=1000,
                    help="features per output file; 0 writes a single file")
    # stored-dataset mode
    ap.add_argument("--activation-path", default=None, help="activation dataset directory (no base model needed)")
    ap.add_argument("--max-batches", type=int, default=100)
    ap.add_argument("--batch-size-tokens", type=int, default=4096)
    ap.add_argument("--context-window", type=int, default=0, help="stored-dataset mode: token indices kept on each side of a hit")
    ap.add_argument("--output-dir", default=None, help="stored-dataset mode: directory of the JSON shards")
    return ap.parse_args(argv)


def load_clt(checkpoint: str, config: str, device) -> CrossLayerTranscoder:
    cfg = CLTConfig.from_json(config)
    model = CrossLayerTranscoder(cfg, device=device)
    if checkpoint.endswith(".safetensors"):
        from safetensors.torch import load_file

        sd = load_file(checkpoint)
    else:
        blob = torch.load(checkpoint, map_location="cpu", weights_only=False)
        sd = blob.get("state_dict", blob) if isinstance(blob, dict) else blob.state_dict()
    sd = {(k[len("module."):] if k.startswith("module.") else k): v for k, v in sd.items()}
    model.load_state_dict(sd)
    model.eval()
    if cfg.activation_fn in ("batchtopk", "topk"):
        cfg.topk_mode = "per_layer"  # encode() of a single layer ranks within that layer
    return model


def load_input_norm(config_path: str, layer: int, d_model: int, device):
    """``(mean [1, d], std [1, d])`` of the layer's inputs from the norm_stats.json beside the config, or None."""
    path = Path(config_path).resolve().parent / "norm_stats.json"
    if not path.exists():
        logger.warning("normalisation requested but %s does not exist; encoding raw activations", path)
        return None
    try:
        stats = json.load(open(path)).get(str(layer), {}).get("inputs")
    except json.JSONDecodeError as exc:
        logger.error("cannot parse %s: %s", path, exc)
        return None
    if not stats or len(stats.get("mean", [])) != d_model or len(stats.get("std", [])) != d_model:
        logger.warning("no usable input statistics for layer %d in %s", layer, path)
        return None
    return (torch.tensor(stats["mean"], device=device).unsqueeze(0), (torch.tensor(stats["std"], device=device) + 1e-6).unsqueeze(0))


def iter_texts(dataset: str, split: str, column: str) -> Iterable[str]:
    if os.path.isfile(dataset):
        with open(dataset) as fh:
            for line in fh:
                line = line.rstrip("\n")
                if not line.strip():
                    continue
                if dataset.endswith(".jsonl"):
                    yield json.loads(line)[column]
                else:
                    yield line
        return
    from datasets import load_dataset

    for item in load_dataset(dataset, split=split, streaming=True):
        text = item[column]
        if isinstance(text, str) and text.strip():
            yield text


class TopSequences:
    """Per-feature top-k sequences, ranked by the sequence's largest activation of that feature."""

    def __init__(self, num_features: int, k: int, device):
        self.k, self.F = k, num_features
        self.score = torch.full((k, num_features), float("-inf"), device=device)
        self.seq = torch.full((k, num_features), -1, dtype=torch.long, device=device)
        self.tokens: Dict[int, List[str]] = {}
        self.values: Dict[tuple, List[float]] = {}

    @torch.no_grad()
    def update(self, acts: torch.Tensor, mask: torch.Tensor, seq_ids: torch.Tensor, decoded: List[List[str]]) -> None:
        """``acts [b, s, F]``, ``mask [b, s]`` (1 = real token), ``seq_ids [b]`` global ids, ``decoded[b]`` token strings."""
        b = acts.shape[0]
        masked = acts.masked_fill(~mask.bool().unsqueeze(-1), float("-inf"))
        best = masked.max(dim=1).values                                   # [b, F]
        cand_score = torch.cat([self.score, best])
        cand_seq = torch.cat([self.seq, seq_ids.unsqueeze(1).expand(b, self.F)])
        top = torch.topk(cand_score, self.k, dim=0)
        self.score = top.values
        self.seq = torch.gather(cand_seq, 0, top.indices)
        entered = top.indices >= self.k                                   # slots now held by a sequence of this batch
        if not bool(entered.any()):
            return
        slot, feat = entered.nonzero(as_tuple=True)
        local = top.indices[slot, feat] - self.k                          # row inside this batch
        lengths = mask.sum(dim=1).tolist()
        vals = acts[local, :, feat].float().cpu()                         # [n, s]
        for j, (row, f) in enumerate(zip(local.tolist(), feat.tolist())):
            sid = int(seq_ids[row])
            self.tokens.setdefault(sid, decoded[row])
            self.values[(sid, f)] = vals[j, : int(lengths[row])].tolist()

    def result(self) -> Dict[str, dict]:
        score, seq = self.score.cpu(), self.seq.cpu()
        out: Dict[str, dict] = {}
        for f in range(self.F):
            entry = {}
            rank = 0
            for r in range(self.k):
                sid = int(seq[r, f])
                if sid < 0 or (sid, f) not in self.values:
                    continue
                entry[str(rank)] = {"text": self.tokens[sid], "values": self.values[(sid, f)], "score": float(score[r, f])}
                rank += 1
            out[str(f)] = {"activations": entry}
        return out


def write_feature_files(result: Dict[str, dict], output_json: str, features_per_file: int) -> List[str]:
    base = Path(output_json)
    base.parent.mkdir(parents=True, exist_ok=True)
    n = len(result)
    per = n if features_per_file <= 0 else features_per_file
    written = []
    keys = sorted(result, key=int)
    for start in range(0, n, max(1, per)):
        part = {k: result[k] for k in keys[start : start + per]}
        path = base if n <= per else base.parent / f"{base.stem}_features_{start}_to_{min(n, start + per) - 1}{base.suffix}"
        with open(path, "w") as fh:
            json.dump(part, fh, indent=2)
        written.append(str(path))
    return written


@torch.no_grad()
def run_with_base_model(args, clt, device, extractor=None, texts: Optional[Iterable[str]] = None) -> List[str]:
    from crosslayer_coding_b200.activation_generation.extractor import ActivationExtractorCLT

    cfg = clt.config
    tin = cfg.mlp_input_template or args.mlp_input_template
    tout = cfg.mlp_output_template or args.mlp_output_template
    if extractor is None:
        extractor = ActivationExtractorCLT(args.model_name, tin, tout, device=device, context_size=args.context_size,
                                           inference_batch_size=args.batch_size)
    norm = load_input_norm(args.clt_config, args.layer, cfg.d_model, device) if cfg.normalization_method in ("auto", "mean_std") else None
    tops = TopSequences(cfg.num_features, args.topk_per_feature, device)
    buf: List[str] = []
    seen = 0

    def flush():
        nonlocal seen
        ids, mask, x = extractor.capture_layer_sequences(buf, args.layer)
        b, s, d = x.shape
        flat = x.reshape(b * s, d).float()
        if norm is not None:
            flat = (flat - norm[0]) / norm[1]
        acts = clt.encode(flat, args.layer).float().reshape(b, s, -1)
        tok = extractor.tokenizer
        decoded = [[tok.decode([int(t)]) for t in ids[i, : int(mask[i].sum())]] for i in range(b)]
        tops.update(acts, mask, torch.arange(seen, seen + b, device=device), decoded)
        seen += b

    source = texts if texts is not None else iter_texts(args.dataset, args.dataset_split, args.dataset_text_column)
    for text in source:
        if args.max_dataset_samples is not None and seen + len(buf) >= args.max_dataset_samples:
            break
        buf.append(text)
        if len(buf) >= args.batch_size:
            flush()
            buf = []
    if buf:
        flush()
    logger.info("processed %d sequences", seen)
    return write_feature_files(tops.result(), args.output_json, args.features_per_file)


@torch.no_grad()
def run_on_stored_dataset(args, clt, device) -> str:
    from crosslayer_coding_b200.training.data import LocalActivationStore

    F, k = clt.config.num_features, args.topk_per_feature
    best_v = torch.full((k, F), float("-inf"), device=device)
    best_i = torch.full((k, F), -1, dtype=torch.long, device=device)
    store = LocalActivationStore(args.activation_path, train_batch_size_tokens=args.batch_size_tokens, device=device, dtype="float32",
                                 normalization_method="auto", shard_data=False)
    seen = 0
    for b, (x, _) in enumerate(store):
        if b >= args.max_batches:
            break
        a = clt.encode(x[args.layer], args.layer).float()
        idx = torch.arange(seen, seen + a.shape[0], device=device).unsqueeze(1).expand_as(a)
        top = torch.topk(torch.cat([best_v, a]), k, dim=0)
        best_v, best_i = top.values, torch.gather(torch.cat([best_i, idx]), 0, top.indices)
        seen += a.shape[0]
    store.close()
    vals, idx = best_v.cpu(), best_i.cpu()
    out_dir = args.output_dir or str(Path(args.output_json).parent)
    os.makedirs(out_dir, exist_ok=True)
    per = F if args.features_per_file <= 0 else args.features_per_file
    w = args.context_window
    for s in range(0, F, per):
        shard = {}
        for f in range(s, min(F, s + per)):
            keep = vals[:, f] > 0
            if keep.any():
                hits = []
                for v, i in zip(vals[keep, f], idx[keep, f]):
                    hit = [float(v), int(i)]
                    if w > 0:
                        hit.append([max(0, int(i) - w), min(seen - 1, int(i) + w)])
                    hits.append(hit)
                shard[str(f)] = hits
        with open(os.path.join(out_dir, f"layer{args.layer}_features_{s}.json"), "w") as fh:
            json.dump({"layer": args.layer, "tokens_seen": seen, "features": shard}, fh)
    return out_dir


def main(argv=None) -> int:
    logging.basicConfig(level=logging.INFO, format="%(asctime)s %(name)s %(levelname)s %(message)s")
    args = parse_args(argv)
    device = torch.device(args.device or ("cuda" if torch.cuda.is_available() else "cpu"))
    clt = load_clt(args.clt_checkpoint, args.clt_config, device)
    if args.activation_path:
        print(run_on_stored_dataset(args, clt, device))
        return 0
    if not args.model_name or not args.dataset:
        raise SystemExit("give --model-name and --dataset (base model in the loop) or --activation-path (stored dataset)")
    for path in run_with_base_model(args, clt, device):
        print(path)
    return 0


if __name__ == "__main__":
    sys.exit(main())
