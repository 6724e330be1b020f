"""Activation extraction with forward hooks on a tiny randomly initialised GPT-2 (built from a config: no network),
and the numeric ordering of layer groups in chunk files (layer_2 before layer_10)."""
import numpy as np
import pytest
import torch

from crosslayer_coding_b200.activation_generation.extractor import ActivationExtractorCLT
from crosslayer_coding_b200.io import hdf5

transformers = pytest.importorskip("transformers")


class _Tok:
    """Whitespace tokenizer with padding: enough of the HF interface for the extractor."""

    pad_token_id, eos_token_id = 0, 1
    all_special_ids = [0, 1]

    def _ids(self, text):
        return [2 + (hash(w) % 90) for w in text.split()]

    def __call__(self, texts, truncation=True, max_length=None, padding=None, return_tensors=None, add_special_tokens=True):
        if isinstance(texts, str):
            return {"input_ids": self._ids(texts)}
        ids = [self._ids(t)[: max_length or 10 ** 9] for t in texts]
        width = max(len(i) for i in ids)
        inp = torch.tensor([i + [0] * (width - len(i)) for i in ids])
        mask = torch.tensor([[1] * len(i) + [0] * (width - len(i)) for i in ids])
        return {"input_ids": inp, "attention_mask": mask}

    def decode(self, ids):
        return " ".join(f"w{i}" for i in ids)


@pytest.fixture(scope="module")
def tiny_gpt2():
    cfg = transformers.GPT2Config(n_layer=3, n_embd=32, n_head=2, n_positions=64, vocab_size=100)
    torch.manual_seed(0)
    return transformers.GPT2LMHeadModel(cfg)


def test_extractor_captures_mlp_inputs_and_outputs(tiny_gpt2):
    ex = ActivationExtractorCLT("tiny-gpt2", "transformer.h.{}.ln_2.input", "transformer.h.{}.mlp.output", device="cpu",
                                context_size=16, inference_batch_size=2, model=tiny_gpt2, tokenizer=_Tok())
    assert ex.num_layers == 3
    ids = torch.randint(2, 100, (2, 7))
    mask = torch.ones_like(ids)
    mask[1, 5:] = 0
    inputs, targets = ex.extract_from_ids(ids, mask)
    assert set(inputs) == {0, 1, 2} and inputs[0].shape == (12, 32) and targets[2].shape == (12, 32)  # padding dropped
    # the hooks see what the modules see: recompute layer 0 by hand
    with torch.no_grad():
        h = tiny_gpt2.transformer.wte(ids) + tiny_gpt2.transformer.wpe(torch.arange(7))[None]
        blk = tiny_gpt2.transformer.h[0]
        h = h + blk.attn(blk.ln_1(h), attention_mask=None)[0]  # no padding effect on the first rows of row 0
    assert torch.allclose(inputs[0][:7], h[0], atol=1e-4)
    with torch.no_grad():
        want = blk.mlp(blk.ln_2(h[0:1]))[0]
    assert torch.allclose(targets[0][:7], want, atol=1e-4)


def test_extractor_streams_batches_from_an_iterable(tiny_gpt2):
    ex = ActivationExtractorCLT("tiny-gpt2", "transformer.h.{}.ln_2.input", "transformer.h.{}.mlp.output", device="cpu",
                                context_size=8, inference_batch_size=2, model=tiny_gpt2, tokenizer=_Tok(), exclude_special_tokens=True)
    docs = [{"text": "a b c d e"}, {"text": "f g h"}, {"text": " ".join(f"t{i}" for i in range(20))}]  # the last one is split
    batches = list(ex.stream_activations(docs))
    total = sum(b[0][0].shape[0] for b in batches)
    assert total == 5 + 3 + 20
    assert all(b[0][l].shape == b[1][l].shape for b in batches for l in range(3))


def test_layer_groups_are_ordered_numerically(tmp_path):
    path = str(tmp_path / "chunk_0.hdf5")
    w = hdf5.H5Writer(path)
    for l in (100, 2, 10, 1, 20):
        w.add(f"layer_{l}", "inputs", np.full((4, 8), float(l), dtype=np.float32))
        w.add(f"layer_{l}", "targets", np.full((4, 8), -float(l), dtype=np.float32))
    w.close()
    with hdf5.H5File(path) as f:
        assert f.layer_groups() == ["layer_1", "layer_2", "layer_10", "layer_20", "layer_100"]
        assert float(f["layer_10/inputs"].read_rows([0])[0, 0]) == 10.0


def test_collect_top_activations_with_base_model_in_the_loop(tiny_gpt2, tmp_path):
    """The analysis script's base-model mode: text -> tiny GPT-2 (hooks) -> clt.encode -> per-feature top sequences with
    token text, in the reference's JSON layout."""
    import importlib.util
    import json
    import os
    import types

    from crosslayer_coding_b200 import CLTConfig, CrossLayerTranscoder

    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("collect_top", os.path.join(repo, "scripts", "analysis", "collect_top_activations.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    cfg = CLTConfig(num_features=12, num_layers=3, d_model=32, activation_fn="relu", normalization_method="none")
    torch.manual_seed(1)
    clt = CrossLayerTranscoder(cfg)
    ex = ActivationExtractorCLT("tiny-gpt2", "transformer.h.{}.ln_2.input", "transformer.h.{}.mlp.output", device="cpu",
                                context_size=8, inference_batch_size=2, model=tiny_gpt2, tokenizer=_Tok())
    texts = ["a b c d", "e f g", "h i j k l", "m n", "o p q r s t"]
    args = types.SimpleNamespace(layer=1, topk_per_feature=2, batch_size=2, max_dataset_samples=None, clt_config=str(tmp_path / "cfg.json"),
                                 output_json=str(tmp_path / "out" / "top.json"), features_per_file=5, mlp_input_template="x", mlp_output_template="y",
                                 context_size=8, model_name="tiny", dataset=None, dataset_split="validation", dataset_text_column="text")
    files = mod.run_with_base_model(args, clt, torch.device("cpu"), extractor=ex, texts=texts)
    assert len(files) == 3 and files[0].endswith("top_features_0_to_4.json")
    merged = {}
    for f in files:
        merged.update(json.load(open(f)))
    assert sorted(merged, key=int) == [str(i) for i in range(12)]
    # oracle: encode every sequence by itself
    best = {}
    for sid, t in enumerate(texts):
        ids, mask, x = ex.capture_layer_sequences([t], 1)
        a = clt.encode(x[0].float(), 1)
        for f in range(12):
            best.setdefault(f, []).append((float(a[:, f].max()), sid, a[:, f].tolist()))
    for f in range(12):
        want = sorted(best[f], reverse=True)[:2]
        got = merged[str(f)]["activations"]
        assert abs(got["0"]["score"] - want[0][0]) < 1e-4 and abs(got["1"]["score"] - want[1][0]) < 1e-4
        assert len(got["0"]["text"]) == len(got["0"]["values"])
        if want[0][0] - sorted(best[f], reverse=True)[1][0] > 1e-6:  # a unique best sequence (equal scores may come in any order)
            assert len(got["0"]["text"]) == len(texts[want[0][1]].split())
            assert all(abs(u - v) < 1e-4 for u, v in zip(got["0"]["values"], want[0][2]))
