"""Paired MLP-input / MLP-output activation extraction from a Hugging Face transformer.

Same constructor and ``stream_activations`` contract as the reference ``ActivationExtractorCLT``
(clt/nnsight/extractor.py:13-441): module paths are dotted templates with ``{}`` for the layer index
(integer path components index into module lists), long documents are split into ``context_size``-token
chunks, batches of ``inference_batch_size`` texts are tokenised with ``padding="longest"``, activations are
flattened ``[batch, seq, d] -> [batch*seq, d]`` and padding tokens are dropped by the attention mask; each
yield is ``(inputs, targets)`` with one ``[n_valid_tokens, d]`` tensor per layer.

The reference traces the model through ``nnsight``; here plain forward hooks on the resolved modules capture the
MLP *input* (pre-hook) and *output* (hook), so nothing beyond ``transformers`` is needed.  The model and the
dataset can also be passed in as objects (used by the tests and for offline work).
"""
from __future__ import annotations

import logging
from typing import Any, Dict, Generator, Iterable, List, Optional, Tuple, Union

import torch

logger = logging.getLogger(__name__)

ActivationPair = Tuple[Dict[int, torch.Tensor], Dict[int, torch.Tensor]]


class ActivationExtractorCLT:
    def __init__(
        self,
        model_name: str,
        mlp_input_module_path_template: str,
        mlp_output_module_path_template: str,
        device: Optional[Union[str, torch.device]] = None,
        model_dtype: Optional[Union[str, torch.dtype]] = None,
        context_size: int = 128,
        inference_batch_size: int = 512,
        exclude_special_tokens: bool = True,
        prepend_bos: bool = False,
        nnsight_tracer_kwargs: Optional[Dict] = None,
        nnsight_invoker_args: Optional[Dict] = None,
        batchtopk_k: Optional[int] = None,
        model: Optional[torch.nn.Module] = None,
        tokenizer: Optional[Any] = None,
    ):
        self.model_name = model_name
        self.device = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
        self.model_dtype = self._resolve_dtype(model_dtype)
        self.context_size = context_size
        self.inference_batch_size = inference_batch_size
        self.mlp_input_module_path_template = mlp_input_module_path_template
        self.mlp_output_module_path_template = mlp_output_module_path_template
        self.exclude_special_tokens = exclude_special_tokens
        self.prepend_bos = prepend_bos
        self.batchtopk_k = batchtopk_k
        self.tokenizer_args = {"truncation": True, "max_length": context_size, "padding": "longest", "return_tensors": "pt"}
        # accepted for signature compatibility; there is no tracer here
        self.nnsight_tracer_kwargs = nnsight_tracer_kwargs or {}
        self.nnsight_invoker_args = nnsight_invoker_args or {}
        if model is not None:
            self.model, self.tokenizer = model.to(self.device), tokenizer
        else:
            self.model, self.tokenizer = self._load_model_and_tokenizer()
        self.model.eval()
        self.num_layers = self._get_num_layers()

    @staticmethod
    def _resolve_dtype(dtype_input) -> Optional[torch.dtype]:
        if isinstance(dtype_input, torch.dtype):
            return dtype_input
        if isinstance(dtype_input, str):
            dt = getattr(torch, dtype_input, None)
            if isinstance(dt, torch.dtype):
                return dt
            logger.warning("Unsupported dtype string %r; ignoring", dtype_input)
        return None

    def _load_model_and_tokenizer(self):
        from transformers import AutoModelForCausalLM, AutoTokenizer

        tok = AutoTokenizer.from_pretrained(self.model_name)
        if tok.pad_token is None:
            tok.pad_token = tok.eos_token
        model = AutoModelForCausalLM.from_pretrained(self.model_name, torch_dtype=self.model_dtype)
        return model.to(self.device), tok

    def _get_num_layers(self) -> int:
        cfg = getattr(self.model, "config", None)
        for name in ("num_hidden_layers", "n_layer", "num_layers", "n_layers"):
            if cfg is not None and isinstance(getattr(cfg, name, None), int):
                return int(getattr(cfg, name))
        # fall back to probing the template
        n = 0
        while True:
            try:
                self._resolve_module(self.mlp_input_module_path_template.format(n))
            except (AttributeError, IndexError, KeyError):
                break
            n += 1
        if n == 0:
            raise ValueError("could not determine the number of layers")
        return n

    def _resolve_module(self, path: str) -> torch.nn.Module:
        obj: Any = self.model
        for part in path.split("."):
            if part in ("input", "output"):  # nnsight-style suffixes name the hook side, not a module
                continue
            obj = obj[int(part)] if part.isdigit() else getattr(obj, part)
        return obj

    def _preprocess_text(self, text: str) -> List[str]:
        """Split a long document into pieces of at most ``context_size`` tokens."""
        if not text:
            return []
        if self.tokenizer is None:
            return [text]
        ids = self.tokenizer(text, truncation=False, add_special_tokens=False)["input_ids"]
        if len(ids) <= self.context_size:
            return [text]
        limit = max(1, self.context_size - (1 if self.prepend_bos else 0))
        return [self.tokenizer.decode(ids[i : i + limit]) for i in range(0, len(ids), limit)]

    @torch.no_grad()
    def _run_batch(self, texts: List[str]) -> ActivationPair:
        enc = self.tokenizer(texts, **self.tokenizer_args)
        input_ids = enc["input_ids"].to(self.device)
        mask = enc.get("attention_mask")
        mask = mask.to(self.device) if mask is not None else torch.ones_like(input_ids)
        if self.exclude_special_tokens and getattr(self.tokenizer, "all_special_ids", None):
            special = torch.tensor(sorted(set(self.tokenizer.all_special_ids)), device=self.device)
            pad_id = getattr(self.tokenizer, "pad_token_id", None)
            eos_id = getattr(self.tokenizer, "eos_token_id", None)
            if pad_id is None or pad_id != eos_id:  # when pad == eos the attention mask already decides
                mask = mask * (~torch.isin(input_ids, special)).to(mask.dtype)
        return self.extract_from_ids(input_ids, mask)

    @torch.no_grad()
    def extract_from_ids(self, input_ids: torch.Tensor, attention_mask: Optional[torch.Tensor] = None) -> ActivationPair:
        captured_in: Dict[int, torch.Tensor] = {}
        captured_out: Dict[int, torch.Tensor] = {}
        handles = []
        for l in range(self.num_layers):
            m_in = self._resolve_module(self.mlp_input_module_path_template.format(l))
            m_out = self._resolve_module(self.mlp_output_module_path_template.format(l))

            def pre_hook(_m, args, kwargs=None, l=l):
                x = args[0] if args else next(iter(kwargs.values()))
                captured_in[l] = x.detach()

            def post_hook(_m, _args, output, l=l):
                captured_out[l] = (output[0] if isinstance(output, (tuple, list)) else output).detach()

            handles.append(m_in.register_forward_pre_hook(pre_hook))
            handles.append(m_out.register_forward_hook(post_hook))
        try:
            kwargs = {"attention_mask": attention_mask} if attention_mask is not None else {}
            self.model(input_ids, **kwargs)
        finally:
            for h in handles:
                h.remove()
        keep = attention_mask.reshape(-1).bool() if attention_mask is not None else None
        inputs, targets = {}, {}
        for l in range(self.num_layers):
            x = captured_in[l].reshape(-1, captured_in[l].shape[-1])
            y = captured_out[l].reshape(-1, captured_out[l].shape[-1])
            if keep is not None:
                x, y = x[keep], y[keep]
            inputs[l], targets[l] = x, y
        return inputs, targets

    @torch.no_grad()
    def capture_layer_sequences(self, texts: List[str], layer: int):
        """MLP-input activations of ``layer`` with the sequence axis kept: ``(input_ids [b, s], attention_mask [b, s],
        activations [b, s, d])`` for one batch of texts (truncated to ``context_size``, padded to the longest).
        Used by the feature-analysis tools, which map activations back to tokens (the reference traces the model per
        batch for the same purpose, scripts/analysis/collect_top_activations.py:362-376)."""
        enc = self.tokenizer(texts, **self.tokenizer_args)
        input_ids = enc["input_ids"].to(self.device)
        mask = enc.get("attention_mask")
        mask = mask.to(self.device) if mask is not None else torch.ones_like(input_ids)
        captured: Dict[str, torch.Tensor] = {}
        module = self._resolve_module(self.mlp_input_module_path_template.format(layer))

        def pre_hook(_m, args, kwargs=None):
            x = args[0] if args else next(iter(kwargs.values()))
            captured["x"] = x.detach()

        handle = module.register_forward_pre_hook(pre_hook)
        try:
            self.model(input_ids, attention_mask=mask)
        finally:
            handle.remove()
        return input_ids, mask, captured["x"]

    def stream_activations(
        self,
        dataset_path: Union[str, Iterable],
        dataset_split: str = "train",
        dataset_text_column: str = "text",
        streaming: bool = True,
        dataset_trust_remote_code: Optional[bool] = False,
        cache_path: Optional[str] = None,
    ) -> Generator[ActivationPair, None, None]:
        if isinstance(dataset_path, str):
            from datasets import load_dataset

            dataset = load_dataset(dataset_path, split=dataset_split, streaming=streaming, cache_dir=cache_path,
                                   trust_remote_code=bool(dataset_trust_remote_code))
        else:
            dataset = dataset_path
        batch: List[str] = []
        for item in dataset:
            text = item[dataset_text_column] if isinstance(item, dict) else item
            batch.extend(self._preprocess_text(text))
            while len(batch) >= self.inference_batch_size:
                cur, batch = batch[: self.inference_batch_size], batch[self.inference_batch_size :]
                yield self._run_batch(cur)
        if batch:
            yield self._run_batch(batch)
