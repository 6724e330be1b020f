"""Cross-layer transcoder with feature-major packed parameters.

Public behaviour follows the reference model (clt/models/clt.py:22-425, encoder.py,
decoder.py, theta.py): ``encode`` / ``decode`` / ``forward`` /
``get_feature_activations`` / ``get_preactivations`` / ``get_decoder_norms`` /
``estimate_theta_posthoc`` / ``convert_to_jumprelu_inplace`` and the reference
``state_dict`` key names.  The storage layout is different, chosen for the fused
sm_100a step:

* ``enc_weight  [L, F_local, d]`` and ``enc_bias [L, F_local]`` — one TMA tensor map
  covers every layer's column-parallel encoder shard.
* ``dec_weight[s]  [F_local, R_s, d]`` — *feature-major*: all ``R_s`` decoder rows of
  one source feature (``R_s = L - s`` targets when untied, 1 when tied) are
  contiguous, so a sparse decode reads one contiguous block per active feature
  and the fused Adam pass owns whole features (decoder norms need no atomics).
* ``log_threshold``, ``feature_offset``, ``feature_scale`` are sharded with the
  features (the reference replicates ``log_threshold`` and all-reduces its gradient).

``state_dict()`` converts to the reference key names and ``[d, F_local]`` decoder
layout; ``load_state_dict()`` accepts those, including the reference's legacy
remaps (clt/models/clt.py:347-425).
"""
from __future__ import annotations

import logging
import math
from collections import OrderedDict
from typing import Callable, Dict, Iterable, List, Optional, Tuple, Union

import torch
import torch.nn as nn

from ..config import CLTConfig
from ..parallel import ops as pops
from . import activations as act
from .base import BaseTranscoder, mark_replicated, shard_width

logger = logging.getLogger(__name__)

_DTYPES = {
    "float32": torch.float32, "fp32": torch.float32, "float": torch.float32,
    "float16": torch.float16, "fp16": torch.float16, "half": torch.float16,
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
    "float64": torch.float64,
}


def resolve_dtype(dtype: Optional[Union[str, torch.dtype]], default: torch.dtype = torch.float32) -> torch.dtype:
    if dtype is None:
        return default
    if isinstance(dtype, torch.dtype):
        return dtype
    key = str(dtype).replace("torch.", "")
    if key in _DTYPES:
        return _DTYPES[key]
    logger.warning("Unknown dtype %r, using %s", dtype, default)
    return default


def pair_index(src: int, tgt: int, num_layers: int) -> int:
    """Row of the (src <= tgt) pair in source-major order."""
    return src * num_layers - (src * (src - 1)) // 2 + (tgt - src)


class CrossLayerTranscoder(BaseTranscoder):
    def __init__(
        self,
        config: CLTConfig,
        process_group=None,
        device: Optional[Union[torch.device, str]] = None,
        profiler=None,
    ):
        super().__init__(config)
        self.process_group = process_group
        self.profiler = profiler
        self.world_size = pops.get_world_size(process_group) if process_group is not None else 1
        self.rank = pops.get_rank(process_group) if process_group is not None else 0
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        self.dtype = resolve_dtype(config.clt_dtype)
        self.bandwidth = 1.0

        L, F, d = config.num_layers, config.num_features, config.d_model
        self.local_features = shard_width(F, self.world_size)  # uniform padding like the reference
        self.feature_start = self.rank * self.local_features
        self.valid_features = max(0, min(F, self.feature_start + self.local_features) - self.feature_start)
        Fl = self.local_features
        tied = config.decoder_tying != "none"
        self.num_pairs = L * (L + 1) // 2
        kw = dict(device=self.device, dtype=self.dtype)

        # --- encoder: U(+-1/sqrt(F)), zero bias (reference parallel.py:82-86)
        enc_bound = 1.0 / math.sqrt(F)
        self.enc_weight = nn.Parameter(torch.empty(L, Fl, d, **kw).uniform_(-enc_bound, enc_bound))
        self.enc_bias = nn.Parameter(torch.zeros(L, Fl, **kw))

        # --- decoders: untied U(+-1/sqrt(L*d)); tied zero-initialised (decoder.py:42-108)
        dec_bound = 1.0 / math.sqrt(L * d)
        dec = []
        for s in range(L):
            rows = 1 if tied else L - s
            w = torch.zeros(Fl, rows, d, **kw)
            if not tied:
                w.uniform_(-dec_bound, dec_bound)
            dec.append(nn.Parameter(w))
        self.dec_weight = nn.ParameterList(dec)
        self.dec_bias = mark_replicated(nn.Parameter(torch.zeros(L if tied else self.num_pairs, d, **kw)))
        if self.valid_features < Fl:
            with torch.no_grad():
                self.enc_weight[:, self.valid_features:].zero_()
                for w in self.dec_weight:
                    w[self.valid_features:].zero_()

        if config.skip_connection:
            self.skip_weight = mark_replicated(nn.Parameter(torch.zeros(L if tied else self.num_pairs, d, d, **kw)))
        else:
            self.register_parameter("skip_weight", None)

        # feature affine exists for tied decoders only (decoder.py:141-172)
        if tied and config.enable_feature_offset:
            self.feature_offset = nn.Parameter(torch.zeros(L, Fl, **kw))
        else:
            self.register_parameter("feature_offset", None)
        if tied and config.enable_feature_scale:
            scale = torch.full((L, Fl), 0.1, **kw)
            scale[0] = 1.0
            self.feature_scale = nn.Parameter(scale)
        else:
            self.register_parameter("feature_scale", None)

        if config.activation_fn == "jumprelu":
            init = math.log(config.jumprelu_threshold) if config.jumprelu_threshold > 0 else math.log(1e-7)
            # thresholds are kept in fp32 whatever the weight type is: a bf16 log-threshold has three significant digits,
            # which moves a layer's L0 by whole features (the reference stores it in the model dtype, theta.py:50-61)
            self.log_threshold = nn.Parameter(torch.full((L, Fl), init, device=self.device, dtype=torch.float32))
        else:
            self.register_parameter("log_threshold", None)

        self._cached_decoder_norms: Optional[torch.Tensor] = None
        # theta-estimation accumulators (created on demand)
        self._theta_stats: Optional[Dict[str, torch.Tensor]] = None

    # ------------------------------------------------------------------ utils
    @property
    def tied(self) -> bool:
        return self.config.decoder_tying != "none"

    def _local_slice(self, full: torch.Tensor) -> torch.Tensor:
        """Bring an activation tensor to this rank's shard: accepts the full ``[..., F]``
        width (sliced), the padded ``F_local`` width or the valid width (returned as is)."""
        w = full.shape[-1]
        if self.world_size == 1:
            if w != self.config.num_features:
                raise ValueError(f"activation width {w} != num_features={self.config.num_features}")
            return full
        if w == self.config.num_features:
            return full[..., self.feature_start : self.feature_start + self.valid_features]
        if w in (self.local_features, self.valid_features):
            return full
        raise ValueError(
            f"activation width {w} matches neither num_features={self.config.num_features} "
            f"nor the local shard width {self.local_features}"
        )

    def _gather(self, local: torch.Tensor) -> torch.Tensor:
        if self.world_size == 1:
            return local
        return pops.gather_cols(local, self.config.num_features, self.process_group)

    def _prep_input(self, x: torch.Tensor) -> torch.Tensor:
        x = x.to(device=self.enc_weight.device, dtype=self.enc_weight.dtype)
        if x.dim() == 3:
            x = x.reshape(-1, x.shape[-1])
        elif x.dim() == 1:
            x = x.unsqueeze(0)
        return x

    # --------------------------------------------------------------- encoding
    def _preact_local(self, x: torch.Tensor, layer_idx: int) -> torch.Tensor:
        x = self._prep_input(x)
        if x.dim() != 2 or x.shape[-1] != self.config.d_model:
            logger.warning(
                "Rank %d: input for layer %d has shape %s, expected [..., %d]; returning zeros.",
                self.rank, layer_idx, tuple(x.shape), self.config.d_model,
            )
            rows = x.shape[0] if x.dim() >= 1 else 0
            return torch.zeros(rows, self.local_features, device=self.enc_weight.device, dtype=self.enc_weight.dtype)
        return torch.nn.functional.linear(x, self.enc_weight[layer_idx], self.enc_bias[layer_idx])

    def get_preactivations(self, x: torch.Tensor, layer_idx: int, gather: bool = True) -> torch.Tensor:
        """``x W_enc^T + b`` for one layer; ``[B, F]`` (gathered) or the local shard."""
        pre = self._preact_local(x, layer_idx)
        if not gather:
            return pre[:, : self.valid_features] if self.valid_features < self.local_features else pre
        return self._gather(pre)

    def _encode_all_layers(self, inputs: Dict[int, torch.Tensor], gather: bool = True):
        pre: Dict[int, torch.Tensor] = {}
        shapes: List[Tuple[int, int, int]] = []
        for l in sorted(inputs.keys()):
            x = inputs[l]
            if x.dim() == 3:
                b, s = x.shape[0], x.shape[1]
            else:
                b, s = (x.shape[0] if x.dim() == 2 else 1), 1
            pre[l] = self.get_preactivations(x, l, gather=gather)
            shapes.append((l, b, s))
        return pre, shapes

    def _theta(self, layer_idx: int) -> torch.Tensor:
        if self.log_threshold is None:
            raise RuntimeError("log_threshold is not initialised; the model is not in JumpReLU mode")
        return self.log_threshold[layer_idx].exp()

    def jumprelu(self, x: torch.Tensor, layer_idx: int) -> torch.Tensor:
        """JumpReLU on a full ``[B, F]`` or local ``[B, F_local]`` pre-activation tensor."""
        theta = self._theta(layer_idx)
        if x.shape[-1] != theta.shape[-1]:
            if x.shape[-1] == self.valid_features:
                theta = theta[: self.valid_features]
            else:  # full width: use the gathered threshold vector
                theta = self._gather(theta.unsqueeze(0)).squeeze(0)
        return act.JumpReLU.apply(x, theta.to(x.device), self.bandwidth)

    def _activate_layer_local(self, pre_local: torch.Tensor, layer_idx: int) -> torch.Tensor:
        """Per-layer activation on the local shard (valid columns only)."""
        fn = self.config.activation_fn
        if fn == "relu":
            return torch.relu(pre_local)
        if fn == "jumprelu":
            return self.jumprelu(pre_local, layer_idx)
        # (batch)topk restricted to one layer: rank on this layer's pre-activations.
        # The reference returns zeros here (clt/models/clt.py:135-149); this is the
        # documented per-layer behaviour of its registry functions.
        shard = {layer_idx: pre_local}
        if fn == "batchtopk":
            out = self._select(shard, batch=True, per_layer=True)
        else:
            out = self._select(shard, batch=False, per_layer=True)
        return out[layer_idx]

    def _select(self, pre_local: Dict[int, torch.Tensor], batch: bool, per_layer: bool = False) -> Dict[int, torch.Tensor]:
        cfg = self.config
        kwargs = dict(full_width=cfg.num_features, shard_offset=self.feature_start,
                      group=self.process_group if self.world_size > 1 else None)
        if batch:
            return act.apply_global_batchtopk(pre_local, cfg.batchtopk_k, **kwargs)
        # a fractional k is a fraction of the ranked row: all layers, or one layer in per-layer mode
        return act.apply_global_tokentopk(pre_local, cfg.topk_k, **kwargs)

    def encode(self, x: torch.Tensor, layer_idx: int, gather: bool = True) -> torch.Tensor:
        pre = self.get_preactivations(x, layer_idx, gather=False)
        out = self._activate_layer_local(pre, layer_idx)
        return self._gather_valid(out) if gather else out

    def _gather_valid(self, local_valid: torch.Tensor) -> torch.Tensor:
        if self.world_size == 1:
            return local_valid
        pad = self.local_features - local_valid.shape[-1]
        if pad:
            local_valid = torch.nn.functional.pad(local_valid, (0, pad))
        return self._gather(local_valid)

    def get_feature_activations(self, inputs: Dict[int, torch.Tensor], gather: bool = True) -> Dict[int, torch.Tensor]:
        """Feature activations for every layer in ``inputs``.

        ``gather=True`` returns full ``[B, F]`` tensors on every rank (the reference's
        contract); ``gather=False`` keeps this rank's ``[B, valid_features]`` shard,
        which is what the trainer, the losses and ``decode`` use internally.
        """
        cfg = self.config
        fn = cfg.activation_fn
        if fn in ("batchtopk", "topk") and cfg.topk_mode == "global":
            pre, _ = self._encode_all_layers(inputs, gather=False)
            out = self._select(pre, batch=(fn == "batchtopk"))
        else:
            out = {l: self.encode(inputs[l], l, gather=False) for l in sorted(inputs.keys())}
        if gather:
            out = {l: self._gather_valid(a) for l, a in out.items()}
        return out

    # --------------------------------------------------------------- decoding
    def _dec_rows(self, src: int, tgt: int) -> torch.Tensor:
        """``[F_local, d]`` decoder rows that map source-layer features to ``tgt``."""
        tying = self.config.decoder_tying
        if tying == "none":
            return self.dec_weight[src][:, tgt - src, :]
        if tying == "per_source":
            return self.dec_weight[src][:, 0, :]
        return self.dec_weight[tgt][:, 0, :]

    def _affine(self, a: torch.Tensor, tgt: int) -> torch.Tensor:
        """``(a + offset_t) * scale_t`` at non-zero entries (tied decoders only)."""
        if self.feature_offset is None and self.feature_scale is None:
            return a
        nz = a != 0
        out = a
        width = a.shape[-1]
        if self.feature_offset is not None:
            out = out + self.feature_offset[tgt][:width].to(a.dtype) * nz.to(a.dtype)
        if self.feature_scale is not None:
            scale = self.feature_scale[tgt][:width].to(a.dtype)
            out = torch.where(nz, out * scale, out)
        return out

    def decode(
        self,
        a: Dict[int, torch.Tensor],
        layer_idx: int,
        source_inputs: Optional[Dict[int, torch.Tensor]] = None,
    ) -> torch.Tensor:
        """Reconstruction of target layer ``layer_idx`` from activations of layers
        ``<= layer_idx`` (full ``[B, F]`` or local-shard tensors)."""
        cfg = self.config
        tying = cfg.decoder_tying
        L = cfg.num_layers
        wdev, wdt = self.dec_bias.device, self.dec_bias.dtype
        srcs = [s for s in range(layer_idx + 1) if s in a and a[s].numel() > 0]
        batch = None
        for s in srcs:
            batch = a[s].reshape(-1, a[s].shape[-1]).shape[0]
            break
        if batch is None:
            if source_inputs:
                batch = next(iter(source_inputs.values())).reshape(-1, cfg.d_model).shape[0]
            else:
                batch = 0
        partial = torch.zeros(batch, cfg.d_model, device=wdev, dtype=wdt)
        bias = torch.zeros(cfg.d_model, device=wdev, dtype=wdt)
        skip = None

        def local(s: int) -> torch.Tensor:
            t = a[s].to(device=wdev, dtype=wdt)
            t = t.reshape(-1, t.shape[-1])
            t = self._local_slice(t)
            return t

        if tying == "per_target":
            if srcs:
                summed = None
                for s in srcs:
                    contrib = self._affine(local(s), layer_idx)
                    summed = contrib if summed is None else summed + contrib
                partial = summed @ self._dec_rows(layer_idx, layer_idx)[: summed.shape[-1]]
            # one bias: the per-target decoder is applied once (decoder.py:249-251)
            bias = self.dec_bias[layer_idx]
        else:
            for s in srcs:
                t = local(s)
                if tying == "per_source":
                    t = self._affine(t, layer_idx)
                    bias = bias + self.dec_bias[s]
                else:
                    bias = bias + self.dec_bias[pair_index(s, layer_idx, L)]
                partial = partial + t @ self._dec_rows(s, layer_idx)[: t.shape[-1]]
                if (tying == "none" and self.skip_weight is not None and source_inputs is not None
                        and s in source_inputs):
                    xs = self._prep_input(source_inputs[s]).to(wdt)
                    term = xs @ self.skip_weight[pair_index(s, layer_idx, L)].T
                    skip = term if skip is None else skip + term
        if tying != "none" and self.skip_weight is not None and source_inputs is not None and layer_idx in source_inputs:
            xs = self._prep_input(source_inputs[layer_idx]).to(wdt)
            skip = xs @ self.skip_weight[layer_idx].T
        out = pops.reduce_sum(partial, self.process_group) if self.world_size > 1 else partial
        out = out + bias
        if skip is not None:
            out = out + skip
        return out

    def forward(self, inputs: Dict[int, torch.Tensor]) -> Dict[int, torch.Tensor]:
        acts = self.get_feature_activations(inputs, gather=False)
        return self.decode_all(acts, inputs)

    def decode_all(self, acts: Dict[int, torch.Tensor], inputs: Optional[Dict[int, torch.Tensor]] = None) -> Dict[int, torch.Tensor]:
        out: Dict[int, torch.Tensor] = {}
        src_inputs = inputs if self.config.skip_connection else None
        for t in range(self.config.num_layers):
            rel = {k: v for k, v in acts.items() if k <= t}
            if not rel and src_inputs is None:
                continue
            if t not in acts and not rel:
                continue
            out[t] = self.decode(rel, t, source_inputs=src_inputs)
        return out

    # ------------------------------------------------------------------ norms
    def get_decoder_norms(self, gather: bool = True) -> torch.Tensor:
        """``[L, F]`` L2 norm of every feature's decoder rows (differentiable, cached
        until :meth:`invalidate_decoder_norms`).  Feature ``(l, f)`` of an untied model owns
        the rows to targets ``t >= l``; ``per_source`` owns its single row; ``per_target``
        sums rows ``t >= l`` (reference decoder.py:342-485)."""
        if self._cached_decoder_norms is not None and gather:
            return self._cached_decoder_norms
        L = self.config.num_layers
        tying = self.config.decoder_tying
        rows = []
        if tying == "per_target":
            sq = torch.stack([w.float().pow(2).sum(dim=(1, 2)) for w in self.dec_weight])  # [L, Fl] by target
            # suffix sums over targets t >= l
            suffix = torch.flip(torch.cumsum(torch.flip(sq, dims=[0]), dim=0), dims=[0])
            local = suffix.sqrt()
        else:
            for s in range(L):
                rows.append(self.dec_weight[s].float().pow(2).sum(dim=(1, 2)))
            local = torch.stack(rows).sqrt()
        local = local.to(self.dtype)
        if not gather:
            return local[:, : self.valid_features]
        full = self._gather(local) if self.world_size > 1 else local
        self._cached_decoder_norms = full
        return full

    def invalidate_decoder_norms(self) -> None:
        self._cached_decoder_norms = None

    # --------------------------------------------------- theta / conversion
    def estimate_theta_posthoc(
        self,
        data_iter: Iterable,
        num_batches: Optional[int] = None,
        default_theta_value: float = 1e6,
        device: Optional[torch.device] = None,
    ) -> torch.Tensor:
        from .theta import estimate_theta_posthoc

        return estimate_theta_posthoc(self, data_iter, num_batches, default_theta_value, device)

    def convert_to_jumprelu_inplace(self, default_theta_value: float = 1e6) -> None:
        from .theta import convert_to_jumprelu_inplace

        convert_to_jumprelu_inplace(self, default_theta_value)

    # ------------------------------------------------------------ state dict
    def packed_state_dict(self) -> "OrderedDict[str, torch.Tensor]":
        """Parameters in the native packed layout (fast path for sharded checkpoints)."""
        return nn.Module.state_dict(self)

    def state_dict(self, *args, destination=None, prefix: str = "", keep_vars: bool = False, **kwargs):
        """Reference key names and layouts (clt/models/encoder.py:34-46, clt/models/decoder.py:58-95):
        ``encoder_module.encoders.{l}.weight|bias_param``,
        ``decoder_module.decoders.{s}->{t}.weight|bias_param`` ...)."""
        cfg = self.config
        L = cfg.num_layers
        sd = destination if destination is not None else OrderedDict()

        def put(key, tensor):
            sd[prefix + key] = tensor if keep_vars else tensor.detach()

        for l in range(L):
            put(f"encoder_module.encoders.{l}.weight", self.enc_weight[l])
            put(f"encoder_module.encoders.{l}.bias_param", self.enc_bias[l])
        if cfg.decoder_tying == "none":
            for s in range(L):
                for t in range(s, L):
                    put(f"decoder_module.decoders.{s}->{t}.weight", self.dec_weight[s][:, t - s, :].transpose(0, 1))
                    put(f"decoder_module.decoders.{s}->{t}.bias_param", self.dec_bias[pair_index(s, t, L)])
                    if self.skip_weight is not None:
                        put(f"decoder_module.skip_weights.{s}->{t}", self.skip_weight[pair_index(s, t, L)])
        else:
            for i in range(L):
                put(f"decoder_module.decoders.{i}.weight", self.dec_weight[i][:, 0, :].transpose(0, 1))
                put(f"decoder_module.decoders.{i}.bias_param", self.dec_bias[i])
                if self.skip_weight is not None:
                    put(f"decoder_module.skip_weights.{i}", self.skip_weight[i])
                if self.feature_offset is not None:
                    put(f"decoder_module.feature_offset.{i}", self.feature_offset[i])
                if self.feature_scale is not None:
                    put(f"decoder_module.feature_scale.{i}", self.feature_scale[i])
        if self.log_threshold is not None:
            put("theta_manager.log_threshold", self.log_threshold)
        return sd

    def load_state_dict(self, state_dict, strict: bool = True, assign: bool = False):
        cfg = self.config
        L = cfg.num_layers
        sd = dict(state_dict)
        if any(k in ("enc_weight", "enc_bias", "dec_bias") for k in sd):
            return nn.Module.load_state_dict(self, sd, strict=strict)
        # legacy: feature affine stored under the encoder (clt.py:389-400)
        for k in list(sd.keys()):
            if k.startswith("encoder_module.feature_offset.") or k.startswith("encoder_module.feature_scale."):
                sd[k.replace("encoder_module.", "decoder_module.", 1)] = sd.pop(k)
        # untied checkpoint into a per-source model: keep the diagonal (clt.py:359-385)
        if cfg.decoder_tying == "per_source" and any("->" in k for k in sd if k.startswith("decoder_module.decoders.")):
            for i in range(L):
                for suffix in ("weight", "bias_param"):
                    key = f"decoder_module.decoders.{i}->{i}.{suffix}"
                    if key in sd:
                        sd[f"decoder_module.decoders.{i}.{suffix}"] = sd[key]
            for k in [k for k in sd if k.startswith("decoder_module.decoders.") and "->" in k]:
                sd.pop(k)
        missing: List[str] = []
        used = set()

        def take(key):
            if key in sd:
                used.add(key)
                return sd[key]
            missing.append(key)
            return None

        def copy_into(dst: torch.Tensor, src: Optional[torch.Tensor], name: str):
            if src is None:
                return
            if tuple(dst.shape) != tuple(src.shape):
                raise RuntimeError(f"size mismatch for {name}: checkpoint {tuple(src.shape)} vs model {tuple(dst.shape)}")
            dst.copy_(src.to(device=dst.device, dtype=dst.dtype))

        with torch.no_grad():
            for l in range(L):
                copy_into(self.enc_weight[l], take(f"encoder_module.encoders.{l}.weight"), f"encoders.{l}.weight")
                copy_into(self.enc_bias[l], take(f"encoder_module.encoders.{l}.bias_param"), f"encoders.{l}.bias_param")
            if cfg.decoder_tying == "none":
                for s in range(L):
                    for t in range(s, L):
                        w = take(f"decoder_module.decoders.{s}->{t}.weight")
                        copy_into(self.dec_weight[s][:, t - s, :], None if w is None else w.transpose(0, 1), f"decoders.{s}->{t}.weight")
                        copy_into(self.dec_bias[pair_index(s, t, L)], take(f"decoder_module.decoders.{s}->{t}.bias_param"), f"decoders.{s}->{t}.bias_param")
                        if self.skip_weight is not None:
                            copy_into(self.skip_weight[pair_index(s, t, L)], take(f"decoder_module.skip_weights.{s}->{t}"), f"skip_weights.{s}->{t}")
            else:
                for i in range(L):
                    w = take(f"decoder_module.decoders.{i}.weight")
                    copy_into(self.dec_weight[i][:, 0, :], None if w is None else w.transpose(0, 1), f"decoders.{i}.weight")
                    copy_into(self.dec_bias[i], take(f"decoder_module.decoders.{i}.bias_param"), f"decoders.{i}.bias_param")
                    if self.skip_weight is not None:
                        copy_into(self.skip_weight[i], take(f"decoder_module.skip_weights.{i}"), f"skip_weights.{i}")
                    if self.feature_offset is not None:
                        copy_into(self.feature_offset[i], take(f"decoder_module.feature_offset.{i}"), f"feature_offset.{i}")
                    if self.feature_scale is not None:
                        copy_into(self.feature_scale[i], take(f"decoder_module.feature_scale.{i}"), f"feature_scale.{i}")
            lt = sd.get("theta_manager.log_threshold")
            if lt is not None:
                used.add("theta_manager.log_threshold")
                if self.log_threshold is None:
                    self.log_threshold = nn.Parameter(torch.empty(L, self.local_features, device=self.enc_weight.device, dtype=torch.float32))
                copy_into(self.log_threshold, lt, "log_threshold")
            elif self.log_threshold is not None:
                missing.append("theta_manager.log_threshold")
        unexpected = [k for k in sd if k not in used]
        self.invalidate_decoder_norms()
        if strict and (missing or unexpected):
            raise RuntimeError(f"Error(s) in loading state_dict: missing keys {missing}, unexpected keys {unexpected}")
        return torch.nn.modules.module._IncompatibleKeys(missing, unexpected)
