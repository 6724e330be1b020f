"""Sparse forward pass on sm_100a for inference and evaluation, for every sparse activation function.

The reference computes ``model(inputs)`` densely: per layer an encoder GEMM, the activation on the dense
``[B, F]`` tensor and one dense decoder GEMM per (source, target) pair over activations that are >99.9 % zeros
(clt/models/clt.py:285-300, clt/models/decoder.py:289-295).  Here the activation is a *selection* that emits a
``(token, feature, value)`` list and the decoder is a gather over the listed rows:

    encoder_gemm (tcgen05)  ->  selection  ->  CSR by token  ->  sparse decode (+ per-layer squared error)

Selections:
  * ``batchtopk``  global top ``k*B`` of the per-feature batch z-scores (same kernels as the training step),
  * ``topk``       every token's top ``k`` of the same z-scores (exact per-token radix selection),
  * ``jumprelu``   ``x >= exp(log_threshold[l, f])``   (the form a converted BatchTopK model is deployed in),
  * ``relu``       ``x > 0`` (only useful while the activations are sparse; dense layers overflow the list and
                   the call reports it, see ``check_status``).
Skip connections and tensor-parallel groups are not covered here; ``supports`` says so and
callers use ``CrossLayerTranscoder.forward`` for those.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..ops import ext as ext_mod

_MIN_POSITIVE_BF16 = 9.183549615799121e-41  # 2**-133, the smallest positive bf16 (subnormal)


def supports(model) -> Optional[str]:
    """``None`` when ``SparseForward`` covers the model's configuration, else the reason it does not."""
    cfg = model.config
    if cfg.activation_fn not in ("batchtopk", "topk", "jumprelu", "relu"):
        return f"activation_fn={cfg.activation_fn!r}"
    if cfg.activation_fn in ("batchtopk", "topk") and cfg.topk_mode != "global":
        return "topk_mode='per_layer'"
    if cfg.skip_connection:
        return "skip_connection"
    if model.world_size > 1:
        return "tensor-parallel model"
    if model.dtype != torch.bfloat16:
        return f"model dtype {model.dtype} (needs bf16 weights)"
    if cfg.d_model % 8 != 0 or cfg.d_model > 2048 or cfg.num_layers > 32 or model.local_features % 8 != 0:
        return "shape limits (d_model % 8, d_model <= 2048, layers <= 32, features % 8)"
    if not model.enc_weight.is_cuda:
        return "model is not on a CUDA device"
    return None


class SparseForward:
    def __init__(self, model, batch_tokens: int, max_active_per_token: int = 2048):
        reason = supports(model)
        if reason is not None:
            raise ValueError(f"SparseForward does not cover this model: {reason}")
        self.model = model
        self.ext = ext_mod.load()
        cfg = model.config
        self.L, self.d, self.B = cfg.num_layers, cfg.d_model, int(batch_tokens)
        self.Fl = model.local_features
        self.fn = cfg.activation_fn
        self.tying = {"none": 0, "per_source": 1, "per_target": 2}[cfg.decoder_tying]
        dev = self.dev = model.enc_weight.device
        L, B, d, Fl = self.L, self.B, self.d, self.Fl
        i32, f32 = torch.int32, torch.float32
        if self.fn == "batchtopk":
            self.k_total = min(int(cfg.batchtopk_k) * B, B * L * Fl)
            cap = max(self.k_total, 8)
        elif self.fn == "topk":
            from .activations import resolve_token_k

            self.k_token = resolve_token_k(float(cfg.topk_k), L * Fl)
            self.k_total = self.k_token * B
            cap = max(self.k_total, 8)
        else:
            cap = int(min(B * L * Fl, max_active_per_token * B))
        self.cap = cap
        self.preact = torch.empty(L, B, Fl, dtype=torch.bfloat16, device=dev)
        self.ctl = torch.zeros(16, dtype=torch.int64, device=dev)
        self.status = torch.zeros(4, dtype=i32, device=dev)
        self.ent_tok = torch.empty(cap, dtype=i32, device=dev)
        self.ent_col = torch.empty(cap, dtype=i32, device=dev)
        self.ent_val = torch.empty(cap, dtype=f32, device=dev)
        if self.fn in ("batchtopk", "topk"):
            self.mean = torch.empty(L, Fl, dtype=f32, device=dev)
            self.rstd = torch.empty(L, Fl, dtype=f32, device=dev)
        if self.fn == "batchtopk":
            from ..training.fused_engine import histogram_range

            self.hist = torch.zeros(2 * 8192 + 32, dtype=i32, device=dev)
            self.key_lo, self.shift = histogram_range(self.k_total, B * L * Fl)
            cand_cap = int(min(B * L * Fl, max(1 << 20, 4 * self.k_total)))
            self.cand = [torch.empty(cand_cap, dtype=i32, device=dev) for _ in range(3)] + [torch.empty(cand_cap, dtype=f32, device=dev)]
            self.sel_state = torch.tensor([self.key_lo, self.shift], dtype=torch.int64, device=dev) if self.key_lo != 0 else None
            self.pool = torch.empty(4, int(min(B * L * Fl, 3 * self.k_total + (1 << 16))), dtype=i32, device=dev) if self.key_lo != 0 else None
        ncols = self.ncols = L * Fl
        self.tok_cnt = torch.zeros(B, dtype=i32, device=dev)
        self.feat_cnt = torch.zeros(ncols, dtype=i32, device=dev)
        self.tok_off = torch.zeros(B + 1, dtype=i32, device=dev)
        self.feat_off = torch.zeros(ncols + 1, dtype=i32, device=dev)
        self.tok_cursor = torch.zeros(B, dtype=i32, device=dev)
        self.feat_cursor = torch.zeros(ncols, dtype=i32, device=dev)
        self.tcsr_col = torch.zeros(cap, dtype=i32, device=dev)
        self.tcsr_val = torch.zeros(cap, dtype=f32, device=dev)
        self.fcsr_tok = torch.zeros(cap, dtype=i32, device=dev)
        self.fcsr_val = torch.zeros(cap, dtype=f32, device=dev)
        self.gs = torch.empty(L, B, d, dtype=torch.bfloat16, device=dev)
        self.sq_err = torch.zeros(L, dtype=torch.float64, device=dev)
        if self.tying == 0:
            from .clt import pair_index

            sel = torch.zeros(L, model.num_pairs, dtype=f32, device=dev)
            for t in range(L):
                for s in range(t + 1):
                    sel[t, pair_index(s, t, L)] = 1.0
        elif self.tying == 1:
            sel = torch.tril(torch.ones(L, L, dtype=f32, device=dev))
        else:
            sel = torch.eye(L, dtype=f32, device=dev)
        self.bias_sel = sel

    # ------------------------------------------------------------------ selection
    def _theta(self) -> torch.Tensor:
        if self.fn == "jumprelu":
            return self.model.log_threshold.data.float().exp().contiguous()
        return torch.full((self.L, self.Fl), _MIN_POSITIVE_BF16, dtype=torch.float32, device=self.dev)

    @torch.no_grad()
    def encode(self, X: torch.Tensor) -> None:
        """Pre-activations, selection and the token-major / feature-major CSR views of the active entries."""
        e, m = self.ext, self.model
        assert X.dtype == torch.bfloat16 and X.shape == (self.L, self.B, self.d), (X.dtype, tuple(X.shape))
        e.encoder_gemm(X, m.enc_weight.data, m.enc_bias.data, self.preact, self.status, None)
        if self.fn == "batchtopk":
            e.colstats(self.preact, self.mean, self.rstd)
            self.hist.zero_()
            e.batchtopk_select(self.preact, self.mean, self.rstd, self.Fl, self.Fl, 0, self.Fl, self.k_total, self.key_lo, self.shift,
                               self.hist, self.ctl, self.ent_tok, self.ent_col, self.ent_val, self.cand[0], self.cand[1], self.cand[2],
                               self.cand[3], self.status, 1, 0, [], [], 0, 0, self.sel_state, self.pool)
        elif self.fn == "topk":
            e.colstats(self.preact, self.mean, self.rstd)
            e.token_topk_select(self.preact, self.mean, self.rstd, self.Fl, self.k_token, self.ctl, self.ent_tok, self.ent_col,
                                self.ent_val, self.status)
        else:
            e.threshold_select(self.preact, self._theta(), self.Fl, self.Fl, self.ctl, self.ent_tok, self.ent_col, self.ent_val, self.status)
        self.tok_cnt.zero_()
        self.feat_cnt.zero_()
        e.build_csr(self.ent_tok, self.ent_col, self.ent_val, self.ctl, self.B, self.ncols, self.tok_cnt, self.feat_cnt, self.tok_off,
                    self.feat_off, self.tok_cursor, self.feat_cursor, self.tcsr_col, self.tcsr_val, self.fcsr_tok, self.fcsr_val,
                    None, 2, self.Fl)

    # ------------------------------------------------------------------ decode
    @torch.no_grad()
    def reconstruct(self, X: torch.Tensor, Y: Optional[torch.Tensor] = None, sigma: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Reconstructions ``[L, B, d]`` (fp32).  With targets ``Y`` the per-layer sums of squared errors
        (scaled by ``sigma [L, d]`` when given) are left in ``self.sq_err``."""
        self.encode(X)
        e, m = self.ext, self.model
        self.sq_err.zero_()
        yhat = torch.empty(self.L, self.B, self.d, dtype=torch.float32, device=self.dev)
        bias_sum = (self.bias_sel @ m.dec_bias.data.float()).contiguous()
        off = scale = None
        if m.feature_offset is not None:
            off = m.feature_offset.data.float().contiguous()
        if m.feature_scale is not None:
            scale = m.feature_scale.data.float().contiguous()
        tgt = Y if Y is not None else torch.zeros_like(X)
        sg = sigma.to(device=self.dev, dtype=torch.float32).reshape(self.L, self.d).contiguous() if sigma is not None else None
        e.sparse_decode([w.data for w in m.dec_weight], self.L, self.B, self.d, self.Fl, self.tying, self.tok_off, self.tcsr_col,
                        self.tcsr_val, off, scale, None, bias_sum, None, tgt, sg, self.gs, yhat, self.sq_err, 1, [], 0, 0, self.status)
        return yhat

    def forward_dict(self, inputs: Dict[int, torch.Tensor]) -> Dict[int, torch.Tensor]:
        """Same contract as ``CrossLayerTranscoder.forward``: ``{layer: [B, d]}`` in, reconstructions out."""
        X = torch.stack([inputs[l].reshape(-1, self.d) for l in range(self.L)]).to(torch.bfloat16)
        yhat = self.reconstruct(X)
        return {l: yhat[l] for l in range(self.L)}

    # ------------------------------------------------------------------ views of the last selection
    def num_entries(self) -> int:
        return int(self.ctl[3].item())

    def l0_per_layer(self) -> torch.Tensor:
        """Mean number of active features per token and layer of the last ``encode``."""
        per_col = (self.feat_off[1:] - self.feat_off[:-1]).view(self.L, self.Fl).sum(dim=1)
        return per_col.float() / self.B

    def activations_dense(self) -> torch.Tensor:
        """Dense ``[L, B, F]`` activations of the last ``encode`` (testing)."""
        n = min(self.num_entries(), self.cap)
        out = torch.zeros(self.L, self.B, self.Fl, dtype=torch.float32, device=self.dev)
        col = self.ent_col[:n].long()
        out[col // self.Fl, self.ent_tok[:n].long(), col % self.Fl] = self.ent_val[:n]
        return out

    def check_status(self) -> None:
        code = int(self.status[0].item())
        if code != 0:
            self.status.zero_()
            names = {1: "wait timeout", 2: "entry list too small (activations too dense for the sparse path)",
                     3: "selection range", 4: "tie overflow"}
            raise RuntimeError(f"sparse forward reported '{names.get(code, code)}'")
