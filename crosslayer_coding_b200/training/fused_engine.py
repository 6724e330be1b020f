"""Fused sm_100a training / inference step for (Batch)TopK transcoders.

One step is a fixed sequence of hand-written kernels and never materialises a dense
``[B, L*F]`` activation tensor or a gradient tensor:

====  =====================================  ============================================
 #    kernel (csrc/)                         replaces in the reference
====  =====================================  ============================================
 1    encoder_gemm  (tcgen05 + TMA)          L x F.linear + all_gather, run 2-4x per step
 2    colstats                               per-layer mean/std temporaries
 3    batchtopk_select                       torch.topk over B*L*F + mask + multiply
 4    build_csr                              (dense mask is the reference's data structure)
 5    sparse_decode (+ loss epilogue)        P dense decoder GEMMs + P all-reduces + MSELoss
 6    sparsity_penalty                       dense tanh over [B, F] per layer
 7    decoder_rows_adam                      autograd decoder GEMMs + AdamW over 1.5 B params
 8    encoder_rows_adam                      autograd encoder GEMMs + AdamW
 9    dense_adam / dead_counter_update       small tensors, dead-feature bookkeeping
====  =====================================  ============================================

(reference call stack: clt/training/trainer.py:661-810, clt/training/losses.py:331-407).

Tensor parallel (features sharded over the ranks): kernels 1-4 and 6-9 run on the shard;
the selection threshold is agreed through in-kernel histogram exchanges over peer memory
(``parallel/symm.py``), and the partial reconstructions are summed across ranks before the
loss epilogue.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from ..config import CLTConfig, TrainingConfig
from ..ops import ext
from ..parallel import ops as pops

STATUS_NAMES = {0: "ok", 1: "wait timeout", 2: "list capacity exceeded", 3: "threshold outside histogram range", 4: "tie overflow"}


class EngineStatusError(RuntimeError):
    """A kernel of the fused step reported a problem through the status word (a bounded wait that ran out, a
    list that did not fit).  The step that reported it skipped its parameter update."""


def histogram_range(k_total: int, numel: int, pool_factor: float = 1.75):
    """First guess ``(key_lo, shift)`` of the selection histogram.  The z-scores are standardised per
    feature, so the range starts at the normal quantile below which all but ``pool_factor * k_total``
    elements fall; the 8192 bins cover the keys from there upwards.  The kernels keep the range in device
    memory and move it every step so that it follows the measured cut; when a step's range misses the cut
    (or holds more elements than the pool takes) the kernels repeat that step's pass over the full key
    range themselves."""
    import struct

    p = pool_factor * k_total / max(1, numel)
    if p >= 0.25 or k_total <= 0:
        return 0, 19
    z_lo = max(0.0, math.sqrt(2.0) * float(torch.erfinv(torch.tensor(1.0 - 2.0 * p, dtype=torch.float64))))
    key_lo = struct.unpack("<I", struct.pack("<f", z_lo))[0] | 0x80000000
    shift = 0
    while ((0xFFFFFFFF - key_lo) >> shift) >= 8192:
        shift += 1
    return key_lo, shift


def engine_supports(clt_config: CLTConfig, training_config: Optional[TrainingConfig], model=None) -> Optional[str]:
    """``None`` when the fused step covers this configuration, else the reason it does not."""
    if clt_config.activation_fn not in ("batchtopk", "jumprelu", "topk"):
        return f"activation_fn={clt_config.activation_fn!r} (fused step covers batchtopk, topk and jumprelu)"
    if clt_config.activation_fn in ("batchtopk", "topk") and clt_config.topk_mode != "global":
        return "topk_mode='per_layer'"
    if clt_config.activation_fn == "topk" and model is not None and model.world_size > 1:
        return "per-token topk under tensor parallelism"
    if clt_config.activation_fn == "jumprelu":
        # the threshold gradient runs as one GEMM per source layer over the packed untied decoder tensors
        if clt_config.decoder_tying != "none":
            return "jumprelu with tied decoders"
    if clt_config.enable_feature_offset or clt_config.enable_feature_scale:
        return "feature offset/scale"
    if clt_config.d_model % 8 != 0 or clt_config.d_model > 2048:
        return "d_model must be a multiple of 8 and <= 2048"
    if clt_config.num_layers > 32:
        return "more than 32 layers"
    if model is not None:
        if model.dtype != torch.bfloat16:
            return f"model dtype {model.dtype} (fused step needs bf16 weights)"
        if model.local_features % 8 != 0:
            return "local feature count must be a multiple of 8"
    if training_config is not None:
        if training_config.gradient_clip_val is not None:
            return "gradient clipping"
        if training_config.aux_loss_factor:
            # AuxK is evaluated by the autograd path whenever dead features exist; the
            # fused step handles the (common) steps without dead features.
            pass
        if training_config.precision == "fp16":
            return "fp16 loss scaling"
    return None


@dataclass
class StepOutput:
    """Device scalars of one step; nothing here forces a host sync."""

    reconstruction: torch.Tensor
    sparsity: torch.Tensor
    preactivation: torch.Tensor
    auxiliary: torch.Tensor
    total: torch.Tensor
    num_entries: torch.Tensor

    def as_dict(self) -> Dict[str, torch.Tensor]:
        return {
            "total": self.total, "reconstruction": self.reconstruction, "sparsity": self.sparsity,
            "preactivation": self.preactivation, "auxiliary": self.auxiliary,
        }


class FusedBatchTopKEngine:
    def __init__(
        self,
        model,
        training_config: Optional[TrainingConfig],
        batch_tokens: int,
        sigma_tg: Optional[torch.Tensor] = None,
        symm=None,
    ):
        reason = engine_supports(model.config, training_config, model)
        if reason is not None:
            raise ValueError(f"fused engine does not cover this configuration: {reason}")
        if not torch.cuda.is_available():
            raise RuntimeError("the fused engine needs a CUDA device")
        self.ext = ext.load()
        self.model = model
        self.tc = training_config
        cfg = model.config
        self.cfg = cfg
        self.L, self.d, self.F = cfg.num_layers, cfg.d_model, cfg.num_features
        self.B = int(batch_tokens)
        self.Fl = model.local_features
        self.Fv = model.valid_features
        self.world = model.world_size
        self.rank = model.rank
        self.group = model.process_group if self.world > 1 else None
        self.symm = symm
        self.dev = model.enc_weight.device
        self.tying = {"none": 0, "per_source": 1, "per_target": 2}[cfg.decoder_tying]
        dev = self.dev
        L, B, d, Fl = self.L, self.B, self.d, self.Fl
        i32, f32 = torch.int32, torch.float32

        self.fn = cfg.activation_fn
        if self.fn == "batchtopk":
            self.k_total = min(int(cfg.batchtopk_k) * B, B * L * self.F)
        elif self.fn == "topk":
            from ..models.activations import resolve_token_k

            self.k_token = resolve_token_k(float(cfg.topk_k), L * self.F)
            if self.k_token < 1:
                raise ValueError("topk_k selects no feature")
            self.k_total = self.k_token * B
        else:
            # JumpReLU: the number of active entries is data dependent; the lists hold up to
            # ``fused_max_active_per_token`` entries per token and a step that needs more reports it
            per_tok = int(getattr(training_config, "fused_max_active_per_token", 1024) or 1024) if training_config is not None else 1024
            self.k_total = int(min(B * L * max(self.Fv, 1), per_tok * B))
        self.key_lo, self.shift = histogram_range(self.k_total, B * L * self.F) if self.fn == "batchtopk" else (0, 19)
        self.preact = torch.empty(L, B, Fl, dtype=torch.bfloat16, device=dev)
        self.mean = torch.empty(L, Fl, dtype=f32, device=dev)
        self.rstd = torch.empty(L, Fl, dtype=f32, device=dev)
        self.tile_stats = None  # [L, ceil(B / 128), Fl, 2] fp32 switches the statistics into the GEMM epilogue
        self.hist = torch.zeros(2 * 8192 + 32, dtype=i32, device=dev)  # two histograms + the pool counter
        # tracked histogram range {key_lo, shift} and the pool filled by the single pass over the pre-activations
        self.sel_state = torch.tensor([self.key_lo, self.shift], dtype=torch.int64, device=dev) if self.key_lo != 0 else None
        k_local = -(-self.k_total // max(1, self.world))
        self.pool = torch.empty(4, int(min(B * L * max(Fl, 1), 3 * k_local + (1 << 16))), dtype=i32, device=dev) if self.key_lo != 0 else None
        self.ctl = torch.zeros(16, dtype=torch.int64, device=dev)
        self.status = torch.zeros(4, dtype=i32, device=dev)
        cap = max(self.k_total, 8)
        self.cap = cap
        numel_local = B * L * max(self.Fv, 1)
        cand_cap = int(min(numel_local, max(1 << 20, 4 * self.k_total, 1 << 23)))
        self.ent_tok = torch.empty(cap, dtype=i32, device=dev)
        self.ent_col = torch.empty(cap, dtype=i32, device=dev)
        self.ent_val = torch.empty(cap, dtype=f32, device=dev)
        self.cand_key = torch.empty(cand_cap, dtype=i32, device=dev)
        self.cand_tok = torch.empty(cand_cap, dtype=i32, device=dev)
        self.cand_col = torch.empty(cand_cap, dtype=i32, device=dev)
        self.cand_val = torch.empty(cand_cap, dtype=f32, device=dev)
        ncols = L * Fl
        self.ncols = ncols
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
        self.fired = torch.zeros(ncols, dtype=torch.uint8, device=dev)
        self.dead_counter = torch.zeros(ncols, dtype=torch.int64, device=dev)
        self.gs = symm.gs if (symm is not None and self.world > 1) else torch.empty(L, B, d, dtype=torch.bfloat16, device=dev)
        self.sq_err = torch.zeros(L, dtype=torch.float64, device=dev)
        self.penalty = torch.zeros(1, dtype=torch.float64, device=dev)
        self.gs_sum = torch.zeros(L, d, dtype=f32, device=dev)
        self.grad_a = torch.zeros(cap, dtype=f32, device=dev)
        self.pen_coef = torch.zeros(ncols, dtype=f32, device=dev)
        self.norm2 = torch.zeros(ncols, dtype=f32, device=dev)      # per decoder tensor rows
        self.norm2_next = torch.zeros(ncols, dtype=f32, device=dev)
        self.norms_valid = False
        self.sigma = None
        if sigma_tg is not None:
            self.sigma = sigma_tg.to(device=dev, dtype=f32).reshape(L, d).contiguous()
        # target t receives the bias of every pair (s <= t) when untied / per_source, one bias when per_target
        if self.tying == 0:
            sel = torch.zeros(L, model.num_pairs, dtype=f32, device=dev)
            from ..models.clt import pair_index

            for t in range(L):
                for s in range(t + 1):
                    sel[t, pair_index(s, t, L)] = 1.0
        elif self.tying == 1:
            sel = torch.tril(torch.ones(L, L, dtype=f32, device=dev))
        else:
            sel = torch.eye(L, dtype=f32, device=dev)
        self.bias_sel = sel  # [L targets, n_bias]

        # optimizer state: fp32 moments; optimizer_states_dtype="bfloat16" keeps the moments of the two big weight
        # families in bf16 with stochastic rounding (12 instead of 20 bytes per parameter and step through HBM)
        self.opt_state: Dict[str, torch.Tensor] = {}
        if training_config is not None:
            z = lambda p: torch.zeros_like(p, dtype=f32)  # noqa: E731
            self.moments_bf16 = str(getattr(training_config, "optimizer_states_dtype", "")).lower() in ("bfloat16", "bf16")
            if self.moments_bf16 and self.tying != 0:
                raise ValueError("optimizer_states_dtype='bfloat16' needs untied decoders (row pipeline)")
            zb = (lambda p: torch.zeros_like(p, dtype=torch.bfloat16)) if self.moments_bf16 else z  # noqa: E731
            self.enc_m, self.enc_v = zb(model.enc_weight), zb(model.enc_weight)
            self.encb_m, self.encb_v = z(model.enc_bias), z(model.enc_bias)
            self.dec_m = [zb(w) for w in model.dec_weight]
            self.dec_v = [zb(w) for w in model.dec_weight]
            self.decb_m, self.decb_v = z(model.dec_bias), z(model.dec_bias)
            if model.skip_weight is not None:
                self.skip_m, self.skip_v = z(model.skip_weight), z(model.skip_weight)
        if self.fn == "jumprelu":
            self.S1 = torch.zeros(L, Fl, dtype=f32, device=dev)
            self.S2 = torch.zeros(L, Fl, dtype=f32, device=dev)
            if training_config is not None:
                self.theta_m = torch.zeros(L, Fl, dtype=f32, device=dev)
                self.theta_v = torch.zeros(L, Fl, dtype=f32, device=dev)
        self.opt_step = 0
        self.seq = 0
        self.kernel_launches = 0  # launches of this package's own kernels (reported by the benchmark)

    # ------------------------------------------------------------------ pieces
    def _exchange_args(self):
        if self.world <= 1 or self.symm is None:
            return 1, 0, [], [], 0, 0
        self.seq += 1
        return (self.world, self.rank, self.symm.hist_data_ptrs, self.symm.hist_flag_ptrs, self.symm.slot_elems, self.seq)

    def encode_select(self, X: torch.Tensor) -> None:
        """Kernels 1-4: pre-activations, batch statistics, global BatchTopK, CSR views."""
        e = self.ext
        m = self.model
        assert X.dtype == torch.bfloat16 and X.shape == (self.L, self.B, self.d), (X.dtype, X.shape)
        self._X_last = X
        # The GEMM can leave per-block column sums behind (tile_stats) so that the batch statistics need no second
        # pass; at K = d_model that epilogue work outlasts the MMAs of a tile (measured: +0.75 ms on the GEMM against
        # 0.37 ms for the separate pass at the GPT-2 shape), so the separate column-statistics pass is used.
        e.encoder_gemm(X, m.enc_weight.data, m.enc_bias.data, self.preact, self.status, self.tile_stats)
        if self.fn == "jumprelu":
            self.theta = m.log_threshold.data.float().exp().contiguous()
            e.threshold_select(self.preact, self.theta, self.Fv, self.Fl, self.ctl, self.ent_tok, self.ent_col, self.ent_val, self.status)
            self.tok_cnt.zero_()
            self.feat_cnt.zero_()
            e.build_csr(
                self.ent_tok, self.ent_col, self.ent_val, self.ctl, self.B, self.ncols,
                self.tok_cnt, self.feat_cnt, self.tok_off, self.feat_off, self.tok_cursor, self.feat_cursor,
                self.tcsr_col, self.tcsr_val, self.fcsr_tok, self.fcsr_val, self.fired, 2, self.Fl,
            )
            self.kernel_launches += 2 + 5  # gemm, threshold selection, csr (5)
            return
        if self.tile_stats is not None:
            e.colstats_from_tiles(self.tile_stats, self.mean, self.rstd, self.B)
        else:
            e.colstats(self.preact, self.mean, self.rstd)
        if self.fn == "topk":
            e.token_topk_select(self.preact, self.mean, self.rstd, self.Fl, self.k_token, self.ctl, self.ent_tok, self.ent_col,
                                self.ent_val, self.status)
            self.tok_cnt.zero_()
            self.feat_cnt.zero_()
            e.build_csr(
                self.ent_tok, self.ent_col, self.ent_val, self.ctl, self.B, self.ncols,
                self.tok_cnt, self.feat_cnt, self.tok_off, self.feat_off, self.tok_cursor, self.feat_cursor,
                self.tcsr_col, self.tcsr_val, self.fcsr_tok, self.fcsr_val, self.fired, 2, self.Fl,
            )
            self.kernel_launches += 3 + 5  # gemm, colstats, per-token selection, csr (5)
            return
        self.hist.zero_()
        world, rank, dptr, fptr, slot, seq = self._exchange_args()
        if self.world > 1 and self.symm is None:
            raise RuntimeError("tensor-parallel fused engine needs a symmetric exchange area (parallel.symm)")
        e.batchtopk_select(
            self.preact, self.mean, self.rstd, self.Fv, self.Fl, m.feature_start, self.F, self.k_total,
            self.key_lo, self.shift, self.hist, self.ctl, self.ent_tok, self.ent_col, self.ent_val,
            self.cand_key, self.cand_tok, self.cand_col, self.cand_val, self.status,
            world, rank, dptr, fptr, slot, seq, self.sel_state, self.pool,
        )
        self.tok_cnt.zero_()
        self.feat_cnt.zero_()
        e.build_csr(
            self.ent_tok, self.ent_col, self.ent_val, self.ctl, self.B, self.ncols,
            self.tok_cnt, self.feat_cnt, self.tok_off, self.feat_off, self.tok_cursor, self.feat_cursor,
            self.tcsr_col, self.tcsr_val, self.fcsr_tok, self.fcsr_val, self.fired, 2, self.Fl,
        )
        # gemm, colstats, select (collect, find_bin, classify, fallback x3, refine, finalize | zhist, find_bin, compact,
        # refine, finalize), csr (5)
        self.kernel_launches += 2 + (8 if self.key_lo != 0 else 5) + 5

    def _bias_sum(self) -> torch.Tensor:
        return (self.bias_sel @ self.model.dec_bias.data.float()).contiguous()

    # The skip connection (reference: clt/models/decoder.py:310,332) is a handful of small dense [B, d] x [d, d]
    # products: library GEMMs.  Its output enters the fused loss epilogue as the `addend` of the decode kernel and
    # its weights are updated by the dense Adam kernel from gs^T @ x.
    def _skip_pairs(self, s: int):
        from ..models.clt import pair_index

        return [pair_index(s, t, self.L) for t in range(s, self.L)]

    def _skip_term(self, X: torch.Tensor) -> Optional[torch.Tensor]:
        W = self.model.skip_weight
        if W is None:
            return None
        out = torch.zeros(self.L, self.B, self.d, dtype=torch.float32, device=self.dev)
        if self.tying == 0:
            for s in range(self.L):
                w = W.data[self._skip_pairs(s)]                     # [R, d, d], row t - s is the pair (s, t)
                out[s:] += torch.matmul(X[s].to(w.dtype), w.transpose(1, 2)).float()
        else:
            out += torch.matmul(X.to(W.dtype), W.data.transpose(1, 2)).float()
        return out

    def _skip_adam(self, X: torch.Tensor, lr: float, c_g: float) -> None:
        W = self.model.skip_weight
        if W is None:
            return
        grad = torch.zeros(W.shape, dtype=torch.float32, device=self.dev)
        gs = self.gs
        if self.tying == 0:
            for s in range(self.L):
                # d loss / d W[s -> t] = c_g * gs[t]^T @ x[s]
                grad[self._skip_pairs(s)] = torch.matmul(gs[s:].transpose(1, 2), X[s].to(gs.dtype)).float()
        else:
            grad = torch.matmul(gs.transpose(1, 2), X.to(gs.dtype)).float()
        self.ext.dense_adam(W.data, self.skip_m, self.skip_v, grad.contiguous(), self._hyper(lr, c_g))

    def decode_loss(self, Y: torch.Tensor, want_yhat: bool = False) -> Optional[torch.Tensor]:
        """Kernel 5: sparse decode, reconstruction loss sums and the gradient seed."""
        e, m = self.ext, self.model
        self.sq_err.zero_()
        yhat = torch.empty(self.L, self.B, self.d, dtype=torch.float32, device=self.dev) if want_yhat else None
        dec_w = [w.data for w in m.dec_weight]
        bias_sum = self._bias_sum()
        addend = self._skip_term(self._X_last) if m.skip_weight is not None else None
        if self.world == 1:
            e.sparse_decode(dec_w, self.L, self.B, self.d, self.Fl, self.tying, self.tok_off, self.tcsr_col, self.tcsr_val,
                            None, None, None, bias_sum, addend, Y, self.sigma, self.gs, yhat, self.sq_err, 1, [], 0, 0, self.status)
            self.kernel_launches += 1
        else:
            sy = self.symm
            if yhat is not None:
                yhat.zero_()
            # 1. decode, pushing every token's partial sums into its owner's staging slot (peer stores)
            e.sparse_decode(dec_w, self.L, self.B, self.d, self.Fl, self.tying, self.tok_off, self.tcsr_col, self.tcsr_val,
                            None, None, None, None, None, None, None, None, None, None, 2, sy.stage_ptrs, sy.rows_per_rank, self.rank, self.status)
            sy.barrier(e, self.status)
            # 2. owners reduce their rows, finish the loss and push the gradient seed to every rank
            e.owner_reduce_loss(sy.stage, sy.gs_ptrs, self.rank, bias_sum, addend, Y, self.sigma, yhat, self.sq_err, sy.rows_per_rank)
            sy.barrier(e, self.status)
            pops.all_reduce(self.sq_err, group=self.group)
            if yhat is not None:
                pops.all_reduce(yhat, group=self.group)
            self.kernel_launches += 4
        return yhat

    def _hyper(self, lr: float, grad_scale: float) -> List[float]:
        tc = self.tc
        b1 = tc.optimizer_beta1 if tc.optimizer_beta1 is not None else 0.9
        b2 = tc.optimizer_beta2 if tc.optimizer_beta2 is not None else 0.999
        decoupled = 1.0 if tc.optimizer == "adamw" else 0.0
        wd = 0.01 if tc.optimizer == "adamw" else 0.0
        t = self.opt_step
        seed = 0.0
        if tc.enable_stochastic_rounding:
            seed = float(((tc.seed * 2654435761 + t * 40503) % 0xFFFFFFFE) + 1)
        mseed = float(((tc.seed * 40503 + t * 2654435761) % 0xFFFFFFFE) + 1)
        return [lr, b1, b2, 1e-8, wd, 1.0 - b1 ** t, 1.0 - b2 ** t, decoupled, grad_scale, seed, mseed]

    def ensure_norms(self) -> None:
        if self.norms_valid:
            return
        for i, w in enumerate(self.model.dec_weight):
            self.ext.decoder_norm2(w.data, self.norm2[i * self.Fl:(i + 1) * self.Fl])
        self.norms_valid = True

    def feature_norm2(self) -> torch.Tensor:
        """Squared decoder norm per (layer, feature) column of this shard."""
        self.ensure_norms()
        if self.tying == 2:
            per_t = self.norm2.view(self.L, self.Fl)
            return torch.flip(torch.cumsum(torch.flip(per_t, dims=[0]), dim=0), dims=[0]).reshape(-1).contiguous()
        return self.norm2

    # -------------------------------------------------------------------- step
    # ------------------------------------------------------- extra loss terms
    def _extra_buffers(self):
        if getattr(self, "_enc_dense", None) is None:
            f32 = torch.float32
            self._enc_dense = torch.zeros(self.L, self.Fl, self.d, dtype=f32, device=self.dev)
            self._encb_dense = torch.zeros(self.L, self.Fl, dtype=f32, device=self.dev)
            self._dec_row0_dense = torch.zeros(len(self.model.dec_weight), self.Fl, self.d, dtype=f32, device=self.dev)
        return self._enc_dense, self._encb_dense, self._dec_row0_dense

    @torch.no_grad()
    def _preactivation_term(self, X: torch.Tensor, coef: float) -> torch.Tensor:
        """``coef * mean(relu(-preact))`` (reference losses.py:203-261) and its dense encoder gradient
        ``-(coef/numel) * 1[preact < 0]^T X`` - a library GEMM per layer on the stored pre-activations."""
        enc_dense, encb_dense, _ = self._extra_buffers()
        numel = float(self.L * self.B * self.F)
        total = torch.zeros((), device=self.dev)
        for l in range(self.L):
            pl = self.preact[l][:, : self.Fv]
            neg = pl < 0
            total = total + torch.where(neg, -pl.float(), torch.zeros((), device=self.dev)).sum()
            g = neg.to(torch.bfloat16)
            enc_dense[l, : self.Fv].add_((g.t() @ X[l]).float(), alpha=-coef / numel)
            encb_dense[l, : self.Fv].add_(g.float().sum(dim=0), alpha=-coef / numel)
        return coef * total / numel

    @torch.no_grad()
    def _auxiliary_term(self, X: torch.Tensor, dead_mask: torch.Tensor, factor: float, k_aux_default: int = 512) -> torch.Tensor:
        """AuxK on dead features (reference losses.py:263-329) in closed form on the few dead rows: per layer the
        top ``k_aux`` dead pre-activations of every token decode to the same layer and are matched to the
        de-normalised residual.  Gradients go to the dense side buffers (encoder rows, same-layer decoder rows,
        that pair's bias) and, because the residual depends on the main reconstruction, into the gradient seed."""
        from ..models import activations as act
        from ..models.clt import pair_index

        enc_dense, encb_dense, dec0_dense = self._extra_buffers()
        m = self.model
        L, B, d = self.L, self.B, self.d
        n_dead = dead_mask.sum(dim=1).float()
        if self.world > 1:
            pops.all_reduce(n_dead, group=self.group)
        n_dead_host = n_dead.tolist()
        total = torch.zeros((), device=self.dev)
        self._aux_bias_grad = torch.zeros_like(self.model.dec_bias.data, dtype=torch.float32)
        for l in range(L):
            nd = int(n_dead_host[l])
            if nd == 0:
                continue
            k_aux = max(1, min(k_aux_default, nd))
            idx = dead_mask[l].nonzero().flatten()
            xl = X[l].float()
            pre = xl @ m.enc_weight.data[l][idx].float().t() + m.enc_bias.data[l][idx].float()  # [B, n_local]
            gidx = (m.feature_start + idx).unsqueeze(0).expand(B, -1)
            mask = act.sharded_row_topk_mask(pre, gidx, k_aux, self.group) if pre.shape[1] > 0 or self.world > 1 else torch.zeros_like(pre, dtype=torch.bool)
            aux = pre * mask
            w_d = m.dec_weight[l].data[idx, 0, :].float()  # the decoder row that maps layer l to itself
            bias_row = pair_index(l, l, L) if self.tying == 0 else l
            recon = aux @ w_d
            if self.world > 1:
                pops.all_reduce(recon, group=self.group)
            recon = recon + m.dec_bias.data[bias_row].float()
            sg = self.sigma[l] if self.sigma is not None else torch.ones(d, device=self.dev)
            residual = -(self.gs[l].float() / sg)  # (y - y_hat) * sigma
            r = recon - residual
            c = factor * min(nd / k_aux, 1.0)
            total = total + c * (r * r).mean()
            g_recon = r * (2.0 * c / (B * d))                      # dL/d recon
            self.gs[l].add_((c * r * sg).to(self.gs.dtype))        # through the residual into the main path
            g_aux = (g_recon @ w_d.t()) * mask                     # STE: gradient at the kept positions
            dec0_dense[l].index_add_(0, idx, aux.t() @ g_recon)
            self._aux_bias_grad[bias_row] += g_recon.sum(dim=0)
            enc_dense[l].index_add_(0, idx, g_aux.t() @ xl)
            encb_dense[l].index_add_(0, idx, g_aux.sum(dim=0))
        return total

    # -------------------------------------------------------------------- step
    def train_step(self, X: torch.Tensor, Y: torch.Tensor, step: int, lr: float, sparsity_lambda: float = 0.0,
                   preactivation_coef: float = 0.0, aux_factor: float = 0.0, dead_mask: Optional[torch.Tensor] = None) -> StepOutput:
        """One optimisation step on inputs/targets ``[L, B, d]`` (bf16, already normalised).

        ``preactivation_coef`` and ``aux_factor`` (with ``dead_mask [L, valid_features]``) switch on the two loss
        terms that are not sparse: they are evaluated with a few library calls on the stored pre-activations /
        the dead rows and enter the fused optimizer kernels as dense side gradients."""
        e, m, tc = self.ext, self.model, self.tc
        L, B, d = self.L, self.B, self.d
        self.opt_step += 1
        self.encode_select(X)
        self.decode_loss(Y)
        c_g = 2.0 / (B * d)
        if self.fn == "jumprelu":
            # window sums for the threshold gradient, from the decoder weights of this step (before their update)
            self.S1.zero_()
            self.S2.zero_()
            e.theta_grad_gemm(self.gs, [w.data for w in m.dec_weight], self.preact, self.theta, float(m.bandwidth), self.S1, self.S2, self.status)
            self.kernel_launches += 1
        zero = torch.zeros((), device=self.dev)
        pre_loss, aux_loss = zero, zero
        enc_dense = encb_dense = dec0_dense = None
        extra_bias_grad = None
        use_pre = abs(preactivation_coef) >= 1e-9
        use_aux = aux_factor and dead_mask is not None
        if use_pre or use_aux:
            enc_dense, encb_dense, dec0_dense = self._extra_buffers()
            enc_dense.zero_()
            encb_dense.zero_()
            if use_pre:
                pre_loss = self._preactivation_term(X, float(preactivation_coef))
            if use_aux:
                dec0_dense.zero_()
                mask = dead_mask
                if mask.shape[-1] != self.Fl:
                    mask = torch.nn.functional.pad(mask, (0, self.Fl - mask.shape[-1]))
                aux_loss = self._auxiliary_term(X, mask, float(aux_factor))
                extra_bias_grad = self._aux_bias_grad
            else:
                dec0_dense = None
        # decoder biases: dL/db[pair (s,t)] = c_g * sum_b gs[t, b, :]
        self.gs_sum.zero_()
        e.gs_colsum(self.gs, self.gs_sum)
        bias_grad = (self.bias_sel.t() @ self.gs_sum).contiguous()
        if extra_bias_grad is not None:
            bias_grad = bias_grad + extra_bias_grad / c_g  # dense_adam multiplies by c_g
        self.grad_a.zero_()
        self.penalty.zero_()
        pen = None
        use_pen = sparsity_lambda > 1e-9 and (self.fn != "batchtopk" or (tc.apply_sparsity_penalty_to_batchtopk if tc is not None else True))
        if use_pen:
            if self.fn == "jumprelu":
                self.norm_at_step = self.feature_norm2().clamp_min(0).sqrt()  # the update below replaces the norms
            e.sparsity_penalty(self.feat_off, self.fcsr_val, self.feature_norm2(), float(sparsity_lambda), float(tc.sparsity_c),
                               self.grad_a, self.pen_coef, self.penalty)
            pen = self.pen_coef
        self.norm2_next.zero_()
        e.decoder_rows_adam([w.data for w in m.dec_weight], self.dec_m, self.dec_v, L, B, d, self.Fl, self.tying,
                            self.feat_off, self.fcsr_tok, self.fcsr_val, self.gs, self.grad_a, pen, self.norm2_next,
                            None, None, dec0_dense, self._hyper(lr, c_g), self.status)
        self.norm2, self.norm2_next = self.norm2_next, self.norm2
        self.norms_valid = True
        e.dense_adam(m.dec_bias.data, self.decb_m, self.decb_v, bias_grad, self._hyper(lr, c_g))
        self._skip_adam(X, lr, c_g)
        e.encoder_rows_adam(m.enc_weight.data, self.enc_m, self.enc_v, m.enc_bias.data, self.encb_m, self.encb_v,
                            self.feat_off, self.fcsr_tok, self.grad_a, X, enc_dense, encb_dense, self._hyper(lr, 1.0), self.status)
        if self.fn == "jumprelu":
            self._update_thresholds(lr, c_g, float(sparsity_lambda) if use_pen else 0.0)
        e.dead_counter_update(self.dead_counter, self.fired)
        self.kernel_launches += 5 + (1 if use_pen else 0)  # gs_colsum, decoder/encoder Adam, dense Adam, dead counters
        m.invalidate_decoder_norms()
        recon = (self.sq_err.sum() / (B * d)).float()
        sparsity = self.penalty[0].float()
        if self.world > 1 and (use_pen or use_pre):
            both = torch.stack([sparsity, pre_loss.float()])
            pops.all_reduce(both, group=self.group)
            sparsity, pre_loss = both[0], both[1]
        return StepOutput(recon, sparsity, pre_loss, aux_loss, recon + sparsity + pre_loss + aux_loss, self.ctl[3])

    @torch.no_grad()
    def _update_thresholds(self, lr: float, c_g: float, lam: float) -> None:
        """AdamW step on ``log_threshold`` from the window sums of ``theta_grad_gemm``.

        ``d loss / d theta[f] = -(1 / bw) * sum_b window * x * G`` with ``G = c_g * (gs . W rows)`` for the
        reconstruction and ``lam * c * n_f * sech^2(c * n_f * a)`` for the sparsity penalty; the latter is a
        per-feature constant except at the active entries, which the entry list corrects
        (reference: clt/models/activations.py:196-220 with clt/training/losses.py:179-185)."""
        m, tc = self.model, self.tc
        bw = float(m.bandwidth)
        g = c_g * self.S1
        if lam > 0.0:
            c = float(tc.sparsity_c)
            norm = self.norm_at_step.view(self.L, self.Fl)
            cap = self.ent_val.numel()
            n = torch.clamp(self.ctl[3], max=cap)
            live = torch.arange(cap, device=self.dev) < n
            # unused slots add zero; they are spread over the columns so that they do not pile up on one address
            col = torch.where(live, self.ent_col, (torch.arange(cap, device=self.dev, dtype=torch.int32) % self.ncols)).long()
            x = torch.where(live, self.ent_val, torch.zeros_like(self.ent_val))
            nf = norm.reshape(-1)[col]
            inside = (x - self.theta.reshape(-1)[col]).abs() <= bw / 2
            t2 = torch.tanh(c * nf * x) ** 2
            corr = torch.zeros(self.ncols, dtype=torch.float32, device=self.dev)
            corr.index_add_(0, col, torch.where(inside & live, x * t2, torch.zeros_like(x)))
            g = g + lam * c * norm * (self.S2 - corr.view(self.L, self.Fl))
        grad_theta = -g / bw
        grad_log = (grad_theta * self.theta).contiguous()  # theta = exp(log_threshold)
        self.grad_log_threshold = grad_log  # kept for diagnostics and tests
        self.ext.dense_adam(m.log_threshold.data, self.theta_m, self.theta_v, grad_log, self._hyper(lr, 1.0))
        self.kernel_launches += 1

    # --------------------------------------------------------------- inference
    @torch.no_grad()
    def forward(self, X: torch.Tensor, Y: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Reconstructions ``[L, B, d]`` (fp32) for inputs ``X``; ``Y`` defaults to zeros."""
        self.encode_select(X)
        if Y is None:
            Y = torch.zeros_like(X)
        return self.decode_loss(Y, want_yhat=True)

    def activations_dense(self) -> torch.Tensor:
        """Dense ``[L, B, F_local]`` view of the last selection (testing / evaluation)."""
        n = int(self.ctl[3].item())
        out = torch.zeros(self.L, self.B, self.Fl, dtype=torch.float32, device=self.dev)
        col = self.ent_col[:n].long()
        l, f = col // self.Fl, col % self.Fl
        out[l, self.ent_tok[:n].long(), f] = self.ent_val[:n]
        return out

    def check_status(self) -> None:
        """Host read of the kernels' status word; raises when a kernel reported a problem."""
        code = int(self.status[0].item())
        if code != 0:
            self.status.zero_()
            raise EngineStatusError(f"rank {self.rank}: fused step reported '{STATUS_NAMES.get(code, code)}'")

    # ------------------------------------------------------- optimizer state io
    def optimizer_state_dict(self) -> Dict[str, torch.Tensor]:
        sd = {"step": torch.tensor(self.opt_step), "enc_m": self.enc_m, "enc_v": self.enc_v, "encb_m": self.encb_m,
              "encb_v": self.encb_v, "decb_m": self.decb_m, "decb_v": self.decb_v, "dead_counter": self.dead_counter}
        for i, (mm, vv) in enumerate(zip(self.dec_m, self.dec_v)):
            sd[f"dec_m.{i}"] = mm
            sd[f"dec_v.{i}"] = vv
        if self.fn == "jumprelu":
            sd["theta_m"], sd["theta_v"] = self.theta_m, self.theta_v
        if self.model.skip_weight is not None:
            sd["skip_m"], sd["skip_v"] = self.skip_m, self.skip_v
        return sd

    def load_optimizer_state_dict(self, sd: Dict[str, torch.Tensor]) -> None:
        self.opt_step = int(sd["step"])
        for name in ("enc_m", "enc_v", "encb_m", "encb_v", "decb_m", "decb_v", "dead_counter"):
            getattr(self, name).copy_(sd[name])
        for i in range(len(self.dec_m)):
            self.dec_m[i].copy_(sd[f"dec_m.{i}"])
            self.dec_v[i].copy_(sd[f"dec_v.{i}"])
        if self.model.skip_weight is not None and "skip_m" in sd:
            self.skip_m.copy_(sd["skip_m"])
            self.skip_v.copy_(sd["skip_v"])
        if self.fn == "jumprelu" and "theta_m" in sd:
            self.theta_m.copy_(sd["theta_m"])
            self.theta_v.copy_(sd["theta_v"])
        self.norms_valid = False
