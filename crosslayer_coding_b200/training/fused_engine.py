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

STATUS_NAMES = {0: "ok", 1: "wait timeout", 2: "list capacity exceeded", 3: "threshold outside histogram range", 4: "tie overflow",
                5: "index out of range (debug build)"}


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
    if clt_config.activation_fn not in ("batchtopk", "jumprelu", "topk", "relu"):
        return f"activation_fn={clt_config.activation_fn!r} (fused step covers batchtopk, topk, jumprelu and relu)"
    if clt_config.activation_fn in ("batchtopk", "topk") and clt_config.topk_mode != "global":
        return "topk_mode='per_layer'"
    if clt_config.activation_fn == "topk" and model is not None and model.world_size > 1:
        from ..models.activations import resolve_token_k

        k_tok = resolve_token_k(float(clt_config.topk_k), clt_config.num_layers * clt_config.num_features)
        if 2 * k_tok > clt_config.num_layers * clt_config.d_model or model.world_size * k_tok * 8 > 200 * 1024:
            return "per-token topk under tensor parallelism with k beyond the key staging area"
        if k_tok > clt_config.num_layers * model.valid_features:
            return "per-token topk with k above the columns of one shard"
    if clt_config.activation_fn == "jumprelu" and (clt_config.enable_feature_offset or clt_config.enable_feature_scale) \
            and clt_config.decoder_tying != "none":
        return "jumprelu with feature offset/scale (the threshold-gradient GEMM has no per-target affine)"
    if (clt_config.enable_feature_offset or clt_config.enable_feature_scale) and clt_config.decoder_tying != "none" \
            and training_config is not None and training_config.aux_loss_factor:
        return "feature offset/scale together with the auxiliary loss (its decode has no affine)"
    if clt_config.d_model % 8 != 0 or clt_config.d_model > 2048:
        return "d_model must be a multiple of 8 and <= 2048"
    if clt_config.num_layers > 32:
        return "more than 32 layers"
    if model is not None:
        if model.dtype not in (torch.bfloat16, torch.float16):
            return f"model dtype {model.dtype} (fused step needs bf16 or fp16 weights)"
        if model.local_features % 8 != 0:
            return "local feature count must be a multiple of 8"
    if training_config is not None:
        if training_config.precision == "fp16" and model is not None and model.dtype != torch.float16:
            return "precision='fp16' needs fp16 weights (clt_dtype='float16' or fp16_convert_weights)"
    return None


@dataclass
class StepOutput:
    """Device scalars of one step; nothing here forces a host sync.  All of them are views of ``vector``
    (fp32 ``[8]``: total, reconstruction, sparsity, pre-activation, auxiliary, gradient norm, skipped steps so far,
    loss scale), which the step-control kernel fills."""

    vector: torch.Tensor
    num_entries: torch.Tensor

    @property
    def total(self): return self.vector[0]

    @property
    def reconstruction(self): return self.vector[1]

    @property
    def sparsity(self): return self.vector[2]

    @property
    def preactivation(self): return self.vector[3]

    @property
    def auxiliary(self): return self.vector[4]

    @property
    def grad_norm(self): return self.vector[5]

    @property
    def skipped_steps(self): return self.vector[6]

    @property
    def loss_scale(self): return self.vector[7]

    def as_dict(self) -> Dict[str, torch.Tensor]:
        return {
            "total": self.total, "reconstruction": self.reconstruction, "sparsity": self.sparsity,
            "preactivation": self.preactivation, "auxiliary": self.auxiliary, "_vector": self.vector,
        }


# rounds of the symmetric exchange area used outside the selection (which owns rounds 0 .. 13)
ROUND_LOSS, ROUND_NORM = 14, 15
# words of the step control block (csrc/common.cuh: StepCtl)
SC_SKIP, SC_INV_SCALE, SC_LOSS_SCALE, SC_GROWTH, SC_FOUND_INF, SC_GRAD_NORM_SQ, SC_CLIP, SC_SKIPPED = range(8)


class _Arena:
    """One allocation for everything a step needs zeroed, so that a step starts with a single memset.  The two
    decoder-norm buffers sit at the two ends: the one that receives this step's norms is zeroed together with the
    middle part (the range to clear is contiguous either way), the other one keeps the norms of the previous step."""

    def __init__(self, device, norm_bytes: int):
        self.device = device
        self.specs = []
        self.norm_bytes = (norm_bytes + 255) // 256 * 256
        self.size = self.norm_bytes

    def add(self, name: str, numel: int, dtype: torch.dtype):
        nbytes = (numel * torch.empty((), dtype=dtype).element_size() + 255) // 256 * 256
        self.specs.append((name, self.size, numel, dtype))
        self.size += nbytes

    def build(self):
        total = self.size + self.norm_bytes
        self.buf = torch.zeros(total, dtype=torch.uint8, device=self.device)
        views = {}
        for name, off, numel, dtype in self.specs:
            es = torch.empty((), dtype=dtype).element_size()
            views[name] = self.buf[off: off + numel * es].view(dtype)
        self.mid_lo, self.mid_hi = self.norm_bytes, self.size
        return views

    def norm_view(self, which: int, numel: int) -> torch.Tensor:
        off = 0 if which == 0 else self.size
        return self.buf[off: off + numel * 4].view(torch.float32)

    def clear_for_step(self, next_norm: int) -> None:
        if next_norm == 0:
            self.buf[: self.mid_hi].zero_()
        else:
            self.buf[self.mid_lo:].zero_()


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
        self.t16 = model.dtype  # bf16 or fp16: storage type of weights, inputs, pre-activations and the gradient seed
        self.tying = {"none": 0, "per_source": 1, "per_target": 2}[cfg.decoder_tying]
        dev = self.dev
        L, B, d, Fl = self.L, self.B, self.d, self.Fl
        i32, f32, f64 = torch.int32, torch.float32, torch.float64

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
            # JumpReLU / ReLU: the number of active entries is data dependent; the lists hold up to
            # ``fused_max_active_per_token`` entries per token and a step that needs more reports it
            per_tok = int(getattr(training_config, "fused_max_active_per_token", 1024) or 1024) if training_config is not None else 1024
            self.k_total = int(min(B * L * max(self.Fv, 1), per_tok * B))
        self.key_lo, self.shift = histogram_range(self.k_total, B * L * self.F) if self.fn == "batchtopk" else (0, 19)
        self.preact = torch.empty(L, B, Fl, dtype=self.t16, device=dev)
        self.mean = torch.empty(L, Fl, dtype=f32, device=dev)
        self.rstd = torch.empty(L, Fl, dtype=f32, device=dev)
        self.tile_stats = None  # [L, ceil(B / 128), Fl, 2] fp32 switches the statistics into the GEMM epilogue
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
        # --- everything that has to be zero when a step starts lives in one arena (one memset per step)
        ar = _Arena(dev, ncols * 4)
        ar.add("hist", 2 * 8192 + 32, i32)          # two histograms + the pool counter
        ar.add("tok_cnt", B, i32)
        ar.add("feat_cnt", ncols, i32)
        ar.add("sq_err", L, f64)
        ar.add("scalars", 4, f64)                    # penalty, pre-activation loss, auxiliary loss (+ spare)
        ar.add("gs_sum", L * d, f32)
        ar.add("grad_a", cap, f32)
        if self.fn == "jumprelu":
            ar.add("S1", L * Fl, f32)
            ar.add("S2", L * Fl, f32)
        views = ar.build()
        self.arena = ar
        self.hist, self.tok_cnt, self.feat_cnt = views["hist"], views["tok_cnt"], views["feat_cnt"]
        self.sq_err, self.scalars = views["sq_err"], views["scalars"]
        self.penalty = self.scalars[0:1]
        self.gs_sum = views["gs_sum"].view(L, d)
        self.grad_a = views["grad_a"]
        if self.fn == "jumprelu":
            self.S1, self.S2 = views["S1"].view(L, Fl), views["S2"].view(L, Fl)
        self._norm_cur = 0                            # which end of the arena holds the current decoder norms
        self.norm2 = ar.norm_view(0, ncols)           # per decoder tensor rows
        self.norm2_next = ar.norm_view(1, ncols)
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
        self.gs = symm.gs if (symm is not None and self.world > 1) else torch.empty(L, B, d, dtype=self.t16, device=dev)
        if self.gs.dtype != self.t16:
            self.gs = self.gs.view(self.t16)  # same width: the symmetric buffer is typed by its user
        self.pen_coef = torch.zeros(ncols, dtype=f32, device=dev)
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
        self.bias_sel = sel.contiguous()  # [L targets, n_bias]
        self.bias_sum = torch.zeros(L, d, dtype=f32, device=dev)
        self._bias_sum_valid = False

        # step control block: skip flag, 1 / loss scale, loss scale, growth counter, found-inf, norm^2, clip, skipped
        self.fp16 = self.t16 == torch.float16
        init_scale = float(getattr(training_config, "loss_scale_init", 65536.0)) if (training_config is not None and self.fp16) else 1.0
        self.step_ctl = torch.zeros(16, dtype=f32, device=dev)
        self.step_ctl[SC_INV_SCALE] = 1.0 / init_scale
        self.step_ctl[SC_LOSS_SCALE] = init_scale
        self.step_ctl[SC_CLIP] = 1.0
        self.growth_interval = int(getattr(training_config, "loss_scale_growth_interval", 2000)) if training_config is not None else 2000
        self.clip_val = float(training_config.gradient_clip_val) if (training_config is not None and training_config.gradient_clip_val) else 0.0

        # optimizer state: fp32 moments; optimizer_states_dtype="bfloat16" keeps the moments of the two big weight
        # families in bf16 with stochastic rounding (12 instead of 20 bytes per parameter and step through HBM)
        self.opt_state: Dict[str, torch.Tensor] = {}
        if training_config is not None:
            z = lambda p: torch.zeros_like(p, dtype=f32)  # noqa: E731
            self.moments_bf16 = str(getattr(training_config, "optimizer_states_dtype", "")).lower() in ("bfloat16", "bf16")
            if self.moments_bf16 and (self.tying != 0 or self.fp16):
                raise ValueError("optimizer_states_dtype='bfloat16' needs untied bf16 decoders (row pipeline)")
            zb = (lambda p: torch.zeros_like(p, dtype=torch.bfloat16)) if self.moments_bf16 else z  # noqa: E731
            self.enc_m, self.enc_v = zb(model.enc_weight), zb(model.enc_weight)
            self.encb_m, self.encb_v = z(model.enc_bias), z(model.enc_bias)
            self.dec_m = [zb(w) for w in model.dec_weight]
            self.dec_v = [zb(w) for w in model.dec_weight]
            self.decb_m, self.decb_v = z(model.dec_bias), z(model.dec_bias)
            if model.skip_weight is not None:
                self.skip_m, self.skip_v = z(model.skip_weight), z(model.skip_weight)
        if self.fn in ("jumprelu", "relu"):
            self.theta = torch.zeros(L, Fl, dtype=f32, device=dev)
            self._theta_valid = False
            if self.fn == "relu":
                # ReLU as a threshold selection: x >= smallest positive value of the storage type
                self.theta.fill_(float(torch.finfo(self.t16).tiny))
                self._theta_valid = True
            if training_config is not None and self.fn == "jumprelu":
                self.theta_m = torch.zeros(L, Fl, dtype=f32, device=dev)
                self.theta_v = torch.zeros(L, Fl, dtype=f32, device=dev)
                self.grad_log_threshold = torch.zeros(L, Fl, dtype=f32, device=dev)  # kept for diagnostics and tests
        # per-source tied decoders: the row of feature (s, f) serves every target t >= s, so its gradient and dL/da only need
        # the gradient seed summed over those targets; with that sum in place of the seed the decoder update is the
        # one-row-per-feature case of the untied row pipeline
        # feature affine of tied decoders (reference clt/models/decoder.py:228-285): a' = (a + offset_t[f]) * scale_t[f] at the
        # active entries, per target layer t.  The kernels read fp32 copies; the gradients of the two terms come out of the
        # tied decoder sweep (per entry and target: scale * (gs_t . w) and (a + offset) * (gs_t . w)), one small Adam kernel each.
        self.affine = self.tying != 0 and (model.feature_offset is not None or model.feature_scale is not None)
        self.foff32 = self.fsc32 = self.d_foff = self.d_fsc = None
        if self.affine:
            if model.feature_offset is not None:
                self.foff32 = model.feature_offset.data.float().contiguous()
                self.d_foff = torch.zeros(L, Fl, dtype=f32, device=dev)
            if model.feature_scale is not None:
                self.fsc32 = model.feature_scale.data.float().contiguous()
                self.d_fsc = torch.zeros(L, Fl, dtype=f32, device=dev)
            if training_config is not None:
                z32 = lambda p: torch.zeros_like(p, dtype=f32)  # noqa: E731
                if model.feature_offset is not None:
                    self.foff_m, self.foff_v = z32(model.feature_offset), z32(model.feature_offset)
                if model.feature_scale is not None:
                    self.fsc_m, self.fsc_v = z32(model.feature_scale), z32(model.feature_scale)
        self.gs_cum = torch.empty(L, B, d, dtype=self.t16, device=dev) if (self.tying == 1 and training_config is not None and not self.affine) else None
        import os as _os

        self._check_guards = _os.environ.get(ext.DEBUG_ENV, "") not in ("", "0")  # debug runs read the guard bytes at every status check
        self.opt_step = 0
        self.seq = 0
        # recorded right before the optimizer sweep of every step: the staging copies of later batches are released at this
        # point (their host-to-device writes slow the read-streaming kernels at the start of a step far more than the sweep)
        self.sweep_begin: Optional[torch.cuda.Event] = None
        self.kernel_launches = 0  # launches of this package's own kernels (reported by the benchmark)
        self.last_output: Optional[StepOutput] = None

    # ------------------------------------------------------------------ pieces
    def _exchange_args(self):
        if self.world <= 1 or self.symm is None:
            return 1, 0, [], [], 0, 0
        self.seq += 1
        return (self.world, self.rank, self.symm.hist_data_ptrs, self.symm.hist_flag_ptrs, self.symm.slot_elems, self.seq)

    def _begin_step(self) -> None:
        """One memset for everything that has to start at zero (histograms, counters, loss sums, dL/da, next norms)."""
        self.arena.clear_for_step(1 - self._norm_cur)
        self._XT_of = None  # the transposed inputs belong to one step

    def _ensure_theta(self) -> None:
        if self.fn == "jumprelu" and not self._theta_valid:
            self.ext.theta_exp(self.model.log_threshold.data, self.theta)
            self._theta_valid = True

    def _build_csr(self) -> None:
        self.ext.build_csr(
            self.ent_tok, self.ent_col, self.ent_val, self.ctl, self.B, self.ncols,
            self.tok_cnt, self.feat_cnt, self.tok_off, self.feat_off, self.tok_cursor, self.feat_cursor,
            self.tcsr_col, self.tcsr_val, self.fcsr_tok, self.fcsr_val, self.fired, 2, self.Fl,
        )

    def encode_select(self, X: torch.Tensor, fresh: bool = True) -> None:
        """Kernels 1-4: pre-activations, batch statistics, selection, CSR views.  ``fresh``: clear the per-step
        arena first (the training step does it itself)."""
        e = self.ext
        m = self.model
        assert X.dtype == self.t16 and X.shape == (self.L, self.B, self.d), (X.dtype, X.shape)
        if fresh:
            self._begin_step()
        self._X_last = X
        # The GEMM can leave per-block column sums behind (tile_stats) so that the batch statistics need no second
        # pass; at K = d_model that epilogue work outlasts the MMAs of a tile (measured: +0.75 ms on the GEMM against
        # 0.37 ms for the separate pass at the GPT-2 shape), so the separate column-statistics pass is used.
        e.encoder_gemm(X, m.enc_weight.data, m.enc_bias.data, self.preact, self.status, self.tile_stats)
        if self.fn in ("jumprelu", "relu"):
            self._ensure_theta()
            e.threshold_select(self.preact, self.theta, self.Fv, self.Fl, self.ctl, self.ent_tok, self.ent_col, self.ent_val, self.status)
            self._build_csr()
            self.kernel_launches += 2 + 5  # gemm, threshold selection, csr (5)
            return
        if self.tile_stats is not None:
            e.colstats_from_tiles(self.tile_stats, self.mean, self.rstd, self.B)
        else:
            e.colstats(self.preact, self.mean, self.rstd)
        if self.fn == "topk" and self.world == 1:
            e.token_topk_select(self.preact, self.mean, self.rstd, self.Fl, self.k_token, self.ctl, self.ent_tok, self.ent_col,
                                self.ent_val, self.status, self.Fv)
            self._build_csr()
            self.kernel_launches += 3 + 5  # gemm, colstats, per-token selection, csr (5)
            return
        if self.fn == "topk":
            self._token_topk_sharded()
            self._build_csr()
            self.kernel_launches += 3 + 5 + 5
            return
        world, rank, dptr, fptr, slot, seq = self._exchange_args()
        if self.world > 1 and self.symm is None:
            raise RuntimeError("tensor-parallel fused engine needs a symmetric exchange area (parallel.symm)")
        e.batchtopk_select(
            self.preact, self.mean, self.rstd, self.Fv, self.Fl, m.feature_start, self.F, self.k_total,
            self.key_lo, self.shift, self.hist, self.ctl, self.ent_tok, self.ent_col, self.ent_val,
            self.cand_key, self.cand_tok, self.cand_col, self.cand_val, self.status,
            world, rank, dptr, fptr, slot, seq, self.sel_state, self.pool,
        )
        self._build_csr()
        # gemm, colstats, select (collect, find_bin, classify, fallback x3, refine, finalize | zhist, find_bin, compact,
        # refine, finalize), csr (5)
        self.kernel_launches += 2 + (8 if self.key_lo != 0 else 5) + 5

    def _token_topk_sharded(self) -> None:
        """TokenTopK across feature shards (reference: clt/models/activations.py:360-491, which gathers the full
        pre-activations and broadcasts the mask).  Every rank takes the exact top k of its own columns, the owners of
        the tokens rank the W * k composite keys that arrive by peer stores and publish the cut, every rank keeps what
        is at or above it.  The keys order by (z-score, lower flat index first), so the result equals the single-GPU
        selection entry for entry.  Staging reuses the decode's partial-sum area (idle during the selection); the cut
        array sits in the histogram section, which this activation does not use otherwise."""
        e, sy = self.ext, self.symm
        if sy is None:
            raise RuntimeError("tensor-parallel fused engine needs a symmetric exchange area (parallel.symm)")
        B, k = self.B, self.k_token
        if getattr(self, "_tk_col", None) is None:
            from ..parallel import symm as symm_mod

            assert B * 8 <= 14 * self.world * symm_mod.HIST_SLOT * 4, "cut array does not fit the histogram section"
            assert 2 * k <= self.L * self.d, "key staging does not fit the partial-sum area"
            self._tk_tok = torch.empty(B * k, dtype=torch.int32, device=self.dev)
            self._tk_col = torch.empty(B * k, dtype=torch.int32, device=self.dev)
            self._tk_val = torch.empty(B * k, dtype=torch.float32, device=self.dev)
            self._tk_key = torch.empty(B * k, dtype=torch.int64, device=self.dev)
        # 1. exact local top k of every token into scratch lists
        e.token_topk_select(self.preact, self.mean, self.rstd, self.Fl, k, self.ctl, self._tk_tok, self._tk_col, self._tk_val, self.status, self.Fv)
        args = (self._tk_col, self._tk_val, self._tk_key, self.mean, self.rstd, self.Fl, self.model.feature_start, self.F, B, k, self.rank,
                sy.rows_per_rank, sy.stage_ptrs, sy.hist_data_ptrs, self.ctl, self.ent_tok, self.ent_col, self.ent_val, self.status)
        e.token_topk_tp(0, *args)   # 2. keys to the token owners
        sy.barrier(e, self.status)
        e.token_topk_tp(1, *args)   # 3. owners publish the cut of their tokens
        sy.barrier(e, self.status)
        e.token_topk_tp(2, *args)   # 4. keep what is at or above the cut

    def _ensure_bias_sum(self) -> None:
        """Per-target sums of the decoder biases; kept current by the last kernel of every training step."""
        if not self._bias_sum_valid:
            self.ext.step_finish(None, None, self.model.dec_bias.data, self.bias_sel, self.bias_sum)
            self._bias_sum_valid = True

    # ------------------------------------------------------------------ dense side terms (grouped tcgen05 GEMM)
    def _seg_tables(self, groups):
        """Device tables of ``ext.dense_gemm``: ``groups`` is a list of segment lists ``[(a_layer, b_layer), ...]``."""
        off, segs = [0], []
        for g in groups:
            segs.extend(g)
            off.append(len(segs))
        return (torch.tensor(off, dtype=torch.int32, device=self.dev),
                torch.tensor(segs, dtype=torch.int32, device=self.dev).view(-1, 2).contiguous())

    def _transposed_inputs(self, X: torch.Tensor) -> torch.Tensor:
        """``x^T [L, d, B]`` of this step's inputs (the gradient GEMMs contract over the tokens)."""
        if getattr(self, "_XT", None) is None:
            self._XT = torch.empty(self.L, self.d, self.B, dtype=self.t16, device=self.dev)
            self._XT_of = None
        if self._XT_of is not X:
            self.ext.transpose16(X, self._XT)
            self._XT_of = X
            self.kernel_launches += 1
        return self._XT

    # The skip connection (reference: clt/models/decoder.py:298-338): y_hat[t] += sum_{s <= t} x[s] W_skip[s -> t]^T (untied)
    # or x[t] W_skip[t]^T (tied).  Forward: one grouped GEMM whose K dimension runs over the source layers; its output
    # enters the loss epilogue of the decode kernel as `addend`.  Backward: dW_skip[s -> t] = gs[t]^T x[s], one grouped
    # GEMM over the transposed seed and inputs (K = tokens), fed to the dense Adam kernel.
    def _skip_setup(self) -> None:
        if getattr(self, "_skip_fwd", None) is not None:
            return
        from ..models.clt import pair_index

        L = self.L
        if self.tying == 0:
            fwd = [[(s, pair_index(s, t, L)) for s in range(t + 1)] for t in range(L)]
            bwd = [None] * self.model.num_pairs
            for s in range(L):
                for t in range(s, L):
                    bwd[pair_index(s, t, L)] = [(t, s)]
        else:
            fwd = [[(l, l)] for l in range(L)]
            bwd = [[(l, l)] for l in range(L)]
        self._skip_fwd = self._seg_tables(fwd)
        self._skip_bwd = self._seg_tables(bwd)
        self._skip_out = torch.empty(L, self.B, self.d, dtype=torch.float32, device=self.dev)
        self._skip_grad_buf = torch.empty(self.model.skip_weight.shape, dtype=torch.float32, device=self.dev)
        self._gsT = torch.empty(L, self.d, self.B, dtype=self.t16, device=self.dev)

    def _skip_term(self, X: torch.Tensor) -> Optional[torch.Tensor]:
        W = self.model.skip_weight
        if W is None:
            return None
        self._skip_setup()
        off, segs = self._skip_fwd
        self.ext.dense_gemm(X, W.data, self._skip_out, off, segs, 1.0, self.status)
        self.kernel_launches += 1
        return self._skip_out

    def _skip_grad(self, X: torch.Tensor) -> torch.Tensor:
        self._skip_setup()
        XT = self._transposed_inputs(X)
        self.ext.transpose16(self.gs, self._gsT)
        off, segs = self._skip_bwd
        self.ext.dense_gemm(self._gsT, XT, self._skip_grad_buf, off, segs, 1.0, self.status)
        self.kernel_launches += 2
        return self._skip_grad_buf

    def decode_loss(self, Y: torch.Tensor, want_yhat: bool = False) -> Optional[torch.Tensor]:
        """Kernel 5: sparse decode, reconstruction loss sums and the gradient seed."""
        e, m = self.ext, self.model
        yhat = torch.empty(self.L, self.B, self.d, dtype=torch.float32, device=self.dev) if want_yhat else None
        dec_w = [w.data for w in m.dec_weight]
        self._ensure_bias_sum()
        bias_sum = self.bias_sum
        addend = self._skip_term(self._X_last) if m.skip_weight is not None else None
        if self.world == 1:
            e.sparse_decode(dec_w, self.L, self.B, self.d, self.Fl, self.tying, self.tok_off, self.tcsr_col, self.tcsr_val,
                            self.foff32, self.fsc32, None, bias_sum, addend, Y, self.sigma, self.gs, yhat, self.sq_err, 1, [], 0, 0, self.status,
                            self.step_ctl)
            self.kernel_launches += 1
        else:
            sy = self.symm
            if yhat is not None:
                yhat.zero_()
            # 1. decode, pushing every token's partial sums into its owner's staging slot (peer stores)
            e.sparse_decode(dec_w, self.L, self.B, self.d, self.Fl, self.tying, self.tok_off, self.tcsr_col, self.tcsr_val,
                            self.foff32, self.fsc32, None, None, None, None, None, None, None, None, 2, sy.stage_ptrs, sy.rows_per_rank, self.rank, self.status)
            sy.barrier(e, self.status)
            # 2. owners reduce their rows, finish their part of the loss and push the gradient seed to every rank; the
            #    exchange inside the step-control kernel that follows is the barrier behind these pushes
            e.owner_reduce_loss(sy.stage, sy.gs_ptrs, self.rank, bias_sum, addend, Y, self.sigma, yhat, self.sq_err, sy.rows_per_rank,
                                self.step_ctl)
            if yhat is not None:
                sy.barrier(e, self.status)
                pops.all_reduce(yhat, group=self.group)
            self.kernel_launches += 3
        return yhat

    def _control(self, phase: int, losses: torch.Tensor) -> None:
        """Device-side decision of the step (sums the loss terms over the ranks, skip flag, loss scale, clip)."""
        world, rank, dptr, fptr, slot, seq = self._exchange_args()
        self.ext.step_control(self.step_ctl, self.status, self.sq_err, self.scalars, losses, 1.0 / (self.B * self.d), phase,
                              self.fp16 and self.tc is not None, self.growth_interval, self.clip_val, world, rank, dptr, fptr, slot, seq,
                              ROUND_LOSS if phase == 0 else ROUND_NORM)
        self.kernel_launches += 1

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

    # ------------------------------------------------------- extra loss terms
    def _extra_buffers(self):
        if getattr(self, "_enc_dense", None) is None:
            f32 = torch.float32
            self._enc_dense = torch.zeros(self.L, self.Fl, self.d, dtype=f32, device=self.dev)
            self._encb_dense = torch.zeros(self.L, self.Fl, dtype=f32, device=self.dev)
            self._dec_row0_dense = torch.zeros(len(self.model.dec_weight), self.Fl, self.d, dtype=f32, device=self.dev)
        return self._enc_dense, self._encb_dense, self._dec_row0_dense

    @torch.no_grad()
    def _preactivation_term(self, X: torch.Tensor, coef: float) -> None:
        """``coef * mean(relu(-preact))`` (reference losses.py:203-261) and its dense encoder gradient
        ``-(coef / numel) * 1[preact < 0]^T x`` on the stored pre-activations: one pass writes the transposed indicator,
        the bias gradient and the loss sum of this shard (``scalars[1]``), one grouped tensor-core GEMM per step (all
        layers in one launch) the ``[F, d]`` weight gradient."""
        enc_dense, encb_dense, _ = self._extra_buffers()
        if getattr(self, "_ind_T", None) is None:
            self._ind_T = torch.empty(self.L, self.Fl, self.B, dtype=self.t16, device=self.dev)
            self._layer_tables = self._seg_tables([[(l, l)] for l in range(self.L)])
        c = coef / float(self.L * self.B * self.F)
        self.ext.negative_indicator(self.preact, self._ind_T, encb_dense, self.scalars[1:2], self.Fv, c)
        XT = self._transposed_inputs(X)
        off, segs = self._layer_tables
        self.ext.dense_gemm(self._ind_T, XT, enc_dense, off, segs, -c, self.status)
        self.kernel_launches += 2

    @torch.no_grad()
    def _auxiliary_term(self, X: torch.Tensor, dead_mask: torch.Tensor, factor: float, k_aux_default: int = 512) -> torch.Tensor:
        """AuxK on dead features (reference losses.py:263-329) in closed form on the few dead rows: per layer the
        top ``k_aux`` dead pre-activations of every token decode to the same layer and are matched to the
        de-normalised residual.  Gradients go to the dense side buffers (encoder rows, same-layer decoder rows,
        that pair's bias) and, because the residual depends on the main reconstruction, into the gradient seed.
        Returns the loss value (the same on every rank)."""
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
        scale = self.step_ctl[SC_LOSS_SCALE]
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
            residual = -(self.gs[l].float() / scale / sg)  # (y - y_hat) * sigma
            r = recon - residual
            c = factor * min(nd / k_aux, 1.0)
            total = total + c * (r * r).mean()
            g_recon = r * (2.0 * c / (B * d))                      # dL/d recon
            self.gs[l].add_((c * r * sg * scale).to(self.gs.dtype))  # through the residual into the main path
            g_aux = (g_recon @ w_d.t()) * mask                     # STE: gradient at the kept positions
            dec0_dense[l].index_add_(0, idx, aux.t() @ g_recon)
            self._aux_bias_grad[bias_row] += g_recon.sum(dim=0)
            enc_dense[l].index_add_(0, idx, g_aux.t() @ xl)
            encb_dense[l].index_add_(0, idx, g_aux.sum(dim=0))
        return total

    AUX_MAX_CAP = 4096  # compact dead features per layer that the selection kernel ranks in shared memory

    def set_dead_count_hint(self, max_dead_per_layer: int, max_dead_per_layer_all_ranks: Optional[int] = None) -> None:
        """Sizes the compact dead-feature set of the auxiliary term from an occasional host read of the counters
        (the largest per-layer dead count of this shard).  The capacity carries 25 % head-room; a layer that outgrows it
        between two hints uses its first ``capacity`` dead features until the next hint.  Counts beyond ``AUX_MAX_CAP``
        take the unfused path.  Under tensor parallelism the kernel path serves runs whose layers have at most ``k_aux``
        (512) dead features over all ranks (``max_dead_per_layer_all_ranks``, the same number on every rank): then every
        dead feature is kept and no selection has to be agreed across the shards."""
        n = int(max_dead_per_layer)
        self._aux_hint = n
        cap = -(-max(256, n + n // 4 + 64) // 256) * 256
        self._aux_cap_wanted = cap if n <= self.AUX_MAX_CAP else 0
        if self._aux_cap_wanted:
            self._aux_cap_wanted = min(self._aux_cap_wanted, self.AUX_MAX_CAP)
        self._aux_global_hint = int(max_dead_per_layer_all_ranks) if max_dead_per_layer_all_ranks is not None else n

    def _aux_buffers(self, cap: int):
        b = getattr(self, "_aux_buf", None)
        if b is not None and b["cap"] == cap:
            return b
        from ..models.clt import pair_index

        L, B, d, dev, t16 = self.L, self.B, self.d, self.dev, self.t16
        i32, f32 = torch.int32, torch.float32
        b = {"cap": cap}
        b["dead_cols"] = torch.zeros(L, cap, dtype=i32, device=dev)
        b["nd"] = torch.zeros(L, dtype=i32, device=dev)
        b["nd_all"] = torch.zeros(L, dtype=i32, device=dev)
        b["extra_idx"] = torch.full((L * self.Fl,), -1, dtype=i32, device=dev)
        for name in ("A", "G"):
            b[name] = torch.empty(L, B, cap, dtype=t16, device=dev)
            b[name + "T"] = torch.empty(L, cap, B, dtype=t16, device=dev)
        b["W0"] = torch.empty(L, cap, d, dtype=t16, device=dev)
        b["W0T"] = torch.empty(L, d, cap, dtype=t16, device=dev)
        b["recon"] = torch.empty(L, B, d, dtype=f32, device=dev)
        b["g"] = torch.empty(L, B, d, dtype=t16, device=dev)
        b["gT"] = torch.empty(L, d, B, dtype=t16, device=dev)
        b["dW0"] = torch.empty(L, cap, d, dtype=f32, device=dev)
        b["dWenc"] = torch.empty(L, cap, d, dtype=f32, device=dev)
        b["dbenc"] = torch.empty(L * cap, dtype=f32, device=dev)
        b["bias_c"] = torch.empty(L, cap, dtype=f32, device=dev)
        b["gsum"] = torch.empty(L, d, dtype=f32, device=dev)
        b["loss"] = torch.zeros(1, dtype=torch.float64, device=dev)
        rows = [pair_index(l, l, L) if self.tying == 0 else l for l in range(L)]
        b["bias_row"] = torch.tensor(rows, dtype=i32, device=dev)
        b["bias_row_long"] = b["bias_row"].long()
        b["bias_grad"] = torch.zeros(self.model.dec_bias.shape, dtype=f32, device=dev)
        b["layers"] = self._seg_tables([[(l, l)] for l in range(L)])
        self._aux_buf = b
        return b

    @torch.no_grad()
    def _auxiliary_term_fused(self, X: torch.Tensor, counter: torch.Tensor, window: int, factor: float, cap: int, k_aux_default: int = 512):
        """The auxiliary term as kernels on the compact dead set (single GPU): compaction of the dead columns, per-token
        exact selection of the top ``k_aux`` dead pre-activations, and four grouped tensor-core GEMMs (all layers in
        one launch each) for the auxiliary reconstruction and its three gradients.  No host read, no per-layer loop.
        Returns the buffers whose ``extra_idx`` / ``dW0`` / ``dWenc`` / ``dbenc`` / ``bias_grad`` feed the optimizer."""
        e, m = self.ext, self.model
        b = self._aux_buffers(cap)
        off, segs = b["layers"]
        e.aux_compact(counter, int(window), self.L, self.Fv, b["dead_cols"], b["nd"], b["nd_all"], b["extra_idx"])
        live = b["nd"]  # layers with dead features (any rank) have an auxiliary term
        if self.world > 1:
            pops.all_reduce(b["nd_all"], group=self.group)  # dead features of the layer over all shards (device side, no host read)
            live = b["nd_all"]
        # A = x W_dead^T on the gathered encoder rows, then bias + per-token top k_aux in place (cheaper than gathering
        # single 16-bit values out of the [B, F] pre-activation rows)
        e.aux_gather_rows([m.enc_weight.data[l].unsqueeze(1) for l in range(self.L)], b["dead_cols"], b["nd"], b["W0"])
        e.dense_gemm(X, b["W0"], b["A"], off, segs, 1.0, self.status)
        e.aux_gather_select(None, m.enc_bias.data, b["dead_cols"], b["nd"], b["nd_all"], int(k_aux_default), b["A"], b["bias_c"])
        e.aux_gather_rows([w.data for w in m.dec_weight][: self.L], b["dead_cols"], b["nd"], b["W0"])
        e.transpose16(b["W0"], b["W0T"])
        e.dense_gemm(b["A"], b["W0T"], b["recon"], off, segs, 1.0, self.status)            # recon = A W0
        if self.world > 1:
            pops.all_reduce(b["recon"], group=self.group)  # every rank goes on with the whole auxiliary reconstruction
        b["loss"].zero_()
        # fp16: dL/d recon (about 1e-8 per element) is kept times the loss scale, the fp32 gradient products are unscaled below
        e.aux_residual(b["recon"], m.dec_bias.data, b["bias_row"], self.sigma, self.gs, b["g"], b["loss"], live, self.step_ctl, float(factor),
                       self.fp16)
        e.dense_gemm(b["g"], b["W0"], b["G"], off, segs, 1.0, self.status)                 # G = g W0^T
        e.transpose16(b["A"], b["AT"])
        e.transpose16(b["G"], b["GT"], b["A"])   # straight-through: the gradient stays at the kept positions
        e.transpose16(b["g"], b["gT"])
        XT = self._transposed_inputs(X)
        e.dense_gemm(b["AT"], b["gT"], b["dW0"], off, segs, 1.0, self.status)              # dW0 = A^T g
        e.dense_gemm(b["GT"], XT, b["dWenc"], off, segs, 1.0, self.status)                 # dW_enc = G^T x
        e.rowsum16(b["GT"], b["dbenc"])
        e.rowsum16(b["gT"], b["gsum"])
        if self.fp16:
            for name in ("dW0", "dWenc", "dbenc", "gsum"):
                e.unscale(b[name], self.step_ctl)
            self.kernel_launches += 4
        b["bias_grad"].zero_()
        b["bias_grad"].index_copy_(0, b["bias_row_long"], b["gsum"])
        self.kernel_launches += 17
        return b

    # -------------------------------------------------------------------- step
    def train_step(self, X: torch.Tensor, Y: torch.Tensor, step: int, lr: float, sparsity_lambda: float = 0.0,
                   preactivation_coef: float = 0.0, aux_factor: float = 0.0, dead_mask: Optional[torch.Tensor] = None,
                   dead_window: Optional[int] = None) -> StepOutput:
        """One optimisation step on inputs/targets ``[L, B, d]`` (bf16 or fp16, already normalised).

        Everything that decides whether and how the update is applied stays on the device: the loss kernels raise a
        flag when the gradient seed overflows (fp16 loss scaling) or is not finite, ``step_control`` turns flag,
        status word and loss into the skip decision, keeps the loss scale and (with ``gradient_clip_val``) computes
        the clip coefficient from the norm pre-pass; the optimizer kernels read all of it from ``step_ctl``.

        ``preactivation_coef`` and ``aux_factor`` switch on the two loss terms that are not sparse; they enter the
        optimizer kernels as side gradients.  The dead features of the auxiliary term come from ``dead_window`` (a
        feature is dead when its counter exceeds it; everything stays on the device) or from an explicit
        ``dead_mask [L, valid_features]``."""
        e, m, tc = self.ext, self.model, self.tc
        L, B, d = self.L, self.B, self.d
        self.opt_step += 1
        self._begin_step()
        self.encode_select(X, fresh=False)
        c_g = 2.0 / (B * d)
        ctl = self.step_ctl
        jr = self.fn == "jumprelu"
        enc_dense = encb_dense = dec0_dense = None
        extra_bias_grad = None
        use_pre = abs(preactivation_coef) >= 1e-9
        use_aux = bool(aux_factor) and (dead_mask is not None or dead_window is not None)
        aux_cap = 0
        if use_aux:
            if getattr(self, "_aux_cap_wanted", None) is None:  # first use without a hint: one host read (agreed over the ranks)
                src = dead_mask if dead_mask is not None else (self.dead_counter.view(L, self.Fl)[:, : self.Fv] > int(dead_window))
                counts = src.sum(dim=1).to(torch.int32)
                local_max = counts.max().reshape(1)
                if self.world > 1:
                    pops.all_reduce(counts, group=self.group)
                    pops.all_reduce(local_max, op=pops.MAX, group=self.group)
                self.set_dead_count_hint(int(local_max.item()), int(counts.max().item()))
            aux_cap = self._aux_cap_wanted
            if self.world > 1 and self._aux_global_hint > 512:
                aux_cap = 0  # more dead features than k_aux: the per-token selection has to be agreed across the shards
        aux = None
        enc_x_idx = enc_x_rows = enc_x_bias = dec_x_idx = dec_x_rows = None
        # loss terms that only need the selection come first, so that their sums are there when the loss is settled
        pen = None
        use_pen = sparsity_lambda > 1e-9 and (self.fn != "batchtopk" or (tc.apply_sparsity_penalty_to_batchtopk if tc is not None else True))
        if use_pen:
            e.sparsity_penalty(self.feat_off, self.fcsr_val, self.feature_norm2(), float(sparsity_lambda), float(tc.sparsity_c),
                               self.grad_a, self.pen_coef, self.penalty)
            pen = self.pen_coef
            self.kernel_launches += 1
        if use_pre or (use_aux and aux_cap == 0):
            enc_dense, encb_dense, dec0_dense = self._extra_buffers()
            encb_dense.zero_()
            if use_pre:
                self._preactivation_term(X, float(preactivation_coef))  # writes every element of enc_dense
            else:
                enc_dense.zero_()
            if not use_aux:
                dec0_dense = None
        self.decode_loss(Y)
        # the loss is settled here; under tensor parallelism the exchange inside is also the barrier behind the
        # all-gather of the gradient seed, so everything below sees every token's seed row
        losses = torch.empty(8, dtype=torch.float32, device=self.dev)
        self._control(0, losses)
        if use_aux and aux_cap > 0:
            if dead_mask is not None:
                counter, window = torch.nn.functional.pad(dead_mask.to(torch.int64), (0, self.Fl - dead_mask.shape[-1])).reshape(-1), 0
            else:
                counter, window = self.dead_counter, int(dead_window)
            aux = self._auxiliary_term_fused(X, counter, window, float(aux_factor), aux_cap)
            extra_bias_grad = aux["bias_grad"]
            dec0_dense = None
            dec_x_idx, dec_x_rows = aux["extra_idx"], aux["dW0"]
            if use_pre:  # the dense encoder gradient of the pre-activation term takes the compact rows in
                e.scatter_add_rows(enc_dense, encb_dense, aux["dWenc"], aux["dbenc"], aux["extra_idx"])
                self.kernel_launches += 1
            else:
                enc_dense = encb_dense = None
                enc_x_idx, enc_x_rows, enc_x_bias = aux["extra_idx"], aux["dWenc"], aux["dbenc"]
            losses[0::4].add_(aux["loss"].float())  # evaluated on the finished residual, after the loss was settled
        elif use_aux:
            dec0_dense.zero_()
            mask = dead_mask if dead_mask is not None else (self.dead_counter.view(L, self.Fl)[:, : self.Fv] > int(dead_window))
            if mask.shape[-1] != self.Fl:
                mask = torch.nn.functional.pad(mask, (0, self.Fl - mask.shape[-1]))
            aux_val = self._auxiliary_term(X, mask, float(aux_factor))
            extra_bias_grad = self._aux_bias_grad
            losses[4] += aux_val  # the auxiliary term is evaluated on the finished residual, after the loss was settled
            losses[0] += aux_val
        gs_dec, tying_dec = self.gs, self.tying
        if self.affine:
            for g in (self.d_foff, self.d_fsc):
                if g is not None:
                    g.zero_()
        if self.tying == 1 and not self.affine:
            e.gs_suffix_sum(self.gs, self.gs_cum)
            gs_dec, tying_dec = self.gs_cum, 0
            self.kernel_launches += 1
        if jr:
            # window sums for the threshold gradient, from the decoder weights of this step (before their update)
            gs_cum = self.gs_cum if (self.tying == 1 and not self.affine) else None
            e.theta_grad_gemm(self.gs, [w.data for w in m.dec_weight], self.preact, self.theta, float(m.bandwidth), self.S1, self.S2,
                              self.status, self.tying, gs_cum)
            self.kernel_launches += 1
        # decoder biases: dL/db[pair (s,t)] = c_g * sum_b gs[t, b, :]
        e.gs_colsum(self.gs, self.gs_sum)
        dec_w = [w.data for w in m.dec_weight]
        skip_grad = self._skip_grad(X) if m.skip_weight is not None else None
        h_dec, h_enc = self._hyper(lr, c_g), self._hyper(lr, 1.0)
        clip = self.clip_val > 0.0
        grad_a_for_update = self.grad_a
        if clip:
            # gradient-norm pre-pass: the row gradients are formed once without touching weights or moments (features
            # without entries have none), dL/da is written on the way; step_control turns the norm into the coefficient
            rep = 1.0 / self.world  # replicated parameters are counted once over the ranks
            e.decoder_rows_adam(dec_w, self.dec_m, self.dec_v, L, B, d, self.Fl, tying_dec, self.feat_off, self.fcsr_tok, self.fcsr_val,
                                gs_dec, self.grad_a, pen, None, self.foff32, self.fsc32, dec0_dense, h_dec, None, dec_x_idx, dec_x_rows, ctl, True,
                                self.d_foff, self.d_fsc)
            self._affine_adam(h_enc, ctl, norm_weight=1.0)
            e.decoder_bias_adam(m.dec_bias.data, self.decb_m, self.decb_v, self.bias_sel, self.gs_sum, extra_bias_grad, h_dec, ctl, rep)
            e.encoder_rows_adam(m.enc_weight.data, self.enc_m, self.enc_v, m.enc_bias.data, self.encb_m, self.encb_v, self.feat_off,
                                self.fcsr_tok, self.grad_a, X, enc_dense, encb_dense, h_enc, None, enc_x_idx, enc_x_rows, enc_x_bias, ctl, True)
            if skip_grad is not None:
                e.dense_adam(m.skip_weight.data, self.skip_m, self.skip_v, skip_grad, h_dec, ctl, True, rep)
            if jr:
                self._theta_update(lr, c_g, float(sparsity_lambda) if use_pen else 0.0, norm_weight=1.0)
            self._control(1, losses)
            grad_a_for_update = None  # dL/da is complete; the update pass must not add to it again
            self.kernel_launches += 4
        if self.sweep_begin is not None:
            self.sweep_begin.record()
        e.decoder_rows_adam(dec_w, self.dec_m, self.dec_v, L, B, d, self.Fl, tying_dec,
                            self.feat_off, self.fcsr_tok, self.fcsr_val, gs_dec, grad_a_for_update, pen, self.norm2_next,
                            self.foff32, self.fsc32, dec0_dense, h_dec, self.status, dec_x_idx, dec_x_rows, ctl, False,
                            self.d_foff, self.d_fsc)
        self._affine_adam(h_enc, ctl)
        if jr:
            # thresholds: uses the decoder norms of this step (before the swap below)
            self._theta_update(lr, c_g, float(sparsity_lambda) if use_pen else 0.0)
        self._swap_norms()
        e.decoder_bias_adam(m.dec_bias.data, self.decb_m, self.decb_v, self.bias_sel, self.gs_sum, extra_bias_grad, h_dec, ctl, 0.0)
        if skip_grad is not None:
            e.dense_adam(m.skip_weight.data, self.skip_m, self.skip_v, skip_grad, h_dec, ctl, True, 0.0)
        e.encoder_rows_adam(m.enc_weight.data, self.enc_m, self.enc_v, m.enc_bias.data, self.encb_m, self.encb_v,
                            self.feat_off, self.fcsr_tok, self.grad_a, X, enc_dense, encb_dense, h_enc, self.status, enc_x_idx, enc_x_rows, enc_x_bias, ctl, False)
        # dead-feature counters and the bias sums of the next step's loss epilogue
        e.step_finish(self.dead_counter, self.fired, m.dec_bias.data, self.bias_sel, self.bias_sum)
        self.kernel_launches += 6  # gs_colsum, decoder rows, decoder biases, encoder rows (+ bias), finish
        m.invalidate_decoder_norms()
        out = StepOutput(losses, self.ctl[3])
        self.last_output = out
        return out

    def _affine_adam(self, hyper, ctl, norm_weight: float = 0.0) -> None:
        """AdamW on the feature offset / scale of tied decoders from the accumulators that the decoder sweep filled; the fp32
        copies that the kernels read follow the stored (16-bit) parameters.  ``norm_weight`` > 0: gradient-norm pre-pass."""
        if not self.affine:
            return
        m = self.model
        for prm, mirror, grad, names in ((m.feature_offset, self.foff32, self.d_foff, ("foff_m", "foff_v")),
                                         (m.feature_scale, self.fsc32, self.d_fsc, ("fsc_m", "fsc_v"))):
            if prm is None:
                continue
            self.ext.dense_adam(prm.data, getattr(self, names[0]), getattr(self, names[1]), grad, hyper, ctl, False, norm_weight)
            if norm_weight == 0.0:
                mirror.copy_(prm.data)
            self.kernel_launches += 1

    def _swap_norms(self) -> None:
        self.norm2, self.norm2_next = self.norm2_next, self.norm2
        self._norm_cur = 1 - self._norm_cur
        self.norms_valid = True

    @torch.no_grad()
    def _theta_update(self, lr: float, c_g: float, lam: float, norm_weight: float = 0.0) -> None:
        """AdamW step on ``log_threshold`` from the window sums of ``theta_grad_gemm`` (one kernel).

        ``d loss / d theta[f] = -(1 / bw) * sum_b window * x * G`` with ``G = c_g * (gs . W rows)`` for the
        reconstruction and ``lam * c * n_f * sech^2(c * n_f * a)`` for the sparsity penalty; the latter is a
        per-feature constant except at the active entries, which the feature's entry list corrects
        (reference: clt/models/activations.py:196-220 with clt/training/losses.py:179-185)."""
        m, tc = self.model, self.tc
        self.ensure_norms()
        self.ext.theta_adam(m.log_threshold.data, self.theta_m, self.theta_v, self.theta, self.S1, self.S2, self.norm2,
                            self.feat_off, self.fcsr_val, self.tying, c_g, lam, float(tc.sparsity_c), float(m.bandwidth),
                            self._hyper(lr, 1.0), self.step_ctl, norm_weight, self.grad_log_threshold)
        self.kernel_launches += 1

    # --------------------------------------------------------------- inference
    @torch.no_grad()
    def forward(self, X: torch.Tensor, Y: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Reconstructions ``[L, B, d]`` (fp32) for inputs ``X``; ``Y`` defaults to zeros."""
        self.encode_select(X)
        if Y is None:
            Y = torch.zeros_like(X)
        keep = self.step_ctl.clone()  # an inference forward must not disturb the loss-scale state
        yhat = self.decode_loss(Y, want_yhat=True)
        self.step_ctl.copy_(keep)
        return yhat

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
        if self.symm is not None and hasattr(self.symm, "check_canaries") and (code != 0 or self._check_guards):
            hit = self.symm.check_canaries()
            if hit:
                raise EngineStatusError(f"rank {self.rank}: guard bytes behind the exchange sections {hit} were overwritten")
        if code != 0:
            detail = f" (site {int(self.status[2])}, value {int(self.status[3])})" if code == 5 else ""
            self.status.zero_()
            raise EngineStatusError(f"rank {self.rank}: fused step reported '{STATUS_NAMES.get(code, code)}'{detail}")

    # ------------------------------------------------------- optimizer state io
    def optimizer_state_dict(self) -> Dict[str, torch.Tensor]:
        sd = {"step": torch.tensor(self.opt_step), "enc_m": self.enc_m, "enc_v": self.enc_v, "encb_m": self.encb_m,
              "encb_v": self.encb_v, "decb_m": self.decb_m, "decb_v": self.decb_v, "dead_counter": self.dead_counter,
              "step_ctl": self.step_ctl}
        for i, (mm, vv) in enumerate(zip(self.dec_m, self.dec_v)):
            sd[f"dec_m.{i}"] = mm
            sd[f"dec_v.{i}"] = vv
        if self.fn == "jumprelu":
            sd["theta_m"], sd["theta_v"] = self.theta_m, self.theta_v
        if self.model.skip_weight is not None:
            sd["skip_m"], sd["skip_v"] = self.skip_m, self.skip_v
        for name in ("foff_m", "foff_v", "fsc_m", "fsc_v"):
            if hasattr(self, name):
                sd[name] = getattr(self, name)
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
        if "step_ctl" in sd:
            self.step_ctl.copy_(sd["step_ctl"].to(self.step_ctl.dtype))
        for name in ("foff_m", "foff_v", "fsc_m", "fsc_v"):
            if hasattr(self, name) and name in sd:
                getattr(self, name).copy_(sd[name])
        self.invalidate_cached()

    def refresh_affine(self) -> None:
        """Re-reads the fp32 copies of the feature offset / scale after the parameters were changed from outside."""
        if getattr(self, "affine", False):
            if self.foff32 is not None:
                self.foff32.copy_(self.model.feature_offset.data)
            if self.fsc32 is not None:
                self.fsc32.copy_(self.model.feature_scale.data)

    def invalidate_cached(self) -> None:
        """Forget everything derived from the parameters (after a checkpoint load or an external weight change)."""
        self.norms_valid = False
        self._bias_sum_valid = False
        if self.fn == "jumprelu":
            self._theta_valid = False
        self.refresh_affine()
