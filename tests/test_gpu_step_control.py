"""Fused step: gradient magnitudes, multi-step trajectories against torch.optim.AdamW, the device-side step control
(non-finite skip, fp16 loss scaling, gradient clipping), ReLU training and JumpReLU with tied decoders.
Every kernel result is compared with a plain PyTorch fp32 restatement of the same step."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

SC_SKIP, SC_INV_SCALE, SC_LOSS_SCALE, SC_GROWTH, SC_FOUND_INF, SC_GRAD_NORM_SQ, SC_CLIP, SC_SKIPPED = range(8)


def _dev():
    return torch.device("cuda:0")


def _make(fn="batchtopk", tying="none", dtype="bfloat16", L=3, B=192, d=64, F=256, k=6, seed=0, theta=0.35, **tc_kw):
    from crosslayer_coding_b200 import CLTConfig, CrossLayerTranscoder, TrainingConfig
    from crosslayer_coding_b200.training.fused_engine import FusedBatchTopKEngine

    torch.manual_seed(seed)
    dev = _dev()
    cfg = CLTConfig(num_features=F, num_layers=L, d_model=d, activation_fn=fn, batchtopk_k=k, clt_dtype=dtype, decoder_tying=tying,
                    jumprelu_threshold=theta)
    model = CrossLayerTranscoder(cfg, device=dev)
    with torch.no_grad():
        model.enc_weight.normal_(0, 1.0 / math.sqrt(d))
        if tying != "none":
            for w in model.dec_weight:
                w.uniform_(-0.05, 0.05)
    kw = dict(learning_rate=1e-3, training_steps=100, activation_path="unused", precision=("fp16" if dtype == "float16" else "bf16"),
              sparsity_lambda=0.0, preactivation_coef=0.0, optimizer="adamw")
    kw.update(tc_kw)
    tc = TrainingConfig(**kw)
    eng = FusedBatchTopKEngine(model, tc, B)
    t16 = torch.float16 if dtype == "float16" else torch.bfloat16
    X = torch.randn(L, B, d, device=dev).to(t16)
    Y = torch.randn(L, B, d, device=dev).to(t16)
    return cfg, model, tc, eng, X, Y


def _fp32_copy(model):
    from crosslayer_coding_b200 import CLTConfig, CrossLayerTranscoder

    cfg = CLTConfig(**{**model.config.to_dict(), "clt_dtype": "float32"})
    ref = CrossLayerTranscoder(cfg, device=model.enc_weight.device)
    with torch.no_grad():
        for (_, a), (_, b) in zip(ref.named_parameters(), model.named_parameters()):
            a.copy_(b.float())
    return ref


def _reference_loss(ref, eng, X, Y, lam, tc):
    """Loss of the fp32 model on the entries that the engine selected (pre-activations as the kernels saw them)."""
    L = ref.config.num_layers
    dense = eng.activations_dense()
    mask = dense != 0
    pre = {l: torch.nn.functional.linear(X[l].float(), ref.enc_weight[l], ref.enc_bias[l]) for l in range(L)}
    acts = {l: (pre[l] + (eng.preact[l].float() - pre[l]).detach()) * mask[l] for l in range(L)}
    loss = sum(torch.nn.functional.mse_loss(ref.decode({s: acts[s] for s in range(t + 1)}, t), Y[t].float()) for t in range(L))
    if lam > 0:
        ref.invalidate_decoder_norms()  # the cached norms belong to the previous step's graph
        norms = ref.get_decoder_norms()
        loss = loss + lam * sum(torch.tanh(tc.sparsity_c * acts[l] * norms[l][None, :]).sum() for l in range(L))
    return loss


def _rel_err(a, b):
    return float((a - b).norm() / (b.norm() + 1e-12))


@pytest.mark.parametrize("tying", ["none", "per_source", "per_target"])
@pytest.mark.parametrize("lam", [0.0, 0.05])
def test_first_moments_equal_autograd_gradients(tying, lam):
    """After one step from zero moments, m / (1 - beta1) is the gradient itself: a wrong factor in the gradient scale, the
    penalty coefficient or dL/da shows up here (the weight update of a first Adam step only shows the sign)."""
    cfg, model, tc, eng, X, Y = _make(tying=tying, seed=11)
    ref = _fp32_copy(model)
    eng.train_step(X, Y, step=0, lr=1e-3, sparsity_lambda=lam)
    torch.cuda.synchronize()
    eng.check_status()
    _reference_loss(ref, eng, X, Y, lam, tc).backward()
    b1 = 0.9
    for i, w in enumerate(ref.dec_weight):
        assert _rel_err(eng.dec_m[i] / (1 - b1), w.grad) < 2e-2, (tying, lam, i)
    assert _rel_err(eng.enc_m / (1 - b1), ref.enc_weight.grad) < 2e-2
    assert _rel_err(eng.encb_m / (1 - b1), ref.enc_bias.grad) < 2e-2
    assert _rel_err(eng.decb_m / (1 - b1), ref.dec_bias.grad) < 2e-2


def test_five_step_trajectory_tracks_adamw():
    """Five fused steps against five steps of torch.optim.AdamW on an fp32 copy fed with the engine's own selections."""
    cfg, model, tc, eng, X, Y = _make(seed=13)
    ref = _fp32_copy(model)
    start = {n: p.detach().float().clone() for n, p in model.named_parameters()}
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-3)
    for step in range(5):
        eng.train_step(X, Y, step=step, lr=1e-3, sparsity_lambda=0.02)
        torch.cuda.synchronize()
        opt.zero_grad()
        _reference_loss(ref, eng, X, Y, 0.02, tc).backward()
        opt.step()
    eng.check_status()
    refp = dict(ref.named_parameters())
    for n, p in model.named_parameters():
        moved = refp[n].detach() - start[n]
        got = p.detach().float() - start[n]
        # bf16 weights: each of the five updates is rounded to 8 bits of mantissa, so the end point is compared in units of
        # the weight's own spacing (2^-8 relative), the direction of the move as a whole
        ulp = torch.maximum(refp[n].detach().abs(), start[n].abs()) * 2.0 ** -8 + 1e-6
        tol = 5.0 * ulp + 0.25 * moved.abs()  # five roundings of up to half a step each, on top of the move itself
        off = ((p.detach().float() - refp[n].detach()).abs() > tol).float().mean().item()
        assert off < 1e-2, (n, off)
        assert _rel_err(got, moved) < 0.35, (n, _rel_err(got, moved))
        cos = float((got * moved).sum() / (got.norm() * moved.norm() + 1e-12))
        assert cos > 0.93, (n, cos)


def test_nonfinite_target_skips_the_step():
    cfg, model, tc, eng, X, Y = _make(seed=3)
    eng.train_step(X, Y, step=0, lr=1e-3)
    torch.cuda.synchronize()
    before = {n: p.detach().clone() for n, p in model.named_parameters()}
    m_before = eng.dec_m[0].clone()
    bad = Y.clone()
    bad[1, 5, 3] = float("nan")
    out = eng.train_step(X, bad, step=1, lr=1e-3)
    torch.cuda.synchronize()
    assert int(eng.step_ctl[SC_SKIP].view(torch.int32)) == 1 and int(out.skipped_steps) == 1
    for n, p in model.named_parameters():
        assert torch.equal(p.detach(), before[n]), n
    assert torch.equal(eng.dec_m[0], m_before)
    out = eng.train_step(X, Y, step=2, lr=1e-3)  # the next clean step is applied again
    torch.cuda.synchronize()
    assert int(eng.step_ctl[SC_SKIP].view(torch.int32)) == 0 and not torch.equal(model.dec_weight[0].detach(), before["dec_weight.0"])
    assert math.isfinite(float(out.total))


@pytest.mark.parametrize("tying", ["none", "per_source"])
def test_fp16_loss_scaling_backs_off_then_trains(tying):
    """fp16 weights and gradient seed with the dynamic loss scale on the device: the initial scale overflows the fp16 seed,
    the step is skipped and the scale halves (GradScaler's policy); once it fits, the update equals the unscaled one."""
    cfg, model, tc, eng, X, Y = _make(tying=tying, dtype="float16", seed=5, loss_scale_init=2.0 ** 17, loss_scale_growth_interval=3)
    assert eng.fp16 and float(eng.step_ctl[SC_LOSS_SCALE]) == 2.0 ** 17
    w0 = model.dec_weight[0].detach().clone()
    out = eng.train_step(X, Y, step=0, lr=1e-3)          # |gs| ~ a few units * 131072 > 65504: overflow
    torch.cuda.synchronize()
    assert int(out.skipped_steps) == 1 and float(eng.step_ctl[SC_LOSS_SCALE]) == 2.0 ** 16
    assert torch.equal(model.dec_weight[0].detach(), w0)
    scales = []
    for step in range(1, 12):
        out = eng.train_step(X, Y, step=step, lr=1e-3)
        scales.append(float(out.loss_scale))
    torch.cuda.synchronize()
    eng.check_status()
    assert min(scales) < 2.0 ** 16 and int(out.skipped_steps) < 11      # it backed off further and then trained
    assert not torch.equal(model.dec_weight[0].detach(), w0)
    # a clean step at a fitting scale: the moments hold unscaled gradients
    cfg2, model2, tc2, eng2, _, _ = _make(tying=tying, dtype="float16", seed=5, loss_scale_init=256.0, loss_scale_growth_interval=4)
    ref = _fp32_copy(model2)
    eng2.train_step(X, Y, step=0, lr=1e-3)
    torch.cuda.synchronize()
    assert int(eng2.step_ctl[SC_SKIP].view(torch.int32)) == 0
    _reference_loss(ref, eng2, X, Y, 0.0, tc2).backward()
    assert _rel_err(eng2.dec_m[0] / 0.1, ref.dec_weight[0].grad) < 2e-2
    assert _rel_err(eng2.enc_m / 0.1, ref.enc_weight.grad) < 2e-2
    # growth: after `growth_interval` clean steps the scale doubles
    for step in range(1, 4):
        out = eng2.train_step(X, Y, step=step, lr=1e-3)
    torch.cuda.synchronize()
    assert float(eng2.step_ctl[SC_LOSS_SCALE]) == 512.0


@pytest.mark.parametrize("tying", ["none", "per_target"])
def test_gradient_clipping_by_global_norm(tying):
    """gradient_clip_val: the norm pre-pass reports the global gradient norm and the update uses clipped gradients."""
    lam = 0.03
    cfg, model, tc, eng, X, Y = _make(tying=tying, seed=17, gradient_clip_val=0.05)
    ref = _fp32_copy(model)
    out = eng.train_step(X, Y, step=0, lr=1e-3, sparsity_lambda=lam)
    torch.cuda.synchronize()
    eng.check_status()
    _reference_loss(ref, eng, X, Y, lam, tc).backward()
    total = torch.sqrt(sum((p.grad.float() ** 2).sum() for p in ref.parameters() if p.grad is not None))
    assert abs(float(out.grad_norm) - float(total)) < 2e-2 * float(total), (float(out.grad_norm), float(total))
    coef = min(1.0, 0.05 / (float(total) + 1e-6))
    assert coef < 1.0 and abs(float(eng.step_ctl[SC_CLIP]) - coef) < 2e-2 * coef
    assert _rel_err(eng.dec_m[0] / 0.1, ref.dec_weight[0].grad * coef) < 3e-2
    assert _rel_err(eng.enc_m / 0.1, ref.enc_weight.grad * coef) < 3e-2
    assert _rel_err(eng.decb_m / 0.1, ref.dec_bias.grad * coef) < 3e-2
    # a generous limit leaves the step unchanged
    _, model_a, _, eng_a, _, _ = _make(tying=tying, seed=17, gradient_clip_val=1e6)
    _, model_b, _, eng_b, _, _ = _make(tying=tying, seed=17)
    eng_a.train_step(X, Y, step=0, lr=1e-3, sparsity_lambda=lam)
    eng_b.train_step(X, Y, step=0, lr=1e-3, sparsity_lambda=lam)
    torch.cuda.synchronize()
    assert torch.allclose(eng_a.enc_m, eng_b.enc_m, rtol=1e-4, atol=1e-7) and torch.equal(model_a.dec_weight[0], model_b.dec_weight[0])


def _jumprelu_reference(ref, eng, X, Y, lam, tc):
    """Dense fp32 JumpReLU step with the straight-through threshold gradient, on the pre-activations the kernels saw."""
    from crosslayer_coding_b200.models import activations as act

    L = ref.config.num_layers
    acts = {}
    for l in range(L):
        pre = torch.nn.functional.linear(X[l].float(), ref.enc_weight[l], ref.enc_bias[l])
        pre = pre + (eng.preact[l].float() - pre).detach()
        acts[l] = act.JumpReLU.apply(pre, ref.log_threshold[l].exp(), ref.bandwidth)
    loss = sum(torch.nn.functional.mse_loss(ref.decode({s: acts[s] for s in range(t + 1)}, t), Y[t].float()) for t in range(L))
    if lam > 0:
        norms = ref.get_decoder_norms()
        loss = loss + lam * sum(torch.tanh(tc.sparsity_c * acts[l] * norms[l][None, :]).sum() for l in range(L))
    return loss


@pytest.mark.parametrize("tying", ["per_source", "per_target"])
@pytest.mark.parametrize("lam", [0.0, 0.02])
def test_fused_jumprelu_with_tied_decoders_matches_autograd(tying, lam):
    cfg, model, tc, eng, X, Y = _make(fn="jumprelu", tying=tying, seed=23, B=256, F=256, d=64, theta=1.2)
    ref = _fp32_copy(model)
    eng.train_step(X, Y, step=0, lr=1e-3, sparsity_lambda=lam)
    torch.cuda.synchronize()
    eng.check_status()
    _jumprelu_reference(ref, eng, X, Y, lam, tc).backward()
    g = ref.log_threshold.grad
    assert _rel_err(eng.grad_log_threshold, g) < 3e-2, _rel_err(eng.grad_log_threshold, g)
    assert _rel_err(eng.theta_m / 0.1, g) < 3e-2
    for i, w in enumerate(ref.dec_weight):
        assert _rel_err(eng.dec_m[i] / 0.1, w.grad) < 2e-2
    assert _rel_err(eng.enc_m / 0.1, ref.enc_weight.grad) < 2e-2


def test_fused_relu_training_step_matches_autograd():
    cfg, model, tc, eng, X, Y = _make(fn="relu", seed=29, B=128, F=128, d=64, fused_max_active_per_token=512)
    with torch.no_grad():
        model.enc_bias.fill_(-1.6)  # sparse enough for the entry lists
    ref = _fp32_copy(model)
    out = eng.train_step(X, Y, step=0, lr=1e-3, sparsity_lambda=0.01)
    torch.cuda.synchronize()
    eng.check_status()
    L = cfg.num_layers
    pre = {l: torch.nn.functional.linear(X[l].float(), ref.enc_weight[l], ref.enc_bias[l]) for l in range(L)}
    acts = {l: torch.relu(pre[l] + (eng.preact[l].float() - pre[l]).detach()) for l in range(L)}
    assert torch.equal(eng.activations_dense() != 0, torch.stack([acts[l] for l in range(L)]) > 0)
    loss = sum(torch.nn.functional.mse_loss(ref.decode({s: acts[s] for s in range(t + 1)}, t), Y[t].float()) for t in range(L))
    norms = ref.get_decoder_norms()
    loss = loss + 0.01 * sum(torch.tanh(tc.sparsity_c * acts[l] * norms[l][None, :]).sum() for l in range(L))
    loss.backward()
    assert abs(float(out.total) - float(loss)) < 5e-3 * abs(float(loss))
    assert _rel_err(eng.enc_m / 0.1, ref.enc_weight.grad) < 2e-2
    assert _rel_err(eng.dec_m[0] / 0.1, ref.dec_weight[0].grad) < 2e-2


def test_exact_cut_with_heavy_ties_is_world_invariant_and_lowest_index_first():
    """Many identical z-scores at the cut (constant columns give equal keys): the gathered exact cut keeps the lowest
    flat indices, whatever the number of candidates; with more ties than the one-round gather holds the radix rounds
    give the same answer."""
    from crosslayer_coding_b200.ops import ext as ext_mod

    e = ext_mod.load()
    dev = _dev()
    for B, F, k in ((8, 16, 5), (64, 128, 5), (512, 1024, 3)):  # gathered cut; radix rounds; radix rounds, large
        L = 2
        x = torch.zeros(L, B, F, device=dev)
        x[:, ::2, :] = 1.0          # every column: half the rows at 1, half at 0 -> two distinct z values, massive ties
        x[0, 1, 7] = 3.0            # a few distinct larger ones
        x = x.bfloat16().contiguous()
        mean = torch.empty(L, F, device=dev)
        rstd = torch.empty(L, F, device=dev)
        e.colstats(x, mean, rstd)
        k_total = k * B
        i32, f32 = torch.int32, torch.float32
        hist = torch.zeros(2 * 8192 + 32, dtype=i32, device=dev)
        ctl = torch.zeros(16, dtype=torch.int64, device=dev)
        status = torch.zeros(4, dtype=i32, device=dev)
        cap = L * B * F
        ent = [torch.empty(cap, dtype=i32, device=dev), torch.empty(cap, dtype=i32, device=dev), torch.empty(cap, dtype=f32, device=dev)]
        cand = [torch.empty(cap, dtype=i32, device=dev), torch.empty(cap, dtype=i32, device=dev), torch.empty(cap, dtype=i32, device=dev),
                torch.empty(cap, dtype=f32, device=dev)]
        e.batchtopk_select(x, mean, rstd, F, F, 0, F, k_total, 0, 19, hist, ctl, ent[0], ent[1], ent[2], cand[0], cand[1], cand[2], cand[3],
                           status, 1, 0, [], [], 0, 0, None, None)
        torch.cuda.synchronize()
        assert int(status[0]) == 0 and int(ctl[3]) == k_total
        n = k_total
        flat = ent[0][:n].long() * (L * F) + ent[1][:n].long()
        z = ((x.float() - mean[:, None, :]) * rstd[:, None, :]).permute(1, 0, 2).reshape(-1)   # flat index = b * L * F + l * F + f
        order = torch.sort(z, descending=True, stable=True).indices[:n]                           # stable: lowest index first among ties
        assert torch.equal(torch.sort(flat).values, torch.sort(order).values)


@pytest.mark.parametrize("in_dtype,out_dtype", [(torch.bfloat16, torch.bfloat16), (torch.float32, torch.float16), (torch.float16, torch.bfloat16)])
def test_normalize_cast_matches_fp32_reference(in_dtype, out_dtype):
    from crosslayer_coding_b200.ops import ext as ext_mod

    e = ext_mod.load()
    dev = _dev()
    torch.manual_seed(0)
    L, B, d = 3, 70, 48
    raw = (torch.randn(2, L, B, d, device=dev) * 3 + 1).to(in_dtype)
    mean = torch.randn(2 * L, d, device=dev)
    std = torch.rand(2 * L, d, device=dev) + 0.5
    out = torch.empty(2, L, B, d, dtype=out_dtype, device=dev)
    e.normalize_cast(raw, out, mean, (1.0 / std).contiguous(), B, 1.0)
    want = ((raw.float() - mean.view(2, L, 1, d)) * (1.0 / std).view(2, L, 1, d)).to(out_dtype)
    assert torch.allclose(out.float(), want.float(), rtol=2 ** -7, atol=1e-6)
    e.normalize_cast(raw, out, None, None, 0, float(d ** 0.5))
    assert torch.allclose(out.float(), (raw.float() * d ** 0.5).to(out_dtype).float(), rtol=2 ** -7, atol=1e-6)


def test_scale_histogram_gives_l0_of_every_scale():
    from crosslayer_coding_b200.conversion import l0_for_scales

    dev = _dev()
    torch.manual_seed(1)
    B, F = 300, 520
    pre = torch.randn(B, F, device=dev).bfloat16()
    theta = torch.rand(F, device=dev) * 0.5 + 0.2
    scales = torch.logspace(-1, 1, 257, device=dev)
    got = l0_for_scales(pre, theta, scales)                          # kernel path (16-bit input on the GPU)
    ratio = pre.float() / theta
    want = torch.stack([(ratio >= s).float().sum() / B for s in scales])
    assert torch.equal((got * B).round(), (want * B).round()), (got - want).abs().max()  # the counts themselves are exact


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("out_dtype", ["f32", "t16"])
def test_grouped_dense_gemm_matches_fp32_reference(dtype, out_dtype):
    """C[g] = alpha * sum over the group's segments of A[a] @ B[b]^T, odd sizes (tile tails in M, N and K)."""
    from crosslayer_coding_b200.ops import ext as ext_mod

    e = ext_mod.load()
    dev = _dev()
    torch.manual_seed(2)
    LA, LB, M, N, K = 4, 5, 200, 328, 136
    A = (torch.randn(LA, M, K, device=dev) * 0.5).to(dtype)
    Bm = (torch.randn(LB, N, K, device=dev) * 0.5).to(dtype)
    groups = [[(0, 1)], [(1, 0), (2, 4), (3, 3)], [(3, 2), (0, 0)]]
    off = torch.tensor([0, 1, 4, 6], dtype=torch.int32, device=dev)
    segs = torch.tensor([p for g in groups for p in g], dtype=torch.int32, device=dev)
    C = torch.empty(len(groups), M, N, dtype=torch.float32 if out_dtype == "f32" else dtype, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    e.dense_gemm(A, Bm, C, off, segs, -0.25, status)
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    for g, seg in enumerate(groups):
        want = -0.25 * sum(A[a].float() @ Bm[b].float().t() for a, b in seg)
        tol = 2e-3 if out_dtype == "f32" else 3e-2
        assert torch.allclose(C[g].float(), want, rtol=tol, atol=tol), (g, (C[g].float() - want).abs().max())
    # transposes and the negative-indicator pass
    T = torch.empty(LA, K, M, dtype=dtype, device=dev)
    e.transpose16(A, T)
    assert torch.equal(T, A.transpose(1, 2).contiguous())
    pre = torch.randn(3, 130, 72, device=dev).to(dtype)
    ind = torch.empty(3, 72, 130, dtype=dtype, device=dev)
    bias_grad = torch.zeros(3, 72, device=dev)
    loss = torch.zeros(1, dtype=torch.float64, device=dev)
    e.negative_indicator(pre, ind, bias_grad, loss, 64, 0.5)     # the last 8 columns are padding
    neg = (pre.float() < 0)
    neg[:, :, 64:] = False
    assert torch.equal(ind.float(), neg.float().transpose(1, 2))
    assert torch.allclose(bias_grad, -0.5 * neg.float().sum(dim=1)) and abs(float(loss) - 0.5 * float((-pre.float() * neg).sum())) < 1e-2


def test_long_csr_segments_are_sorted_by_the_cooperative_path():
    """A feature that fires on every token and a token with hundreds of entries: both CSR views come out sorted."""
    from crosslayer_coding_b200.ops import ext as ext_mod

    e = ext_mod.load()
    dev = _dev()
    g = torch.Generator().manual_seed(4)
    T, L, pitch = 700, 2, 512
    ncols = L * pitch
    toks = torch.randperm(T, generator=g)                                   # column 5 on every token, shuffled
    ent_tok = [toks, torch.full((600,), 3)]                                  # token 3 with 600 more columns
    ent_col = [torch.full((T,), 5), torch.randperm(ncols - 10, generator=g)[:600] + 10]
    more = torch.randperm(T * ncols, generator=g)[:2000]
    more = more[((more % ncols) >= 10) & ((more // ncols) != 3)]
    ent_tok.append(more // ncols)
    ent_col.append(more % ncols)
    tok = torch.cat(ent_tok).to(torch.int32).to(dev)
    col = torch.cat(ent_col).to(torch.int32).to(dev)
    n = tok.numel()
    val = torch.randn(n, generator=g).to(dev)
    ctl = torch.zeros(16, dtype=torch.int64, device=dev)
    ctl[3] = n
    i32, f32 = torch.int32, torch.float32
    z = lambda k, dt=i32: torch.zeros(k, dtype=dt, device=dev)  # noqa: E731
    tok_off, feat_off = z(T + 1), z(ncols + 1)
    tcsr_col, tcsr_val, fcsr_tok, fcsr_val = z(n), z(n, f32), z(n), z(n, f32)
    e.build_csr(tok, col, val, ctl, T, ncols, z(T), z(ncols), tok_off, feat_off, z(T), z(ncols), tcsr_col, tcsr_val, fcsr_tok, fcsr_val, None, 3, pitch)
    torch.cuda.synchronize()
    b, en = int(feat_off[5]), int(feat_off[6])
    assert en - b == T and torch.equal(fcsr_tok[b:en].cpu(), torch.arange(T, dtype=torch.int32))
    order = torch.argsort(toks)
    assert torch.equal(fcsr_val[b:en].cpu(), val[:T].cpu()[order])          # values moved with their keys
    b, en = int(tok_off[3]), int(tok_off[4])
    seg = tcsr_col[b:en].cpu()
    assert en - b >= 600 and bool((seg[1:] > seg[:-1]).all())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_aux_compaction_and_per_token_selection(dtype):
    """Dead-column compaction and the exact per-token top-k of the dead pre-activations (ties by lowest index)."""
    from crosslayer_coding_b200.ops import ext as ext_mod

    ext = ext_mod.load()
    dev = _dev()
    torch.manual_seed(5)
    L, B, F, Fv, cap, k_aux = 3, 70, 1024, 1000, 512, 24
    counter = torch.zeros(L, F, dtype=torch.int64, device=dev)
    counter[0, ::3] = 11          # 342 dead (some beyond the valid range are ignored)
    counter[1, 5:17] = 99         # 12 dead: fewer than k_aux, all kept
    counter[2, :] = 50            # every valid feature dead: more than the capacity, truncated to the first `cap`
    dead_cols = torch.zeros(L, cap, dtype=torch.int32, device=dev)
    nd = torch.zeros(L, dtype=torch.int32, device=dev)
    nd_all = torch.zeros(L, dtype=torch.int32, device=dev)
    extra_idx = torch.zeros(L * F, dtype=torch.int32, device=dev)
    ext.aux_compact(counter.reshape(-1), 10, L, Fv, dead_cols, nd, nd_all, extra_idx)
    dead = (counter > 10) & (torch.arange(F, device=dev) < Fv)
    assert nd_all.tolist() == dead.sum(dim=1).tolist()
    assert nd.tolist() == [min(cap, n) for n in nd_all.tolist()]
    xi = extra_idx.view(L, F)
    for l in range(L):
        cols = dead[l].nonzero().flatten()[:cap]
        assert torch.equal(dead_cols[l, : len(cols)].long(), cols)
        assert torch.equal(xi[l, cols].long(), l * cap + torch.arange(len(cols), device=dev))
        rest = torch.ones(F, dtype=torch.bool, device=dev)
        rest[cols] = False
        assert bool((xi[l, rest] == -1).all())
    # values on a coarse grid, so that many of them tie at the cut
    pre = (torch.randint(-6, 7, (L, B, F), device=dev).float() * 0.25).to(dtype)
    A = torch.full((L, B, cap), 7.0, dtype=dtype, device=dev)
    ext.aux_gather_select(pre, None, dead_cols, nd, nd_all, k_aux, A)
    # second source: A holds the bias-free products, the bias of each dead column is added in the kernel
    bias = (torch.randint(-3, 4, (L, F), device=dev).float() * 0.25)
    A2 = torch.zeros(L, B, cap, dtype=dtype, device=dev)
    for l in range(L):
        cols = dead_cols[l, : int(nd[l])].long()
        A2[l, :, : len(cols)] = (pre[l][:, cols].float() - bias[l, cols]).to(dtype)
    ext.aux_gather_select(None, bias, dead_cols, nd, nd_all, k_aux, A2, torch.empty(L, cap, device=dev))
    assert torch.equal(A2, A)
    for l in range(L):
        n = int(nd[l])
        vals = pre[l][:, dead_cols[l, :n].long()].float()
        k = min(k_aux, int(nd_all[l]))
        want = torch.zeros(B, cap, device=dev)
        if n <= k:
            want[:, :n] = vals
        else:
            # stable descending sort = ties resolved towards the lowest index
            order = torch.sort(vals, dim=1, descending=True, stable=True).indices[:, :k]
            want[:, :n] = torch.zeros_like(vals).scatter_(1, order, vals.gather(1, order))
        assert torch.equal(A[l].float(), want), l
    # masked transpose: the gradient survives where the selection kept a value
    Bp = 72
    Gp = torch.randn(L, Bp, cap, device=dev).to(dtype)
    Ap = torch.zeros(L, Bp, cap, dtype=dtype, device=dev)
    Ap[:, :B] = A
    GT = torch.empty(L, cap, Bp, dtype=dtype, device=dev)
    ext.transpose16(Gp, GT, Ap)
    assert torch.equal(GT, (Gp * (Ap != 0)).transpose(1, 2).contiguous())
    ext.transpose16(Gp, GT)
    assert torch.equal(GT, Gp.transpose(1, 2).contiguous())


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
def test_fused_auxiliary_term_matches_loss_manager_beyond_k_aux(dtype):
    """More dead features than k_aux = 512: the kernel path (selection + grouped GEMMs + compact extra rows) against
    the PyTorch loss and one AdamW step; then the same step through the unfused per-layer path.  In fp16 the gradient of
    the auxiliary reconstruction travels times the loss scale and the fp32 products are unscaled on the device."""
    import copy

    from crosslayer_coding_b200.training.losses import LossManager

    cfg, model, tc, eng, X, Y = _make(L=2, B=128, d=64, F=2048, k=16, seed=21, dtype=dtype, loss_scale_init=4096.0)
    tc.aux_loss_factor = 0.25
    ref = _fp32_copy(model)
    twin = copy.deepcopy(model)
    snap = {n: p.detach().float().clone() for n, p in model.named_parameters()}
    L, F = 2, 2048
    dead = torch.zeros(L, F, dtype=torch.bool, device=X.device)
    dead[0, 100:1500] = True   # 1400 dead, 512 kept per token
    dead[1, ::9] = True        # 228 dead, all kept
    out = eng.train_step(X, Y, step=0, lr=1e-3, aux_factor=0.25, dead_mask=dead)
    torch.cuda.synchronize()
    eng.check_status()
    assert eng._aux_buf["cap"] >= 1400
    x = {l: X[l].float() for l in range(L)}
    y = {l: Y[l].float() for l in range(L)}
    acts_k = eng.activations_dense()
    pre = {l: torch.nn.functional.linear(x[l], ref.enc_weight[l], ref.enc_bias[l]) for l in range(L)}
    acts = {l: (pre[l] + (eng.preact[l].float() - pre[l]).detach()) * (acts_k[l] != 0) for l in range(L)}
    preds = {t: ref.decode({s: acts[s] for s in range(t + 1)}, t) for t in range(L)}
    lm = LossManager(tc)
    recon = lm.compute_reconstruction_loss(preds, y)
    pre_k = {l: pre[l] + (eng.preact[l].float() - pre[l]).detach() for l in range(L)}  # the values the kernels ranked
    aux = lm.compute_auxiliary_loss(ref, x, {l: y[l] - preds[l] for l in range(L)}, dead, preacts=pre_k)
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-3)
    (recon + aux).backward()
    opt.step()
    assert abs(out.auxiliary.item() - aux.item()) < 3e-2 * max(1e-3, aux.item()), (out.auxiliary.item(), aux.item())
    assert abs(out.total.item() - (recon + aux).item()) < 1e-2 * (recon + aux).item()
    ref_params = dict(ref.named_parameters())
    for name, p in model.named_parameters():
        old = snap[name]
        upd, ref_upd = p.detach().float() - old, ref_params[name].detach() - old
        bad = ((upd - ref_upd).abs() > 0.008 * old.abs() + 3e-4).float().mean().item()
        assert bad < 2e-2, (name, bad)
    # the unfused path (taken under tensor parallelism and for very large dead sets) gives the same step
    from crosslayer_coding_b200.training.fused_engine import FusedBatchTopKEngine

    eng2 = FusedBatchTopKEngine(twin, tc, X.shape[1])
    eng2._aux_cap_wanted = 0
    out2 = eng2.train_step(X, Y, step=0, lr=1e-3, aux_factor=0.25, dead_mask=dead)
    eng2.check_status()
    assert abs(out2.auxiliary.item() - out.auxiliary.item()) < 2e-2 * max(1e-3, out.auxiliary.item())
    for (name, p), (_, q) in zip(model.named_parameters(), twin.named_parameters()):
        diff = ((p.detach().float() - q.detach().float()).abs() > 0.008 * snap[name].abs() + 3e-4).float().mean().item()
        assert diff < 2e-2, (name, diff)


@pytest.mark.parametrize("tying,fn", [("per_source", "batchtopk"), ("per_target", "batchtopk"), ("per_source", "relu")])
def test_fused_feature_affine_of_tied_decoders_matches_autograd(tying, fn):
    """Feature offset / scale of tied decoders on the fused step: loss, first moments of every parameter (gradients) and the
    updated offset / scale against autograd on the entries that the engine selected."""
    from crosslayer_coding_b200 import CLTConfig, CrossLayerTranscoder, TrainingConfig
    from crosslayer_coding_b200.training.fused_engine import FusedBatchTopKEngine, engine_supports

    torch.manual_seed(31)
    dev = _dev()
    L, B, d, F, k = 3, 192, 64, 256, 6
    cfg = CLTConfig(num_features=F, num_layers=L, d_model=d, activation_fn=fn, batchtopk_k=k, clt_dtype="bfloat16", decoder_tying=tying,
                    enable_feature_offset=True, enable_feature_scale=True)
    model = CrossLayerTranscoder(cfg, device=dev)
    with torch.no_grad():
        model.enc_weight.normal_(0, 1.0 / math.sqrt(d))
        if fn == "relu":
            model.enc_bias.fill_(-1.2)
        for w in model.dec_weight:
            w.uniform_(-0.05, 0.05)
        model.feature_offset.copy_(torch.randn_like(model.feature_offset) * 0.2)
        model.feature_scale.copy_(1.0 + torch.randn_like(model.feature_scale) * 0.2)
    tc = TrainingConfig(learning_rate=1e-3, training_steps=100, activation_path="unused", precision="bf16", sparsity_lambda=0.0,
                        preactivation_coef=0.0, aux_loss_factor=0.0, optimizer="adamw")
    assert engine_supports(cfg, tc, model) is None
    eng = FusedBatchTopKEngine(model, tc, B)
    ref = _fp32_copy(model)
    snap = {n: p.detach().float().clone() for n, p in model.named_parameters()}
    X = torch.randn(L, B, d, device=dev).bfloat16()
    Y = torch.randn(L, B, d, device=dev).bfloat16()
    lr = 2e-2  # large enough to move a 16-bit scale near 1.0 by more than half an ulp
    out = eng.train_step(X, Y, 0, lr)
    torch.cuda.synchronize()
    eng.check_status()
    acts_k = eng.activations_dense()
    x = {l: X[l].float() for l in range(L)}
    pre = {l: torch.nn.functional.linear(x[l], ref.enc_weight[l], ref.enc_bias[l]) for l in range(L)}
    acts = {l: (pre[l] + (eng.preact[l].float() - pre[l]).detach()) * (acts_k[l] != 0) for l in range(L)}
    loss = sum(torch.nn.functional.mse_loss(ref.decode({s: acts[s] for s in range(t + 1)}, t), Y[t].float()) for t in range(L))
    loss.backward()
    assert abs(float(out.reconstruction) - float(loss)) < 3e-3 * float(loss), (float(out.reconstruction), float(loss))
    for name, mom in (("feature_offset", eng.foff_m), ("feature_scale", eng.fsc_m)):
        g_ref = dict(ref.named_parameters())[name].grad
        g = mom / 0.1  # first moment after one step = (1 - beta1) * gradient
        assert _rel_err(g, g_ref) < 0.03, (name, _rel_err(g, g_ref))
    assert _rel_err(eng.enc_m / 0.1, ref.enc_weight.grad) < 0.03
    for i, w in enumerate(ref.dec_weight):
        assert _rel_err(eng.dec_m[i] / 0.1, w.grad) < 0.03, i
    opt = torch.optim.AdamW(ref.parameters(), lr=lr)
    opt.step()
    for name in ("feature_offset", "feature_scale"):
        new = dict(model.named_parameters())[name].detach().float()
        want = dict(ref.named_parameters())[name].detach()
        moved = want.bfloat16().float() != snap[name]  # updates that survive the rounding to the storage type
        assert moved.float().mean().item() > 0.5
        agree = (torch.sign(new - snap[name])[moved] == torch.sign(want - snap[name])[moved]).float().mean().item()
        assert agree > 0.97, (name, agree)
    # the copies that the kernels read follow the stored parameters
    assert torch.equal(eng.foff32, model.feature_offset.data.float()) and torch.equal(eng.fsc32, model.feature_scale.data.float())
