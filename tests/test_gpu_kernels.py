"""Numerics of every sm_100a kernel against a plain PyTorch fp32 restatement of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ext():
    from crosslayer_coding_b200.ops import ext as ext_mod

    return ext_mod.load()


def _dev():
    return torch.device("cuda:0")


@pytest.mark.parametrize(
    "L,M,N,K",
    [(1, 128, 256, 64), (2, 300, 520, 136), (1, 256, 512, 768), (3, 130, 8, 72), (1, 4096, 1024, 768)],
)
def test_encoder_gemm_matches_fp32(ext, L, M, N, K):
    torch.manual_seed(0)
    dev = _dev()
    x = torch.randn(L, M, K, device=dev).bfloat16()
    w = (torch.randn(L, N, K, device=dev) / math.sqrt(K)).bfloat16()
    b = torch.randn(L, N, device=dev).bfloat16()
    out = torch.full((L, M, N), float("nan"), device=dev, dtype=torch.bfloat16)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    tile_stats = torch.full((L, (M + 127) // 128, N, 2), float("nan"), device=dev)
    ext.encoder_gemm(x, w, b, out, status, tile_stats)
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    # the epilogue's per-block column sums give the batch statistics of the stored (rounded) outputs
    mean = torch.empty(L, N, device=dev)
    rstd = torch.empty(L, N, device=dev)
    ext.colstats_from_tiles(tile_stats, mean, rstd, M)
    of = out.float()
    assert torch.isfinite(tile_stats).all()
    assert torch.allclose(mean, of.mean(dim=1), atol=2e-4, rtol=1e-4)
    assert torch.allclose(rstd, 1.0 / (of.std(dim=1) + 1e-6), rtol=2e-3)
    ref = torch.einsum("lmk,lnk->lmn", x.float(), w.float()) + b.float()[:, None, :]
    err = (out.float() - ref).abs().max().item()
    assert torch.isfinite(out.float()).all()
    assert err < 0.03 * max(1.0, ref.abs().max().item()), err
    # bf16 rounding of an fp32 accumulation: relative error of a few 1e-3
    rel = ((out.float() - ref).norm() / ref.norm()).item()
    assert rel < 4e-3, rel


@pytest.mark.parametrize("L,B,F", [(3, 257, 72), (2, 1030, 256)])  # the second shape takes the row-split path
def test_colstats(ext, L, B, F):
    torch.manual_seed(1)
    dev = _dev()
    x = (torch.randn(L, B, F, device=dev) * 2 + 5).bfloat16()
    mean = torch.empty(L, F, device=dev)
    rstd = torch.empty(L, F, device=dev)
    ext.colstats(x, mean, rstd)
    xf = x.float()
    assert torch.allclose(mean, xf.mean(dim=1), atol=1e-4, rtol=1e-5)
    assert torch.allclose(rstd, 1.0 / (xf.std(dim=1) + 1e-6), rtol=1e-4)


def _run_select(ext, x, k_total, f_valid=None, feat_offset=0, full_F=None, full_range=False, cand_cap=None, key_range=None,
                sel_state=None, pool=None):
    dev = x.device
    L, B, Fl = x.shape
    f_valid = Fl if f_valid is None else f_valid
    full_F = Fl if full_F is None else full_F
    mean = torch.empty(L, Fl, device=dev)
    rstd = torch.empty(L, Fl, device=dev)
    ext.colstats(x, mean, rstd)
    hist = torch.zeros(2 * 8192 + 32, dtype=torch.int32, device=dev)
    ctl = torch.zeros(16, dtype=torch.int64, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    cap = max(k_total, 8)
    cc = cand_cap or x.numel()
    i32, f32 = torch.int32, torch.float32
    ent = [torch.empty(cap, dtype=i32, device=dev), torch.empty(cap, dtype=i32, device=dev), torch.empty(cap, dtype=f32, device=dev)]
    cand = [torch.empty(cc, dtype=i32, device=dev), torch.empty(cc, dtype=i32, device=dev), torch.empty(cc, dtype=i32, device=dev),
            torch.empty(cc, dtype=f32, device=dev)]
    key_lo, shift = (0, 19) if full_range else (0x80000000, 18)
    if key_range is not None:
        key_lo, shift = key_range
    ext.batchtopk_select(x, mean, rstd, f_valid, Fl, feat_offset, full_F, k_total, key_lo, shift, hist, ctl,
                         ent[0], ent[1], ent[2], cand[0], cand[1], cand[2], cand[3], status, 1, 0, [], [], 0, 0, sel_state, pool)
    torch.cuda.synchronize()
    return mean, rstd, ctl, status, ent


def _oracle_mask(x, mean, rstd, k_total, f_valid):
    """Top k_total of z = (x - mean) * rstd over [B, L*F] with lowest-flat-index tie-break."""
    L, B, Fl = x.shape
    z = (x.float() - mean[:, None, :]) * rstd[:, None, :]
    z = z[:, :, :f_valid]
    flat = z.permute(1, 0, 2).reshape(-1)  # token-major: b, l, f
    _, order = torch.sort(flat, descending=True, stable=True)
    mask = torch.zeros_like(flat, dtype=torch.bool)
    mask[order[:k_total]] = True
    return mask.view(B, L, f_valid).permute(1, 0, 2)


@pytest.mark.parametrize("full_range", [False, True])
@pytest.mark.parametrize("L,B,F,k", [(2, 64, 128, 5), (3, 200, 264, 17), (1, 33, 40, 3)])
def test_batchtopk_select_matches_oracle(ext, L, B, F, k, full_range):
    torch.manual_seed(2)
    dev = _dev()
    x = torch.randn(L, B, F, device=dev).bfloat16()
    k_total = k * B
    mean, rstd, ctl, status, ent = _run_select(ext, x, k_total, full_range=full_range)
    assert int(status[0]) == 0
    n = int(ctl[3])
    assert n == k_total
    got = torch.zeros(L, B, F, dtype=torch.bool, device=dev)
    col = ent[1][:n].long()
    got[col // F, ent[0][:n].long(), col % F] = True
    assert int(got.sum()) == n, "duplicate entries"
    want = _oracle_mask(x, mean, rstd, k_total, F)
    assert torch.equal(got, want)
    vals = x.float()[col // F, ent[0][:n].long(), col % F]
    assert torch.equal(vals, ent[2][:n])


def test_batchtopk_select_ties_use_lowest_flat_index(ext):
    dev = _dev()
    L, B, F = 2, 16, 64
    # two distinct values only: massive ties at the cut
    x = torch.zeros(L, B, F, device=dev)
    x[:, ::2, :] = 1.0
    x = x.bfloat16()
    k_total = 3 * B + 5
    mean, rstd, ctl, status, ent = _run_select(ext, x, k_total)
    assert int(status[0]) == 0
    n = int(ctl[3])
    assert n == k_total
    got = torch.zeros(L, B, F, dtype=torch.bool, device=dev)
    col = ent[1][:n].long()
    got[col // F, ent[0][:n].long(), col % F] = True
    want = _oracle_mask(x, mean, rstd, k_total, F)
    assert torch.equal(got, want)


def test_batchtopk_select_falls_back_when_guess_misses(ext):
    """A histogram range that starts above every key (z >= 50) must trigger the full-range pass."""
    import struct

    torch.manual_seed(4)
    dev = _dev()
    L, B, F = 2, 80, 96
    x = torch.randn(L, B, F, device=dev).bfloat16()
    k_total = 6 * B
    key_lo = struct.unpack("<I", struct.pack("<f", 50.0))[0] | 0x80000000
    shift = 0
    while ((0xFFFFFFFF - key_lo) >> shift) >= 8192:
        shift += 1
    mean, rstd, ctl, status, ent = _run_select(ext, x, k_total, key_range=(key_lo, shift))
    assert int(status[0]) == 0 and int(ctl[10]) == 1  # retry flag raised, no error
    n = int(ctl[3])
    assert n == k_total
    got = torch.zeros(L, B, F, dtype=torch.bool, device=dev)
    col = ent[1][:n].long()
    got[col // F, ent[0][:n].long(), col % F] = True
    assert torch.equal(got, _oracle_mask(x, mean, rstd, k_total, F))


def _selected_mask(ent, n, L, B, F, dev):
    got = torch.zeros(L, B, F, dtype=torch.bool, device=dev)
    col = ent[1][:n].long()
    got[col // F, ent[0][:n].long(), col % F] = True
    return got


def test_batchtopk_select_tracked_range_follows_the_cut(ext):
    """Tracked range + pool: the state starts far too high (first step falls back), then follows the data
    through a change of distribution; every step must equal the oracle."""
    import struct

    torch.manual_seed(11)
    dev = _dev()
    L, B, F = 3, 256, 512
    k_total = 9 * B
    key_lo = struct.unpack("<I", struct.pack("<f", 40.0))[0] | 0x80000000
    shift = 0
    while ((0xFFFFFFFF - key_lo) >> shift) >= 8192:
        shift += 1
    state = torch.tensor([key_lo, shift], dtype=torch.int64, device=dev)
    pool = torch.empty(4, 3 * k_total + 4096, dtype=torch.int32, device=dev)
    retries = []
    for step in range(6):
        x = torch.randn(L, B, F, device=dev)
        if step >= 3:  # heavier tails: the cut moves
            x = x * (1.0 + 2.0 * (torch.rand(L, B, F, device=dev) < 0.05).float())
        x = x.bfloat16()
        mean, rstd, ctl, status, ent = _run_select(ext, x, k_total, key_range=(key_lo, shift), sel_state=state, pool=pool)
        assert int(status[0]) == 0, f"status {status.tolist()} at step {step}"
        n = int(ctl[3])
        assert n == k_total
        assert torch.equal(_selected_mask(ent, n, L, B, F, dev), _oracle_mask(x, mean, rstd, k_total, F)), f"step {step}"
        retries.append(int(ctl[10]))
    assert retries[0] == 1, "first range was above every key: fallback expected"
    assert retries[1] == 0 and retries[2] == 0, f"range did not lock on: {retries}"
    assert retries[5] == 0, f"range did not recover after the distribution changed: {retries}"
    z_lo = struct.unpack("<f", struct.pack("<I", int(state[0]) & 0x7FFFFFFF))[0]
    assert 0.0 < z_lo < 6.0


def test_batchtopk_select_pool_overflow_falls_back(ext):
    """A pool that cannot hold the elements inside the range: the full-range pass must take over."""
    torch.manual_seed(12)
    dev = _dev()
    L, B, F = 2, 128, 256
    k_total = 8 * B
    state = torch.tensor([0x80000000, 18], dtype=torch.int64, device=dev)  # z >= 0: half of all elements
    pool = torch.empty(4, 64, dtype=torch.int32, device=dev)
    x = torch.randn(L, B, F, device=dev).bfloat16()
    mean, rstd, ctl, status, ent = _run_select(ext, x, k_total, sel_state=state, pool=pool)
    assert int(status[0]) == 0 and int(ctl[10]) == 1
    n = int(ctl[3])
    assert n == k_total
    assert torch.equal(_selected_mask(ent, n, L, B, F, dev), _oracle_mask(x, mean, rstd, k_total, F))
    assert int(state[0]) > 0x80000000  # the range moved up for the next step


def test_histogram_range_guess():
    from crosslayer_coding_b200.training.fused_engine import histogram_range

    key_lo, shift = histogram_range(200 * 4096, 4096 * 12 * 24576)
    assert key_lo > 0x80000000 and ((0xFFFFFFFF - key_lo) >> shift) < 8192
    assert histogram_range(10, 20) == (0, 19)


def test_batchtopk_select_respects_valid_columns(ext):
    torch.manual_seed(3)
    dev = _dev()
    L, B, Fl, Fv = 2, 48, 64, 52
    x = torch.randn(L, B, Fl, device=dev)
    x[:, :, Fv:] = 100.0  # padding columns must never be selected
    x = x.bfloat16()
    k_total = 4 * B
    mean, rstd, ctl, status, ent = _run_select(ext, x, k_total, f_valid=Fv, feat_offset=7, full_F=Fv + 7)
    n = int(ctl[3])
    assert n == k_total and int(status[0]) == 0
    col = ent[1][:n].long()
    assert int((col % Fl).max()) < Fv
    got = torch.zeros(L, B, Fv, dtype=torch.bool, device=dev)
    got[col // Fl, ent[0][:n].long(), col % Fl] = True
    assert torch.equal(got, _oracle_mask(x, mean, rstd, k_total, Fv))


def _engine_and_model(L=3, d=64, F=256, B=96, k=8, tying="none", seed=0, lr_cfg=None):
    from crosslayer_coding_b200 import CLTConfig, CrossLayerTranscoder, TrainingConfig
    from crosslayer_coding_b200.training.fused_engine import FusedBatchTopKEngine

    torch.manual_seed(seed)
    dev = _dev()
    cfg = CLTConfig(num_features=F, num_layers=L, d_model=d, activation_fn="batchtopk", batchtopk_k=k,
                    clt_dtype="bfloat16", decoder_tying=tying)
    model = CrossLayerTranscoder(cfg, device=dev)
    if tying != "none":
        with torch.no_grad():
            for w in model.dec_weight:
                w.uniform_(-0.05, 0.05)
    tc = TrainingConfig(learning_rate=1e-3, training_steps=100, activation_path="unused", precision="bf16",
                        sparsity_lambda=0.0, preactivation_coef=0.0, optimizer="adamw", **(lr_cfg or {}))
    eng = FusedBatchTopKEngine(model, tc, B)
    X = torch.randn(L, B, d, device=dev).bfloat16()
    Y = torch.randn(L, B, d, device=dev).bfloat16()
    return cfg, model, tc, eng, X, Y


@pytest.mark.parametrize("tying", ["none", "per_source", "per_target"])
def test_sparse_decode_and_loss_match_dense(tying):
    cfg, model, tc, eng, X, Y = _engine_and_model(tying=tying)
    yhat = eng.forward(X, Y)
    torch.cuda.synchronize()
    eng.check_status()
    acts = eng.activations_dense()  # [L, B, F]
    L = cfg.num_layers
    ref_model = _fp32_copy(model)
    a = {l: acts[l] for l in range(L)}
    for t in range(L):
        ref = ref_model.decode({s: a[s] for s in range(t + 1)}, t)
        assert torch.allclose(yhat[t], ref, atol=2e-3, rtol=2e-3), (t, (yhat[t] - ref).abs().max())
    # loss sums and gradient seed
    sq = torch.stack([((yhat[t] - Y[t].float()) ** 2).sum() for t in range(L)]).double()
    assert torch.allclose(eng.sq_err, sq, rtol=1e-3)
    assert torch.allclose(eng.gs.float(), (yhat - Y.float()), atol=2e-2, rtol=1e-2)
    # the selection itself equals the PyTorch model's BatchTopK on the same pre-activations
    want = _oracle_mask(eng.preact, eng.mean, eng.rstd, eng.k_total, cfg.num_features)
    assert torch.equal(acts != 0, want & (eng.preact.float() != 0))


def _fp32_copy(model):
    from crosslayer_coding_b200 import CLTConfig, CrossLayerTranscoder

    cfg = CLTConfig(**{**model.config.to_dict(), "clt_dtype": "float32"})
    ref = CrossLayerTranscoder(cfg, device=model.enc_weight.device)
    with torch.no_grad():
        ref.enc_weight.copy_(model.enc_weight.float())
        ref.enc_bias.copy_(model.enc_bias.float())
        for a, b in zip(ref.dec_weight, model.dec_weight):
            a.copy_(b.float())
        ref.dec_bias.copy_(model.dec_bias.float())
    return ref


@pytest.mark.parametrize("tying", ["none", "per_source", "per_target"])
@pytest.mark.parametrize("lam", [0.0, 0.05])
def test_fused_step_losses_match_autograd(tying, lam):
    """Loss terms reported by the fused step equal the dense PyTorch losses for the same selection."""
    cfg, model, tc, eng, X, Y = _engine_and_model(tying=tying, seed=5)
    ref = _fp32_copy(model)
    L, B, d = cfg.num_layers, eng.B, cfg.d_model
    out = eng.train_step(X, Y, step=0, lr=1e-3, sparsity_lambda=lam)
    torch.cuda.synchronize()
    eng.check_status()
    # reference step with the engine's own mask (the selection is tested elsewhere)
    mask = _oracle_mask(eng.preact, eng.mean, eng.rstd, eng.k_total, cfg.num_features)
    pre = {l: torch.nn.functional.linear(X[l].float(), ref.enc_weight[l], ref.enc_bias[l]) for l in range(L)}
    # the kernels see bf16-rounded pre-activations
    acts = {l: (pre[l] + (eng.preact[l].float() - pre[l]).detach()) * mask[l] for l in range(L)}
    recon = sum(torch.nn.functional.mse_loss(ref.decode({s: acts[s] for s in range(t + 1)}, t), Y[t].float()) for t in range(L))
    pen = torch.zeros((), device=X.device)
    if lam > 0:
        norms = ref.get_decoder_norms()
        pen = lam * sum(torch.tanh(tc.sparsity_c * acts[l] * norms[l][None, :]).sum() for l in range(L))
    assert abs(out.reconstruction.item() - recon.item()) < 2e-3 * max(1.0, abs(recon.item()))
    if lam > 0:
        assert abs(out.sparsity.item() - pen.item()) < 1e-2 * max(1.0, abs(pen.item()))


@pytest.mark.parametrize("tying", ["none", "per_source", "per_target"])
@pytest.mark.parametrize("lam", [0.0, 0.05])
def test_fused_step_weight_updates(tying, lam):
    cfg, model, tc, eng, X, Y = _engine_and_model(tying=tying, seed=7)
    ref = _fp32_copy(model)
    snap = {n: p.detach().float().clone() for n, p in model.named_parameters()}
    L = cfg.num_layers
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-3)
    eng.train_step(X, Y, step=0, lr=1e-3, sparsity_lambda=lam)
    torch.cuda.synchronize()
    eng.check_status()
    mask = _oracle_mask(eng.preact, eng.mean, eng.rstd, eng.k_total, cfg.num_features)
    pre = {l: torch.nn.functional.linear(X[l].float(), ref.enc_weight[l], ref.enc_bias[l]) for l in range(L)}
    acts = {l: (pre[l] + (eng.preact[l].float() - pre[l]).detach()) * mask[l] for l in range(L)}
    recon = sum(torch.nn.functional.mse_loss(ref.decode({s: acts[s] for s in range(t + 1)}, t), Y[t].float()) for t in range(L))
    if lam > 0:
        norms = ref.get_decoder_norms()
        recon = recon + lam * sum(torch.tanh(tc.sparsity_c * acts[l] * norms[l][None, :]).sum() for l in range(L))
    recon.backward()
    opt.step()
    ref_params = dict(ref.named_parameters())
    for name, p in model.named_parameters():
        old = snap[name]
        upd = p.detach().float() - old
        ref_upd = ref_params[name].detach() - old
        # Adam's first step moves every touched weight by ~lr; compare the sign/magnitude pattern
        tol = 0.008 * old.abs() + 3e-4
        bad = ((upd - ref_upd).abs() > tol).float().mean().item()
        assert bad < 2e-3, (name, bad, (upd - ref_upd).abs().max().item())
        touched = ref_upd.abs() > 5e-4
        if touched.any():
            agree = (torch.sign(upd[touched]) == torch.sign(ref_upd[touched])).float().mean().item()
            assert agree > 0.98, (name, agree)


def test_dead_counter_and_csr_consistency():
    cfg, model, tc, eng, X, Y = _engine_and_model(seed=9)
    eng.train_step(X, Y, step=0, lr=1e-3)
    torch.cuda.synchronize()
    n = int(eng.ctl[3])
    assert n == eng.k_total
    assert int(eng.tok_off[-1]) == n and int(eng.feat_off[-1]) == n
    acts = eng.activations_dense()
    fired = (acts > 1e-6).any(dim=1).reshape(-1)
    assert torch.equal(eng.dead_counter == 0, fired)
    # feature-major CSR lists tokens in increasing order per feature (sorted segments)
    off = eng.feat_off.cpu()
    tok = eng.fcsr_tok.cpu()
    for c in torch.nonzero(eng.feat_cnt.cpu() > 1).flatten()[:50].tolist():
        seg = tok[off[c]:off[c + 1]]
        assert torch.all(seg[1:] >= seg[:-1])


@pytest.mark.parametrize("L,d", [(16, 2048), (6, 1536), (5, 2048)])
def test_sparse_decode_wide_rows_take_the_bulk_ring(L, d):
    """d_model above 1024: two column chunks per thread and a ring of fewer, larger stages (64 KB per stage at 16 layers x 2048)."""
    cfg, model, tc, eng, X, Y = _engine_and_model(L=L, d=d, F=256, B=64, k=6, seed=5)
    yhat = eng.forward(X, Y)
    torch.cuda.synchronize()
    eng.check_status()
    acts = eng.activations_dense()
    ref_model = _fp32_copy(model)
    a = {l: acts[l] for l in range(L)}
    for t in range(L):
        ref = ref_model.decode({s: a[s] for s in range(t + 1)}, t)
        assert torch.allclose(yhat[t], ref, atol=3e-3, rtol=3e-3), (t, (yhat[t] - ref).abs().max())
    sq = torch.stack([((yhat[t] - Y[t].float()) ** 2).sum() for t in range(L)]).double()
    assert torch.allclose(eng.sq_err, sq, rtol=1e-3)


def test_decoder_norm2(ext):
    dev = _dev()
    w = torch.randn(40, 3, 64, device=dev).bfloat16()
    out = torch.empty(40, device=dev)
    ext.decoder_norm2(w, out)
    assert torch.allclose(out, w.float().pow(2).sum(dim=(1, 2)), rtol=1e-4)


def test_loss_decreases_over_steps():
    cfg, model, tc, eng, X, Y = _engine_and_model(L=2, d=64, F=512, B=128, k=16, seed=11)
    # learnable target: a fixed linear map of the inputs
    A = torch.randn(cfg.d_model, cfg.d_model, device=X.device) / math.sqrt(cfg.d_model)
    Y = (X.float() @ A).bfloat16()
    losses = []
    for step in range(60):
        out = eng.train_step(X, Y, step=step, lr=2e-3)
        losses.append(out.reconstruction.item())
    eng.check_status()
    assert losses[-1] < 0.7 * losses[0], losses[::10]


@pytest.mark.parametrize("tying", ["none", "per_source"])
def test_fused_step_with_preactivation_and_auxk_terms(tying):
    """The two dense side terms (pre-activation loss, AuxK on dead features) against the PyTorch LossManager."""
    from crosslayer_coding_b200.training.losses import LossManager

    cfg, model, tc, eng, X, Y = _engine_and_model(tying=tying, seed=13)
    tc.preactivation_coef = 0.05
    tc.aux_loss_factor = 0.5
    ref = _fp32_copy(model)
    snap = {n: p.detach().float().clone() for n, p in model.named_parameters()}
    L, F = cfg.num_layers, cfg.num_features
    dead = torch.zeros(L, F, dtype=torch.bool, device=X.device)
    dead[0, ::5] = True
    dead[2, 3:40] = True
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-3)
    out = eng.train_step(X, Y, step=0, lr=1e-3, preactivation_coef=0.05, aux_factor=0.5, dead_mask=dead)
    torch.cuda.synchronize()
    eng.check_status()
    mask = _oracle_mask(eng.preact, eng.mean, eng.rstd, eng.k_total, F)
    x = {l: X[l].float() for l in range(L)}
    y = {l: Y[l].float() for l in range(L)}
    pre = {l: torch.nn.functional.linear(x[l], ref.enc_weight[l], ref.enc_bias[l]) for l in range(L)}
    acts = {l: (pre[l] + (eng.preact[l].float() - pre[l]).detach()) * mask[l] for l in range(L)}
    preds = {t: ref.decode({s: acts[s] for s in range(t + 1)}, t) for t in range(L)}
    lm = LossManager(tc)
    recon = lm.compute_reconstruction_loss(preds, y)
    preact = lm.compute_preactivation_loss(ref, x, pre)
    aux = lm.compute_auxiliary_loss(ref, x, {l: y[l] - preds[l] for l in range(L)}, dead, preacts=pre)
    (recon + preact + aux).backward()
    opt.step()
    assert abs(out.reconstruction.item() - recon.item()) < 2e-3 * max(1.0, recon.item())
    assert abs(out.preactivation.item() - preact.item()) < 2e-2 * max(1e-3, preact.item())
    assert abs(out.auxiliary.item() - aux.item()) < 3e-2 * max(1e-3, aux.item()), (out.auxiliary.item(), aux.item())
    ref_params = dict(ref.named_parameters())
    for name, p in model.named_parameters():
        old = snap[name]
        upd = p.detach().float() - old
        ref_upd = ref_params[name].detach() - old
        bad = ((upd - ref_upd).abs() > 0.008 * old.abs() + 3e-4).float().mean().item()
        assert bad < 2e-2, (name, bad)
        touched = ref_upd.abs() > 5e-4
        agree = (torch.sign(upd[touched]) == torch.sign(ref_upd[touched])).float().mean().item()
        assert agree > 0.95, (name, agree)


@pytest.mark.parametrize("fn,tying", [("jumprelu", "none"), ("jumprelu", "per_source"), ("relu", "none"), ("batchtopk", "none")])
def test_sparse_forward_matches_dense_model(ext, fn, tying):
    """Inference path: encoder GEMM -> selection -> sparse decode against the dense PyTorch forward."""
    from crosslayer_coding_b200 import CLTConfig, CrossLayerTranscoder
    from crosslayer_coding_b200.models.sparse_forward import SparseForward, supports

    torch.manual_seed(3)
    dev = _dev()
    L, d, F, B = 3, 64, 256, 192
    kw = dict(num_features=F, num_layers=L, d_model=d, activation_fn=fn, decoder_tying=tying, clt_dtype="bfloat16")
    if fn == "batchtopk":
        kw["batchtopk_k"] = 12
    if tying != "none":
        kw.update(enable_feature_offset=True, enable_feature_scale=True)
    model = CrossLayerTranscoder(CLTConfig(**kw), device=dev)
    with torch.no_grad():
        for w in model.dec_weight:
            w.copy_(torch.randn_like(w) * 0.05)
        model.enc_bias.copy_(torch.randn_like(model.enc_bias) * 0.1 - (0.6 if fn == "relu" else 0.0))
        if model.log_threshold is not None:
            model.log_threshold.copy_(torch.log(torch.rand_like(model.log_threshold) * 0.4 + 0.5))
        if model.feature_offset is not None:
            model.feature_offset.copy_(torch.randn_like(model.feature_offset) * 0.1)
            model.feature_scale.copy_(1.0 + torch.randn_like(model.feature_scale) * 0.1)
    assert supports(model) is None
    X = (torch.randn(L, B, d, device=dev) * 0.7).bfloat16()
    Y = torch.randn(L, B, d, device=dev).bfloat16()
    sf = SparseForward(model, B)
    yhat = sf.reconstruct(X, Y)
    sf.check_status()
    inputs = {l: X[l] for l in range(L)}
    with torch.no_grad():
        acts = model.get_feature_activations(inputs)
        want = model(inputs)
    dense = torch.stack([acts[l].float() for l in range(L)])
    got_acts = sf.activations_dense()
    if fn != "batchtopk":
        # exact against the kernel's own pre-activations and thresholds ...
        theta = sf._theta()
        assert torch.equal(got_acts != 0, sf.preact.float() >= theta[:, None, :]), "selection differs from x >= theta"
        assert torch.equal(got_acts[got_acts != 0], sf.preact.float()[got_acts != 0])
        # ... and the same set as the dense model up to elements within bf16 rounding of their threshold
        mism = (got_acts != 0) != (dense != 0)
        gap = (sf.preact.float() - theta[:, None, :]).abs() / theta[:, None, :]
        assert mism.float().mean().item() < 1e-3 and (gap[mism] < 0.02).all(), "sets differ away from the thresholds"
    assert int((got_acts != 0).sum()) == sf.num_entries()
    # the decode, given the kernel's own active set (elements at their threshold may differ from the dense
    # model by bf16 rounding of the pre-activation, which would move the reconstruction by a whole feature)
    with torch.no_grad():
        own = {l: got_acts[l].to(torch.bfloat16) for l in range(L)}
        ref = torch.stack([model.decode(own, l).float() for l in range(L)])
    err = (yhat - ref).abs().max().item()
    assert err < 0.03 * max(1.0, ref.abs().max().item()), err
    full = torch.stack([want[l].float() for l in range(L)])
    assert ((yhat - full).norm() / full.norm()).item() < 0.35
    l0 = sf.l0_per_layer()
    assert torch.allclose(l0, (got_acts != 0).float().sum(dim=(1, 2)) / B)
    sq = ((yhat - Y.float()) ** 2).sum(dim=(1, 2)).double()
    assert torch.allclose(sf.sq_err, sq, rtol=2e-3)
    # contract of model.forward
    out = sf.forward_dict(inputs)
    assert set(out) == set(range(L)) and out[0].shape == (B, d)


@pytest.mark.parametrize("L,B,F,d", [(3, 256, 256, 64), (2, 200, 264, 72), (4, 384, 512, 128)])
def test_theta_grad_gemm_matches_dense(ext, L, B, F, d):
    """S1 = sum_b window * x * (gs . W rows over the target layers), S2 = sum_b window * x."""
    torch.manual_seed(5)
    dev = _dev()
    gs = (torch.randn(L, B, d, device=dev) * 0.1).bfloat16()
    ws = [(torch.randn(F, L - s, d, device=dev) * 0.2).bfloat16() for s in range(L)]
    x = (torch.randn(L, B, F, device=dev) * 0.6).bfloat16()
    theta = torch.rand(L, F, device=dev) * 0.5 + 0.05
    S1 = torch.zeros(L, F, device=dev)
    S2 = torch.zeros(L, F, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    ext.theta_grad_gemm(gs, ws, x, theta, 1.0, S1, S2, status)
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    for s in range(L):
        G = torch.zeros(B, F, device=dev)
        for r in range(L - s):
            G += gs[s + r].float() @ ws[s][:, r, :].float().t()
        xf = x[s].float()
        win = ((xf - theta[s][None, :]).abs() <= 0.5).float()
        want1 = (win * xf * G).sum(dim=0)
        want2 = (win * xf).sum(dim=0)
        assert torch.allclose(S2[s], want2, rtol=1e-4, atol=1e-3), (S2[s] - want2).abs().max()
        scale = want1.abs().max().item()
        assert (S1[s] - want1).abs().max().item() < 5e-3 * max(scale, 1.0), ((S1[s] - want1).abs().max().item(), scale)


@pytest.mark.parametrize("lam", [0.0, 0.05])
def test_fused_jumprelu_step_matches_autograd(lam):
    """Fused JumpReLU training step (threshold selection, sparse decode, threshold-gradient GEMM, fused AdamW)
    against autograd on an fp32 copy of the model fed with the kernel's own pre-activations."""
    from crosslayer_coding_b200 import CLTConfig, CrossLayerTranscoder, TrainingConfig
    from crosslayer_coding_b200.models import activations as act
    from crosslayer_coding_b200.training.fused_engine import FusedBatchTopKEngine

    torch.manual_seed(21)
    dev = _dev()
    L, d, F, B = 3, 64, 256, 128
    cfg = CLTConfig(num_features=F, num_layers=L, d_model=d, activation_fn="jumprelu", jumprelu_threshold=0.4, clt_dtype="bfloat16")
    model = CrossLayerTranscoder(cfg, device=dev)
    with torch.no_grad():
        model.log_threshold.copy_(torch.log(torch.rand_like(model.log_threshold.float()) * 0.5 + 0.3))
        for w in model.dec_weight:
            w.copy_(torch.randn_like(w) * 0.08)
    tc = TrainingConfig(learning_rate=1e-3, training_steps=100, activation_path="unused", precision="bf16",
                        sparsity_lambda=lam, sparsity_c=1.0, preactivation_coef=0.0, optimizer="adamw")
    eng = FusedBatchTopKEngine(model, tc, B)
    X = torch.randn(L, B, d, device=dev).bfloat16()
    Y = torch.randn(L, B, d, device=dev).bfloat16()
    ref = _fp32_copy(model)
    with torch.no_grad():
        ref.log_threshold.copy_(model.log_threshold.float())
    snap = {n: p.detach().float().clone() for n, p in model.named_parameters()}
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-3)
    out = eng.train_step(X, Y, step=0, lr=1e-3, sparsity_lambda=lam)
    torch.cuda.synchronize()
    eng.check_status()
    # autograd reference on the same pre-activation values (straight-through to the fp32 encoder)
    pre = {l: torch.nn.functional.linear(X[l].float(), ref.enc_weight[l], ref.enc_bias[l]) for l in range(L)}
    acts = {}
    for l in range(L):
        x = pre[l] + (eng.preact[l].float() - pre[l]).detach()
        acts[l] = act.JumpReLU.apply(x, ref.log_threshold[l].exp(), 1.0)
    loss = sum(torch.nn.functional.mse_loss(ref.decode({s: acts[s] for s in range(t + 1)}, t), Y[t].float()) for t in range(L))
    recon_ref = loss.item()
    pen_ref = 0.0
    if lam > 0:
        norms = ref.get_decoder_norms()
        pen = lam * sum(torch.tanh(tc.sparsity_c * acts[l] * norms[l][None, :]).sum() for l in range(L))
        pen_ref = pen.item()
        loss = loss + pen
    loss.backward()
    assert abs(out.reconstruction.item() - recon_ref) < 2e-3 * max(1.0, recon_ref)
    assert abs(out.sparsity.item() - pen_ref) < 2e-3 * max(1.0, pen_ref)
    # threshold gradient itself: recover it from the engine's window sums
    g_ref = ref.log_threshold.grad  # d loss / d log_threshold
    assert g_ref.abs().max().item() > 0
    g_err = (eng.grad_log_threshold - g_ref).abs().max().item()
    assert g_err < 0.02 * g_ref.abs().max().item() + 1e-6, (g_err, g_ref.abs().max().item())
    opt.step()
    ref_params = dict(ref.named_parameters())
    for name, p in model.named_parameters():
        old = snap[name]
        upd = p.detach().float() - old
        ref_upd = ref_params[name].detach() - old
        tol = 0.008 * old.abs() + 3e-4
        bad = ((upd - ref_upd).abs() > tol).float().mean().item()
        assert bad < 4e-3, (name, bad, (upd - ref_upd).abs().max().item())
        touched = ref_upd.abs() > 5e-4
        if touched.any() and "log_threshold" not in name:  # a 1e-3 step is below the bf16 spacing of log theta
            agree = (torch.sign(upd[touched]) == torch.sign(ref_upd[touched])).float().mean().item()
            assert agree > 0.97, (name, agree)


def test_fused_step_with_bf16_moments_tracks_fp32_moments():
    """optimizer_states_dtype='bfloat16': stochastically rounded bf16 moments; the run stays close to fp32 moments."""
    from crosslayer_coding_b200 import CLTConfig, CrossLayerTranscoder, TrainingConfig
    from crosslayer_coding_b200.training.fused_engine import FusedBatchTopKEngine

    dev = _dev()
    L, d, F, B, k = 2, 64, 512, 128, 16
    runs = {}
    for states in ("float32", "bfloat16"):
        torch.manual_seed(31)
        cfg = CLTConfig(num_features=F, num_layers=L, d_model=d, activation_fn="batchtopk", batchtopk_k=k, clt_dtype="bfloat16")
        model = CrossLayerTranscoder(cfg, device=dev)
        tc = TrainingConfig(learning_rate=2e-3, training_steps=100, activation_path="unused", precision="bf16", sparsity_lambda=0.0,
                            preactivation_coef=0.0, optimizer_states_dtype=states)
        eng = FusedBatchTopKEngine(model, tc, B)
        assert eng.dec_m[0].dtype == (torch.bfloat16 if states == "bfloat16" else torch.float32)
        g = torch.Generator(device="cpu").manual_seed(5)
        X = torch.randn(L, B, d, generator=g).bfloat16().to(dev)
        A = torch.randn(d, d, generator=g) / math.sqrt(d)
        Y = (X.float().cpu() @ A).bfloat16().to(dev)
        losses = [eng.train_step(X, Y, step=s, lr=2e-3).reconstruction.item() for s in range(40)]
        eng.check_status()
        runs[states] = (losses, model.dec_weight[0].detach().float().clone(), eng.dec_v[0].float().clone())
    lf, wf, vf = runs["float32"]
    lb, wb, vb = runs["bfloat16"]
    assert lb[-1] < 0.8 * lb[0], lb[::8]
    assert abs(lb[-1] - lf[-1]) < 0.05 * lf[-1], (lb[-1], lf[-1])
    # second moments agree on average (stochastic rounding is unbiased) although single entries differ
    touched = vf > 1e-12
    ratio = (vb[touched] / vf[touched]).mean().item()
    assert 0.9 < ratio < 1.1, ratio
    assert ((wb - wf).abs().mean() / wf.abs().mean()).item() < 0.05


def _token_topk_oracle(x, mean, rstd, k):
    """[L, B, F] -> bool mask of every token's k largest z-scores over all layers (ties: lowest column first)."""
    L, B, F = x.shape
    z = ((x.float() - mean[:, None, :]) * rstd[:, None, :]).permute(1, 0, 2).reshape(B, L * F)
    _, order = torch.sort(z, dim=-1, descending=True, stable=True)
    mask = torch.zeros_like(z, dtype=torch.bool)
    mask.scatter_(-1, order[:, :k], True)
    return mask.view(B, L, F).permute(1, 0, 2)


@pytest.mark.parametrize("L,B,F,k,ties", [(3, 50, 264, 7, False), (2, 33, 512, 40, False), (2, 20, 64, 9, True)])
def test_token_topk_select_matches_oracle(ext, L, B, F, k, ties):
    torch.manual_seed(8)
    dev = _dev()
    if ties:
        x = torch.zeros(L, B, F, device=dev)
        x[:, ::2, ::3] = 1.0   # few distinct values: the cut falls among exact ties
        x[:, 1::2, 1::4] = -0.5
        x = x.bfloat16()
    else:
        x = torch.randn(L, B, F, device=dev).bfloat16()
    mean = torch.empty(L, F, device=dev)
    rstd = torch.empty(L, F, device=dev)
    ext.colstats(x, mean, rstd)
    ctl = torch.zeros(16, dtype=torch.int64, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    ent = [torch.full((B * k,), -1, dtype=torch.int32, device=dev), torch.full((B * k,), -1, dtype=torch.int32, device=dev),
           torch.zeros(B * k, device=dev)]
    ext.token_topk_select(x, mean, rstd, F, k, ctl, ent[0], ent[1], ent[2], status)
    torch.cuda.synchronize()
    assert int(status[0]) == 0 and int(ctl[3]) == B * k
    tok, col = ent[0].long(), ent[1].long()
    assert (tok >= 0).all() and torch.equal(tok.view(B, k), torch.arange(B, device=dev)[:, None].expand(B, k))
    got = torch.zeros(L, B, F, dtype=torch.bool, device=dev)
    got[col // F, tok, col % F] = True
    assert int(got.sum()) == B * k, "duplicate entries"
    assert torch.equal(got, _token_topk_oracle(x, mean, rstd, k))
    assert torch.equal(ent[2], x.float()[col // F, tok, col % F])


def test_fused_token_topk_step_matches_autograd():
    from crosslayer_coding_b200 import CLTConfig, CrossLayerTranscoder, TrainingConfig
    from crosslayer_coding_b200.training.fused_engine import FusedBatchTopKEngine

    torch.manual_seed(41)
    dev = _dev()
    L, d, F, B, k = 3, 64, 256, 96, 12
    cfg = CLTConfig(num_features=F, num_layers=L, d_model=d, activation_fn="topk", topk_k=k, clt_dtype="bfloat16")
    model = CrossLayerTranscoder(cfg, device=dev)
    tc = TrainingConfig(learning_rate=1e-3, training_steps=100, activation_path="unused", precision="bf16", sparsity_lambda=0.0,
                        preactivation_coef=0.0, optimizer="adamw")
    eng = FusedBatchTopKEngine(model, tc, B)
    X = torch.randn(L, B, d, device=dev).bfloat16()
    Y = torch.randn(L, B, d, device=dev).bfloat16()
    ref = _fp32_copy(model)
    snap = {n: p.detach().float().clone() for n, p in model.named_parameters()}
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-3)
    out = eng.train_step(X, Y, step=0, lr=1e-3)
    torch.cuda.synchronize()
    eng.check_status()
    assert int(out.num_entries) == B * k
    mask = _token_topk_oracle(eng.preact, eng.mean, eng.rstd, k)
    assert torch.equal(eng.activations_dense() != 0, mask & (eng.preact.float() != 0))
    pre = {l: torch.nn.functional.linear(X[l].float(), ref.enc_weight[l], ref.enc_bias[l]) for l in range(L)}
    acts = {l: (pre[l] + (eng.preact[l].float() - pre[l]).detach()) * mask[l] for l in range(L)}
    loss = sum(torch.nn.functional.mse_loss(ref.decode({s: acts[s] for s in range(t + 1)}, t), Y[t].float()) for t in range(L))
    assert abs(out.reconstruction.item() - loss.item()) < 2e-3 * max(1.0, loss.item())
    loss.backward()
    opt.step()
    ref_params = dict(ref.named_parameters())
    for name, p in model.named_parameters():
        old = snap[name]
        upd, ref_upd = p.detach().float() - old, ref_params[name].detach() - old
        bad = ((upd - ref_upd).abs() > 0.008 * old.abs() + 3e-4).float().mean().item()
        assert bad < 2e-3, (name, bad)


@pytest.mark.parametrize("tying", ["none", "per_source"])
def test_fused_step_with_skip_connection(tying):
    """Skip connection inside the fused step: forward term through the loss epilogue, weight update from gs^T x."""
    from crosslayer_coding_b200 import CLTConfig, CrossLayerTranscoder, TrainingConfig
    from crosslayer_coding_b200.training.fused_engine import FusedBatchTopKEngine

    torch.manual_seed(51)
    dev = _dev()
    L, d, F, B, k = 3, 64, 256, 96, 8
    cfg = CLTConfig(num_features=F, num_layers=L, d_model=d, activation_fn="batchtopk", batchtopk_k=k, clt_dtype="bfloat16",
                    decoder_tying=tying, skip_connection=True)
    model = CrossLayerTranscoder(cfg, device=dev)
    with torch.no_grad():
        model.skip_weight.copy_(torch.randn_like(model.skip_weight) * 0.05)
        if tying != "none":
            for w in model.dec_weight:
                w.uniform_(-0.05, 0.05)
    tc = TrainingConfig(learning_rate=1e-3, training_steps=100, activation_path="unused", precision="bf16", sparsity_lambda=0.0,
                        preactivation_coef=0.0, optimizer="adamw")
    eng = FusedBatchTopKEngine(model, tc, B)
    X = torch.randn(L, B, d, device=dev).bfloat16()
    Y = torch.randn(L, B, d, device=dev).bfloat16()
    ref = _fp32_copy(model)
    with torch.no_grad():
        ref.skip_weight.copy_(model.skip_weight.float())
    snap = {n: p.detach().float().clone() for n, p in model.named_parameters()}
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-3)
    out = eng.train_step(X, Y, step=0, lr=1e-3)
    torch.cuda.synchronize()
    eng.check_status()
    mask = _oracle_mask(eng.preact, eng.mean, eng.rstd, eng.k_total, F)
    pre = {l: torch.nn.functional.linear(X[l].float(), ref.enc_weight[l], ref.enc_bias[l]) for l in range(L)}
    acts = {l: (pre[l] + (eng.preact[l].float() - pre[l]).detach()) * mask[l] for l in range(L)}
    src = {l: X[l].float() for l in range(L)}
    loss = sum(torch.nn.functional.mse_loss(ref.decode({s: acts[s] for s in range(t + 1)}, t, source_inputs=src), Y[t].float()) for t in range(L))
    assert abs(out.reconstruction.item() - loss.item()) < 3e-3 * max(1.0, loss.item()), (out.reconstruction.item(), loss.item())
    loss.backward()
    assert ref.skip_weight.grad.abs().max().item() > 0
    opt.step()
    ref_params = dict(ref.named_parameters())
    for name, p in model.named_parameters():
        old = snap[name]
        upd, ref_upd = p.detach().float() - old, ref_params[name].detach() - old
        bad = ((upd - ref_upd).abs() > 0.008 * old.abs() + 3e-4).float().mean().item()
        # Adam's first step is +-lr: an element whose gradient is ~0 may flip; allow a handful per tensor
        assert bad < max(3e-3, 4.0 / old.numel()), (name, bad, (upd - ref_upd).abs().max().item())


def test_evaluator_metrics_from_engine_match_dense_path():
    """Evaluation through the sparse forward gives the dense evaluator's numbers."""
    from crosslayer_coding_b200.training.evaluator import CLTEvaluator

    cfg, model, tc, eng, X, Y = _engine_and_model(L=3, d=64, F=256, B=96, k=8, seed=13)
    for s in range(3):
        eng.train_step(X, Y, step=s, lr=1e-3)
    fired = eng.fired.clone()
    ev = CLTEvaluator(model, X.device, None, normalization_method="none", d_model=cfg.d_model)
    dead = torch.zeros(3, 256, dtype=torch.bool, device=X.device)
    dead[1, :5] = True
    got = ev.compute_metrics_from_engine(eng, X, Y, dead_neuron_mask=dead)
    assert torch.equal(eng.fired, fired)
    with torch.autocast(device_type="cuda", dtype=torch.bfloat16):
        want = ev.compute_metrics({l: X[l] for l in range(3)}, {l: Y[l] for l in range(3)}, dead_neuron_mask=dead)
    assert got["sparsity/total_l0"] == pytest.approx(8.0) and want["sparsity/total_l0"] == pytest.approx(8.0, abs=0.05)
    for key in ("reconstruction/normalized_mean_reconstruction_error", "reconstruction/explained_variance"):
        assert got[key] == pytest.approx(want[key], rel=0.02, abs=0.01), key
    assert got["dead_features/total_eval"] == want["dead_features/total_eval"] == 5
    gd = torch.tensor(got["layerwise/log_feature_density"]["layer_0"])
    wd = torch.tensor(want["layerwise/log_feature_density"]["layer_0"])
    assert ((gd - wd).abs() > 1e-4).float().mean().item() < 0.05  # selections differ only by bf16 ties of the dense path
    assert set(got["layerwise/preactivation_std_dev"]) == {"layer_0", "layer_1", "layer_2"}


@pytest.mark.parametrize("fn", ["batchtopk", "topk"])
def test_theta_estimation_through_the_sparse_forward_matches_dense(fn):
    """BatchTopK / TopK -> JumpReLU threshold statistics from the entry list against the dense accumulation."""
    import copy

    from crosslayer_coding_b200 import CLTConfig, CrossLayerTranscoder
    from crosslayer_coding_b200.models import theta as theta_mod
    from crosslayer_coding_b200.models.sparse_forward import SparseForward

    torch.manual_seed(61)
    dev = _dev()
    L, d, F, B = 3, 64, 256, 128
    cfg = CLTConfig(num_features=F, num_layers=L, d_model=d, activation_fn=fn, batchtopk_k=10, topk_k=10, clt_dtype="bfloat16")
    model = CrossLayerTranscoder(cfg, device=dev)
    batches = [torch.randn(L, B, d, device=dev).bfloat16() for _ in range(4)]
    dense_stats = theta_mod._new_stats(model)
    sparse_stats = theta_mod._new_stats(model)
    sf = SparseForward(model, B)
    for X in batches:
        theta_mod.accumulate_theta_batch(model, {l: X[l] for l in range(L)}, dense_stats)
        theta_mod.accumulate_theta_batch_sparse(sf, X, sparse_stats)
    sf.check_status()
    assert torch.allclose(sparse_stats["mean"], dense_stats["mean"], atol=2e-3)
    assert torch.allclose(sparse_stats["std"], dense_stats["std"], rtol=2e-2, atol=1e-3)
    # the selections agree except for bf16 near-ties: compare the per-feature statistic where both paths saw the feature
    both = (sparse_stats["cnt_min"] > 0) & (dense_stats["cnt_min"] > 0)
    assert both.float().mean().item() > 0.3
    assert ((sparse_stats["cnt_min"] != dense_stats["cnt_min"]).float().mean().item()) < 0.02
    a = sparse_stats["sum_min"][both] / sparse_stats["cnt_min"][both]
    b = dense_stats["sum_min"][both] / dense_stats["cnt_min"][both]
    assert ((a - b).abs() > 0.02 * b.abs() + 0.02).float().mean().item() < 0.02
    # and the public entry point takes the sparse path on its own
    m2 = copy.deepcopy(model)
    th = theta_mod.estimate_theta_posthoc(m2, iter([({l: X[l] for l in range(L)}, None) for X in batches]), num_batches=4)
    assert m2.config.activation_fn == "jumprelu" and torch.isfinite(th).all() and (th > 0).all()


def test_strided_copy_places_a_row_range(ext):
    """The staging copy: rows [r0, r0 + n) of every outer index, pinned host -> device and device -> device."""
    dev = _dev()
    outer, rows, inner, r0, n = 6, 32, 40, 8, 8
    host = torch.randn(outer, rows, inner).bfloat16().pin_memory()
    a = torch.zeros(outer, rows, inner, dtype=torch.bfloat16, device=dev)
    b = torch.zeros_like(a)
    es = host.element_size()
    pitch, width, off = rows * inner * es, n * inner * es, r0 * inner * es
    ext.memcpy_2d(a.data_ptr() + off, pitch, host.data_ptr() + off, pitch, width, outer)
    ext.memcpy_2d(b.data_ptr() + off, pitch, a.data_ptr() + off, pitch, width, outer)
    torch.cuda.synchronize()
    want = torch.zeros_like(host)
    want[:, r0:r0 + n] = host[:, r0:r0 + n]
    assert torch.equal(a.cpu(), want) and torch.equal(b.cpu(), want)
    with pytest.raises(RuntimeError):
        ext.memcpy_2d(a.data_ptr(), 8, host.data_ptr(), 8, 16, 1)  # pitch below the width
