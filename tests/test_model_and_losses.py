import math

import pytest
import torch

from crosslayer_coding_b200 import CLTConfig, CrossLayerTranscoder, TrainingConfig
from crosslayer_coding_b200.models.clt import pair_index
from crosslayer_coding_b200.training.losses import LossManager, sparsity_lambda_at


def _cfg(**kw):
    base = dict(num_features=32, num_layers=3, d_model=8, activation_fn="relu")
    base.update(kw)
    return CLTConfig(**base)


def _inputs(cfg, batch=6, seed=0):
    g = torch.Generator().manual_seed(seed)
    return {l: torch.randn(batch, cfg.d_model, generator=g) for l in range(cfg.num_layers)}


def test_shapes_and_3d_inputs():
    cfg = _cfg()
    m = CrossLayerTranscoder(cfg)
    x3 = {l: torch.randn(2, 5, cfg.d_model) for l in range(cfg.num_layers)}
    out = m(x3)
    assert set(out) == {0, 1, 2} and out[1].shape == (10, cfg.d_model)
    acts = m.get_feature_activations(x3)
    assert acts[0].shape == (10, cfg.num_features)
    assert m.get_preactivations(x3[0], 0).shape == (10, cfg.num_features)


def test_wrong_input_width_gives_zero_preactivations(caplog):
    m = CrossLayerTranscoder(_cfg())
    out = m.get_preactivations(torch.randn(4, 5), 0)
    assert out.shape == (4, 32) and float(out.abs().sum()) == 0.0


def test_init_bounds_and_tied_zero_init():
    cfg = _cfg()
    m = CrossLayerTranscoder(cfg)
    assert float(m.enc_weight.abs().max()) <= 1 / math.sqrt(cfg.num_features) + 1e-6
    assert float(m.dec_weight[0].abs().max()) <= 1 / math.sqrt(cfg.num_layers * cfg.d_model) + 1e-6
    assert float(m.enc_bias.abs().sum()) == 0 and float(m.dec_bias.abs().sum()) == 0
    t = CrossLayerTranscoder(_cfg(decoder_tying="per_source", enable_feature_offset=True, enable_feature_scale=True, skip_connection=True))
    assert all(float(w.abs().sum()) == 0 for w in t.dec_weight)
    assert float(t.feature_offset.abs().sum()) == 0
    assert torch.all(t.feature_scale[0] == 1) and torch.all(t.feature_scale[1:] == 0.1)
    assert float(t.skip_weight.abs().sum()) == 0 and t.skip_weight.shape == (3, 8, 8)


def test_untied_decode_matches_manual_sum():
    cfg = _cfg()
    m = CrossLayerTranscoder(cfg)
    with torch.no_grad():
        m.dec_bias.normal_()
    a = {l: torch.relu(torch.randn(5, cfg.num_features)) for l in range(3)}
    for t in range(3):
        want = torch.zeros(5, cfg.d_model)
        for s in range(t + 1):
            want = want + a[s] @ m.dec_weight[s][:, t - s, :] + m.dec_bias[pair_index(s, t, 3)]
        assert torch.allclose(m.decode({s: a[s] for s in range(t + 1)}, t), want, atol=1e-6)


@pytest.mark.parametrize("tying", ["per_source", "per_target"])
def test_tied_decode_with_affine_and_skip(tying):
    cfg = _cfg(decoder_tying=tying, enable_feature_offset=True, enable_feature_scale=True, skip_connection=True)
    m = CrossLayerTranscoder(cfg)
    with torch.no_grad():
        for w in m.dec_weight:
            w.normal_(std=0.1)
        m.feature_offset.normal_(std=0.1)
        m.feature_scale.uniform_(0.5, 1.5)
        m.skip_weight.normal_(std=0.1)
        m.dec_bias.normal_()
    a = {l: torch.relu(torch.randn(4, cfg.num_features)) for l in range(3)}
    x = _inputs(cfg, 4)
    t = 2

    def aff(v):
        nz = (v != 0).float()
        return torch.where(v != 0, (v + m.feature_offset[t] * nz) * m.feature_scale[t], v)

    if tying == "per_target":
        want = sum(aff(a[s]) for s in range(t + 1)) @ m.dec_weight[t][:, 0, :] + m.dec_bias[t]
    else:
        want = sum(aff(a[s]) @ m.dec_weight[s][:, 0, :] + m.dec_bias[s] for s in range(t + 1))
    want = want + x[t] @ m.skip_weight[t].T
    got = m.decode({s: a[s] for s in range(t + 1)}, t, source_inputs=x)
    assert torch.allclose(got, want, atol=1e-5)


def test_decoder_norms_definition_and_cache():
    m = CrossLayerTranscoder(_cfg())
    n = m.get_decoder_norms()
    assert n.shape == (3, 32)
    want0 = m.dec_weight[0].float().pow(2).sum(dim=(1, 2)).sqrt()
    assert torch.allclose(n[0], want0, atol=1e-6)
    assert m.get_decoder_norms() is n
    m.invalidate_decoder_norms()
    assert m.get_decoder_norms() is not n
    pt = CrossLayerTranscoder(_cfg(decoder_tying="per_target"))
    with torch.no_grad():
        for w in pt.dec_weight:
            w.normal_()
    n = pt.get_decoder_norms()
    want = sum(pt.dec_weight[t].float().pow(2).sum(dim=(1, 2)) for t in range(1, 3)).sqrt()
    assert torch.allclose(n[1], want, atol=1e-5)


def test_state_dict_uses_reference_keys_and_roundtrips():
    cfg = _cfg(activation_fn="jumprelu", skip_connection=True)
    m = CrossLayerTranscoder(cfg)
    sd = m.state_dict()
    assert sd["encoder_module.encoders.1.weight"].shape == (32, 8)
    assert sd["encoder_module.encoders.1.bias_param"].shape == (32,)
    assert sd["decoder_module.decoders.0->2.weight"].shape == (8, 32)
    assert sd["decoder_module.decoders.1->1.bias_param"].shape == (8,)
    assert sd["decoder_module.skip_weights.0->1"].shape == (8, 8)
    assert sd["theta_manager.log_threshold"].shape == (3, 32)
    m2 = CrossLayerTranscoder(cfg)
    m2.load_state_dict(sd)
    x = _inputs(cfg)
    assert all(torch.allclose(m(x)[l], m2(x)[l]) for l in range(3))
    with pytest.raises(RuntimeError):
        m2.load_state_dict({k: v for k, v in sd.items() if "encoders.0.weight" not in k})


def test_untied_checkpoint_loads_into_per_source_model():
    src = CrossLayerTranscoder(_cfg())
    tied = CrossLayerTranscoder(_cfg(decoder_tying="per_source"))
    tied.load_state_dict(src.state_dict(), strict=False)
    assert torch.allclose(tied.dec_weight[1][:, 0, :], src.dec_weight[1][:, 0, :])


def test_legacy_feature_affine_keys_migrate():
    cfg = _cfg(decoder_tying="per_source", enable_feature_offset=True)
    m = CrossLayerTranscoder(cfg)
    sd = dict(m.state_dict())
    for i in range(3):
        sd[f"encoder_module.feature_offset.{i}"] = sd.pop(f"decoder_module.feature_offset.{i}") + 1.0
    m.load_state_dict(sd)
    assert torch.allclose(m.feature_offset, torch.ones_like(m.feature_offset))


def test_per_layer_topk_mode_is_a_real_selection():
    cfg = _cfg(activation_fn="batchtopk", batchtopk_k=4, topk_mode="per_layer")
    m = CrossLayerTranscoder(cfg)
    acts = m.get_feature_activations(_inputs(cfg, 6))
    assert all(int((a != 0).sum()) == 4 * 6 for a in acts.values())
    enc = m.encode(_inputs(cfg, 6)[1], 1)
    assert int((enc != 0).sum()) == 24


def test_save_load_roundtrip(tmp_path):
    cfg = _cfg(activation_fn="batchtopk", batchtopk_k=3)
    m = CrossLayerTranscoder(cfg)
    p = str(tmp_path / "m.pt")
    m.save(p)
    m2 = CrossLayerTranscoder.load(p)
    x = _inputs(cfg)
    assert all(torch.allclose(m(x)[l], m2(x)[l]) for l in range(3))


# ------------------------------------------------------------------------------------------- losses
def _tc(**kw):
    base = dict(learning_rate=1e-3, training_steps=100, activation_path="x", normalization_method="none")
    base.update(kw)
    return TrainingConfig(**base)


def test_lambda_schedules():
    tc = _tc(sparsity_lambda=2.0)
    assert sparsity_lambda_at(tc, 0, 100) == 0.0 and sparsity_lambda_at(tc, 50, 100) == 1.0
    assert sparsity_lambda_at(tc, 200, 100) == 2.0
    td = _tc(sparsity_lambda=2.0, sparsity_lambda_schedule="delayed_linear", sparsity_lambda_delay_frac=0.5)
    assert sparsity_lambda_at(td, 49, 100) == 0.0 and sparsity_lambda_at(td, 75, 100) == 1.0


def test_reconstruction_loss_denormalises():
    tc = _tc(normalization_method="mean_std")
    mean = {0: torch.full((1, 4), 2.0)}
    std = {0: torch.full((1, 4), 3.0)}
    lm = LossManager(tc, mean_tg=mean, std_tg=std)
    pred, tgt = {0: torch.zeros(5, 4)}, {0: torch.ones(5, 4)}
    assert torch.isclose(lm.compute_reconstruction_loss(pred, tgt), torch.tensor(9.0))
    lm2 = LossManager(_tc(normalization_method="sqrt_d_model"), clt_config=_cfg(d_model=4))
    assert torch.isclose(lm2.compute_reconstruction_loss(pred, tgt), torch.tensor(0.25))


def test_sparsity_penalty_closed_form_and_batchtopk_switch():
    cfg = _cfg()
    m = CrossLayerTranscoder(cfg)
    tc = _tc(sparsity_lambda=0.5, sparsity_c=2.0)
    lm = LossManager(tc)
    acts = {l: torch.rand(4, cfg.num_features) for l in range(3)}
    pen, lam = lm.compute_sparsity_penalty(m, acts, 50, 100)
    norms = m.get_decoder_norms()
    want = 0.25 * sum(torch.tanh(2.0 * acts[l] * norms[l][None]).sum() for l in range(3))
    assert lam == 0.25 and torch.isclose(pen, want, rtol=1e-5)
    mb = CrossLayerTranscoder(_cfg(activation_fn="batchtopk", batchtopk_k=2))
    off = LossManager(_tc(sparsity_lambda=0.5, apply_sparsity_penalty_to_batchtopk=False))
    assert float(off.compute_sparsity_penalty(mb, acts, 50, 100)[0]) == 0.0


def test_preactivation_loss_mean_of_negative_part():
    cfg = _cfg()
    m = CrossLayerTranscoder(cfg)
    lm = LossManager(_tc(preactivation_coef=2.0))
    x = _inputs(cfg)
    pre = torch.cat([m.get_preactivations(x[l], l) for l in range(3)])
    want = 2.0 * torch.relu(-pre).sum() / pre.numel()
    assert torch.isclose(lm.compute_preactivation_loss(m, x), want, rtol=1e-5)
    assert float(LossManager(_tc(preactivation_coef=0.0)).compute_preactivation_loss(m, x)) == 0.0


def test_aux_loss_only_with_dead_features_and_has_grad():
    cfg = _cfg(activation_fn="batchtopk", batchtopk_k=3)
    m = CrossLayerTranscoder(cfg)
    lm = LossManager(_tc(aux_loss_factor=0.5, sparsity_lambda=0.0, preactivation_coef=0.0))
    x, y = _inputs(cfg, 8, 1), _inputs(cfg, 8, 2)
    dead = torch.zeros(3, 32, dtype=torch.bool)
    loss, parts = lm.compute_total_loss(m, x, y, 0, 10, dead_neuron_mask=dead)
    assert parts["auxiliary"] == 0.0
    dead[1, :10] = True
    loss, parts = lm.compute_total_loss(m, x, y, 0, 10, dead_neuron_mask=dead)
    assert parts["auxiliary"] > 0 and abs(parts["total"] - parts["reconstruction"] - parts["auxiliary"]) < 1e-5
    loss.backward()
    assert float(m.enc_weight.grad[1, :10].abs().sum()) > 0


def test_total_loss_components_sum():
    cfg = _cfg(activation_fn="jumprelu")
    m = CrossLayerTranscoder(cfg)
    lm = LossManager(_tc(sparsity_lambda=0.1))
    loss, parts = lm.compute_total_loss(m, _inputs(cfg), _inputs(cfg, seed=3), 50, 100)
    s = parts["reconstruction"] + parts["sparsity"] + parts["preactivation"] + parts["auxiliary"]
    assert abs(parts["total"] - s) < 1e-5 and abs(float(loss) - s) < 1e-4
    loss.backward()
    assert m.log_threshold.grad is not None
