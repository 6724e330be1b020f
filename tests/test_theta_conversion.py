import math

import torch

from crosslayer_coding_b200 import CLTConfig, CrossLayerTranscoder
from crosslayer_coding_b200.models.registry import get_activation_fn, register_activation_fn
import pytest


def _model(fn="batchtopk", **kw):
    cfg = CLTConfig(num_features=48, num_layers=2, d_model=8, activation_fn=fn, **kw)
    torch.manual_seed(0)
    return CrossLayerTranscoder(cfg)


def _batches(n=6, batch=64):
    g = torch.Generator().manual_seed(3)
    for _ in range(n):
        x = {l: torch.randn(batch, 8, generator=g) for l in range(2)}
        yield x, x


@pytest.mark.parametrize("fn,kw", [("batchtopk", {"batchtopk_k": 6}), ("topk", {"topk_k": 6})])
def test_estimate_theta_converts_model_and_roughly_preserves_l0(fn, kw):
    m = _model(fn, **kw)
    x = next(_batches(1, 256))[0]
    l0_before = sum(float((a != 0).float().sum(1).mean()) for a in m.get_feature_activations(x).values())
    theta = m.estimate_theta_posthoc(_batches(), num_batches=5)
    cfg = m.config
    assert cfg.activation_fn == "jumprelu" and cfg.batchtopk_k is None and cfg.jumprelu_threshold == 0.0
    assert theta.shape == (2, 48) and torch.isfinite(theta).all() and (theta > 0).all()
    assert torch.allclose(m.log_threshold.exp(), theta)
    acts = m.get_feature_activations(x)
    l0_after = sum(float((a != 0).float().sum(1).mean()) for a in acts.values())
    assert 0.3 * l0_before < l0_after < 3.0 * l0_before, (l0_before, l0_after)
    # encode() now goes through JumpReLU and matches get_feature_activations
    assert torch.equal(m.encode(x[1], 1), acts[1])


def test_theta_formula_from_accumulated_statistics():
    from crosslayer_coding_b200.models.theta import convert_to_jumprelu_inplace

    m = _model(batchtopk_k=4)
    L, F = 2, 48
    stats = {"sum_min": torch.zeros(L, F), "cnt_min": torch.zeros(L, F), "mean": torch.full((L, F), 0.5),
             "std": torch.full((L, F), 2.0), "batches": torch.ones(L)}
    stats["sum_min"][0, :10] = 3.0  # ten features selected twice with min z = 1.5 each
    stats["cnt_min"][0, :10] = 2.0
    m._theta_stats = stats
    convert_to_jumprelu_inplace(m)
    theta = m.log_threshold.exp()
    assert torch.allclose(theta[0], torch.full((F,), 1.5 * 2.0 + 0.5))      # theta_norm * std + mean
    assert torch.allclose(theta[1], torch.full((F,), 1e-5 * 2.0 + 0.5))     # fallback layer scalar 1e-5
    with pytest.raises(RuntimeError):
        convert_to_jumprelu_inplace(_model(batchtopk_k=4))


def test_registry():
    m = _model("relu")
    pre = torch.tensor([[-1.0, 2.0]])
    assert torch.equal(get_activation_fn("relu")(m, pre, 0), torch.tensor([[0.0, 2.0]]))
    for name in ("jumprelu", "batchtopk", "topk"):
        assert callable(get_activation_fn(name))
    with pytest.raises(ValueError):
        get_activation_fn("nope")
    with pytest.raises(ValueError):
        register_activation_fn("relu")(lambda m, p, l: p)


def test_l0_for_scales_matches_direct_count():
    from crosslayer_coding_b200.conversion import l0_for_scales

    torch.manual_seed(0)
    pre = torch.randn(200, 40)
    theta = torch.rand(40) * 0.5 + 0.1
    scales = torch.logspace(-1, 1, 33)
    got = l0_for_scales(pre, theta, scales)
    want = torch.stack([(pre >= s * theta).float().sum() / 200 for s in scales])
    assert torch.allclose(got, want, atol=1e-5)


def test_layerwise_calibration_matches_original_l0():
    from crosslayer_coding_b200.conversion import convert_model_to_jumprelu, layer_l0

    m = _model(batchtopk_k=8)
    calib = next(_batches(1, 512))[0]
    report, scales = convert_model_to_jumprelu(m, _batches(), num_batches=4, calibration_inputs=calib, l0_tolerance=0.25)
    assert m.config.activation_fn == "jumprelu" and set(scales) == {0, 1}
    after = layer_l0(m, calib)
    for l, tgt in report["l0_original"].items():
        assert abs(after[l] - tgt) <= 0.5, (l, after[l], tgt)
        assert abs(after[l] - tgt) <= abs(report["l0_converted"][l] - tgt) + 1e-6
