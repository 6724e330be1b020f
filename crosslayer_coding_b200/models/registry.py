"""Name -> per-layer activation callable ``(model, preact, layer_idx) -> activated``.

Mirrors the reference registry (clt/activations/registry.py:15-108).  Unlike the
reference, the model really dispatches through the per-layer (batch)topk entries
when ``topk_mode="per_layer"`` (the reference returns zeros there).
"""
from __future__ import annotations

from typing import Callable, Dict

import torch

from . import activations as act

ActivationCallable = Callable[["object", torch.Tensor, int], torch.Tensor]
ACTIVATION_REGISTRY: Dict[str, ActivationCallable] = {}


def register_activation_fn(name: str) -> Callable[[ActivationCallable], ActivationCallable]:
    def decorator(fn: ActivationCallable) -> ActivationCallable:
        if name in ACTIVATION_REGISTRY:
            raise ValueError(f"Activation function '{name}' already registered.")
        ACTIVATION_REGISTRY[name] = fn
        return fn

    return decorator


def get_activation_fn(name: str) -> ActivationCallable:
    try:
        return ACTIVATION_REGISTRY[name]
    except KeyError as exc:
        raise ValueError(f"Activation function '{name}' not registered. Available: {list(ACTIVATION_REGISTRY)}") from exc


@register_activation_fn("relu")
def relu_activation(model, preact: torch.Tensor, layer_idx: int) -> torch.Tensor:
    return torch.relu(preact)


@register_activation_fn("jumprelu")
def jumprelu_activation(model, preact: torch.Tensor, layer_idx: int) -> torch.Tensor:
    return model.jumprelu(preact, layer_idx)


@register_activation_fn("batchtopk")
def batchtopk_per_layer_activation(model, preact: torch.Tensor, layer_idx: int) -> torch.Tensor:
    k = model.config.batchtopk_k
    if k is None:
        return preact
    return act.BatchTopK.apply(preact, int(k), model.config.batchtopk_straight_through, preact)


@register_activation_fn("topk")
def topk_per_layer_activation(model, preact: torch.Tensor, layer_idx: int) -> torch.Tensor:
    k = model.config.topk_k
    if k is None:
        return preact
    return act.TokenTopK.apply(preact, float(k), model.config.topk_straight_through, preact)
