"""Glue between a model description and the oracle (test infrastructure only).

``spec`` is any object with the attributes of ``megabake_b200.models.ModelSpec``; this module
does not import the product package.
"""

from __future__ import annotations

import torch

from .decoder_oracle import OracleConfig, OracleWeights


def oracle_config(spec) -> OracleConfig:
    return OracleConfig(
        hidden=spec.hidden, layers=spec.layers, heads=spec.heads, kv_heads=spec.kv_heads,
        head_dim=spec.head_dim, intermediate=spec.intermediate, vocab=spec.vocab, eps=spec.eps,
        norm=spec.norm, activation=spec.activation, embed_scale=spec.embed_scale,
        rope_scale=1.0, qkv_bias=spec.qkv_bias, query_rescale=None,
    )


def oracle_weights(weights: dict[str, torch.Tensor], inv_freq: torch.Tensor) -> OracleWeights:
    cpu = {name: tensor.detach().to("cpu") for name, tensor in weights.items()}
    return OracleWeights(cpu, inv_freq.detach().to("cpu"), tied="lm_head.weight" not in cpu)
