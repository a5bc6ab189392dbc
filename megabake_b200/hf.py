"""Hugging Face glue: the ``megabake`` attention implementation and the decode
wrappers that give a causal LM the explicit-state calling convention.

Calling convention (reference ``src/megabake/fx_handler/hf_attention.py:168-207``):
``forward(input_ids[B,1] int64, position_ids[B,1] int64, *state) -> logits[B,1,V]``
with ``state`` holding, per layer and in this order, a key cache and a value cache
of shape ``[B, capacity, kv_heads, head_dim]`` and one int32 ``[1]`` valid length
shared by the batch.  ``megabake::kv_attention`` appends to the caches and bumps the
length, so after a call the state tensors already describe the next step.

Two wrappers produce that convention:

``DecodeStep``       runs the model's own ``forward`` with a pass-through cache and
                     routes every attention module to ``megabake::kv_attention``
                     through transformers' ``AttentionInterface`` (any attention
                     model; same class name and semantics as the reference).
``StatefulDecoder``  walks embed -> layers -> norm -> head itself for the plain
                     pre-norm decoder families (Llama, Qwen2, Gemma, ...); the
                     counterpart of the reference's benchmark wrapper
                     ``benchmarks/stateful_models.py:152-187``, restricted to
                     attention layers, and batch-aware in ``state_shapes``.
``GroupedStateDecoder`` the same step with the state in the order of the reference's Llama
                     wrapper (``tests/fixtures.py:236-238``): all key caches, then all value
                     caches, then all valid lengths.

``megabake_attention_forward``, ``megabake_decode_attention``,
``register_transformers_attention`` and ``_PassThroughLayer`` below restate the reference's
``src/megabake/fx_handler/hf_attention.py:28-162`` closely -- same branches, same error texts:
they are the operator boundary a model written against the reference binds to, and their
signatures are dictated by ``transformers``' ``AttentionInterface`` and cache protocol.
"""

from __future__ import annotations

import sys
from typing import Any

import torch
from transformers.cache_utils import Cache, CacheLayerMixin

from . import ops as _ops  # noqa: F401  (registers torch.ops.megabake.*)
from .ops import attention as _attention_op

ATTENTION_IMPLEMENTATION = "megabake"


def megabake_attention_forward(
    module: torch.nn.Module,
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    attention_mask: torch.Tensor | None,
    dropout: float = 0.0,
    scaling: float | None = None,
    softcap: float | None = None,
    **kwargs: Any,
) -> tuple[torch.Tensor, None]:
    """``AttentionInterface`` entry for prefill: ``query`` ``[B, H, T, D]``,
    ``key``/``value`` ``[B, Hkv, S, D]``; returns ``[B, T, H, D]``."""
    unsupported = (
        (dropout and module.training)
        or softcap is not None
        or kwargs.get("s_aux") is not None
        or kwargs.get("output_attentions")
    )
    if unsupported:
        eager = sys.modules[type(module).__module__].eager_attention_forward
        return eager(
            module, query, key, value, attention_mask,
            dropout=dropout, scaling=scaling, softcap=softcap, **kwargs,
        )
    batch, heads, length, dim = query.shape
    scale = dim**-0.5 if scaling is None else scaling
    mask = attention_mask
    if mask is not None:
        mask = mask[:, :, :, : key.shape[-2]]
    mixed = _attention_op(
        query.transpose(1, 2), key.transpose(1, 2), value.transpose(1, 2), mask, float(scale)
    )
    return mixed.view(batch, heads, length, dim).transpose(1, 2).contiguous(), None


def megabake_decode_attention(
    module: torch.nn.Module,
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    attention_mask: torch.Tensor | None,
    dropout: float = 0.0,
    scaling: float | None = None,
    softcap: float | None = None,
    megabake_state: tuple[tuple[torch.Tensor, ...], ...] | None = None,
    **kwargs: Any,
) -> tuple[torch.Tensor, None]:
    """One-token decode on the layer's own ``(key_cache, value_cache, length)``
    triple; without ``megabake_state`` it is the prefill entry above."""
    if megabake_state is None:
        return megabake_attention_forward(
            module, query, key, value, attention_mask,
            dropout=dropout, scaling=scaling, softcap=softcap, **kwargs,
        )
    if softcap is not None or kwargs.get("s_aux") is not None:
        raise NotImplementedError("decode attention with soft cap or sinks is not declared")
    key_cache, value_cache, valid_length = megabake_state[module.layer_idx]
    window = getattr(module, "sliding_window", None)
    if window is not None and key_cache.shape[1] > window:
        raise NotImplementedError(
            f"cache capacity {key_cache.shape[1]} exceeds the {window}-token sliding window"
        )
    batch, heads, length, dim = query.shape
    if scaling is not None and abs(scaling * dim**0.5 - 1.0) > 1e-6:
        query = query * (scaling * dim**0.5)  # the op always scales by dim ** -0.5
    mixed = torch.ops.megabake.kv_attention(
        query.transpose(1, 2), key.transpose(1, 2), value.transpose(1, 2),
        key_cache, value_cache, valid_length,
    )
    return mixed.view(batch, heads, length, dim).transpose(1, 2).contiguous(), None


def register_transformers_attention() -> str:
    """Register attention + mask functions under the name ``"megabake"``."""
    from transformers import AttentionInterface
    from transformers.masking_utils import AttentionMaskInterface, eager_mask

    AttentionInterface.register(ATTENTION_IMPLEMENTATION, megabake_decode_attention)
    AttentionMaskInterface.register(ATTENTION_IMPLEMENTATION, eager_mask)
    return ATTENTION_IMPLEMENTATION


class _PassThroughLayer(CacheLayerMixin):
    """Stores nothing: the new key/value go straight to the attention call, which owns the
    real cache."""

    is_compileable = True
    is_sliding = False

    def __init__(self, capacity: int):
        super().__init__()
        self.capacity = capacity
        self.is_initialized = True

    def lazy_initialization(self, *args, **kwargs) -> None:
        pass

    def update(self, key_states, value_states, *args, **kwargs):
        return key_states, value_states

    def get_mask_sizes(self, *args, **kwargs) -> tuple[int, int]:
        return self.capacity, 0

    def get_seq_length(self, *args, **kwargs) -> int:
        return 0

    def get_max_cache_shape(self) -> int:
        return self.capacity

    def get_max_length(self) -> int:
        return self.capacity


def _pass_through_cache(layer_count: int, capacity: int) -> Cache:
    return Cache(layers=[_PassThroughLayer(capacity) for _ in range(layer_count)])


def _text_config(model: torch.nn.Module):
    config = model.config
    getter = getattr(config, "get_text_config", None)
    return getter(decoder=True) if getter is not None else config


def _head_dim(config) -> int:
    return getattr(config, "head_dim", None) or config.hidden_size // config.num_attention_heads


class _ExplicitState(torch.nn.Module):
    layer_count: int
    kv_heads: int
    head_dim: int
    capacity: int | None

    def state_shapes(self, batch: int = 1, dtype: torch.dtype = torch.bfloat16,
                     capacity: int | None = None, per_row_lengths: bool = False):
        """Per layer ``[key_cache, value_cache, valid_length]``.  The valid length is int32
        ``[1]``, shared by the batch (the reference's contract,
        ``fx_handler/hf_attention.py:194-196``), or ``[batch]`` with ``per_row_lengths``: rows
        then hold different numbers of keys."""
        capacity = self.capacity if capacity is None else capacity
        cache = ((batch, capacity, self.kv_heads, self.head_dim), dtype)
        lengths = ((batch if per_row_lengths else 1,), torch.int32)
        return [[cache, cache, lengths] for _ in range(self.layer_count)]

    def make_state(self, batch: int = 1, *, capacity: int | None = None, device=None,
                   dtype: torch.dtype = torch.bfloat16,
                   per_row_lengths: bool = False) -> list[torch.Tensor]:
        """Zeroed state tensors in ``forward`` order."""
        flat = []
        for layer in self.state_shapes(batch, dtype, capacity, per_row_lengths):
            for shape, kind in layer:
                flat.append(torch.zeros(shape, dtype=kind, device=device))
        return flat


class DecodeStep(_ExplicitState):
    """One-token decode of any Hugging Face attention model over explicit state."""

    def __init__(self, model: torch.nn.Module, capacity: int):
        super().__init__()
        register_transformers_attention()
        model.set_attn_implementation(ATTENTION_IMPLEMENTATION)
        self.model = model
        self.capacity = capacity
        config = _text_config(model)
        kinds = set(getattr(config, "layer_types", None) or ())
        if kinds - {"full_attention", "sliding_attention"}:
            raise NotImplementedError(f"decode of {sorted(kinds)} layers is not declared")
        self.layer_count = config.num_hidden_layers
        self.kv_heads = config.num_key_value_heads
        self.head_dim = _head_dim(config)

    def forward(self, input_ids: torch.Tensor, position_ids: torch.Tensor, *state: torch.Tensor):
        triples = tuple(tuple(state[3 * i : 3 * i + 3]) for i in range(self.layer_count))
        return self.model(
            input_ids=input_ids,
            position_ids=position_ids,
            past_key_values=_pass_through_cache(self.layer_count, self.capacity),
            use_cache=True,
            megabake_state=triples,
        ).logits


class StatefulDecoder(_ExplicitState):
    """Explicit embed -> (norm, attention, residual, norm, MLP, residual)* -> norm ->
    head loop over a Hugging Face pre-norm decoder, one token per call."""

    def __init__(self, model: torch.nn.Module, capacity: int | None = None):
        super().__init__()
        inner = model.model
        self.model = getattr(inner, "language_model", inner)
        self.lm_head = model.lm_head
        self.config = _text_config(model)
        self.capacity = capacity
        self.layer_count = self.config.num_hidden_layers
        self.kv_heads = self.config.num_key_value_heads
        self.head_dim = _head_dim(self.config)
        kinds = set(getattr(self.config, "layer_types", None) or ())
        if kinds - {"full_attention"}:
            raise NotImplementedError(f"decode of {sorted(kinds)} layers is not declared")

    def _attend(self, module, normalized, rotary, key_cache, value_cache, valid_length):
        batch, steps, _ = normalized.shape
        dim = self.head_dim
        query = module.q_proj(normalized).view(batch, steps, -1, dim)
        key = module.k_proj(normalized).view(batch, steps, -1, dim)
        value = module.v_proj(normalized).view(batch, steps, -1, dim)
        rotate = sys.modules[type(module).__module__].apply_rotary_pos_emb
        query, key = rotate(query, key, rotary[0], rotary[1], unsqueeze_dim=2)
        rescale = module.scaling * dim**0.5
        if abs(rescale - 1.0) > 1e-6:
            query = query * rescale
        mixed = torch.ops.megabake.kv_attention(
            query, key, value, key_cache, value_cache, valid_length
        )
        return module.o_proj(mixed.reshape(batch, steps, -1))

    def forward(self, input_ids: torch.Tensor, position_ids: torch.Tensor, *state: torch.Tensor):
        if len(state) != 3 * self.layer_count:
            raise ValueError(f"expected {3 * self.layer_count} state tensors, got {len(state)}")
        hidden = self.model.embed_tokens(input_ids)
        position_ids = position_ids.to(torch.int64)
        rotary = self.model.rotary_emb(hidden, position_ids)
        for index, layer in enumerate(self.model.layers):
            key_cache, value_cache, valid_length = state[3 * index : 3 * index + 3]
            mixed = self._attend(
                layer.self_attn, layer.input_layernorm(hidden), rotary,
                key_cache, value_cache, valid_length,
            )
            hidden = hidden + mixed
            hidden = hidden + layer.mlp(layer.post_attention_layernorm(hidden))
        return self.lm_head(self.model.norm(hidden))


class GroupedStateDecoder(StatefulDecoder):
    """``StatefulDecoder`` with the state tensors grouped by kind instead of by layer:
    ``forward(input_ids, position_ids, K_0..K_{L-1}, V_0..V_{L-1}, len_0..len_{L-1})`` -- the
    calling convention of the reference's ``StatefulSmolLM`` (``tests/fixtures.py:220-238``), which
    its benchmark uses for Llama-family models (``benchmarks/full_model.py:235-255``)."""

    def state_shapes(self, batch: int = 1, dtype: torch.dtype = torch.bfloat16,
                     capacity: int | None = None, per_row_lengths: bool = False):
        per_layer = super().state_shapes(batch, dtype, capacity, per_row_lengths)
        return [[layer[kind] for layer in per_layer] for kind in range(3)]

    def forward(self, input_ids: torch.Tensor, position_ids: torch.Tensor, *state: torch.Tensor):
        count = self.layer_count
        if len(state) != 3 * count:
            raise ValueError(f"expected {3 * count} state tensors, got {len(state)}")
        by_layer = [state[kind * count + index] for index in range(count) for kind in range(3)]
        return super().forward(input_ids, position_ids, *by_layer)


class PrefillLogits(torch.nn.Module):
    """``forward(input_ids[B, T]) -> logits[B, T, V]``: a full causal prefill at positions
    0..T-1 with every attention module routed to ``megabake::attention``.  This is the callable
    the reference's prefill benchmark compiles (``benchmarks/full_model.py:178-200``: the model
    itself, called on the prompt), reduced to its logits so that the compiled graph has one
    output."""

    def __init__(self, model: torch.nn.Module):
        super().__init__()
        register_transformers_attention()
        model.config._attn_implementation = ATTENTION_IMPLEMENTATION
        self.model = model

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        return self.model(input_ids=input_ids, use_cache=False).logits


class StatefulPrefill(StatefulDecoder):
    """``forward(input_ids[B, T], *state) -> logits[B, T, V]``: a full causal prefill at
    positions 0..T-1 that also fills the explicit decode state (rows 0..T-1 of every layer's
    caches, valid lengths = T) through ``megabake::prefill_kv_attention``.  Same state tensors and
    order as ``StatefulDecoder`` / ``DecodeStep``: compile this with ``mode="prefill"``, the decode
    wrapper with ``mode="decode"``, and generation is prefill once, then one decode call per
    token."""

    def _attend(self, module, normalized, rotary, key_cache, value_cache, valid_length):
        batch, tokens, _ = normalized.shape
        dim = self.head_dim
        query = module.q_proj(normalized).view(batch, tokens, -1, dim)
        key = module.k_proj(normalized).view(batch, tokens, -1, dim)
        value = module.v_proj(normalized).view(batch, tokens, -1, dim)
        rotate = sys.modules[type(module).__module__].apply_rotary_pos_emb
        query, key = rotate(query, key, rotary[0], rotary[1], unsqueeze_dim=2)
        mixed = torch.ops.megabake.prefill_kv_attention(
            query, key, value, key_cache, value_cache, valid_length, float(module.scaling)
        )
        mixed = mixed.view(batch, -1, tokens, dim).transpose(1, 2)
        return module.o_proj(mixed.reshape(batch, tokens, -1))

    def forward(self, input_ids: torch.Tensor, *state: torch.Tensor):
        batch, tokens = input_ids.shape
        positions = torch.arange(tokens, device=input_ids.device)[None].expand(batch, -1)
        return super().forward(input_ids, positions, *state)
