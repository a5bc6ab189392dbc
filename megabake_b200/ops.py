"""The two attention operators a model declares to the backend.

``megabake::kv_attention`` (one-token decode over an explicit, caller-owned KV
cache that the op itself appends to) and ``megabake::attention`` (prefill
attention with an additive mask).  Names, schemas, mutation annotations, result
layout ``[batch * heads, query, dim]`` and the rounding points of the eager
definitions are those of the reference (``src/megabake/ops/attention.py:52-87``
for the stateful op, ``:113-140`` for the stateless one, fake kernels at
``:90-107`` and ``:143-149``) so a model written against the reference traces to
the same FX nodes here.

The eager bodies below are what runs when the op is called outside a compiled
megakernel, and what the ``compile_kernel=False`` FX forward runs.  Rounding
contract they fix (and the CUDA bodies reproduce):

* stateful decode: scores are a bf16 matmul result, widened to fp32 and scaled by
  ``dim ** -0.5`` *in fp32*; softmax in fp32; probabilities rounded to bf16;
  value product accumulated in fp32 and rounded once.
* prefill: scores are a bf16 matmul result scaled *in bf16*, the additive mask is
  added in bf16, softmax runs in fp32 and is rounded to bf16 before the value
  product.
"""

from __future__ import annotations

import torch

__all__ = ["kv_attention", "attention", "prefill_kv_attention", "KV_ATTENTION_OP", "ATTENTION_OP",
           "PREFILL_KV_ATTENTION_OP"]


def _repeat_kv(tensor: torch.Tensor, groups: int) -> torch.Tensor:
    # [batch, kv_heads, keys, dim] -> [batch, kv_heads * groups, keys, dim]
    return tensor if groups == 1 else tensor.repeat_interleave(groups, dim=1)


@torch.library.custom_op(
    "megabake::kv_attention",
    mutates_args=("key_cache", "value_cache", "valid_length"),
)
def kv_attention(
    source: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    valid_length: torch.Tensor,
) -> torch.Tensor:
    """Append ``key``/``value`` (``[batch, 1, kv_heads, dim]``) to the caches
    (``[batch, capacity, kv_heads, dim]``) at ``valid_length``, add one to it, and attend
    ``source`` (``[batch, 1, heads, dim]``) over every valid key.  ``valid_length`` is int32
    ``[1]`` (one length shared by the batch: the reference's operator,
    ``src/megabake/ops/attention.py:52-87``) or ``[batch]`` (one length per row, so that rows may
    hold prompts of different lengths: the reference's roadmap step 12,
    ``docs/roadmap.md:178``); with per-row lengths every row is the shared-length operator
    applied to that row alone."""
    batch, steps, heads, dim = source.shape
    if steps != 1:
        raise RuntimeError("megabake kv_attention supports one-token decode only")
    if valid_length.numel() not in (1, batch):
        raise RuntimeError(f"valid_length must hold 1 or {batch} lengths, got {valid_length.numel()}")
    if valid_length.numel() == batch and batch > 1:
        rows = [kv_attention(source[b:b + 1], key[b:b + 1], value[b:b + 1], key_cache[b:b + 1],
                             value_cache[b:b + 1], valid_length[b:b + 1]) for b in range(batch)]
        return torch.cat(rows, dim=0)
    first = int(valid_length.item())
    last = first + steps
    capacity = key_cache.shape[1]
    if first < 0 or last > capacity:
        raise RuntimeError(f"KV cache length {first} plus {steps} exceeds capacity {capacity}")
    key_cache[:, first:last].copy_(key)
    value_cache[:, first:last].copy_(value)
    valid_length.fill_(last)
    groups = heads // key_cache.shape[2]
    q = source.permute(0, 2, 1, 3)
    k = _repeat_kv(key_cache[:, :last].permute(0, 2, 1, 3), groups)
    v = _repeat_kv(value_cache[:, :last].permute(0, 2, 1, 3), groups)
    scores = torch.matmul(q, k.transpose(-2, -1)).float() * dim**-0.5
    weights = torch.softmax(scores, dim=-1).to(source.dtype)
    mixed = torch.matmul(weights, v)
    return mixed.permute(0, 2, 1, 3).reshape(batch * heads, steps, dim)


@kv_attention.register_fake
def _(source, key, value, key_cache, value_cache, valid_length):
    batch, steps, heads, dim = source.shape
    return source.new_empty((batch * heads, steps, dim))


@torch.library.custom_op("megabake::attention", mutates_args=())
def attention(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    mask: torch.Tensor | None,
    scale: float,
) -> torch.Tensor:
    """Masked softmax attention with Hugging Face eager numerics.  ``query`` is
    ``[batch, query, heads, dim]``, ``key``/``value`` ``[batch, key, kv_heads, dim]``,
    ``mask`` additive and broadcastable to ``[batch, heads, query, key]``."""
    q = query.transpose(1, 2)
    groups = q.shape[1] // key.shape[2]
    k = _repeat_kv(key.transpose(1, 2), groups)
    v = _repeat_kv(value.transpose(1, 2), groups)
    scores = torch.matmul(q, k.transpose(2, 3)) * scale
    if mask is not None:
        scores = scores + mask
    weights = torch.softmax(scores, dim=-1, dtype=torch.float32).to(q.dtype)
    mixed = torch.matmul(weights, v)
    return mixed.reshape(-1, mixed.shape[2], mixed.shape[3])


@attention.register_fake
def _(query, key, value, mask, scale):
    batch, length, heads, dim = query.shape
    return query.new_empty((batch * heads, length, dim))


@torch.library.custom_op(
    "megabake::prefill_kv_attention",
    mutates_args=("key_cache", "value_cache", "valid_length"),
)
def prefill_kv_attention(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    valid_length: torch.Tensor,
    scale: float,
) -> torch.Tensor:
    """Causal prefill attention that also hands the prompt's keys and values to the decode
    state: ``key``/``value`` (``[batch, tokens, kv_heads, dim]``) are written to rows
    ``0 .. tokens - 1`` of the caches (``[batch, capacity, kv_heads, dim]``) and
    ``valid_length`` (int32 ``[1]``) is set to ``tokens``, so that ``megabake::kv_attention``
    can continue from there.  The attention itself is ``megabake::attention`` with the causal
    mask (same rounding points).  The reference has no such operator: its prefill cannot seed
    its decode state (``examples/single_gpu_generate.py:3-4``)."""
    batch, tokens, heads, dim = query.shape
    capacity = key_cache.shape[1]
    if tokens > capacity:
        raise RuntimeError(f"prompt of {tokens} tokens exceeds the KV capacity {capacity}")
    key_cache[:, :tokens].copy_(key)
    value_cache[:, :tokens].copy_(value)
    valid_length.fill_(tokens)
    allowed = torch.tril(torch.ones(tokens, tokens, dtype=torch.bool, device=query.device))
    mask = torch.where(allowed, torch.zeros((), dtype=query.dtype, device=query.device),
                       torch.full((), torch.finfo(query.dtype).min, dtype=query.dtype,
                                  device=query.device))[None, None]
    q = query.transpose(1, 2)
    groups = heads // key.shape[2]
    k = _repeat_kv(key.transpose(1, 2), groups)
    v = _repeat_kv(value.transpose(1, 2), groups)
    scores = torch.matmul(q, k.transpose(2, 3)) * scale + mask
    weights = torch.softmax(scores, dim=-1, dtype=torch.float32).to(q.dtype)
    mixed = torch.matmul(weights, v)
    return mixed.reshape(-1, mixed.shape[2], mixed.shape[3])


@prefill_kv_attention.register_fake
def _(query, key, value, key_cache, value_cache, valid_length, scale):
    batch, length, heads, dim = query.shape
    return query.new_empty((batch * heads, length, dim))


KV_ATTENTION_OP = torch.ops.megabake.kv_attention.default
PREFILL_KV_ATTENTION_OP = torch.ops.megabake.prefill_kv_attention.default
ATTENTION_OP = torch.ops.megabake.attention.default
