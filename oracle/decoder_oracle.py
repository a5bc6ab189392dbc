"""CPU oracle for the decoder hot path -- TEST INFRASTRUCTURE, not a product path.

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline / reference arm
may import this module; nothing under ``megabake_b200/`` does.

It restates, op by op and with every bf16 rounding point, the eager forward the reference
treats as truth for one-token decode and for prefill:

* decode loop over explicit ``[K, V, len]`` state -- reference
  ``benchmarks/stateful_models.py:152-187`` (``StatefulCausalLM.forward``; attention at
  ``:87-116``) and ``tests/fixtures.py:220-288`` (``StatefulSmolLM.forward``);
* the stateful attention op -- reference ``src/megabake/ops/attention.py:52-87``;
* the prefill attention op -- reference ``src/megabake/ops/attention.py:113-140``;
* the layer math that lives in the third-party ``transformers`` package (pinned 5.21.0 in
  the reference's ``uv.lock``, 5.5.0 installed here): Llama/Qwen2 RMSNorm
  ``w * bf16(x * rsqrt(mean(x^2) + eps))``, Gemma RMSNorm ``bf16(x * rsqrt(...) * (1 + w))``,
  rotary tables ``cos/sin(float(pos) * inv_freq) * attention_scaling -> bf16`` and
  ``q * cos + rotate_half(q) * sin``, SwiGLU / GeGLU-tanh MLP, Gemma's ``sqrt(hidden)``
  embedding scale as a bf16 scalar.

Parity pin: ``tests/golden/make_golden.py`` runs the reference's own wrappers and custom ops
(imported from the reference checkout) on seeded tiny and full-size models and stores their
outputs; ``tests/test_oracle_golden.py`` requires this module to reproduce them bit for bit.

Everything runs with plain ``torch`` CPU ops on bf16 tensors, so each op rounds exactly as
ATen's eager kernels do.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

BF16 = torch.bfloat16


@dataclass
class OracleConfig:
    hidden: int
    layers: int
    heads: int
    kv_heads: int
    head_dim: int
    intermediate: int
    vocab: int
    eps: float
    norm: str = "llama"          # "llama" | "gemma"
    activation: str = "silu"     # "silu" | "gelu_tanh"
    embed_scale: float | None = None
    rope_scale: float = 1.0      # attention_scaling
    qkv_bias: bool = False
    query_rescale: float | None = None  # attention.scaling * sqrt(head_dim) when != 1


@dataclass
class OracleWeights:
    """bf16 tensors under Hugging Face parameter names (``model.layers.0.self_attn...``),
    plus ``inv_freq`` exactly as the model's rotary buffer holds it (bf16 after
    ``model.to(bfloat16)``)."""

    tensors: dict[str, torch.Tensor]
    inv_freq: torch.Tensor
    tied: bool = True

    def __getitem__(self, name: str) -> torch.Tensor:
        return self.tensors[name]

    def get(self, name: str):
        return self.tensors.get(name)

    def lm_head(self) -> torch.Tensor:
        return self.tensors["model.embed_tokens.weight"] if self.tied else self.tensors["lm_head.weight"]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, kind: str) -> torch.Tensor:
    wide = x.float()
    variance = wide.pow(2).mean(-1, keepdim=True)
    scaled = wide * torch.rsqrt(variance + eps)
    if kind == "gemma":
        return (scaled * (1.0 + weight.float())).to(x.dtype)
    return weight * scaled.to(x.dtype)


def rotary_tables(inv_freq: torch.Tensor, positions: torch.Tensor, scale: float, dtype=BF16):
    """``positions`` int64 ``[B, T]`` -> cos, sin ``[B, T, D]`` in ``dtype``."""
    expanded = inv_freq[None, :, None].float().expand(positions.shape[0], -1, 1)
    freqs = (expanded @ positions[:, None, :].float()).transpose(1, 2)
    emb = torch.cat((freqs, freqs), dim=-1)
    return (emb.cos() * scale).to(dtype), (emb.sin() * scale).to(dtype)


def _rotate_half(x: torch.Tensor) -> torch.Tensor:
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """``x`` ``[B, T, heads, D]``; cos/sin ``[B, T, D]``."""
    cos = cos.unsqueeze(2)
    sin = sin.unsqueeze(2)
    return (x * cos) + (_rotate_half(x) * sin)


def _expand_kv(t: torch.Tensor, groups: int) -> torch.Tensor:
    return t if groups == 1 else t.repeat_interleave(groups, dim=1)


def kv_attention(query, key, value, key_cache, value_cache, valid_length) -> torch.Tensor:
    """Stateful one-token attention; mutates the caches and the length.
    Shapes as ``megabake::kv_attention``; returns ``[B * heads, 1, D]``."""
    batch, steps, heads, dim = query.shape
    assert steps == 1
    if valid_length.numel() == batch and batch > 1:
        # one length per row: the shared-length operator applied to every row alone (pinned by
        # tests/golden/ops_per_row.npz, made by calling the reference's operator row by row)
        rows = [kv_attention(query[b:b + 1], key[b:b + 1], value[b:b + 1], key_cache[b:b + 1],
                             value_cache[b:b + 1], valid_length[b:b + 1]) for b in range(batch)]
        return torch.cat(rows, dim=0)
    start = int(valid_length.item())
    stop = start + 1
    if stop > key_cache.shape[1]:
        raise RuntimeError(f"KV cache length {start} plus 1 exceeds capacity {key_cache.shape[1]}")
    key_cache[:, start:stop].copy_(key)
    value_cache[:, start:stop].copy_(value)
    valid_length.fill_(stop)
    groups = heads // key_cache.shape[2]
    q = query.permute(0, 2, 1, 3)
    k = _expand_kv(key_cache[:, :stop].permute(0, 2, 1, 3), groups)
    v = _expand_kv(value_cache[:, :stop].permute(0, 2, 1, 3), groups)
    scores = (q @ k.transpose(-2, -1)).float() * dim**-0.5
    weights = torch.softmax(scores, dim=-1).to(query.dtype)
    mixed = weights @ v
    return mixed.permute(0, 2, 1, 3).reshape(batch * heads, 1, dim)


def prefill_attention(query, key, value, mask, scale: float) -> torch.Tensor:
    """``megabake::attention``: q ``[B, T, H, D]``, k/v ``[B, S, Hkv, D]``, additive mask."""
    q = query.transpose(1, 2)
    groups = q.shape[1] // key.shape[2]
    k = _expand_kv(key.transpose(1, 2), groups)
    v = _expand_kv(value.transpose(1, 2), groups)
    scores = torch.matmul(q, k.transpose(2, 3)) * scale
    if mask is not None:
        scores = scores + mask
    weights = torch.softmax(scores, dim=-1, dtype=torch.float32).to(q.dtype)
    mixed = torch.matmul(weights, v)
    return mixed.reshape(-1, mixed.shape[2], mixed.shape[3])


def causal_mask(batch: int, length: int, dtype=BF16) -> torch.Tensor:
    """The additive mask Hugging Face's ``eager_mask`` builds for a full causal prefill:
    0 where key <= query, the dtype's most negative finite value elsewhere."""
    allowed = torch.tril(torch.ones(length, length, dtype=torch.bool))
    floor = torch.finfo(dtype).min
    mask = torch.where(allowed, torch.tensor(0.0, dtype=dtype), torch.tensor(floor, dtype=dtype))
    return mask[None, None].expand(batch, 1, length, length)


def _linear(x, weight, bias=None):
    return torch.nn.functional.linear(x, weight, bias)


def _activation(x: torch.Tensor, kind: str) -> torch.Tensor:
    if kind == "silu":
        return torch.nn.functional.silu(x)
    return torch.nn.functional.gelu(x, approximate="tanh")


@dataclass
class DecodeTrace:
    """Optional per-layer intermediates, for locating the first divergent region."""

    entries: dict[str, torch.Tensor] = field(default_factory=dict)

    def put(self, name: str, value: torch.Tensor) -> None:
        self.entries[name] = value.detach().clone()


def _embed(cfg: OracleConfig, w: OracleWeights, ids: torch.Tensor) -> torch.Tensor:
    hidden = torch.nn.functional.embedding(ids, w["model.embed_tokens.weight"])
    if cfg.embed_scale is not None:
        hidden = hidden * torch.tensor(cfg.embed_scale, dtype=hidden.dtype)
    return hidden


def _mlp(cfg, w, prefix, x):
    gate = _linear(x, w[prefix + "mlp.gate_proj.weight"])
    up = _linear(x, w[prefix + "mlp.up_proj.weight"])
    return _linear(_activation(gate, cfg.activation) * up, w[prefix + "mlp.down_proj.weight"])


def decode_step(cfg: OracleConfig, w: OracleWeights, input_ids: torch.Tensor,
                position_ids: torch.Tensor, state: list[torch.Tensor],
                trace: DecodeTrace | None = None) -> torch.Tensor:
    """One token per row.  ``state`` is per layer ``[key_cache, value_cache, valid_length]``
    flattened in that order; caches and lengths are updated in place.  Returns logits
    ``[B, 1, V]`` bf16."""
    hidden = _embed(cfg, w, input_ids)
    batch = hidden.shape[0]
    cos, sin = rotary_tables(w.inv_freq, position_ids.to(torch.int64), cfg.rope_scale, hidden.dtype)
    for index in range(cfg.layers):
        prefix = f"model.layers.{index}."
        key_cache, value_cache, valid_length = state[3 * index: 3 * index + 3]
        normed = rms_norm(hidden, w[prefix + "input_layernorm.weight"], cfg.eps, cfg.norm)
        q = _linear(normed, w[prefix + "self_attn.q_proj.weight"], w.get(prefix + "self_attn.q_proj.bias"))
        k = _linear(normed, w[prefix + "self_attn.k_proj.weight"], w.get(prefix + "self_attn.k_proj.bias"))
        v = _linear(normed, w[prefix + "self_attn.v_proj.weight"], w.get(prefix + "self_attn.v_proj.bias"))
        q = q.view(batch, 1, cfg.heads, cfg.head_dim)
        k = k.view(batch, 1, cfg.kv_heads, cfg.head_dim)
        v = v.view(batch, 1, cfg.kv_heads, cfg.head_dim)
        q = apply_rope(q, cos, sin)
        k = apply_rope(k, cos, sin)
        if cfg.query_rescale is not None:
            q = q * cfg.query_rescale
        mixed = kv_attention(q, k, v, key_cache, value_cache, valid_length)
        mixed = mixed.reshape(batch, 1, cfg.heads * cfg.head_dim)
        if trace is not None:
            trace.put(f"{index}.attention", mixed)
        hidden = hidden + _linear(mixed, w[prefix + "self_attn.o_proj.weight"])
        normed = rms_norm(hidden, w[prefix + "post_attention_layernorm.weight"], cfg.eps, cfg.norm)
        hidden = hidden + _mlp(cfg, w, prefix, normed)
        if trace is not None:
            trace.put(f"{index}.hidden", hidden)
    final = rms_norm(hidden, w["model.norm.weight"], cfg.eps, cfg.norm)
    return _linear(final, w.lm_head())


def prefill(cfg: OracleConfig, w: OracleWeights, input_ids: torch.Tensor,
            return_kv: bool = False):
    """Full causal prefill of ``input_ids`` ``[B, T]`` (positions 0..T-1).  Returns logits
    ``[B, T, V]`` bf16 and, if asked, the per-layer post-RoPE keys and the values
    ``[B, T, Hkv, D]`` (what a decode cache would hold)."""
    batch, length = input_ids.shape
    hidden = _embed(cfg, w, input_ids)
    positions = torch.arange(length, dtype=torch.int64)[None].expand(batch, -1)
    cos, sin = rotary_tables(w.inv_freq, positions, cfg.rope_scale, hidden.dtype)
    mask = causal_mask(batch, length, hidden.dtype)
    scale = cfg.head_dim**-0.5 if cfg.query_rescale is None else cfg.head_dim**-0.5 * cfg.query_rescale
    kv = []
    for index in range(cfg.layers):
        prefix = f"model.layers.{index}."
        normed = rms_norm(hidden, w[prefix + "input_layernorm.weight"], cfg.eps, cfg.norm)
        q = _linear(normed, w[prefix + "self_attn.q_proj.weight"], w.get(prefix + "self_attn.q_proj.bias"))
        k = _linear(normed, w[prefix + "self_attn.k_proj.weight"], w.get(prefix + "self_attn.k_proj.bias"))
        v = _linear(normed, w[prefix + "self_attn.v_proj.weight"], w.get(prefix + "self_attn.v_proj.bias"))
        q = apply_rope(q.view(batch, length, cfg.heads, cfg.head_dim), cos, sin)
        k = apply_rope(k.view(batch, length, cfg.kv_heads, cfg.head_dim), cos, sin)
        v = v.view(batch, length, cfg.kv_heads, cfg.head_dim)
        if return_kv:
            kv.append((k.clone(), v.clone()))
        mixed = prefill_attention(q, k, v, mask, scale)
        mixed = mixed.view(batch, cfg.heads, length, cfg.head_dim).transpose(1, 2)
        mixed = mixed.reshape(batch, length, cfg.heads * cfg.head_dim)
        hidden = hidden + _linear(mixed, w[prefix + "self_attn.o_proj.weight"])
        normed = rms_norm(hidden, w[prefix + "post_attention_layernorm.weight"], cfg.eps, cfg.norm)
        hidden = hidden + _mlp(cfg, w, prefix, normed)
    final = rms_norm(hidden, w["model.norm.weight"], cfg.eps, cfg.norm)
    logits = _linear(final, w.lm_head())
    return (logits, kv) if return_kv else logits


def make_state(cfg: OracleConfig, batch: int, capacity: int, dtype=BF16,
               per_row_lengths: bool = False) -> list[torch.Tensor]:
    state = []
    for _ in range(cfg.layers):
        state.append(torch.zeros(batch, capacity, cfg.kv_heads, cfg.head_dim, dtype=dtype))
        state.append(torch.zeros(batch, capacity, cfg.kv_heads, cfg.head_dim, dtype=dtype))
        state.append(torch.zeros(batch if per_row_lengths else 1, dtype=torch.int32))
    return state


def greedy_decode(cfg: OracleConfig, w: OracleWeights, prompt: torch.Tensor, steps: int,
                  capacity: int, step_fn=None):
    """The decode protocol of the benchmark configs: feed ``prompt`` ``[B, P]`` one token per
    call (P calls), then ``steps`` more calls that each feed the previous call's greedy
    token.  Returns the greedy ids after every call ``[B, P + steps]``, the logits of every
    call and the final state.  ``step_fn(ids, pos, state)`` replaces the oracle step (used
    to drive another implementation through the same protocol)."""
    batch, plen = prompt.shape
    state = make_state(cfg, batch, capacity)
    if step_fn is None:
        step_fn = lambda ids, pos, st: decode_step(cfg, w, ids, pos, st)  # noqa: E731
    logits_log, picks = [], []
    token = prompt[:, :1].contiguous()
    for call in range(plen + steps):
        pos = torch.full((batch, 1), call, dtype=torch.int64)
        logits = step_fn(token, pos, state)
        logits_log.append(logits)
        pick = logits[:, -1].float().argmax(-1, keepdim=True)
        picks.append(pick)
        token = prompt[:, call + 1: call + 2].contiguous() if call + 1 < plen else pick
    return torch.cat(picks, dim=1), logits_log, state
