"""Decoder shapes of the benchmark configurations, seeded random-init weights, and the two
ways to get a ``DecoderProgram`` for them: from explicit tensors (``direct_program``, no
Dynamo) or through Hugging Face modules and ``make_backend`` (``build_hf_model``).

Weights follow the synthetic-data protocol of the benchmark: every >= 2-D parameter and every
bias is N(0, 0.02) drawn in fp32 from one seeded CPU generator in Hugging Face
``named_parameters()`` order and cast to bf16; RMSNorm weights are 1.0 (Gemma stores ``w`` with
``1 + w`` applied, so 0.0); embeddings are tied to the LM head.  ``inv_freq`` is computed as
the Hugging Face rotary module does (including the ``llama3`` frequency scaling) and then
rounded to bf16, which is what ``model.to(torch.bfloat16)`` does to that buffer.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, replace

import torch

from .program import DecoderProgram, LayerBinding


@dataclass(frozen=True)
class ModelSpec:
    name: str
    family: str  # "llama" | "qwen2" | "gemma"
    hidden: int
    layers: int
    heads: int
    kv_heads: int
    head_dim: int
    intermediate: int
    vocab: int
    eps: float
    rope_theta: float
    qkv_bias: bool = False
    rope_scaling: tuple | None = None  # ("llama3", factor, low, high, original_max_positions)
    max_positions: int = 16384

    @property
    def norm(self) -> str:
        return "gemma" if self.family == "gemma" else "llama"

    @property
    def activation(self) -> str:
        return "gelu_tanh" if self.family == "gemma" else "silu"

    @property
    def embed_scale(self) -> float | None:
        if self.family != "gemma":
            return None
        # the model multiplies by tensor(sqrt(hidden)).to(bf16)
        return float(torch.tensor(self.hidden**0.5).to(torch.bfloat16))

    def parameter_count(self) -> int:
        d = self.head_dim
        per_layer = (self.heads * d * self.hidden + 2 * self.kv_heads * d * self.hidden
                     + self.hidden * self.heads * d + 3 * self.hidden * self.intermediate
                     + 2 * self.hidden)
        if self.qkv_bias:
            per_layer += (self.heads + 2 * self.kv_heads) * d
        return self.layers * per_layer + self.vocab * self.hidden + self.hidden


PRESETS: dict[str, ModelSpec] = {
    "smollm-135m": ModelSpec("smollm-135m", "llama", 576, 30, 9, 3, 64, 1536, 49152, 1e-5, 1e4),
    "qwen2-0.5b": ModelSpec("qwen2-0.5b", "qwen2", 896, 24, 14, 2, 64, 4864, 151936, 1e-6, 1e6,
                            qkv_bias=True),
    "llama-3.2-1b": ModelSpec("llama-3.2-1b", "llama", 2048, 16, 32, 8, 64, 8192, 128256, 1e-5,
                              5e5, rope_scaling=("llama3", 32.0, 1.0, 4.0, 8192)),
    "smollm-1.7b": ModelSpec("smollm-1.7b", "llama", 2048, 24, 32, 32, 64, 8192, 49152, 1e-5,
                             1e4),
    "gemma-2b": ModelSpec("gemma-2b", "gemma", 2048, 18, 8, 1, 256, 16384, 256000, 1e-6, 1e4),
    # small shapes for tests (same families, every code path, seconds on CPU)
    "tiny-llama": ModelSpec("tiny-llama", "llama", 256, 2, 4, 2, 64, 512, 512, 1e-5, 1e4),
    "tiny-llama3": ModelSpec("tiny-llama3", "llama", 256, 2, 4, 1, 64, 512, 640, 1e-5, 5e5,
                             rope_scaling=("llama3", 32.0, 1.0, 4.0, 8192)),
    "tiny-qwen2": ModelSpec("tiny-qwen2", "qwen2", 448, 2, 7, 1, 64, 1216, 1024, 1e-6, 1e6,
                            qkv_bias=True),
    "tiny-mha": ModelSpec("tiny-mha", "llama", 256, 2, 4, 4, 64, 512, 512, 1e-5, 1e4),
    "tiny-gemma": ModelSpec("tiny-gemma", "gemma", 256, 2, 2, 1, 128, 768, 768, 1e-6, 1e4),
    "tiny-gemma256": ModelSpec("tiny-gemma256", "gemma", 256, 1, 8, 1, 256, 512, 512, 1e-6, 1e4),
}


def get_spec(name: str, **overrides) -> ModelSpec:
    spec = PRESETS[name]
    return replace(spec, **overrides) if overrides else spec


# ---------------------------------------------------------------------------------------
# Weights
# ---------------------------------------------------------------------------------------
def parameter_shapes(spec: ModelSpec) -> list[tuple[str, tuple[int, ...]]]:
    """(name, shape) in Hugging Face ``named_parameters()`` order (tied LM head omitted)."""
    d = spec.head_dim
    out: list[tuple[str, tuple[int, ...]]] = [("model.embed_tokens.weight", (spec.vocab, spec.hidden))]
    for index in range(spec.layers):
        prefix = f"model.layers.{index}."
        for proj, rows in (("q_proj", spec.heads * d), ("k_proj", spec.kv_heads * d),
                           ("v_proj", spec.kv_heads * d)):
            out.append((prefix + f"self_attn.{proj}.weight", (rows, spec.hidden)))
            if spec.qkv_bias:
                out.append((prefix + f"self_attn.{proj}.bias", (rows,)))
        out.append((prefix + "self_attn.o_proj.weight", (spec.hidden, spec.heads * d)))
        out.append((prefix + "mlp.gate_proj.weight", (spec.intermediate, spec.hidden)))
        out.append((prefix + "mlp.up_proj.weight", (spec.intermediate, spec.hidden)))
        out.append((prefix + "mlp.down_proj.weight", (spec.hidden, spec.intermediate)))
        out.append((prefix + "input_layernorm.weight", (spec.hidden,)))
        out.append((prefix + "post_attention_layernorm.weight", (spec.hidden,)))
    out.append(("model.norm.weight", (spec.hidden,)))
    return out


def fill_parameter(name: str, shape: tuple[int, ...], generator: torch.Generator,
                   norm_value: float) -> torch.Tensor:
    device = generator.device
    if name.endswith("layernorm.weight") or name.endswith("norm.weight"):
        return torch.full(shape, norm_value, dtype=torch.bfloat16, device=device)
    values = torch.empty(shape, dtype=torch.float32, device=device)
    values.normal_(0.0, 0.02, generator=generator)
    return values.to(torch.bfloat16)


def init_weights(spec: ModelSpec, seed: int = 0, device: str | torch.device = "cpu",
                 on_device: bool = False) -> dict[str, torch.Tensor]:
    """Seeded random-init bf16 weights.  By default they are drawn on CPU (bit-reproducible
    everywhere, what the parity tests need) and then moved; ``on_device=True`` draws them with
    the target device's generator instead (same distribution, seconds faster for the
    billion-parameter benchmark shapes, not bit-equal to the CPU draw)."""
    where = torch.device(device) if on_device else torch.device("cpu")
    generator = torch.Generator(device=where).manual_seed(seed)
    norm_value = 0.0 if spec.family == "gemma" else 1.0
    weights = {}
    for name, shape in parameter_shapes(spec):
        weights[name] = fill_parameter(name, shape, generator, norm_value).to(device)
    return weights


def inverse_frequencies(spec: ModelSpec) -> torch.Tensor:
    """fp32 ``inv_freq`` as ``transformers`` computes it for the spec's rope settings."""
    dim = spec.head_dim
    inv = 1.0 / (spec.rope_theta ** (torch.arange(0, dim, 2, dtype=torch.int64).float() / dim))
    if spec.rope_scaling is None:
        return inv
    kind, factor, low, high, original = spec.rope_scaling
    if kind != "llama3":
        raise ValueError(f"rope scaling {kind!r} is not covered")
    low_wavelen = original / low
    high_wavelen = original / high
    wavelen = 2 * math.pi / inv
    scaled = torch.where(wavelen > low_wavelen, inv / factor, inv)
    smooth = (original / wavelen - low) / (high - low)
    smoothed = (1 - smooth) * scaled / factor + smooth * scaled
    medium = ~(wavelen < high_wavelen) * ~(wavelen > low_wavelen)
    return torch.where(medium, smoothed, scaled)


def inv_freq_buffer(spec: ModelSpec, device: str | torch.device = "cpu") -> torch.Tensor:
    """The rotary buffer as a bf16-cast model holds it."""
    return inverse_frequencies(spec).to(torch.bfloat16).to(device)


# ---------------------------------------------------------------------------------------
# Direct program (explicit tensors, no Dynamo): argument order is
#   input_ids, position_ids, [key_cache, value_cache, valid_length] per layer, inv_freq,
#   then the weights in parameter_shapes() order.
# ---------------------------------------------------------------------------------------
def direct_arguments(spec: ModelSpec, weights: dict[str, torch.Tensor], inv_freq: torch.Tensor,
                     input_ids: torch.Tensor, position_ids: torch.Tensor,
                     state: list[torch.Tensor]) -> list[torch.Tensor]:
    return [input_ids, position_ids, *state, inv_freq,
            *[weights[name] for name, _ in parameter_shapes(spec)]]


def direct_program(spec: ModelSpec, batch: int, capacity: int,
                   per_row_lengths: bool = False) -> DecoderProgram:
    names = [name for name, _ in parameter_shapes(spec)]
    base = 2 + 3 * spec.layers + 1
    where = {name: base + index for index, name in enumerate(names)}
    layers = []
    for index in range(spec.layers):
        prefix = f"model.layers.{index}."
        layers.append(LayerBinding(
            input_norm=where[prefix + "input_layernorm.weight"],
            q_weight=where[prefix + "self_attn.q_proj.weight"],
            k_weight=where[prefix + "self_attn.k_proj.weight"],
            v_weight=where[prefix + "self_attn.v_proj.weight"],
            o_weight=where[prefix + "self_attn.o_proj.weight"],
            post_norm=where[prefix + "post_attention_layernorm.weight"],
            gate_weight=where[prefix + "mlp.gate_proj.weight"],
            up_weight=where[prefix + "mlp.up_proj.weight"],
            down_weight=where[prefix + "mlp.down_proj.weight"],
            key_cache=2 + 3 * index,
            value_cache=3 + 3 * index,
            valid_length=4 + 3 * index,
            q_bias=where.get(prefix + "self_attn.q_proj.bias"),
            k_bias=where.get(prefix + "self_attn.k_proj.bias"),
            v_bias=where.get(prefix + "self_attn.v_proj.bias"),
        ))
    return DecoderProgram(
        mode="decode", batch=batch, tokens=1, hidden=spec.hidden, heads=spec.heads,
        kv_heads=spec.kv_heads, head_dim=spec.head_dim, intermediate=spec.intermediate,
        vocab=spec.vocab, capacity=capacity, norm=spec.norm, eps=spec.eps,
        activation=spec.activation, embed_scale=spec.embed_scale, rope_scale=1.0, q_scale=None,
        softmax_scale=spec.head_dim**-0.5, inv_freq_dtype="bf16",
        input_ids=0, position_ids=1, embed_weight=where["model.embed_tokens.weight"],
        inv_freq=2 + 3 * spec.layers, final_norm=where["model.norm.weight"],
        lm_head_weight=where["model.embed_tokens.weight"], layers=tuple(layers),
        length_count=batch if per_row_lengths else 1,
    )


def direct_prefill_arguments(spec: ModelSpec, weights: dict[str, torch.Tensor],
                             inv_freq: torch.Tensor, input_ids: torch.Tensor) -> list[torch.Tensor]:
    """Argument list of ``direct_prefill_program``: input_ids, inv_freq, then the weights."""
    return [input_ids, inv_freq, *[weights[name] for name, _ in parameter_shapes(spec)]]


def direct_prefill_program(spec: ModelSpec, batch: int, tokens: int) -> DecoderProgram:
    """Causal prefill of ``[batch, tokens]`` ids at positions 0..tokens-1 (held by the plan)."""
    names = [name for name, _ in parameter_shapes(spec)]
    where = {name: 2 + index for index, name in enumerate(names)}
    layers = []
    for index in range(spec.layers):
        prefix = f"model.layers.{index}."
        layers.append(LayerBinding(
            input_norm=where[prefix + "input_layernorm.weight"],
            q_weight=where[prefix + "self_attn.q_proj.weight"],
            k_weight=where[prefix + "self_attn.k_proj.weight"],
            v_weight=where[prefix + "self_attn.v_proj.weight"],
            o_weight=where[prefix + "self_attn.o_proj.weight"],
            post_norm=where[prefix + "post_attention_layernorm.weight"],
            gate_weight=where[prefix + "mlp.gate_proj.weight"],
            up_weight=where[prefix + "mlp.up_proj.weight"],
            down_weight=where[prefix + "mlp.down_proj.weight"],
            key_cache=-1, value_cache=-1, valid_length=-1,
            q_bias=where.get(prefix + "self_attn.q_proj.bias"),
            k_bias=where.get(prefix + "self_attn.k_proj.bias"),
            v_bias=where.get(prefix + "self_attn.v_proj.bias"),
        ))
    return DecoderProgram(
        mode="prefill", batch=batch, tokens=tokens, hidden=spec.hidden, heads=spec.heads,
        kv_heads=spec.kv_heads, head_dim=spec.head_dim, intermediate=spec.intermediate,
        vocab=spec.vocab, capacity=0, norm=spec.norm, eps=spec.eps,
        activation=spec.activation, embed_scale=spec.embed_scale, rope_scale=1.0, q_scale=None,
        softmax_scale=spec.head_dim**-0.5, inv_freq_dtype="bf16",
        input_ids=0, position_ids=None, embed_weight=where["model.embed_tokens.weight"],
        inv_freq=1, final_norm=where["model.norm.weight"],
        lm_head_weight=where["model.embed_tokens.weight"], layers=tuple(layers), causal=True,
    )


def make_state(spec: ModelSpec, batch: int, capacity: int, device: str | torch.device = "cpu",
               per_row_lengths: bool = False) -> list[torch.Tensor]:
    """Zeroed ``[key_cache, value_cache, valid_length]`` per layer; one valid length shared by
    the batch, or one per row."""
    state = []
    for _ in range(spec.layers):
        shape = (batch, capacity, spec.kv_heads, spec.head_dim)
        state.append(torch.zeros(shape, dtype=torch.bfloat16, device=device))
        state.append(torch.zeros(shape, dtype=torch.bfloat16, device=device))
        state.append(torch.zeros(batch if per_row_lengths else 1, dtype=torch.int32, device=device))
    return state


# ---------------------------------------------------------------------------------------
# Hugging Face modules with the same weights (for the make_backend / torch.compile path)
# ---------------------------------------------------------------------------------------
def hf_config(spec: ModelSpec):
    common = dict(
        hidden_size=spec.hidden, intermediate_size=spec.intermediate,
        num_attention_heads=spec.heads, num_key_value_heads=spec.kv_heads,
        num_hidden_layers=spec.layers, vocab_size=spec.vocab, rms_norm_eps=spec.eps,
        max_position_embeddings=spec.max_positions, tie_word_embeddings=True,
    )
    rope: dict = {"rope_type": "default", "rope_theta": spec.rope_theta}
    if spec.rope_scaling is not None:
        kind, factor, low, high, original = spec.rope_scaling
        rope = {"rope_type": kind, "rope_theta": spec.rope_theta, "factor": factor,
                "low_freq_factor": low, "high_freq_factor": high,
                "original_max_position_embeddings": original}
    if spec.family == "llama":
        from transformers import LlamaConfig
        return LlamaConfig(head_dim=spec.head_dim, rope_parameters=rope, **common)
    if spec.family == "qwen2":
        from transformers import Qwen2Config
        return Qwen2Config(rope_parameters=rope, **common)
    if spec.family == "gemma":
        from transformers import GemmaConfig
        return GemmaConfig(head_dim=spec.head_dim, hidden_act="gelu_pytorch_tanh",
                           hidden_activation="gelu_pytorch_tanh", rope_parameters=rope, **common)
    raise ValueError(spec.family)


def build_hf_model(spec: ModelSpec, seed: int = 0, device: str | torch.device = "cpu",
                   weights: dict[str, torch.Tensor] | None = None):
    """A bf16 Hugging Face causal LM of the spec's shape carrying ``init_weights(spec, seed)``."""
    from transformers import AutoModelForCausalLM

    config = hf_config(spec)
    with torch.device("meta"):
        model = AutoModelForCausalLM.from_config(config)
    model = model.to(torch.bfloat16).to_empty(device=device)
    weights = weights if weights is not None else init_weights(spec, seed, device)
    with torch.no_grad():
        for name, parameter in model.named_parameters():
            if name == "lm_head.weight":
                continue
            parameter.copy_(weights[name])
        model.tie_weights()
        rotary = model.model.rotary_emb
        rotary.inv_freq = inv_freq_buffer(spec, device)
        if hasattr(rotary, "original_inv_freq"):
            rotary.original_inv_freq = rotary.inv_freq
        scale = getattr(model.model.embed_tokens, "embed_scale", None)
        if scale is not None:
            model.model.embed_tokens.embed_scale = torch.tensor(
                spec.hidden**0.5, device=device).to(torch.bfloat16)
    model.config.use_cache = False
    return model.eval()


# ---------------------------------------------------------------------------------------
# Cache filling for long-context decode workloads (input preparation, never timed)
# ---------------------------------------------------------------------------------------
@torch.no_grad()
def fill_cache_by_prefill(spec: ModelSpec, weights: dict[str, torch.Tensor],
                          inv_freq: torch.Tensor, state: list[torch.Tensor], keys: int,
                          seed: int = 0, chunk_rows: int = 2) -> None:
    """Fill ``state`` with the keys (after RoPE) and values of a seeded causal prefill of ``keys``
    uniform-random token ids per row, and set every valid length to ``keys``.

    Plain library torch on the tensors' device (fused SDPA for the attention itself): this
    prepares the benchmark's *input*, the same tensors then go to the kernel and to the CPU
    baseline.  Rows are processed ``chunk_rows`` at a time to bound memory."""
    device = state[0].device
    batch = state[0].shape[0]
    ids = torch.randint(0, spec.vocab, (batch, keys), generator=torch.Generator().manual_seed(seed))
    positions = torch.arange(keys, device=device, dtype=torch.float32)
    freqs = torch.outer(positions, inv_freq.to(device).float())
    emb = torch.cat((freqs, freqs), dim=-1)
    cos, sin = emb.cos().to(torch.bfloat16)[None, :, None], emb.sin().to(torch.bfloat16)[None, :, None]

    def rope(x):
        half = x.shape[-1] // 2
        return x * cos + torch.cat((-x[..., half:], x[..., :half]), dim=-1) * sin

    def norm(x, w):
        wide = x.float()
        scaled = wide * torch.rsqrt(wide.pow(2).mean(-1, keepdim=True) + spec.eps)
        if spec.norm == "gemma":
            return (scaled * (1.0 + w.float())).to(x.dtype)
        return w * scaled.to(x.dtype)

    lin = torch.nn.functional.linear
    for start in range(0, batch, chunk_rows):
        rows = slice(start, min(batch, start + chunk_rows))
        hidden = torch.nn.functional.embedding(ids[rows].to(device), weights["model.embed_tokens.weight"])
        if spec.embed_scale is not None:
            hidden = hidden * torch.tensor(spec.embed_scale, dtype=hidden.dtype, device=device)
        n = hidden.shape[0]
        for index in range(spec.layers):
            pre = f"model.layers.{index}."
            x = norm(hidden, weights[pre + "input_layernorm.weight"])
            q = lin(x, weights[pre + "self_attn.q_proj.weight"], weights.get(pre + "self_attn.q_proj.bias"))
            k = lin(x, weights[pre + "self_attn.k_proj.weight"], weights.get(pre + "self_attn.k_proj.bias"))
            v = lin(x, weights[pre + "self_attn.v_proj.weight"], weights.get(pre + "self_attn.v_proj.bias"))
            q = rope(q.view(n, keys, spec.heads, spec.head_dim))
            k = rope(k.view(n, keys, spec.kv_heads, spec.head_dim))
            v = v.view(n, keys, spec.kv_heads, spec.head_dim)
            state[3 * index][rows, :keys] = k
            state[3 * index + 1][rows, :keys] = v
            mixed = torch.nn.functional.scaled_dot_product_attention(
                q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True,
                enable_gqa=spec.heads != spec.kv_heads)
            mixed = mixed.transpose(1, 2).reshape(n, keys, spec.heads * spec.head_dim)
            hidden = hidden + lin(mixed, weights[pre + "self_attn.o_proj.weight"])
            x = norm(hidden, weights[pre + "post_attention_layernorm.weight"])
            gate = lin(x, weights[pre + "mlp.gate_proj.weight"])
            act = (torch.nn.functional.silu(gate) if spec.activation == "silu"
                   else torch.nn.functional.gelu(gate, approximate="tanh"))
            hidden = hidden + lin(act * lin(x, weights[pre + "mlp.up_proj.weight"]),
                                  weights[pre + "mlp.down_proj.weight"])
    for index in range(spec.layers):
        state[3 * index + 2].fill_(keys)
