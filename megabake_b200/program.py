"""What the recogniser hands the planner: a decoder invocation described by its shapes,
numerics switches and *where each tensor comes from* (argument positions of the captured
graph), never by tensor values.

``DecoderProgram`` is deliberately small: every decoder family this backend covers (Llama,
Qwen2, Gemma, SmolLM shapes; MHA / GQA / MQA) is the same sequence of regions

    [embed] -> { rmsnorm -> q|k|v (+bias) -> rope -> kv attention -> o_proj + residual ->
                 rmsnorm -> gate|up -> act * up -> down + residual }* -> rmsnorm -> lm head

and differs only in the switches below.  The planner packs those regions into barrier
intervals; nothing else of the FX graph survives recognition.
"""

from __future__ import annotations

from dataclasses import dataclass, field


@dataclass(frozen=True)
class LayerBinding:
    """Argument positions of one decoder layer's tensors (None = absent)."""

    input_norm: int
    q_weight: int
    k_weight: int
    v_weight: int
    o_weight: int
    post_norm: int
    gate_weight: int
    up_weight: int
    down_weight: int
    key_cache: int
    value_cache: int
    valid_length: int
    q_bias: int | None = None
    k_bias: int | None = None
    v_bias: int | None = None
    o_bias: int | None = None
    gate_bias: int | None = None
    up_bias: int | None = None
    down_bias: int | None = None


@dataclass(frozen=True)
class DecoderProgram:
    mode: str  # "decode" | "prefill"
    batch: int
    tokens: int  # query positions per row (1 for decode)
    hidden: int
    heads: int
    kv_heads: int
    head_dim: int
    intermediate: int
    vocab: int
    capacity: int  # KV capacity (decode); 0 for prefill
    norm: str  # "llama": w * bf16(x * r)   |  "gemma": bf16(x * r * (1 + w))
    eps: float
    activation: str  # "silu" | "gelu_tanh"
    embed_scale: float | None  # bf16 scalar multiplied into the embedding rows (Gemma)
    rope_scale: float  # attention_scaling multiplied into cos / sin
    q_scale: float | None  # extra scale folded into q after RoPE (None = none)
    softmax_scale: float
    inv_freq_dtype: str  # "bf16" | "f32"
    input_ids: int
    position_ids: int | None  # None (prefill only): positions 0..tokens-1, held by the plan
    embed_weight: int
    inv_freq: int
    final_norm: int
    lm_head_weight: int
    layers: tuple[LayerBinding, ...] = field(default_factory=tuple)
    lm_head_bias: int | None = None
    embed_scale_arg: int | None = None  # graph input holding the embedding scale (read at bind)
    length_count: int = 1  # valid lengths per layer: 1 (shared by the batch) or ``batch``
    causal: bool = True  # prefill mask kind
    mask: object = field(default=None, compare=False, repr=False)  # additive bf16 mask tensor of a
    # non-causal prefill, [1 or batch, 1, tokens, tokens]

    @property
    def group(self) -> int:
        return self.heads // self.kv_heads

    def weight_bytes(self) -> int:
        """Bytes of weights one decode step must read (the algorithmic figure of the
        HBM roofline): every projection once, the LM head once, norm vectors."""
        h, d = self.hidden, self.head_dim
        per_layer = (self.heads * d * h + 2 * self.kv_heads * d * h + h * self.heads * d
                     + 3 * h * self.intermediate + 2 * h)
        return 2 * (len(self.layers) * per_layer + self.vocab * h + h)

    def kv_bytes_per_key(self) -> int:
        """KV-cache bytes per cached key per batch row, all layers."""
        return 2 * len(self.layers) * self.kv_heads * self.head_dim * 2
