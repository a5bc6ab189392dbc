"""Execution planner: packs a ``DecoderProgram`` into phases and emits the phase records +
address-table layout of the C ABI.

Decode packing (five phases per layer; the activations between them travel as flagged cells,
so no grid barrier separates them -- a consumer polls the very cells it needs and starts on
them as soon as their producers have stored them):

    [embed gather (layer 0) . rmsnorm . q|k|v (+bias)]          -> q, k, v cells
    [rope(q, new k) . kv append . split-key attention . merge]   -> attention cells
    [o_proj + residual]                                          -> hidden cells (buffer B)
    [rmsnorm . gate|up . act(gate) * up]                         -> gated cells
    [down + residual]                                            -> hidden cells (A or C)   x layers
    [rmsnorm . lm head]                                          -> logits (plain bf16)

The kernel keeps its CTAs within two phases of one another, so a cell buffer may be rewritten
from the third phase after its last reader on.  Every buffer is five phases apart from itself
except the residual stream, which o_proj reads (as the residual) three phases after ``down`` of
the layer before wrote it: it rotates through three buffers -- a layer reads its input from A
(even layers) or C (odd layers), o_proj writes B, ``down`` writes the other of A and C.  The
valid lengths are advanced when the launch ends.

RMSNorm, the embedding gather, RoPE, bias, residual adds and the gated activation never get
an interval of their own: they are folded into the consumer's prologue (recomputed by every
CTA, the rows are tiny) or the producer's epilogue.  That is the 5-intervals-per-layer
shape the reference's schedule reaches with interval folding
(``src/megabake/schedule.py:1220-1245,1298-1409``; ``docs/roadmap.md:56-59``), with the gate/up
pair fused (the reference's sm100 provider cannot, ``bodies/cuda/sm100/table.py:28-30``) and
the embedding + RoPE-table intervals removed.

The planner runs without a GPU (it only asks the native library for its shared-memory
constants), so the tables are unit-testable on CPU.
"""

from __future__ import annotations

import math
import os
from dataclasses import dataclass, field

from . import runtime as rt
from .diagnostics import fail
from .program import DecoderProgram

DYN_INPUT_IDS, DYN_POSITION_IDS, DYN_LOGITS = 0, 1, 2
N_DYNAMIC = 3
CONSUMER_WARPS = 8
EXACT_SOFTMAX_KEYS = 128  # contexts up to here use the reference-rounding softmax (one CTA)
MAX_GEMV_ROWS = 8
# Activations that EVERY CTA reads whole (the input rows of a skinny GEMM) stay plain bf16: their
# producers fence and report the phase finished, a consumer waits on that one counter and fetches
# the rows with bulk copies -- measured on B200, the copy engine brings 14-78 KB per CTA into
# shared memory in about a microsecond, where polling as many flagged cells with ordinary loads
# took 5-13.  Flagged cells carry what a consumer reads a FEW rows of: q, k and v on their way to
# the attention items (always), and GEMV inputs up to this many bytes per CTA (0: none).
CELL_LIMIT_BYTES = 0


@dataclass(frozen=True)
class SlotSpec:
    kind: str  # "dynamic" | "arg" | "workspace" | "constant" (tensor in PlanLayout.constants)
    index: int = 0  # argument position, or dynamic ordinal
    offset: int = 0  # byte offset into the workspace
    name: str = ""


@dataclass
class PlanLayout:
    program: DecoderProgram
    phases: list[rt.Phase]
    slots: list[SlotSpec]
    workspace_bytes: int
    zero_ranges: list[tuple[int, int]]  # workspace byte ranges that must start zeroed
    activation_bytes: int
    intervals: int
    notes: list[str] = field(default_factory=list)
    mode: int = rt.MODE_DECODE
    stage_bytes: int = 0  # decode: weight-ring stage size handed to mb_plan_create (0 = default)
    constants: dict = field(default_factory=dict)  # name -> CPU tensor uploaded at bind


@dataclass(frozen=True)
class PlannerOptions:
    ctas: int = 148  # CTAs the tile split is planned for (one per SM on B200)
    row_tile: int | None = None  # force the GEMV row tile (tuning sweeps)
    max_chunks: int = 32
    merge_slots: int | None = None
    exact_keys: int = EXACT_SOFTMAX_KEYS
    stage_bytes: int | None = None  # force the ring stage size (tuning sweeps)
    cell_limit: int = CELL_LIMIT_BYTES  # largest per-CTA copy of an activation kept as cells
    qkv_cells: bool = True  # q, k and v reach the attention items as flagged cells
    distinct_buffers: bool = False  # every layer gets activation buffers of its own (race check:
    #                                 the results must not depend on the buffers being reused)

    @classmethod
    def resolve(cls, program, device_index: int | None = None, **overrides) -> "PlannerOptions":
        """Options for one program: defaults, then the tuning file's choice for this model shape
        and device (``cache.tuned_choice``), then the sweep variables of ``from_env``, then
        ``overrides``."""
        from .cache import tuned_choice

        values = dict(tuned_choice(program, device_index))
        values.update(cls._env_values())
        values.update(overrides)
        return cls(**values)

    @staticmethod
    def _env_values() -> dict:
        values = {}
        if os.environ.get("MEGABAKE_B200_ROW_TILE"):
            values["row_tile"] = int(os.environ["MEGABAKE_B200_ROW_TILE"])
        if os.environ.get("MEGABAKE_B200_STAGE_BYTES"):
            values["stage_bytes"] = int(os.environ["MEGABAKE_B200_STAGE_BYTES"])
        if os.environ.get("MEGABAKE_B200_CELL_LIMIT"):
            values["cell_limit"] = int(os.environ["MEGABAKE_B200_CELL_LIMIT"])
        if os.environ.get("MEGABAKE_B200_QKV_CELLS"):
            values["qkv_cells"] = os.environ["MEGABAKE_B200_QKV_CELLS"] != "0"
        return values

    @classmethod
    def from_env(cls, **overrides) -> "PlannerOptions":
        """Defaults plus the sweep variables (``MEGABAKE_B200_STAGE_BYTES`` ...): for tuning runs
        that compare settings inside one process; measured choices belong in the tuning file."""
        values = cls._env_values()
        values.update(overrides)
        return cls(**values)


def _align(value: int, to: int) -> int:
    return (value + to - 1) // to * to


class _Slots:
    def __init__(self):
        self.specs: list[SlotSpec] = [
            SlotSpec("dynamic", DYN_INPUT_IDS, name="input_ids"),
            SlotSpec("dynamic", DYN_POSITION_IDS, name="position_ids"),
            SlotSpec("dynamic", DYN_LOGITS, name="logits"),
        ]
        self._args: dict[int, int] = {}
        self.workspace = 0
        self.zero: list[tuple[int, int]] = []

    def arg(self, position: int | None, name: str = "") -> int:
        if position is None:
            return -1
        if position not in self._args:
            self._args[position] = len(self.specs)
            self.specs.append(SlotSpec("arg", position, name=name))
        return self._args[position]

    def buffer(self, nbytes: int, name: str, zero: bool = False) -> int:
        offset = _align(self.workspace, 256)
        self.workspace = offset + nbytes
        if zero:
            self.zero.append((offset, nbytes))
        self.specs.append(SlotSpec("workspace", offset=offset, name=name))
        return len(self.specs) - 1

    def constant(self, name: str) -> int:
        self.specs.append(SlotSpec("constant", name=name))
        return len(self.specs) - 1


ROW_TILE = 8  # weight rows per pipeline stage (one n8 MMA tile); a consumer warp owns a block


def gemv_geometry(n_total: int, k: int, nmat: int, ctas: int, stage_bytes: int, row_pad: int,
                  forced_row_tile: int | None = None) -> tuple[int, int]:
    """(row_tile, k_chunk) of a skinny-GEMM phase.

    A CTA owns ``ceil(n_total / ctas)`` consecutive weight rows and streams them as blocks of
    8 rows; a block is cut along K into equal chunks (multiples of 32 elements, preferably of
    64 so that staged rows stay bank-staggered) that fit one ring stage together with the
    paired matrix.  Whole rows per copy whenever they fit: the bulk-copy engine is at its best
    from 2 KB per copy upwards.

    Rows of at most 1,024 elements (Qwen2-0.5B, SmolLM-135M) would leave a stage half empty,
    and with three stages per SM too few bytes in flight to cover the HBM latency: a plain
    (unpaired) phase then stages 16 rows, two MMA tiles, per stage.
    """
    del n_total, ctas
    tile = ROW_TILE
    if forced_row_tile in (ROW_TILE, 2 * ROW_TILE) and nmat == 1:
        tile = forced_row_tile
    elif nmat == 1 and 2 * ROW_TILE * (k * 2 + row_pad) <= stage_bytes:
        tile = 2 * ROW_TILE
    limit = ((stage_bytes // (tile * nmat)) - row_pad) // 2 // 32 * 32
    if limit < 32:
        fail("resource-admission", f"a ring stage cannot hold {tile} rows of {nmat} matrices")
    chunks = math.ceil(k / min(limit, k))
    k_chunk = _align(math.ceil(k / chunks), 64)
    if k_chunk > limit:
        k_chunk = _align(math.ceil(k / chunks), 32)
    while k_chunk > limit:
        chunks += 1
        k_chunk = _align(math.ceil(k / chunks), 32)
    return tile, min(k_chunk, k)


def attention_state_bytes(head_dim: int, group: int, merge_slots: int) -> int:
    """Query rows, new K/V rows, tables, statistics and head states of the decode attention
    body (mirrors the native layout)."""
    stats = 4 * (2 * 8 * 8 + 8 * 64 + 16)
    return (16 * (head_dim + 32) + 4 * head_dim + 4 * head_dim + stats
            + 4 * (head_dim + 2) * group * (merge_slots + 2))


def attention_staging_bytes(head_dim: int) -> int:
    """Per-warp K/V tile slots of the split-key loop (64-wide heads only): 8 warps x 2 slots x
    16 keys x (a K row padded by 64 B + a V row padded by 16 B)."""
    if head_dim != 64:
        return 0
    return CONSUMER_WARPS * 2 * 16 * ((head_dim * 2 + 64) + (head_dim * 2 + 16))


def attention_merge_slots(head_dim: int, group: int, wanted: int = CONSUMER_WARPS) -> int:
    """Per-warp states merged at once: as many as keep the state area within 48 KB."""
    slots = wanted
    while slots > 1 and attention_state_bytes(head_dim, group, slots) > 48 * 1024:
        slots //= 2
    return slots


def attention_scratch_bytes(head_dim: int, group: int, merge_slots: int) -> int:
    """Shared-memory scratch of the decode attention body."""
    return attention_state_bytes(head_dim, group, merge_slots) + attention_staging_bytes(head_dim)


def exact_softmax_keys(capacity: int, limit: int = EXACT_SOFTMAX_KEYS) -> int:
    return min(capacity, limit, 128)


def _check_program(p: DecoderProgram) -> None:
    if p.mode != "decode":
        fail("planning", f"plan_decode got a {p.mode!r} program")
    if p.tokens != 1:
        fail("planning", "decode plans take one token per row")
    if not 1 <= p.batch <= MAX_GEMV_ROWS:
        fail("resource-admission", f"decode batch {p.batch} outside 1..{MAX_GEMV_ROWS}",
             requirement="batch <= 8 rows per GPU")
    if p.head_dim not in (64, 128, 256):
        fail("resource-admission", f"head_dim {p.head_dim} not in (64, 128, 256)")
    if p.heads % p.kv_heads or p.group > 8:
        fail("resource-admission",
             f"{p.heads} query heads over {p.kv_heads} kv heads (group size must divide, <= 8)")
    for name, value in (("hidden", p.hidden), ("intermediate", p.intermediate)):
        if value % 32:
            fail("resource-admission", f"{name} size {value} is not a multiple of 32")
    if p.norm not in ("llama", "gemma"):
        fail("planning", f"unknown norm kind {p.norm!r}")
    if p.activation not in ("silu", "gelu_tanh"):
        fail("planning", f"unknown activation {p.activation!r}")


def plan_decode(program: DecoderProgram, options: PlannerOptions | None = None) -> PlanLayout:
    """Plan one decode step.  The ring stage size is the library's largest unless forced:
    measured on B200, smaller stages (a deeper ring) never paid -- the consumers' per-stage
    work, not the bytes in flight, bounds the weight stream."""
    options = options or PlannerOptions.resolve(program)
    largest = rt.load_library().mb_stage_bytes(rt.MODE_DECODE)
    return _plan_decode(program, options, options.stage_bytes or largest)


def _plan_decode(program: DecoderProgram, options: PlannerOptions, stage_bytes: int) -> PlanLayout:
    _check_program(program)
    lib = rt.load_library()
    fixed_bytes = lib.mb_fixed_smem_bytes(rt.MODE_DECODE)
    max_smem = lib.mb_max_smem_bytes()
    row_pad = 64
    p = program
    B, H, D = p.batch, p.hidden, p.head_dim
    q_dim, kv_dim = p.heads * D, p.kv_heads * D
    slots = _Slots()
    pro = rt.PRO_RMS_LLAMA if p.norm == "llama" else rt.PRO_RMS_GEMMA
    act = rt.EPI_SILU_MUL if p.activation == "silu" else rt.EPI_GELU_TANH_MUL

    # activations between phases: flagged cells, 8 bytes per pair of bf16 values, zero at first
    hidden_a = slots.buffer(B * H * 4, "hidden_a", zero=True)
    hidden_b = slots.buffer(B * H * 4, "hidden_b", zero=True)
    hidden_c = slots.buffer(B * H * 4, "hidden_c", zero=True)
    q_buf = slots.buffer(B * q_dim * 4, "q", zero=True)
    k_buf = slots.buffer(B * kv_dim * 4, "k", zero=True)
    v_buf = slots.buffer(B * kv_dim * 4, "v", zero=True)
    attn = slots.buffer(B * q_dim * 4, "attention", zero=True)
    glu = slots.buffer(B * p.intermediate * 4, "gated", zero=True)
    max_chunks = max(1, min(options.max_chunks, math.ceil(p.capacity / 16)))
    pairs = B * p.kv_heads
    partial = slots.buffer(pairs * max_chunks * p.group * (D + 2) * 4, "attention_partials")
    counters = slots.buffer(_align(pairs * 4, 16), "attention_arrivals", zero=True)

    merge_slots = options.merge_slots or CONSUMER_WARPS
    exact_keys = exact_softmax_keys(p.capacity, options.exact_keys)
    merge_slots = attention_merge_slots(D, p.group, merge_slots)
    activation = attention_scratch_bytes(D, p.group, merge_slots)

    phases: list[rt.Phase] = []
    if options.distinct_buffers:
        shared = dict(hidden_a=hidden_a, hidden_b=hidden_b, hidden_c=hidden_c, q=q_buf, k=k_buf,
                      v=v_buf, attention=attn, gated=glu)
        widths = dict(hidden_a=H, hidden_b=H, hidden_c=H, q=q_dim, k=kv_dim, v=kv_dim,
                      attention=q_dim, gated=p.intermediate)

    def layer_buffers(index: int):
        """The activation buffers layer ``index`` works in: the shared set, or its own."""
        if not options.distinct_buffers or index == 0:
            return hidden_a, hidden_b, hidden_c, q_buf, k_buf, v_buf, attn, glu
        own = {name: slots.buffer(B * widths[name] * 4, f"{name}.{index}", zero=True)
               for name in shared}
        return (own["hidden_a"], own["hidden_b"], own["hidden_c"], own["q"], own["k"], own["v"],
                own["attention"], own["gated"])

    def as_cells(width: int) -> bool:
        return B * width * 4 <= options.cell_limit

    def gemv(*, k, segments, x_slot, prologue=rt.PRO_NONE, norm_slot=-1, epilogue=rt.EPI_NONE,
             pair_slot=-1, residual_slot=-1, gather=False, store_x=-1, x_source=-1,
             residual_source=-1, out_cells=True, out_fenced=False, x_cells=True,
             residual_cells=True, store_x_cells=True):
        """``x_source`` / ``residual_source``: index of the phase that wrote that operand earlier
        in the launch (-1: it comes from outside).  ``*_cells``: the operand is flagged cells
        (else plain bf16, whose producing phase fences: ``out_fenced``).  Returns the index of
        the new phase."""
        nonlocal activation
        n_total = sum(n for n, _, _, _ in segments)
        nmat = 2 if pair_slot >= 0 else 1
        row_tile, k_chunk = gemv_geometry(n_total, k, nmat, options.ctas, stage_bytes, row_pad,
                                          options.row_tile)
        phase = rt.Phase.blank(rt.BODY_GEMV, rt.FLAG_FENCE if out_fenced else 0)
        cells = rt.CELLS_OUT if out_cells else 0
        if x_source >= 0:
            cells |= rt.CELLS_X_WAIT | (rt.CELLS_X if x_cells else 0)
            phase.i[rt.GV_I_X_SOURCE] = x_source
        if residual_source >= 0 and residual_cells:
            cells |= rt.CELLS_RESIDUAL
            phase.i[rt.GV_I_RES_SOURCE] = residual_source
        if store_x >= 0 and store_x_cells:
            cells |= rt.CELLS_XSTORE
        phase.i[rt.GV_I_CELLS] = cells
        phase.i[rt.GV_I_ROWS] = B
        phase.i[rt.GV_I_K] = k
        phase.i[rt.GV_I_NSEG] = len(segments)
        phase.i[rt.GV_I_NMAT] = nmat
        phase.i[rt.GV_I_PROLOGUE] = prologue
        phase.i[rt.GV_I_EPILOGUE] = epilogue
        phase.i[rt.GV_I_ROW_TILE] = row_tile
        phase.i[rt.GV_I_K_CHUNK] = k_chunk
        phase.f[rt.GV_F_EPS] = p.eps
        phase.slot[rt.GV_S_X] = x_slot
        phase.slot[rt.GV_S_NORM_W] = norm_slot
        for index, (n, weight, bias, out) in enumerate(segments):
            phase.i[rt.GV_I_N0 + index] = n
            phase.slot[rt.GV_S_W0 + index] = weight
            phase.slot[rt.GV_S_BIAS0 + index] = bias
            phase.slot[rt.GV_S_OUT0 + index] = out
        phase.slot[rt.GV_S_W_PAIR] = pair_slot
        phase.slot[rt.GV_S_RESIDUAL] = residual_slot
        if gather:
            phase.i[rt.GV_I_GATHER] = 1
            phase.i[rt.GV_I_VOCAB] = p.vocab
            phase.f[rt.GV_F_EMBED_SCALE] = float(p.embed_scale or 0.0)
            phase.slot[rt.GV_S_IDS] = DYN_INPUT_IDS
            if store_x >= 0:
                phase.i[rt.GV_I_STORE_X] = 1
                phase.slot[rt.GV_S_XSTORE] = store_x
        staged_rows = B + (1 if prologue != rt.PRO_NONE else 0)  # + the norm weight row
        activation = max(activation, staged_rows * (k + 32) * 2)
        phases.append(phase)
        return len(phases) - 1

    inv_freq = slots.arg(p.inv_freq, "inv_freq")
    embed = slots.arg(p.embed_weight, "embed_tokens.weight")
    hidden_source = 0  # phase that last wrote the residual stream (buffer A): the gather
    stream = hidden_a  # the buffer that holds the residual stream at the start of a layer
    hidden_cells, attn_cells, glu_cells = as_cells(H), as_cells(q_dim), as_cells(p.intermediate)
    qkv_cells = options.qkv_cells
    for index, layer in enumerate(p.layers):
        tag = f"layers.{index}."
        first = index == 0
        if options.distinct_buffers:
            # the layer reads what the previous layer's `down` wrote and writes buffers of its own
            _, hidden_b, layer_out, q_buf, k_buf, v_buf, attn, glu = layer_buffers(index + 1)
            layer_in = stream
        else:
            layer_in, layer_out = (hidden_a, hidden_c) if index % 2 == 0 else (hidden_c, hidden_a)
        stream_in, stream = layer_in, layer_out
        qkv_phase = gemv(
            k=H,
            segments=[
                (q_dim, slots.arg(layer.q_weight, tag + "q_proj.weight"),
                 slots.arg(layer.q_bias, tag + "q_proj.bias"), q_buf),
                (kv_dim, slots.arg(layer.k_weight, tag + "k_proj.weight"),
                 slots.arg(layer.k_bias, tag + "k_proj.bias"), k_buf),
                (kv_dim, slots.arg(layer.v_weight, tag + "v_proj.weight"),
                 slots.arg(layer.v_bias, tag + "v_proj.bias"), v_buf),
            ],
            x_slot=embed if first else layer_in,
            x_source=-1 if first else hidden_source,
            x_cells=hidden_cells,
            prologue=pro,
            norm_slot=slots.arg(layer.input_norm, tag + "input_layernorm.weight"),
            gather=first,
            store_x=stream_in if first else -1,
            store_x_cells=hidden_cells,
            out_cells=qkv_cells,
            # fenced for plain q, k, v and for the gathered rows stored plain
            out_fenced=not qkv_cells or (first and not hidden_cells),
        )
        attention = rt.Phase.blank(rt.BODY_ATTN_DECODE, rt.FLAG_BUMP_LENGTH
                                   | (0 if attn_cells else rt.FLAG_FENCE))
        attention.i[rt.AT_I_BATCH] = B
        attention.i[rt.AT_I_HEADS] = p.heads
        attention.i[rt.AT_I_KV_HEADS] = p.kv_heads
        attention.i[rt.AT_I_HEAD_DIM] = D
        attention.i[rt.AT_I_CAPACITY] = p.capacity
        attention.i[rt.AT_I_INVFREQ_BF16] = 1 if p.inv_freq_dtype == "bf16" else 0
        attention.i[rt.AT_I_MAX_CHUNKS] = max_chunks
        attention.i[rt.AT_I_MERGE_SLOTS] = merge_slots
        attention.i[rt.AT_I_EXACT_KEYS] = exact_keys
        attention.i[rt.AT_I_CELLS] = ((rt.CELLS_X if qkv_cells else rt.CELLS_X_WAIT)
                                      | (rt.CELLS_OUT if attn_cells else 0))
        attention.i[rt.AT_I_QKV_SOURCE] = qkv_phase
        attention.i[rt.AT_I_LEN_COUNT] = p.length_count
        attention.f[rt.AT_F_SCALE] = p.softmax_scale
        attention.f[rt.AT_F_ROPE_SCALE] = p.rope_scale
        attention.f[rt.AT_F_Q_SCALE] = float(p.q_scale or 0.0)
        attention.slot[rt.AT_S_Q] = q_buf
        attention.slot[rt.AT_S_K] = k_buf
        attention.slot[rt.AT_S_V] = v_buf
        attention.slot[rt.AT_S_KCACHE] = slots.arg(layer.key_cache, tag + "key_cache")
        attention.slot[rt.AT_S_VCACHE] = slots.arg(layer.value_cache, tag + "value_cache")
        attention.slot[rt.AT_S_LEN] = slots.arg(layer.valid_length, tag + "valid_length")
        attention.slot[rt.AT_S_POS] = DYN_POSITION_IDS
        attention.slot[rt.AT_S_INVFREQ] = inv_freq
        attention.slot[rt.AT_S_OUT] = attn
        attention.slot[rt.AT_S_PARTIAL] = partial
        attention.slot[rt.AT_S_COUNTER] = counters
        phases.append(attention)
        attention_phase = len(phases) - 1
        o_phase = gemv(
            k=q_dim,
            segments=[(H, slots.arg(layer.o_weight, tag + "o_proj.weight"),
                       slots.arg(layer.o_bias, tag + "o_proj.bias"), hidden_b)],
            x_slot=attn,
            x_source=attention_phase,
            x_cells=attn_cells,
            epilogue=rt.EPI_RESIDUAL,
            residual_slot=layer_in,
            residual_source=hidden_source,
            residual_cells=hidden_cells,
            out_cells=hidden_cells,
            out_fenced=not hidden_cells,
        )
        if layer.gate_bias is not None or layer.up_bias is not None:
            fail("pattern-recognition", "biased gate/up projections are not covered")
        gated_phase = gemv(
            k=H,
            segments=[(p.intermediate, slots.arg(layer.gate_weight, tag + "gate_proj.weight"),
                       -1, glu)],
            x_slot=hidden_b,
            x_source=o_phase,
            x_cells=hidden_cells,
            prologue=pro,
            norm_slot=slots.arg(layer.post_norm, tag + "post_attention_layernorm.weight"),
            epilogue=act,
            pair_slot=slots.arg(layer.up_weight, tag + "up_proj.weight"),
            out_cells=glu_cells,
            out_fenced=not glu_cells,
        )
        hidden_source = gemv(
            k=p.intermediate,
            segments=[(H, slots.arg(layer.down_weight, tag + "down_proj.weight"),
                       slots.arg(layer.down_bias, tag + "down_proj.bias"), layer_out)],
            x_slot=glu,
            x_source=gated_phase,
            x_cells=glu_cells,
            epilogue=rt.EPI_RESIDUAL,
            residual_slot=hidden_b,
            residual_source=o_phase,
            residual_cells=hidden_cells,
            out_cells=hidden_cells,
            out_fenced=not hidden_cells,
        )
    gemv(
        k=H,
        segments=[(p.vocab, slots.arg(p.lm_head_weight, "lm_head.weight"),
                   slots.arg(p.lm_head_bias, "lm_head.bias"), DYN_LOGITS)],
        x_slot=stream,
        x_source=hidden_source,
        x_cells=hidden_cells,
        prologue=pro,
        norm_slot=slots.arg(p.final_norm, "norm.weight"),
        out_cells=False,
    )

    activation = _align(activation, 128)
    if fixed_bytes + activation + 2 * stage_bytes > max_smem:
        fail("resource-admission",
             f"activations need {activation} B of shared memory; with {fixed_bytes} B fixed and two "
             f"{stage_bytes} B weight stages that exceeds {max_smem} B",
             requirement="batch * max(hidden, intermediate) * 2 B must leave room for the ring")
    # grid barriers per launch: none between phases, one closes the launch
    intervals = sum(1 for phase in phases if phase.flags & rt.FLAG_BARRIER) + 1
    return PlanLayout(
        program=p,
        phases=phases,
        slots=slots.specs,
        workspace_bytes=_align(slots.workspace, 256),
        zero_ranges=slots.zero,
        activation_bytes=activation,
        intervals=intervals,
        notes=[f"{len(phases)} phases handed off through flagged cells, {intervals} grid barrier(s)",
               f"attention: max_chunks={max_chunks} merge_slots={merge_slots} "
               f"exact_keys={exact_keys}", f"ring stage {stage_bytes} B"],
        stage_bytes=stage_bytes,
    )


def plan_prefill(program: DecoderProgram, options: PlannerOptions | None = None,
                 mask=None) -> PlanLayout:
    """Prefill packing: one kernel launch per phase, in stream order (no grid barriers).

        [embed rows]                                   (layer 0)
        [rmsnorm rows] [q|k|v GEMM (+bias)] [rope rows] [attention] [o GEMM + residual]
        [rmsnorm rows] [gate|up GEMM . act(gate) * up] [down GEMM + residual]      x layers
        [rmsnorm rows] [lm head GEMM]

    GEMMs run on tcgen05 with TMA-fed operands, so their activations must sit in memory: the
    norms are phases of their own here (a [rows, hidden] round trip through L2, negligible
    next to the weights), while bias, residual and the gated activation stay in the GEMM
    epilogues.  ``mask`` is an additive bf16 ``[1 or B, 1, T, T]`` tensor for a non-causal
    program (``program.causal`` False); causal programs need none.
    """
    del options
    p = program
    if p.mode != "prefill":
        fail("planning", f"plan_prefill got a {p.mode!r} program")
    if p.head_dim not in (64, 128, 256):
        fail("resource-admission", f"head_dim {p.head_dim} not in (64, 128, 256)")
    if p.heads % p.kv_heads:
        fail("resource-admission", "query heads must be a multiple of kv heads")
    for name, value in (("hidden", p.hidden), ("intermediate", p.intermediate)):
        if value % 8:
            fail("resource-admission", f"{name} size {value} is not a multiple of 8")
    if p.norm not in ("llama", "gemma") or p.activation not in ("silu", "gelu_tanh"):
        fail("planning", "unknown norm or activation kind")
    if not p.causal and mask is None:
        fail("planning", "a non-causal prefill program needs its mask tensor")
    B, T, H, D = p.batch, p.tokens, p.hidden, p.head_dim
    R = B * T
    q_dim, kv_dim = p.heads * D, p.kv_heads * D
    slots = _Slots()
    kind = rt.PRO_RMS_LLAMA if p.norm == "llama" else rt.PRO_RMS_GEMMA
    act = rt.EPI_SILU_MUL if p.activation == "silu" else rt.EPI_GELU_TANH_MUL
    hidden = slots.buffer(R * H * 2, "hidden")
    normed = slots.buffer(R * H * 2, "normed")
    q_buf = slots.buffer(R * q_dim * 2, "q")
    k_buf = slots.buffer(R * kv_dim * 2, "k")
    v_buf = slots.buffer(R * kv_dim * 2, "v")
    attn = slots.buffer(R * q_dim * 2, "attention")
    glu = slots.buffer(R * p.intermediate * 2, "gated")
    padded = (T + 63) // 64 * 64
    v_t = slots.buffer(B * kv_dim * padded * 2, "values_transposed")
    # state handoff: keys and values go straight into the caller's KV caches (rows 0..T-1 of
    # every batch row) and the valid lengths are set to T
    handoff = all(layer.key_cache >= 0 for layer in p.layers)
    if handoff and p.capacity < T:
        fail("state-capacity", f"prompt of {T} tokens exceeds the KV capacity {p.capacity}")
    constants = {}
    mask_slot = -1
    if not p.causal:
        mask_slot = slots.constant("mask")
        constants["mask"] = mask.contiguous()
    phases: list[rt.Phase] = []

    def norm(weight_slot):
        phase = rt.Phase.blank(rt.BODY_RMSNORM_ROWS, 0)
        phase.i[rt.RN_I_ROWS], phase.i[rt.RN_I_K], phase.i[rt.RN_I_KIND] = R, H, kind
        phase.f[rt.RN_F_EPS] = p.eps
        phase.slot[rt.RN_S_X], phase.slot[rt.RN_S_W], phase.slot[rt.RN_S_OUT] = hidden, weight_slot, normed
        phases.append(phase)

    def gemm(*, k, x_slot, segments, epilogue=rt.EPI_NONE, pair_slot=-1, residual_slot=-1):
        phase = rt.Phase.blank(rt.BODY_GEMM_TC, 0)
        phase.i[rt.GV_I_ROWS] = R
        phase.i[rt.GV_I_K] = k
        phase.i[rt.GV_I_NSEG] = len(segments)
        phase.i[rt.GV_I_NMAT] = 2 if pair_slot >= 0 else 1
        phase.i[rt.GV_I_EPILOGUE] = epilogue
        phase.slot[rt.GV_S_X] = x_slot
        for index, (n, weight, bias, out) in enumerate(segments):
            phase.i[rt.GV_I_N0 + index] = n
            phase.slot[rt.GV_S_W0 + index] = weight
            phase.slot[rt.GV_S_BIAS0 + index] = bias
            phase.slot[rt.GV_S_OUT0 + index] = out
        phase.slot[rt.GV_S_W_PAIR] = pair_slot
        phase.slot[rt.GV_S_RESIDUAL] = residual_slot
        phases.append(phase)

    embed = rt.Phase.blank(rt.BODY_EMBED_ROWS, 0)
    embed.i[rt.EM_I_ROWS], embed.i[rt.EM_I_K], embed.i[rt.EM_I_VOCAB] = R, H, p.vocab
    embed.f[rt.EM_F_SCALE] = float(p.embed_scale or 0.0)
    embed.slot[rt.EM_S_TABLE] = slots.arg(p.embed_weight, "embed_tokens.weight")
    embed.slot[rt.EM_S_IDS] = DYN_INPUT_IDS
    embed.slot[rt.EM_S_OUT] = hidden
    phases.append(embed)
    inv_freq = slots.arg(p.inv_freq, "inv_freq")
    for index, layer in enumerate(p.layers):
        tag = f"layers.{index}."
        norm(slots.arg(layer.input_norm, tag + "input_layernorm.weight"))
        k_out = slots.arg(layer.key_cache, tag + "key_cache") if handoff else k_buf
        v_out = slots.arg(layer.value_cache, tag + "value_cache") if handoff else v_buf
        gemm(k=H, x_slot=normed, segments=[
            (q_dim, slots.arg(layer.q_weight, tag + "q_proj.weight"),
             slots.arg(layer.q_bias, tag + "q_proj.bias"), q_buf),
            (kv_dim, slots.arg(layer.k_weight, tag + "k_proj.weight"),
             slots.arg(layer.k_bias, tag + "k_proj.bias"), k_out),
            (kv_dim, slots.arg(layer.v_weight, tag + "v_proj.weight"),
             slots.arg(layer.v_bias, tag + "v_proj.bias"), v_out),
        ])
        if handoff:
            phases[-1].i[rt.GV_I_OUT_TOKENS], phases[-1].i[rt.GV_I_OUT_CAPACITY] = T, p.capacity
        rope = rt.Phase.blank(rt.BODY_ROPE_ROWS, 0)
        rope.i[rt.RP_I_ROWS], rope.i[rt.RP_I_HEADS], rope.i[rt.RP_I_KV_HEADS] = R, p.heads, p.kv_heads
        rope.i[rt.RP_I_HEAD_DIM] = D
        rope.i[rt.RP_I_INVFREQ_BF16] = 1 if p.inv_freq_dtype == "bf16" else 0
        rope.f[rt.RP_F_ROPE_SCALE] = p.rope_scale
        rope.f[rt.RP_F_Q_SCALE] = float(p.q_scale or 0.0)
        rope.slot[rt.RP_S_Q], rope.slot[rt.RP_S_K] = q_buf, k_out
        if handoff:
            rope.i[rt.RP_I_K_TOKENS], rope.i[rt.RP_I_K_CAPACITY] = T, p.capacity
            rope.i[rt.RP_I_LEN_VALUE] = T
            rope.i[rt.RP_I_LEN_COUNT] = p.length_count
            rope.slot[rt.RP_S_LEN] = slots.arg(layer.valid_length, tag + "valid_length")
        rope.slot[rt.RP_S_POS], rope.slot[rt.RP_S_INVFREQ] = DYN_POSITION_IDS, inv_freq
        phases.append(rope)
        attention = rt.Phase.blank(rt.BODY_ATTN_PREFILL, 0)
        attention.i[rt.AP_I_BATCH], attention.i[rt.AP_I_TOKENS] = B, T
        attention.i[rt.AP_I_HEADS], attention.i[rt.AP_I_KV_HEADS] = p.heads, p.kv_heads
        attention.i[rt.AP_I_HEAD_DIM] = D
        attention.i[rt.AP_I_CAUSAL] = 1 if p.causal else 0
        attention.i[rt.AP_I_MASK_BATCH] = 1 if mask is None else int(mask.shape[0])
        attention.f[rt.AP_F_SCALE] = p.softmax_scale
        attention.slot[rt.AP_S_Q], attention.slot[rt.AP_S_K], attention.slot[rt.AP_S_V] = q_buf, k_out, v_out
        attention.i[rt.AP_I_KV_CAPACITY] = p.capacity if handoff else 0
        attention.slot[rt.AP_S_OUT], attention.slot[rt.AP_S_MASK] = attn, mask_slot
        attention.slot[rt.AP_S_VT] = v_t
        phases.append(attention)
        gemm(k=q_dim, x_slot=attn, epilogue=rt.EPI_RESIDUAL, residual_slot=hidden, segments=[
            (H, slots.arg(layer.o_weight, tag + "o_proj.weight"),
             slots.arg(layer.o_bias, tag + "o_proj.bias"), hidden)])
        if layer.gate_bias is not None or layer.up_bias is not None:
            fail("pattern-recognition", "biased gate/up projections are not covered")
        norm(slots.arg(layer.post_norm, tag + "post_attention_layernorm.weight"))
        gemm(k=H, x_slot=normed, epilogue=act,
             pair_slot=slots.arg(layer.up_weight, tag + "up_proj.weight"),
             segments=[(p.intermediate, slots.arg(layer.gate_weight, tag + "gate_proj.weight"), -1, glu)])
        gemm(k=p.intermediate, x_slot=glu, epilogue=rt.EPI_RESIDUAL, residual_slot=hidden, segments=[
            (H, slots.arg(layer.down_weight, tag + "down_proj.weight"),
             slots.arg(layer.down_bias, tag + "down_proj.bias"), hidden)])
    norm(slots.arg(p.final_norm, "norm.weight"))
    gemm(k=H, x_slot=normed, segments=[
        (p.vocab, slots.arg(p.lm_head_weight, "lm_head.weight"),
         slots.arg(p.lm_head_bias, "lm_head.bias"), DYN_LOGITS)])
    return PlanLayout(
        program=p, phases=phases, slots=slots.specs,
        workspace_bytes=_align(slots.workspace, 256), zero_ranges=[], activation_bytes=0,
        intervals=len(phases), notes=[f"{len(phases)} kernel launches per prefill"],
        mode=rt.MODE_PREFILL, constants=constants)
