/*
 * megabake_b200 -- C ABI of the B200 (sm_100a) persistent-megakernel decoder backend.
 *
 * The Python host (megabake_b200.planner) turns one captured decoder invocation into a
 * table of fixed-size phase records plus a table of device addresses ("slots") and hands
 * both to this library.  One call of mb_plan_launch() is one cooperative persistent
 * kernel launch that executes every phase in order.  Phases hand their activations to one
 * another either through flagged cells (below) that the consumers poll -- no barrier at all --
 * or, where a record asks for one, across a grid barrier.
 *
 * Flagged cells.  An activation tensor [rows, N] of bf16 that one phase produces and a later
 * phase of the same launch consumes can be kept as [rows, N / 2] 64-bit cells: two bf16 values
 * in the low word, a 32-bit sequence number in the high word (launch epoch x phases + producing
 * phase + 1), written with one 8-byte store.  A consumer loads the cells it needs and retries
 * until the sequence number is the one it expects: data and "ready" arrive in one round trip
 * through L2.  This is the per-region flag wait of the reference's event-counter scheduler
 * (src/megabake/runtime.py:279-316) taken down to the single activation element.  A cell
 * buffer may be overwritten at the earliest two phases after its last reader; the kernel checks
 * that (a counter of CTAs that finished each phase) before every cell store.  Cell buffers
 * belong to the plan's workspace and start zeroed.
 *
 * What each entry point replaces in the reference (paths relative to the reference
 * project root):
 *   mb_plan_create   compile_plan(): emit + JIT the CuTe module, occupancy admission
 *                    (src/megabake/compiler.py:625-796) and the phase/GEMM tables built by
 *                    _emit_table_module (src/megabake/codegen.py:728-1784)
 *   mb_plan_bind     _RuntimeState.rebind / _fast_table_rebind: static slot addresses
 *                    (src/megabake/compiler.py:2156-2208)
 *   mb_plan_launch   _RuntimeState.prepare_launch + run_compiled_program: per-call dynamic
 *                    addresses and the cooperative launch
 *                    (src/megabake/compiler.py:2464-2524, src/megabake/runtime.py:153-190)
 *   mb_plan_status   the device-side trap_if sites (src/megabake/runtime.py:139-149,
 *                    src/megabake/bodies/cuda/sm100/attention.py:982): here a status word
 *                    the host reads after it synchronised, never a trap
 *   mb_plan_reset    no counterpart (the reference traps; a trapped context is lost)
 *   mb_plan_destroy  release of _RuntimeState buffers
 *   mb_plan_query    CompiledResources / launch requirements
 *                    (src/megabake/codegen.py:100-143)
 *
 * Conventions: every function returns an int code (MB_OK == 0) and never throws, aborts
 * or exits.  Pointers are borrowed for the duration of the call; slot addresses are
 * copied.  A plan is not re-entrant (the caller serialises calls on one plan); different
 * plans are independent.  No function synchronises the device except mb_plan_create,
 * mb_plan_bind, mb_plan_status, mb_plan_reset and mb_plan_destroy.  mb_plan_launch
 * performs no allocation and no host synchronisation and always passes the same kernel
 * parameters for the same dynamic addresses, so it can be captured in a CUDA graph.
 */
#ifndef MEGABAKE_B200_H
#define MEGABAKE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MB_ABI_VERSION 2

/* ---- return codes of the host API ------------------------------------------------ */
enum mb_error {
    MB_OK = 0,
    MB_ERR_INVALID = 1,     /* bad argument / malformed descriptor                      */
    MB_ERR_CUDA = 2,        /* a CUDA runtime call failed (mb_last_cuda_error())         */
    MB_ERR_UNSUPPORTED = 3, /* body / shape outside what the kernels implement           */
    MB_ERR_RESOURCE = 4,    /* shared memory or co-residency admission failed            */
    MB_ERR_UNBOUND = 5,     /* launch before every static slot was bound                 */
    MB_ERR_VERSION = 6      /* descriptor abi_version != MB_ABI_VERSION                  */
};

/* ---- device status word (read back by mb_plan_status) ---------------------------- */
enum mb_status_code {
    MB_ST_OK = 0,
    MB_ST_BARRIER_TIMEOUT = 1, /* a grid-barrier wait ran out                            */
    MB_ST_PIPE_TIMEOUT = 2,    /* a shared-memory pipeline (mbarrier) wait ran out       */
    MB_ST_KV_OVERFLOW = 3,     /* valid_length + 1 > cache capacity                      */
    MB_ST_TOKEN_RANGE = 4,     /* an input id outside [0, vocab)                         */
    MB_ST_BAD_PHASE = 5,       /* unknown body id in the phase table                     */
    MB_ST_TMEM = 6,            /* tensor-memory allocation failed                        */
    MB_ST_HANDOFF_TIMEOUT = 7  /* a flagged cell never showed the expected sequence number */
};

typedef struct mb_status {
    int32_t code;   /* enum mb_status_code of the first fault, 0 if none                */
    int32_t phase;  /* phase index that recorded it                                     */
    int32_t detail; /* body-specific (CTA index, offending value ...)                   */
    int32_t calls;  /* launches completed on this plan since create/reset               */
} mb_status;

/* ---- plan modes ------------------------------------------------------------------- */
enum mb_mode { MB_MODE_DECODE = 0, MB_MODE_PREFILL = 1 };

/* ---- device bodies ---------------------------------------------------------------- */
enum mb_body {
    MB_BODY_NOP = 0,
    /* Skinny GEMM for <= 8 activation rows: out[r, n] = epi(pro(x)[r, :] . W[n, :] + b[n]).
     * Weight rows are streamed by a dedicated producer warp with bulk async copies into a
     * shared-memory ring; up to three weight segments share one activation (q|k|v), or two
     * matrices are paired (gate|up) for a gated-activation epilogue.                      */
    MB_BODY_GEMV = 1,
    /* One-token attention over the KV cache: RoPE of q and the new k, append of k/v at
     * valid_length, split-key flash decoding with an online softmax, last-arriver merge.  */
    MB_BODY_ATTN_DECODE = 2,
    /* ---- prefill bodies ---- */
    MB_BODY_EMBED_ROWS = 3,   /* gather embedding rows (+ scalar scale)                    */
    MB_BODY_RMSNORM_ROWS = 4, /* row-wise RMSNorm                                          */
    MB_BODY_GEMM_TC = 5,      /* tcgen05/TMEM GEMM fed by TMA                              */
    MB_BODY_ROPE_ROWS = 6,    /* rotary embedding of q and k rows, in place                */
    MB_BODY_ATTN_PREFILL = 7, /* causal / masked softmax attention, tensor-core flash form */
    MB_BODY_COUNT = 8
};

/* mb_phase.flags */
#define MB_FLAG_BARRIER 1      /* grid barrier after the phase                            */
#define MB_FLAG_BUMP_LENGTH 2  /* attention phases: when the launch has finished without a
                                  fault, 1 is added to every valid length at
                                  slot[MB_AT_S_LEN]                                         */

#define MB_FLAG_FENCE 4        /* the phase's results are plain memory that a later phase reads
                                  after MB_CELLS_X_WAIT: every CTA makes its stores visible
                                  (a gpu-scope fence) before it reports the phase finished   */

/* bits of MB_GV_I_CELLS / MB_AT_I_CELLS: which tensors of the phase are flagged cells */
#define MB_CELLS_X 1           /* activations in (GEMV x; attention q, k and v)            */
#define MB_CELLS_OUT 2         /* every output segment                                     */
#define MB_CELLS_RESIDUAL 4    /* the residual operand                                     */
#define MB_CELLS_XSTORE 8      /* the copy of the gathered rows                            */
#define MB_CELLS_X_WAIT 16     /* GEMV: before x is read, wait until every CTA has reported
                                  phase MB_GV_I_X_SOURCE finished (one thread polls one
                                  counter: thousands of threads polling their cells would
                                  queue up in front of the very stores they wait for).  With
                                  cell x it is a hint -- the sequence numbers still decide;
                                  with plain x it is the synchronisation, and the producing
                                  phase must carry MB_FLAG_FENCE                              */

/* GEMV / GEMM prologues (applied to the activation rows) */
enum mb_prologue {
    MB_PRO_NONE = 0,
    MB_PRO_RMS_LLAMA = 1, /* bf16(w * bf16(x * rsqrt(mean(x^2) + eps)))                    */
    MB_PRO_RMS_GEMMA = 2  /* bf16(x * rsqrt(mean(x^2) + eps) * (1 + w)), all in fp32       */
};

/* GEMV / GEMM epilogues.  acc is the fp32 accumulator (+ fp32 bias); y = bf16(acc). */
enum mb_epilogue {
    MB_EPI_NONE = 0,          /* out = y                                                   */
    MB_EPI_RESIDUAL = 1,      /* out = bf16(res + y)                                       */
    MB_EPI_SILU_MUL = 2,      /* paired: out = bf16(bf16(silu(y_gate)) * y_up)             */
    MB_EPI_GELU_TANH_MUL = 3  /* paired: out = bf16(bf16(gelu_tanh(y_gate)) * y_up)        */
};

/* ---- phase record ------------------------------------------------------------------ */
#define MB_PHASE_INTS 24
#define MB_PHASE_FLOATS 4
#define MB_PHASE_SLOTS 20

typedef struct mb_phase {
    int32_t body;
    int32_t flags;
    int32_t i[MB_PHASE_INTS];
    float f[MB_PHASE_FLOATS];
    int32_t slot[MB_PHASE_SLOTS]; /* indices into the address table; -1 = absent         */
} mb_phase;

/* MB_BODY_GEMV: integer fields */
#define MB_GV_I_ROWS 0     /* activation rows (batch), 1..8                               */
#define MB_GV_I_K 1        /* reduction length, multiple of 16                            */
#define MB_GV_I_NSEG 2     /* weight segments, 1..3                                       */
#define MB_GV_I_N0 3       /* output features of segment 0 (1 and 2 follow), each even    */
#define MB_GV_I_NMAT 6     /* 1, or 2 for a paired gate/up phase (then NSEG == 1)         */
#define MB_GV_I_PROLOGUE 7
#define MB_GV_I_EPILOGUE 8
#define MB_GV_I_ROW_TILE 9 /* output rows per pipeline stage: 8 (always for a paired phase)
                              or 16 (two 8-row tiles per stage: rows of at most 1,024
                              elements, so that a stage still carries ~30 KB)              */
#define MB_GV_I_K_CHUNK 10 /* reduction elements per pipeline stage, multiple of 16       */
#define MB_GV_I_GATHER 11  /* 1: activation rows are gathered from an embedding table     */
#define MB_GV_I_VOCAB 12   /* rows of that table (range check)                            */
#define MB_GV_I_STORE_X 13 /* 1: CTA 0 also stores the un-normalised rows at S_XSTORE     */
#define MB_GV_I_SPLIT_Q 14 /* filled by mb_plan_create: output row PAIRS per CTA (floor) ...  */
#define MB_GV_I_SPLIT_R 15 /* ... and how many leading CTAs take one pair more              */
#define MB_GV_I_CELLS 20   /* MB_CELLS_* bits                                             */
#define MB_GV_I_X_SOURCE 21   /* phase index that wrote the x cells                        */
#define MB_GV_I_RES_SOURCE 22 /* phase index that wrote the residual cells                 */
/* floats */
#define MB_GV_F_EPS 0
#define MB_GV_F_EMBED_SCALE 1 /* 0 = none; else gathered rows are bf16(row * scale)       */
/* slots */
#define MB_GV_S_X 0        /* activations [rows, K] bf16, or the embedding table [V, K]   */
#define MB_GV_S_NORM_W 1   /* [K] bf16                                                    */
#define MB_GV_S_W0 2       /* weights [N, K] bf16 row-major, segments 0..2                */
#define MB_GV_S_BIAS0 5    /* [N] bf16, segments 0..2, -1 if absent                       */
#define MB_GV_S_OUT0 8     /* [rows, N] bf16, segments 0..2                               */
#define MB_GV_S_W_PAIR 11  /* second matrix of a paired phase                             */
#define MB_GV_S_RESIDUAL 12
#define MB_GV_S_IDS 13     /* int64 [rows] token ids (gather)                             */
#define MB_GV_S_XSTORE 14

/* MB_BODY_ATTN_DECODE */
#define MB_AT_I_BATCH 0
#define MB_AT_I_HEADS 1
#define MB_AT_I_KV_HEADS 2
#define MB_AT_I_HEAD_DIM 3   /* 64, 128 or 256                                            */
#define MB_AT_I_CAPACITY 4
#define MB_AT_I_INVFREQ_BF16 5 /* 1 if the inv_freq buffer is bf16, 0 if fp32             */
#define MB_AT_I_MAX_CHUNKS 6 /* key chunks per (batch, kv head) the workspace is sized for */
#define MB_AT_I_MERGE_SLOTS 7 /* per-warp states that fit the shared scratch at once      */
#define MB_AT_I_EXACT_KEYS 8 /* contexts up to this many keys (<= 128, 0 = never) use the
                                softmax that rounds normalised probabilities to bf16
                                like the eager operator                                */
#define MB_AT_I_CELLS 9      /* MB_CELLS_X: q, k and v are cells; MB_CELLS_OUT: out is      */
#define MB_AT_I_QKV_SOURCE 10 /* phase index that wrote the q, k and v cells               */
#define MB_AT_I_LEN_COUNT 11 /* valid lengths at MB_AT_S_LEN: 1 (shared by the batch; 0 means
                                1) or batch (one per row: rows may hold different numbers of
                                keys)                                                     */
#define MB_AT_F_SCALE 0      /* head_dim ** -0.5, applied in fp32                          */
#define MB_AT_F_ROPE_SCALE 1 /* attention_scaling multiplied into cos/sin                  */
#define MB_AT_F_Q_SCALE 2    /* 0 or 1 = none; else q = bf16(q * this) after RoPE          */
#define MB_AT_S_Q 0          /* [B, Hq*D] bf16 before RoPE                                 */
#define MB_AT_S_K 1          /* [B, Hkv*D]                                                 */
#define MB_AT_S_V 2
#define MB_AT_S_KCACHE 3     /* [B, capacity, Hkv, D] bf16                                 */
#define MB_AT_S_VCACHE 4
#define MB_AT_S_LEN 5        /* int32 [1] or [batch] (MB_AT_I_LEN_COUNT)                    */
#define MB_AT_S_POS 6        /* int64 [B]                                                  */
#define MB_AT_S_INVFREQ 7    /* [D/2]                                                      */
#define MB_AT_S_OUT 8        /* [B, Hq*D] bf16                                             */
#define MB_AT_S_PARTIAL 9    /* fp32 [B*Hkv, max_chunks, Hq/Hkv, D+2]                      */
#define MB_AT_S_COUNTER 10   /* int32 [B*Hkv], zero before the first launch                */

/* ---- prefill bodies (MB_MODE_PREFILL plans: one kernel launch per phase, in order) ----- */
/* MB_BODY_EMBED_ROWS: out[r, :] = table[ids[r], :] (x scale, rounded to bf16)              */
#define MB_EM_I_ROWS 0
#define MB_EM_I_K 1
#define MB_EM_I_VOCAB 2
#define MB_EM_F_SCALE 0      /* 0 = none                                                   */
#define MB_EM_S_TABLE 0      /* [vocab, K] bf16                                            */
#define MB_EM_S_IDS 1        /* int64 [rows]                                               */
#define MB_EM_S_OUT 2        /* [rows, K] bf16                                             */
/* MB_BODY_RMSNORM_ROWS: out[r, :] = rmsnorm(x[r, :]) in the spelling MB_RN_I_KIND names    */
#define MB_RN_I_ROWS 0
#define MB_RN_I_K 1          /* multiple of 8                                              */
#define MB_RN_I_KIND 2       /* enum mb_prologue, not NONE                                 */
#define MB_RN_F_EPS 0
#define MB_RN_S_X 0
#define MB_RN_S_W 1
#define MB_RN_S_OUT 2
/* MB_BODY_GEMM_TC: the MB_BODY_GEMV record (MB_GV_* fields: any number of rows, K a multiple
 * of 8, segments, paired gate/up, epilogues; no prologue, no gather) computed by a TMA-fed
 * tcgen05 GEMM with TMEM accumulators.  mb_plan_create fills MB_GV_I_SPLIT_K and
 * MB_GV_I_TILE_N.                                                                          */
#define MB_GV_I_SPLIT_K 16   /* CTAs sharing one output tile along the reduction           */
#define MB_GV_I_TILE_N 17    /* output columns per tile: 128 or 256 (per matrix: half)     */
#define MB_GV_I_OUT_TOKENS 18   /* > 0: segments 1 and 2 (k, v) write row r at                 */
#define MB_GV_I_OUT_CAPACITY 19 /* (r / TOKENS) * CAPACITY + r % TOKENS: straight into KV caches */
/* MB_BODY_ROPE_ROWS: rotary embedding of q and k rows, in place                            */
#define MB_RP_I_ROWS 0
#define MB_RP_I_HEADS 1
#define MB_RP_I_KV_HEADS 2
#define MB_RP_I_HEAD_DIM 3
#define MB_RP_I_INVFREQ_BF16 4
#define MB_RP_I_K_TOKENS 5    /* > 0: k rows live in a cache, row r at (r / TOKENS) * CAPACITY   */
#define MB_RP_I_K_CAPACITY 6  /*      + r % TOKENS                                                */
#define MB_RP_I_LEN_VALUE 7   /* written to the int32(s) at MB_RP_S_LEN, if that slot is given    */
#define MB_RP_I_LEN_COUNT 8   /* how many: 1 (0 means 1), or up to 256 (one per batch row)       */
#define MB_RP_F_ROPE_SCALE 0
#define MB_RP_F_Q_SCALE 1    /* 0 or 1 = none; else q = bf16(q * this) after the rotation  */
#define MB_RP_S_Q 0          /* [rows, heads * D] bf16                                     */
#define MB_RP_S_K 1          /* [rows, kv_heads * D] bf16                                  */
#define MB_RP_S_POS 2        /* int64 [rows]                                               */
#define MB_RP_S_INVFREQ 3    /* [D / 2]                                                    */
#define MB_RP_S_LEN 4        /* optional int32 [MB_RP_I_LEN_COUNT]: the layer's valid length(s)
                                (state handoff)                                              */
/* MB_BODY_ATTN_PREFILL: softmax attention with the eager operator's rounding points:
 * s = bf16(q . k), s = bf16(s * scale), s = bf16(s + mask), p = bf16(softmax_fp32(s)),
 * out = bf16(sum p v).                                                                     */
#define MB_AP_I_BATCH 0
#define MB_AP_I_TOKENS 1
#define MB_AP_I_HEADS 2
#define MB_AP_I_KV_HEADS 3
#define MB_AP_I_HEAD_DIM 4   /* 64, 128 or 256                                             */
#define MB_AP_I_CAUSAL 5     /* 1: key j visible to query i iff j <= i, no mask tensor      */
#define MB_AP_I_MASK_BATCH 6 /* leading extent of the mask tensor: 1 or batch              */
#define MB_AP_I_KV_CAPACITY 7 /* rows per batch of the K and V tensors (a KV cache); 0 = tokens */
#define MB_AP_F_SCALE 0
#define MB_AP_S_Q 0          /* [batch * tokens, heads * D] bf16 (after RoPE)              */
#define MB_AP_S_K 1          /* [batch * tokens, kv_heads * D]                             */
#define MB_AP_S_V 2
#define MB_AP_S_OUT 3        /* [batch * tokens, heads * D]                                */
#define MB_AP_S_MASK 4       /* additive bf16 [mask_batch, 1, tokens, tokens], or absent   */
#define MB_AP_S_VT 5         /* scratch [batch * kv_heads * D, tokens rounded up to 64] bf16:
                                given, the phase runs on tcgen05 (Q.K^T and P.V as tensor-memory
                                MMAs, V transposed into this buffer first); absent, on mma.sync */

/* ---- plan descriptor ---------------------------------------------------------------- */
#define MB_MAX_DYNAMIC 8

typedef struct mb_plan_desc {
    uint32_t abi_version;     /* MB_ABI_VERSION                                           */
    int32_t device;           /* CUDA device ordinal                                      */
    int32_t mode;             /* enum mb_mode                                             */
    uint32_t n_phases;
    const mb_phase* phases;
    uint32_t n_slots;         /* size of the address table                                */
    uint32_t n_dynamic;       /* slots [0, n_dynamic) are given per launch, <= 8          */
    uint32_t activation_bytes;/* shared memory for activations / attention scratch        */
    uint32_t ctas;            /* 0 = one per SM                                           */
    uint32_t stage_bytes;     /* decode: bytes of one weight-ring stage, a multiple of 1024 up
                                 to mb_stage_bytes(); 0 = mb_stage_bytes().  Small stages give
                                 a deeper ring when the reduction length is short            */
    uint32_t wait_limit_ms;   /* bound of every device-side wait (hand-off cells, pipeline
                                 stages, grid barrier) in milliseconds; 0 = 2000.  When a wait
                                 runs out the kernel records a status, drains and returns   */
    uint32_t reserved[2];
} mb_plan_desc;

typedef struct mb_plan_info {
    int32_t ctas;             /* cooperative grid size                                    */
    int32_t threads;          /* threads per CTA                                          */
    int32_t smem_bytes;       /* dynamic shared memory per CTA                            */
    int32_t stages;           /* weight-ring stages                                       */
    int32_t barriers;         /* grid barriers per launch                                 */
    int32_t sm_count;
    int32_t launches;         /* kernel launches one mb_plan_launch enqueues              */
    int32_t reserved[1];
} mb_plan_info;

typedef struct mb_plan mb_plan;

int mb_plan_create(const mb_plan_desc* desc, mb_plan** out);
int mb_plan_query(const mb_plan* plan, mb_plan_info* out);
int mb_plan_bind(mb_plan* plan, const uint64_t* slot_addresses, size_t n);
int mb_plan_launch(mb_plan* plan, const uint64_t* dynamic_addresses, size_t n, void* stream);
int mb_plan_status(mb_plan* plan, mb_status* out);
int mb_plan_reset(mb_plan* plan);
/* Per-phase trace (no counterpart in the reference API; its MEGABAKE_PHASE_TIMER build flag,
 * src/megabake/runtime.py:22-47, is the same idea): `device_address` points at
 * ctas * n_phases * 8 uint64 the kernel fills with global-timer stamps (0 phase start,
 * 1 prologue done, 2 body done, 3 barrier passed, 4..7 body-specific) on every later
 * launch; 0 switches it off. */
int mb_plan_set_trace(mb_plan* plan, uint64_t device_address, size_t bytes);
void mb_plan_destroy(mb_plan* plan);

/* ---- decode attention that allocates nothing ---------------------------------------------
 * No counterpart in the reference (its attention body only exists inside a compiled plan).
 * For callers that must not allocate device memory where they need an attention step (a
 * plugin inside a foreign stream-ordered pipeline, a process living on an amount of memory fixed
 * at start-up, a region where cudaMalloc would synchronise the device): the same decode
 * attention as MB_BODY_ATTN_DECODE -- RoPE of q and the new k, append at valid_length,
 * valid_length += 1, attention over every valid key -- with its scratch (split-key partials,
 * arrival counters, status) in a fixed 4 MiB array inside the library's device image instead
 * of allocated memory.  It calls no cudaMalloc/cudaFree or allocating library routine.
 *
 * Limits: batch * kv_heads <= 1024 and batch * heads * (head_dim + 2) * 4 B must fit the array
 * (MB_ERR_RESOURCE otherwise); heads / kv_heads <= 8; head_dim in {64, 128, 256}.
 * The first call on a device does the one-time set-up (address of the array on that device,
 * kernel attribute): make it before any stream capture.  Every call shares the array: calls
 * that may overlap on the GPU race on it and must be serialised by the caller.  Non-blocking:
 * a device-side fault (KV cache full = MB_ST_KV_OVERFLOW) is written to `status` if given.  */
typedef struct mb_attention_args {
    int32_t batch, heads, kv_heads, head_dim, capacity;
    int32_t inv_freq_is_bf16;  /* 1: inv_freq holds bf16, 0: fp32                              */
    float rope_scale;          /* attention_scaling multiplied into cos/sin (usually 1)        */
    float query_scale;         /* 0 or 1 = none; else q = bf16(q * this) after RoPE            */
    uint64_t query;            /* [batch, heads * head_dim] bf16, before RoPE                  */
    uint64_t key;              /* [batch, kv_heads * head_dim] bf16, before RoPE               */
    uint64_t value;            /* [batch, kv_heads * head_dim] bf16                            */
    uint64_t key_cache;        /* [batch, capacity, kv_heads, head_dim] bf16, appended to      */
    uint64_t value_cache;
    uint64_t valid_length;     /* int32 [1], incremented                                       */
    uint64_t position_ids;     /* int64 [batch]                                                */
    uint64_t inv_freq;         /* [head_dim / 2]                                               */
    uint64_t out;              /* [batch, heads * head_dim] bf16                               */
    uint64_t status;           /* optional int32 [1] receiving enum mb_status_code, or 0       */
} mb_attention_args;

int mb_attention_decode_static(const mb_attention_args* args, void* stream);

/* ---- greedy pick on the device ------------------------------------------------------------
 * Replaces the host-side pick of the reference's generation loop
 * (`int(logits[0, -1].argmax().item())`, examples/single_gpu_generate.py:76) and provides what
 * its roadmap lists as missing (multi-step decode loop with on-device argmax,
 * docs/roadmap.md:180,223): for every batch row, the index of the largest logit (lowest index
 * on ties, NaN above every number -- torch.argmax's rules) is written into `input_ids`, the
 * tensor the next decode launch reads; `position_ids` (optional) is advanced by one; the id is
 * appended to `out_tokens[row][cursor[row]]` and `cursor[row]` incremented (optional; the
 * cursor keeps counting when the log is full, ids past `out_capacity` are dropped).
 * One launch, no allocation, no host synchronisation: a decode launch followed by this call
 * can be enqueued back to back any number of times, or captured in a CUDA graph.           */
typedef struct mb_greedy_args {
    int32_t rows;             /* batch rows                                               */
    int32_t vocab;            /* logits per row                                           */
    int32_t out_capacity;     /* ids per row that out_tokens can hold                     */
    int32_t reserved;
    uint64_t logits;          /* [rows, vocab] bf16, contiguous                           */
    uint64_t input_ids;       /* int64 [rows], overwritten with the picks                 */
    uint64_t position_ids;    /* int64 [rows], incremented; 0 = leave alone               */
    uint64_t out_tokens;      /* int64 [rows, out_capacity] log of picks; 0 = none        */
    uint64_t cursor;          /* int32 [rows] next free column of out_tokens (with it)    */
} mb_greedy_args;

int mb_greedy_advance(const mb_greedy_args* args, void* stream);

const char* mb_strerror(int code);
const char* mb_status_string(int status_code);
const char* mb_last_cuda_error(void);
int mb_abi_version(void);

/* Shared-memory need of the fixed parts, so the host planner can size activation_bytes
 * and predict the ring depth without a device: returns bytes, or -1 for a bad mode. */
int mb_fixed_smem_bytes(int mode);
int mb_stage_bytes(int mode);
int mb_max_smem_bytes(void);

#ifdef __cplusplus
}
#endif
#endif /* MEGABAKE_B200_H */
