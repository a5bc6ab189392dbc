// Decode megakernel: one cooperative persistent launch runs every phase of a one-token
// decoder step.  Phases hand activations to one another through flagged cells (two bf16 values
// and a sequence number per 8-byte store, polled by the consumers), so that a layer needs no
// grid barrier; a record may still ask for one.  Thread layout per CTA (one CTA per SM):
//   warps 0..7   consumers: activation prologues (RMSNorm, embedding gather), the skinny
//                GEMM inner loop on mma.sync with fp32 accumulation, epilogues, decode
//                attention, and the grid barriers between barrier intervals
//   warp 8       weight producer: walks the same phase table and streams this CTA's weight
//                rows into a shared-memory ring with bulk async copies (TMA, 1-D), running
//                ahead of the consumers across phase and grid-barrier boundaries because
//                weights never depend on earlier phases
//
// Replaces, for decode, the reference's generated persistent kernel
// (src/megabake/codegen.py:1634-1703), its sm100 swapAB GEMM bodies
// (src/megabake/bodies/cuda/sm100/cutlass_gemm.py:1072-1316), the split decode attention
// body (src/megabake/bodies/cuda/sm100/attention.py:909-1417), the generic row-reduction /
// map bodies used for RMSNorm, RoPE, residual and gated activations
// (src/megabake/bodies/cuda/generic.py:175-613) and the counting grid barrier
// (src/megabake/runtime.py:153-190).
#include <cmath>
#include <cstring>
#include <mutex>

#include "mb_device.cuh"
#include "mb_kernels.h"

namespace mb {
namespace decode {

constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 32;
constexpr int kMaxStages = 16;
constexpr int kRowTile = 8;          // weight rows of one n8 MMA tile; a stage holds one or two
constexpr int kRowPad = 64;          // bytes added to each staged row: with row lengths that are
                                     // multiples of 128 B this makes 16-byte fragment loads of
                                     // two neighbouring rows hit disjoint banks
constexpr int kStageBytes = 34816;   // largest ring stage: 8 rows x (2048 * 2 + 64) B plus slack,
                                     // whole 4 KB rows; plans may ask for smaller stages
constexpr int kCtlBytes = 2048;
constexpr int kReduceBytes = 16384;  // partial sums of one reduction group of row blocks
constexpr int kFixedBytes = kCtlBytes + kReduceBytes;
constexpr int kBarConsumers = 1;     // named barrier id of the consumer warps
constexpr int kFoldFloats = 8 * 64 + 16;  // attention: chunk weights + denominators
constexpr int kEntryVectors = sizeof(PhaseEntry) / 16;
constexpr int kTraceEvents = 8;  // stamps per phase and CTA in the optional trace buffer

// Trace stamp from inside a body (events 4..7 are body-specific); thread 0 only.
__device__ __forceinline__ void trace_stamp(const KernelParams& p, int ph, int event, int tid) {
    if (p.trace != nullptr && tid == 0)
        p.trace[(static_cast<size_t>(blockIdx.x) * p.n_phases + ph) * kTraceEvents + event] =
            global_timer_ns();
}

struct SharedCtl {
    unsigned long long full[kMaxStages];
    unsigned long long empty[kMaxStages];
    unsigned long long act_full;     // bulk copies of the current GEMV phase's prologue have landed
    unsigned long long limit_ns;     // bound of every wait of this launch
    volatile int abort_flag;
    volatile unsigned int issued;    // stages the producer armed
    int bcast[4];                    // small broadcasts (attention chunking, arrival order)
    volatile int verdict;            // thread 0's go / drain decision at a barrier
    unsigned int tag_base;           // cells of phase q carry tag_base + q + 1 in this launch
    unsigned int calls;              // launches completed before this one
    __align__(16) unsigned int guard[4];  // a counter of Control::finished, fetched asynchronously
    float red[kConsumerWarps][8];    // per-warp partials of the activation prologue
    __align__(16) PhaseEntry entry[2];  // current / next phase record with resolved addresses
    __align__(16) PhaseEntry producer_entry;  // the producer warp's own copy of its phase
};
static_assert(sizeof(SharedCtl) <= kCtlBytes, "control block too large");
static_assert(sizeof(PhaseEntry) % 16 == 0, "phase entries are copied in 16-byte vectors");

// Entries reach the bodies with per-launch (dynamic) slots already replaced by their addresses
// (patch_dynamic below), so reading an address is one shared-memory load.
__device__ __forceinline__ unsigned long long entry_address(const KernelParams&,
                                                            const PhaseEntry* e, int j) {
    return e->addr[j];
}

__device__ __forceinline__ unsigned long long resolve_dynamic(const KernelParams& p,
                                                              unsigned long long v) {
    if (v >> 63) {  // dynamic slot: the address comes with the launch
        const int s = static_cast<int>(v & 0xffu);
        unsigned long long a = p.dyn[0];
#pragma unroll
        for (int i = 1; i < MB_MAX_DYNAMIC; ++i)
            if (s == i) a = p.dyn[i];
        return a;
    }
    return v;
}

// One thread per slot rewrites the tagged slots of an entry that sits in shared memory.
__device__ __forceinline__ void patch_dynamic(const KernelParams& p, PhaseEntry* e, int lane) {
    if (lane < MB_PHASE_SLOTS) e->addr[lane] = resolve_dynamic(p, e->addr[lane]);
}

// ---------------------------------------------------------------------------------------
// Waiting for flagged cells.  The fast path (the cell already carries the expected sequence
// number) is inline at the call sites; these are the retry loops.  A wait gives up when the
// launch's limit has run out (status MB_ST_HANDOFF_TIMEOUT) or when this CTA or any other has
// recorded a fault; the caller goes on with whatever it has and the CTA drains at the end of
// the phase.
// ---------------------------------------------------------------------------------------
__device__ __noinline__ bool wait_gave_up(const KernelParams& p, SharedCtl* sc, int ph,
                                          unsigned long long start) {
    if (sc->abort_flag) return true;
    if (peek_status(p.ctl) != 0) {
        sc->abort_flag = 1;
        return true;
    }
    if (global_timer_ns() - start > sc->limit_ns) {
        record_status(p.ctl, MB_ST_HANDOFF_TIMEOUT, ph, static_cast<int>(blockIdx.x));
        sc->abort_flag = 1;
        return true;
    }
    return false;
}

__device__ __noinline__ void cell_pair_wait(const void* src, unsigned int tag,
                                            unsigned long long& a, unsigned long long& b,
                                            const KernelParams& p, SharedCtl* sc, int ph) {
    const unsigned long long start = global_timer_ns();
    for (unsigned int tries = 1;; ++tries) {
        __nanosleep(32);
        ld_cell_pair(src, a, b);
        if (cell_tag(a) == tag && cell_tag(b) == tag) return;
        if ((tries & 63u) == 0u && wait_gave_up(p, sc, ph, start)) return;
    }
}

__device__ __noinline__ unsigned long long cell_wait(const void* src, unsigned int tag,
                                                     const KernelParams& p, SharedCtl* sc,
                                                     int ph) {
    const unsigned long long start = global_timer_ns();
    for (unsigned int tries = 1;; ++tries) {
        __nanosleep(32);
        const unsigned long long v = ld_cell(src);
        if (cell_tag(v) == tag) return v;
        if ((tries & 63u) == 0u && wait_gave_up(p, sc, ph, start)) return v;
    }
}

// Lock-step within two phases.  A cell buffer is rewritten at the earliest three phases after
// its last reader (the planner's rule).  So a CTA may enter phase q + 1 only when every CTA has
// finished phase q - 2 ... the kernel asks for a little more, q - 2 at the END of phase q:
// Control::finished[q % 4] counts the CTAs that finished phase q, and thread 0 of every CTA
// checks the counter of phase q - 2 before it reports phase q finished.  `seen` is a value of
// that counter fetched while the phase ran; in the steady state it is already large enough and
// nothing waits.
__device__ __forceinline__ unsigned int finished_target(const KernelParams& p, const SharedCtl* sc,
                                                        int q) {
    const unsigned int slot = static_cast<unsigned int>(q) & 3u;
    // phases of one launch that count on this slot, and how many of them up to phase q
    const unsigned int per_launch = (static_cast<unsigned int>(p.n_phases) + 3u - slot) >> 2;
    return gridDim.x * (sc->calls * per_launch + (static_cast<unsigned int>(q) >> 2) + 1u);
}

// One thread: wait until every CTA has reported phase `q` finished.  The load is an acquire, so
// what those CTAs stored before a fenced report is visible to this thread afterwards (and,
// through a CTA barrier, to its CTA).
__device__ __noinline__ void finished_wait(const KernelParams& p, SharedCtl* sc, int ph, int q) {
    const unsigned int target = finished_target(p, sc, q);
    const unsigned int* counter = &p.ctl->finished[q & 3].count;
    const unsigned long long start = global_timer_ns();
    for (unsigned int tries = 1;; ++tries) {
        unsigned int seen;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
        if (static_cast<int>(seen - target) >= 0) return;
        if ((tries & 63u) == 0u && wait_gave_up(p, sc, ph, start)) return;
        __nanosleep(40);
    }
}

// Geometry of one GEMV phase for one CTA; producer and consumers derive it identically.
// A CTA owns output rows [r0, r1) of the phase's (virtually concatenated) output rows -- whole
// pairs of rows, so that a lane's two neighbouring results always form one cell -- and streams
// their weight rows as blocks of `row_tile` rows (8, or 16 = two MMA tiles), each cut into
// n_chunks stages of k_chunk elements.
struct GemvGeom {
    int rows, K, nseg, nmat, n[3], ntotal;
    int k_chunk, n_chunks, pitch, row_tile;
    int r0, r1, n_blocks;
};

__device__ __forceinline__ GemvGeom gemv_geometry(const mb_phase& P, int cta) {
    GemvGeom g;
    g.rows = P.i[MB_GV_I_ROWS];
    g.K = P.i[MB_GV_I_K];
    g.nseg = P.i[MB_GV_I_NSEG];
    g.nmat = P.i[MB_GV_I_NMAT];
    g.n[0] = P.i[MB_GV_I_N0];
    g.n[1] = g.nseg > 1 ? P.i[MB_GV_I_N0 + 1] : 0;
    g.n[2] = g.nseg > 2 ? P.i[MB_GV_I_N0 + 2] : 0;
    g.ntotal = g.n[0] + g.n[1] + g.n[2];
    g.k_chunk = P.i[MB_GV_I_K_CHUNK];
    g.n_chunks = (g.K + g.k_chunk - 1) / g.k_chunk;  // small operands: cheap
    g.pitch = g.k_chunk * 2 + kRowPad;
    g.row_tile = P.i[MB_GV_I_ROW_TILE];
    // balanced split precomputed by the host, in pairs of rows: the first `rem` CTAs own one
    // pair more
    const int q = P.i[MB_GV_I_SPLIT_Q], rem = P.i[MB_GV_I_SPLIT_R];
    g.r0 = 2 * (cta * q + min(cta, rem));
    g.r1 = g.r0 + 2 * (q + (cta < rem ? 1 : 0));
    g.n_blocks = (g.r1 - g.r0 + g.row_tile - 1) / g.row_tile;
    return g;
}

// ---------------------------------------------------------------------------------------
// Producer warp: for every GEMV phase, in phase order, stream this CTA's weight rows into
// the ring -- stage order is (row block, k chunk), the order the consumers expect.
// ---------------------------------------------------------------------------------------
__device__ __noinline__ void producer_loop(const KernelParams& p, SharedCtl* sc, char* ring,
                                           int lane) {
    const int cta = blockIdx.x;
    unsigned int it = 0;
    // The producer runs phases ahead of the consumers, so it would meet every phase entry
    // cold in DRAM and chase its fields one dependent load at a time.  Instead: pull the whole
    // table into L2 once, and per phase fetch the entry with one coalesced 16-byte load per
    // lane (the next entry's load is already in flight while this one is worked on).
    {
        const char* table = reinterpret_cast<const char*>(p.entries);
        const size_t bytes = sizeof(PhaseEntry) * static_cast<size_t>(p.n_phases);
        for (size_t off = static_cast<size_t>(lane) * 128; off < bytes; off += 32 * 128)
            prefetch_l2(table + off);
    }
    PhaseEntry* mine = &sc->producer_entry;
    uint4 next_vector = make_uint4(0u, 0u, 0u, 0u);
    if (lane < kEntryVectors)
        next_vector = __ldg(reinterpret_cast<const uint4*>(p.entries) + lane);
    for (int ph = 0; ph < p.n_phases; ++ph) {
        __syncwarp();  // everybody is done with the previous entry
        if (lane < kEntryVectors) {
            reinterpret_cast<uint4*>(mine)[lane] = next_vector;
            if (ph + 1 < p.n_phases)
                next_vector = __ldg(reinterpret_cast<const uint4*>(p.entries + ph + 1) + lane);
        }
        __syncwarp();
        patch_dynamic(p, mine, lane);
        __syncwarp();
        const PhaseEntry* E = mine;
        if (E->rec.body == MB_BODY_ATTN_DECODE) {
            // the few scalars the attention body starts from: pull them into L2 ahead of time
            if (lane == 0) prefetch_l2(reinterpret_cast<const void*>(entry_address(p, E, MB_AT_S_LEN)));
            if (lane == 1) prefetch_l2(reinterpret_cast<const void*>(entry_address(p, E, MB_AT_S_POS)));
            if (lane == 2)
                prefetch_l2(reinterpret_cast<const void*>(entry_address(p, E, MB_AT_S_INVFREQ)));
            continue;
        }
        if (E->rec.body != MB_BODY_GEMV) continue;
        const GemvGeom g = gemv_geometry(E->rec, cta);
        if (E->rec.i[MB_GV_I_PROLOGUE] != MB_PRO_NONE) {
            // norm weights are read by every CTA right after the barrier: have them in L2
            const char* nw = reinterpret_cast<const char*>(entry_address(p, E, MB_GV_S_NORM_W));
            for (int line = lane; line * 128 < g.K * 2; line += 32) prefetch_l2(nw + line * 128);
        }
        if (E->rec.slot[MB_GV_S_BIAS0] >= 0 && g.nseg == 1 && lane < 8) {
            // this CTA's slice of a single-segment bias (a few lines at most per 8 lanes)
            const char* bias = reinterpret_cast<const char*>(entry_address(p, E, MB_GV_S_BIAS0));
            const int stop = g.r1 * 2;  // byte range [r0 * 2, r1 * 2) of the vector
            for (int off = (g.r0 * 2 / 128 + lane) * 128; off < stop; off += 8 * 128)
                prefetch_l2(bias + off);
        }
        const char* w0 = reinterpret_cast<const char*>(entry_address(p, E, MB_GV_S_W0));
        const char* w1 = g.nseg > 1
                             ? reinterpret_cast<const char*>(entry_address(p, E, MB_GV_S_W0 + 1))
                             : nullptr;
        const char* w2 = g.nseg > 2
                             ? reinterpret_cast<const char*>(entry_address(p, E, MB_GV_S_W0 + 2))
                             : nullptr;
        const char* wpair = g.nmat > 1 ? reinterpret_cast<const char*>(
                                             entry_address(p, E, MB_GV_S_W_PAIR))
                                       : nullptr;
        const size_t row_bytes = static_cast<size_t>(g.K) * 2;
        // ring position: one division per phase, then counted up (a division per stage costs
        // more than the rest of the stage's bookkeeping)
        int stage = static_cast<int>(it % static_cast<unsigned int>(p.stages));
        unsigned int wraps = it / static_cast<unsigned int>(p.stages);
        for (int blk = 0; blk < g.n_blocks; ++blk) {
            const int block0 = g.r0 + blk * g.row_tile;
            const int nrows = min(g.row_tile, g.r1 - block0);
            // this lane's copy: matrix m, row r of the block (at most 16 copies per stage)
            const int m = lane / nrows, r = lane - m * nrows;
            const bool mine = lane < nrows * g.nmat;
            const char* src_row = nullptr;
            if (mine) {
                int local = block0 + r;
                const char* base;
                if (m == 1) {
                    base = wpair;
                } else if (local < g.n[0]) {
                    base = w0;
                } else if (local < g.n[0] + g.n[1]) {
                    base = w1;
                    local -= g.n[0];
                } else {
                    base = w2;
                    local -= g.n[0] + g.n[1];
                }
                src_row = base + static_cast<size_t>(local) * row_bytes;
            }
            for (int c = 0; c < g.n_chunks; ++c) {
                const unsigned int parity = (wraps & 1u) ^ 1u;
                if (!mbar_wait_bounded(&sc->empty[stage], parity, &sc->abort_flag, sc->limit_ns)) {
                    if (lane == 0 && !sc->abort_flag) {
                        record_status(p.ctl, MB_ST_PIPE_TIMEOUT, ph, cta);
                        sc->abort_flag = 1;
                    }
                    return;
                }
                const int kc = min(g.k_chunk, g.K - c * g.k_chunk);
                const unsigned int seg_bytes = static_cast<unsigned int>(kc) * 2u;
                if (lane == 0) {
                    mbar_arrive_expect_tx(&sc->full[stage], seg_bytes * nrows * g.nmat);
                    sc->issued = it + 1;
                }
                __syncwarp();
                if (mine) {
                    char* dst = ring + static_cast<size_t>(stage) * p.stage_bytes +
                                static_cast<size_t>(m * kRowTile + r) * g.pitch;
                    bulk_copy_g2s(dst, src_row + static_cast<size_t>(c) * g.k_chunk * 2, seg_bytes,
                                  &sc->full[stage]);
                }
                ++it;
                if (++stage == p.stages) {
                    stage = 0;
                    ++wraps;
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// Activation prologue: bring the phase's activation rows into shared memory as bf16,
// applying the embedding gather and/or RMSNorm.  All consumer threads.
// xs layout: [rows][K + 32] bf16 (the 64-byte pad spreads rows over banks).
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ const char* activation_row(const PhaseEntry* E, const char* xbase,
                                                      const long long* ids, int r, int K,
                                                      bool* bad_token) {
    if (ids != nullptr) {
        long long id = ids[r];
        if (id < 0 || id >= E->rec.i[MB_GV_I_VOCAB]) {
            *bad_token = true;
            id = 0;
        }
        return xbase + static_cast<size_t>(id) * K * 2;
    }
    return xbase + static_cast<size_t>(r) * K * 2;
}

__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src_gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)),
                 "l"(src_gmem)
                 : "memory");
}
// 16 bytes, or 16 zero bytes when `valid` is false (the source is not read then).
__device__ __forceinline__ void cp_async16_or_zero(void* dst_smem, const void* src_gmem,
                                                   bool valid) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(valid ? 16 : 0)
                 : "memory");
}

// Does this GEMV phase arm the activation mbarrier?  Plain activations come by bulk copy (one
// per row); so do the norm weights (one more row).  Cell activations with no norm arm nothing.
__device__ __forceinline__ bool activation_arms(const mb_phase& P) {
    return !(P.i[MB_GV_I_CELLS] & MB_CELLS_X) || P.i[MB_GV_I_PROLOGUE] != MB_PRO_NONE;
}

// Part 1 (activation_issue) starts the bulk copies global -> shared of whatever the phase takes
// from plain memory: every activation row when they are plain bf16 (one copy per row: the
// bulk-copy engine takes a row in one instruction, where 16-byte cp.async copies by all threads
// stalled the issuing warps for about a microsecond on the load/store unit's miss tracking), and
// the norm weight vector, staged as one extra row.  Part 2 waits for them (activation_finish for
// plain rows, activation_cells for rows that arrive as flagged cells) and normalises.
// `round` counts the phases of this CTA that armed the barrier: its parity.
__device__ __noinline__ void activation_issue(const KernelParams& p, const PhaseEntry* E, int ph,
                                              SharedCtl* sc, __nv_bfloat16* xs, int tid) {
    if (tid >= 32) return;
    const mb_phase& P = E->rec;
    const int cells = P.i[MB_GV_I_CELLS];
    const bool waits = (cells & MB_CELLS_X_WAIT) != 0;  // x was written earlier in this launch
    const int rows = P.i[MB_GV_I_ROWS];
    const int K = P.i[MB_GV_I_K];
    const int xpitch = K + 32;
    const bool gather = P.i[MB_GV_I_GATHER] != 0;
    const bool normed = P.i[MB_GV_I_PROLOGUE] != MB_PRO_NONE;
    const bool plain = !(cells & MB_CELLS_X);
    const unsigned int row_bytes = static_cast<unsigned int>(K) * 2u;
    const int lane = tid;
    if (sc->abort_flag) return;  // a faulted CTA arms nothing (part 2 will not wait)
    if (activation_arms(P)) {
        if (lane == 0) {
            // The destination was last touched by ordinary loads and stores: hand it to the
            // async proxy.  All bytes of the phase are expected on one barrier phase; the norm
            // weights (they depend on nothing in this launch) are requested at once, the rows
            // below when their producers are done.
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive_expect_tx(&sc->act_full,
                                  row_bytes * static_cast<unsigned int>((plain ? rows : 0) + (normed ? 1 : 0)));
            if (normed)  // the norm weights travel as row number `rows`
                bulk_copy_g2s(xs + static_cast<size_t>(rows) * xpitch,
                              reinterpret_cast<const char*>(entry_address(p, E, MB_GV_S_NORM_W)),
                              row_bytes, &sc->act_full);
        }
    }
    if (waits) {
        // lane 0 polls one counter until every CTA has reported the producing phase finished
        if (lane == 0) finished_wait(p, sc, ph, P.i[MB_GV_I_X_SOURCE]);
        __syncwarp();
        if (sc->abort_flag) return;
    }
    if (!plain) return;
    const char* xbase = reinterpret_cast<const char*>(entry_address(p, E, MB_GV_S_X));
    const long long* ids =
        gather ? reinterpret_cast<const long long*>(entry_address(p, E, MB_GV_S_IDS)) : nullptr;
    bool bad_token = false;
    const char* src = nullptr;
    if (lane < rows) src = activation_row(E, xbase, ids, lane, K, &bad_token);
    // Rows written with ordinary stores by other CTAs earlier in this launch were made visible
    // by their fence and this warp's acquire; the bulk copies below read them through the async
    // proxy, which is ordered after that by this fence.
    if (waits) asm volatile("fence.proxy.async.global;" ::: "memory");
    __syncwarp();
    if (src != nullptr)
        bulk_copy_g2s(xs + static_cast<size_t>(lane) * xpitch, src, row_bytes, &sc->act_full);
    if (__any_sync(0xffffffffu, bad_token) && lane == 0)
        record_status(p.ctl, MB_ST_TOKEN_RANGE, ph, blockIdx.x);
}

__device__ __forceinline__ void wait_activation_copies(const KernelParams& p, int ph, SharedCtl* sc,
                                                       unsigned int round) {
    if (!mbar_wait_bounded(&sc->act_full, round & 1u, &sc->abort_flag, sc->limit_ns)) {
        if (!sc->abort_flag) {
            record_status(p.ctl, MB_ST_PIPE_TIMEOUT, ph, blockIdx.x);
            sc->abort_flag = 1;
        }
        // fall through: the rows are garbage, the CTA drains at the end of the phase
    }
}

// Eight raw bf16 values of the gathered (un-normalised) rows go to the residual stream, as
// plain bf16 or as four cells.
__device__ __forceinline__ void store_gathered(char* store, bool cells, unsigned int tag,
                                               size_t element, uint4 raw) {
    if (cells) {
        char* c = store + element * 4;
        st_cell(c, raw.x, tag);
        st_cell(c + 8, raw.y, tag);
        st_cell(c + 16, raw.z, tag);
        st_cell(c + 24, raw.w, tag);
    } else {
        *reinterpret_cast<uint4*>(store + element * 2) = raw;
    }
}

__device__ __noinline__ void activation_finish(const KernelParams& p, const PhaseEntry* E, int ph,
                                               SharedCtl* sc, __nv_bfloat16* xs, unsigned int round,
                                               int tid) {
    const mb_phase& P = E->rec;
    const int rows = P.i[MB_GV_I_ROWS];
    const int K = P.i[MB_GV_I_K];
    const int xpitch = K + 32;
    const int pro = P.i[MB_GV_I_PROLOGUE];
    const bool gather = P.i[MB_GV_I_GATHER] != 0;
    const float embed_scale = P.f[MB_GV_F_EMBED_SCALE];
    const bool scaled = gather && embed_scale != 0.f;
    const bool store_x = gather && P.i[MB_GV_I_STORE_X] && blockIdx.x == 0;
    const bool store_cells = (P.i[MB_GV_I_CELLS] & MB_CELLS_XSTORE) != 0;
    const unsigned int tag = sc->tag_base + static_cast<unsigned int>(ph) + 1u;
    const int warp = tid >> 5, lane = tid & 31;
    const int vec_per_row = K / 8;  // 16-byte vectors
    const __nv_bfloat16* wrow = xs + static_cast<size_t>(rows) * xpitch;  // staged norm weights
    wait_activation_copies(p, ph, sc, round);

    if (rows >= 2 && (pro != MB_PRO_NONE || gather)) {
        // one warp per row: sum of squares and normalisation of a row need no CTA barrier
        // between them
        char* store = store_x ? reinterpret_cast<char*>(entry_address(p, E, MB_GV_S_XSTORE))
                              : nullptr;
        for (int r = warp; r < rows; r += kConsumerWarps) {
            __nv_bfloat16* row = xs + static_cast<size_t>(r) * xpitch;
            float ss = 0.f;
            for (int v = lane; v < vec_per_row; v += 32) {
                uint4* cell = reinterpret_cast<uint4*>(row + v * 8);
                uint4 raw = *cell;
                if (scaled) {
                    raw = scale_vector(raw, embed_scale);
                    *cell = raw;
                }
                ss += sum_squares(raw);
                if (store_x)
                    store_gathered(store, store_cells, tag, static_cast<size_t>(r) * K + v * 8, raw);
            }
            if (pro != MB_PRO_NONE) {
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                const float inv = 1.0f / sqrtf(ss / static_cast<float>(K) + P.f[MB_GV_F_EPS]);
                for (int v = lane; v < vec_per_row; v += 32) {
                    uint4* cell = reinterpret_cast<uint4*>(row + v * 8);
                    *cell = normalise_vector(*cell, *reinterpret_cast<const uint4*>(wrow + v * 8),
                                             inv, pro);
                }
            }
        }
        named_barrier(kBarConsumers, kConsumerThreads);
        return;
    }

    if (scaled || store_x || pro != MB_PRO_NONE) {
        // every thread works on its own vectors in both passes
        char* store = store_x ? reinterpret_cast<char*>(entry_address(p, E, MB_GV_S_XSTORE))
                              : nullptr;
        for (int r = 0; r < rows; ++r) {
            float ss = 0.f;
            for (int v = tid; v < vec_per_row; v += kConsumerThreads) {
                uint4* cell = reinterpret_cast<uint4*>(xs + static_cast<size_t>(r) * xpitch + v * 8);
                uint4 raw = *cell;
                if (scaled) {
                    raw = scale_vector(raw, embed_scale);
                    *cell = raw;
                }
                ss += sum_squares(raw);
                if (store_x)  // the residual stream needs the un-normalised rows
                    store_gathered(store, store_cells, tag, static_cast<size_t>(r) * K + v * 8, raw);
            }
            if (pro != MB_PRO_NONE) {
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                if (lane == 0) sc->red[warp][r] = ss;
            }
        }
        if (pro != MB_PRO_NONE) {
            named_barrier(kBarConsumers, kConsumerThreads);
            for (int r = 0; r < rows; ++r) {
                float total = 0.f;
#pragma unroll
                for (int w = 0; w < kConsumerWarps; ++w) total += sc->red[w][r];
                const float inv = 1.0f / sqrtf(total / static_cast<float>(K) + P.f[MB_GV_F_EPS]);
                for (int v = tid; v < vec_per_row; v += kConsumerThreads) {
                    uint4* cell =
                        reinterpret_cast<uint4*>(xs + static_cast<size_t>(r) * xpitch + v * 8);
                    *cell = normalise_vector(*cell, *reinterpret_cast<const uint4*>(wrow + v * 8),
                                             inv, pro);
                }
            }
        }
    }
    named_barrier(kBarConsumers, kConsumerThreads);
}

// Two packed pairs of bf16 values (four elements) through the RMSNorm.
__device__ __forceinline__ uint2 normalise_quad(uint2 x, uint2 w, float inv, int kind) {
    unsigned int xv[2] = {x.x, x.y};
    const unsigned int wv[2] = {w.x, w.y};
#pragma unroll
    for (int q = 0; q < 2; ++q) {
        float a = lo_bf16(xv[q]), b = hi_bf16(xv[q]);
        const float wa = lo_bf16(wv[q]), wb = hi_bf16(wv[q]);
        if (kind == MB_PRO_RMS_LLAMA) {
            a = bf16_round(a * inv) * wa;
            b = bf16_round(b * inv) * wb;
        } else {
            a = (a * inv) * (1.0f + wa);
            b = (b * inv) * (1.0f + wb);
        }
        xv[q] = pack_bf16(a, b);
    }
    return make_uint2(xv[0], xv[1]);
}

// Activation rows that arrive as flagged cells, written by other CTAs earlier in this launch:
// every thread loads its share of the cells (two per 16-byte load, four loads in flight) and
// retries the ones that do not yet carry the producing phase's sequence number -- the wait for
// the producers and the fetch of their data are one round trip through L2.  The values go to
// shared memory as plain bf16 rows; sums of squares are gathered on the way.
// A row is shared by `S` warps (8 for one row, 4 for two, 2 for up to four, else 1), each lane
// works on the same quads in both passes, so RMSNorm needs a CTA barrier only when S > 1.
__device__ __noinline__ void activation_cells(const KernelParams& p, const PhaseEntry* E, int ph,
                                              SharedCtl* sc, __nv_bfloat16* xs, unsigned int round,
                                              int tid) {
    const mb_phase& P = E->rec;
    const int rows = P.i[MB_GV_I_ROWS];
    const int K = P.i[MB_GV_I_K];
    const int xpitch = K + 32;
    const int pro = P.i[MB_GV_I_PROLOGUE];
    const unsigned int tag = sc->tag_base + static_cast<unsigned int>(P.i[MB_GV_I_X_SOURCE]) + 1u;
    const int warp = tid >> 5, lane = tid & 31;
    const int quads = K / 4;  // 16-byte loads (two cells, four values) per row
    const int S = rows >= 5 ? 1 : (rows >= 3 ? 2 : (rows == 2 ? 4 : 8));
    const int r = warp / S, s = warp - r * S;
    const bool works = r < rows;
    const char* src = reinterpret_cast<const char*>(entry_address(p, E, MB_GV_S_X)) +
                      static_cast<size_t>(r) * K * 4;
    __nv_bfloat16* row = xs + static_cast<size_t>(r) * xpitch;
    const int first = s * 32 + lane, step = 32 * S;
    float ss = 0.f;
    // warp 0 has waited for the producers in activation_issue; the others wait for warp 0
    if (P.i[MB_GV_I_CELLS] & MB_CELLS_X_WAIT) named_barrier(kBarConsumers, kConsumerThreads);
    if (works) {
        constexpr int kInFlight = 8;
        for (int j0 = first; j0 < quads; j0 += kInFlight * step) {
            unsigned long long c[kInFlight][2];
#pragma unroll
            for (int u = 0; u < kInFlight; ++u) {
                const int j = j0 + u * step;
                if (j < quads) ld_cell_pair(src + static_cast<size_t>(j) * 16, c[u][0], c[u][1]);
            }
#pragma unroll
            for (int u = 0; u < kInFlight; ++u) {
                const int j = j0 + u * step;
                if (j < quads) {
                    if (cell_tag(c[u][0]) != tag || cell_tag(c[u][1]) != tag)
                        cell_pair_wait(src + static_cast<size_t>(j) * 16, tag, c[u][0], c[u][1], p,
                                       sc, ph);
                    const unsigned int lo = cell_data(c[u][0]), hi = cell_data(c[u][1]);
                    const float a0 = lo_bf16(lo), a1 = hi_bf16(lo), a2 = lo_bf16(hi), a3 = hi_bf16(hi);
                    ss += a0 * a0;
                    ss += a1 * a1;
                    ss += a2 * a2;
                    ss += a3 * a3;
                    *reinterpret_cast<uint2*>(row + 4 * j) = make_uint2(lo, hi);
                }
            }
        }
    }
    if (pro != MB_PRO_NONE) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (S > 1) {
            if (lane == 0) sc->red[warp][0] = ss;
            named_barrier(kBarConsumers, kConsumerThreads);
            ss = 0.f;
            for (int w = 0; w < S; ++w) ss += sc->red[min(r, rows - 1) * S + w][0];
        }
        wait_activation_copies(p, ph, sc, round);  // the norm weights (row number `rows`)
        if (works) {
            const float inv = 1.0f / sqrtf(ss / static_cast<float>(K) + P.f[MB_GV_F_EPS]);
            const __nv_bfloat16* wrow = xs + static_cast<size_t>(rows) * xpitch;
            for (int j = first; j < quads; j += step) {
                uint2* cell = reinterpret_cast<uint2*>(row + 4 * j);
                *cell = normalise_quad(*cell, *reinterpret_cast<const uint2*>(wrow + 4 * j), inv, pro);
            }
        }
    }
    named_barrier(kBarConsumers, kConsumerThreads);
}

// ---------------------------------------------------------------------------------------
// Consumer side of a GEMV phase.
// ---------------------------------------------------------------------------------------
struct EpilogueCtx {
    char* out[3];
    const char* bias[3];
    const char* residual;
    int n[3];
    int epilogue;
    bool out_cells, res_cells;
    unsigned int tag, res_tag;
};

// One lane's pair of neighbouring results: token `gid`, output rows v and v + 1 (v even, both in
// the same segment because segment sizes are even).  Operands that come from global memory are
// fetched before the reduction loop so that their latency hides behind it.
struct PairIO {
    char* out;             // address of the pair: a cell, or two bf16
    const char* res;       // address of the residual pair (a cell, or two bf16)
    unsigned long long residual;  // what was loaded from there
    unsigned int bias;     // packed bf16 pair, 0 if absent
    bool live;
};

__device__ __forceinline__ PairIO locate_pair(const EpilogueCtx& e, int token, int vrow, bool live) {
    PairIO io;
    io.live = live;
    io.out = nullptr;
    io.res = nullptr;
    io.residual = 0ull;
    io.bias = 0u;
    if (!live) return io;
    int local = vrow, n = e.n[0];
    char* out = e.out[0];
    const char* bias = e.bias[0];
    if (local >= e.n[0]) {  // segment lookup without dynamically indexed arrays
        local -= e.n[0];
        n = e.n[1];
        out = e.out[1];
        bias = e.bias[1];
        if (local >= e.n[1]) {
            local -= e.n[1];
            n = e.n[2];
            out = e.out[2];
            bias = e.bias[2];
        }
    }
    const size_t index = static_cast<size_t>(token) * n + local;  // even
    io.out = out + index * (e.out_cells ? 4 : 2);
    if (bias != nullptr) io.bias = __ldg(reinterpret_cast<const unsigned int*>(bias + local * 2));
    if (e.epilogue == MB_EPI_RESIDUAL) {
        io.res = e.residual + index * (e.res_cells ? 4 : 2);
        io.residual = e.res_cells ? ld_cell(io.res) : static_cast<unsigned long long>(ld_cg_u32(io.res));
    }
    return io;
}

__device__ __forceinline__ void store_pair(const KernelParams& p, SharedCtl* sc, int ph,
                                           const EpilogueCtx& e, PairIO& io, float acc0, float acc1,
                                           float pair0, float pair1) {
    const float y0 = bf16_round(acc0 + lo_bf16(io.bias));
    const float y1 = bf16_round(acc1 + hi_bf16(io.bias));
    float r0, r1;
    switch (e.epilogue) {
        case MB_EPI_RESIDUAL: {
            if (e.res_cells && cell_tag(io.residual) != e.res_tag)
                io.residual = cell_wait(io.res, e.res_tag, p, sc, ph);
            const unsigned int res = cell_data(io.residual);
            r0 = lo_bf16(res) + y0;
            r1 = hi_bf16(res) + y1;
            break;
        }
        case MB_EPI_SILU_MUL:
            r0 = bf16_round(silu_f32(y0)) * bf16_round(pair0);
            r1 = bf16_round(silu_f32(y1)) * bf16_round(pair1);
            break;
        case MB_EPI_GELU_TANH_MUL:
            r0 = bf16_round(gelu_tanh_f32(y0)) * bf16_round(pair0);
            r1 = bf16_round(gelu_tanh_f32(y1)) * bf16_round(pair1);
            break;
        default:
            r0 = y0;
            r1 = y1;
            break;
    }
    const unsigned int packed = pack_bf16(r0, r1);
    if (e.out_cells)
        st_cell(io.out, packed, e.tag);
    else
        *reinterpret_cast<unsigned int*>(io.out) = packed;
}

// All consumer warps work on every stage together, in ring order (so no warp is ever more
// than one mbarrier phase behind the slot it waits on).  A stage holds SUBS tiles of 8 weight
// rows x k_chunk elements: the gate and up rows of a paired phase (PAIRED), or 16 consecutive
// output rows of a plain one (SUBS == 2, rows of at most 1,024 elements: more bytes per stage
// and so more bytes in flight per SM), or 8 rows.  The 32-element groups of a stage are dealt
// round-robin to the 8 warps.  A = activations (row = token), B = weights (n = weight row); the
// reduction index is permuted identically in both so that every lane reads 16 contiguous bytes
// per group.  Each warp parks its partial sums of a block in shared memory; once a group of
// blocks is through, one CTA barrier lets warp w add up the eight partials of block w and run
// that block's epilogue.  That is one barrier pair per 8 (SUBS == 2: 4) blocks instead of a
// reduction per stage.
template <int SUBS, bool PAIRED>
__device__ __noinline__ bool gemv_consume(const KernelParams& p, const PhaseEntry* E, int ph,
                                          SharedCtl* sc, const __nv_bfloat16* xs, float* red,
                                          const char* ring, unsigned int& it,
                                          unsigned int act_round, int tid) {
    static_assert(!PAIRED || SUBS == 2, "a paired phase stages two tiles");
    constexpr int NB = SUBS == 1 ? 8 : 4;     // blocks per reduction group
    constexpr int PV = 2 * SUBS;              // partial values per lane and block
    constexpr int OUTS = PAIRED ? 1 : SUBS;   // result pairs per lane and block
    constexpr int RT = 8 * OUTS;              // output rows per block
    const int cta = blockIdx.x;
    const GemvGeom g = gemv_geometry(E->rec, cta);
    trace_stamp(p, ph, 7, tid);
    const int warp = tid >> 5, lane = tid & 31;
    const int gid = lane >> 2, tq = lane & 3;
    const int xpitch = g.K + 32;
    const __nv_bfloat16* xrow = xs + static_cast<size_t>(min(gid, g.rows - 1)) * xpitch + 8 * tq;
    const int cells = E->rec.i[MB_GV_I_CELLS];

    EpilogueCtx e;
    e.epilogue = E->rec.i[MB_GV_I_EPILOGUE];
    e.out_cells = (cells & MB_CELLS_OUT) != 0;
    e.res_cells = (cells & MB_CELLS_RESIDUAL) != 0;
    e.tag = sc->tag_base + static_cast<unsigned int>(ph) + 1u;
    e.res_tag = sc->tag_base + static_cast<unsigned int>(E->rec.i[MB_GV_I_RES_SOURCE]) + 1u;
#pragma unroll
    for (int s = 0; s < 3; ++s) {
        e.n[s] = g.n[s];
        e.out[s] = s < g.nseg ? reinterpret_cast<char*>(entry_address(p, E, MB_GV_S_OUT0 + s))
                              : nullptr;
        e.bias[s] = (s < g.nseg && E->rec.slot[MB_GV_S_BIAS0 + s] >= 0)
                        ? reinterpret_cast<const char*>(entry_address(p, E, MB_GV_S_BIAS0 + s))
                        : nullptr;
    }
    e.residual = e.epilogue == MB_EPI_RESIDUAL
                     ? reinterpret_cast<const char*>(entry_address(p, E, MB_GV_S_RESIDUAL))
                     : nullptr;

    bool dead = false;
    bool staged = false;  // activation rows not yet waited for / normalised
    // ring position: one division per phase, then counted up
    int stage = static_cast<int>(it % static_cast<unsigned int>(p.stages));
    unsigned int wraps = it / static_cast<unsigned int>(p.stages);
    for (int group0 = 0; group0 < g.n_blocks; group0 += NB) {
        const int nb = min(NB, g.n_blocks - group0);
        // The block this warp finalises, this lane's result pairs in it and their global
        // epilogue operands: requested now, used after the reduction.
        PairIO io[OUTS];
#pragma unroll
        for (int o = 0; o < OUTS; ++o) {
            const int v = g.r0 + (group0 + warp) * RT + 8 * o + 2 * tq;
            io[o] = locate_pair(e, gid, v, warp < nb && gid < g.rows && v < g.r1);
        }

        if (!staged) {
            if (cells & MB_CELLS_X)
                activation_cells(p, E, ph, sc, const_cast<__nv_bfloat16*>(xs), act_round, tid);
            else
                activation_finish(p, E, ph, sc, const_cast<__nv_bfloat16*>(xs), act_round, tid);
            staged = true;
        }
        for (int b = 0; b < nb; ++b) {
            // two accumulator sets per tile keep the MMA dependency chains short
            float acc[SUBS][4][4];
#pragma unroll
            for (int m = 0; m < SUBS; ++m)
#pragma unroll
                for (int u = 0; u < 4; ++u)
#pragma unroll
                    for (int q = 0; q < 4; ++q) acc[m][u][q] = 0.f;
            // a plain 16-row block whose second tile is past the CTA's rows multiplies one tile
            const bool both = PAIRED || SUBS == 1 ||
                              g.r1 - (g.r0 + (group0 + b) * RT) > kRowTile;

            for (int c = 0; c < g.n_chunks; ++c) {
                const int this_stage = stage;
                const unsigned int parity = wraps & 1u;
                ++it;
                if (++stage == p.stages) {
                    stage = 0;
                    ++wraps;
                }
                if (group0 == 0 && b == 0 && c == 0) trace_stamp(p, ph, 6, tid);
                // A wait that runs out must not make this warp leave: the others would hang
                // at the next CTA barrier.  It records the fault, and every warp then falls
                // through the remaining loops without waiting or computing.
                // (the bounded wait itself watches the CTA's abort flag while it spins)
                if (dead || !mbar_wait_bounded(&sc->full[this_stage], parity, &sc->abort_flag,
                                               sc->limit_ns)) {
                    if (!dead && !sc->abort_flag) {
                        record_status(p.ctl, MB_ST_PIPE_TIMEOUT, ph, cta);
                        sc->abort_flag = 1;
                    }
                    dead = true;
                    continue;
                }
                if (group0 == 0 && b == 0 && c == 0) trace_stamp(p, ph, 4, tid);
                const int kc = min(g.k_chunk, g.K - c * g.k_chunk);
                const char* wrow = ring + static_cast<size_t>(this_stage) * p.stage_bytes +
                                   static_cast<size_t>(gid) * g.pitch + 16 * tq;
                const __nv_bfloat16* xk = xrow + c * g.k_chunk;
                const int groups = kc >> 5;  // 32 reduction elements per group
                // groups are taken two at a time onto four independent accumulator sets: the
                // tensor-core latency of this MMA shape is long, the dependent chain must be short
                for (int grp = warp; grp < groups; grp += 2 * kConsumerWarps) {
                    const int grp2 = grp + kConsumerWarps;
                    const bool second = grp2 < groups;
                    const uint4 a = *reinterpret_cast<const uint4*>(xk + 32 * grp);
                    const uint4 a2 = second ? *reinterpret_cast<const uint4*>(xk + 32 * grp2)
                                            : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
                    for (int m = 0; m < SUBS; ++m) {
                        if (m == 1 && !both) break;
                        const char* wm = wrow + static_cast<size_t>(m) * kRowTile * g.pitch;
                        const uint4 w = *reinterpret_cast<const uint4*>(wm + 64 * grp);
                        const uint4 w2 = second ? *reinterpret_cast<const uint4*>(wm + 64 * grp2)
                                                : make_uint4(0u, 0u, 0u, 0u);
                        mma_bf16_16816(acc[m][0], a.x, 0u, a.y, 0u, w.x, w.y);
                        mma_bf16_16816(acc[m][1], a.z, 0u, a.w, 0u, w.z, w.w);
                        mma_bf16_16816(acc[m][2], a2.x, 0u, a2.y, 0u, w2.x, w2.y);
                        mma_bf16_16816(acc[m][3], a2.z, 0u, a2.w, 0u, w2.z, w2.w);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&sc->empty[this_stage]);
            }
            float* cell = red + (static_cast<size_t>(b * kConsumerWarps + warp) * 32 + lane) * PV;
#pragma unroll
            for (int m = 0; m < SUBS; ++m) {
                cell[2 * m] = (acc[m][0][0] + acc[m][1][0]) + (acc[m][2][0] + acc[m][3][0]);
                cell[2 * m + 1] = (acc[m][0][1] + acc[m][1][1]) + (acc[m][2][1] + acc[m][3][1]);
            }
        }
        if (group0 == 0) trace_stamp(p, ph, 5, tid);
        named_barrier(kBarConsumers, kConsumerThreads);
        if (warp < nb && !dead) {
            float total[PV];
#pragma unroll
            for (int v = 0; v < PV; ++v) total[v] = 0.f;
#pragma unroll
            for (int w = 0; w < kConsumerWarps; ++w) {
                const float* cell =
                    red + (static_cast<size_t>(warp * kConsumerWarps + w) * 32 + lane) * PV;
#pragma unroll
                for (int v = 0; v < PV; ++v) total[v] += cell[v];
            }
            if (PAIRED) {
                if (io[0].live) store_pair(p, sc, ph, e, io[0], total[0], total[1], total[2], total[3]);
            } else {
#pragma unroll
                for (int o = 0; o < OUTS; ++o)
                    if (io[o].live)
                        store_pair(p, sc, ph, e, io[o], total[2 * o], total[2 * o + 1], 0.f, 0.f);
            }
        }
        if (group0 + NB < g.n_blocks) named_barrier(kBarConsumers, kConsumerThreads);
    }
    if (!staged) {
        // No rows here.  Plain activations still run their prologue (CTA 0 may have to store the
        // gathered rows for the residual stream); cells are simply not read, but a bulk copy
        // of norm weights this CTA started must land before its shared memory is used again.
        if (!(cells & MB_CELLS_X)) {
            activation_finish(p, E, ph, sc, const_cast<__nv_bfloat16*>(xs), act_round, tid);
        } else if (activation_arms(E->rec)) {
            wait_activation_copies(p, ph, sc, act_round);
            named_barrier(kBarConsumers, kConsumerThreads);
        }
    }
    return !dead && !sc->abort_flag;
}

// ---------------------------------------------------------------------------------------
// Decode attention.
// ---------------------------------------------------------------------------------------
// Key chunks per (batch row, kv head): pick the count that minimises
//   waves(items over CTAs) * (rounds of 16-key blocks over the consumer warps + fixed overhead).
// Evaluated by one warp, two candidates per lane, identical in every CTA.
__device__ __forceinline__ int choose_chunks(int pairs, int nblocks, int ctas, int max_chunks,
                                             int lane) {
    int best_cost = 0x7fffffff, best_nc = 1;
#pragma unroll
    for (int rep = 0; rep < 2; ++rep) {
        const int nc = lane + 1 + 32 * rep;
        if (nc <= max_chunks && nc <= nblocks) {
            const int waves = (pairs * nc + ctas - 1) / ctas;
            const int blocks = (nblocks + nc - 1) / nc;
            const int rounds = (blocks + kConsumerWarps - 1) / kConsumerWarps;
            // per wave: block rounds + fixed prologue/merge; plus the last arriver's fold, whose
            // dependent batches of L2 loads grow with the chunk count
            const int cost = 4 * waves * (rounds + 3) + nc;
            if (cost < best_cost) {
                best_cost = cost;
                best_nc = nc;
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const int oc = __shfl_xor_sync(0xffffffffu, best_cost, o);
        const int on = __shfl_xor_sync(0xffffffffu, best_nc, o);
        if (oc < best_cost || (oc == best_cost && on < best_nc)) {
            best_cost = oc;
            best_nc = on;
        }
    }
    return best_nc;
}

// Shared scratch of the attention body (carved from the activation region):
//   qs       [8][D + 32] bf16   rotated query rows of one kv-head group
//   kn, vn   [D] bf16 each      the new (rotated) key row and the new value row
//   cs       [D] fp32           cos (first half) and sin (second half), already bf16-rounded
//   wstat    [2][8 warps][8] fp32   per-warp row maxima / row sums of the exact mode
//   fold     [8][64] + [16] fp32    chunk weights and denominators of the cross-CTA fold
//   merge    [merge_slots][group][D + 2] fp32   per-warp (max, sum, values) states
//   running  [2][group][D + 2] fp32             CTA state, ping-pong over merge rounds
//
// Two softmax modes.  The reference normalises the probabilities in fp32 and rounds them to
// bf16 *before* the value product (ops/attention.py:82-84).
//   exact  (contexts of at most `exact_keys` <= 128 keys: one CTA per (row, kv head), one
//          16-key block per warp, scores stay in registers): row max and row sum are
//          exchanged through shared memory, then bf16(exp / sum) feeds the value product --
//          the reference's rounding.
//   split  (longer contexts): online softmax per warp with unnormalised bf16 probabilities,
//          states merged across warps and, through global partials, across CTAs by the last
//          chunk to arrive.  With hundreds of keys the rounding of single probabilities
//          averages out far below one bf16 ulp of the result.
// The new key/value row is appended to the cache in global memory and, for this launch's own
// arithmetic, taken from shared memory, so nothing waits on that store.
// `Lmax` is the largest valid length of the batch (the chunk count is chosen for it); every
// (row, kv head) item reads its own row's length, so rows may hold different numbers of keys.
template <int D, bool EXACT>
__device__ __noinline__ void attention_body(const KernelParams& p, const PhaseEntry* E, int Lmax,
                                            int ph, SharedCtl* sc, char* scratch, int tid) {
    constexpr int QP = D + 32;  // bf16 pitch of the rotated query rows
    constexpr int DC = D / 32;  // 32-element chunks of the head dimension (QK^T)
    constexpr int DB = D / 64;  // 64-element blocks of the head dimension (PV)
    constexpr int SW = D + 2;   // floats per head state: max, sum, D values
    constexpr bool kEarlyKeys = false;      // register prefetch spills at 168 registers: off
    constexpr bool kEarlyValues = false;    // same for the value tile
    const mb_phase* P = &E->rec;
    const int B = P->i[MB_AT_I_BATCH];
    const int Hq = P->i[MB_AT_I_HEADS];
    const int Hkv = P->i[MB_AT_I_KV_HEADS];
    const int merge_slots = P->i[MB_AT_I_MERGE_SLOTS];
    const int group = Hq / Hkv;  // query heads per kv head, <= 8
    const float scale = P->f[MB_AT_F_SCALE];
    const int warp = tid >> 5, lane = tid & 31;
    const int gid = lane >> 2, tq = lane & 3;
    const int cta = blockIdx.x, ctas = gridDim.x;

    // Addresses and rarely used scalars are read from the phase entry (shared memory) where
    // they are needed instead of being kept in registers across the key loop.
    auto slot = [&](int j) { return entry_address(p, E, j); };

    const int pairs = B * Hkv;
    constexpr bool exact = EXACT;  // contexts of at most 128 keys: at most 8 blocks
    const int cells = P->i[MB_AT_I_CELLS];
    const bool in_cells = (cells & MB_CELLS_X) != 0, out_cells = (cells & MB_CELLS_OUT) != 0;
    const unsigned int in_tag =
        sc->tag_base + static_cast<unsigned int>(P->i[MB_AT_I_QKV_SOURCE]) + 1u;
    const unsigned int out_tag = sc->tag_base + static_cast<unsigned int>(ph) + 1u;
    const int* lengths = reinterpret_cast<const int*>(entry_address(p, E, MB_AT_S_LEN));
    const bool per_row = P->i[MB_AT_I_LEN_COUNT] > 1;
    // plain q, k and v written earlier in this launch: wait until their phase is finished
    // everywhere (the named barrier below, or the one before the rotation, publishes it)
    if ((cells & MB_CELLS_X_WAIT) && tid == 0 && !sc->abort_flag)
        finished_wait(p, sc, ph, P->i[MB_AT_I_QKV_SOURCE]);
    if ((cells & MB_CELLS_X_WAIT) && exact) named_barrier(kBarConsumers, kConsumerThreads);
    int nc = 1;
    if (!exact) {
        if (warp == 0) {
            const int nc_pick = choose_chunks(pairs, (Lmax + 16) >> 4, ctas,
                                              P->i[MB_AT_I_MAX_CHUNKS], lane);
            if (lane == 0) sc->bcast[0] = nc_pick;
        }
        named_barrier(kBarConsumers, kConsumerThreads);
        nc = sc->bcast[0];
    }
    const int items = pairs * nc;

    __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(scratch);
    __nv_bfloat16* kn = qs + 8 * QP;
    __nv_bfloat16* vn = kn + D;
    float* cs = reinterpret_cast<float*>(vn + D);
    float* wstat = cs + D;                         // [2][kConsumerWarps][8]
    float* fold = wstat + 2 * kConsumerWarps * 8;  // [8][64] chunk weights + denominators
    float* merge = fold + kFoldFloats;
    float* running = merge + static_cast<size_t>(merge_slots) * group * SW;
    // Split mode with 64-wide heads: every warp streams its 16-key K and V tiles through two
    // private shared-memory slots with cp.async, one tile ahead of the one it works on, so that
    // the two dependent global round trips per block leave the critical path.
    constexpr bool kStaged = D == 64 && !EXACT;
    constexpr int kKPitch = D * 2 + 64, kVPitch = D * 2 + 16;  // bank-conflict-free fragment reads
    constexpr int kTileBytes = 16 * (kKPitch + kVPitch);
    char* staging = reinterpret_cast<char*>(running + 2 * static_cast<size_t>(group) * SW) +
                    static_cast<size_t>(warp) * 2 * kTileBytes;
    const size_t key_stride = static_cast<size_t>(Hkv) * D;  // elements between keys

    for (int item = cta; item < items; item += ctas) {
        const int pair = item / nc, chunk = item - pair * nc;
        const int b = pair / Hkv, h = pair - b * Hkv;
        // this row's own length: it may need fewer chunks than the longest row
        const int L = __ldg(lengths + (per_row ? b : 0));
        const int nkeys = L + 1;
        const int nblocks = (nkeys + 15) >> 4;
        const int row_chunks = min(nc, nblocks);
        if (chunk >= row_chunks) continue;  // the whole CTA takes this branch together
        // chunk * nblocks stays far below 2^32: 32-bit division is enough
        const int blk0 = static_cast<int>(static_cast<unsigned>(chunk) * static_cast<unsigned>(nblocks) /
                                          static_cast<unsigned>(row_chunks));
        const int blk1 = static_cast<int>(static_cast<unsigned>(chunk + 1) *
                                          static_cast<unsigned>(nblocks) /
                                          static_cast<unsigned>(row_chunks));
        const size_t cache_row0 =
            (static_cast<size_t>(b) * P->i[MB_AT_I_CAPACITY] * Hkv + h) * D;  // (b, key 0, h)
        const unsigned short* kc0 =
            reinterpret_cast<const unsigned short*>(slot(MB_AT_S_KCACHE)) + cache_row0;
        const unsigned short* vc0 =
            reinterpret_cast<const unsigned short*>(slot(MB_AT_S_VCACHE)) + cache_row0;

        // Register tiles of one 16-key block.  kt[j][i]: key kb + 8j + gid, dims 32i + 8tq..+7.
        // vt[x][q]: key kb + {2tq, 2tq+1, 2tq+8, 2tq+9}[q], dims 64x + 8gid..+7.  Only keys
        // already in the cache (< L) come from global memory; the new key (== L) is patched in
        // from shared memory and later keys are zeros (their probabilities are zero too).
        auto load_keys = [&](int blk, uint4 (&kt)[2][DC]) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int key = (blk << 4) + 8 * j + gid;
                const bool ok = key < L;
                const unsigned short* kp = kc0 + static_cast<size_t>(ok ? key : 0) * key_stride;
#pragma unroll
                for (int i = 0; i < DC; ++i)
                    kt[j][i] = ok ? *reinterpret_cast<const uint4*>(kp + 32 * i + 8 * tq)
                                  : make_uint4(0u, 0u, 0u, 0u);
            }
        };
        auto load_values = [&](int blk, uint4 (&vt)[DB][4]) {
            const int k0 = (blk << 4) + 2 * tq;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int key = k0 + (q & 1) + ((q >> 1) << 3);
                const bool ok = key < L;
                const unsigned short* vp =
                    vc0 + static_cast<size_t>(ok ? key : 0) * key_stride + 8 * gid;
#pragma unroll
                for (int x = 0; x < DB; ++x)
                    vt[x][q] = ok ? *reinterpret_cast<const uint4*>(vp + 64 * x)
                                  : make_uint4(0u, 0u, 0u, 0u);
            }
        };
        // staged variant: this warp's tile `blk` into slot `slot` (rows past the valid length
        // become zeros: their probabilities are zero, but 0 * stale bits may be NaN)
        auto issue_tile = [&](int blk, int slot) {
            char* kdst = staging + slot * kTileBytes;
            char* vdst = kdst + 16 * kKPitch;
            constexpr int kChunks = D / 8;  // 16-byte pieces per row
#pragma unroll
            for (int t = 0; t < 16 * kChunks / 32; ++t) {
                const int c = lane + 32 * t, row = c / kChunks, piece = c - row * kChunks;
                const int key = (blk << 4) + row;
                const bool ok = key < L;
                const size_t at = static_cast<size_t>(ok ? key : 0) * key_stride + piece * 8;
                cp_async16_or_zero(kdst + row * kKPitch + piece * 16, kc0 + at, ok);
                cp_async16_or_zero(vdst + row * kVPitch + piece * 16, vc0 + at, ok);
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        auto staged_keys = [&](int slot, uint4 (&kt)[2][DC]) {
            const char* kbase = staging + slot * kTileBytes;
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int i = 0; i < DC; ++i)
                    kt[j][i] = *reinterpret_cast<const uint4*>(kbase + (8 * j + gid) * kKPitch +
                                                               (32 * i + 8 * tq) * 2);
        };
        auto staged_values = [&](int slot, uint4 (&vt)[DB][4]) {
            const char* vbase = staging + slot * kTileBytes + 16 * kKPitch;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int row = 2 * tq + (q & 1) + ((q >> 1) << 3);
#pragma unroll
                for (int x = 0; x < DB; ++x)
                    vt[x][q] = *reinterpret_cast<const uint4*>(vbase + row * kVPitch +
                                                               (64 * x + 8 * gid) * 2);
            }
        };
        auto patch_new_row = [&](int blk, uint4 (&kt)[2][DC], uint4 (&vt)[DB][4]) {
            if ((L >> 4) != blk) return;
#pragma unroll
            for (int j = 0; j < 2; ++j)
                if ((blk << 4) + 8 * j + gid == L) {
#pragma unroll
                    for (int i = 0; i < DC; ++i)
                        kt[j][i] = *reinterpret_cast<const uint4*>(kn + 32 * i + 8 * tq);
                }
#pragma unroll
            for (int q = 0; q < 4; ++q)
                if ((blk << 4) + 2 * tq + (q & 1) + ((q >> 1) << 3) == L) {
#pragma unroll
                    for (int x = 0; x < DB; ++x)
                        vt[x][q] = *reinterpret_cast<const uint4*>(vn + 64 * x + 8 * gid);
                }
        };

        // ---- prologue in one memory round trip.  The raw query rows, the new key row and the
        // new value row go global -> shared with asynchronous 16-byte copies (no registers are
        // held across the trigonometry below); cos/sin are computed meanwhile; the first K/V
        // tiles are requested right after, so they fly during the barrier and the rotation.
        constexpr int kRowVectors = D / 8;  // 16-byte vectors per head row
        const int first = blk0 + warp;
        if (kStaged && in_cells) {
            // the cache tiles do not depend on this layer's projections: request the first one
            // before waiting for q, k and v
            if (first < blk1)
                issue_tile(first, 0);
            else
                asm volatile("cp.async.commit_group;" ::: "memory");
        }
        // cos / sin of this row's position: independent of the projections, so before the wait
        if (tid < D / 2) {
            const void* invf = reinterpret_cast<const void*>(slot(MB_AT_S_INVFREQ));
            const float f =
                P->i[MB_AT_I_INVFREQ_BF16] != 0
                    ? bf16_bits_to_float(reinterpret_cast<const unsigned short*>(invf)[tid])
                    : reinterpret_cast<const float*>(invf)[tid];
            const float angle =
                static_cast<float>(reinterpret_cast<const long long*>(slot(MB_AT_S_POS))[b]) * f;
            const float rope_scale = P->f[MB_AT_F_ROPE_SCALE];
            float sn, cn;
            sincosf(angle, &sn, &cn);
            cs[tid] = bf16_round(cn * rope_scale);
            cs[D / 2 + tid] = bf16_round(sn * rope_scale);
        }
        if (in_cells) {
            // q, k and v of this (row, kv head) as flagged cells of the projection phase: load,
            // retry until they carry its sequence number, park the values in shared memory
            constexpr int kRowQuads = D / 4;  // 16-byte loads (two cells, four values) per row
            for (int v = tid; v < (group + 2) * kRowQuads; v += kConsumerThreads) {
                const int row = v / kRowQuads, part = v - row * kRowQuads;
                const char* src;
                __nv_bfloat16* dst;
                if (row < group) {
                    src = reinterpret_cast<const char*>(slot(MB_AT_S_Q)) +
                          ((static_cast<size_t>(b) * Hq + h * group + row) * D + part * 4) * 4;
                    dst = qs + row * QP;
                } else if (row == group) {
                    src = reinterpret_cast<const char*>(slot(MB_AT_S_K)) +
                          ((static_cast<size_t>(b) * Hkv + h) * D + part * 4) * 4;
                    dst = kn;
                } else {
                    src = reinterpret_cast<const char*>(slot(MB_AT_S_V)) +
                          ((static_cast<size_t>(b) * Hkv + h) * D + part * 4) * 4;
                    dst = vn;
                }
                unsigned long long c0, c1;
                ld_cell_pair(src, c0, c1);
                if (cell_tag(c0) != in_tag || cell_tag(c1) != in_tag)
                    cell_pair_wait(src, in_tag, c0, c1, p, sc, ph);
                *reinterpret_cast<uint2*>(dst + part * 4) = make_uint2(cell_data(c0), cell_data(c1));
            }
        }
        for (int v = tid; !in_cells && v < (group + 2) * kRowVectors; v += kConsumerThreads) {
            const int row = v / kRowVectors, part = v - row * kRowVectors;
            const unsigned short* src;
            __nv_bfloat16* dst;
            if (row < group) {
                src = reinterpret_cast<const unsigned short*>(slot(MB_AT_S_Q)) +
                      (static_cast<size_t>(b) * Hq + h * group + row) * D;
                dst = qs + row * QP;
            } else if (row == group) {
                src = reinterpret_cast<const unsigned short*>(slot(MB_AT_S_K)) +
                      (static_cast<size_t>(b) * Hkv + h) * D;
                dst = kn;
            } else {
                src = reinterpret_cast<const unsigned short*>(slot(MB_AT_S_V)) +
                      (static_cast<size_t>(b) * Hkv + h) * D;
                dst = vn;
            }
            cp_async16(dst + part * 8, src + part * 8);
        }
        if (!in_cells) asm volatile("cp.async.commit_group;" ::: "memory");
        uint4 kt[2][DC];
        uint4 vt[DB][4];
        if (first < blk1) {
            if (kEarlyKeys) load_keys(first, kt);
            if (kEarlyValues) load_values(first, vt);
        }
        if (kStaged) {
            // the first tile flies during the barrier and the rotation below; an empty group
            // keeps the group count the same for warps without a tile
            if (!in_cells) {
                if (first < blk1)
                    issue_tile(first, 0);
                else
                    asm volatile("cp.async.commit_group;" ::: "memory");
                asm volatile("cp.async.wait_group 1;" ::: "memory");  // the prologue rows only
            }
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        named_barrier(kBarConsumers, kConsumerThreads);
        // rotate in place: thread e owns the element pair (i, i + D/2) of row e / (D/2); rows
        // 0..group-1 are query heads, row `group` is the new key
        const bool appends = chunk == row_chunks - 1;  // the chunk that holds key L stores the new row
        const size_t new_row = cache_row0 + static_cast<size_t>(L) * key_stride;
        const float q_scale = P->f[MB_AT_F_Q_SCALE];
        unsigned short* kcache = reinterpret_cast<unsigned short*>(slot(MB_AT_S_KCACHE));
        for (int e = tid; e < (group + 1) * (D / 2); e += kConsumerThreads) {
            const int gq = e / (D / 2), i = e - gq * (D / 2);
            __nv_bfloat16* row = gq == group ? kn : qs + gq * QP;
            const float x1 = __bfloat162float(row[i]), x2 = __bfloat162float(row[i + D / 2]);
            const float c = cs[i], sn = cs[D / 2 + i];
            float r1 = bf16_round(bf16_round(x1 * c) + bf16_round(-x2 * sn));
            float r2 = bf16_round(bf16_round(x2 * c) + bf16_round(x1 * sn));
            if (gq != group && q_scale != 0.f && q_scale != 1.f) {
                r1 = bf16_round(r1 * q_scale);
                r2 = bf16_round(r2 * q_scale);
            }
            row[i] = __float2bfloat16_rn(r1);
            row[i + D / 2] = __float2bfloat16_rn(r2);
            if (gq == group && appends) {
                kcache[new_row + i] = float_to_bf16_bits(r1);
                kcache[new_row + i + D / 2] = float_to_bf16_bits(r2);
            }
        }
        if (appends && tid < D)
            reinterpret_cast<unsigned short*>(slot(MB_AT_S_VCACHE))[new_row + tid] =
                reinterpret_cast<unsigned short*>(vn)[tid];
        named_barrier(kBarConsumers, kConsumerThreads);
        trace_stamp(p, ph, 4, tid);

        // QK^T: A = rotated queries (row = head of the group), B = keys (n = key).  The head
        // dimension is permuted identically in both operands so that every lane fetches 16
        // contiguous bytes of its key per 32-element chunk.
        uint4 qf[DC];
#pragma unroll
        for (int i = 0; i < DC; ++i)
            qf[i] = gid < group ? *reinterpret_cast<const uint4*>(qs + gid * QP + 32 * i + 8 * tq)
                                : make_uint4(0u, 0u, 0u, 0u);
        float m_run = -INFINITY, l_run = 0.f;
        // PV^T: A = V^T (row = head dim, via byte-permute of per-key vectors), B = P^T, which
        // is the score fragment as it stands.  acc[x][mt]: dims 64x + 8*gid + 2*mt (+1),
        // heads 2*tq (+1).
        float acc[DB][4][4];
#pragma unroll
        for (int x = 0; x < DB; ++x)
#pragma unroll
            for (int mt = 0; mt < 4; ++mt)
#pragma unroll
                for (int q = 0; q < 4; ++q) acc[x][mt][q] = 0.f;

        // scores of one block: sv[2j + q] <-> head gid, key kb + 8j + 2tq + q; bf16-rounded
        // product, scale applied in fp32, keys past the valid length masked
        auto block_scores = [&](int kb, const uint4 (&kt_)[2][DC], float (&sv)[4]) {
            float frag[2][4], frag2[2][4];  // two independent chains per tile, added at the end
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                frag[j][0] = frag[j][1] = frag[j][2] = frag[j][3] = 0.f;
                frag2[j][0] = frag2[j][1] = frag2[j][2] = frag2[j][3] = 0.f;
            }
#pragma unroll
            for (int i = 0; i < DC; ++i)
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    mma_bf16_16816(frag[j], qf[i].x, 0u, qf[i].y, 0u, kt_[j][i].x, kt_[j][i].y);
                    mma_bf16_16816(frag2[j], qf[i].z, 0u, qf[i].w, 0u, kt_[j][i].z, kt_[j][i].w);
                }
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                frag[j][0] += frag2[j][0];
                frag[j][1] += frag2[j][1];
            }
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    const int key = kb + 8 * j + 2 * tq + q;
                    const float sval = bf16_round(frag[j][q]) * scale;
                    sv[2 * j + q] = key < nkeys ? sval : -INFINITY;
                }
        };
        // acc += V^T P^T for one block; pb0/pb1 = probabilities of keys (2tq, 2tq+1) and
        // (8+2tq, 9+2tq) of head gid, packed bf16
        auto block_values = [&](const uint4 (&vt_)[DB][4], unsigned int pb0, unsigned int pb1) {
#pragma unroll
            for (int x = 0; x < DB; ++x) {
                const unsigned int ra[4] = {vt_[x][0].x, vt_[x][0].y, vt_[x][0].z, vt_[x][0].w};
                const unsigned int rb[4] = {vt_[x][1].x, vt_[x][1].y, vt_[x][1].z, vt_[x][1].w};
                const unsigned int rc[4] = {vt_[x][2].x, vt_[x][2].y, vt_[x][2].z, vt_[x][2].w};
                const unsigned int rd[4] = {vt_[x][3].x, vt_[x][3].y, vt_[x][3].z, vt_[x][3].w};
#pragma unroll
                for (int mt = 0; mt < 4; ++mt) {
                    const unsigned int a0 = __byte_perm(ra[mt], rb[mt], 0x5410u);
                    const unsigned int a1 = __byte_perm(ra[mt], rb[mt], 0x7632u);
                    const unsigned int a2 = __byte_perm(rc[mt], rd[mt], 0x5410u);
                    const unsigned int a3 = __byte_perm(rc[mt], rd[mt], 0x7632u);
                    mma_bf16_16816(acc[x][mt], a0, a1, a2, a3, pb0, pb1);
                }
            }
        };

        if (exact) {
            // one block per warp at most; warps without a block still join the two exchanges
            const bool has = first < blk1;
            float sv[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            if (has) {
                if (!kEarlyKeys) load_keys(first, kt);
                if (!kEarlyValues) load_values(first, vt);
                patch_new_row(first, kt, vt);
                block_scores(first << 4, kt, sv);
            }
            float rmax = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
            rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, 1));
            rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, 2));
            if (tq == 0) wstat[warp * 8 + gid] = rmax;
            named_barrier(kBarConsumers, kConsumerThreads);
            float row_max = -INFINITY;
#pragma unroll
            for (int w = 0; w < kConsumerWarps; ++w) row_max = fmaxf(row_max, wstat[w * 8 + gid]);
            float ev[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) ev[q] = expf(sv[q] - row_max);  // 0 for masked keys
            float rsum = (ev[0] + ev[1]) + (ev[2] + ev[3]);
            rsum += __shfl_xor_sync(0xffffffffu, rsum, 1);
            rsum += __shfl_xor_sync(0xffffffffu, rsum, 2);
            if (tq == 0) wstat[(kConsumerWarps + warp) * 8 + gid] = rsum;
            named_barrier(kBarConsumers, kConsumerThreads);
            float row_sum = 0.f;
#pragma unroll
            for (int w = 0; w < kConsumerWarps; ++w)
                row_sum += wstat[(kConsumerWarps + w) * 8 + gid];
            if (has)  // normalised probabilities rounded to bf16, as the eager operator does
                block_values(vt, pack_bf16(ev[0] / row_sum, ev[1] / row_sum),
                             pack_bf16(ev[2] / row_sum, ev[3] / row_sum));
            // already normalised: merge as plain sums (max 0, total weight 1)
            m_run = 0.f;
            l_run = (warp == 0 && tq == 0) ? 1.f : 0.f;
        } else {
            // online softmax, one 16-key block per iteration, the next block requested ahead
            uint4 kt_next[2][DC];
            uint4 vt_next[DB][4];
            int slot = 0;
            for (int blk = first; blk < blk1; blk += kConsumerWarps) {
                const int kb = blk << 4;
                const int following = blk + kConsumerWarps;
                if (kStaged) {
                    if (following < blk1) {
                        issue_tile(following, slot ^ 1);
                        asm volatile("cp.async.wait_group 1;" ::: "memory");
                    } else {
                        asm volatile("cp.async.wait_group 0;" ::: "memory");
                    }
                    __syncwarp();  // every lane's pieces of the current tile have landed
                    staged_keys(slot, kt);
                    staged_values(slot, vt);
                    __syncwarp();  // the slot may be refilled from the next iteration on
                    slot ^= 1;
                } else {
                    if (!kEarlyKeys) load_keys(blk, kt);
                    if (!kEarlyValues) load_values(blk, vt);
                }
                if (following < blk1) {
                    if (kEarlyKeys) load_keys(following, kt_next);
                    if (kEarlyValues) load_values(following, vt_next);
                }
                patch_new_row(blk, kt, vt);
                float sv[4];
                block_scores(kb, kt, sv);
                float bmax = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
                bmax = fmaxf(bmax, __shfl_xor_sync(0xffffffffu, bmax, 1));
                bmax = fmaxf(bmax, __shfl_xor_sync(0xffffffffu, bmax, 2));
                const float m_new = fmaxf(m_run, bmax);
                const float alpha = expf(m_run - m_new);
                float pv[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) pv[q] = expf(sv[q] - m_new);
                l_run = l_run * alpha + ((pv[0] + pv[1]) + (pv[2] + pv[3]));
                m_run = m_new;
                // rescale factors of the two heads this lane accumulates (columns 2tq, 2tq+1)
                const float alpha0 = __shfl_sync(0xffffffffu, alpha, (2 * tq) * 4);
                const float alpha1 = __shfl_sync(0xffffffffu, alpha, (2 * tq + 1) * 4);
#pragma unroll
                for (int x = 0; x < DB; ++x)
#pragma unroll
                    for (int mt = 0; mt < 4; ++mt) {
                        acc[x][mt][0] *= alpha0;
                        acc[x][mt][1] *= alpha1;
                        acc[x][mt][2] *= alpha0;
                        acc[x][mt][3] *= alpha1;
                    }
                block_values(vt, pack_bf16(pv[0], pv[1]), pack_bf16(pv[2], pv[3]));
                if (following < blk1) {
                    if (kEarlyKeys) {
#pragma unroll
                        for (int j = 0; j < 2; ++j)
#pragma unroll
                            for (int i = 0; i < DC; ++i) kt[j][i] = kt_next[j][i];
                    }
                    if (kEarlyValues) {
#pragma unroll
                        for (int x = 0; x < DB; ++x)
#pragma unroll
                            for (int q = 0; q < 4; ++q) vt[x][q] = vt_next[x][q];
                    }
                }
            }
        }
        l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
        l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
        trace_stamp(p, ph, 5, tid);

        // ---- merge the warp states into one CTA state, `merge_slots` warps per round
        const int rounds = (kConsumerWarps + merge_slots - 1) / merge_slots;
        for (int round = 0; round < rounds; ++round) {
            const int lead = round * merge_slots;
            if (warp >= lead && warp < lead + merge_slots) {
                float* base = merge + static_cast<size_t>(warp - lead) * group * SW;
                if (tq == 0 && gid < group) {
                    base[gid * SW] = m_run;
                    base[gid * SW + 1] = l_run;
                }
                const int h0 = 2 * tq, h1 = 2 * tq + 1;
#pragma unroll
                for (int x = 0; x < DB; ++x)
#pragma unroll
                    for (int mt = 0; mt < 4; ++mt) {
                        const int d = 64 * x + 8 * gid + 2 * mt;
                        if (h0 < group) {
                            base[h0 * SW + 2 + d] = acc[x][mt][0];
                            base[h0 * SW + 2 + d + 1] = acc[x][mt][2];
                        }
                        if (h1 < group) {
                            base[h1 * SW + 2 + d] = acc[x][mt][1];
                            base[h1 * SW + 2 + d + 1] = acc[x][mt][3];
                        }
                    }
            }
            named_barrier(kBarConsumers, kConsumerThreads);
            const int live = min(merge_slots, kConsumerWarps - lead);
            const float* prev = running + static_cast<size_t>((round & 1) ^ 1) * group * SW;
            float* next = running + static_cast<size_t>(round & 1) * group * SW;
            for (int e = tid; e < group * SW; e += kConsumerThreads) {
                const int gq = e / SW, col = e - gq * SW;
                float mx = round == 0 ? -INFINITY : prev[gq * SW];
                for (int w = 0; w < live; ++w)
                    mx = fmaxf(mx, merge[(static_cast<size_t>(w) * group + gq) * SW]);
                float sum_l = 0.f, sum_v = 0.f;
                if (round > 0) {
                    const float wgt = __expf(prev[gq * SW] - mx);
                    sum_l = prev[gq * SW + 1] * wgt;
                    sum_v = prev[gq * SW + col] * wgt;
                }
                for (int w = 0; w < live; ++w) {
                    const float* st = merge + (static_cast<size_t>(w) * group + gq) * SW;
                    // weights between partial softmax states: no rounding point of the operator
                    // sits here, the fast exponential is accurate to 2^-21
                    const float wgt = __expf(st[0] - mx);  // 0 for a warp that saw no block
                    sum_l += st[1] * wgt;
                    sum_v += st[col] * wgt;
                }
                next[e] = col == 0 ? mx : (col == 1 ? sum_l : sum_v);
            }
            named_barrier(kBarConsumers, kConsumerThreads);
        }
        const float* state = running + static_cast<size_t>((rounds - 1) & 1) * group * SW;
        trace_stamp(p, ph, 6, tid);

        // results leave in pairs of neighbouring elements: one 4-byte store, or one cell
        char* out = reinterpret_cast<char*>(slot(MB_AT_S_OUT));
        auto store_out = [&](int gq, int d, float v0, float v1) {
            const size_t index = (static_cast<size_t>(b) * Hq + h * group + gq) * D + d;
            const unsigned int packed = pack_bf16(v0, v1);
            if (out_cells)
                st_cell(out + index * 4, packed, out_tag);
            else
                *reinterpret_cast<unsigned int*>(out + index * 2) = packed;
        };
        if (row_chunks == 1) {
            for (int e = tid; e < group * (D / 2); e += kConsumerThreads) {
                const int gq = e / (D / 2), d = 2 * (e - gq * (D / 2));
                const float denom_ = state[gq * SW + 1];
                store_out(gq, d, state[gq * SW + 2 + d] / denom_, state[gq * SW + 3 + d] / denom_);
            }
        } else {
            float* partial = reinterpret_cast<float*>(slot(MB_AT_S_PARTIAL));
            int* counter = reinterpret_cast<int*>(slot(MB_AT_S_COUNTER));
            const int max_chunks = P->i[MB_AT_I_MAX_CHUNKS];
            float* mine = partial + (static_cast<size_t>(pair) * max_chunks + chunk) * group * SW;
            for (int e = tid; e < group * SW; e += kConsumerThreads) mine[e] = state[e];
            __threadfence();
            named_barrier(kBarConsumers, kConsumerThreads);
            if (tid == 0) {
                const int arrived = atomicAdd(counter + pair, 1);
                __threadfence();
                sc->bcast[1] = arrived;
            }
            named_barrier(kBarConsumers, kConsumerThreads);
            trace_stamp(p, ph, 7, tid);
            const int nc_row = row_chunks;
            if (sc->bcast[1] == nc_row - 1) {
                // Last chunk of this (row, kv head) to arrive folds all chunks, in chunk order.
                // Step 1: (max, sum) of every chunk into shared memory, all loads in flight
                // together, then the per-chunk weights and the denominator.
                const float* all = partial + static_cast<size_t>(pair) * max_chunks * group * SW;
                float* weight = fold;          // [group][nc] chunk maxima, then weights
                float* denom = fold + 8 * 64;  // [group]
                float* sums = merge;           // [group][nc] chunk sums (merge slots are free)
                for (int e = tid; e < group * nc_row; e += kConsumerThreads) {
                    const int gq = e / nc_row, c = e - gq * nc_row;
                    const float* st = all + (static_cast<size_t>(c) * group + gq) * SW;
                    weight[e] = ld_cg_f32(st);
                    sums[e] = ld_cg_f32(st + 1);
                }
                named_barrier(kBarConsumers, kConsumerThreads);
                if (tid < group) {
                    float mx = -INFINITY;
                    for (int c = 0; c < nc_row; ++c) mx = fmaxf(mx, weight[tid * nc_row + c]);
                    float total = 0.f;
                    for (int c = 0; c < nc_row; ++c) {
                        const float wgt = expf(weight[tid * nc_row + c] - mx);
                        weight[tid * nc_row + c] = wgt;
                        total += sums[tid * nc_row + c] * wgt;
                    }
                    denom[tid] = total;
                }
                named_barrier(kBarConsumers, kConsumerThreads);
                // Step 2: weighted sums of the value partials, two neighbouring elements per
                // thread; loads are independent.
                for (int e = tid; e < group * (D / 2); e += kConsumerThreads) {
                    const int gq = e / (D / 2), d = 2 * (e - gq * (D / 2));
                    const float* col = all + static_cast<size_t>(gq) * SW + 2 + d;
                    float sum0 = 0.f, sum1 = 0.f;
                    for (int c0 = 0; c0 < nc_row; c0 += 8) {  // eight loads in flight per batch
                        float2 part[8];
#pragma unroll
                        for (int u = 0; u < 8; ++u)
                            part[u] = c0 + u < nc_row
                                          ? __ldcg(reinterpret_cast<const float2*>(
                                                col + static_cast<size_t>(c0 + u) * group * SW))
                                          : make_float2(0.f, 0.f);
#pragma unroll
                        for (int u = 0; u < 8; ++u)
                            if (c0 + u < nc_row) {
                                const float wgt = weight[gq * nc_row + c0 + u];
                                sum0 += part[u].x * wgt;
                                sum1 += part[u].y * wgt;
                            }
                    }
                    store_out(gq, d, sum0 / denom[gq], sum1 / denom[gq]);
                }
                if (tid == 0) counter[pair] = 0;  // ready for the next launch
            }
        }
        named_barrier(kBarConsumers, kConsumerThreads);  // scratch is reused by the next item
    }
}

// Reads the valid lengths (one shared by the batch, or one per row), refuses a full cache --
// every thread of every CTA sees the same lengths, so all of them take the same branch -- and
// picks the softmax mode from the longest row.  The two modes are separate functions so that a
// launch only ever executes one of them: instruction-cache footprint matters more here than
// code sharing.  The lengths do not change during a launch (they are advanced when it ends).
template <int D>
__device__ __forceinline__ void attention_decode(const KernelParams& p, const PhaseEntry* E,
                                                 int ph, SharedCtl* sc, char* scratch, int tid) {
    const int* lenp = reinterpret_cast<const int*>(entry_address(p, E, MB_AT_S_LEN));
    const int count = E->rec.i[MB_AT_I_LEN_COUNT] > 1 ? E->rec.i[MB_AT_I_BATCH] : 1;
    const int capacity = E->rec.i[MB_AT_I_CAPACITY];
    int longest = 0, bad = 0, bad_length = 0;
    for (int r = 0; r < count; ++r) {
        const int L = __ldg(lenp + r);
        if (L < 0 || L + 1 > capacity) {
            bad = 1;
            bad_length = L;
        }
        longest = max(longest, L);
    }
    if (bad) {
        if (tid == 0) {
            record_status(p.ctl, MB_ST_KV_OVERFLOW, ph, bad_length);
            sc->abort_flag = 1;
        }
        return;
    }
    if (longest + 1 <= E->rec.i[MB_AT_I_EXACT_KEYS])
        attention_body<D, true>(p, E, longest, ph, sc, scratch, tid);
    else
        attention_body<D, false>(p, E, longest, ph, sc, scratch, tid);
}

// ---------------------------------------------------------------------------------------
// The kernel.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void prefetch_entry(const PhaseEntry* src, PhaseEntry* dst, int tid) {
    // 16-byte asynchronous copies global -> shared of one phase entry
    if (src != nullptr && tid < kEntryVectors) {
        const unsigned int d = smem_u32(reinterpret_cast<char*>(dst) + 16 * tid);
        const char* g = reinterpret_cast<const char*>(src) + 16 * tid;
        asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(d), "l"(g) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}

// Thread 0, at the start of phase `ph`: fetch the counter of phase ph - 2 from L2 (not L1: other
// SMs add to it) into shared memory, in the same group as the entry prefetch, so that the check
// at the end of the phase finds it there without a round trip of its own.
__device__ __forceinline__ void prefetch_guard(const KernelParams& p, SharedCtl* sc, int ph) {
    const unsigned int d = smem_u32(sc->guard);
    const void* g = &p.ctl->finished[(ph - 2) & 3];
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(g) : "memory");
}

// Every thread waits for its own copies; the 16-byte vectors of one address pair (two slots)
// were copied by one thread, which then patches them -- no extra barrier is needed before the
// CTA barrier that publishes the entry.
__device__ __forceinline__ void wait_entry(const KernelParams& p, PhaseEntry* dst, int tid) {
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (dst == nullptr) return;
    constexpr int kFirstAddrVector = offsetof(PhaseEntry, addr) / 16;
    static_assert(offsetof(PhaseEntry, addr) % 16 == 8, "addr[] starts mid-vector");
    // vector kFirstAddrVector holds addr[0] in its upper half; vector v > that holds
    // addr[2 (v - first) - 1] and addr[2 (v - first)]
    if (tid >= kFirstAddrVector && tid < kEntryVectors) {
        const int hi = 2 * (tid - kFirstAddrVector), lo = hi - 1;
        if (lo >= 0 && lo < MB_PHASE_SLOTS) dst->addr[lo] = resolve_dynamic(p, dst->addr[lo]);
        if (hi < MB_PHASE_SLOTS) dst->addr[hi] = resolve_dynamic(p, dst->addr[hi]);
    }
}

__global__ void __launch_bounds__(kThreads, 1)
decode_kernel(const __grid_constant__ KernelParams p) {
    extern __shared__ __align__(128) char smem[];
    SharedCtl* sc = reinterpret_cast<SharedCtl*>(smem);
    float* red = reinterpret_cast<float*>(smem + kCtlBytes);
    char* act = smem + kFixedBytes;
    char* ring = act + p.activation_bytes;
    const int tid = threadIdx.x;

    if (tid == 0) {
        for (int s = 0; s < kMaxStages; ++s) {
            mbar_init(&sc->full[s], 1);
            mbar_init(&sc->empty[s], kConsumerWarps);
        }
        mbar_init(&sc->act_full, 1);
        sc->abort_flag = peek_status(p.ctl) != 0 ? 1 : 0;  // a faulted plan runs nothing
        sc->issued = 0;
        sc->limit_ns = static_cast<unsigned long long>(p.wait_limit_us) * 1000ull;
        // Both words only change after the closing barrier of a launch (or by a host reset).
        const unsigned int calls = *reinterpret_cast<volatile unsigned int*>(&p.ctl->calls);
        const unsigned int epoch = *reinterpret_cast<volatile unsigned int*>(&p.ctl->epoch);
        sc->tag_base = epoch * static_cast<unsigned int>(p.n_phases);
        sc->calls = calls;
        mbar_init_fence();
    }
    if (tid < kConsumerThreads) {
        prefetch_entry(p.entries, &sc->entry[0], tid);
        wait_entry(p, &sc->entry[0], tid);
    }
    __syncthreads();
    if (sc->abort_flag) return;

    if (tid >= kConsumerThreads) {
        producer_loop(p, sc, ring, tid & 31);
    } else {
        const unsigned int calls = *reinterpret_cast<volatile unsigned int*>(&p.ctl->calls);
        const unsigned int base = calls * static_cast<unsigned int>(p.barriers_per_launch);
        unsigned int it = 0;
        unsigned int act_round = 0;  // GEMV phases run so far: parity of the activation barrier
        int barrier_index = 0;
        bool ok = true;
        // Optional per-phase trace: thread 0 of every CTA stamps the global timer at phase
        // start (0), after the activation copies were started (1), after the body (2) and after
        // the closing grid barrier, if the phase has one (3).
        auto stamp = [&](int ph, int event) {
            if (p.trace != nullptr && tid == 0)
                p.trace[(static_cast<size_t>(blockIdx.x) * p.n_phases + ph) * kTraceEvents + event] =
                    global_timer_ns();
        };
        for (int ph = 0; ph < p.n_phases && ok; ++ph) {
            // The entry of this phase is in shared memory already; fetch the next one now so
            // that no phase starts with a dependent chain of global loads.
            const PhaseEntry* E = &sc->entry[ph & 1];
            const bool more = ph + 1 < p.n_phases;
            if (ph >= 2 && tid == 0) prefetch_guard(p, sc, ph);
            prefetch_entry(more ? p.entries + ph + 1 : nullptr, &sc->entry[(ph + 1) & 1], tid);
            stamp(ph, 0);
            switch (E->rec.body) {
                case MB_BODY_NOP:
                    break;
                case MB_BODY_GEMV: {
                    __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(act);
                    activation_issue(p, E, ph, sc, xs, tid);
                    stamp(ph, 1);
                    if (E->rec.i[MB_GV_I_NMAT] == 2)
                        gemv_consume<2, true>(p, E, ph, sc, xs, red, ring, it, act_round, tid);
                    else if (E->rec.i[MB_GV_I_ROW_TILE] == 2 * kRowTile)
                        gemv_consume<2, false>(p, E, ph, sc, xs, red, ring, it, act_round, tid);
                    else
                        gemv_consume<1, false>(p, E, ph, sc, xs, red, ring, it, act_round, tid);
                    if (activation_arms(E->rec)) ++act_round;
                    break;
                }
                case MB_BODY_ATTN_DECODE: {
                    const int D = E->rec.i[MB_AT_I_HEAD_DIM];
                    if (D == 64)
                        attention_decode<64>(p, E, ph, sc, act, tid);
                    else if (D == 128)
                        attention_decode<128>(p, E, ph, sc, act, tid);
                    else
                        attention_decode<256>(p, E, ph, sc, act, tid);
                    break;
                }
                default:
                    if (tid == 0) {
                        record_status(p.ctl, MB_ST_BAD_PHASE, ph, E->rec.body);
                        sc->abort_flag = 1;
                    }
                    break;
            }
            // Whether to go on is decided once per CTA, by thread 0 inside the barrier below
            // (a fault raises the CTA's abort flag; bodies never leave early on their own
            // except for conditions every thread evaluates identically).
            stamp(ph, 2);
            const int flags = E->rec.flags;
            wait_entry(p, more ? &sc->entry[(ph + 1) & 1] : nullptr, tid);  // published by the barrier below
            if (ph >= 2 && tid == 0 && !sc->abort_flag) {
                const unsigned int target = finished_target(p, sc, ph - 2);
                if (static_cast<int>(sc->guard[0] - target) < 0) finished_wait(p, sc, ph, ph - 2);
            }
            if (flags & MB_FLAG_BARRIER) {
                ++barrier_index;
                ok = grid_barrier(p.ctl, base + barrier_index, kBarConsumers, kConsumerThreads, tid,
                                  &sc->abort_flag, &sc->verdict, ph, sc->limit_ns);
                stamp(ph, 3);
            } else {
                // one CTA barrier: every warp is done with the phase's shared memory, and all of
                // them learn together whether one of them raised the abort flag
                ok = !named_barrier_or(kBarConsumers, kConsumerThreads, sc->abort_flag != 0);
            }
            // This CTA has finished phase `ph` (all its loads of the phase's inputs are done):
            // counted for the CTAs that are about to leave phase ph + 2.  No ordering is needed
            // beyond the CTA barrier above.
            if (ok && tid == 0) {
                // plain results that a later phase fetches after waiting on this counter: make
                // the CTA's stores (ordered before this point by the CTA barrier) visible first
                if (flags & MB_FLAG_FENCE) asm volatile("fence.acq_rel.gpu;" ::: "memory");
                asm volatile("red.relaxed.gpu.global.add.u32 [%0], 1;" ::"l"(
                                 &p.ctl->finished[ph & 3].count)
                             : "memory");
            }
        }
        if (ok) {
            // Closing barrier: every CTA has read the valid lengths, `calls` and `epoch` and is
            // done with them; CTA 0 may now advance them.
            ++barrier_index;
            ok = grid_barrier(p.ctl, base + barrier_index, kBarConsumers, kConsumerThreads, tid,
                              &sc->abort_flag, &sc->verdict, p.n_phases, sc->limit_ns);
            // a launch that recorded a fault anywhere (a token outside the table ...) leaves the
            // lengths and the launch counters alone: the host has to reset the plan anyway
            if (ok && blockIdx.x == 0 && peek_status(p.ctl) == 0) {
                // valid_length += 1 for every attention phase that asks for it, one thread per
                // phase (the table is in L2: the producers prefetched it)
                for (int q = tid; q < p.n_phases; q += kConsumerThreads) {
                    const PhaseEntry* G = p.entries + q;
                    if (G->rec.body != MB_BODY_ATTN_DECODE || !(G->rec.flags & MB_FLAG_BUMP_LENGTH))
                        continue;
                    int* lenp = reinterpret_cast<int*>(resolve_dynamic(p, G->addr[MB_AT_S_LEN]));
                    const int count = G->rec.i[MB_AT_I_LEN_COUNT] > 1 ? G->rec.i[MB_AT_I_BATCH] : 1;
                    for (int r = 0; r < count; ++r) lenp[r] = lenp[r] + 1;
                }
                if (tid == 0) {
                    p.ctl->calls = calls + 1;
                    p.ctl->epoch = *reinterpret_cast<volatile unsigned int*>(&p.ctl->epoch) + 1u;
                }
            }
        }
    }

    // Drain: never leave while one of this CTA's bulk copies is still in flight.  After an
    // abort the producer stopped issuing; wait (bounded) for every stage it armed.
    __syncthreads();
    if (sc->abort_flag && tid == 0) {
        const unsigned int issued = sc->issued;
        const unsigned int first = issued > static_cast<unsigned int>(p.stages)
                                       ? issued - p.stages : 0u;
        for (unsigned int s = first; s < issued; ++s) {
            const int stage = s % p.stages;
            const unsigned int parity = (s / p.stages) & 1u;
            for (unsigned int tries = 0; tries < kDrainTryLimit; ++tries)
                if (mbar_try_wait(&sc->full[stage], parity)) break;
        }
    }
}

}  // namespace decode

int decode_threads() { return decode::kThreads; }
int decode_fixed_smem() { return decode::kFixedBytes; }
int decode_stage_bytes() { return decode::kStageBytes; }
int decode_max_stages() { return decode::kMaxStages; }
int decode_row_pad() { return decode::kRowPad; }
int decode_row_tile() { return decode::kRowTile; }

cudaError_t decode_configure(int smem_bytes) {
    return cudaFuncSetAttribute(decode::decode_kernel,
                                cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
}

cudaError_t decode_occupancy(int smem_bytes, int* blocks_per_sm) {
    return cudaOccupancyMaxActiveBlocksPerMultiprocessor(blocks_per_sm, decode::decode_kernel,
                                                         decode::kThreads, smem_bytes);
}

cudaError_t decode_launch(const KernelParams& params, int ctas, int smem_bytes,
                          cudaStream_t stream) {
    KernelParams copy = params;
    void* args[] = {&copy};
    return cudaLaunchCooperativeKernel(reinterpret_cast<void*>(decode::decode_kernel), dim3(ctas),
                                       dim3(decode::kThreads), args,
                                       static_cast<size_t>(smem_bytes), stream);
}

}  // namespace mb

// =======================================================================================
// Decode attention without any allocation.
//
// Some hosts may not allocate device memory at the point where they need one attention
// step: a plugin called from inside someone else's stream-ordered pipeline, a process that
// runs inside a fixed amount of memory handed out at start-up, a caller inside a region where
// cudaMalloc would synchronise the device.  For them this entry point runs the same
// attention body as the plan path, but everything the plan path keeps in allocated memory
// (phase table, control block, split-key partials, arrival counters) lives either in the
// kernel parameters or in one fixed-size array inside this library's device image.
//
// The array is a file-scope `static __device__` object of kStaticScratchBytes (4 MiB); every
// GPU that loads the library holds it until the process exits.  In host code its name is only
// a host-side stand-in, not a device address: the address the kernel gets is asked for once
// per device with cudaGetSymbolAddress, with that device current.
//
// All calls share the array.  The arrival counters and the control words are cleared on the
// stream before every launch; the partials need no clearing (they are written before they
// are read).  Two calls that overlap on the GPU (different streams, no dependency) race on
// it -- callers serialise them.
// =======================================================================================
namespace mb {
namespace decode {

constexpr size_t kStaticScratchBytes = 4u << 20;
constexpr size_t kStaticControlBytes = 256;        // status words of Control + "CTAs done" counter
// The attention body only touches Control::status through the pointer it is given (record_status,
// peek_status); those words must lie inside the first 128 bytes, before the "done" counter.
static_assert(offsetof(Control, status) + sizeof(int) * 4 <= 128,
              "the status words must precede the done counter of the static control area");
constexpr size_t kStaticCounterBytes = 4096;       // arrival counters: up to 1024 (row, kv head)
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

__global__ void __launch_bounds__(kConsumerThreads, 1)
attention_static_kernel(const __grid_constant__ PhaseEntry entry, Control* ctl, int* done,
                        int* status_out) {
    extern __shared__ __align__(128) char smem[];
    SharedCtl* sc = reinterpret_cast<SharedCtl*>(smem);
    char* scratch = smem + kCtlBytes;
    const int tid = threadIdx.x;
    if (tid < kEntryVectors)
        reinterpret_cast<uint4*>(&sc->entry[0])[tid] = reinterpret_cast<const uint4*>(&entry)[tid];
    if (tid == 0) {
        sc->abort_flag = 0;
        sc->tag_base = 0;
        sc->calls = 0;
        sc->limit_ns = kPipeTimeoutNs;
    }
    __syncthreads();
    KernelParams p;
    p.entries = nullptr;
    p.ctl = ctl;
    p.trace = nullptr;
    p.n_phases = 1;
    p.n_dynamic = 0;
    p.barriers_per_launch = 0;
    p.stages = 0;
    p.stage_bytes = 0;
    p.activation_bytes = 0;
    p.wait_limit_us = 2000000u;
    const PhaseEntry* E = &sc->entry[0];
    const int D = E->rec.i[MB_AT_I_HEAD_DIM];
    if (D == 64)
        attention_decode<64>(p, E, 0, sc, scratch, tid);
    else if (D == 128)
        attention_decode<128>(p, E, 0, sc, scratch, tid);
    else
        attention_decode<256>(p, E, 0, sc, scratch, tid);
    __syncthreads();
    if (tid == 0) {
        // The valid length may only move once every CTA has read it: the last CTA to finish
        // advances it, reports the status and re-arms the counter for the next call.
        __threadfence();
        const int finished = atomicAdd(done, 1);
        if (finished == static_cast<int>(gridDim.x) - 1) {
            __threadfence();
            const int code = *reinterpret_cast<volatile int*>(&ctl->status[0]);
            if (code == 0) {
                int* lenp = reinterpret_cast<int*>(E->addr[MB_AT_S_LEN]);
                *lenp = *lenp + 1;
            }
            if (status_out != nullptr) *status_out = code;
            *done = 0;
        }
    }
}

struct StaticDevice {
    unsigned char* scratch = nullptr;  // device address of g_static_scratch on this device
    int sm_count = 0;
    int max_smem = 0;
    bool ready = false;
};

}  // namespace decode
}  // namespace mb

namespace {
mb::decode::StaticDevice g_static_devices[64];
std::mutex g_static_mutex;

long long static_attention_smem(int head_dim, int group, int merge_slots) {
    return mb::decode::kCtlBytes + 8LL * (head_dim + 32) * 2 + 2LL * head_dim * 2 + 4LL * head_dim +
           4LL * (2 * 8 * 8 + mb::decode::kFoldFloats) +
           4LL * (head_dim + 2) * group * (merge_slots + 2) +
           (head_dim == 64 ? 8LL * 2 * 16 * ((head_dim * 2 + 64) + (head_dim * 2 + 16)) : 0);
}
}  // namespace

// Declared in include/megabake_b200.h.  The first call on a device performs the one-time
// set-up (symbol address, kernel attribute); make that call before any stream capture.
extern "C" int mb_attention_decode_static(const mb_attention_args* a, void* stream) {
    using namespace mb::decode;
    if (a == nullptr) return MB_ERR_INVALID;
    if (a->batch < 1 || a->heads < 1 || a->kv_heads < 1 || a->capacity < 1) return MB_ERR_INVALID;
    if (a->heads % a->kv_heads != 0 || a->heads / a->kv_heads > 8) return MB_ERR_UNSUPPORTED;
    if (a->head_dim != 64 && a->head_dim != 128 && a->head_dim != 256) return MB_ERR_UNSUPPORTED;
    const unsigned long long pointers[] = {a->query, a->key, a->value, a->key_cache,
                                           a->value_cache, a->valid_length, a->position_ids,
                                           a->inv_freq, a->out};
    for (unsigned long long ptr : pointers)
        if (ptr == 0) return MB_ERR_INVALID;
    if ((a->query | a->key | a->value | a->key_cache | a->value_cache | a->out) & 15ull)
        return MB_ERR_INVALID;
    if ((a->position_ids & 7ull) || (a->valid_length & 3ull) || (a->inv_freq & 3ull) ||
        (a->status & 3ull))
        return MB_ERR_INVALID;

    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return MB_ERR_CUDA;
    StaticDevice& dev = g_static_devices[device];
    {
        std::lock_guard<std::mutex> lock(g_static_mutex);
        if (!dev.ready) {
            void* address = nullptr;
            cudaError_t err = cudaGetSymbolAddress(&address, g_static_scratch);
            if (err != cudaSuccess || address == nullptr) return MB_ERR_CUDA;
            cudaDeviceProp prop;
            if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return MB_ERR_CUDA;
            if (prop.major != 10) return MB_ERR_UNSUPPORTED;
            dev.max_smem = 160 * 1024;
            if (cudaFuncSetAttribute(attention_static_kernel,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     dev.max_smem) != cudaSuccess)
                return MB_ERR_CUDA;
            dev.scratch = static_cast<unsigned char*>(address);
            dev.sm_count = prop.multiProcessorCount;
            dev.ready = true;
        }
    }

    const int group = a->heads / a->kv_heads;
    const int pairs = a->batch * a->kv_heads;
    int merge_slots = 8;
    while (merge_slots > 1 &&
           static_attention_smem(a->head_dim, group, merge_slots) - kCtlBytes -
                   (a->head_dim == 64 ? 8 * 2 * 16 * ((64 * 2 + 64) + (64 * 2 + 16)) : 0) >
               48 * 1024)
        merge_slots /= 2;
    if (static_attention_smem(a->head_dim, group, merge_slots) > dev.max_smem) return MB_ERR_RESOURCE;
    // What fits the fixed array: arrival counters for every (row, kv head) and at least one
    // key chunk of partials each; more chunks if there is room, up to 32.
    if (static_cast<size_t>(pairs) * 4 > kStaticCounterBytes) return MB_ERR_RESOURCE;
    const size_t per_chunk = static_cast<size_t>(pairs) * group * (a->head_dim + 2) * 4;
    const size_t room = kStaticScratchBytes - kStaticControlBytes - kStaticCounterBytes;
    if (per_chunk > room) return MB_ERR_RESOURCE;  // shapes beyond the 4 MiB scratch
    int max_chunks = static_cast<int>(room / per_chunk);
    if (max_chunks > 32) max_chunks = 32;
    const int by_capacity = (a->capacity + 15) / 16;
    if (max_chunks > by_capacity) max_chunks = by_capacity;

    mb::PhaseEntry entry;
    std::memset(&entry, 0, sizeof(entry));
    entry.rec.body = MB_BODY_ATTN_DECODE;
    entry.rec.i[MB_AT_I_BATCH] = a->batch;
    entry.rec.i[MB_AT_I_HEADS] = a->heads;
    entry.rec.i[MB_AT_I_KV_HEADS] = a->kv_heads;
    entry.rec.i[MB_AT_I_HEAD_DIM] = a->head_dim;
    entry.rec.i[MB_AT_I_CAPACITY] = a->capacity;
    entry.rec.i[MB_AT_I_INVFREQ_BF16] = a->inv_freq_is_bf16 ? 1 : 0;
    entry.rec.i[MB_AT_I_MAX_CHUNKS] = max_chunks;
    entry.rec.i[MB_AT_I_MERGE_SLOTS] = merge_slots;
    entry.rec.i[MB_AT_I_EXACT_KEYS] = a->capacity < 128 ? a->capacity : 128;
    entry.rec.i[MB_AT_I_LEN_COUNT] = 1;
    entry.rec.f[MB_AT_F_SCALE] = 1.0f / sqrtf(static_cast<float>(a->head_dim));
    entry.rec.f[MB_AT_F_ROPE_SCALE] = a->rope_scale;
    entry.rec.f[MB_AT_F_Q_SCALE] = a->query_scale;
    unsigned char* control = dev.scratch;
    unsigned char* counters = dev.scratch + kStaticControlBytes;
    unsigned char* partials = counters + kStaticCounterBytes;
    entry.addr[MB_AT_S_Q] = a->query;
    entry.addr[MB_AT_S_K] = a->key;
    entry.addr[MB_AT_S_V] = a->value;
    entry.addr[MB_AT_S_KCACHE] = a->key_cache;
    entry.addr[MB_AT_S_VCACHE] = a->value_cache;
    entry.addr[MB_AT_S_LEN] = a->valid_length;
    entry.addr[MB_AT_S_POS] = a->position_ids;
    entry.addr[MB_AT_S_INVFREQ] = a->inv_freq;
    entry.addr[MB_AT_S_OUT] = a->out;
    entry.addr[MB_AT_S_PARTIAL] = reinterpret_cast<unsigned long long>(partials);
    entry.addr[MB_AT_S_COUNTER] = reinterpret_cast<unsigned long long>(counters);

    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // control words + arrival counters start every call at zero (a faulted earlier call may
    // have left them set); the partials are always written before they are read
    if (cudaMemsetAsync(control, 0, kStaticControlBytes + kStaticCounterBytes, s) != cudaSuccess)
        return MB_ERR_CUDA;
    mb::Control* ctl = reinterpret_cast<mb::Control*>(control);
    int* done = reinterpret_cast<int*>(control + 128);
    const int smem = static_cast<int>(static_attention_smem(a->head_dim, group, merge_slots));
    attention_static_kernel<<<dev.sm_count, kConsumerThreads, smem, s>>>(
        entry, ctl, done, reinterpret_cast<int*>(a->status));
    return cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_CUDA;
}
