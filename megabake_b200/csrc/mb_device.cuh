// Device-side primitives shared by the decode and prefill megakernels: bf16 rounding
// helpers, mbarrier / bulk-copy / mma wrappers, bounded waits, the counting grid barrier
// and the status word.  sm_100a only.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/megabake_b200.h"

namespace mb {

// ---------------------------------------------------------------------------------------
// Control block in global memory, one per plan.
// ---------------------------------------------------------------------------------------
constexpr int kBarrierLanes = 8;
struct Control {
    unsigned int epoch;     // base of the hand-off sequence numbers: grows with every completed
                            // launch and every reset, so that no cell of an earlier launch can
                            // ever be mistaken for one of this launch
    unsigned int calls;     // completed launches; the barrier targets derive from it
    int status[4];          // code, phase, detail, (unused)
    unsigned int pad0[26];
    // CTAs that finished a phase: a ring of four counters (a line each), phase q counts on
    // counter q % 4.  Every CTA, before it leaves phase q, waits until all CTAs have finished
    // phase q - 2; so no CTA is ever more than two phases ahead of another, a counter never
    // mixes arrivals of two phases, and a cell buffer may be overwritten from the third phase
    // after its last reader on.
    struct Finished {
        unsigned int count;
        unsigned int pad[31];
    } finished[4];
    // Counting grid barrier, spread over eight counters 128 bytes apart: CTA c arrives on
    // counter c % 8, so the arrivals (atomics on one address serialise in L2) proceed on eight
    // addresses at once.  Counter j grows by the number of CTAs mapped to it per barrier.
    struct Lane {
        unsigned int count;
        unsigned int pad[31];
    } lanes[kBarrierLanes];
};

// One phase as the kernel reads it: the record plus the device address of every slot it
// names, resolved by the host at bind time so that the kernel never chases a slot index
// through a second table.  A per-launch (dynamic) slot holds kDynamicTag | ordinal instead.
struct PhaseEntry {
    mb_phase rec;
    unsigned long long addr[MB_PHASE_SLOTS];
    unsigned long long pad;  // keeps sizeof a multiple of 16 (copied in 16-byte vectors)
};
static_assert(sizeof(PhaseEntry) % 16 == 0, "PhaseEntry must be a whole number of 16-byte vectors");
constexpr unsigned long long kDynamicTag = 1ull << 63;

struct KernelParams {
    const PhaseEntry* entries;
    Control* ctl;
    unsigned long long* trace;  // optional [ctas][n_phases][4] global-timer stamps, or null
    unsigned long long dyn[MB_MAX_DYNAMIC];
    int n_phases;
    int n_dynamic;
    int barriers_per_launch;
    int stages;            // weight-ring depth
    int stage_bytes;       // bytes of one ring stage
    int activation_bytes;  // shared bytes reserved for activations / attention scratch
    unsigned int wait_limit_us;  // bound of every device-side wait, microseconds
};

// Wait limits.  Every wait in the kernels is bounded: when one runs out the kernel records
// a status, raises the CTA's abort flag and drains instead of spinning forever.  The decode
// kernel takes its limit from the plan (KernelParams::wait_limit_us); these are the defaults.
constexpr unsigned long long kBarrierTimeoutNs = 2000000000ull;  // 2 s
constexpr unsigned long long kPipeTimeoutNs = 2000000000ull;     // 2 s
constexpr unsigned int kDrainTryLimit = 1000000u;                 // try_wait calls while draining

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void record_status(Control* ctl, int code, int phase, int detail) {
    if (atomicCAS(&ctl->status[0], 0, code) == 0) {
        ctl->status[1] = phase;
        ctl->status[2] = detail;
        __threadfence();
    }
}

__device__ __forceinline__ int peek_status(const Control* ctl) {
    return *reinterpret_cast<const volatile int*>(&ctl->status[0]);
}

// ---------------------------------------------------------------------------------------
// bf16 helpers.  Every rounding point of the eager forward is an explicit call here.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float bf16_round(float v) {
    return __bfloat162float(__float2bfloat16_rn(v));
}
__device__ __forceinline__ float bf16_bits_to_float(unsigned short bits) {
    return __uint_as_float(static_cast<unsigned int>(bits) << 16);
}
__device__ __forceinline__ unsigned short float_to_bf16_bits(float v) {
    return __bfloat16_as_ushort(__float2bfloat16_rn(v));
}
__device__ __forceinline__ float lo_bf16(unsigned int packed) {
    return __uint_as_float(packed << 16);
}
__device__ __forceinline__ float hi_bf16(unsigned int packed) {
    return __uint_as_float(packed & 0xffff0000u);
}
__device__ __forceinline__ unsigned int pack_bf16(float lo, float hi) {
    return static_cast<unsigned int>(float_to_bf16_bits(lo)) |
           (static_cast<unsigned int>(float_to_bf16_bits(hi)) << 16);
}

// Eight bf16 values at a time (one 16-byte vector): embedding scale, sum of squares and the
// two RMSNorm spellings.
__device__ __forceinline__ uint4 scale_vector(uint4 raw, float scale) {
    raw.x = pack_bf16(lo_bf16(raw.x) * scale, hi_bf16(raw.x) * scale);
    raw.y = pack_bf16(lo_bf16(raw.y) * scale, hi_bf16(raw.y) * scale);
    raw.z = pack_bf16(lo_bf16(raw.z) * scale, hi_bf16(raw.z) * scale);
    raw.w = pack_bf16(lo_bf16(raw.w) * scale, hi_bf16(raw.w) * scale);
    return raw;
}

__device__ __forceinline__ float sum_squares(uint4 v) {
    float s = 0.f;
    const unsigned int w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const float a = lo_bf16(w[q]), b = hi_bf16(w[q]);
        s += a * a;
        s += b * b;
    }
    return s;
}

__device__ __forceinline__ uint4 normalise_vector(uint4 x, uint4 w, float inv, int kind) {
    unsigned int xv[4] = {x.x, x.y, x.z, x.w};
    const unsigned int wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
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
    return make_uint4(xv[0], xv[1], xv[2], xv[3]);
}

// x / (1 + exp(-x)) with the operation order of the decomposed graph.
__device__ __forceinline__ float silu_f32(float x) { return x / (1.0f + expf(-x)); }
// 0.5 * x * (1 + tanh(sqrt(2/pi) * (x + 0.044715 x^3)))
__device__ __forceinline__ float gelu_tanh_f32(float x) {
    const float kBeta = 0.7978845608028654f;
    const float kKappa = 0.044715f;
    float inner = kBeta * (x + kKappa * (x * x * x));
    return 0.5f * x * (1.0f + tanhf(inner));
}

// ---------------------------------------------------------------------------------------
// Loads that bypass L1 for data another CTA produced earlier in the same launch.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 ld_cg_u4(const void* p) {
    return __ldcg(reinterpret_cast<const uint4*>(p));
}
__device__ __forceinline__ unsigned int ld_cg_u32(const void* p) {
    return __ldcg(reinterpret_cast<const unsigned int*>(p));
}
__device__ __forceinline__ unsigned short ld_cg_u16(const void* p) {
    return __ldcg(reinterpret_cast<const unsigned short*>(p));
}
__device__ __forceinline__ float ld_cg_f32(const void* p) {
    return __ldcg(reinterpret_cast<const float*>(p));
}

// ---------------------------------------------------------------------------------------
// Shared-memory addresses, named barriers, mbarriers, bulk async copies.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned int smem_u32(const void* p) {
    return static_cast<unsigned int>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void named_barrier(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Named barrier that also ORs a predicate over the arriving threads.
__device__ __forceinline__ bool named_barrier_or(int id, int threads, bool value) {
    unsigned int out;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 p, %3, 0;\n\t"
        "barrier.cta.red.or.pred q, %1, %2, p;\n\t"
        "selp.u32 %0, 1, 0, q;\n\t}"
        : "=r"(out)
        : "r"(id), "r"(threads), "r"(value ? 1u : 0u)
        : "memory");
    return out != 0;
}

// ---------------------------------------------------------------------------------------
// Flagged cells: 64 bits = two bf16 values (low word) + a 32-bit sequence number (high word),
// written and read as ONE 8-byte access, so a reader that sees the number it expects has the
// data of that very store.  Loads go to L2 (gpu scope): the cells are written by other SMs.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void st_cell(void* p, unsigned int data, unsigned int tag) {
    const unsigned long long v =
        static_cast<unsigned long long>(data) | (static_cast<unsigned long long>(tag) << 32);
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_cell(const void* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
// two neighbouring cells (16-byte aligned); each is read atomically
__device__ __forceinline__ void ld_cell_pair(const void* p, unsigned long long& a,
                                             unsigned long long& b) {
    asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];"
                 : "=l"(a), "=l"(b)
                 : "l"(p)
                 : "memory");
}
__device__ __forceinline__ unsigned int cell_tag(unsigned long long v) {
    return static_cast<unsigned int>(v >> 32);
}
__device__ __forceinline__ unsigned int cell_data(unsigned long long v) {
    return static_cast<unsigned int>(v);
}
__device__ __forceinline__ unsigned int ld_relaxed_u32(const void* p) {
    unsigned int v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count)
                 : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned long long* bar,
                                                      unsigned int bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, unsigned int parity) {
    unsigned int done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return done != 0;
}

// Bounded mbarrier wait.  `abort_flag` is a CTA-shared int that any thread raises when a
// wait of its own ran out; everybody else then stops waiting too.
__device__ __forceinline__ bool mbar_wait_bounded(unsigned long long* bar, unsigned int parity,
                                                  volatile int* abort_flag,
                                                  unsigned long long limit_ns = kPipeTimeoutNs) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long start = global_timer_ns();
    for (unsigned int tries = 1;; ++tries) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((tries & 127u) == 0u) {
            if (*abort_flag) return false;
            if (global_timer_ns() - start > limit_ns) return false;
        }
    }
}

__device__ __forceinline__ void prefetch_l2(const void* p) {
    asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}

// 1-D bulk async copy global -> shared, completion counted in bytes on an mbarrier.
// Source, destination and size must be multiples of 16 bytes.
__device__ __forceinline__ void bulk_copy_g2s(void* dst_smem, const void* src_gmem,
                                              unsigned int bytes, unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// D(16x8, fp32) += A(16x16, bf16, row) * B(16x8, bf16, col)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], unsigned int a0, unsigned int a1,
                                               unsigned int a2, unsigned int a3, unsigned int b0,
                                               unsigned int b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---------------------------------------------------------------------------------------
// Counting grid barrier.  Called by `threads` threads of every CTA (named barrier `bar_id`).
// `generation` counts barriers since the plan was created or reset (the same in every CTA).
// Lanes 0..7 of warp 0 each watch one of the eight counters; together they decide for the
// whole CTA -- go on, or drain because a wait ran out / a fault was recorded here or in
// another CTA -- and publish the decision through `verdict` in shared memory, so that every
// thread of the CTA takes the same branch afterwards.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ bool grid_barrier(Control* ctl, unsigned int generation, int bar_id,
                                             int threads, int tid, volatile int* abort_flag,
                                             volatile int* verdict, int phase,
                                             unsigned long long limit_ns = kBarrierTimeoutNs) {
    named_barrier(bar_id, threads);
    if (tid < kBarrierLanes) {
        constexpr unsigned int kMask = (1u << kBarrierLanes) - 1u;
        const unsigned int ctas = gridDim.x;
        bool go = *abort_flag == 0;
        if (go) {
            if (tid == 0) {
                // release: orders every write this CTA made before the bar.sync above
                asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(
                                 &ctl->lanes[blockIdx.x % kBarrierLanes].count)
                             : "memory");
            }
            const unsigned int mapped = ctas / kBarrierLanes +
                                        (static_cast<unsigned int>(tid) < ctas % kBarrierLanes ? 1u : 0u);
            const unsigned int target = generation * mapped;
            unsigned long long start = 0;
            unsigned int polls = 0;
            for (;;) {
                unsigned int seen;
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];"
                             : "=r"(seen)
                             : "l"(&ctl->lanes[tid].count)
                             : "memory");
                if (__all_sync(kMask, static_cast<int>(seen - target) >= 0)) break;
                if ((++polls & 63u) == 0u) {  // the eight lanes take this branch together
                    if (start == 0) start = global_timer_ns();
                    const bool faulted = peek_status(ctl) != 0 || *abort_flag != 0;
                    const bool late = global_timer_ns() - start > limit_ns;
                    if (__any_sync(kMask, faulted || late)) {
                        if (tid == 0 && !faulted)
                            record_status(ctl, MB_ST_BARRIER_TIMEOUT, phase,
                                          static_cast<int>(blockIdx.x));
                        go = false;
                        break;
                    }
                }
            }
        }
        if (tid == 0) {
            if (!go) *abort_flag = 1;
            *verdict = go ? 1 : 0;
        }
    }
    named_barrier(bar_id, threads);
    return *verdict != 0;
}

}  // namespace mb
