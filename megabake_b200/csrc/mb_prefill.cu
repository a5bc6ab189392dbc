// Prefill path: one kernel launch per phase of an MB_MODE_PREFILL plan, enqueued in order on
// the caller's stream (and captured as a whole by a CUDA graph when the caller does so).
//
//   embed_rows_kernel      gather of embedding rows (+ Gemma's bf16 scalar scale)
//   rmsnorm_block_kernel   row-wise RMSNorm, Llama and Gemma spellings, one CTA per row
//                          (rmsnorm_rows_kernel: rows longer than 8192 elements)
//   gemm_tc_persistent_kernel   C[M, N] = A[M, K] . W[N, K]^T on the 5th-generation tensor
//                          cores, one CTA per SM walking (tile, reduction slice) units:
//                          TMA (cp.async.bulk.tensor, 128-byte swizzle) -> 192 KB shared-
//                          memory ring -> tcgen05.mma issued by one thread into one of two
//                          tensor-memory accumulators -> tcgen05.ld epilogue on eight warps
//                          (bias / residual / gated activation) behind the next unit's MMAs
//   gemm_tc_kernel         the same contraction with one tile per CTA and two CTAs per SM
//                          (kept selectable: MEGABAKE_B200_GEMM_PERSISTENT=0)
//   rope_transpose_kernel  rotary embedding of q and k rows in place and, in the same launch,
//                          the transpose of v the tensor-core attention reads
//   attention_tc_kernel    masked softmax attention with the eager rounding points, S and O in
//                          tensor memory (attention_prefill_kernel: the mma.sync fallback)
//
// Every load in this file is a plain (single-CTA) TMA or cp.async load, so the library runs
// unchanged at any GPU count.  Every wait is bounded and reports through
// the plan's status word.
#include <cuda.h>
#include <cuda_runtime.h>

#include <climits>
#include <cstdlib>
#include <cmath>
#include <cstring>
#include <new>
#include <vector>

#include "mb_device.cuh"
#include "mb_kernels.h"

namespace mb {
namespace prefill {

// Programmatic dependent launch: a phase's kernel is launched while the previous phase's
// kernel is still draining, runs its prologue (barrier set-up, tensor-memory allocation)
// beside it, and blocks in chain_wait() until that kernel has completed and its writes are
// visible.  chain_release() lets the next kernel in the stream start its own prologue; in
// kernels that allocate tensor memory it comes after the allocation, so a successor never
// queues for columns ahead of a CTA of this grid.
__device__ __forceinline__ void chain_release() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void chain_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

// Two floats to a bf16 pair in one instruction (same bits as two cvt.rn.bf16.f32, checked over
// every finite float): the attention's softmax warps and the GEMM epilogue are bound by the
// instructions they issue, and packing was four of them per pair.
__device__ __forceinline__ float exp2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ unsigned int pack_bf16_pair(float lo, float hi) {
    unsigned int packed;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(packed) : "f"(hi), "f"(lo));
    return packed;
}

// ---------------------------------------------------------------------------------------
// Row kernels
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) embed_rows_kernel(const unsigned short* table,
                                                         const long long* ids,
                                                         unsigned short* out, int rows, int K,
                                                         int vocab, float scale, Control* ctl,
                                                         int phase) {
    const int r = blockIdx.x;
    chain_release();
    chain_wait();
    if (r >= rows) return;
    long long id = ids[r];
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) record_status(ctl, MB_ST_TOKEN_RANGE, phase, r);
        id = 0;
    }
    const uint4* src = reinterpret_cast<const uint4*>(table + static_cast<size_t>(id) * K);
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(r) * K);
    for (int v = threadIdx.x; v < K / 8; v += blockDim.x) {
        uint4 raw = __ldg(src + v);
        if (scale != 0.f) raw = scale_vector(raw, scale);
        dst[v] = raw;
    }
}

// One warp per row, two passes over the row (the second one hits L1/L2).
__global__ void __launch_bounds__(128) rmsnorm_rows_kernel(const unsigned short* x,
                                                           const unsigned short* w,
                                                           unsigned short* out, int rows, int K,
                                                           int kind, float eps) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.x * 4 + warp;
    chain_release();
    chain_wait();
    if (r >= rows) return;
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(r) * K);
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(r) * K);
    const uint4* wv = reinterpret_cast<const uint4*>(w);
    float ss = 0.f;
    for (int v = lane; v < K / 8; v += 32) ss += sum_squares(src[v]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = 1.0f / sqrtf(ss / static_cast<float>(K) + eps);
    for (int v = lane; v < K / 8; v += 32) dst[v] = normalise_vector(src[v], __ldg(wv + v), inv, kind);
}

// One CTA per row, the row held in registers between the sum of squares and the scaling: one
// read of x where the warp-per-row kernel makes two, at a third of its latency (these kernels
// are latency, not bandwidth: a 128-token step runs 37 of them).  Rows of up to 8192 elements.
__global__ void __launch_bounds__(256) rmsnorm_block_kernel(const unsigned short* x,
                                                            const unsigned short* w,
                                                            unsigned short* out, int K, int kind,
                                                            float eps) {
    __shared__ float partial[8];
    chain_release();
    chain_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int vectors = K / 8;
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(blockIdx.x) * K);
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(blockIdx.x) * K);
    const uint4* wv = reinterpret_cast<const uint4*>(w);
    uint4 v[4], g[4];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int idx = static_cast<int>(threadIdx.x) + j * 256;
        if (idx < vectors) {
            v[j] = src[idx];
            g[j] = __ldg(wv + idx);
            ss += sum_squares(v[j]);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) partial[warp] = ss;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) total += partial[i];
    const float inv = 1.0f / sqrtf(total / static_cast<float>(K) + eps);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int idx = static_cast<int>(threadIdx.x) + j * 256;
        if (idx < vectors) dst[idx] = normalise_vector(v[j], g[j], inv, kind);
    }
}

// One thread per (row, i): the cos / sin pair of that position and frequency is computed once
// and applied to element pair (i, i + D/2) of every q and k head of the row, with the rounding
// points of the eager graph: tables in bf16, every product and the sum rounded to bf16.
struct RopeArgs {
    unsigned short* q;
    unsigned short* k;
    const long long* pos;
    const void* inv_freq;
    int rows, heads, kv_heads, D, invfreq_bf16;
    float rope_scale, q_scale;
    int k_tokens, k_capacity;
    int* length;
    int length_value, length_count;
};

// block / blocks: this CTA's index among the CTAs that share the work
__device__ __forceinline__ void rope_rows_body(const RopeArgs& a, int block, int blocks) {
    unsigned short* q = a.q;
    unsigned short* k = a.k;
    const long long* pos = a.pos;
    const void* inv_freq = a.inv_freq;
    const int rows = a.rows, heads = a.heads, kv_heads = a.kv_heads, D = a.D;
    const int invfreq_bf16 = a.invfreq_bf16, k_tokens = a.k_tokens, k_capacity = a.k_capacity;
    const float rope_scale = a.rope_scale, q_scale = a.q_scale;
    const int half = D / 2;
    const long long total = static_cast<long long>(rows) * half;
    // state handoff: the layer's valid length(s), one shared by the batch or one per row
    if (a.length != nullptr && block == 0 && static_cast<int>(threadIdx.x) < a.length_count)
        a.length[threadIdx.x] = a.length_value;
    for (long long e = block * static_cast<long long>(blockDim.x) + threadIdx.x; e < total;
         e += static_cast<long long>(blocks) * blockDim.x) {
        const int r = static_cast<int>(e / half);
        const int i = static_cast<int>(e - static_cast<long long>(r) * half);
        const float f = invfreq_bf16
                            ? bf16_bits_to_float(reinterpret_cast<const unsigned short*>(inv_freq)[i])
                            : reinterpret_cast<const float*>(inv_freq)[i];
        const float angle = static_cast<float>(pos[r]) * f;
        float sn, cn;
        sincosf(angle, &sn, &cn);
        const float c = bf16_round(cn * rope_scale), s = bf16_round(sn * rope_scale);
        for (int head = 0; head < heads + kv_heads; ++head) {
            const bool is_q = head < heads;
            // k rows may live in a KV cache: batch b's rows start at b * capacity
            const size_t k_row = k_tokens > 0 ? static_cast<size_t>(r / k_tokens) * k_capacity + r % k_tokens
                                              : static_cast<size_t>(r);
            unsigned short* row = is_q ? q + (static_cast<size_t>(r) * heads + head) * D
                                       : k + (k_row * kv_heads + (head - heads)) * D;
            const float x1 = bf16_bits_to_float(row[i]), x2 = bf16_bits_to_float(row[i + half]);
            float r1 = bf16_round(bf16_round(x1 * c) + bf16_round(-x2 * s));
            float r2 = bf16_round(bf16_round(x2 * c) + bf16_round(x1 * s));
            if (is_q && q_scale != 0.f && q_scale != 1.f) {
                r1 = bf16_round(r1 * q_scale);
                r2 = bf16_round(r2 * q_scale);
            }
            row[i] = float_to_bf16_bits(r1);
            row[i + half] = float_to_bf16_bits(r2);
        }
    }
}

__global__ void __launch_bounds__(256) rope_rows_kernel(const RopeArgs a) {
    chain_release();
    chain_wait();
    rope_rows_body(a, blockIdx.x, gridDim.x);
}

// ---------------------------------------------------------------------------------------
// tcgen05 / TMA wrappers
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void* dst_smem, const CUtensorMap* map, int x, int y,
                                            unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(dst_smem)),
        "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tmem_alloc(unsigned int* slot_smem, unsigned int columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(slot_smem)),
                 "r"(columns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(unsigned int base, unsigned int columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns)
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// The mbarrier gets one arrival once every tcgen05.mma this thread issued before has finished.
__device__ __forceinline__ void umma_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     smem_u32(bar))
                 : "memory");
}
// D[tmem] (+)= A[smem] . B[smem]^T, bf16 operands, fp32 accumulate, M = 128.
__device__ __forceinline__ void umma_bf16(unsigned int tmem_d, unsigned long long desc_a,
                                          unsigned long long desc_b, unsigned int idesc,
                                          unsigned int accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Shared-memory operand descriptor: K-major tile of 128-byte rows, 128-byte swizzle, groups of
// 8 rows 1024 bytes apart (the layout TMA writes with CU_TENSOR_MAP_SWIZZLE_128B).
__device__ __forceinline__ unsigned long long umma_desc(unsigned int smem_addr) {
    unsigned long long d = 0;
    d |= static_cast<unsigned long long>((smem_addr & 0x3ffffu) >> 4);  // start address
    d |= 1ull << 16;                                                     // leading byte offset (unused)
    d |= static_cast<unsigned long long>(1024 >> 4) << 32;               // stride byte offset
    d |= 1ull << 46;                                                     // descriptor version
    d |= 2ull << 61;                                                     // SWIZZLE_128B
    return d;
}
// 32 consecutive fp32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_load32(unsigned int taddr, float (&v)[32]) {
    unsigned int r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// 16 consecutive fp32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_load16(unsigned int taddr, float (&v)[16]) {
    unsigned int r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// ---------------------------------------------------------------------------------------
// The GEMM
// ---------------------------------------------------------------------------------------
constexpr int kTileM = 128;
constexpr int kTileK = 64;  // bf16 elements = one 128-byte swizzle row
constexpr int kGemmThreads = 192;  // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2-5: epilogue
constexpr int kStageA = kTileM * kTileK * 2;

struct GemmMaps {
    CUtensorMap a;
    CUtensorMap w[4];  // segments 0..2, [3] = second matrix of a pair
};

struct GemmArgs {
    int M, K, kblocks, split_k, stages, phase;
    int nseg, pair, epilogue;
    int out_tokens, out_capacity;  // > 0: segments 1, 2 write row r at (r / tokens) * capacity + r % tokens
    int n[3];
    int tile_start[3];  // first n-tile of each segment
    int tiles_n;        // n-tiles over all segments
    int tiles_m;        // 128-row m-tiles (persistent kernel)
    unsigned short* out[3];
    const unsigned short* bias[3];
    const unsigned short* residual;
    float* workspace;  // split-K partials [tile][split][128][BN] fp32
    int* counters;     // split-K arrivals per tile, zero between launches
    Control* ctl;
    unsigned long long* trace;  // optional: 8 global-timer stamps of CTA (0, 0, 0), or null
};

// Epilogue, step 1: 32 accumulator columns of this thread's row -> bf16 results in the
// staging tile (shared memory, the drained operand ring).  v: accumulators of output columns
// col0.. of segment seg; u: the paired matrix's accumulators for the same columns (gated
// epilogues only).  The residual is added in step 2, where rows are read back coalesced.
__device__ __forceinline__ void gemm_stage_chunk(const GemmArgs& a, int seg, int col0, int width,
                                                 const float (&v)[32], const float (&u)[32],
                                                 unsigned char* stage_row) {
    const unsigned short* bias = a.bias[seg];
    // one uniform branch per chunk, not per element: the activation functions are long and
    // must not be evaluated speculatively for epilogues that do not use them
    float y[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        const float b = (bias != nullptr && i < width) ? bf16_bits_to_float(__ldg(bias + col0 + i)) : 0.f;
        y[i] = bf16_round(v[i] + b);
    }
    if (a.epilogue == MB_EPI_SILU_MUL) {
#pragma unroll
        for (int i = 0; i < 32; ++i) y[i] = bf16_round(silu_f32(y[i])) * bf16_round(u[i]);
    } else if (a.epilogue == MB_EPI_GELU_TANH_MUL) {
#pragma unroll
        for (int i = 0; i < 32; ++i) y[i] = bf16_round(gelu_tanh_f32(y[i])) * bf16_round(u[i]);
    }
    uint4* dst = reinterpret_cast<uint4*>(stage_row);
#pragma unroll
    for (int q = 0; q < 4; ++q)
        dst[q] = make_uint4(pack_bf16(y[8 * q], y[8 * q + 1]), pack_bf16(y[8 * q + 2], y[8 * q + 3]),
                            pack_bf16(y[8 * q + 4], y[8 * q + 5]), pack_bf16(y[8 * q + 6], y[8 * q + 7]));
}

// Epilogue, step 2: a warp writes the 32 rows it staged, 16 bytes per lane along the row.
__device__ __forceinline__ void gemm_write_rows(const GemmArgs& a, int seg, int row0, int n0,
                                                int per_tile, const unsigned char* stage,
                                                int pitch, int lane) {
    const int n = a.n[seg];
    unsigned short* out = a.out[seg];
    const unsigned short* res = a.epilogue == MB_EPI_RESIDUAL ? a.residual : nullptr;
    const int vectors = per_tile / 8;
    for (int idx = lane; idx < 32 * vectors; idx += 32) {
        const int r = idx / vectors, c = (idx - r * vectors) * 8;
        const int row = row0 + r, col = n0 + c;
        if (row >= a.M || col >= n) continue;
        uint4 t = *reinterpret_cast<const uint4*>(stage + r * pitch + c * 2);
        const size_t out_row = (seg >= 1 && a.out_tokens > 0)
                                   ? static_cast<size_t>(row / a.out_tokens) * a.out_capacity + row % a.out_tokens
                                   : static_cast<size_t>(row);
        const size_t at = out_row * n + col;
        if ((n & 7) == 0) {
            if (res != nullptr) {
                const uint4 h = *reinterpret_cast<const uint4*>(res + at);
                t.x = pack_bf16(lo_bf16(h.x) + lo_bf16(t.x), hi_bf16(h.x) + hi_bf16(t.x));
                t.y = pack_bf16(lo_bf16(h.y) + lo_bf16(t.y), hi_bf16(h.y) + hi_bf16(t.y));
                t.z = pack_bf16(lo_bf16(h.z) + lo_bf16(t.z), hi_bf16(h.z) + hi_bf16(t.z));
                t.w = pack_bf16(lo_bf16(h.w) + lo_bf16(t.w), hi_bf16(h.w) + hi_bf16(t.w));
            }
            *reinterpret_cast<uint4*>(out + at) = t;
        } else {
            const unsigned int w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if (col + i >= n) break;
                float y = i & 1 ? hi_bf16(w[i / 2]) : lo_bf16(w[i / 2]);
                if (res != nullptr) y = bf16_bits_to_float(res[at + i]) + y;
                out[at + i] = float_to_bf16_bits(y);
            }
        }
    }
}

template <int BN>
__global__ void __launch_bounds__(kGemmThreads, 2)
gemm_tc_kernel(const __grid_constant__ GemmMaps maps, const GemmArgs a) {
    constexpr int kStageW = BN * kTileK * 2;
    constexpr int kStage = kStageA + kStageW;
    constexpr int kHalf = BN / 2;  // columns per matrix of a gated pair
    extern __shared__ unsigned char smem_raw[];
    // operand tiles need 1024-byte alignment for the 128-byte swizzle
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    unsigned long long* full = reinterpret_cast<unsigned long long*>(smem + a.stages * kStage);
    unsigned long long* empty = full + 8;
    unsigned long long* accum = empty + 8;
    unsigned int* tmem_slot = reinterpret_cast<unsigned int*>(accum + 1);
    int* abort_flag = reinterpret_cast<int*>(tmem_slot + 1);
    int* last_flag = abort_flag + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool traced = a.trace != nullptr && (blockIdx.x | blockIdx.y | blockIdx.z) == 0;
    auto stamp = [&](int slot) {
        if (traced) a.trace[slot] = global_timer_ns();
    };
    if (threadIdx.x == 0) stamp(0);
    // m-tiles vary fastest: CTAs that run together share the same weight tile (read from HBM
    // once) and differ in the activation tile, which stays in L2
    const int mt = blockIdx.x, tile = blockIdx.y, z = blockIdx.z;
    const int seg = (tile >= a.tile_start[1] ? 1 : 0) + (tile >= a.tile_start[2] ? 1 : 0);
    const int per_tile = a.pair ? kHalf : BN;  // output columns of one n-tile
    const int n0 = (tile - a.tile_start[seg]) * per_tile;
    const int m0 = mt * kTileM;
    const int kb0 = static_cast<int>(static_cast<long long>(z) * a.kblocks / a.split_k);
    const int kb1 = static_cast<int>(static_cast<long long>(z + 1) * a.kblocks / a.split_k);
    const int nkb = kb1 - kb0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(accum, 1);
        *abort_flag = 0;
        *last_flag = 0;
        mbar_init_fence();
    }
    if (warp == 1) tmem_alloc(tmem_slot, BN);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned int tmem_base = *tmem_slot;
    chain_release();
    chain_wait();  // nothing above reads or writes global memory
    if (threadIdx.x == 0) stamp(1);

    if (warp == 0) {
        if (lane == 0) {
            for (int it = 0; it < nkb; ++it) {
                const int s = it % a.stages;
                if (it >= a.stages &&
                    !mbar_wait_bounded(&empty[s], ((it / a.stages) - 1) & 1, abort_flag)) {
                    record_status(a.ctl, MB_ST_PIPE_TIMEOUT, a.phase, 1);
                    *abort_flag = 1;
                    break;
                }
                unsigned char* stage = smem + s * kStage;
                mbar_arrive_expect_tx(&full[s], kStage);
                const int kx = (kb0 + it) * kTileK;
                tma_load_2d(stage, &maps.a, kx, m0, &full[s]);
                if (a.pair) {
                    tma_load_2d(stage + kStageA, &maps.w[0], kx, n0, &full[s]);
                    tma_load_2d(stage + kStageA + kHalf * kTileK * 2, &maps.w[3], kx, n0, &full[s]);
                } else {
                    tma_load_2d(stage + kStageA, &maps.w[seg], kx, n0, &full[s]);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            // instruction descriptor: fp32 accumulate, bf16 x bf16, both operands K-major,
            // N = BN, M = 128
            const unsigned int idesc = (1u << 4) | (1u << 7) | (1u << 10) |
                                       (static_cast<unsigned int>(BN >> 3) << 17) |
                                       (static_cast<unsigned int>(kTileM >> 4) << 24);
            bool ok = true;
            for (int it = 0; it < nkb; ++it) {
                const int s = it % a.stages;
                if (!mbar_wait_bounded(&full[s], (it / a.stages) & 1, abort_flag)) {
                    record_status(a.ctl, MB_ST_PIPE_TIMEOUT, a.phase, 2);
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
                tc_fence_after();
                if (it == 0) stamp(2);
                const unsigned int base = smem_u32(smem + s * kStage);
                const unsigned long long da = umma_desc(base);
                const unsigned long long db = umma_desc(base + kStageA);
#pragma unroll
                for (int k = 0; k < kTileK / 16; ++k)  // 32 bytes along K per step: +2 encoded
                    umma_bf16(tmem_base, da + 2 * k, db + 2 * k, idesc, (it | k) != 0 ? 1u : 0u);
                umma_commit(&empty[s]);  // the stage is free once these MMAs have read it
            }
            if (ok) umma_commit(accum);
            stamp(3);
        }
        __syncwarp();
    } else {
        const int quarter = warp & 3;  // the TMEM lanes a warp may read: 32 * (warp % 4) ...
        const int row_in_tile = quarter * 32 + lane;
        // `ok` is warp-uniform: the tcgen05.ld below must be executed by whole warps
        bool ok = __all_sync(0xffffffffu, mbar_wait_bounded(accum, 0, abort_flag));
        if (!ok) {
            if (lane == 0) record_status(a.ctl, MB_ST_PIPE_TIMEOUT, a.phase, 3);
            *abort_flag = 1;
        }
        tc_fence_after();
        if (threadIdx.x == 64) stamp(4);
        const unsigned int lane_addr = tmem_base + (static_cast<unsigned int>(quarter * 32) << 16);
        const int chunks = per_tile / 32;
        const int tile_id = mt * a.tiles_n + tile;
        if (ok && a.split_k > 1) {
            // park this CTA's partial sums; the CTA that arrives last adds them up in split
            // order (so the result does not depend on arrival order) and runs the epilogue
            // layout [tile][split][column][row]: a warp's 32 rows are contiguous, so every
            // store and every load of the reduction is one 128-byte line per warp
            float* mine = a.workspace +
                          (static_cast<size_t>(tile_id) * a.split_k + z) * (kTileM * BN) + row_in_tile;
            for (int c = 0; c < BN / 32; ++c) {
                float v[32];
                tmem_load32(lane_addr + c * 32, v);
#pragma unroll
                for (int i = 0; i < 32; ++i) __stcg(mine + (c * 32 + i) * kTileM, v[i]);
            }
            __threadfence();
            named_barrier(1, 128);
            if (warp == 2 && lane == 0) {
                const int arrived = atomicAdd(a.counters + tile_id, 1);
                *last_flag = arrived == a.split_k - 1 ? 1 : 0;
                if (arrived == a.split_k - 1) a.counters[tile_id] = 0;  // re-arm for the next launch
                __threadfence();
            }
            named_barrier(1, 128);
            ok = *last_flag != 0;
        }
        if (ok) {
            // every MMA has finished reading the operand ring: its first bytes become the
            // staging tile, rows padded by 16 bytes against bank conflicts
            unsigned char* stage_rows = smem;
            const int pitch = per_tile * 2 + 16;
            const float* parts = a.workspace +
                                 static_cast<size_t>(tile_id) * a.split_k * (kTileM * BN) + row_in_tile;
            for (int c = 0; c < chunks; ++c) {
                const int col0 = n0 + c * 32;
                if (col0 >= a.n[seg]) break;
                const int width = min(32, a.n[seg] - col0);
                float v[32], u[32];
                if (a.split_k > 1) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = u[i] = 0.f;
                    for (int s = 0; s < a.split_k; ++s) {
                        const float* p = parts + static_cast<size_t>(s) * (kTileM * BN);
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] += __ldcg(p + (c * 32 + i) * kTileM);
                        if (a.pair) {
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                u[i] += __ldcg(p + (kHalf + c * 32 + i) * kTileM);
                        }
                    }
                } else {
                    tmem_load32(lane_addr + c * 32, v);
                    if (c == 0 && threadIdx.x == 64) stamp(7);
                    if (a.pair)
                        tmem_load32(lane_addr + kHalf + c * 32, u);
                    else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) u[i] = 0.f;
                    }
                }
                gemm_stage_chunk(a, seg, col0, width, v, u, stage_rows + row_in_tile * pitch + c * 64);
            }
            __syncwarp();
            gemm_write_rows(a, seg, m0 + quarter * 32, n0, per_tile, stage_rows + quarter * 32 * pitch,
                            pitch, lane);
        }
    }
    if (threadIdx.x == 64) stamp(5);
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        // copies this CTA issued may still be landing in its shared memory: give them time
        const unsigned long long start = global_timer_ns();
        while (global_timer_ns() - start < 200000ull) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) tmem_dealloc(tmem_base, BN);
    if (threadIdx.x == 32) stamp(6);
}

// ---------------------------------------------------------------------------------------
// The persistent GEMM: one CTA per SM walks output tiles (m-tiles fastest, so the CTAs that run
// together share a weight tile), with the three roles decoupled across tiles:
//   warp 0      TMA producer: keeps the operand ring (192 KB) full, across tile boundaries
//   warp 1      MMA issuer: accumulates tile j into tensor-memory buffer j & 1
//   warps 2-9   epilogue: drain buffer j & 1 while the MMAs of tile j + 1 fill the other one;
//               warps 2-5 take the first half of the tile's output columns, warps 6-9 the
//               second half (a warp reads the 32 TMEM lanes of its index modulo 4)
// Measured on the one-tile-per-CTA kernel at 2048 rows: two co-resident CTAs start together
// and stay in step, so their epilogues (a third of a CTA's life) leave the tensor cores
// idle; here the epilogue of a tile is hidden behind the next tile's MMAs by construction,
// and a ring twice as deep per CTA covers the load latency of single-wave problems.
// The epilogue stores straight from registers: a lane owns 64 contiguous bytes of its output
// row per 32-column chunk (whole 32-byte sectors), so no staging tile and no second pass.
// ---------------------------------------------------------------------------------------
constexpr int kPersistThreads = 320;
constexpr int kPersistRingBytes = 192 * 1024;
constexpr int kPersistSmemBytes = kPersistRingBytes + 256 + 1024;  // ring + barriers + alignment slack

__device__ __forceinline__ void tmem_load32_pair(unsigned int addr_v, unsigned int addr_u, bool pair,
                                                 float (&v)[32], float (&u)[32]) {
    unsigned int r[32], q[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(addr_v)
        : "memory");
    if (pair) {
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
            "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
            : "=r"(q[0]), "=r"(q[1]), "=r"(q[2]), "=r"(q[3]), "=r"(q[4]), "=r"(q[5]), "=r"(q[6]),
              "=r"(q[7]), "=r"(q[8]), "=r"(q[9]), "=r"(q[10]), "=r"(q[11]), "=r"(q[12]),
              "=r"(q[13]), "=r"(q[14]), "=r"(q[15]), "=r"(q[16]), "=r"(q[17]), "=r"(q[18]),
              "=r"(q[19]), "=r"(q[20]), "=r"(q[21]), "=r"(q[22]), "=r"(q[23]), "=r"(q[24]),
              "=r"(q[25]), "=r"(q[26]), "=r"(q[27]), "=r"(q[28]), "=r"(q[29]), "=r"(q[30]),
              "=r"(q[31])
            : "r"(addr_u)
            : "memory");
    }
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        v[i] = __uint_as_float(r[i]);
        u[i] = pair ? __uint_as_float(q[i]) : 0.f;
    }
}

// Epilogue of one 32-column chunk of this thread's output row, registers -> global memory.
// h: the residual's 32 values of the same place (read before the accumulators were awaited),
// used by the fast path only.
__device__ __forceinline__ void gemm_store_chunk(const GemmArgs& a, int seg, int row, int col0,
                                                 const float (&v)[32], const float (&u)[32],
                                                 const uint4 (&h)[4], bool fast) {
    const int n = a.n[seg];
    const int width = min(32, n - col0);
    const unsigned short* bias = a.bias[seg];
    float y[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        const float b = (bias != nullptr && i < width) ? bf16_bits_to_float(__ldg(bias + col0 + i)) : 0.f;
        y[i] = bf16_round(v[i] + b);
    }
    if (a.epilogue == MB_EPI_SILU_MUL) {
#pragma unroll
        for (int i = 0; i < 32; ++i) y[i] = bf16_round(silu_f32(y[i])) * bf16_round(u[i]);
    } else if (a.epilogue == MB_EPI_GELU_TANH_MUL) {
#pragma unroll
        for (int i = 0; i < 32; ++i) y[i] = bf16_round(gelu_tanh_f32(y[i])) * bf16_round(u[i]);
    }
    if (row >= a.M) return;
    const size_t out_row = (seg >= 1 && a.out_tokens > 0)
                               ? static_cast<size_t>(row / a.out_tokens) * a.out_capacity + row % a.out_tokens
                               : static_cast<size_t>(row);
    const size_t at = out_row * n + col0;
    unsigned short* out = a.out[seg] + at;
    if (fast) {
        const bool res = a.epilogue == MB_EPI_RESIDUAL;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const unsigned int hw[4] = {h[q].x, h[q].y, h[q].z, h[q].w};
            unsigned int t[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                t[e] = pack_bf16_pair(y[8 * q + 2 * e], y[8 * q + 2 * e + 1]);
                if (res)
                    t[e] = pack_bf16_pair(lo_bf16(hw[e]) + lo_bf16(t[e]), hi_bf16(hw[e]) + hi_bf16(t[e]));
            }
            reinterpret_cast<uint4*>(out)[q] = make_uint4(t[0], t[1], t[2], t[3]);
        }
    } else {
        const unsigned short* res = a.epilogue == MB_EPI_RESIDUAL ? a.residual + at : nullptr;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            if (i < width) {
                float r = bf16_round(y[i]);
                if (res != nullptr) r = bf16_bits_to_float(res[i]) + r;
                out[i] = float_to_bf16_bits(r);
            }
        }
    }
}

template <int BN>
__global__ void __launch_bounds__(kPersistThreads, 1)
gemm_tc_persistent_kernel(const __grid_constant__ GemmMaps maps, const GemmArgs a) {
    constexpr int kStageW = BN * kTileK * 2;
    constexpr int kStage = kStageA + kStageW;
    constexpr int kStages = kPersistRingBytes / kStage;  // 4 at BN = 256, 6 at BN = 128
    constexpr int kHalf = BN / 2;                        // columns per matrix of a gated pair
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    unsigned long long* full = reinterpret_cast<unsigned long long*>(smem + kStages * kStage);
    unsigned long long* empty = full + 8;
    unsigned long long* acc_full = empty + 8;
    unsigned long long* acc_empty = acc_full + 2;
    unsigned int* tmem_slot = reinterpret_cast<unsigned int*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool traced = a.trace != nullptr && blockIdx.x == 0;
    auto stamp = [&](int slot) {
        if (traced) a.trace[slot] = global_timer_ns();
    };
    if (threadIdx.x == 0) stamp(0);
    // work units: (output tile, slice of the reduction), slices of a tile adjacent so that they
    // finish together and the last one to arrive finds the others' partial sums in L2.  Every
    // unit starts at the same k offsets as its neighbours, so CTAs that share an operand tile
    // ask for the same k-block at the same time and L2 serves all but one of them.  (Measured
    // and dropped: equal runs of k-blocks per CTA cut across tiles.  They balance the CTAs
    // exactly but skew the k offsets, the operands then overflow L2 between two uses, and
    // every shape that needed them ran 20-60 % slower.)
    const int total = a.tiles_n * a.tiles_m * a.split_k;
    const int per_tile = a.pair ? kHalf : BN;  // output columns of one n-tile
    int* last_flag = const_cast<int*>(abort_flag) + 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 8);  // one arrival per epilogue warp
        }
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 1) tmem_alloc(tmem_slot, 2 * BN);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned int tmem_base = *tmem_slot;
    chain_release();
    chain_wait();  // nothing above reads or writes global memory
    if (threadIdx.x == 0) stamp(1);

    if (warp == 0) {
        if (lane == 0) {
            int s = 0, round = 0;  // ring position; `round` counts wraps
            bool ok = true;
            for (int unit = blockIdx.x; unit < total && ok; unit += gridDim.x) {
                const int t = unit / a.split_k, z = unit - t * a.split_k;
                const int mt = t % a.tiles_m, tile = t / a.tiles_m;
                const int seg = (tile >= a.tile_start[1] ? 1 : 0) + (tile >= a.tile_start[2] ? 1 : 0);
                const int n0 = (tile - a.tile_start[seg]) * per_tile;
                const int m0 = mt * kTileM;
                const int kb0 = static_cast<int>(static_cast<long long>(z) * a.kblocks / a.split_k);
                const int kb1 = static_cast<int>(static_cast<long long>(z + 1) * a.kblocks / a.split_k);
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (round > 0 && !mbar_wait_bounded(&empty[s], (round - 1) & 1, abort_flag)) {
                        record_status(a.ctl, MB_ST_PIPE_TIMEOUT, a.phase, 1);
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                    unsigned char* stage = smem + s * kStage;
                    mbar_arrive_expect_tx(&full[s], kStage);
                    const int kx = kb * kTileK;
                    tma_load_2d(stage, &maps.a, kx, m0, &full[s]);
                    if (a.pair) {
                        tma_load_2d(stage + kStageA, &maps.w[0], kx, n0, &full[s]);
                        tma_load_2d(stage + kStageA + kHalf * kTileK * 2, &maps.w[3], kx, n0, &full[s]);
                    } else {
                        tma_load_2d(stage + kStageA, &maps.w[seg], kx, n0, &full[s]);
                    }
                    if (++s == kStages) {
                        s = 0;
                        ++round;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            // instruction descriptor: fp32 accumulate, bf16 x bf16, both operands K-major,
            // N = BN, M = 128
            const unsigned int idesc = (1u << 4) | (1u << 7) | (1u << 10) |
                                       (static_cast<unsigned int>(BN >> 3) << 17) |
                                       (static_cast<unsigned int>(kTileM >> 4) << 24);
            int s = 0, round = 0, j = 0;
            bool ok = true;
            for (int unit = blockIdx.x; unit < total && ok; unit += gridDim.x, ++j) {
                const int buf = j & 1;
                const int z = unit % a.split_k;
                const int kb0 = static_cast<int>(static_cast<long long>(z) * a.kblocks / a.split_k);
                const int kb1 = static_cast<int>(static_cast<long long>(z + 1) * a.kblocks / a.split_k);
                // the epilogue must have drained this buffer's previous tile
                if (j >= 2 && !mbar_wait_bounded(&acc_empty[buf], ((j >> 1) - 1) & 1, abort_flag)) {
                    record_status(a.ctl, MB_ST_PIPE_TIMEOUT, a.phase, 4);
                    *abort_flag = 1;
                    break;
                }
                tc_fence_after();
                const unsigned int acc = tmem_base + buf * BN;
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait_bounded(&full[s], round & 1, abort_flag)) {
                        record_status(a.ctl, MB_ST_PIPE_TIMEOUT, a.phase, 2);
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    if (j == 0 && kb == kb0) stamp(2);
                    const unsigned int base = smem_u32(smem + s * kStage);
                    const unsigned long long da = umma_desc(base);
                    const unsigned long long db = umma_desc(base + kStageA);
#pragma unroll
                    for (int k = 0; k < kTileK / 16; ++k)  // 32 bytes along K per step: +2 encoded
                        umma_bf16(acc, da + 2 * k, db + 2 * k, idesc, (kb != kb0 || k != 0) ? 1u : 0u);
                    umma_commit(&empty[s]);  // the stage is free once these MMAs have read it
                    if (++s == kStages) {
                        s = 0;
                        ++round;
                    }
                }
                if (ok) umma_commit(&acc_full[buf]);
                if (j == 0) stamp(3);
            }
        }
        __syncwarp();
    } else {
        const int quarter = warp & 3;        // the TMEM lanes a warp may read: 32 * (warp % 4) ...
        const int column_half = (warp - 2) >> 2;
        const int chunks = per_tile / 32;
        const int c_begin = column_half * (chunks / 2), c_end = c_begin + chunks / 2;
        int j = 0;
        for (int unit = blockIdx.x; unit < total; unit += gridDim.x, ++j) {
            const int buf = j & 1;
            const int t = unit / a.split_k, z = unit - t * a.split_k;
            const int mt = t % a.tiles_m, tile = t / a.tiles_m;
            const int seg = (tile >= a.tile_start[1] ? 1 : 0) + (tile >= a.tile_start[2] ? 1 : 0);
            const int n0 = (tile - a.tile_start[seg]) * per_tile;
            const int row = mt * kTileM + quarter * 32 + lane;
            const int n = a.n[seg];
            // warp-uniform: the tcgen05.ld below must be executed by whole warps
            const bool ok = __all_sync(0xffffffffu,
                                       mbar_wait_bounded(&acc_full[buf], (j >> 1) & 1, abort_flag));
            if (!ok) {
                if (lane == 0) record_status(a.ctl, MB_ST_PIPE_TIMEOUT, a.phase, 3);
                *abort_flag = 1;
                if (a.split_k == 1) break;
            }
            tc_fence_after();
            if (j == 0 && threadIdx.x == 64) stamp(4);
            const unsigned int lane_addr =
                tmem_base + buf * BN + (static_cast<unsigned int>(quarter * 32) << 16);
            const bool row_fast = (n & 7) == 0;
            if (a.split_k > 1) {
                // the eight warps meet at barriers below: leave together or not at all
                if (named_barrier_or(2, 256, !ok)) {
                    *abort_flag = 1;
                    break;
                }
                // park the partial sums ([tile][slice][column][row]: a warp's 32 rows are one
                // 128-byte line per column), give the buffer back, and let the slice that
                // arrives last add all of them up in slice order, so that the result does not
                // depend on the order of arrival
                const int row_in_tile = quarter * 32 + lane;
                float* parts = a.workspace + static_cast<size_t>(t) * a.split_k * (kTileM * BN) + row_in_tile;
                float* mine = parts + static_cast<size_t>(z) * (kTileM * BN);
                for (int c = column_half * (BN / 64); c < (column_half + 1) * (BN / 64); ++c) {
                    float v[32];
                    tmem_load32(lane_addr + c * 32, v);
#pragma unroll
                    for (int i = 0; i < 32; ++i) __stcg(mine + (c * 32 + i) * kTileM, v[i]);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[buf]);
                __threadfence();
                named_barrier(1, 256);
                if (warp == 2 && lane == 0) {
                    const int arrived = atomicAdd(a.counters + t, 1);
                    *last_flag = arrived == a.split_k - 1 ? 1 : 0;
                    if (arrived == a.split_k - 1) a.counters[t] = 0;  // re-arm for the next launch
                    __threadfence();
                }
                named_barrier(1, 256);
                if (*last_flag != 0) {
                    for (int c = c_begin; c < c_end; ++c) {
                        const int col0 = n0 + c * 32;
                        if (col0 >= n) break;
                        const bool fast = row_fast && col0 + 32 <= n;
                        uint4 h[4] = {};
                        if (fast && a.epilogue == MB_EPI_RESIDUAL && row < a.M) {
                            const uint4* src = reinterpret_cast<const uint4*>(
                                a.residual + static_cast<size_t>(row) * n + col0);
#pragma unroll
                            for (int q = 0; q < 4; ++q) h[q] = src[q];
                        }
                        float v[32], u[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = u[i] = 0.f;
                        for (int sl = 0; sl < a.split_k; ++sl) {
                            const float* p = parts + static_cast<size_t>(sl) * (kTileM * BN);
#pragma unroll
                            for (int i = 0; i < 32; ++i) v[i] += __ldcg(p + (c * 32 + i) * kTileM);
                            if (a.pair) {
#pragma unroll
                                for (int i = 0; i < 32; ++i)
                                    u[i] += __ldcg(p + (kHalf + c * 32 + i) * kTileM);
                            }
                        }
                        gemm_store_chunk(a, seg, row, col0, v, u, h, fast);
                    }
                }
                named_barrier(1, 256);  // last_flag is rewritten by the next unit
                continue;
            }
            for (int c = c_begin; c < c_end; ++c) {
                const int col0 = n0 + c * 32;
                if (col0 >= n) break;
                const bool fast = row_fast && col0 + 32 <= n;
                uint4 h[4] = {};
                if (fast && a.epilogue == MB_EPI_RESIDUAL && row < a.M) {
                    const uint4* src =
                        reinterpret_cast<const uint4*>(a.residual + static_cast<size_t>(row) * n + col0);
#pragma unroll
                    for (int q = 0; q < 4; ++q) h[q] = src[q];
                }
                float v[32], u[32];
                tmem_load32_pair(lane_addr + c * 32, lane_addr + kHalf + c * 32, a.pair != 0, v, u);
                gemm_store_chunk(a, seg, row, col0, v, u, h, fast);
            }
            // this warp's reads of the buffer are complete: hand it back to the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
            if (j == 0 && threadIdx.x == 64) stamp(5);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        // copies this CTA issued may still be landing in its shared memory: give them time
        const unsigned long long start = global_timer_ns();
        while (global_timer_ns() - start < 200000ull) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) tmem_dealloc(tmem_base, 2 * BN);
    if (threadIdx.x == 32) stamp(6);
}


// ---------------------------------------------------------------------------------------
// Prefill attention.  One CTA (4 warps) per 64 query rows of one head; keys in blocks of 64.
// Two sweeps over the visible keys so that the probabilities can be rounded to bf16 *after*
// normalisation, as the eager operator does: sweep 1 finds each row's maximum and
// denominator, sweep 2 recomputes the scores, forms p = bf16(exp(s - max) / sum) and
// accumulates p . V.  Scores carry the operator's rounding points:
// s = bf16(q . k); s = bf16(s * scale); s = bf16(s + mask).
// ---------------------------------------------------------------------------------------
struct AttnArgs {
    const unsigned short* q;
    const unsigned short* k;
    const unsigned short* v;
    unsigned short* out;
    const unsigned short* mask;  // additive, [mask_batch, 1, T, T], or null
    int batch, tokens, heads, kv_heads, causal, mask_batch;
    int kv_rows;  // rows per batch of the K and V tensors (tokens, or a cache's capacity)
    float scale;
    // attention_tc_kernel with the keys of a query tile shared out (see there); 0 = one CTA per tile
    int mode;           // kAttnWhole, kAttnStats or kAttnValues
    int chunk;          // key blocks per CTA at most
    int parts_max;      // ceil(all key blocks / chunk): stride of the scratch below
    float* stats_ws;    // [item][part][128 rows][2]: row maximum and denominator over the part's keys
    float* o_ws;        // [item][part][head_dim][128 rows]: fp32 partial outputs
    int* counters;      // [item]: parts arrived, zero between launches
};

constexpr int kAttnWhole = 0, kAttnStats = 1, kAttnValues = 2;

constexpr int kAttnKeys = 64;  // keys per block

__device__ __forceinline__ void ldmatrix_x4(unsigned int (&r)[4], const void* smem_ptr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(smem_ptr)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned int (&r)[4], const void* smem_ptr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(smem_ptr)));
}
__device__ __forceinline__ void cp_async_16(void* dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(src)
                 : "memory");
}

// `rows` rows of D bf16 each into a tile with pitch D + 8; rows past `limit` repeat the last one
template <int D, int THREADS>
__device__ __forceinline__ void attn_load_rows(unsigned short* dst, const unsigned short* src,
                                               size_t row_stride, int row0, int rows, int limit) {
    constexpr int kVectors = D / 8;
    for (int e = threadIdx.x; e < rows * kVectors; e += THREADS) {
        const int r = e / kVectors, c = e - r * kVectors;
        const int row = min(row0 + r, limit - 1);
        cp_async_16(dst + r * (D + 8) + c * 8, src + static_cast<size_t>(row) * row_stride + c * 8);
    }
}

template <int D>
__device__ __forceinline__ void attn_scores(float (&sacc)[8][4], const unsigned short* Qs,
                                            const unsigned short* Ks, int warp, int lane) {
    constexpr int P = D + 8;
#pragma unroll
    for (int t = 0; t < 8; ++t)
#pragma unroll
        for (int q = 0; q < 4; ++q) sacc[t][q] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
        unsigned int a[4];
        ldmatrix_x4(a, Qs + (warp * 16 + (lane & 15)) * P + kk * 16 + (lane >> 4) * 8);
#pragma unroll
        for (int np = 0; np < 4; ++np) {
            unsigned int b[4];
            ldmatrix_x4(b, Ks + (np * 16 + ((lane >> 4) & 1) * 8 + (lane & 7)) * P + kk * 16 +
                               ((lane >> 3) & 1) * 8);
            mma_bf16_16816(sacc[2 * np], a[0], a[1], a[2], a[3], b[0], b[1]);
            mma_bf16_16816(sacc[2 * np + 1], a[0], a[1], a[2], a[3], b[2], b[3]);
        }
    }
}

// WARPS warps per CTA, 16 query rows each; K (and V) blocks double-buffered with cp.async so
// that the next block streams in while the tensor cores work on the current one.
template <int D, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, 1) attention_prefill_kernel(const AttnArgs a) {
    constexpr int P = D + 8;
    constexpr int THREADS = WARPS * 32;
    constexpr int ROWS = WARPS * 16;
    extern __shared__ __align__(16) unsigned char attn_smem[];
    unsigned short* Qs = reinterpret_cast<unsigned short*>(attn_smem);
    unsigned short* Kbuf = Qs + ROWS * P;               // [2][64][P]
    unsigned short* Vbuf = Kbuf + 2 * kAttnKeys * P;    // [2][64][P]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gid = lane >> 2, tq = lane & 3;
    const int T = a.tokens;
    const int qt = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);  // long rows first
    const int head = blockIdx.y, b = blockIdx.z;
    const int kvh = head / (a.heads / a.kv_heads);
    const int q0 = qt * ROWS;
    const size_t q_stride = static_cast<size_t>(a.heads) * D;
    const size_t kv_stride = static_cast<size_t>(a.kv_heads) * D;
    const unsigned short* qbase = a.q + static_cast<size_t>(b) * T * q_stride + head * D;
    const unsigned short* kbase = a.k + static_cast<size_t>(b) * a.kv_rows * kv_stride + kvh * D;
    const unsigned short* vbase = a.v + static_cast<size_t>(b) * a.kv_rows * kv_stride + kvh * D;
    const int all_blocks = (T + kAttnKeys - 1) / kAttnKeys;
    const int last_row = min(q0 + ROWS, T) - 1;
    const int nblocks = a.causal ? min(last_row / kAttnKeys + 1, all_blocks) : all_blocks;
    const int row_lo = q0 + warp * 16 + gid, row_hi = row_lo + 8;
    // causal: key blocks that start past this warp's last row contribute nothing to it
    const int warp_blocks = a.causal ? min((q0 + warp * 16 + 15) / kAttnKeys + 1, nblocks) : nblocks;
    const unsigned short* mask_lo = nullptr;
    const unsigned short* mask_hi = nullptr;
    if (a.mask != nullptr) {
        const unsigned short* mb = a.mask + (a.mask_batch > 1 ? static_cast<size_t>(b) * T * T : 0);
        mask_lo = mb + static_cast<size_t>(min(row_lo, T - 1)) * T;
        mask_hi = mb + static_cast<size_t>(min(row_hi, T - 1)) * T;
    }

    // score of (row, key) with the operator's rounding points; false if the key is not visible
    auto score = [&](float acc, int row, int key, const unsigned short* mrow, float* s) {
        float t = bf16_round(acc);
        t = bf16_round(t * a.scale);
        if (mrow != nullptr && key < T) t = bf16_round(t + bf16_bits_to_float(__ldg(mrow + key)));
        *s = t;
        return key < T && (!a.causal || key <= row);
    };

    attn_load_rows<D, THREADS>(Qs, qbase, q_stride, q0, ROWS, T);
    attn_load_rows<D, THREADS>(Kbuf, kbase, kv_stride, 0, kAttnKeys, T);
    asm volatile("cp.async.commit_group;" ::: "memory");

    // ---- sweep 1: row maxima and denominators --------------------------------------------
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
    for (int jb = 0; jb < nblocks; ++jb) {
        const unsigned short* Ks = Kbuf + (jb & 1) * kAttnKeys * P;
        if (jb + 1 < nblocks) {
            attn_load_rows<D, THREADS>(Kbuf + ((jb + 1) & 1) * kAttnKeys * P, kbase, kv_stride,
                                       (jb + 1) * kAttnKeys, kAttnKeys, T);
            asm volatile("cp.async.commit_group;" ::: "memory");
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        if (jb < warp_blocks) {
            float sacc[8][4];
            attn_scores<D>(sacc, Qs, Ks, warp, lane);
            float s_lo[16], s_hi[16];
            float bm_lo = -INFINITY, bm_hi = -INFINITY;
#pragma unroll
            for (int t = 0; t < 8; ++t)
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int key = jb * kAttnKeys + t * 8 + 2 * tq + j;
                    float s;
                    s_lo[2 * t + j] = score(sacc[t][j], row_lo, key, mask_lo, &s) ? s : -INFINITY;
                    s_hi[2 * t + j] = score(sacc[t][2 + j], row_hi, key, mask_hi, &s) ? s : -INFINITY;
                    bm_lo = fmaxf(bm_lo, s_lo[2 * t + j]);
                    bm_hi = fmaxf(bm_hi, s_hi[2 * t + j]);
                }
#pragma unroll
            for (int o = 1; o <= 2; o <<= 1) {
                bm_lo = fmaxf(bm_lo, __shfl_xor_sync(0xffffffffu, bm_lo, o));
                bm_hi = fmaxf(bm_hi, __shfl_xor_sync(0xffffffffu, bm_hi, o));
            }
            const float n_lo = fmaxf(m_lo, bm_lo), n_hi = fmaxf(m_hi, bm_hi);
            // a row with no visible key yet keeps max = -inf; exp(-inf - -inf) must not be formed
            l_lo = n_lo == -INFINITY ? 0.f : l_lo * expf(m_lo - n_lo);
            l_hi = n_hi == -INFINITY ? 0.f : l_hi * expf(m_hi - n_hi);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                if (s_lo[i] != -INFINITY) l_lo += expf(s_lo[i] - n_lo);
                if (s_hi[i] != -INFINITY) l_hi += expf(s_hi[i] - n_hi);
            }
            m_lo = n_lo;
            m_hi = n_hi;
        }
        __syncthreads();  // the buffer just used is the target of the load after next
    }
#pragma unroll
    for (int o = 1; o <= 2; o <<= 1) {
        l_lo += __shfl_xor_sync(0xffffffffu, l_lo, o);
        l_hi += __shfl_xor_sync(0xffffffffu, l_hi, o);
    }

    // ---- sweep 2: probabilities and p . V -------------------------------------------------
    float oacc[D / 8][4];
#pragma unroll
    for (int t = 0; t < D / 8; ++t)
#pragma unroll
        for (int q = 0; q < 4; ++q) oacc[t][q] = 0.f;
    attn_load_rows<D, THREADS>(Kbuf, kbase, kv_stride, 0, kAttnKeys, T);
    attn_load_rows<D, THREADS>(Vbuf, vbase, kv_stride, 0, kAttnKeys, T);
    asm volatile("cp.async.commit_group;" ::: "memory");
    for (int jb = 0; jb < nblocks; ++jb) {
        const unsigned short* Ks = Kbuf + (jb & 1) * kAttnKeys * P;
        const unsigned short* Vs = Vbuf + (jb & 1) * kAttnKeys * P;
        if (jb + 1 < nblocks) {
            attn_load_rows<D, THREADS>(Kbuf + ((jb + 1) & 1) * kAttnKeys * P, kbase, kv_stride,
                                       (jb + 1) * kAttnKeys, kAttnKeys, T);
            attn_load_rows<D, THREADS>(Vbuf + ((jb + 1) & 1) * kAttnKeys * P, vbase, kv_stride,
                                       (jb + 1) * kAttnKeys, kAttnKeys, T);
            asm volatile("cp.async.commit_group;" ::: "memory");
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        if (jb < warp_blocks) {
            float sacc[8][4];
            attn_scores<D>(sacc, Qs, Ks, warp, lane);
            unsigned int pfrag[4][4];  // A fragments of P for the four 16-key steps
#pragma unroll
            for (int t = 0; t < 8; ++t) {
                float p[4];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int key = jb * kAttnKeys + t * 8 + 2 * tq + j;
                    float s;
                    p[j] = score(sacc[t][j], row_lo, key, mask_lo, &s)
                               ? __fdiv_rn(expf(s - m_lo), l_lo) : 0.f;
                    p[2 + j] = score(sacc[t][2 + j], row_hi, key, mask_hi, &s)
                                   ? __fdiv_rn(expf(s - m_hi), l_hi) : 0.f;
                }
                pfrag[t >> 1][(t & 1) * 2] = pack_bf16(p[0], p[1]);
                pfrag[t >> 1][(t & 1) * 2 + 1] = pack_bf16(p[2], p[3]);
            }
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
                for (int dp = 0; dp < D / 16; ++dp) {
                    unsigned int vb[4];
                    ldmatrix_x4_trans(vb, Vs + (kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * P +
                                              dp * 16 + (lane >> 4) * 8);
                    mma_bf16_16816(oacc[2 * dp], pfrag[kk][0], pfrag[kk][1], pfrag[kk][2],
                                   pfrag[kk][3], vb[0], vb[1]);
                    mma_bf16_16816(oacc[2 * dp + 1], pfrag[kk][0], pfrag[kk][1], pfrag[kk][2],
                                   pfrag[kk][3], vb[2], vb[3]);
                }
            }
        }
        __syncthreads();
    }

    unsigned short* obase = a.out + static_cast<size_t>(b) * T * q_stride + head * D;
#pragma unroll
    for (int t = 0; t < D / 8; ++t) {
        const int d = t * 8 + 2 * tq;
        if (row_lo < T)
            *reinterpret_cast<unsigned int*>(obase + static_cast<size_t>(row_lo) * q_stride + d) =
                pack_bf16(oacc[t][0], oacc[t][1]);
        if (row_hi < T)
            *reinterpret_cast<unsigned int*>(obase + static_cast<size_t>(row_hi) * q_stride + d) =
                pack_bf16(oacc[t][2], oacc[t][3]);
    }
}

// Launch geometry: 8 warps (128 query rows) per CTA for long prompts, 4 for short ones so
// that more CTAs exist.
inline int attn_warps(int tokens) { return tokens > 256 ? 8 : 4; }
inline int attn_smem_bytes(int D, int warps) { return (warps * 16 + 4 * kAttnKeys) * (D + 8) * 2; }

template <int D>
cudaError_t attn_launch(const AttnArgs& a, cudaStream_t stream) {
    const int warps = attn_warps(a.tokens);
    const dim3 grid((a.tokens + warps * 16 - 1) / (warps * 16), a.heads, a.batch);
    const int smem = attn_smem_bytes(D, warps);
    if (warps == 8)
        attention_prefill_kernel<D, 8><<<grid, 256, smem, stream>>>(a);
    else
        attention_prefill_kernel<D, 4><<<grid, 128, smem, stream>>>(a);
    return cudaGetLastError();
}

template <int D>
cudaError_t attn_configure() {
    cudaError_t err = cudaFuncSetAttribute(attention_prefill_kernel<D, 8>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           attn_smem_bytes(D, 8));
    if (err == cudaSuccess)
        err = cudaFuncSetAttribute(attention_prefill_kernel<D, 4>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   attn_smem_bytes(D, 4));
    return err;
}

// ---------------------------------------------------------------------------------------
// Prefill attention on the 5th-generation tensor cores.
//
// One CTA per 128 query rows of one head.  S = Q . K^T and O += P . V both run as tcgen05.mma
// with accumulators in tensor memory; the softmax between them runs on eight warps that read
// S with tcgen05.ld (one thread per row and half a key block, so no shuffles), and write the
// bf16 probabilities into shared memory in the 128-byte-swizzled K-major layout the second
// MMA reads them in.  exp and the division by the row sum use the device's fast forms
// (ex2.approx, multiplication by the reciprocal): the result is rounded to bf16 right after, so
// they change a probability only when it sits within 2^-14 of a rounding boundary.  V is consumed transposed ([head_dim, keys], keys contiguous) so that
// every operand is K-major; a small kernel transposes V once per layer.
//
// Same two sweeps and rounding points as attention_prefill_kernel above.
//   warp 0      TMA producers: lane 0 loads Q once and then K blocks, lane 1 the V^T blocks,
//               each into its own two-stage ring (a K stage is free again as soon as the
//               scores that read it are done, a V stage after the P . V that read it)
//   warp 1      MMA issuer, owner of the tensor-memory allocation
//   warps 2-17  softmax; warp w works on TMEM lanes 32 * (w % 4) .. and key columns
//               16 * ((w - 2) / 4) .. of a block (sixteen warps: the softmax, not the tensor
//               cores, is the long pole of a step, and it is latency-bound per warp)
// Tensor memory: S double-buffered in columns [0, 64) and [64, 128), O in [128, 128 + D).
//
// Few query tiles: 512 tokens of 8 heads are 32 tiles on 148 SMs, and under a causal mask the
// last tile has four times the key blocks of the first.  The keys of a tile can therefore be
// shared out in parts of at most `chunk` blocks (the host decides how: attention_parts), and
// the two sweeps become two launches, so that no CTA ever waits for another one: kAttnStats runs the first sweep over
// its part and leaves each row's maximum and denominator; kAttnValues combines the parts'
// statistics (as the column parts inside a CTA are combined), runs the second sweep over its part
// and, when a tile has several parts, parks its fp32 output -- the part that arrives last adds
// them in key order and rounds once.  Probabilities are still rounded after normalisation by
// the whole row's sum; only the order of the fp32 additions changes.
// ---------------------------------------------------------------------------------------
struct AttnMaps {
    CUtensorMap q;   // [batch * tokens, heads * D], boxes of 128 rows x 64 columns
    CUtensorMap k;   // [batch * tokens, kv_heads * D], boxes of 64 rows x 64 columns
    CUtensorMap vt;  // [batch * kv_heads * D, padded tokens], boxes of D rows x 64 columns
};

constexpr int kTcRows = 128;
constexpr int kTcThreads = 64 + 16 * 32;
constexpr int kTcSoftmaxWarps = 16;  // one elected lane per warp arrives on the shared barriers

// V [batch * tokens, kv_heads * D] -> V^T [batch * kv_heads * D, padded], zero beyond `tokens`
struct TransposeArgs {
    const unsigned short* v;
    unsigned short* vt;
    int tokens, padded, kv_heads, D, kv_rows;
};

// block: index among padded / 64 x D / 64 x batch * kv_heads tiles, tokens fastest
__device__ __forceinline__ void transpose_values_body(const TransposeArgs& a, int block) {
    __shared__ unsigned short tile[64][66];
    const unsigned short* v = a.v;
    unsigned short* vt = a.vt;
    const int tokens = a.tokens, padded = a.padded, kv_heads = a.kv_heads, D = a.D, kv_rows = a.kv_rows;
    const int tiles_t = padded / 64, tiles_d = D / 64;
    const int t0 = (block % tiles_t) * 64, d0 = ((block / tiles_t) % tiles_d) * 64;
    const int bh = block / (tiles_t * tiles_d), b = bh / kv_heads, h = bh - b * kv_heads;
    const size_t row_stride = static_cast<size_t>(kv_heads) * D;
    for (int e = threadIdx.x; e < 64 * 64; e += 256) {
        const int t = e >> 6, d = e & 63;
        tile[t][d] = t0 + t < tokens
                         ? v[(static_cast<size_t>(b) * kv_rows + t0 + t) * row_stride + h * D + d0 + d]
                         : static_cast<unsigned short>(0);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < 64 * 64; e += 256) {
        const int d = e >> 6, t = e & 63;
        if (t0 + t < padded)
            vt[(static_cast<size_t>(bh) * D + d0 + d) * padded + t0 + t] = tile[t][d];
    }
}

__global__ void __launch_bounds__(256) transpose_values_kernel(const TransposeArgs a) {
    chain_release();
    chain_wait();
    transpose_values_body(a, blockIdx.x);
}

// The rotary embedding of q and k and the transpose of v both follow the q|k|v projection and
// touch disjoint tensors: one launch, the first `rope_blocks` CTAs rotate, the others transpose.
__global__ void __launch_bounds__(256) rope_transpose_kernel(const RopeArgs rope,
                                                             const TransposeArgs transpose,
                                                             int rope_blocks) {
    chain_release();
    chain_wait();
    if (static_cast<int>(blockIdx.x) < rope_blocks)
        rope_rows_body(rope, blockIdx.x, rope_blocks);
    else
        transpose_values_body(transpose, blockIdx.x - rope_blocks);
}

template <int D>
__global__ void __launch_bounds__(kTcThreads, 1)
attention_tc_kernel(const __grid_constant__ AttnMaps maps, const AttnArgs a, Control* ctl,
                    int phase) {
    constexpr int kQBytes = kTcRows * D * 2;         // D / 64 boxes of 128 x 64
    constexpr int kKBytes = kAttnKeys * D * 2;       // D / 64 boxes of 64 x 64
    constexpr int kVBytes = D * kAttnKeys * 2;       // one box of D x 64
    constexpr int kPBytes = kTcRows * kAttnKeys * 2; // 128 rows of 128 bytes
    constexpr unsigned int kTmemCols = D > 128 ? 512 : 256;
    constexpr unsigned int kColO = 128;
    // operand tiles need 1024-byte alignment for the 128-byte swizzle; the tile set of
    // head_dim 256 leaves no room for alignment slack, so the base is checked instead
    extern __shared__ __align__(1024) unsigned char tc_smem_raw[];
    unsigned char* smem = tc_smem_raw;
    if ((smem_u32(smem) & 1023u) != 0u) {
        chain_wait();
        if (threadIdx.x == 0) record_status(ctl, MB_ST_BAD_PHASE, phase, -1);
        return;
    }
    unsigned char* Qs = smem;
    unsigned char* Kst = Qs + kQBytes;               // [2][kKBytes]
    unsigned char* Vst = Kst + 2 * kKBytes;          // [2][kVBytes]
    unsigned char* Ps = Vst + 2 * kVBytes;           // [2][kPBytes]
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(Ps + 2 * kPBytes);
    unsigned long long* q_full = bars;
    unsigned long long* k_full = bars + 1;     // [2]
    unsigned long long* k_empty = bars + 3;    // [2]
    unsigned long long* s_full = bars + 5;     // [2]
    unsigned long long* s_empty = bars + 7;    // [2]
    unsigned long long* p_full = bars + 9;     // [2]
    unsigned long long* p_empty = bars + 11;   // [2]
    unsigned long long* o_full = bars + 13;
    unsigned long long* x_full = bars + 14;    // the column parts of every row exchanged their statistics
    unsigned long long* v_full = bars + 15;    // [2]
    unsigned long long* v_empty = bars + 17;   // [2]
    unsigned int* tmem_slot = reinterpret_cast<unsigned int*>(bars + 19);
    int* abort_flag = reinterpret_cast<int*>(tmem_slot + 1);
    int* last_flag = abort_flag + 1;
    // row statistics of the four column parts meet here once, between the sweeps (the first P
    // buffer is idle until then)
    float* stats = reinterpret_cast<float*>(Ps);  // [4 parts][128 rows][2]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int T = a.tokens;
    // heads vary fastest in the grid: CTAs are handed out heaviest work first over the whole
    // grid, not head by head, so light CTAs fill in behind heavy ones
    const int head = blockIdx.x, b = blockIdx.z;
    const int kvh = head / (a.heads / a.kv_heads);
    const int all_blocks = (T + kAttnKeys - 1) / kAttnKeys;
    const int q_tiles = (T + kTcRows - 1) / kTcRows;
    auto visible_blocks = [&](int tile) {
        const int last_row = min(tile * kTcRows + kTcRows, T) - 1;
        return a.causal ? min(last_row / kAttnKeys + 1, all_blocks) : all_blocks;
    };
    // blockIdx.y -> (query tile, part of its keys), long rows first
    int qt = q_tiles - 1, part_index = 0, parts = 1;
    if (a.mode == kAttnWhole) {
        qt = q_tiles - 1 - static_cast<int>(blockIdx.y);
    } else {
        int x = blockIdx.y;
        for (;; --qt) {
            parts = (visible_blocks(qt) + a.chunk - 1) / a.chunk;
            if (x < parts || qt == 0) break;
            x -= parts;
        }
        part_index = min(x, parts - 1);
    }
    const int q0 = qt * kTcRows;
    const int visible = visible_blocks(qt);
    const int per_part = (visible + parts - 1) / parts;
    const int j_begin = min(part_index * per_part, visible);
    const int n = min(visible, j_begin + per_part) - j_begin;  // key blocks of this CTA
    const int n1 = a.mode == kAttnValues ? 0 : n;              // steps of the first sweep
    const int steps = n1 + (a.mode == kAttnStats ? 0 : n);     // of both
    const int item = (b * a.heads + head) * q_tiles + qt;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&k_full[s], 1);
            mbar_init(&k_empty[s], 1);
            mbar_init(&v_full[s], 1);
            mbar_init(&v_empty[s], 1);
            mbar_init(&s_full[s], 1);
            mbar_init(&s_empty[s], kTcSoftmaxWarps);
            mbar_init(&p_full[s], kTcSoftmaxWarps);
            mbar_init(&p_empty[s], 1);
        }
        mbar_init(o_full, 1);
        mbar_init(x_full, kTcSoftmaxWarps);
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 1) tmem_alloc(tmem_slot, kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned int tmem_base = *tmem_slot;
    chain_release();
    chain_wait();  // nothing above reads or writes global memory

    auto give_up = [&](int where) {
        record_status(ctl, MB_ST_PIPE_TIMEOUT, phase, where);
        *abort_flag = 1;
    };

    if (warp == 0) {
        if (lane == 0) {
            mbar_arrive_expect_tx(q_full, kQBytes);
            for (int kb = 0; kb < D / 64; ++kb)
                tma_load_2d(Qs + kb * (kTcRows * 128), &maps.q, head * D + kb * 64, b * T + q0, q_full);
            for (int g = 0; g < steps; ++g) {
                const int st = g & 1, jb = j_begin + (g < n1 ? g : g - n1);
                if (g >= 2 && !mbar_wait_bounded(&k_empty[st], ((g >> 1) - 1) & 1, abort_flag)) {
                    give_up(10);
                    break;
                }
                mbar_arrive_expect_tx(&k_full[st], kKBytes);
                for (int kb = 0; kb < D / 64; ++kb)
                    tma_load_2d(Kst + st * kKBytes + kb * (kAttnKeys * 128), &maps.k,
                                kvh * D + kb * 64, b * a.kv_rows + jb * kAttnKeys, &k_full[st]);
            }
        } else if (lane == 1) {
            for (int j = 0; j < steps - n1; ++j) {  // second sweep only
                const int sv = j & 1;
                if (j >= 2 && !mbar_wait_bounded(&v_empty[sv], ((j >> 1) - 1) & 1, abort_flag)) {
                    give_up(11);
                    break;
                }
                mbar_arrive_expect_tx(&v_full[sv], kVBytes);
                tma_load_2d(Vst + sv * kVBytes, &maps.vt, (j_begin + j) * kAttnKeys,
                            (b * a.kv_heads + kvh) * D, &v_full[sv]);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            const unsigned int idesc_s = (1u << 4) | (1u << 7) | (1u << 10) |
                                         (static_cast<unsigned int>(kAttnKeys >> 3) << 17) |
                                         (static_cast<unsigned int>(kTcRows >> 4) << 24);
            const unsigned int idesc_o = (1u << 4) | (1u << 7) | (1u << 10) |
                                         (static_cast<unsigned int>(D >> 3) << 17) |
                                         (static_cast<unsigned int>(kTcRows >> 4) << 24);
            bool ok = mbar_wait_bounded(q_full, 0, abort_flag);
            if (!ok) give_up(20);
            // values . probabilities of step g (second sweep), issued one step late so that the
            // scores of step g + 1 are already under way while the softmax of step g runs
            auto issue_pv = [&](int g) {
                const int st = g & 1, sv = (g - n1) & 1;
                if (!mbar_wait_bounded(&v_full[sv], ((g - n1) >> 1) & 1, abort_flag) ||
                    !mbar_wait_bounded(&p_full[st], ((g - n1) >> 1) & 1, abort_flag)) {
                    give_up(21);
                    return false;
                }
                tc_fence_after();
                const unsigned long long dp = umma_desc(smem_u32(Ps + st * kPBytes));
                const unsigned long long dv = umma_desc(smem_u32(Vst + sv * kVBytes));
#pragma unroll
                for (int k = 0; k < kAttnKeys / 16; ++k)
                    umma_bf16(tmem_base + kColO, dp + 2 * k, dv + 2 * k, idesc_o,
                              (g > n1 || k > 0) ? 1u : 0u);
                umma_commit(&v_empty[sv]);
                umma_commit(&p_empty[st]);
                return true;
            };
            for (int g = 0; ok && g < steps; ++g) {
                const int st = g & 1;
                if (!mbar_wait_bounded(&k_full[st], (g >> 1) & 1, abort_flag) ||
                    (g >= 2 && !mbar_wait_bounded(&s_empty[st], ((g >> 1) - 1) & 1, abort_flag))) {
                    give_up(22);
                    ok = false;
                    break;
                }
                tc_fence_after();
#pragma unroll
                for (int kb = 0; kb < D / 64; ++kb) {
                    const unsigned long long dq = umma_desc(smem_u32(Qs + kb * (kTcRows * 128)));
                    const unsigned long long dk =
                        umma_desc(smem_u32(Kst + st * kKBytes + kb * (kAttnKeys * 128)));
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma_bf16(tmem_base + st * kAttnKeys, dq + 2 * k, dk + 2 * k, idesc_s,
                                  (kb | k) != 0 ? 1u : 0u);
                }
                umma_commit(&s_full[st]);
                umma_commit(&k_empty[st]);  // the K stage is free as soon as these MMAs have read it
                if (g > n1) ok = issue_pv(g - 1);
            }
            if (ok && steps > n1) ok = issue_pv(steps - 1);
            if (ok && steps > n1) umma_commit(o_full);
        }
        __syncwarp();
    } else {
        const int quarter = warp & 3;            // TMEM lanes this warp may touch
        const int part = (warp - 2) >> 2;        // which 16 key columns of a block
        const int r = quarter * 32 + lane;       // row of the tile
        const int row = q0 + r;
        const unsigned int lane_addr = tmem_base + (static_cast<unsigned int>(quarter * 32) << 16);
        const unsigned short* mrow = nullptr;
        if (a.mask != nullptr)
            mrow = a.mask + (a.mask_batch > 1 ? static_cast<size_t>(b) * T * T : 0) +
                   static_cast<size_t>(min(row, T - 1)) * T;
        float m_run = -INFINITY, l_run = 0.f, inv_l = 0.f;
        bool ok = true;
        // a power of two times a bf16 value is exact: rounding the product again is a no-op
        const bool scale_exact = (__float_as_uint(a.scale) & 0x007fffffu) == 0u;
        const size_t stats_row = (static_cast<size_t>(item) * a.parts_max) * kTcRows + r;
        if (a.mode == kAttnValues) {
            // the first sweep ran as a launch of its own: combine the parts' statistics, in
            // part order, exactly as the column parts of one CTA are combined below
            float fm = -INFINITY;
            for (int q = 0; q < parts; ++q)
                fm = fmaxf(fm, __ldcg(a.stats_ws + (stats_row + static_cast<size_t>(q) * kTcRows) * 2));
            const float fbase = fm == -INFINITY ? 0.f : fm;
            float total = 0.f;
            for (int q = 0; q < parts; ++q) {
                const float* entry = a.stats_ws + (stats_row + static_cast<size_t>(q) * kTcRows) * 2;
                total += __ldcg(entry + 1) * __expf(__ldcg(entry) - fbase);
            }
            m_run = fbase;
            inv_l = total > 0.f ? __frcp_rn(total) : 0.f;
        }
        for (int g = 0; g < steps; ++g) {
            const int st = g & 1, jb = j_begin + (g < n1 ? g : g - n1);
            ok = ok && __all_sync(0xffffffffu, mbar_wait_bounded(&s_full[st], (g >> 1) & 1, abort_flag));
            if (!ok) {
                if (lane == 0) give_up(30);
                break;
            }
            tc_fence_after();
            float v[16];
            tmem_load16(lane_addr + st * kAttnKeys + part * 16, v);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_empty[st]);  // per-thread arrivals would serialise
            const int key0 = jb * kAttnKeys + part * 16;
            // scores with the operator's rounding points; -inf marks keys that are not visible.
            // The softmax warps are bound by the instructions they issue (measured: two sets
            // of warps on alternate steps gain nothing), so the common block -- every key
            // visible to every row of the tile, no mask tensor -- skips the visibility tests,
            // and a power-of-two scale (head sizes 64 and 256) skips a rounding that changes
            // nothing.
            const bool interior = mrow == nullptr && jb * kAttnKeys + kAttnKeys <= T &&
                                  (!a.causal || jb * kAttnKeys + kAttnKeys - 1 <= q0);
            // `unit`: what one unit of v is worth in scaled scores.  On the common path v stays
            // unscaled and the scale rides along in the exponent's multiplier and in the row
            // maximum (a power of two commutes with both): one multiplication per element less.
            const bool folded = interior && scale_exact;
            const float unit = folded ? a.scale : 1.0f;
            const float to_log2 = unit * 1.4426950408889634f;
            if (folded) {
#pragma unroll
                for (int i = 0; i < 16; ++i) v[i] = bf16_round(v[i]);
            } else if (interior) {
#pragma unroll
                for (int i = 0; i < 16; ++i) v[i] = bf16_round(bf16_round(v[i]) * a.scale);
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int key = key0 + i;
                    float t = bf16_round(v[i]);
                    t = bf16_round(t * a.scale);
                    if (mrow != nullptr && key < T) t = bf16_round(t + bf16_bits_to_float(__ldg(mrow + key)));
                    v[i] = (key < T && (!a.causal || key <= row)) ? t : -INFINITY;
                }
            }
            if (g < n1) {
                float bm = -INFINITY;
#pragma unroll
                for (int i = 0; i < 16; ++i) bm = fmaxf(bm, v[i]);
                const float nm = fmaxf(m_run, bm * unit);
                // exp(-inf - x) is 0 for every finite x: invisible keys need no branch, only a
                // maximum that is still -inf must not be subtracted
                const float base = nm == -INFINITY ? 0.f : nm;
                float sum = l_run * __expf(m_run - base);
                // exp(s - base) as 2^(v * to_log2 - base * log2 e), one fused multiply-add and one
                // ex2 per element (the softmax warps are bound by the instructions they issue)
                // (a mask tensor of finite minima can leave a maximum near -3.4e38, whose product
                // with log2 e overflows: such rows subtract first, as the plain formula does)
                const float base_log2 = base * 1.4426950408889634f;
                if (base > -1e30f) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) sum += exp2_approx(__fmaf_rn(v[i], to_log2, -base_log2));
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) sum += __expf(v[i] * unit - base);
                }
                l_run = sum;
                m_run = nm;
                if (g == n1 - 1) {
                    // the four parts of a row meet: combine their maxima and denominators, in
                    // part order, so that all four get the same sum
                    stats[(part * kTcRows + r) * 2] = m_run;
                    stats[(part * kTcRows + r) * 2 + 1] = l_run;
                    __syncwarp();
                    if (lane == 0) mbar_arrive(x_full);
                    if (!__all_sync(0xffffffffu, mbar_wait_bounded(x_full, 0, abort_flag))) {
                        if (lane == 0) give_up(33);
                        ok = false;
                        break;
                    }
                    float fm = -INFINITY;
#pragma unroll
                    for (int q = 0; q < 4; ++q) fm = fmaxf(fm, stats[(q * kTcRows + r) * 2]);
                    const float fbase = fm == -INFINITY ? 0.f : fm;
                    float total = 0.f;
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        total += stats[(q * kTcRows + r) * 2 + 1] *
                                 __expf(stats[(q * kTcRows + r) * 2] - fbase);
                    m_run = fbase;
                    inv_l = total > 0.f ? __frcp_rn(total) : 0.f;
                    if (a.mode == kAttnStats && part == 0) {
                        float* entry = a.stats_ws + (stats_row + static_cast<size_t>(part_index) * kTcRows) * 2;
                        __stcg(entry, fm);
                        __stcg(entry + 1, total);
                    }
                    // nobody may overwrite the statistics (they alias the first P tile) before
                    // every warp has read them
                    __syncwarp();
                    if (lane == 0) mbar_arrive(x_full);
                    if (!__all_sync(0xffffffffu, mbar_wait_bounded(x_full, 1, abort_flag))) {
                        if (lane == 0) give_up(34);
                        ok = false;
                        break;
                    }
                }
            } else {
                if (g >= n1 + 2 &&
                    !__all_sync(0xffffffffu,
                                mbar_wait_bounded(&p_empty[st], (((g - n1) >> 1) - 1) & 1, abort_flag))) {
                    if (lane == 0) give_up(31);
                    ok = false;
                    break;
                }
                const float max_log2 = m_run * 1.4426950408889634f;
                unsigned int packed[8];
                if (m_run > -1e30f) {
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        packed[i] = pack_bf16_pair(
                            exp2_approx(__fmaf_rn(v[2 * i], to_log2, -max_log2)) * inv_l,
                            exp2_approx(__fmaf_rn(v[2 * i + 1], to_log2, -max_log2)) * inv_l);
                } else {  // a row whose every key is masked by a finite minimum: subtract first
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        packed[i] = pack_bf16_pair(__expf(v[2 * i] * unit - m_run) * inv_l,
                                                   __expf(v[2 * i + 1] * unit - m_run) * inv_l);
                }
                // row r of the P tile: 128 bytes, 16-byte chunk c stored at c ^ (r % 8) (the
                // 128-byte swizzle the MMA's shared-memory descriptor expects)
                unsigned char* prow = Ps + st * kPBytes + r * 128;
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int chunk = (part * 2 + c) ^ (r & 7);
                    *reinterpret_cast<uint4*>(prow + chunk * 16) =
                        make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
                }
                // generic-proxy writes must be visible to the tensor core's async-proxy reads
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(&p_full[st]);
            }
        }
        if (a.mode != kAttnStats) {
            ok = ok && __all_sync(0xffffffffu, mbar_wait_bounded(o_full, 0, abort_flag));
            if (!ok && lane == 0 && *abort_flag == 0) give_up(32);
            tc_fence_after();
        }
        if (a.mode == kAttnValues && parts > 1) {
            // Several CTAs hold parts of this tile's output: park this one ([column][row], a warp's
            // 32 rows are one 128-byte line), and let the part that arrives last add them in key
            // order and round once.  The sixteen warps meet at barriers: all leave or none.
            if (!named_barrier_or(3, kTcSoftmaxWarps * 32, !ok)) {
                const size_t tile_floats = static_cast<size_t>(D) * kTcRows;
                float* parts_base = a.o_ws + static_cast<size_t>(item) * a.parts_max * tile_floats + r;
                float* mine = parts_base + part_index * tile_floats;
#pragma unroll 1
                for (int c = 0; c < D / 64; ++c) {
                    float o[16];
                    tmem_load16(lane_addr + kColO + part * (D / 4) + c * 16, o);
#pragma unroll
                    for (int i = 0; i < 16; ++i) __stcg(mine + (part * (D / 4) + c * 16 + i) * kTcRows, o[i]);
                }
                __threadfence();
                named_barrier(4, kTcSoftmaxWarps * 32);
                if (warp == 2 && lane == 0) {
                    const int arrived = atomicAdd(a.counters + item, 1);
                    *last_flag = arrived == parts - 1 ? 1 : 0;
                    if (arrived == parts - 1) a.counters[item] = 0;  // re-arm for the next launch
                    __threadfence();
                }
                named_barrier(4, kTcSoftmaxWarps * 32);
                if (*last_flag != 0 && row < T) {
                    unsigned short* orow = a.out + (static_cast<size_t>(b) * T + row) * (static_cast<size_t>(a.heads) * D) +
                                           head * D + part * (D / 4);
#pragma unroll 1
                    for (int c = 0; c < D / 64; ++c) {
                        float o[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) o[i] = 0.f;
                        for (int q = 0; q < parts; ++q) {
                            const float* theirs = parts_base + q * tile_floats;
#pragma unroll
                            for (int i = 0; i < 16; ++i)
                                o[i] += __ldcg(theirs + (part * (D / 4) + c * 16 + i) * kTcRows);
                        }
#pragma unroll
                        for (int q = 0; q < 2; ++q)
                            reinterpret_cast<uint4*>(orow + c * 16)[q] =
                                make_uint4(pack_bf16(o[8 * q], o[8 * q + 1]), pack_bf16(o[8 * q + 2], o[8 * q + 3]),
                                           pack_bf16(o[8 * q + 4], o[8 * q + 5]), pack_bf16(o[8 * q + 6], o[8 * q + 7]));
                    }
                }
            }
        } else if (ok && a.mode != kAttnStats) {
            unsigned short* orow = a.out + (static_cast<size_t>(b) * T + row) * (static_cast<size_t>(a.heads) * D) +
                                   head * D + part * (D / 4);
#pragma unroll 1
            for (int c = 0; c < D / 64; ++c) {
                float o[16];
                tmem_load16(lane_addr + kColO + part * (D / 4) + c * 16, o);
                if (row < T) {
#pragma unroll
                    for (int q = 0; q < 2; ++q)
                        reinterpret_cast<uint4*>(orow + c * 16)[q] =
                            make_uint4(pack_bf16(o[8 * q], o[8 * q + 1]), pack_bf16(o[8 * q + 2], o[8 * q + 3]),
                                       pack_bf16(o[8 * q + 4], o[8 * q + 5]), pack_bf16(o[8 * q + 6], o[8 * q + 7]));
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        const unsigned long long start = global_timer_ns();
        while (global_timer_ns() - start < 200000ull) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

inline int attention_tc_smem_bytes(int D) {
    return kTcRows * D * 2 + 2 * kAttnKeys * D * 2 + 2 * D * kAttnKeys * 2 + 2 * kTcRows * kAttnKeys * 2 +
           21 * 8;
}

// How attention_tc_kernel shares out the keys of a query tile (host side of the kernel's own
// arithmetic): parts of at most `chunk` key blocks, at most four per tile.
struct AttnParts {
    int chunk = 0;      // 0: one CTA per tile, both sweeps in one launch
    int parts_max = 1;
    int grid_x = 0;     // CTAs per (head, batch row)
    int items = 0;      // query tiles x heads x batch rows
    size_t stats_floats = 0, output_floats = 0;
};

inline AttnParts attention_parts(int batch, int tokens, int heads, int D, bool causal, int sm_count) {
    AttnParts p;
    const int all_blocks = (tokens + kAttnKeys - 1) / kAttnKeys;
    const int q_tiles = (tokens + kTcRows - 1) / kTcRows;
    p.items = q_tiles * heads * batch;
    p.grid_x = q_tiles;
    const char* env = std::getenv("MEGABAKE_B200_ATTN_PARTS");
    const bool allowed = env == nullptr || std::atoi(env) != 0;
    if (!allowed || all_blocks < 4) return p;
    // Which chunk?  Measured on the gemma-2b shape: a CTA costs 4.5 us before and after its key
    // blocks and 1.84 us per block and sweep, CTAs run one per SM and are handed out in grid
    // order, heaviest first.  The host plays that schedule for every way of cutting the keys
    // into at most eight parts per tile, and for whole tiles, and keeps the shortest.
    auto visible_blocks = [&](int qt) {
        const int last_row = (qt * kTcRows + kTcRows < tokens ? qt * kTcRows + kTcRows : tokens) - 1;
        const int visible = causal ? last_row / kAttnKeys + 1 : all_blocks;
        return visible < all_blocks ? visible : all_blocks;
    };
    auto makespan = [&](int chunk, double per_block, double merge) {
        std::vector<double> free_at(sm_count, 0.0);
        double end = 0.0;
        for (int qt = q_tiles - 1; qt >= 0; --qt) {
            const int visible = visible_blocks(qt);
            const int parts = chunk > 0 ? (visible + chunk - 1) / chunk : 1;
            const int per_part = (visible + parts - 1) / parts;
            for (int part = 0; part < parts; ++part) {
                const int begin = part * per_part < visible ? part * per_part : visible;
                const int blocks = (begin + per_part < visible ? begin + per_part : visible) - begin;
                for (int copy = 0; copy < heads * batch; ++copy) {
                    size_t first = 0;
                    for (size_t m = 1; m < free_at.size(); ++m)
                        if (free_at[m] < free_at[first]) first = m;
                    free_at[first] += 4.5 + blocks * per_block + (parts > 1 ? merge : 0.0);
                    if (free_at[first] > end) end = free_at[first];
                }
            }
        }
        return end;
    };
    double best = makespan(0, 2 * 1.84, 0.0);
    for (int parts = 2; parts <= 8 && parts <= all_blocks; ++parts) {
        const int chunk = (all_blocks + parts - 1) / parts;
        if ((all_blocks + chunk - 1) / chunk != parts) continue;  // same cut as a smaller count
        const double cost = makespan(chunk, 1.84, 0.0) + makespan(chunk, 1.84, 2.0) + 3.0;
        if (cost < best) {
            best = cost;
            p.chunk = chunk;
        }
    }
    if (const char* forced = std::getenv("MEGABAKE_B200_ATTN_CHUNK")) {
        const int value = std::atoi(forced);
        if (value >= 1 && (all_blocks + value - 1) / value <= 8) p.chunk = value;
    }
    if (p.chunk == 0) return p;
    p.parts_max = (all_blocks + p.chunk - 1) / p.chunk;
    p.grid_x = 0;
    for (int qt = 0; qt < q_tiles; ++qt) {
        const int last_row = (qt * kTcRows + kTcRows < tokens ? qt * kTcRows + kTcRows : tokens) - 1;
        int visible = causal ? last_row / kAttnKeys + 1 : all_blocks;
        if (visible > all_blocks) visible = all_blocks;
        p.grid_x += (visible + p.chunk - 1) / p.chunk;
    }
    p.stats_floats = static_cast<size_t>(p.items) * p.parts_max * kTcRows * 2;
    p.output_floats = static_cast<size_t>(p.items) * p.parts_max * kTcRows * D;
    return p;
}

// ---------------------------------------------------------------------------------------
// Host side: validation, tile / split-K geometry, tensor maps, launches.
// ---------------------------------------------------------------------------------------
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &result) ==
                cudaSuccess &&
            result == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

// [rows, K] bf16 row-major, boxes of `box_rows` x 64 elements, 128-byte swizzle, zero fill
// outside the tensor.
bool make_map(CUtensorMap* map, unsigned long long base, int rows, int K, int box_rows) {
    EncodeTiledFn fn = encode_tiled();
    if (fn == nullptr) return false;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(K) * 2};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(kTileK), static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, reinterpret_cast<void*>(base), dims,
              strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int gemm_smem_bytes(int bn, int stages) {
    return stages * (kStageA + bn * kTileK * 2) + 256 + 1024;  // ring + barriers + alignment slack
}

struct GemmGeometry {
    int bn, stages, tiles_n, tiles_m, split_k, kblocks;
    int persistent;  // 1: gemm_tc_persistent_kernel on `grid` CTAs
    int grid;
    int tile_start[3];
};

GemmGeometry gemm_geometry(const mb_phase& P, int sm_count) {
    GemmGeometry g;
    const int M = P.i[MB_GV_I_ROWS], K = P.i[MB_GV_I_K];
    const bool pair = P.i[MB_GV_I_NMAT] == 2;
    g.tiles_m = (M + kTileM - 1) / kTileM;
    g.kblocks = (K + kTileK - 1) / kTileK;
    // wide tiles once there are enough of them to fill the machine; they halve the shared-
    // memory traffic per flop
    auto count = [&](int bn) {
        int tiles = 0;
        const int per = pair ? bn / 2 : bn;
        for (int s = 0; s < P.i[MB_GV_I_NSEG]; ++s) tiles += (P.i[MB_GV_I_N0 + s] + per - 1) / per;
        return tiles;
    };
    g.bn = count(256) * g.tiles_m >= sm_count ? 256 : 128;
    // the persistent kernel once its tiles fill most of the machine: wide tiles from 80 % of
    // the SMs on (a single wave of them moves a third less operand bytes than two CTAs per SM
    // on narrow ones), narrow tiles when only those reach one per SM
    g.persistent = 0;
    int persistent_split = 1;
    const char* persistent_env = std::getenv("MEGABAKE_B200_GEMM_PERSISTENT");
    if (persistent_env == nullptr || std::atoi(persistent_env) != 0) {
        // Tile width and number of reduction slices by a cost model in microseconds, fitted to
        // a sweep of both over the twelve GEMM shapes of the gemma-2b prefill (128 / 512 / 2048
        // rows): a CTA takes a k-block every 0.44 us (256 columns) or 0.30 us (128) when every
        // SM streams operands; the weights cannot arrive faster than HBM delivers them; a wave
        // of sliced tiles pays 4 us (2 us) for parking its partial sums and the last slice
        // 2 us (1 us) per slice for its pass over them, a chain of L2 round trips.
        g.persistent = 1;
        double best = 1e30;
        const double weight_bytes = 2.0 * K * (pair ? 2 : 1) * [&] {
            long long n = 0;
            for (int s = 0; s < P.i[MB_GV_I_NSEG]; ++s) n += P.i[MB_GV_I_N0 + s];
            return static_cast<double>(n);
        }();
        for (int bn = 256; bn >= 128; bn -= 128) {
            const int tiles = count(bn) * g.tiles_m;
            for (int split = 1; split <= 16; ++split) {
                if (split > 1 && g.kblocks / split < 4) break;
                const int units = tiles * split;
                const int waves = (units + sm_count - 1) / sm_count;
                const int per_unit = (g.kblocks + split - 1) / split;
                double stream = waves * per_unit * (bn == 256 ? 0.44 : 0.30);
                const double hbm = weight_bytes / 6.0e6;
                if (stream < hbm) stream = hbm;
                const double slices =
                    split > 1 ? (bn == 256 ? 4.0 : 2.0) * waves + (bn == 256 ? 2.0 : 1.0) * split : 0.0;
                const double cost = stream + slices;
                if (cost < best - 1e-9) {
                    best = cost;
                    g.bn = bn;
                    persistent_split = split;
                }
            }
        }
    }
    if (const char* forced = std::getenv("MEGABAKE_B200_GEMM_BN")) {
        const int value = std::atoi(forced);
        if (value == 128 || value == 256) g.bn = value;
    }
    // two CTAs per SM: while one runs its epilogue the other one keeps the tensor cores busy
    g.stages = g.bn == 256 ? 2 : 3;
    if (const char* forced = std::getenv("MEGABAKE_B200_GEMM_STAGES")) {
        const int value = std::atoi(forced);
        if (value >= 2 && value <= (g.bn == 256 ? 4 : 6)) g.stages = value;
    }
    const int per = pair ? g.bn / 2 : g.bn;
    int tiles = 0;
    for (int s = 0; s < 3; ++s) {
        g.tile_start[s] = s < P.i[MB_GV_I_NSEG] ? tiles : INT_MAX;
        if (s < P.i[MB_GV_I_NSEG]) tiles += (P.i[MB_GV_I_N0 + s] + per - 1) / per;
    }
    g.tiles_n = tiles;
    // split the reduction when the output tiles alone leave SMs idle: aim at two CTAs per SM,
    // keep at least eight k-blocks per CTA (measured: shorter slices lose more to the pipeline
    // fill and the partial-sum round trip than they gain)
    int split = 1;
    const int ctas = g.tiles_n * g.tiles_m;
    if (ctas < sm_count) {
        split = 2 * sm_count / ctas;
        if (split > g.kblocks / 8) split = g.kblocks / 8;
        if (split > 16) split = 16;
        if (split < 1) split = 1;
    }
    if (const char* forced = std::getenv("MEGABAKE_B200_GEMM_SPLIT")) {
        const int value = std::atoi(forced);
        if (value >= 1 && value <= 16 && value <= g.kblocks) split = value;
    }
    if (g.persistent) {
        split = persistent_split;
        if (const char* forced = std::getenv("MEGABAKE_B200_GEMM_SPLIT")) {
            const int value = std::atoi(forced);
            if (value >= 1 && value <= 16 && value <= g.kblocks) split = value;
        }
    }
    g.split_k = split;
    const int units = g.tiles_n * g.tiles_m * g.split_k;
    g.grid = units < sm_count ? units : sm_count;
    return g;
}

}  // namespace

struct PrefillLaunch {
    int body = MB_BODY_NOP;
    GemmMaps maps;
    GemmArgs gemm;
    GemmGeometry geometry;
    AttnArgs attn;
    AttnMaps attn_maps;
    unsigned short* vt = nullptr;  // transposed values of the tensor-core attention, or null
    int padded_tokens = 0;
    bool tensor_core = false;      // the phase names scratch for transposed values
    AttnParts parts;
};

}  // namespace prefill

struct PrefillState {
    std::vector<prefill::PrefillLaunch> launches;
    float* workspace = nullptr;
    int* counters = nullptr;
    size_t workspace_floats = 0;
    size_t counter_count = 0;
    int sm_count = 0;
};

int prefill_validate(const mb_phase& P, unsigned int n_slots, unsigned int n_dynamic) {
    auto slot_ok = [&](int s, bool required, bool may_be_dynamic) {
        if (s < 0) return !required;
        if (static_cast<unsigned int>(s) >= n_slots) return false;
        return may_be_dynamic || static_cast<unsigned int>(s) >= n_dynamic;
    };
    switch (P.body) {
        case MB_BODY_NOP:
            return MB_OK;
        case MB_BODY_EMBED_ROWS:
            if (P.i[MB_EM_I_ROWS] < 1 || P.i[MB_EM_I_K] < 8 || P.i[MB_EM_I_K] % 8 ||
                P.i[MB_EM_I_VOCAB] < 1)
                return MB_ERR_INVALID;
            if (!slot_ok(P.slot[MB_EM_S_TABLE], true, false) ||
                !slot_ok(P.slot[MB_EM_S_IDS], true, true) || !slot_ok(P.slot[MB_EM_S_OUT], true, false))
                return MB_ERR_INVALID;
            return MB_OK;
        case MB_BODY_RMSNORM_ROWS:
            if (P.i[MB_RN_I_ROWS] < 1 || P.i[MB_RN_I_K] < 8 || P.i[MB_RN_I_K] % 8)
                return MB_ERR_INVALID;
            if (P.i[MB_RN_I_KIND] != MB_PRO_RMS_LLAMA && P.i[MB_RN_I_KIND] != MB_PRO_RMS_GEMMA)
                return MB_ERR_INVALID;
            for (int s = 0; s < 3; ++s)
                if (!slot_ok(P.slot[s], true, false)) return MB_ERR_INVALID;
            return MB_OK;
        case MB_BODY_GEMM_TC: {
            const int nseg = P.i[MB_GV_I_NSEG], nmat = P.i[MB_GV_I_NMAT], epi = P.i[MB_GV_I_EPILOGUE];
            if (P.i[MB_GV_I_ROWS] < 1 || P.i[MB_GV_I_K] < 8 || P.i[MB_GV_I_K] % 8) return MB_ERR_INVALID;
            if (nseg < 1 || nseg > 3 || (nmat != 1 && nmat != 2)) return MB_ERR_INVALID;
            if (P.i[MB_GV_I_PROLOGUE] != MB_PRO_NONE || P.i[MB_GV_I_GATHER] != 0)
                return MB_ERR_UNSUPPORTED;
            const bool gated = epi == MB_EPI_SILU_MUL || epi == MB_EPI_GELU_TANH_MUL;
            if (gated != (nmat == 2) || (nmat == 2 && nseg != 1)) return MB_ERR_INVALID;
            if (epi < MB_EPI_NONE || epi > MB_EPI_GELU_TANH_MUL) return MB_ERR_INVALID;
            if (P.i[MB_GV_I_OUT_TOKENS] < 0 ||
                (P.i[MB_GV_I_OUT_TOKENS] > 0 && P.i[MB_GV_I_OUT_CAPACITY] < P.i[MB_GV_I_OUT_TOKENS]))
                return MB_ERR_INVALID;
            if (!slot_ok(P.slot[MB_GV_S_X], true, false)) return MB_ERR_INVALID;
            for (int s = 0; s < nseg; ++s) {
                if (P.i[MB_GV_I_N0 + s] < 1) return MB_ERR_INVALID;
                if (!slot_ok(P.slot[MB_GV_S_W0 + s], true, false) ||
                    !slot_ok(P.slot[MB_GV_S_OUT0 + s], true, true) ||
                    !slot_ok(P.slot[MB_GV_S_BIAS0 + s], false, false))
                    return MB_ERR_INVALID;
            }
            if (nmat == 2 && !slot_ok(P.slot[MB_GV_S_W_PAIR], true, false)) return MB_ERR_INVALID;
            if (epi == MB_EPI_RESIDUAL &&
                (nseg != 1 || !slot_ok(P.slot[MB_GV_S_RESIDUAL], true, false)))
                return MB_ERR_INVALID;
            return MB_OK;
        }
        case MB_BODY_ROPE_ROWS: {
            const int D = P.i[MB_RP_I_HEAD_DIM];
            if (P.i[MB_RP_I_ROWS] < 1 || P.i[MB_RP_I_HEADS] < 1 || P.i[MB_RP_I_KV_HEADS] < 1 ||
                D < 2 || D % 2)
                return MB_ERR_INVALID;
            for (int s = 0; s < 4; ++s)
                if (!slot_ok(P.slot[s], true, s == MB_RP_S_POS)) return MB_ERR_INVALID;
            if (!slot_ok(P.slot[MB_RP_S_LEN], false, false)) return MB_ERR_INVALID;
            if (P.i[MB_RP_I_K_TOKENS] > 0 && P.i[MB_RP_I_K_CAPACITY] < P.i[MB_RP_I_K_TOKENS])
                return MB_ERR_INVALID;
            return MB_OK;
        }
        case MB_BODY_ATTN_PREFILL: {
            const int D = P.i[MB_AP_I_HEAD_DIM];
            if (D != 64 && D != 128 && D != 256) return MB_ERR_UNSUPPORTED;
            if (P.i[MB_AP_I_BATCH] < 1 || P.i[MB_AP_I_TOKENS] < 1 || P.i[MB_AP_I_HEADS] < 1 ||
                P.i[MB_AP_I_KV_HEADS] < 1 || P.i[MB_AP_I_HEADS] % P.i[MB_AP_I_KV_HEADS])
                return MB_ERR_INVALID;
            if (P.i[MB_AP_I_BATCH] > 65535 || P.i[MB_AP_I_HEADS] > 65535) return MB_ERR_UNSUPPORTED;
            for (int s = 0; s < 4; ++s)
                if (!slot_ok(P.slot[s], true, false)) return MB_ERR_INVALID;
            if (!slot_ok(P.slot[MB_AP_S_MASK], false, false)) return MB_ERR_INVALID;
            if (!slot_ok(P.slot[MB_AP_S_VT], false, false)) return MB_ERR_INVALID;
            if (P.slot[MB_AP_S_MASK] >= 0 && P.i[MB_AP_I_MASK_BATCH] != 1 &&
                P.i[MB_AP_I_MASK_BATCH] != P.i[MB_AP_I_BATCH])
                return MB_ERR_INVALID;
            return MB_OK;
        }
        default:
            return MB_ERR_UNSUPPORTED;
    }
}

// Creates the per-plan state: geometry of every GEMM (written back into the phase records so
// that mb_plan users can read it) and the split-K workspace.
cudaError_t prefill_create(std::vector<mb_phase>& phases, int sm_count, PrefillState** out) {
    using namespace prefill;
    PrefillState* st = new (std::nothrow) PrefillState();
    if (st == nullptr) return cudaErrorMemoryAllocation;
    st->sm_count = sm_count;
    st->launches.resize(phases.size());
    size_t floats = 0, counters = 0;
    for (size_t i = 0; i < phases.size(); ++i) {
        mb_phase& P = phases[i];
        st->launches[i].body = P.body;
        if (P.body == MB_BODY_ATTN_PREFILL && P.slot[MB_AP_S_VT] >= 0) {
            const AttnParts parts = attention_parts(P.i[MB_AP_I_BATCH], P.i[MB_AP_I_TOKENS], P.i[MB_AP_I_HEADS],
                                                    P.i[MB_AP_I_HEAD_DIM], P.i[MB_AP_I_CAUSAL] != 0, sm_count);
            st->launches[i].parts = parts;
            st->launches[i].tensor_core = true;
            if (parts.chunk > 0) {
                const size_t need = parts.stats_floats + parts.output_floats;
                if (need > floats) floats = need;
                if (static_cast<size_t>(parts.items) > counters) counters = parts.items;
            }
        }
        if (P.body != MB_BODY_GEMM_TC) continue;
        GemmGeometry g = gemm_geometry(P, sm_count);
        st->launches[i].geometry = g;
        P.i[MB_GV_I_SPLIT_K] = g.split_k;
        P.i[MB_GV_I_TILE_N] = g.bn;
        const size_t tiles = static_cast<size_t>(g.tiles_n) * g.tiles_m;
        if (g.split_k > 1) {
            const size_t need = tiles * g.split_k * kTileM * g.bn;
            if (need > floats) floats = need;
            if (tiles > counters) counters = tiles;
        }
    }
    cudaError_t err = cudaSuccess;
    if (floats > 0) {
        err = cudaMalloc(&st->workspace, floats * sizeof(float));
        if (err == cudaSuccess) err = cudaMalloc(&st->counters, counters * sizeof(int));
        if (err == cudaSuccess) err = cudaMemset(st->counters, 0, counters * sizeof(int));
    }
    if (err == cudaSuccess)
        err = cudaFuncSetAttribute(gemm_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   gemm_smem_bytes(128, 6));
    if (err == cudaSuccess)
        err = cudaFuncSetAttribute(gemm_tc_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   gemm_smem_bytes(256, 4));
    if (err == cudaSuccess)
        err = cudaFuncSetAttribute(gemm_tc_persistent_kernel<128>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, kPersistSmemBytes);
    if (err == cudaSuccess)
        err = cudaFuncSetAttribute(gemm_tc_persistent_kernel<256>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, kPersistSmemBytes);
    if (err == cudaSuccess)
        err = cudaFuncSetAttribute(attention_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   attention_tc_smem_bytes(64));
    if (err == cudaSuccess)
        err = cudaFuncSetAttribute(attention_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   attention_tc_smem_bytes(128));
    if (err == cudaSuccess)
        err = cudaFuncSetAttribute(attention_tc_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   attention_tc_smem_bytes(256));
    if (err == cudaSuccess) err = attn_configure<64>();
    if (err == cudaSuccess) err = attn_configure<128>();
    if (err == cudaSuccess) err = attn_configure<256>();
    if (err != cudaSuccess) {
        prefill_destroy(st);
        return err;
    }
    st->workspace_floats = floats;
    st->counter_count = counters;
    *out = st;
    return cudaSuccess;
}

int prefill_launch_count(const PrefillState* st) {
    using namespace prefill;
    if (st == nullptr) return 0;
    int count = 0;
    for (size_t i = 0; i < st->launches.size(); ++i) {
        const PrefillLaunch& L = st->launches[i];
        if (L.body == MB_BODY_NOP) continue;
        if (L.body != MB_BODY_ATTN_PREFILL || !L.tensor_core) {
            ++count;
            continue;
        }
        // values transposed by the rotary phase just before, or by a launch of their own
        if (i == 0 || st->launches[i - 1].body != MB_BODY_ROPE_ROWS) ++count;
        count += L.parts.chunk > 0 ? 2 : 1;
    }
    return count;
}

void prefill_destroy(PrefillState* st) {
    if (st == nullptr) return;
    if (st->workspace != nullptr) cudaFree(st->workspace);
    if (st->counters != nullptr) cudaFree(st->counters);
    delete st;
}

// Resolves the static addresses of every phase into launch arguments and tensor maps.
int prefill_bind(PrefillState* st, const std::vector<mb_phase>& phases,
                 const std::vector<unsigned long long>& slots, Control* ctl) {
    using namespace prefill;
    auto addr = [&](int s) -> unsigned long long { return s < 0 ? 0ull : slots[s]; };
    for (size_t i = 0; i < phases.size(); ++i) {
        const mb_phase& P = phases[i];
        PrefillLaunch& L = st->launches[i];
        if (P.body == MB_BODY_GEMM_TC) {
            const GemmGeometry& g = L.geometry;
            GemmArgs& a = L.gemm;
            std::memset(&a, 0, sizeof(a));
            a.M = P.i[MB_GV_I_ROWS];
            a.K = P.i[MB_GV_I_K];
            a.kblocks = g.kblocks;
            a.split_k = g.split_k;
            a.stages = g.stages;
            a.phase = static_cast<int>(i);
            a.nseg = P.i[MB_GV_I_NSEG];
            a.pair = P.i[MB_GV_I_NMAT] == 2 ? 1 : 0;
            a.epilogue = P.i[MB_GV_I_EPILOGUE];
            a.out_tokens = P.i[MB_GV_I_OUT_TOKENS];
            a.out_capacity = P.i[MB_GV_I_OUT_CAPACITY];
            a.tiles_n = g.tiles_n;
            a.tiles_m = g.tiles_m;
            for (int s = 0; s < 3; ++s) {
                a.n[s] = s < a.nseg ? P.i[MB_GV_I_N0 + s] : 0;
                a.tile_start[s] = g.tile_start[s];
                a.out[s] = reinterpret_cast<unsigned short*>(addr(s < a.nseg ? P.slot[MB_GV_S_OUT0 + s] : -1));
                a.bias[s] = reinterpret_cast<const unsigned short*>(
                    addr(s < a.nseg ? P.slot[MB_GV_S_BIAS0 + s] : -1));
            }
            a.residual = reinterpret_cast<const unsigned short*>(
                addr(a.epilogue == MB_EPI_RESIDUAL ? P.slot[MB_GV_S_RESIDUAL] : -1));
            a.workspace = st->workspace;
            a.counters = st->counters;
            a.ctl = ctl;
            if (!make_map(&L.maps.a, addr(P.slot[MB_GV_S_X]), a.M, a.K, kTileM)) return MB_ERR_CUDA;
            const int box = a.pair ? g.bn / 2 : g.bn;
            for (int s = 0; s < a.nseg; ++s)
                if (!make_map(&L.maps.w[s], addr(P.slot[MB_GV_S_W0 + s]), a.n[s], a.K, box))
                    return MB_ERR_CUDA;
            if (a.pair &&
                !make_map(&L.maps.w[3], addr(P.slot[MB_GV_S_W_PAIR]), a.n[0], a.K, box))
                return MB_ERR_CUDA;
        } else if (P.body == MB_BODY_ATTN_PREFILL) {
            AttnArgs& a = L.attn;
            a.q = reinterpret_cast<const unsigned short*>(addr(P.slot[MB_AP_S_Q]));
            a.k = reinterpret_cast<const unsigned short*>(addr(P.slot[MB_AP_S_K]));
            a.v = reinterpret_cast<const unsigned short*>(addr(P.slot[MB_AP_S_V]));
            a.out = reinterpret_cast<unsigned short*>(addr(P.slot[MB_AP_S_OUT]));
            a.mask = reinterpret_cast<const unsigned short*>(addr(P.slot[MB_AP_S_MASK]));
            a.batch = P.i[MB_AP_I_BATCH];
            a.tokens = P.i[MB_AP_I_TOKENS];
            a.heads = P.i[MB_AP_I_HEADS];
            a.kv_heads = P.i[MB_AP_I_KV_HEADS];
            a.causal = P.i[MB_AP_I_CAUSAL];
            a.mask_batch = P.i[MB_AP_I_MASK_BATCH];
            a.kv_rows = P.i[MB_AP_I_KV_CAPACITY] > 0 ? P.i[MB_AP_I_KV_CAPACITY] : a.tokens;
            a.scale = P.f[MB_AP_F_SCALE];
            a.mode = kAttnWhole;
            a.chunk = L.parts.chunk;
            a.parts_max = L.parts.parts_max;
            a.stats_ws = st->workspace;
            a.o_ws = st->workspace == nullptr ? nullptr : st->workspace + L.parts.stats_floats;
            a.counters = st->counters;
            L.vt = reinterpret_cast<unsigned short*>(addr(P.slot[MB_AP_S_VT]));
            if (L.vt != nullptr) {
                const int D = P.i[MB_AP_I_HEAD_DIM];
                const int rows = a.batch * a.tokens;
                L.padded_tokens = (a.tokens + kAttnKeys - 1) / kAttnKeys * kAttnKeys;
                if (!make_map(&L.attn_maps.q, addr(P.slot[MB_AP_S_Q]), rows, a.heads * D, kTcRows) ||
                    !make_map(&L.attn_maps.k, addr(P.slot[MB_AP_S_K]), a.batch * a.kv_rows, a.kv_heads * D,
                              kAttnKeys) ||
                    !make_map(&L.attn_maps.vt, addr(P.slot[MB_AP_S_VT]), a.batch * a.kv_heads * D,
                              L.padded_tokens, D))
                    return MB_ERR_CUDA;
            }
        }
    }
    return MB_OK;
}

namespace {

// One phase's kernel; `chained`: launched with programmatic stream serialization, so that it
// may start while its predecessor drains (every kernel of this file blocks in chain_wait()
// before it touches global memory).
template <typename... Params, typename... Args>
cudaError_t launch_phase(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem,
                         cudaStream_t stream, bool chained, Args&&... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = chained ? 1 : 0;
    return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

prefill::TransposeArgs transpose_args(const prefill::PrefillLaunch& L, int head_dim) {
    prefill::TransposeArgs t;
    t.v = L.attn.v;
    t.vt = L.vt;
    t.tokens = L.attn.tokens;
    t.padded = L.padded_tokens;
    t.kv_heads = L.attn.kv_heads;
    t.D = head_dim;
    t.kv_rows = L.attn.kv_rows;
    return t;
}

int transpose_blocks(const prefill::TransposeArgs& t, int batch) {
    return (t.padded / 64) * (t.D / 64) * batch * t.kv_heads;
}

// Whether the kernels of one prefill are chained by programmatic dependent launch.  Measured
// on the gemma-2b shape: a launch boundary between two dependent kernels costs about 5 us on a
// stream (CTA-level stamps of consecutive GEMMs), chaining takes 3-4 % off a step launched
// kernel by kernel at 128 and 512 tokens, and adds 1-2 % to the same step replayed from a CUDA
// graph.  So: on for plain stream launches, off while the stream is being captured;
// MEGABAKE_B200_PREFILL_CHAIN = 0 / 1 forces it (read at every launch, not cached, so that one
// process can run both ways).
bool chaining_enabled(cudaStream_t stream) {
    if (const char* value = std::getenv("MEGABAKE_B200_PREFILL_CHAIN")) return std::atoi(value) != 0;
    cudaStreamCaptureStatus status = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &status) != cudaSuccess) return false;
    return status == cudaStreamCaptureStatusNone;
}

}  // namespace

// Enqueues every phase in order.  Dynamic slots (token ids) are resolved here on the host.
cudaError_t prefill_launch(PrefillState* st, const std::vector<mb_phase>& phases,
                           const std::vector<unsigned long long>& slots, unsigned int n_dynamic,
                           const unsigned long long* dyn, Control* ctl,
                           unsigned long long* trace, cudaStream_t stream) {
    using namespace prefill;
    auto addr = [&](int s) -> unsigned long long {
        if (s < 0) return 0ull;
        return static_cast<unsigned int>(s) < n_dynamic ? dyn[s] : slots[s];
    };
    const bool chain = chaining_enabled(stream);
    bool chained = false;  // the first kernel of an invocation follows foreign work: plain launch
    size_t transposed_by = phases.size() + 1;  // the rotary phase that transposed the values, if any
    cudaError_t err = cudaSuccess;
    for (size_t i = 0; i < phases.size(); ++i) {
        const mb_phase& P = phases[i];
        const PrefillLaunch& L = st->launches[i];
        switch (P.body) {
            case MB_BODY_EMBED_ROWS:
                err = launch_phase(embed_rows_kernel, dim3(P.i[MB_EM_I_ROWS]), dim3(128), 0, stream, chained,
                    reinterpret_cast<const unsigned short*>(addr(P.slot[MB_EM_S_TABLE])),
                    reinterpret_cast<const long long*>(addr(P.slot[MB_EM_S_IDS])),
                    reinterpret_cast<unsigned short*>(addr(P.slot[MB_EM_S_OUT])), P.i[MB_EM_I_ROWS],
                    P.i[MB_EM_I_K], P.i[MB_EM_I_VOCAB], P.f[MB_EM_F_SCALE], ctl, static_cast<int>(i));
                break;
            case MB_BODY_RMSNORM_ROWS:
                if (P.i[MB_RN_I_K] <= 8192) {
                    err = launch_phase(rmsnorm_block_kernel, dim3(P.i[MB_RN_I_ROWS]), dim3(256), 0, stream,
                                       chained,
                                       reinterpret_cast<const unsigned short*>(addr(P.slot[MB_RN_S_X])),
                                       reinterpret_cast<const unsigned short*>(addr(P.slot[MB_RN_S_W])),
                                       reinterpret_cast<unsigned short*>(addr(P.slot[MB_RN_S_OUT])),
                                       P.i[MB_RN_I_K], P.i[MB_RN_I_KIND], P.f[MB_RN_F_EPS]);
                    break;
                }
                err = launch_phase(rmsnorm_rows_kernel, dim3((P.i[MB_RN_I_ROWS] + 3) / 4), dim3(128), 0, stream, chained,
                    reinterpret_cast<const unsigned short*>(addr(P.slot[MB_RN_S_X])),
                    reinterpret_cast<const unsigned short*>(addr(P.slot[MB_RN_S_W])),
                    reinterpret_cast<unsigned short*>(addr(P.slot[MB_RN_S_OUT])), P.i[MB_RN_I_ROWS],
                    P.i[MB_RN_I_K], P.i[MB_RN_I_KIND], P.f[MB_RN_F_EPS]);
                break;
            case MB_BODY_GEMM_TC: {
                const GemmGeometry& g = L.geometry;
                const dim3 grid(g.tiles_m, g.tiles_n, g.split_k);
                GemmArgs args = L.gemm;
                args.trace = trace == nullptr ? nullptr : trace + 8 * i;
                for (int s = 0; s < args.nseg; ++s)  // outputs may be per-launch tensors (logits)
                    args.out[s] = reinterpret_cast<unsigned short*>(addr(P.slot[MB_GV_S_OUT0 + s]));
                if (g.persistent && g.bn == 256)
                    err = launch_phase(gemm_tc_persistent_kernel<256>, dim3(g.grid), dim3(kPersistThreads),
                                       kPersistSmemBytes, stream, chained, L.maps, args);
                else if (g.persistent)
                    err = launch_phase(gemm_tc_persistent_kernel<128>, dim3(g.grid), dim3(kPersistThreads),
                                       kPersistSmemBytes, stream, chained, L.maps, args);
                else if (g.bn == 256)
                    err = launch_phase(gemm_tc_kernel<256>, grid, dim3(kGemmThreads),
                                       gemm_smem_bytes(256, g.stages), stream, chained, L.maps, args);
                else
                    err = launch_phase(gemm_tc_kernel<128>, grid, dim3(kGemmThreads),
                                       gemm_smem_bytes(128, g.stages), stream, chained, L.maps, args);
                break;
            }
            case MB_BODY_ROPE_ROWS: {
                const long long work = static_cast<long long>(P.i[MB_RP_I_ROWS]) *
                                       (P.i[MB_RP_I_HEAD_DIM] / 2);
                long long blocks = (work + 255) / 256;
                if (blocks > 4 * 148 * 8) blocks = 4 * 148 * 8;
                RopeArgs rope;
                rope.q = reinterpret_cast<unsigned short*>(addr(P.slot[MB_RP_S_Q]));
                rope.k = reinterpret_cast<unsigned short*>(addr(P.slot[MB_RP_S_K]));
                rope.pos = reinterpret_cast<const long long*>(addr(P.slot[MB_RP_S_POS]));
                rope.inv_freq = reinterpret_cast<const void*>(addr(P.slot[MB_RP_S_INVFREQ]));
                rope.rows = P.i[MB_RP_I_ROWS];
                rope.heads = P.i[MB_RP_I_HEADS];
                rope.kv_heads = P.i[MB_RP_I_KV_HEADS];
                rope.D = P.i[MB_RP_I_HEAD_DIM];
                rope.invfreq_bf16 = P.i[MB_RP_I_INVFREQ_BF16];
                rope.rope_scale = P.f[MB_RP_F_ROPE_SCALE];
                rope.q_scale = P.f[MB_RP_F_Q_SCALE];
                rope.k_tokens = P.i[MB_RP_I_K_TOKENS];
                rope.k_capacity = P.i[MB_RP_I_K_CAPACITY];
                rope.length = reinterpret_cast<int*>(addr(P.slot[MB_RP_S_LEN]));
                rope.length_value = P.i[MB_RP_I_LEN_VALUE];
                rope.length_count = P.i[MB_RP_I_LEN_COUNT] > 1 ? P.i[MB_RP_I_LEN_COUNT] : 1;
                // the attention phase that follows wants its values transposed: same launch
                const bool with_transpose = i + 1 < phases.size() &&
                                            phases[i + 1].body == MB_BODY_ATTN_PREFILL &&
                                            st->launches[i + 1].vt != nullptr;
                if (with_transpose) {
                    const PrefillLaunch& next = st->launches[i + 1];
                    const TransposeArgs transpose = transpose_args(next, phases[i + 1].i[MB_AP_I_HEAD_DIM]);
                    const int tblocks = transpose_blocks(transpose, next.attn.batch);
                    err = launch_phase(rope_transpose_kernel, dim3(static_cast<int>(blocks) + tblocks),
                                       dim3(256), 0, stream, chained, rope, transpose,
                                       static_cast<int>(blocks));
                    transposed_by = i;
                } else {
                    err = launch_phase(rope_rows_kernel, dim3(static_cast<int>(blocks)), dim3(256), 0,
                                       stream, chained, rope);
                }
                break;
            }
            case MB_BODY_ATTN_PREFILL: {
                const int D = P.i[MB_AP_I_HEAD_DIM];
                if (L.vt != nullptr) {
                    const AttnArgs& a = L.attn;
                    if (transposed_by + 1 != i) {  // not done by the rotary phase just before
                        const TransposeArgs transpose = transpose_args(L, D);
                        err = launch_phase(transpose_values_kernel,
                                           dim3(transpose_blocks(transpose, a.batch)), dim3(256), 0,
                                           stream, chained, transpose);
                        if (err != cudaSuccess) return err;
                        chained = chain;
                    }
                    const dim3 grid(a.heads, L.parts.grid_x, a.batch);
                    const int smem = attention_tc_smem_bytes(D);
                    const int ph = static_cast<int>(i);
                    // keys shared out: the first sweep and the second one as two launches
                    for (int pass = 0; pass < (L.parts.chunk > 0 ? 2 : 1) && err == cudaSuccess; ++pass) {
                        AttnArgs args = a;
                        args.mode = L.parts.chunk == 0 ? kAttnWhole : (pass == 0 ? kAttnStats : kAttnValues);
                        if (D == 64)
                            err = launch_phase(attention_tc_kernel<64>, grid, dim3(kTcThreads), smem, stream,
                                               chained, L.attn_maps, args, ctl, ph);
                        else if (D == 128)
                            err = launch_phase(attention_tc_kernel<128>, grid, dim3(kTcThreads), smem, stream,
                                               chained, L.attn_maps, args, ctl, ph);
                        else
                            err = launch_phase(attention_tc_kernel<256>, grid, dim3(kTcThreads), smem, stream,
                                               chained, L.attn_maps, args, ctl, ph);
                        chained = chain;
                    }
                    break;
                }
                cudaError_t launched = D == 64    ? attn_launch<64>(L.attn, stream)
                                       : D == 128 ? attn_launch<128>(L.attn, stream)
                                                  : attn_launch<256>(L.attn, stream);
                if (launched != cudaSuccess) return launched;
                break;
            }
            default:
                break;
        }
        if (err == cudaSuccess) err = cudaGetLastError();
        if (err != cudaSuccess) return err;
        if (P.body != MB_BODY_NOP) chained = chain;
    }
    return cudaSuccess;
}

}  // namespace mb
