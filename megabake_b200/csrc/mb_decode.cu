// Decode megakernel: one cooperative persistent launch runs every phase of a one-token
// decoder step.  Thread layout per CTA (one CTA per SM):
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
#include "mb_device.cuh"
#include "mb_kernels.h"

namespace mb {
namespace decode {

constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 32;
constexpr int kMaxStages = 8;
constexpr int kStageBytes = 34816;  // 32 KiB of weights + room for per-row padding
constexpr int kRowPad = 16;         // bytes added to each staged row (bank spreading)
constexpr int kReduceBytes = 8192;  // two parities of cross-warp partial sums
constexpr int kCtlBytes = 1024;
constexpr int kFixedBytes = kCtlBytes + kReduceBytes;
constexpr int kBarConsumers = 1;    // named barrier ids
constexpr int kBarReduce = 2;

struct SharedCtl {
    unsigned long long full[kMaxStages];
    unsigned long long empty[kMaxStages];
    volatile int abort_flag;
    volatile unsigned int issued;    // stages the producer armed
    volatile unsigned int consumed;  // stages the consumers released
    int bcast[4];                    // small broadcasts (attention chunking, arrival order)
    float red[kConsumerWarps][8];    // per-warp partials of the activation prologue
};
static_assert(sizeof(SharedCtl) <= kCtlBytes, "control block too large");

// Geometry of one GEMV phase for one CTA; producer and consumers derive it identically.
struct GemvGeom {
    int rows, K, nseg, nmat, n[3], ntotal;
    int row_tile, k_chunk, n_chunks, pitch;
    int r0, r1;
};

__device__ __forceinline__ GemvGeom gemv_geometry(const mb_phase* P, int cta, int ctas) {
    GemvGeom g;
    g.rows = P->i[MB_GV_I_ROWS];
    g.K = P->i[MB_GV_I_K];
    g.nseg = P->i[MB_GV_I_NSEG];
    g.nmat = P->i[MB_GV_I_NMAT];
    g.n[0] = P->i[MB_GV_I_N0];
    g.n[1] = g.nseg > 1 ? P->i[MB_GV_I_N0 + 1] : 0;
    g.n[2] = g.nseg > 2 ? P->i[MB_GV_I_N0 + 2] : 0;
    g.ntotal = g.n[0] + g.n[1] + g.n[2];
    g.row_tile = P->i[MB_GV_I_ROW_TILE];
    g.k_chunk = P->i[MB_GV_I_K_CHUNK];
    g.n_chunks = (g.K + g.k_chunk - 1) / g.k_chunk;
    g.pitch = g.k_chunk * 2 + kRowPad;
    g.r0 = static_cast<int>((static_cast<long long>(cta) * g.ntotal) / ctas);
    g.r1 = static_cast<int>((static_cast<long long>(cta + 1) * g.ntotal) / ctas);
    return g;
}

// ---------------------------------------------------------------------------------------
// Producer warp.
// ---------------------------------------------------------------------------------------
__device__ __noinline__ void producer_loop(const KernelParams& p, SharedCtl* sc, char* ring, int lane) {
    const int cta = blockIdx.x, ctas = gridDim.x;
    unsigned int it = 0;
    for (int ph = 0; ph < p.n_phases; ++ph) {
        const mb_phase* P = p.phases + ph;
        if (P->body != MB_BODY_GEMV) continue;
        const GemvGeom g = gemv_geometry(P, cta, ctas);
        const char* wbase[3];
        wbase[0] = reinterpret_cast<const char*>(slot_address(p, P->slot[MB_GV_S_W0]));
        wbase[1] = g.nseg > 1
                       ? reinterpret_cast<const char*>(slot_address(p, P->slot[MB_GV_S_W0 + 1]))
                       : nullptr;
        wbase[2] = g.nseg > 2
                       ? reinterpret_cast<const char*>(slot_address(p, P->slot[MB_GV_S_W0 + 2]))
                       : nullptr;
        const char* wpair =
            g.nmat > 1 ? reinterpret_cast<const char*>(slot_address(p, P->slot[MB_GV_S_W_PAIR]))
                       : nullptr;
        const size_t row_bytes = static_cast<size_t>(g.K) * 2;
        for (int block0 = g.r0; block0 < g.r1; block0 += g.row_tile) {
            const int nrows = min(g.row_tile, g.r1 - block0);
            for (int c = 0; c < g.n_chunks; ++c) {
                const int stage = it % p.stages;
                const unsigned int parity = ((it / p.stages) & 1u) ^ 1u;
                if (!mbar_wait_bounded(&sc->empty[stage], parity, &sc->abort_flag)) {
                    if (lane == 0 && !sc->abort_flag) {
                        record_status(p.ctl, MB_ST_PIPE_TIMEOUT, ph, cta);
                        sc->abort_flag = 1;
                    }
                    return;
                }
                const int kc = min(g.k_chunk, g.K - c * g.k_chunk);
                const unsigned int seg_bytes = static_cast<unsigned int>(kc) * 2u;
                char* dst_stage = ring + static_cast<size_t>(stage) * kStageBytes;
                if (lane == 0) {
                    mbar_arrive_expect_tx(&sc->full[stage], seg_bytes * nrows * g.nmat);
                    sc->issued = it + 1;
                }
                __syncwarp();
                const int copies = nrows * g.nmat;
                for (int idx = lane; idx < copies; idx += 32) {
                    const int m = idx / nrows;
                    const int r = idx - m * nrows;
                    int local = block0 + r;
                    const char* base;
                    if (m == 1) {
                        base = wpair;
                    } else if (local < g.n[0]) {
                        base = wbase[0];
                    } else if (local < g.n[0] + g.n[1]) {
                        base = wbase[1];
                        local -= g.n[0];
                    } else {
                        base = wbase[2];
                        local -= g.n[0] + g.n[1];
                    }
                    const char* src = base + static_cast<size_t>(local) * row_bytes +
                                      static_cast<size_t>(c) * g.k_chunk * 2;
                    char* dst = dst_stage + static_cast<size_t>(m * g.row_tile + r) * g.pitch;
                    bulk_copy_g2s(dst, src, seg_bytes, &sc->full[stage]);
                }
                ++it;
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// Activation prologue: bring the phase's activation rows into shared memory as bf16,
// applying the embedding gather and/or RMSNorm.  All consumer threads.
// xs layout: [rows][K + 8] bf16.
// ---------------------------------------------------------------------------------------
__device__ __noinline__ bool activation_prologue(const KernelParams& p, const mb_phase* P, int ph,
                                    SharedCtl* sc, __nv_bfloat16* xs, int tid) {
    const int rows = P->i[MB_GV_I_ROWS];
    const int K = P->i[MB_GV_I_K];
    const int xpitch = K + 8;
    const int pro = P->i[MB_GV_I_PROLOGUE];
    const bool gather = P->i[MB_GV_I_GATHER] != 0;
    const float embed_scale = P->f[MB_GV_F_EMBED_SCALE];
    const char* xbase = reinterpret_cast<const char*>(slot_address(p, P->slot[MB_GV_S_X]));
    const long long* ids =
        gather ? reinterpret_cast<const long long*>(slot_address(p, P->slot[MB_GV_S_IDS]))
               : nullptr;
    const int warp = tid >> 5, lane = tid & 31;
    const int vec_per_row = K / 8;  // 16-byte vectors

    // Pass 1: copy raw rows (gathered / scaled) into xs and accumulate sums of squares.
    float ss[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) ss[r] = 0.f;
    bool bad_token = false;
#pragma unroll
    for (int r = 0; r < 8; ++r) {
        if (r >= rows) break;
        const char* src;
        if (gather) {
            long long id = ids[r];
            if (id < 0 || id >= P->i[MB_GV_I_VOCAB]) {
                bad_token = true;
                id = 0;
            }
            src = xbase + static_cast<size_t>(id) * K * 2;
        } else {
            src = xbase + static_cast<size_t>(r) * K * 2;
        }
        for (int v = tid; v < vec_per_row; v += kConsumerThreads) {
            uint4 raw = ld_cg_u4(src + static_cast<size_t>(v) * 16);
            unsigned int w[4] = {raw.x, raw.y, raw.z, raw.w};
            if (gather && embed_scale != 0.f) {
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    w[q] = pack_bf16(lo_bf16(w[q]) * embed_scale, hi_bf16(w[q]) * embed_scale);
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                float a = lo_bf16(w[q]), b = hi_bf16(w[q]);
                ss[r] += a * a;
                ss[r] += b * b;
            }
            *reinterpret_cast<uint4*>(xs + static_cast<size_t>(r) * xpitch + v * 8) =
                make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
    if (bad_token && tid == 0) record_status(p.ctl, MB_ST_TOKEN_RANGE, ph, blockIdx.x);

    if (gather && P->i[MB_GV_I_STORE_X] && blockIdx.x == 0) {
        // The residual stream needs the un-normalised rows in global memory.
        named_barrier(kBarConsumers, kConsumerThreads);
        char* store = reinterpret_cast<char*>(slot_address(p, P->slot[MB_GV_S_XSTORE]));
        for (int r = 0; r < rows; ++r)
            for (int v = tid; v < vec_per_row; v += kConsumerThreads)
                *reinterpret_cast<uint4*>(store + (static_cast<size_t>(r) * K + v * 8) * 2) =
                    *reinterpret_cast<const uint4*>(xs + static_cast<size_t>(r) * xpitch + v * 8);
    }

    if (pro == MB_PRO_NONE) {
        named_barrier(kBarConsumers, kConsumerThreads);
        return true;
    }

#pragma unroll
    for (int r = 0; r < 8; ++r) {
        float v = ss[r];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0) sc->red[warp][r] = v;
    }
    named_barrier(kBarConsumers, kConsumerThreads);
    float inv[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) {
        float total = 0.f;
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) total += sc->red[w][r];
        const float mean = total / static_cast<float>(K);
        inv[r] = 1.0f / sqrtf(mean + P->f[MB_GV_F_EPS]);
    }
    const char* nw = reinterpret_cast<const char*>(slot_address(p, P->slot[MB_GV_S_NORM_W]));
    // Pass 2: each thread rescales the vectors it wrote itself (same indices as pass 1).
    for (int v = tid; v < vec_per_row; v += kConsumerThreads) {
        uint4 wraw = __ldg(reinterpret_cast<const uint4*>(nw + static_cast<size_t>(v) * 16));
        const unsigned int wv[4] = {wraw.x, wraw.y, wraw.z, wraw.w};
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            if (r >= rows) break;
            uint4* cell = reinterpret_cast<uint4*>(xs + static_cast<size_t>(r) * xpitch + v * 8);
            uint4 raw = *cell;
            unsigned int xv[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                float a = lo_bf16(xv[q]), b = hi_bf16(xv[q]);
                float wa = lo_bf16(wv[q]), wb = hi_bf16(wv[q]);
                if (pro == MB_PRO_RMS_LLAMA) {
                    a = bf16_round(a * inv[r]) * wa;
                    b = bf16_round(b * inv[r]) * wb;
                } else {
                    a = (a * inv[r]) * (1.0f + wa);
                    b = (b * inv[r]) * (1.0f + wb);
                }
                xv[q] = pack_bf16(a, b);
            }
            *cell = make_uint4(xv[0], xv[1], xv[2], xv[3]);
        }
    }
    named_barrier(kBarConsumers, kConsumerThreads);
    return true;
}

// ---------------------------------------------------------------------------------------
// Consumer side of a GEMV phase.
// ---------------------------------------------------------------------------------------
struct EpilogueCtx {
    const mb_phase* P;
    char* out[3];
    const char* bias[3];
    const char* residual;
    int n[3];
    int rows;
    int epilogue;
};

__device__ __forceinline__ void store_output(const EpilogueCtx& e, int token, int vrow, float acc,
                                             float acc_pair) {
    // Segment lookup without dynamically indexed arrays (those would live in local memory).
    int local = vrow, n = e.n[0];
    char* out = e.out[0];
    const char* bias = e.bias[0];
    if (local >= e.n[0]) {
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
    if (bias != nullptr)
        acc += bf16_bits_to_float(__ldg(reinterpret_cast<const unsigned short*>(bias) + local));
    const float y = bf16_round(acc);
    const size_t index = static_cast<size_t>(token) * n + local;
    float result;
    switch (e.epilogue) {
        case MB_EPI_RESIDUAL: {
            const float res = bf16_bits_to_float(
                ld_cg_u16(reinterpret_cast<const unsigned short*>(e.residual) + index));
            result = res + y;
            break;
        }
        case MB_EPI_SILU_MUL:
            result = bf16_round(silu_f32(y)) * bf16_round(acc_pair);
            break;
        case MB_EPI_GELU_TANH_MUL:
            result = bf16_round(gelu_tanh_f32(y)) * bf16_round(acc_pair);
            break;
        default:
            result = y;
            break;
    }
    reinterpret_cast<unsigned short*>(out)[index] = float_to_bf16_bits(result);
}

template <int NMAT>
__device__ __noinline__ bool gemv_consume(const KernelParams& p, const mb_phase* P, int ph, SharedCtl* sc,
                             const __nv_bfloat16* xs, float* red, const char* ring,
                             unsigned int& it, int tid) {
    const int cta = blockIdx.x, ctas = gridDim.x;
    const GemvGeom g = gemv_geometry(P, cta, ctas);
    const int warp = tid >> 5, lane = tid & 31;
    const int gid = lane >> 2, tq = lane & 3;
    const int row_groups = g.row_tile / 8;
    const int ksplit = kConsumerWarps / row_groups;
    const int rg = warp % row_groups;
    const int ks = warp / row_groups;
    const int xpitch = g.K + 8;
    const __nv_bfloat16* xrow = xs + static_cast<size_t>(min(gid, g.rows - 1)) * xpitch;

    EpilogueCtx e;
    e.P = P;
    e.rows = g.rows;
    e.epilogue = P->i[MB_GV_I_EPILOGUE];
#pragma unroll
    for (int s = 0; s < 3; ++s) {
        e.n[s] = g.n[s];
        e.out[s] = s < g.nseg ? reinterpret_cast<char*>(slot_address(p, P->slot[MB_GV_S_OUT0 + s]))
                              : nullptr;
        e.bias[s] = (s < g.nseg && P->slot[MB_GV_S_BIAS0 + s] >= 0)
                        ? reinterpret_cast<const char*>(slot_address(p, P->slot[MB_GV_S_BIAS0 + s]))
                        : nullptr;
    }
    e.residual = e.epilogue == MB_EPI_RESIDUAL
                     ? reinterpret_cast<const char*>(slot_address(p, P->slot[MB_GV_S_RESIDUAL]))
                     : nullptr;

    int parity_red = 0;
    for (int block0 = g.r0; block0 < g.r1; block0 += g.row_tile) {
        float acc[NMAT][4];
#pragma unroll
        for (int m = 0; m < NMAT; ++m)
#pragma unroll
            for (int q = 0; q < 4; ++q) acc[m][q] = 0.f;

        for (int c = 0; c < g.n_chunks; ++c) {
            const int stage = it % p.stages;
            const unsigned int parity = (it / p.stages) & 1u;
            if (!mbar_wait_bounded(&sc->full[stage], parity, &sc->abort_flag)) {
                if (!sc->abort_flag) {
                    record_status(p.ctl, MB_ST_PIPE_TIMEOUT, ph, cta);
                    sc->abort_flag = 1;
                }
                return false;
            }
            const int kc = min(g.k_chunk, g.K - c * g.k_chunk);
            const char* st = ring + static_cast<size_t>(stage) * kStageBytes;
            const char* wrow = st + static_cast<size_t>(rg * 8 + gid) * g.pitch;
            const __nv_bfloat16* xk = xrow + c * g.k_chunk;
            const int kblocks = kc >> 4;
#pragma unroll 4
            for (int b = ks; b < kblocks; b += ksplit) {
                const unsigned int a0 =
                    *reinterpret_cast<const unsigned int*>(xk + b * 16 + 2 * tq);
                const unsigned int a2 =
                    *reinterpret_cast<const unsigned int*>(xk + b * 16 + 8 + 2 * tq);
#pragma unroll
                for (int m = 0; m < NMAT; ++m) {
                    const char* wm = wrow + static_cast<size_t>(m) * g.row_tile * g.pitch;
                    const unsigned int b0 =
                        *reinterpret_cast<const unsigned int*>(wm + (b * 16 + 2 * tq) * 2);
                    const unsigned int b1 =
                        *reinterpret_cast<const unsigned int*>(wm + (b * 16 + 8 + 2 * tq) * 2);
                    mma_bf16_16816(acc[m], a0, 0u, a2, 0u, b0, b1);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&sc->empty[stage]);
            ++it;
            if (tid == 0) sc->consumed = it;
        }

        // Cross-warp reduction over the k-split, then the epilogue in the ks == 0 warps.
        if (ksplit > 1) {
            float* slab = red + parity_red * (kReduceBytes / 8);
            if (ks > 0) {
                float* cell = slab + ((static_cast<size_t>(ks - 1) * row_groups + rg) * 32 + lane) *
                                         (2 * NMAT);
#pragma unroll
                for (int m = 0; m < NMAT; ++m) {
                    cell[2 * m] = acc[m][0];
                    cell[2 * m + 1] = acc[m][1];
                }
            }
            named_barrier(kBarReduce, kConsumerThreads);
            if (ks == 0) {
                for (int other = 1; other < ksplit; ++other) {
                    const float* cell =
                        slab + ((static_cast<size_t>(other - 1) * row_groups + rg) * 32 + lane) *
                                   (2 * NMAT);
#pragma unroll
                    for (int m = 0; m < NMAT; ++m) {
                        acc[m][0] += cell[2 * m];
                        acc[m][1] += cell[2 * m + 1];
                    }
                }
            }
            parity_red ^= 1;
        }
        if (ks == 0 && gid < g.rows) {
            const int v0 = block0 + rg * 8 + 2 * tq;
            if (v0 < g.r1) store_output(e, gid, v0, acc[0][0], NMAT > 1 ? acc[NMAT - 1][0] : 0.f);
            if (v0 + 1 < g.r1)
                store_output(e, gid, v0 + 1, acc[0][1], NMAT > 1 ? acc[NMAT - 1][1] : 0.f);
        }
    }
    return true;
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
            const int cost = waves * (rounds + 3);
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
//   cs       [D] fp32           cos (first half) and sin (second half), already bf16-rounded
//   merge    [merge_slots][group][D + 2] fp32   per-warp (max, sum, values) states
//   running  [2][group][D + 2] fp32             CTA state, ping-pong over merge rounds
template <int D>
__device__ __noinline__ bool attention_decode(const KernelParams& p, const mb_phase* P, int ph, SharedCtl* sc,
                                 char* scratch, int tid) {
    constexpr int QP = D + 32;  // bf16 pitch of the rotated query rows
    constexpr int DC = D / 32;  // 32-element chunks of the head dimension (QK^T)
    constexpr int DB = D / 64;  // 64-element blocks of the head dimension (PV)
    constexpr int SW = D + 2;   // floats per head state: max, sum, D values
    const int B = P->i[MB_AT_I_BATCH];
    const int Hq = P->i[MB_AT_I_HEADS];
    const int Hkv = P->i[MB_AT_I_KV_HEADS];
    const int cap = P->i[MB_AT_I_CAPACITY];
    const int max_chunks = P->i[MB_AT_I_MAX_CHUNKS];
    const int merge_slots = P->i[MB_AT_I_MERGE_SLOTS];
    const int group = Hq / Hkv;  // query heads per kv head, <= 8
    const float scale = P->f[MB_AT_F_SCALE];
    const float rope_scale = P->f[MB_AT_F_ROPE_SCALE];
    const float q_scale = P->f[MB_AT_F_Q_SCALE];
    const int warp = tid >> 5, lane = tid & 31;
    const int gid = lane >> 2, tq = lane & 3;
    const int cta = blockIdx.x, ctas = gridDim.x;

    const unsigned short* qbuf =
        reinterpret_cast<const unsigned short*>(slot_address(p, P->slot[MB_AT_S_Q]));
    const unsigned short* kbuf =
        reinterpret_cast<const unsigned short*>(slot_address(p, P->slot[MB_AT_S_K]));
    const unsigned short* vbuf =
        reinterpret_cast<const unsigned short*>(slot_address(p, P->slot[MB_AT_S_V]));
    unsigned short* kcache =
        reinterpret_cast<unsigned short*>(slot_address(p, P->slot[MB_AT_S_KCACHE]));
    unsigned short* vcache =
        reinterpret_cast<unsigned short*>(slot_address(p, P->slot[MB_AT_S_VCACHE]));
    const int* lenp = reinterpret_cast<const int*>(slot_address(p, P->slot[MB_AT_S_LEN]));
    const long long* pos =
        reinterpret_cast<const long long*>(slot_address(p, P->slot[MB_AT_S_POS]));
    const void* invf = reinterpret_cast<const void*>(slot_address(p, P->slot[MB_AT_S_INVFREQ]));
    const bool invf_bf16 = P->i[MB_AT_I_INVFREQ_BF16] != 0;
    unsigned short* out = reinterpret_cast<unsigned short*>(slot_address(p, P->slot[MB_AT_S_OUT]));
    float* partial = reinterpret_cast<float*>(slot_address(p, P->slot[MB_AT_S_PARTIAL]));
    int* counter = reinterpret_cast<int*>(slot_address(p, P->slot[MB_AT_S_COUNTER]));

    const int L = __ldcg(lenp);
    if (L < 0 || L + 1 > cap) {
        if (tid == 0) {
            record_status(p.ctl, MB_ST_KV_OVERFLOW, ph, L);
            sc->abort_flag = 1;
        }
        named_barrier(kBarConsumers, kConsumerThreads);
        return false;
    }
    const int nkeys = L + 1;
    const int nblocks = (nkeys + 15) >> 4;
    const int pairs = B * Hkv;
    if (warp == 0) {
        const int nc_pick = choose_chunks(pairs, nblocks, ctas, max_chunks, lane);
        if (lane == 0) sc->bcast[0] = nc_pick;
    }
    named_barrier(kBarConsumers, kConsumerThreads);
    const int nc = sc->bcast[0];
    const int items = pairs * nc;

    __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(scratch);
    float* cs = reinterpret_cast<float*>(scratch + 8 * QP * 2);
    float* merge = cs + D;
    float* running = merge + static_cast<size_t>(merge_slots) * group * SW;
    const size_t key_stride = static_cast<size_t>(Hkv) * D;  // elements between keys

    for (int item = cta; item < items; item += ctas) {
        const int pair = item / nc, chunk = item - pair * nc;
        const int b = pair / Hkv, h = pair - b * Hkv;
        const int blk0 = static_cast<int>((static_cast<long long>(chunk) * nblocks) / nc);
        const int blk1 = static_cast<int>((static_cast<long long>(chunk + 1) * nblocks) / nc);

        // ---- prologue: cos/sin, RoPE of the group's query heads, append of the new key/value
        if (tid < D / 2) {
            const float f =
                invf_bf16 ? bf16_bits_to_float(reinterpret_cast<const unsigned short*>(invf)[tid])
                          : reinterpret_cast<const float*>(invf)[tid];
            const float angle = static_cast<float>(pos[b]) * f;
            cs[tid] = bf16_round(cosf(angle) * rope_scale);
            cs[D / 2 + tid] = bf16_round(sinf(angle) * rope_scale);
        }
        named_barrier(kBarConsumers, kConsumerThreads);
        for (int e = tid; e < group * (D / 2); e += kConsumerThreads) {
            const int gq = e / (D / 2), i = e - gq * (D / 2);
            const unsigned short* qrow = qbuf + (static_cast<size_t>(b) * Hq + h * group + gq) * D;
            const float x1 = bf16_bits_to_float(ld_cg_u16(qrow + i));
            const float x2 = bf16_bits_to_float(ld_cg_u16(qrow + i + D / 2));
            const float c = cs[i], s = cs[D / 2 + i];
            float r1 = bf16_round(bf16_round(x1 * c) + bf16_round(-x2 * s));
            float r2 = bf16_round(bf16_round(x2 * c) + bf16_round(x1 * s));
            if (q_scale != 0.f && q_scale != 1.f) {
                r1 = bf16_round(r1 * q_scale);
                r2 = bf16_round(r2 * q_scale);
            }
            qs[gq * QP + i] = __float2bfloat16_rn(r1);
            qs[gq * QP + i + D / 2] = __float2bfloat16_rn(r2);
        }
        if (chunk == nc - 1) {
            const size_t row = ((static_cast<size_t>(b) * cap + L) * Hkv + h) * D;
            const unsigned short* krow = kbuf + (static_cast<size_t>(b) * Hkv + h) * D;
            const unsigned short* vrow = vbuf + (static_cast<size_t>(b) * Hkv + h) * D;
            for (int i = tid; i < D / 2; i += kConsumerThreads) {
                const float x1 = bf16_bits_to_float(ld_cg_u16(krow + i));
                const float x2 = bf16_bits_to_float(ld_cg_u16(krow + i + D / 2));
                const float c = cs[i], s = cs[D / 2 + i];
                kcache[row + i] = float_to_bf16_bits(bf16_round(x1 * c) + bf16_round(-x2 * s));
                kcache[row + i + D / 2] =
                    float_to_bf16_bits(bf16_round(x2 * c) + bf16_round(x1 * s));
            }
            for (int i = tid; i < D; i += kConsumerThreads) vcache[row + i] = ld_cg_u16(vrow + i);
        }
        named_barrier(kBarConsumers, kConsumerThreads);

        // ---- main loop: each warp owns the 16-key blocks blk0 + warp, + 8, ...
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

        const unsigned short* kc0 = kcache + (static_cast<size_t>(b) * cap * Hkv + h) * D;
        const unsigned short* vc0 = vcache + (static_cast<size_t>(b) * cap * Hkv + h) * D;

        // Register tiles of one 16-key block.  kt[j][i]: key kb + 8j + gid, dims 32i + 8tq..+7.
        // vt[x][q]: key kb + {2tq, 2tq+1, 2tq+8, 2tq+9}[q], dims 64x + 8gid..+7.
        // Keys past the valid length load as zeros (their probabilities are zero as well).
        auto load_keys = [&](int blk, uint4 (&kt)[2][DC]) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int key = (blk << 4) + 8 * j + gid;
                const bool ok = key < nkeys;
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
                const bool ok = key < nkeys;
                const unsigned short* vp =
                    vc0 + static_cast<size_t>(ok ? key : 0) * key_stride + 8 * gid;
#pragma unroll
                for (int x = 0; x < DB; ++x)
                    vt[x][q] = ok ? *reinterpret_cast<const uint4*>(vp + 64 * x)
                                  : make_uint4(0u, 0u, 0u, 0u);
            }
        };
        constexpr bool kPrefetchKeys = D <= 128;
        constexpr bool kPrefetchValues = D <= 64;

        uint4 kt[2][DC], kt_next[2][DC];
        uint4 vt[DB][4], vt_next[DB][4];
        int blk = blk0 + warp;
        if (blk < blk1) {
            if (kPrefetchKeys) load_keys(blk, kt);
            if (kPrefetchValues) load_values(blk, vt);
        }
        for (; blk < blk1; blk += kConsumerWarps) {
            const int kb = blk << 4;
            const int following = blk + kConsumerWarps;
            if (!kPrefetchKeys) load_keys(blk, kt);
            if (!kPrefetchValues) load_values(blk, vt);
            if (following < blk1) {
                if (kPrefetchKeys) load_keys(following, kt_next);
                if (kPrefetchValues) load_values(following, vt_next);
            }
            float sc_[2][4];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                sc_[j][0] = sc_[j][1] = sc_[j][2] = sc_[j][3] = 0.f;
#pragma unroll
                for (int i = 0; i < DC; ++i) {
                    mma_bf16_16816(sc_[j], qf[i].x, 0u, qf[i].y, 0u, kt[j][i].x, kt[j][i].y);
                    mma_bf16_16816(sc_[j], qf[i].z, 0u, qf[i].w, 0u, kt[j][i].z, kt[j][i].w);
                }
            }
            // bf16-rounded score, fp32 scale, key mask; sv[2j+q] <-> key kb + 8j + 2tq + q
            float sv[4];
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    const int key = kb + 8 * j + 2 * tq + q;
                    const float s = bf16_round(sc_[j][q]) * scale;
                    sv[2 * j + q] = key < nkeys ? s : -INFINITY;
                }
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
            const unsigned int pb0 = pack_bf16(pv[0], pv[1]);  // keys 2tq, 2tq+1 of head gid
            const unsigned int pb1 = pack_bf16(pv[2], pv[3]);  // keys 8+2tq, 9+2tq
            // rescale factors of the two heads this lane accumulates (columns 2tq, 2tq+1)
            const float alpha0 = __shfl_sync(0xffffffffu, alpha, (2 * tq) * 4);
            const float alpha1 = __shfl_sync(0xffffffffu, alpha, (2 * tq + 1) * 4);
#pragma unroll
            for (int x = 0; x < DB; ++x) {
                const unsigned int ra[4] = {vt[x][0].x, vt[x][0].y, vt[x][0].z, vt[x][0].w};
                const unsigned int rb[4] = {vt[x][1].x, vt[x][1].y, vt[x][1].z, vt[x][1].w};
                const unsigned int rc[4] = {vt[x][2].x, vt[x][2].y, vt[x][2].z, vt[x][2].w};
                const unsigned int rd[4] = {vt[x][3].x, vt[x][3].y, vt[x][3].z, vt[x][3].w};
#pragma unroll
                for (int mt = 0; mt < 4; ++mt) {
                    acc[x][mt][0] *= alpha0;
                    acc[x][mt][1] *= alpha1;
                    acc[x][mt][2] *= alpha0;
                    acc[x][mt][3] *= alpha1;
                    const unsigned int a0 = __byte_perm(ra[mt], rb[mt], 0x5410u);
                    const unsigned int a1 = __byte_perm(ra[mt], rb[mt], 0x7632u);
                    const unsigned int a2 = __byte_perm(rc[mt], rd[mt], 0x5410u);
                    const unsigned int a3 = __byte_perm(rc[mt], rd[mt], 0x7632u);
                    mma_bf16_16816(acc[x][mt], a0, a1, a2, a3, pb0, pb1);
                }
            }
            if (following < blk1) {
                if (kPrefetchKeys) {
#pragma unroll
                    for (int j = 0; j < 2; ++j)
#pragma unroll
                        for (int i = 0; i < DC; ++i) kt[j][i] = kt_next[j][i];
                }
                if (kPrefetchValues) {
#pragma unroll
                    for (int x = 0; x < DB; ++x)
#pragma unroll
                        for (int q = 0; q < 4; ++q) vt[x][q] = vt_next[x][q];
                }
            }
        }
        l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
        l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);

        // ---- merge the warp states into one CTA state, `merge_slots` warps per round
        const int rounds = (kConsumerWarps + merge_slots - 1) / merge_slots;
        for (int round = 0; round < rounds; ++round) {
            const int first = round * merge_slots;
            if (warp >= first && warp < first + merge_slots) {
                float* base = merge + static_cast<size_t>(warp - first) * group * SW;
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
            const int live = min(merge_slots, kConsumerWarps - first);
            const float* prev = running + static_cast<size_t>((round & 1) ^ 1) * group * SW;
            float* next = running + static_cast<size_t>(round & 1) * group * SW;
            for (int e = tid; e < group * SW; e += kConsumerThreads) {
                const int gq = e / SW, col = e - gq * SW;
                float mx = round == 0 ? -INFINITY : prev[gq * SW];
                for (int s = 0; s < live; ++s)
                    mx = fmaxf(mx, merge[(static_cast<size_t>(s) * group + gq) * SW]);
                float sum_l = 0.f, sum_v = 0.f;
                if (round > 0) {
                    const float w = expf(prev[gq * SW] - mx);
                    sum_l = prev[gq * SW + 1] * w;
                    sum_v = prev[gq * SW + col] * w;
                }
                for (int s = 0; s < live; ++s) {
                    const float* st = merge + (static_cast<size_t>(s) * group + gq) * SW;
                    const float w = expf(st[0] - mx);  // 0 for a warp that saw no block
                    sum_l += st[1] * w;
                    sum_v += st[col] * w;
                }
                next[e] = col == 0 ? mx : (col == 1 ? sum_l : sum_v);
            }
            named_barrier(kBarConsumers, kConsumerThreads);
        }
        const float* state = running + static_cast<size_t>((rounds - 1) & 1) * group * SW;

        if (nc == 1) {
            for (int e = tid; e < group * D; e += kConsumerThreads) {
                const int gq = e / D, d = e - gq * D;
                const float v = state[gq * SW + 2 + d] / state[gq * SW + 1];
                out[(static_cast<size_t>(b) * Hq + h * group + gq) * D + d] = float_to_bf16_bits(v);
            }
        } else {
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
            if (sc->bcast[1] == nc - 1) {
                // last chunk of this (row, kv head) to arrive: fold all chunks in chunk order
                const float* all = partial + static_cast<size_t>(pair) * max_chunks * group * SW;
                for (int e = tid; e < group * D; e += kConsumerThreads) {
                    const int gq = e / D, d = e - gq * D;
                    float mx = -INFINITY;
                    for (int c = 0; c < nc; ++c)
                        mx = fmaxf(mx, ld_cg_f32(all + (static_cast<size_t>(c) * group + gq) * SW));
                    float sum_l = 0.f, sum_v = 0.f;
                    for (int c = 0; c < nc; ++c) {
                        const float* st = all + (static_cast<size_t>(c) * group + gq) * SW;
                        const float w = expf(ld_cg_f32(st) - mx);
                        sum_l += ld_cg_f32(st + 1) * w;
                        sum_v += ld_cg_f32(st + 2 + d) * w;
                    }
                    out[(static_cast<size_t>(b) * Hq + h * group + gq) * D + d] =
                        float_to_bf16_bits(sum_v / sum_l);
                }
                if (tid == 0) counter[pair] = 0;  // ready for the next launch
            }
        }
        named_barrier(kBarConsumers, kConsumerThreads);  // scratch is reused by the next item
    }
    return true;
}

// ---------------------------------------------------------------------------------------
// The kernel.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads, 1) decode_kernel(const __grid_constant__ KernelParams p) {
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
        sc->abort_flag = peek_status(p.ctl) != 0 ? 1 : 0;  // a faulted plan runs nothing
        sc->issued = 0;
        sc->consumed = 0;
        mbar_init_fence();
    }
    __syncthreads();
    if (sc->abort_flag) return;

    if (tid >= kConsumerThreads) {
        producer_loop(p, sc, ring, tid & 31);
    } else {
        const unsigned int calls = *reinterpret_cast<volatile unsigned int*>(&p.ctl->calls);
        const unsigned int base =
            calls * static_cast<unsigned int>(p.barriers_per_launch) * gridDim.x;
        unsigned int it = 0;
        int barrier_index = 0;
        bool ok = true;
        for (int ph = 0; ph < p.n_phases && ok; ++ph) {
            const mb_phase* P = p.phases + ph;
            switch (P->body) {
                case MB_BODY_NOP:
                    break;
                case MB_BODY_GEMV:
                    activation_prologue(p, P, ph, sc, reinterpret_cast<__nv_bfloat16*>(act), tid);
                    if (P->i[MB_GV_I_NMAT] == 2)
                        ok = gemv_consume<2>(p, P, ph, sc,
                                             reinterpret_cast<const __nv_bfloat16*>(act), red, ring,
                                             it, tid);
                    else
                        ok = gemv_consume<1>(p, P, ph, sc,
                                             reinterpret_cast<const __nv_bfloat16*>(act), red, ring,
                                             it, tid);
                    break;
                case MB_BODY_ATTN_DECODE: {
                    const int D = P->i[MB_AT_I_HEAD_DIM];
                    if (D == 64)
                        ok = attention_decode<64>(p, P, ph, sc, act, tid);
                    else if (D == 128)
                        ok = attention_decode<128>(p, P, ph, sc, act, tid);
                    else
                        ok = attention_decode<256>(p, P, ph, sc, act, tid);
                    break;
                }
                default:
                    if (tid == 0) {
                        record_status(p.ctl, MB_ST_BAD_PHASE, ph, P->body);
                        sc->abort_flag = 1;
                    }
                    ok = false;
                    break;
            }
            if (!ok) break;
            if (P->flags & MB_FLAG_BARRIER) {
                ++barrier_index;
                ok = grid_barrier(p.ctl, base + barrier_index * gridDim.x, kBarConsumers,
                                  kConsumerThreads, tid, &sc->abort_flag, ph);
                if (ok && (P->flags & MB_FLAG_BUMP_LENGTH) && blockIdx.x == 0 && tid == 0) {
                    int* lenp = reinterpret_cast<int*>(slot_address(p, P->slot[MB_AT_S_LEN]));
                    *lenp = *lenp + 1;
                }
            }
        }
        if (ok) {
            // Closing barrier: nobody may still read `calls` when CTA 0 advances it.
            ++barrier_index;
            ok = grid_barrier(p.ctl, base + barrier_index * gridDim.x, kBarConsumers,
                              kConsumerThreads, tid, &sc->abort_flag, p.n_phases);
            if (ok && blockIdx.x == 0 && tid == 0) p.ctl->calls = calls + 1;
        }
    }

    // Drain: never leave while one of this CTA's bulk copies is still in flight.
    __syncthreads();
    if (sc->abort_flag && tid == 0) {
        const unsigned int issued = sc->issued, consumed = sc->consumed;
        for (unsigned int s = consumed; s < issued; ++s) {
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
