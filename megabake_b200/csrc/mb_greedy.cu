// Greedy pick on the device: the step between two decode launches of a multi-step loop.
//
// The reference picks the next token on the host (`int(logits[0, -1].argmax().item())`,
// examples/single_gpu_generate.py:76) and lists a multi-step decode loop with on-device argmax
// as future work (docs/roadmap.md:180).  With the pick on the device a whole run of decode
// steps can be enqueued -- or captured in one CUDA graph -- without the host ever reading a
// logit: the kernel below writes the chosen id straight into the `input_ids` tensor the next
// decode launch reads, advances `position_ids`, and logs the id.
//
// One CTA of 1,024 threads per batch row, two sweeps over the row (inputs come from L2: the LM
// head wrote them a moment ago).  Sweep 1 finds the row maximum on packed bf16 pairs
// (`__hmax2_nan`: one instruction per two logits, a NaN wins); sweep 2 finds the first index
// that holds it (`__heq2_mask` on pairs, so -0 and +0 count as equal), each thread stopping at
// its own first hit.  Keeping (value, index) in one sweep costs about 14 instructions per
// logit and made the scan issue-bound; the two sweeps cost about 3.  Shuffles and one
// shared-memory step reduce the CTA each time.  Ties go to the lowest index and a NaN beats
// every number, which is what torch.argmax does.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "megabake_b200.h"

namespace mb {
namespace greedy {

constexpr int kThreads = 1024;
constexpr int kWarps = kThreads / 32;
constexpr int kUnroll = 4;  // 16-byte loads in flight per thread: the sweeps are latency bound
constexpr int kNone = 0x7fffffff;

// maximum with a NaN winning over every number
__device__ __forceinline__ float max_nan(float a, float b) {
    return (a != a || b != b) ? __int_as_float(0x7fc00000) : fmaxf(a, b);
}

__device__ __forceinline__ float bf16_bits(unsigned int bits16) {
    return __uint_as_float(bits16 << 16);
}

__device__ __forceinline__ __nv_bfloat162 as_pair(unsigned int word) {
    return *reinterpret_cast<const __nv_bfloat162*>(&word);
}

__device__ __forceinline__ bool hits(float v, float target) {
    return target != target ? v != v : v == target;
}

__global__ void __launch_bounds__(kThreads)
greedy_pick_kernel(const unsigned short* __restrict__ logits, int vocab, long long* ids,
                   long long* positions, long long* out_tokens, int out_capacity, int* cursor) {
    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const unsigned short* x = logits + static_cast<size_t>(row) * vocab;
    __shared__ float warp_max[kWarps];
    __shared__ int warp_first[kWarps];
    __shared__ float row_max;

    // 16-byte body when the row starts on a 16-byte boundary, scalar head/tail otherwise
    const uintptr_t address = reinterpret_cast<uintptr_t>(x);
    int head = static_cast<int>(((16 - (address & 15)) & 15) / 2);
    if (head > vocab) head = vocab;
    const int vectors = (vocab - head) / 8;
    const uint4* body = reinterpret_cast<const uint4*>(x + head);
    const int tail0 = head + 8 * vectors;

    // ---- sweep 1: the maximum
    const unsigned int lowest = 0xff80ff80u;  // (-inf, -inf)
    __nv_bfloat162 best2 = as_pair(lowest);
    for (int v0 = tid; v0 < vectors; v0 += kThreads * kUnroll) {
        uint4 raw[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int v = v0 + u * kThreads;
            raw[u] = v < vectors ? __ldg(body + v) : make_uint4(lowest, lowest, lowest, lowest);
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            best2 = __hmax2_nan(best2, as_pair(raw[u].x));
            best2 = __hmax2_nan(best2, as_pair(raw[u].y));
            best2 = __hmax2_nan(best2, as_pair(raw[u].z));
            best2 = __hmax2_nan(best2, as_pair(raw[u].w));
        }
    }
    float best = max_nan(__bfloat162float(best2.x), __bfloat162float(best2.y));
    for (int i = tid; i < head; i += kThreads) best = max_nan(best, bf16_bits(x[i]));
    for (int i = tail0 + tid; i < vocab; i += kThreads) best = max_nan(best, bf16_bits(x[i]));
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1)
        best = max_nan(best, __shfl_xor_sync(0xffffffffu, best, offset));
    if (lane == 0) warp_max[warp] = best;
    __syncthreads();
    if (warp == 0) {
        float m = warp_max[lane];
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1)
            m = max_nan(m, __shfl_xor_sync(0xffffffffu, m, offset));
        if (lane == 0) row_max = m;
    }
    __syncthreads();
    const float target = row_max;

    // ---- sweep 2: the first index holding it (every thread's indices only grow)
    int first = kNone;
    for (int i = tid; i < head; i += kThreads)
        if (hits(bf16_bits(x[i]), target)) {
            first = i;
            break;
        }
    if (first == kNone) {
        const bool nan_target = target != target;
        const __nv_bfloat16 t16 = __float2bfloat16_rn(target);  // exact: it is one of the logits
        const __nv_bfloat162 target2 = __halves2bfloat162(t16, t16);
        for (int v0 = tid; v0 < vectors && first == kNone; v0 += kThreads * kUnroll) {
            uint4 raw[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const int v = v0 + u * kThreads;
                raw[u] = v < vectors ? __ldg(body + v) : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int u = kUnroll - 1; u >= 0; --u) {  // downwards: the lowest index is assigned last
                const int v = v0 + u * kThreads;
                if (v >= vectors) continue;
                const unsigned int w[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
                if (!nan_target) {
                    unsigned int any = 0;
#pragma unroll
                    for (int q = 0; q < 4; ++q) any |= __heq2_mask(as_pair(w[q]), target2);
                    if (any == 0) continue;
                }
#pragma unroll
                for (int q = 3; q >= 0; --q) {
                    if (hits(bf16_bits(w[q] >> 16), target)) first = head + 8 * v + 2 * q + 1;
                    if (hits(bf16_bits(w[q] & 0xffffu), target)) first = head + 8 * v + 2 * q;
                }
            }
        }
    }
    if (first == kNone)
        for (int i = tail0 + tid; i < vocab; i += kThreads)
            if (hits(bf16_bits(x[i]), target)) {
                first = i;
                break;
            }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1)
        first = min(first, __shfl_xor_sync(0xffffffffu, first, offset));
    if (lane == 0) warp_first[warp] = first;
    __syncthreads();
    if (warp == 0) {
        int f = warp_first[lane];
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1)
            f = min(f, __shfl_xor_sync(0xffffffffu, f, offset));
        if (lane == 0) {
            const long long chosen = f;
            ids[row] = chosen;
            if (positions != nullptr) positions[row] += 1;
            if (out_tokens != nullptr) {
                const int at = cursor[row];
                if (at < out_capacity)
                    out_tokens[static_cast<size_t>(row) * out_capacity + at] = chosen;
                cursor[row] = at + 1;  // keeps counting past the end: the host sees an overrun
            }
        }
    }
}

}  // namespace greedy
}  // namespace mb

extern "C" int mb_greedy_advance(const mb_greedy_args* a, void* stream) {
    if (a == nullptr) return MB_ERR_INVALID;
    if (a->rows < 1 || a->vocab < 1 || a->logits == 0 || a->input_ids == 0) return MB_ERR_INVALID;
    if (a->logits % 2 || a->input_ids % 8 || a->position_ids % 8 || a->out_tokens % 8 ||
        a->cursor % 4)
        return MB_ERR_INVALID;
    if (a->out_tokens != 0 && (a->cursor == 0 || a->out_capacity < 1)) return MB_ERR_INVALID;
    mb::greedy::greedy_pick_kernel<<<a->rows, mb::greedy::kThreads, 0,
                                     static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const unsigned short*>(a->logits), a->vocab,
        reinterpret_cast<long long*>(a->input_ids), reinterpret_cast<long long*>(a->position_ids),
        reinterpret_cast<long long*>(a->out_tokens), a->out_capacity,
        reinterpret_cast<int*>(a->cursor));
    return cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_CUDA;
}
