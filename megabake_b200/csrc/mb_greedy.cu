// Greedy pick on the device: the step between two decode launches of a multi-step loop.
//
// The reference picks the next token on the host (`int(logits[0, -1].argmax().item())`,
// examples/single_gpu_generate.py:76) and lists a multi-step decode loop with on-device argmax
// as future work (docs/roadmap.md:180).  With the pick on the device a whole run of decode
// steps can be enqueued -- or captured in one CUDA graph -- without the host ever reading a
// logit: the kernel below writes the chosen id straight into the `input_ids` tensor the next
// decode launch reads, advances `position_ids`, and logs the id.
//
// One CTA of 1,024 threads per batch row.  Each thread scans a strided share of the row's logits
// with 16-byte loads, four in flight (inputs come from L2: the LM head wrote them a moment ago,
// and the scan is bound by that latency), keeping (value, first index of that value);
// shuffles and one shared-memory step reduce the CTA.  Ties go to the lowest index and a NaN
// beats every number, which is what torch.argmax does.
#include <cuda_runtime.h>

#include <cstdint>

#include "megabake_b200.h"

namespace mb {
namespace greedy {

constexpr int kThreads = 1024;
constexpr int kUnroll = 4;  // 16-byte loads in flight per thread: the scan is L2-latency bound

struct Pick {
    float value;
    int index;
};

// true when candidate (v, i) should replace (best, bi)
__device__ __forceinline__ bool beats(float v, int i, float best, int bi) {
    const bool v_nan = v != v, b_nan = best != best;
    if (v_nan || b_nan) return v_nan && (!b_nan || i < bi);
    return v > best || (v == best && i < bi);
}

__device__ __forceinline__ float bf16_bits(unsigned int bits16) {
    return __uint_as_float(bits16 << 16);
}

__global__ void __launch_bounds__(kThreads)
greedy_pick_kernel(const unsigned short* __restrict__ logits, int vocab, long long* ids,
                   long long* positions, long long* out_tokens, int out_capacity, int* cursor) {
    const int row = blockIdx.x, tid = threadIdx.x;
    const unsigned short* x = logits + static_cast<size_t>(row) * vocab;
    Pick mine = {-INFINITY, 0x7fffffff};

    // 16-byte body when the row starts on a 16-byte boundary, scalar head/tail otherwise
    const uintptr_t address = reinterpret_cast<uintptr_t>(x);
    int head = static_cast<int>(((16 - (address & 15)) & 15) / 2);
    if (head > vocab) head = vocab;
    const int vectors = (vocab - head) / 8;
    const uint4* body = reinterpret_cast<const uint4*>(x + head);
    for (int v0 = tid; v0 < vectors; v0 += kThreads * kUnroll) {
        uint4 raw[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int v = v0 + u * kThreads;
            raw[u] = v < vectors ? __ldg(body + v) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int v = v0 + u * kThreads;
            if (v >= vectors) break;
            const unsigned int w[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
            const int base = head + 8 * v;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float lo = bf16_bits(w[q] & 0xffffu), hi = bf16_bits(w[q] >> 16);
                if (beats(lo, base + 2 * q, mine.value, mine.index)) mine = {lo, base + 2 * q};
                if (beats(hi, base + 2 * q + 1, mine.value, mine.index))
                    mine = {hi, base + 2 * q + 1};
            }
        }
    }
    for (int i = tid; i < head; i += kThreads) {
        const float v = bf16_bits(x[i]);
        if (beats(v, i, mine.value, mine.index)) mine = {v, i};
    }
    for (int i = head + 8 * vectors + tid; i < vocab; i += kThreads) {
        const float v = bf16_bits(x[i]);
        if (beats(v, i, mine.value, mine.index)) mine = {v, i};
    }

#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, mine.value, offset);
        const int oi = __shfl_xor_sync(0xffffffffu, mine.index, offset);
        if (beats(ov, oi, mine.value, mine.index)) mine = {ov, oi};
    }
    __shared__ Pick warp_best[kThreads / 32];
    if ((tid & 31) == 0) warp_best[tid >> 5] = mine;
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < kThreads / 32; ++w)
            if (beats(warp_best[w].value, warp_best[w].index, mine.value, mine.index))
                mine = warp_best[w];
        const long long chosen = mine.index;
        ids[row] = chosen;
        if (positions != nullptr) positions[row] += 1;
        if (out_tokens != nullptr) {
            const int at = cursor[row];
            if (at < out_capacity) out_tokens[static_cast<size_t>(row) * out_capacity + at] = chosen;
            cursor[row] = at + 1;  // keeps counting past the end: the host sees an overrun
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
