// The C ABI declared in include/megabake_b200.h: plan objects, validation, admission,
// binding and launch.  No torch types cross this boundary; device memory for tensors is the
// caller's, the plan only owns its own small tables (phase records, address table, control
// block).
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include "mb_device.cuh"
#include "mb_kernels.h"

namespace {

thread_local std::string g_last_cuda_error;

int cuda_fail(cudaError_t err, const char* what) {
    g_last_cuda_error = std::string(what) + ": " + cudaGetErrorName(err) + " (" +
                        cudaGetErrorString(err) + ")";
    return MB_ERR_CUDA;
}

#define MB_CUDA(call)                                       \
    do {                                                    \
        cudaError_t err__ = (call);                         \
        if (err__ != cudaSuccess) return cuda_fail(err__, #call); \
    } while (0)

// Makes `device` current for the lifetime of the object and restores the previous one.
struct DeviceGuard {
    int previous = -1;
    bool switched = false;
    cudaError_t error = cudaSuccess;
    explicit DeviceGuard(int device) {
        error = cudaGetDevice(&previous);
        if (error == cudaSuccess && previous != device) {
            error = cudaSetDevice(device);
            switched = error == cudaSuccess;
        }
    }
    ~DeviceGuard() {
        if (switched) cudaSetDevice(previous);
    }
};


}  // namespace

struct mb_plan {
    int device = 0;
    int mode = MB_MODE_DECODE;
    std::vector<mb_phase> phases;
    std::vector<unsigned long long> slots;
    unsigned int n_dynamic = 0;
    unsigned int activation_bytes = 0;
    bool bound = false;
    int sm_count = 0;
    int ctas = 0;
    int threads = 0;
    int smem_bytes = 0;
    int stages = 0;
    int stage_bytes = 0;
    int barriers = 0;
    unsigned int wait_limit_us = 2000000u;
    mb::PhaseEntry* d_entries = nullptr;
    mb::Control* d_ctl = nullptr;
    unsigned long long trace = 0;
    mb::PrefillState* prefill = nullptr;  // MB_MODE_PREFILL plans only
};

namespace {

// Shared-memory scratch the decode attention body carves from the activation region.
long long attention_scratch_bytes(int head_dim, int group, int merge_slots) {
    const long long qs = 8LL * (head_dim + 32) * 2;
    const long long new_rows = 2LL * head_dim * 2;
    const long long cs = 4LL * head_dim;
    const long long stats = 4LL * (2 * 8 * 8 + 8 * 64 + 16);
    const long long states = 4LL * (head_dim + 2) * group * (merge_slots + 2);
    // per-warp K/V tile slots of the split-key loop (64-wide heads): 8 warps x 2 slots x 16 keys
    const long long staging = head_dim == 64 ? 8LL * 2 * 16 * ((head_dim * 2 + 64) + (head_dim * 2 + 16)) : 0;
    return qs + new_rows + cs + stats + states + staging;
}

int check_slot(const mb_plan_desc* d, int s, bool required) {
    if (s < 0) return required ? MB_ERR_INVALID : MB_OK;
    return static_cast<unsigned int>(s) < d->n_slots ? MB_OK : MB_ERR_INVALID;
}

int plan_stage_bytes(const mb_plan_desc* d) {
    return d->stage_bytes == 0 ? mb::decode_stage_bytes() : static_cast<int>(d->stage_bytes);
}

int validate_gemv(const mb_plan_desc* d, const mb_phase& P) {
    const int rows = P.i[MB_GV_I_ROWS], K = P.i[MB_GV_I_K], nseg = P.i[MB_GV_I_NSEG];
    const int nmat = P.i[MB_GV_I_NMAT], rt = P.i[MB_GV_I_ROW_TILE], kc = P.i[MB_GV_I_K_CHUNK];
    const int epi = P.i[MB_GV_I_EPILOGUE], pro = P.i[MB_GV_I_PROLOGUE];
    if (rows < 1 || rows > 8) return MB_ERR_UNSUPPORTED;
    if (K < 32 || K % 32 != 0) return MB_ERR_UNSUPPORTED;
    if (nseg < 1 || nseg > 3) return MB_ERR_INVALID;
    if (nmat != 1 && nmat != 2) return MB_ERR_INVALID;
    if (nmat == 2 && nseg != 1) return MB_ERR_INVALID;
    // a stage holds one 8-row tile, or two: the gate and up tiles of a paired phase, or 16
    // consecutive rows of a plain one
    if (rt != mb::decode_row_tile() && !(nmat == 1 && rt == 2 * mb::decode_row_tile()))
        return MB_ERR_INVALID;
    if (kc < 32 || kc % 32 != 0 || kc > K) return MB_ERR_INVALID;
    if (static_cast<long long>(rt) * nmat * (kc * 2 + mb::decode_row_pad()) > plan_stage_bytes(d))
        return MB_ERR_RESOURCE;
    const int cells = P.i[MB_GV_I_CELLS];
    if (cells & ~(MB_CELLS_X | MB_CELLS_OUT | MB_CELLS_RESIDUAL | MB_CELLS_XSTORE | MB_CELLS_X_WAIT))
        return MB_ERR_INVALID;
    if ((cells & MB_CELLS_X_WAIT) &&
        (P.i[MB_GV_I_X_SOURCE] < 0 || static_cast<unsigned int>(P.i[MB_GV_I_X_SOURCE]) >= d->n_phases))
        return MB_ERR_INVALID;
    if ((cells & MB_CELLS_X) && (P.i[MB_GV_I_GATHER] || K % 4 != 0)) return MB_ERR_INVALID;
    if ((cells & MB_CELLS_X) &&
        (P.i[MB_GV_I_X_SOURCE] < 0 || static_cast<unsigned int>(P.i[MB_GV_I_X_SOURCE]) >= d->n_phases))
        return MB_ERR_INVALID;
    if ((cells & MB_CELLS_RESIDUAL) &&
        (P.i[MB_GV_I_RES_SOURCE] < 0 ||
         static_cast<unsigned int>(P.i[MB_GV_I_RES_SOURCE]) >= d->n_phases))
        return MB_ERR_INVALID;
    // activation rows, plus one staged row of norm weights when the phase normalises
    const long long staged_rows = rows + (P.i[MB_GV_I_PROLOGUE] != MB_PRO_NONE ? 1 : 0);
    if (staged_rows * (K + 32) * 2 > d->activation_bytes) return MB_ERR_RESOURCE;
    if (pro < MB_PRO_NONE || pro > MB_PRO_RMS_GEMMA) return MB_ERR_INVALID;
    if (epi < MB_EPI_NONE || epi > MB_EPI_GELU_TANH_MUL) return MB_ERR_INVALID;
    const bool paired_epi = epi == MB_EPI_SILU_MUL || epi == MB_EPI_GELU_TANH_MUL;
    if (paired_epi != (nmat == 2)) return MB_ERR_INVALID;
    for (int s = 0; s < nseg; ++s) {
        if (P.i[MB_GV_I_N0 + s] < 2) return MB_ERR_INVALID;
        // results are stored as pairs of neighbouring rows (one 4-byte store or one cell)
        if (P.i[MB_GV_I_N0 + s] % 2 != 0) return MB_ERR_UNSUPPORTED;
        if (check_slot(d, P.slot[MB_GV_S_W0 + s], true)) return MB_ERR_INVALID;
        if (check_slot(d, P.slot[MB_GV_S_OUT0 + s], true)) return MB_ERR_INVALID;
        if (check_slot(d, P.slot[MB_GV_S_BIAS0 + s], false)) return MB_ERR_INVALID;
    }
    if (check_slot(d, P.slot[MB_GV_S_X], true)) return MB_ERR_INVALID;
    if (pro != MB_PRO_NONE && check_slot(d, P.slot[MB_GV_S_NORM_W], true)) return MB_ERR_INVALID;
    if (nmat == 2 && check_slot(d, P.slot[MB_GV_S_W_PAIR], true)) return MB_ERR_INVALID;
    if (epi == MB_EPI_RESIDUAL && check_slot(d, P.slot[MB_GV_S_RESIDUAL], true))
        return MB_ERR_INVALID;
    if (P.i[MB_GV_I_GATHER]) {
        if (check_slot(d, P.slot[MB_GV_S_IDS], true)) return MB_ERR_INVALID;
        if (P.i[MB_GV_I_VOCAB] < 1) return MB_ERR_INVALID;
        if (P.i[MB_GV_I_STORE_X] && check_slot(d, P.slot[MB_GV_S_XSTORE], true))
            return MB_ERR_INVALID;
    }
    return MB_OK;
}

int validate_attention(const mb_plan_desc* d, const mb_phase& P) {
    const int B = P.i[MB_AT_I_BATCH], Hq = P.i[MB_AT_I_HEADS], Hkv = P.i[MB_AT_I_KV_HEADS];
    const int D = P.i[MB_AT_I_HEAD_DIM], cap = P.i[MB_AT_I_CAPACITY];
    const int chunks = P.i[MB_AT_I_MAX_CHUNKS], slots = P.i[MB_AT_I_MERGE_SLOTS];
    if (B < 1 || Hq < 1 || Hkv < 1 || cap < 1) return MB_ERR_INVALID;
    if (Hq % Hkv != 0 || Hq / Hkv > 8) return MB_ERR_UNSUPPORTED;
    if (D != 64 && D != 128 && D != 256) return MB_ERR_UNSUPPORTED;
    if (chunks < 1 || chunks > 64) return MB_ERR_INVALID;
    if (slots < 1 || slots > 8) return MB_ERR_INVALID;
    const int exact = P.i[MB_AT_I_EXACT_KEYS];
    if (exact < 0 || exact > 128) return MB_ERR_INVALID;
    if (attention_scratch_bytes(D, Hq / Hkv, slots) > d->activation_bytes)
        return MB_ERR_RESOURCE;
    for (int s = MB_AT_S_Q; s <= MB_AT_S_COUNTER; ++s)
        if (check_slot(d, P.slot[s], true)) return MB_ERR_INVALID;
    const int cells = P.i[MB_AT_I_CELLS];
    if (cells & ~(MB_CELLS_X | MB_CELLS_OUT | MB_CELLS_X_WAIT)) return MB_ERR_INVALID;
    if ((cells & (MB_CELLS_X | MB_CELLS_X_WAIT)) &&
        (P.i[MB_AT_I_QKV_SOURCE] < 0 ||
         static_cast<unsigned int>(P.i[MB_AT_I_QKV_SOURCE]) >= d->n_phases))
        return MB_ERR_INVALID;
    const int lengths = P.i[MB_AT_I_LEN_COUNT];
    if (lengths != 0 && lengths != 1 && lengths != B) return MB_ERR_INVALID;
    return MB_OK;
}

// A prefill plan is a list of kernel launches; it shares the descriptor, the slot table, the
// status word and the entry points with decode plans.
int create_prefill_plan(const mb_plan_desc* desc, mb_plan** out) {
    for (unsigned int i = 0; i < desc->n_phases; ++i) {
        const int rc = mb::prefill_validate(desc->phases[i], desc->n_slots, desc->n_dynamic);
        if (rc != MB_OK) return rc;
    }
    DeviceGuard guard(desc->device);
    if (guard.error != cudaSuccess) return cuda_fail(guard.error, "cudaSetDevice");
    cudaDeviceProp prop;
    MB_CUDA(cudaGetDeviceProperties(&prop, desc->device));
    if (prop.major != 10) {
        g_last_cuda_error = "device is not sm_100 (compute capability " +
                            std::to_string(prop.major) + "." + std::to_string(prop.minor) + ")";
        return MB_ERR_UNSUPPORTED;
    }
    mb_plan* plan = new (std::nothrow) mb_plan();
    if (plan == nullptr) return MB_ERR_RESOURCE;
    plan->device = desc->device;
    plan->mode = desc->mode;
    plan->phases.assign(desc->phases, desc->phases + desc->n_phases);
    plan->slots.assign(desc->n_slots, 0ull);
    plan->n_dynamic = desc->n_dynamic;
    plan->sm_count = prop.multiProcessorCount;
    plan->ctas = prop.multiProcessorCount;
    cudaError_t err = cudaMalloc(&plan->d_ctl, sizeof(mb::Control));
    if (err == cudaSuccess) err = cudaMemset(plan->d_ctl, 0, sizeof(mb::Control));
    if (err == cudaSuccess) err = mb::prefill_create(plan->phases, plan->sm_count, &plan->prefill);
    if (err != cudaSuccess) {
        cuda_fail(err, "prefill plan allocation");
        mb_plan_destroy(plan);
        return MB_ERR_CUDA;
    }
    *out = plan;
    return MB_OK;
}

}  // namespace

extern "C" {

int mb_abi_version(void) { return MB_ABI_VERSION; }

const char* mb_last_cuda_error(void) { return g_last_cuda_error.c_str(); }

const char* mb_strerror(int code) {
    switch (code) {
        case MB_OK: return "ok";
        case MB_ERR_INVALID: return "invalid argument or malformed plan descriptor";
        case MB_ERR_CUDA: return "a CUDA runtime call failed";
        case MB_ERR_UNSUPPORTED: return "body or shape not implemented by the kernels";
        case MB_ERR_RESOURCE: return "shared memory or co-residency admission failed";
        case MB_ERR_UNBOUND: return "plan launched before its static slots were bound";
        case MB_ERR_VERSION: return "plan descriptor ABI version mismatch";
        default: return "unknown error code";
    }
}

const char* mb_status_string(int status_code) {
    switch (status_code) {
        case MB_ST_OK: return "ok";
        case MB_ST_BARRIER_TIMEOUT: return "grid barrier wait timed out";
        case MB_ST_PIPE_TIMEOUT: return "shared-memory pipeline wait timed out";
        case MB_ST_KV_OVERFLOW: return "KV cache is full";
        case MB_ST_TOKEN_RANGE: return "token id outside the embedding table";
        case MB_ST_BAD_PHASE: return "unknown body in the phase table";
        case MB_ST_TMEM: return "tensor memory allocation failed";
        case MB_ST_HANDOFF_TIMEOUT: return "an activation hand-off wait timed out";
        default: return "unknown status";
    }
}

int mb_max_smem_bytes(void) { return 232448; }  // 227 KiB opt-in limit of sm_100

int mb_fixed_smem_bytes(int mode) {
    if (mode == MB_MODE_DECODE) return mb::decode_fixed_smem();
    return -1;
}

int mb_stage_bytes(int mode) {
    if (mode == MB_MODE_DECODE) return mb::decode_stage_bytes();
    return -1;
}

int mb_plan_create(const mb_plan_desc* desc, mb_plan** out) {
    if (desc == nullptr || out == nullptr) return MB_ERR_INVALID;
    *out = nullptr;
    if (desc->abi_version != MB_ABI_VERSION) return MB_ERR_VERSION;
    if (desc->n_phases == 0 || desc->phases == nullptr) return MB_ERR_INVALID;
    if (desc->n_dynamic > MB_MAX_DYNAMIC || desc->n_dynamic > desc->n_slots) return MB_ERR_INVALID;
    if (desc->mode == MB_MODE_PREFILL) return create_prefill_plan(desc, out);
    if (desc->mode != MB_MODE_DECODE) return MB_ERR_UNSUPPORTED;
    if (desc->activation_bytes % 128 != 0) return MB_ERR_INVALID;
    if (desc->stage_bytes % 1024 != 0 ||
        desc->stage_bytes > static_cast<unsigned int>(mb::decode_stage_bytes()))
        return MB_ERR_INVALID;

    int barriers = 1;  // the closing barrier
    for (unsigned int i = 0; i < desc->n_phases; ++i) {
        const mb_phase& P = desc->phases[i];
        int rc = MB_OK;
        switch (P.body) {
            case MB_BODY_NOP: break;
            case MB_BODY_GEMV: rc = validate_gemv(desc, P); break;
            case MB_BODY_ATTN_DECODE: rc = validate_attention(desc, P); break;
            default: rc = MB_ERR_UNSUPPORTED; break;
        }
        if (rc != MB_OK) return rc;
        if (P.flags & MB_FLAG_BARRIER) ++barriers;
    }

    DeviceGuard guard(desc->device);
    if (guard.error != cudaSuccess) return cuda_fail(guard.error, "cudaSetDevice");
    cudaDeviceProp prop;
    MB_CUDA(cudaGetDeviceProperties(&prop, desc->device));
    if (prop.major != 10) {
        g_last_cuda_error = "device is not sm_100 (compute capability " +
                            std::to_string(prop.major) + "." + std::to_string(prop.minor) + ")";
        return MB_ERR_UNSUPPORTED;
    }
    if (!prop.cooperativeLaunch) return MB_ERR_UNSUPPORTED;

    const int fixed = mb::decode_fixed_smem();
    const int stage = plan_stage_bytes(desc);
    const int limit = static_cast<int>(prop.sharedMemPerBlockOptin);
    int stages = (limit - fixed - static_cast<int>(desc->activation_bytes)) / stage;
    if (stages > mb::decode_max_stages()) stages = mb::decode_max_stages();
    if (stages < 2) return MB_ERR_RESOURCE;
    const int smem = fixed + static_cast<int>(desc->activation_bytes) + stages * stage;

    // The attribute belongs to the kernel, not to a plan: set it to the device's opt-in limit so
    // that plans of different sizes (two batch sizes, two models) can be launched in any order.
    MB_CUDA(mb::decode_configure(limit));
    int per_sm = 0;
    MB_CUDA(mb::decode_occupancy(smem, &per_sm));
    if (per_sm < 1) return MB_ERR_RESOURCE;
    int ctas = desc->ctas == 0 ? prop.multiProcessorCount : static_cast<int>(desc->ctas);
    if (ctas < 1 || ctas > prop.multiProcessorCount * per_sm) return MB_ERR_RESOURCE;

    mb_plan* plan = new (std::nothrow) mb_plan();
    if (plan == nullptr) return MB_ERR_RESOURCE;
    plan->device = desc->device;
    plan->mode = desc->mode;
    plan->phases.assign(desc->phases, desc->phases + desc->n_phases);
    for (mb_phase& P : plan->phases) {
        if (P.body != MB_BODY_GEMV) continue;
        // balanced split of the output rows over the CTAs, so the kernel needs no division
        // (in pairs of rows: a lane's two neighbouring results are stored together)
        int total = 0;
        for (int s = 0; s < P.i[MB_GV_I_NSEG]; ++s) total += P.i[MB_GV_I_N0 + s];
        P.i[MB_GV_I_SPLIT_Q] = (total / 2) / ctas;
        P.i[MB_GV_I_SPLIT_R] = (total / 2) % ctas;
    }
    plan->slots.assign(desc->n_slots, 0ull);
    plan->n_dynamic = desc->n_dynamic;
    plan->activation_bytes = desc->activation_bytes;
    plan->sm_count = prop.multiProcessorCount;
    plan->ctas = ctas;
    plan->threads = mb::decode_threads();
    plan->smem_bytes = smem;
    plan->stages = stages;
    plan->stage_bytes = stage;
    plan->barriers = barriers;
    if (desc->wait_limit_ms != 0)
        plan->wait_limit_us = desc->wait_limit_ms > 4000000u ? 4000000000u : desc->wait_limit_ms * 1000u;

    cudaError_t err = cudaMalloc(&plan->d_entries, sizeof(mb::PhaseEntry) * desc->n_phases);
    if (err == cudaSuccess) err = cudaMalloc(&plan->d_ctl, sizeof(mb::Control));
    if (err == cudaSuccess) err = cudaMemset(plan->d_ctl, 0, sizeof(mb::Control));
    if (err != cudaSuccess) {
        cuda_fail(err, "plan table allocation");
        mb_plan_destroy(plan);
        return MB_ERR_CUDA;
    }
    *out = plan;
    return MB_OK;
}

int mb_plan_query(const mb_plan* plan, mb_plan_info* out) {
    if (plan == nullptr || out == nullptr) return MB_ERR_INVALID;
    std::memset(out, 0, sizeof(*out));
    out->ctas = plan->ctas;
    out->threads = plan->threads;
    out->smem_bytes = plan->smem_bytes;
    out->stages = plan->stages;
    out->barriers = plan->barriers;
    out->sm_count = plan->sm_count;
    out->launches = plan->mode == MB_MODE_PREFILL ? mb::prefill_launch_count(plan->prefill) : 1;
    return MB_OK;
}

int mb_plan_bind(mb_plan* plan, const uint64_t* slot_addresses, size_t n) {
    if (plan == nullptr || slot_addresses == nullptr) return MB_ERR_INVALID;
    if (n != plan->slots.size()) return MB_ERR_INVALID;
    for (size_t i = plan->n_dynamic; i < n; ++i) {
        if (slot_addresses[i] == 0 || (slot_addresses[i] & 15ull) != 0) return MB_ERR_INVALID;
        plan->slots[i] = slot_addresses[i];
    }
    if (plan->mode == MB_MODE_PREFILL) {
        DeviceGuard guard(plan->device);
        if (guard.error != cudaSuccess) return cuda_fail(guard.error, "cudaSetDevice");
        const int rc = mb::prefill_bind(plan->prefill, plan->phases, plan->slots, plan->d_ctl);
        if (rc != MB_OK) {
            g_last_cuda_error = "tensor map encoding failed";
            return rc;
        }
        plan->bound = true;
        return MB_OK;
    }
    // Resolve every slot a phase names into its entry, so the kernel reads one record per
    // phase and never a second table.
    std::vector<mb::PhaseEntry> entries(plan->phases.size());
    for (size_t ph = 0; ph < plan->phases.size(); ++ph) {
        entries[ph].rec = plan->phases[ph];
        for (int j = 0; j < MB_PHASE_SLOTS; ++j) {
            const int slot = plan->phases[ph].slot[j];
            if (slot < 0)
                entries[ph].addr[j] = 0ull;
            else if (static_cast<unsigned int>(slot) < plan->n_dynamic)
                entries[ph].addr[j] = mb::kDynamicTag | static_cast<unsigned long long>(slot);
            else
                entries[ph].addr[j] = plan->slots[slot];
        }
    }
    DeviceGuard guard(plan->device);
    if (guard.error != cudaSuccess) return cuda_fail(guard.error, "cudaSetDevice");
    MB_CUDA(cudaMemcpy(plan->d_entries, entries.data(), sizeof(mb::PhaseEntry) * entries.size(),
                       cudaMemcpyHostToDevice));
    plan->bound = true;
    return MB_OK;
}

int mb_plan_launch(mb_plan* plan, const uint64_t* dynamic_addresses, size_t n, void* stream) {
    if (plan == nullptr) return MB_ERR_INVALID;
    if (!plan->bound) return MB_ERR_UNBOUND;
    if (n != plan->n_dynamic || (n > 0 && dynamic_addresses == nullptr)) return MB_ERR_INVALID;
    if (plan->mode == MB_MODE_PREFILL) {
        for (size_t i = 0; i < n; ++i)
            if (dynamic_addresses[i] == 0 || (dynamic_addresses[i] & 7ull) != 0) return MB_ERR_INVALID;
        DeviceGuard guard(plan->device);
        if (guard.error != cudaSuccess) return cuda_fail(guard.error, "cudaSetDevice");
        MB_CUDA(mb::prefill_launch(plan->prefill, plan->phases, plan->slots, plan->n_dynamic,
                                   reinterpret_cast<const unsigned long long*>(dynamic_addresses),
                                   plan->d_ctl, reinterpret_cast<unsigned long long*>(plan->trace),
                                   static_cast<cudaStream_t>(stream)));
        return MB_OK;
    }
    mb::KernelParams params;
    std::memset(&params, 0, sizeof(params));
    params.entries = plan->d_entries;
    params.ctl = plan->d_ctl;
    params.trace = reinterpret_cast<unsigned long long*>(plan->trace);
    for (size_t i = 0; i < n; ++i) {
        if (dynamic_addresses[i] == 0 || (dynamic_addresses[i] & 7ull) != 0) return MB_ERR_INVALID;
        params.dyn[i] = dynamic_addresses[i];
    }
    params.n_phases = static_cast<int>(plan->phases.size());
    params.n_dynamic = static_cast<int>(plan->n_dynamic);
    params.barriers_per_launch = plan->barriers;
    params.stages = plan->stages;
    params.stage_bytes = plan->stage_bytes;
    params.activation_bytes = static_cast<int>(plan->activation_bytes);
    params.wait_limit_us = plan->wait_limit_us;
    DeviceGuard guard(plan->device);
    if (guard.error != cudaSuccess) return cuda_fail(guard.error, "cudaSetDevice");
    MB_CUDA(mb::decode_launch(params, plan->ctas, plan->smem_bytes,
                              static_cast<cudaStream_t>(stream)));
    return MB_OK;
}

int mb_plan_status(mb_plan* plan, mb_status* out) {
    if (plan == nullptr || out == nullptr) return MB_ERR_INVALID;
    DeviceGuard guard(plan->device);
    if (guard.error != cudaSuccess) return cuda_fail(guard.error, "cudaSetDevice");
    mb::Control host;
    MB_CUDA(cudaMemcpy(&host, plan->d_ctl, sizeof(host), cudaMemcpyDeviceToHost));
    out->code = host.status[0];
    out->phase = host.status[1];
    out->detail = host.status[2];
    out->calls = static_cast<int32_t>(host.calls);
    return MB_OK;
}

int mb_plan_set_trace(mb_plan* plan, uint64_t device_address, size_t bytes) {
    if (plan == nullptr) return MB_ERR_INVALID;
    if (device_address != 0) {
        // decode: 8 stamps per CTA and phase; prefill: 8 stamps per phase (CTA 0 of each GEMM)
        const size_t per_phase = plan->mode == MB_MODE_PREFILL ? 1 : static_cast<size_t>(plan->ctas);
        const size_t need = per_phase * plan->phases.size() * 8 * sizeof(uint64_t);
        if (bytes < need || (device_address & 7ull) != 0) return MB_ERR_INVALID;
    }
    plan->trace = device_address;
    return MB_OK;
}

int mb_plan_reset(mb_plan* plan) {
    if (plan == nullptr) return MB_ERR_INVALID;
    DeviceGuard guard(plan->device);
    if (guard.error != cudaSuccess) return cuda_fail(guard.error, "cudaSetDevice");
    MB_CUDA(cudaDeviceSynchronize());
    // Everything starts over except the epoch, which moves on: hand-off cells written by the
    // abandoned launch must never look like cells of the next one.
    unsigned int epoch = 0;
    MB_CUDA(cudaMemcpy(&epoch, &plan->d_ctl->epoch, sizeof(epoch), cudaMemcpyDeviceToHost));
    epoch += 1;
    MB_CUDA(cudaMemset(plan->d_ctl, 0, sizeof(mb::Control)));
    MB_CUDA(cudaMemcpy(&plan->d_ctl->epoch, &epoch, sizeof(epoch), cudaMemcpyHostToDevice));
    return MB_OK;
}

void mb_plan_destroy(mb_plan* plan) {
    if (plan == nullptr) return;
    {
        DeviceGuard guard(plan->device);
        if (plan->d_entries) cudaFree(plan->d_entries);
        if (plan->d_ctl) cudaFree(plan->d_ctl);
        mb::prefill_destroy(plan->prefill);
    }
    delete plan;
}

}  // extern "C"
