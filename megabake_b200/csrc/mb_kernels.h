// Host-visible handles of the megakernels (one translation unit per kernel).
#pragma once
#include <cuda_runtime.h>

#include <vector>

#include "../../include/megabake_b200.h"

namespace mb {
struct KernelParams;

int decode_threads();
int decode_fixed_smem();
int decode_stage_bytes();
int decode_max_stages();
int decode_row_pad();
int decode_row_tile();
cudaError_t decode_configure(int smem_bytes);
cudaError_t decode_occupancy(int smem_bytes, int* blocks_per_sm);
cudaError_t decode_launch(const KernelParams& params, int ctas, int smem_bytes,
                          cudaStream_t stream);

// Prefill plans (mb_prefill.cu): one kernel launch per phase.
struct PrefillState;
struct Control;
int prefill_validate(const mb_phase& phase, unsigned int n_slots, unsigned int n_dynamic);
cudaError_t prefill_create(std::vector<mb_phase>& phases, int sm_count, PrefillState** out);
int prefill_launch_count(const PrefillState* state);  // kernels one prefill_launch enqueues
void prefill_destroy(PrefillState* state);
int prefill_bind(PrefillState* state, const std::vector<mb_phase>& phases,
                 const std::vector<unsigned long long>& slots, Control* ctl);
cudaError_t prefill_launch(PrefillState* state, const std::vector<mb_phase>& phases,
                           const std::vector<unsigned long long>& slots, unsigned int n_dynamic,
                           const unsigned long long* dynamic_addresses, Control* ctl,
                           unsigned long long* trace, cudaStream_t stream);
}  // namespace mb
