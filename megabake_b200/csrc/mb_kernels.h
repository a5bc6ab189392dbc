// Host-visible handles of the megakernels (one translation unit per kernel).
#pragma once
#include <cuda_runtime.h>

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
}  // namespace mb
