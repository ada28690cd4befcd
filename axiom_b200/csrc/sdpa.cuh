// sdpa.cuh — launcher of the fused attention forward (sdpa.cu).  dk <= 128.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace axb {

int launch_sdpa_fwd(const float *Q, const float *K, const float *V, float *O, float *L, int64_t BH,
                    int64_t S, int64_t dk, float scale, int causal, cudaStream_t st);

}  // namespace axb
