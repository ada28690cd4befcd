// sdpa.cuh — launcher of the fused attention forward (sdpa.cu).  dk <= 128.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace axb {

int launch_sdpa_fwd(const float *Q, const float *K, const float *V, float *O, float *L, int64_t BH,
                    int64_t S, int64_t dk, float scale, int causal, cudaStream_t st);

// Tensor-core route (sdpa_tc.cu): head dim <= 64.  The split pre-pass writes six tf32 planes (Q, K, V as hi/lo)
// into `workspace` (sdpa_tc_workspace_bytes); the attention kernel reads them through TMA.  A bounded wait that
// runs out inside the kernel is reported through *err_word.
bool sdpa_tc_applicable(int64_t BH, int64_t S, int64_t dk, float scale);
size_t sdpa_tc_workspace_bytes(int64_t BH, int64_t S, int64_t dk);
int launch_sdpa_tc_split(const float *Q, const float *K, const float *V, int64_t BH, int64_t S, int64_t dk,
                         void *workspace, int sm_count, cudaStream_t st);
int launch_sdpa_tc(const void *workspace, float *O, float *L, int64_t BH, int64_t S, int64_t dk, float scale,
                   int causal, int *err_word, cudaStream_t st);

}  // namespace axb
