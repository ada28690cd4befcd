// sdpa.cuh — launcher of the fused attention forward (sdpa.cu).  dk <= 128.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace axb {

int launch_sdpa_fwd(const float *Q, const float *K, const float *V, float *O, float *L, int64_t BH,
                    int64_t S, int64_t dk, float scale, int causal, cudaStream_t st);

// P[BH,S,S] = exp(scale*Q.K^T - L), 0 above the diagonal when causal (the probabilities a caller may ask to keep).
int launch_sdpa_probs(const float *Q, const float *K, const float *L, float *P, int64_t BH, int64_t S, int64_t dk,
                      float scale, int causal, cudaStream_t st);

// Backward (sdpa_bwd.cu): dQ, dK, dV are overwritten; workspace holds BH*S floats (sdpa_bwd_workspace_bytes).
size_t sdpa_bwd_workspace_bytes(int64_t BH, int64_t S);
// Head dims <= 64 (multiples of 4, 16-byte aligned tensors, S >= 128, scale > 0) run on the tensor cores
// (sdpa_bwd_tc.cu), the rest on the fp32 FMA kernels.  *launches receives the number of kernels enqueued.
int launch_sdpa_bwd(const float *Q, const float *K, const float *V, const float *O, const float *dO, const float *L,
                    float *dQ, float *dK, float *dV, int64_t BH, int64_t S, int64_t dk, float scale, int causal,
                    float *workspace, int sm_count, int *err_word, cudaStream_t st, int *launches);
bool sdpa_bwd_tc_applicable(const float *Q, const float *K, const float *V, const float *dO, int64_t BH, int64_t S, int64_t dk,
                            float scale);
// D = rowsum(dO o O) [BH][S] must have been computed; one kernel in three roles (dQ, dK, dV)
int launch_sdpa_bwd_tc(const float *Q, const float *K, const float *V, const float *dO, const float *L, const float *D,
                       float *dQ, float *dK, float *dV, int64_t BH, int64_t S, int64_t dk, float scale, int causal,
                       int *err_word, cudaStream_t st);

// Tensor-core route (sdpa_tc.cu): head dim <= 64 and a multiple of 4, 16-byte aligned tensors, scale > 0.
// Reads the caller's tensors through TMA and splits them inside the kernel: no pre-pass, no scratch.  A bounded
// wait that runs out inside the kernel is reported through *err_word.
bool sdpa_tc_applicable(const float *Q, const float *K, const float *V, int64_t BH, int64_t S, int64_t dk,
                        float scale);
int launch_sdpa_tc(const float *Q, const float *K, const float *V, float *O, float *L, int64_t BH, int64_t S,
                   int64_t dk, float scale, int causal, int *err_word, cudaStream_t st);

}  // namespace axb
