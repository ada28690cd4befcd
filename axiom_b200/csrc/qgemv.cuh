// qgemv.cuh — W8A32 GEMV for skinny activations (qgemv.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace axb {

// M <= 8, K a multiple of 16 that fits shared memory, q 16-byte aligned
bool qgemv_w8a32_applicable(int64_t M, int64_t N, int64_t K, const void *q);
// out = act(scale[n] * sum_k a*q (+ bias[n])); bias may be null, act 0 none / 1 ReLU / 2 GELU (tanh form)
int launch_qgemv_w8a32(const float *a, const int8_t *q, const float *scales, const float *bias, int act, float *out,
                       int64_t M, int64_t N, int64_t K, int sm_count, cudaStream_t st);

}  // namespace axb
