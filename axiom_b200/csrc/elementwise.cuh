// elementwise.cuh — launchers for the stand-alone bias_add / relu / gelu passes.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace axb {

int launch_unary(int op /*0 relu, 1 gelu*/, const float *in, float *out, int64_t n, int sm_count,
                 cudaStream_t st);
int launch_bias_add(const float *in, const float *bias, int axis, float *out, int64_t M, int64_t N,
                    int sm_count, cudaStream_t st);

int launch_head_split(const float *qkv, float *Qh, float *Kh, float *Vh, int64_t rows, int64_t S, int64_t H, int64_t dk,
                      int sm_count, cudaStream_t st);

}  // namespace axb
