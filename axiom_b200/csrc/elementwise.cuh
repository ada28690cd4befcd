// elementwise.cuh — launchers for the stand-alone bias_add / relu / gelu passes and the attention layout passes.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace axb {

int launch_unary(int op /*0 relu, 1 gelu*/, const float *in, float *out, int64_t n, int sm_count,
                 cudaStream_t st);
int launch_fill(float *out, int64_t n, float value, int sm_count, cudaStream_t st);
// axis 0: out[i,j] = in[i,j] + bias[i % period] (period 0 = M); axis 1: + bias[j]
int launch_bias_add(const float *in, const float *bias, int axis, float *out, int64_t M, int64_t N,
                    int sm_count, cudaStream_t st, int64_t period = 0);

// head_layout.cu: rows of dk floats between the flat [B*S, nslot*H*dk] matrix and head-major [B*H, S, dk] buffers.
// to_head: flat -> head[0..nslot) (+ bias[nslot*H*dk] when given; accumulate adds to what head[] holds);
// otherwise head[0..nslot) -> flat.
int launch_head_layout(bool to_head, float *flat, float *const head[3], const float *bias, int nslot, int64_t B,
                       int64_t S, int64_t H, int64_t dk, int sm_count, cudaStream_t st, bool accumulate = false);

}  // namespace axb
