// qskinny_tc.cuh — W8A32 for skinny activations (M <= 64) on the integer tensor cores (qskinny_tc.cu).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace axb {

// 1 <= M <= 64, K a multiple of 16 in [128, 65536], activations and weights 16-byte aligned
bool qskinny_tc_applicable(int64_t M, int64_t N, int64_t K, const float *a, const int8_t *q);
// bytes of device scratch one call needs (digit planes of the activations + one scale per row)
size_t qskinny_tc_workspace_bytes(int64_t M, int64_t K);
// out = act(scale[n] * sum_k a*q (+ bias[n])); bias may be null, act 0 none / 1 ReLU / 2 GELU (tanh form).
// Two launches on `st`: the digit pre-pass and the tensor-core kernel, which is launched as a programmatic dependent
// and requests its first weight tiles while the pre-pass runs.  `err` receives a code if a wait in the kernel runs out.
int launch_qskinny_tc(const float *a, const int8_t *q, const float *scales, const float *bias, int act, float *out,
                      int64_t M, int64_t N, int64_t K, void *workspace, int *err, int sm_count, cudaStream_t st);

// M > 64: the same digit planes as the A operand of one int8 GEMM.  launch_qx_digits writes digits[4][plane_rows][K]
// (row m of plane j at (j * plane_rows + m) * K) and 2^-s per row; launch_qx_combine turns the s32 result
// [4 * M, N] of digits x weights^T into out[M, N] with the per-column scale, bias and activation.
int launch_qx_digits(const float *a, int64_t M, int64_t K, int64_t plane_rows, int8_t *digits, float *inv_s,
                     cudaStream_t st);
int launch_qx_combine(const int32_t *acc, const float *inv_s, const float *scales, const float *bias, int act, float *out,
                      int64_t M, int64_t N, int sm_count, cudaStream_t st);

}  // namespace axb
