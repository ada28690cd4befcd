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
// M <= 4: ONE launch — the tensor-core kernel makes the digits itself; it releases its own dependents early, and is
// launched as a programmatic dependent when `pdl` says the kernel before it did not write these weights (it requests
// its first weight tiles before that kernel has finished; everything else waits).  M > 4: two launches on `st`, the
// digit pre-pass and the tensor-core kernel, which requests its first weight tiles while the pre-pass runs.  `err` receives a code if a wait in the kernel runs out.
int launch_qskinny_tc(const float *a, const int8_t *q, const float *scales, const float *bias, int act, float *out,
                      int64_t M, int64_t N, int64_t K, void *workspace, int *err, int sm_count, cudaStream_t st, int pdl);

// M > 64: the same digit planes as an operand of one int8 GEMM.  launch_qx_digits writes digits[4][plane_rows][K]
// (row m of plane j at (j * plane_rows + m) * K; plane_rows == 0: interleaved, digit j of row m at (4 * m + j) * K)
// and 2^-s per row.  The interleaved form is the B operand of the int8 GEMM core, whose epilogue recombines the four
// digit sums of every output (OUT_DIGITS_T).
int launch_qx_digits(const float *a, int64_t M, int64_t K, int64_t plane_rows, int8_t *digits, float *inv_s,
                     cudaStream_t st);

#ifdef __CUDACC__
// Exact integer sum of digit products -> fp32 result: total * 2^-s * scale (+ bias) -> activation.  |total| < 2^47 is cut
// into a signed head and 24 low bits, which convert with 32-bit instructions.
__device__ __forceinline__ float qt_finish(long long total, float inv_s, float scale, float bias, int act)
{
    const float head = (float)(int)(total >> 24);
    const float tail = (float)(int)((unsigned)total & 0xFFFFFFu);
    float v = fmaf(head, 16777216.0f, tail) * scale * inv_s + bias;
    if (act == 1) v = fmaxf(v, 0.0f);
    else if (act == 2) v = 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
    return v;
}
#endif

}  // namespace axb
