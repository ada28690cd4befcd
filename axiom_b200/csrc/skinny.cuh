// skinny.cuh — launcher interface of the skinny-M (GEMV) route, see skinny.cu.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace axb {

struct SkinnyArgs {
    const float *X;     // [M,K]
    const float *W;     // [K,N]
    const float *bias;  // [N] or null
    float *Y;           // [M,N]
    int M;
    int64_t N, K;
    float alpha, beta;
    int act;
    int ksplit, kchunk;
    int stages;         // TMA ring depth (skinny_tma.cu)
    int cluster;        // 1: the K-slices of a strip are one thread-block cluster and reduce through shared memory
    float *partial;     // [ksplit][M][N] scratch when ksplit > 1
    int *counters;      // [strips] zero between calls
    int *err;           // device word that receives a code when a bounded wait runs out, or null
    // 1: launch as a programmatic dependent of the kernel before it in the stream.  The TMA-staged kernels request
    // their first ring of WEIGHT tiles before they wait for that kernel to finish (X, bias and Y are only touched
    // afterwards), so the caller sets this only when W cannot be that kernel's output.
    int pdl = 0;
};

struct SkinnyPlan {
    int use_tma;             // 1: TMA-staged kernel (skinny_tma.cu), 0: plain-load kernel (skinny.cu)
    int mt, strips, ksplit, kchunk, stages, cluster;
    int64_t partial_floats;  // scratch the plan needs (0 when K is not split)
    size_t smem_bytes;
};

void skinny_plan(int64_t M, int64_t N, int64_t K, const float *W, int sm_count, SkinnyPlan *plan);
int launch_skinny(const SkinnyArgs &args, const SkinnyPlan &plan, cudaStream_t st);

// TMA-staged variant (skinny_tma.cu)
int skinny_tma_strip_cols(int mt, int cluster);
int skinny_tma_stage_rows(int mt, int cluster);
size_t skinny_tma_smem_bytes(int mt, int kchunk, int stages);
int launch_skinny_tma(const SkinnyArgs &args, const SkinnyPlan &plan, cudaStream_t st);

// Tensor-core variant for 8 < M <= 32 (skinny_tc.cu): needs no scratch; X and W are read in place through TMA
// (N % 4 == 0, K % 4 == 0, 16-byte aligned bases).
bool skinny_tc_applicable(int64_t M, int64_t N, int64_t K, const float *X, const float *W);
int launch_skinny_tc(const SkinnyArgs &args, int sm_count, cudaStream_t st);

}  // namespace axb
