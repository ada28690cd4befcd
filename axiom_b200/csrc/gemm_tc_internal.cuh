// gemm_tc_internal.cuh — definitions shared by the two tcgen05 GEMM kernels
// (gemm_tc.cu: one CTA per tile; gemm_tc2.cu: a CTA pair per tile).
#pragma once
#include "gemm_tc.cuh"
#include "ptx.cuh"

#include <cuda.h>

namespace axb {

static constexpr int BM = 128;
static constexpr int GROUP_M = 16;
static constexpr int NUM_THREADS = 320;  // producer warp, MMA warp, 8 epilogue warps
static constexpr int HEADER_BYTES = 1024;
static constexpr int MAX_STAGES = 8;
static constexpr int SMEM_BUDGET = 227 * 1024;

struct alignas(64) TmapPack {
    CUtensorMap a[TC_MAX_PLANES];
    CUtensorMap b[TC_MAX_PLANES];
};

struct KernelArgs {
    int M, N, K;
    int npa, npb, nprod;
    int8_t pa[TC_MAX_PRODUCTS], pb[TC_MAX_PRODUCTS];
    int m_tiles, n_tiles, k_blocks, stages;
    int chunk_kb;  // k-blocks accumulated in TMEM before the epilogue warps drain them
    float alpha, beta;
    const float *bias;
    const float *colscale;
    int act, out_mode;
    void *C;
    int32_t *acc_out;
    long long ldc;
    int *err;
};

// error words written to *err (first writer wins)
enum { ERR_PRODUCER_WAIT = 1, ERR_MMA_WAIT_FULL = 2, ERR_MMA_WAIT_TMEM = 3, ERR_EPI_WAIT = 4 };

__device__ __forceinline__ void report(int *err, int code)
{
    if (err) atomicCAS(err, 0, code);
}

__device__ __forceinline__ void tile_coords(int t, int m_tiles, int n_tiles, int &mt, int &nt)
{
    const int per_group = GROUP_M * n_tiles;
    const int g = t / per_group;
    const int first_m = g * GROUP_M;
    const int gm = min(GROUP_M, m_tiles - first_m);
    const int r = t - g * per_group;
    mt = first_m + r % gm;
    nt = r / gm;
}

__device__ __forceinline__ float gelu_tanh(float v)
{
    const float inner = 0.7978845608028654f * (v + 0.044715f * v * v * v);
    return 0.5f * v * (1.0f + tanhf(inner));
}

// gemm_tc2.cu: the CTA-pair kernel (256 x 256 tiles; ka.m_tiles counts 256-row tiles, the B maps have 128-row boxes)
int launch_gemm_tc_pair(int kind, int swb, const TmapPack &tm, KernelArgs &ka, int npa, int npb, int sm_count,
                        cudaStream_t stream, char *err, size_t err_len);

}  // namespace axb
