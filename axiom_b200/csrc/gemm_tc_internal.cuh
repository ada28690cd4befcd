// gemm_tc_internal.cuh — definitions shared by the two tcgen05 GEMM kernels
// (gemm_tc.cu: one CTA per tile; gemm_tc2.cu: a CTA pair per tile).
#pragma once
#include "gemm_tc.cuh"
#include "ptx.cuh"

#include <cuda.h>

namespace axb {

static constexpr int BM = 128;
static constexpr int GROUP_M = 16;
static constexpr int NUM_THREADS = 352;  // A-producer warp, MMA warp, 8 epilogue warps, B-producer warp
static constexpr int B_PRODUCER_WARP = 10;
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
    uint32_t prod_a, prod_b;  // plane index of product i in bits [4i, 4i+4): registers, never indexed memory
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
    float *c_extra[TC_MAX_EXTRA];
    int n_extra;
    int hs_dk, hs_S, hs_H;   // head-major scatter of the output (hs_dk > 0), see TcEpilogue
    float *hs_out[3];
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

// where the 32 output columns starting at col0 of output row `row` go
__device__ __forceinline__ float *out_piece_ptr(const KernelArgs &p, long long row, int col0)
{
    if (p.hs_dk == 0) return reinterpret_cast<float *>(p.C) + row * p.ldc + col0;
    const int D = p.hs_H * p.hs_dk;
    const int which = col0 / D, rem = col0 - which * D, h = rem / p.hs_dk, d0 = rem - h * p.hs_dk;
    const long long b = row / p.hs_S, s = row - b * p.hs_S;
    return p.hs_out[which] + ((b * p.hs_H + h) * p.hs_S + s) * p.hs_dk + d0;
}

__device__ __forceinline__ float gelu_tanh(float v)
{
    const float inner = 0.7978845608028654f * (v + 0.044715f * v * v * v);
    return 0.5f * v * (1.0f + tanhf(inner));
}


// All MMAs of one pipeline stage, fully unrolled.  tcgen05.mma holds the issuing thread while
// the tensor pipe is busy and the pipe queues next to nothing, so every scalar instruction
// between two MMAs is time the pipe idles: descriptors are one OR and one ADD away from
// registers, the product list is a bitfield, there are no loops, divisions or memory accesses.
template <int KIND, int SWB, int NPROD, bool PAIR, int A_BYTES, int B_BYTES>
__device__ __forceinline__ void issue_stage_mmas(uint32_t d_tmem, uint32_t sa, uint32_t sb, uint32_t prod_a,
                                                 uint32_t prod_b, uint64_t desc_hi, uint32_t idesc, bool first)
{
    constexpr int KSTEPS = SWB / 32;
#pragma unroll
    for (int pr = 0; pr < NPROD; ++pr) {
        const uint32_t ia = (prod_a >> (4 * pr)) & 15u, ib = (prod_b >> (4 * pr)) & 15u;
        const uint64_t da = desc_hi | (uint64_t)((sa + ia * A_BYTES) >> 4);
        const uint64_t db = desc_hi | (uint64_t)((sb + ib * B_BYTES) >> 4);
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            const uint32_t accumulate = (pr == 0 && ks == 0) ? (first ? 0u : 1u) : 1u;
            if constexpr (PAIR) tc_mma_pair<KIND>(d_tmem, da + 2u * ks, db + 2u * ks, idesc, accumulate);
            else tc_mma<KIND>(d_tmem, da + 2u * ks, db + 2u * ks, idesc, accumulate);
        }
    }
}

// gemm_tc2.cu: the CTA-pair kernel (256 x 256 tiles; ka.m_tiles counts 256-row tiles, the B maps have 128-row boxes)
int launch_gemm_tc_pair(int kind, int swb, int nprod, const TmapPack &tm, KernelArgs &ka, int npa, int npb, int sm_count,
                        cudaStream_t stream, char *err, size_t err_len);

}  // namespace axb
