// sdpa_bwd.cu — backward of scaled-dot-product attention in fp32 (slot sdpa_bwd of ax_cuda_extension_t,
// include/axiom/internal/cuda_extension.h:96-100; CPU path src/compute/backends/cpu_opt.c:9112-9180; the
// reference CUDA path, cuda/ops_attention.cu:443-590, materialises P and dP as two BH*S*S buffers):
//     P  = exp(scale*Q.K^T - L)            (L = row log-sum-exp from the forward; masked entries 0)
//     dV = P^T.dO      dP = dO.V^T      D_i = dO_i . O_i
//     dS = P o (dP - D) * scale          dQ = dS.K      dK = dS^T.Q
// Nothing of size S x S is stored: scores are recomputed from Q, K and L block by block.  Two kernels so that
// every output has exactly one writer and a fixed summation order (no atomics, bitwise repeatable):
//   sdpa_bwd_dq_kernel  — one CTA per 64 query rows, sweeps the key blocks, accumulates dQ;
//   sdpa_bwd_dkv_kernel — one CTA per 64 key rows, sweeps the query blocks, accumulates dK and dV.
// Both run on the fp32 FMA pipe from shared-memory tiles (4x4 register micro-tiles), like the fp32 forward
// kernel in sdpa.cu; dQ, dK and dV are overwritten, as both reference implementations do.
#include "sdpa.cuh"

#include <math.h>
#include <stdint.h>

namespace axb {

static constexpr int BB = 64, BW_THREADS = 256, PP = BB + 4;

// rows r0.. of a [S, dk] matrix -> dst[64][DKP] (zero fill past S and dk)
template <int DKP>
__device__ __forceinline__ void bw_load_rows(float *dst, const float *Xh, int r0, int S, int dk, bool vec, int tid)
{
    for (int i = tid; i < BB * (DKP / 4); i += BW_THREADS) {
        const int r = i / (DKP / 4), c = (i - r * (DKP / 4)) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r0 + r < S) {
            const float *src = Xh + (int64_t)(r0 + r) * dk + c;
            if (vec && c + 4 <= dk) v = __ldg(reinterpret_cast<const float4 *>(src));
            else {
                if (c + 0 < dk) v.x = __ldg(src + 0);
                if (c + 1 < dk) v.y = __ldg(src + 1);
                if (c + 2 < dk) v.z = __ldg(src + 2);
                if (c + 3 < dk) v.w = __ldg(src + 3);
            }
        }
        *reinterpret_cast<float4 *>(dst + r * DKP + c) = v;
    }
}

// the same rows transposed -> dst[DKP][64]
template <int DKP>
__device__ __forceinline__ void bw_load_rows_t(float *dst, const float *Xh, int r0, int S, int dk, bool vec, int tid)
{
    for (int i = tid; i < BB * (DKP / 4); i += BW_THREADS) {
        const int j = i % BB, c = (i / BB) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r0 + j < S) {
            const float *src = Xh + (int64_t)(r0 + j) * dk + c;
            if (vec && c + 4 <= dk) v = __ldg(reinterpret_cast<const float4 *>(src));
            else {
                if (c + 0 < dk) v.x = __ldg(src + 0);
                if (c + 1 < dk) v.y = __ldg(src + 1);
                if (c + 2 < dk) v.z = __ldg(src + 2);
                if (c + 3 < dk) v.w = __ldg(src + 3);
            }
        }
        dst[(c + 0) * BB + j] = v.x;
        dst[(c + 1) * BB + j] = v.y;
        dst[(c + 2) * BB + j] = v.z;
        dst[(c + 3) * BB + j] = v.w;
    }
}

// s[a][b] = sum_d A[ty*4+a][d] * Bt[d][tx*4+b]     (A: [64][DKP], Bt: [DKP][64])
template <int DKP>
__device__ __forceinline__ void bw_mm_nt(const float *A, const float *Bt, int ty, int tx, float (&s)[4][4])
{
#pragma unroll
    for (int a = 0; a < 4; ++a) s[a][0] = s[a][1] = s[a][2] = s[a][3] = 0.f;
#pragma unroll 4
    for (int d = 0; d < DKP; d += 4) {
        float4 q[4], k[4];
#pragma unroll
        for (int a = 0; a < 4; ++a) q[a] = *reinterpret_cast<const float4 *>(A + (ty * 4 + a) * DKP + d);
#pragma unroll
        for (int e = 0; e < 4; ++e) k[e] = *reinterpret_cast<const float4 *>(Bt + (d + e) * BB + tx * 4);
#pragma unroll
        for (int a = 0; a < 4; ++a) {
            const float qa[4] = { q[a].x, q[a].y, q[a].z, q[a].w };
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                s[a][0] = fmaf(qa[e], k[e].x, s[a][0]);
                s[a][1] = fmaf(qa[e], k[e].y, s[a][1]);
                s[a][2] = fmaf(qa[e], k[e].z, s[a][2]);
                s[a][3] = fmaf(qa[e], k[e].w, s[a][3]);
            }
        }
    }
}

// o[a][cg*4+e] += sum_j P[ty*4+a][j] * B[j][cg*64 + tx*4 + e]     (P: [64][PP], B: [64][DKP])
template <int DKP>
__device__ __forceinline__ void bw_mm_acc(const float *P, const float *B, int ty, int tx, float (&o)[4][DKP / 16])
{
    constexpr int NCG = DKP / 64;
#pragma unroll 2
    for (int j = 0; j < BB; j += 4) {
        float4 p[4];
#pragma unroll
        for (int a = 0; a < 4; ++a) p[a] = *reinterpret_cast<const float4 *>(P + (ty * 4 + a) * PP + j);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
#pragma unroll
            for (int cg = 0; cg < NCG; ++cg) {
                const float4 v = *reinterpret_cast<const float4 *>(B + (j + e) * DKP + cg * 64 + tx * 4);
#pragma unroll
                for (int a = 0; a < 4; ++a) {
                    const float pe = e == 0 ? p[a].x : e == 1 ? p[a].y : e == 2 ? p[a].z : p[a].w;
                    o[a][cg * 4 + 0] = fmaf(pe, v.x, o[a][cg * 4 + 0]);
                    o[a][cg * 4 + 1] = fmaf(pe, v.y, o[a][cg * 4 + 1]);
                    o[a][cg * 4 + 2] = fmaf(pe, v.z, o[a][cg * 4 + 2]);
                    o[a][cg * 4 + 3] = fmaf(pe, v.w, o[a][cg * 4 + 3]);
                }
            }
        }
    }
}

// rows r0 + ty*4 + a of a [S, dk] output <- o[a][*]
template <int DKP>
__device__ __forceinline__ void bw_store(float *Xh, int r0, int S, int dk, bool vec, int ty, int tx, const float (&o)[4][DKP / 16])
{
    constexpr int NCG = DKP / 64;
#pragma unroll
    for (int a = 0; a < 4; ++a) {
        const int r = r0 + ty * 4 + a;
        if (r >= S) continue;
        float *dst = Xh + (int64_t)r * dk;
#pragma unroll
        for (int cg = 0; cg < NCG; ++cg) {
            const int c = cg * 64 + tx * 4;
            if (vec && c + 4 <= dk) {
                *reinterpret_cast<float4 *>(dst + c) = make_float4(o[a][cg * 4 + 0], o[a][cg * 4 + 1], o[a][cg * 4 + 2], o[a][cg * 4 + 3]);
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (c + e < dk) dst[c + e] = o[a][cg * 4 + e];
            }
        }
    }
}

// D[h, i] = dO[h, i, :] . O[h, i, :]; one warp per row
__global__ void __launch_bounds__(256) sdpa_bwd_rowdot_kernel(const float *__restrict__ O, const float *__restrict__ dO,
                                                              float *__restrict__ D, int64_t rows, int dk)
{
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t r = warp; r < rows; r += nwarps) {
        float s = 0.f;
        for (int d = lane; d < dk; d += 32) s = fmaf(__ldg(dO + r * dk + d), __ldg(O + r * dk + d), s);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
        if (lane == 0) D[r] = s;
    }
}

template <int DKP>
__global__ void __launch_bounds__(BW_THREADS) sdpa_bwd_dq_kernel(const float *__restrict__ Q, const float *__restrict__ K,
                                                                 const float *__restrict__ V, const float *__restrict__ dO,
                                                                 const float *__restrict__ L, const float *__restrict__ D,
                                                                 float *__restrict__ dQ, int S, int dk, float scale,
                                                                 int causal, int vec)
{
    extern __shared__ __align__(16) float sm[];
    float *Qs = sm;                    // [64][DKP]
    float *dOs = Qs + BB * DKP;        // [64][DKP]
    float *Kt = dOs + BB * DKP;        // [DKP][64]
    float *Vt = Kt + DKP * BB;         // [DKP][64]
    float *Ks = Vt + DKP * BB;         // [64][DKP]
    float *dSs = Ks + BB * DKP;        // [64][PP]

    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int qb = (int)gridDim.x - 1 - (int)blockIdx.x;   // longest causal rows first
    const int64_t head = blockIdx.y;
    const int64_t hoff = head * (int64_t)S * dk;
    const int q0 = qb * BB;
    bw_load_rows<DKP>(Qs, Q + hoff, q0, S, dk, vec, tid);
    bw_load_rows<DKP>(dOs, dO + hoff, q0, S, dk, vec, tid);
    float Li[4], Di[4];
#pragma unroll
    for (int a = 0; a < 4; ++a) {
        const int gi = q0 + ty * 4 + a;
        Li[a] = gi < S ? __ldg(L + head * S + gi) : 0.f;
        Di[a] = gi < S ? __ldg(D + head * S + gi) : 0.f;
    }
    float dq[4][DKP / 16];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int c = 0; c < DKP / 16; ++c) dq[a][c] = 0.f;

    const int nkb = causal ? (qb + 1) : (S + BB - 1) / BB;
    for (int kb = 0; kb < nkb; ++kb) {
        const int k0 = kb * BB;
        __syncthreads();   // the previous block's tiles are consumed
        bw_load_rows_t<DKP>(Kt, K + hoff, k0, S, dk, vec, tid);
        bw_load_rows_t<DKP>(Vt, V + hoff, k0, S, dk, vec, tid);
        bw_load_rows<DKP>(Ks, K + hoff, k0, S, dk, vec, tid);
        __syncthreads();
        float s[4][4], dp[4][4];
        bw_mm_nt<DKP>(Qs, Kt, ty, tx, s);
        bw_mm_nt<DKP>(dOs, Vt, ty, tx, dp);
#pragma unroll
        for (int a = 0; a < 4; ++a) {
            const int gi = q0 + ty * 4 + a;
            float ds[4];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const int gj = k0 + tx * 4 + b;
                const bool dead = gi >= S || gj >= S || (causal && gj > gi);
                const float p = dead ? 0.f : expf(fmaf(s[a][b], scale, -Li[a]));
                ds[b] = p * (dp[a][b] - Di[a]) * scale;
            }
            *reinterpret_cast<float4 *>(dSs + (ty * 4 + a) * PP + tx * 4) = make_float4(ds[0], ds[1], ds[2], ds[3]);
        }
        __syncthreads();
        bw_mm_acc<DKP>(dSs, Ks, ty, tx, dq);
    }
    bw_store<DKP>(dQ + hoff, q0, S, dk, vec, ty, tx, dq);
}

template <int DKP>
__global__ void __launch_bounds__(BW_THREADS) sdpa_bwd_dkv_kernel(const float *__restrict__ Q, const float *__restrict__ K,
                                                                  const float *__restrict__ V, const float *__restrict__ dO,
                                                                  const float *__restrict__ L, const float *__restrict__ D,
                                                                  float *__restrict__ dK, float *__restrict__ dV, int S, int dk,
                                                                  float scale, int causal, int vec)
{
    extern __shared__ __align__(16) float sm[];
    float *Kt = sm;                    // [DKP][64]
    float *Vt = Kt + DKP * BB;         // [DKP][64]
    float *Qs = Vt + DKP * BB;         // [64][DKP]
    float *dOs = Qs + BB * DKP;        // [64][DKP]
    float *Pt = dOs + BB * DKP;        // [64 keys][PP]  P transposed
    float *dSt = Pt + BB * PP;         // [64 keys][PP]  dS transposed

    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int kb = blockIdx.x;         // early key blocks see the most query blocks under the causal mask: first
    const int64_t head = blockIdx.y;
    const int64_t hoff = head * (int64_t)S * dk;
    const int k0 = kb * BB;
    bw_load_rows_t<DKP>(Kt, K + hoff, k0, S, dk, vec, tid);
    bw_load_rows_t<DKP>(Vt, V + hoff, k0, S, dk, vec, tid);
    float dkacc[4][DKP / 16], dvacc[4][DKP / 16];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int c = 0; c < DKP / 16; ++c) dkacc[a][c] = dvacc[a][c] = 0.f;

    const int nqb = (S + BB - 1) / BB;
    for (int qb = causal ? kb : 0; qb < nqb; ++qb) {
        const int q0 = qb * BB;
        __syncthreads();
        bw_load_rows<DKP>(Qs, Q + hoff, q0, S, dk, vec, tid);
        bw_load_rows<DKP>(dOs, dO + hoff, q0, S, dk, vec, tid);
        __syncthreads();
        float s[4][4], dp[4][4];
        bw_mm_nt<DKP>(Qs, Kt, ty, tx, s);      // rows: queries (ty), columns: keys (tx)
        bw_mm_nt<DKP>(dOs, Vt, ty, tx, dp);
        float pt[4][4], dst[4][4];             // [key b][query a]
#pragma unroll
        for (int a = 0; a < 4; ++a) {
            const int gi = q0 + ty * 4 + a;
            const float Li = gi < S ? __ldg(L + head * S + gi) : 0.f;
            const float Di = gi < S ? __ldg(D + head * S + gi) : 0.f;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const int gj = k0 + tx * 4 + b;
                const bool dead = gi >= S || gj >= S || (causal && gj > gi);
                const float p = dead ? 0.f : expf(fmaf(s[a][b], scale, -Li));
                pt[b][a] = p;
                dst[b][a] = p * (dp[a][b] - Di) * scale;
            }
        }
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            *reinterpret_cast<float4 *>(Pt + (tx * 4 + b) * PP + ty * 4) = make_float4(pt[b][0], pt[b][1], pt[b][2], pt[b][3]);
            *reinterpret_cast<float4 *>(dSt + (tx * 4 + b) * PP + ty * 4) = make_float4(dst[b][0], dst[b][1], dst[b][2], dst[b][3]);
        }
        __syncthreads();
        bw_mm_acc<DKP>(Pt, dOs, ty, tx, dvacc);    // dV[key][d] += sum_query P[query][key] * dO[query][d]
        bw_mm_acc<DKP>(dSt, Qs, ty, tx, dkacc);    // dK[key][d] += sum_query dS[query][key] * Q[query][d]
    }
    bw_store<DKP>(dK + hoff, k0, S, dk, vec, ty, tx, dkacc);
    bw_store<DKP>(dV + hoff, k0, S, dk, vec, ty, tx, dvacc);
}

size_t sdpa_bwd_workspace_bytes(int64_t BH, int64_t S) { return (size_t)BH * S * sizeof(float); }

template <int DKP>
static int launch_bwd(const float *Q, const float *K, const float *V, const float *dO, const float *L, const float *D,
                      float *dQ, float *dK, float *dV, int64_t BH, int64_t S, int64_t dk, float scale, int causal, int vec,
                      cudaStream_t st)
{
    const size_t smem_q = (size_t)(5 * BB * DKP + BB * PP) * 4, smem_kv = (size_t)(4 * BB * DKP + 2 * BB * PP) * 4;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(sdpa_bwd_dq_kernel<DKP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_q);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(sdpa_bwd_dkv_kernel<DKP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_kv);
        if (e != cudaSuccess) return (int)e;
        attr_set[dev] = true;
    }
    dim3 grid((unsigned)((S + BB - 1) / BB), (unsigned)BH);
    sdpa_bwd_dq_kernel<DKP><<<grid, BW_THREADS, smem_q, st>>>(Q, K, V, dO, L, D, dQ, (int)S, (int)dk, scale, causal, vec);
    sdpa_bwd_dkv_kernel<DKP><<<grid, BW_THREADS, smem_kv, st>>>(Q, K, V, dO, L, D, dK, dV, (int)S, (int)dk, scale, causal, vec);
    return (int)cudaGetLastError();
}

int launch_sdpa_bwd(const float *Q, const float *K, const float *V, const float *O, const float *dO, const float *L,
                    float *dQ, float *dK, float *dV, int64_t BH, int64_t S, int64_t dk, float scale, int causal,
                    float *workspace, int sm_count, int *err_word, cudaStream_t st, int *launches)
{
    if (launches) *launches = 0;
    if (BH <= 0 || S <= 0) return 0;
    const int64_t rows = BH * S;
    int64_t blocks = (rows + 7) / 8;
    if (blocks > (int64_t)sm_count * 8) blocks = (int64_t)sm_count * 8;
    sdpa_bwd_rowdot_kernel<<<(unsigned)blocks, 256, 0, st>>>(O, dO, workspace, rows, (int)dk);
    int e = (int)cudaGetLastError();
    if (e) return e;
    if (sdpa_bwd_tc_applicable(Q, K, V, dO, BH, S, dk, scale)) {
        if (launches) *launches = 4;
        return launch_sdpa_bwd_tc(Q, K, V, dO, L, workspace, dQ, dK, dV, BH, S, dk, scale, causal, err_word, st);
    }
    if (launches) *launches = 3;
    const uintptr_t align = reinterpret_cast<uintptr_t>(Q) | reinterpret_cast<uintptr_t>(K) | reinterpret_cast<uintptr_t>(V) |
                            reinterpret_cast<uintptr_t>(dO) | reinterpret_cast<uintptr_t>(dQ) | reinterpret_cast<uintptr_t>(dK) |
                            reinterpret_cast<uintptr_t>(dV);
    const int vec = (dk % 4 == 0) && ((align & 15) == 0);
    return dk <= 64 ? launch_bwd<64>(Q, K, V, dO, L, workspace, dQ, dK, dV, BH, S, dk, scale, causal, vec, st)
                    : launch_bwd<128>(Q, K, V, dO, L, workspace, dQ, dK, dV, BH, S, dk, scale, causal, vec, st);
}

}  // namespace axb
