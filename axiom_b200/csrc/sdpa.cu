// sdpa.cu — fused scaled-dot-product attention forward in fp32:
//     O = softmax(scale * Q.K^T [+ causal mask]) . V,   L = rowmax + log(rowsum)
// on head-major [BH,S,dk] buffers.  One CTA owns 64 query rows of one head and
// sweeps the keys in blocks of 64 with the online-softmax recurrence, so the
// S x S score matrix is never written to memory (the reference CUDA path
// materialises it: BH*S*S floats).  Both contractions run on the fp32 FMA pipe
// from shared-memory tiles (4x4 register micro-tiles, 128-bit shared loads);
// causal blocks above the diagonal are skipped.  Results match an fp32
// restatement to ~1e-6, which the bf16 tensor-core route cannot do without
// operand splitting.
#include "sdpa.cuh"
#include "errors.cuh"

#include <math.h>
#include <stdint.h>

namespace axb {

static constexpr int BQ = 64, BKV = 64, SD_THREADS = 256;
static constexpr int PS_PITCH = BKV + 4;

template <int DKP>
__global__ void __launch_bounds__(SD_THREADS) sdpa_fwd_kernel(const float *__restrict__ Q,
                                                              const float *__restrict__ K,
                                                              const float *__restrict__ V,
                                                              float *__restrict__ O, float *__restrict__ L,
                                                              int S, int dk, float scale, int causal)
{
    constexpr int NCG = DKP / 64;  // column groups of 64: thread owns cols cg*64 + tx*4 .. +3
    extern __shared__ __align__(16) float sm[];
    float *Qs = sm;                       // [BQ][DKP]
    float *Kt = Qs + BQ * DKP;            // [DKP][BKV]   (transposed)
    float *Vs = Kt + DKP * BKV;           // [BKV][DKP]
    float *Ps = Vs + BKV * DKP;           // [BQ][PS_PITCH]

    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int qb = (int)gridDim.x - 1 - (int)blockIdx.x;  // longest causal rows first
    const int64_t head = blockIdx.y;
    const float *Qh = Q + head * (int64_t)S * dk;
    const float *Kh = K + head * (int64_t)S * dk;
    const float *Vh = V + head * (int64_t)S * dk;
    const int q0 = qb * BQ;
    // 128-bit accesses need rows that are multiples of 16 bytes on 16-byte aligned bases
    const bool vec = (dk % 4 == 0) && (((reinterpret_cast<uintptr_t>(Q) | reinterpret_cast<uintptr_t>(K) |
                                         reinterpret_cast<uintptr_t>(V) | reinterpret_cast<uintptr_t>(O)) & 15) == 0);

    // Q block -> shared (rows past S and columns past dk are zero)
    for (int i = tid; i < BQ * (DKP / 4); i += SD_THREADS) {
        const int r = i / (DKP / 4), c = (i - r * (DKP / 4)) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (q0 + r < S) {
            const float *src = Qh + (int64_t)(q0 + r) * dk + c;
            if (vec && c + 4 <= dk) v = __ldg(reinterpret_cast<const float4 *>(src));
            else {
                if (c + 0 < dk) v.x = __ldg(src + 0);
                if (c + 1 < dk) v.y = __ldg(src + 1);
                if (c + 2 < dk) v.z = __ldg(src + 2);
                if (c + 3 < dk) v.w = __ldg(src + 3);
            }
        }
        *reinterpret_cast<float4 *>(Qs + r * DKP + c) = v;
    }

    float o[4][NCG * 4];
    float m_run[4], l_run[4];
#pragma unroll
    for (int a = 0; a < 4; ++a) {
        m_run[a] = -INFINITY;
        l_run[a] = 0.f;
#pragma unroll
        for (int c = 0; c < NCG * 4; ++c) o[a][c] = 0.f;
    }

    const int nkb = causal ? (qb + 1) : (S + BKV - 1) / BKV;
    for (int kb = 0; kb < nkb; ++kb) {
        const int k0 = kb * BKV;
        __syncthreads();  // previous block's Kt / Vs / Ps fully consumed
        // K block -> Kt (lanes along the key index: conflict-free transposed stores)
        for (int i = tid; i < BKV * (DKP / 4); i += SD_THREADS) {
            const int j = i % BKV, c = (i / BKV) * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (k0 + j < S) {
                const float *src = Kh + (int64_t)(k0 + j) * dk + c;
                if (vec && c + 4 <= dk) v = __ldg(reinterpret_cast<const float4 *>(src));
                else {
                    if (c + 0 < dk) v.x = __ldg(src + 0);
                    if (c + 1 < dk) v.y = __ldg(src + 1);
                    if (c + 2 < dk) v.z = __ldg(src + 2);
                    if (c + 3 < dk) v.w = __ldg(src + 3);
                }
            }
            Kt[(c + 0) * BKV + j] = v.x;
            Kt[(c + 1) * BKV + j] = v.y;
            Kt[(c + 2) * BKV + j] = v.z;
            Kt[(c + 3) * BKV + j] = v.w;
        }
        // V block -> Vs
        for (int i = tid; i < BKV * (DKP / 4); i += SD_THREADS) {
            const int r = i / (DKP / 4), c = (i - r * (DKP / 4)) * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (k0 + r < S) {
                const float *src = Vh + (int64_t)(k0 + r) * dk + c;
                if (vec && c + 4 <= dk) v = __ldg(reinterpret_cast<const float4 *>(src));
                else {
                    if (c + 0 < dk) v.x = __ldg(src + 0);
                    if (c + 1 < dk) v.y = __ldg(src + 1);
                    if (c + 2 < dk) v.z = __ldg(src + 2);
                    if (c + 3 < dk) v.w = __ldg(src + 3);
                }
            }
            *reinterpret_cast<float4 *>(Vs + r * DKP + c) = v;
        }
        __syncthreads();

        // S tile: rows ty*4.., cols tx*4..
        float s[4][4];
#pragma unroll
        for (int a = 0; a < 4; ++a) s[a][0] = s[a][1] = s[a][2] = s[a][3] = 0.f;
#pragma unroll 4
        for (int d = 0; d < DKP; d += 4) {
            float4 q[4], k[4];
#pragma unroll
            for (int a = 0; a < 4; ++a) q[a] = *reinterpret_cast<const float4 *>(Qs + (ty * 4 + a) * DKP + d);
#pragma unroll
            for (int e = 0; e < 4; ++e) k[e] = *reinterpret_cast<const float4 *>(Kt + (d + e) * BKV + tx * 4);
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
        // scale, mask, online softmax
        const bool diag = causal && (kb == qb);
        const bool tail = (k0 + BKV > S);
#pragma unroll
        for (int a = 0; a < 4; ++a) {
            const int gi = q0 + ty * 4 + a;
            float mx = -INFINITY;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const int gj = k0 + tx * 4 + b;
                float v = s[a][b] * scale;
                if ((diag && gj > gi) || (tail && gj >= S)) v = -INFINITY;
                s[a][b] = v;
                mx = fmaxf(mx, v);
            }
#pragma unroll
            for (int off = 1; off < 16; off <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
            const float m_new = fmaxf(m_run[a], mx);
            const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
            const float corr = expf(m_run[a] - m_safe);  // exp(-inf) = 0 on the first block
            float sum = 0.f;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                s[a][b] = expf(s[a][b] - m_safe);
                sum += s[a][b];
            }
#pragma unroll
            for (int off = 1; off < 16; off <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
            l_run[a] = l_run[a] * corr + sum;
            m_run[a] = m_new;
#pragma unroll
            for (int c = 0; c < NCG * 4; ++c) o[a][c] *= corr;
            *reinterpret_cast<float4 *>(Ps + (ty * 4 + a) * PS_PITCH + tx * 4) =
                make_float4(s[a][0], s[a][1], s[a][2], s[a][3]);
        }
        __syncthreads();
        // O += P . V
#pragma unroll 2
        for (int j = 0; j < BKV; j += 4) {
            float4 p[4];
#pragma unroll
            for (int a = 0; a < 4; ++a) p[a] = *reinterpret_cast<const float4 *>(Ps + (ty * 4 + a) * PS_PITCH + j);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
#pragma unroll
                for (int cg = 0; cg < NCG; ++cg) {
                    const float4 v = *reinterpret_cast<const float4 *>(Vs + (j + e) * DKP + cg * 64 + tx * 4);
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

    // normalise and store
#pragma unroll
    for (int a = 0; a < 4; ++a) {
        const int gi = q0 + ty * 4 + a;
        if (gi >= S) continue;
        const float inv = l_run[a] > 0.f ? 1.0f / l_run[a] : 0.f;
        float *dst = O + (head * (int64_t)S + gi) * dk;
#pragma unroll
        for (int cg = 0; cg < NCG; ++cg) {
            const int c = cg * 64 + tx * 4;
            if (vec && c + 4 <= dk) {
                *reinterpret_cast<float4 *>(dst + c) = make_float4(o[a][cg * 4 + 0] * inv, o[a][cg * 4 + 1] * inv,
                                                                   o[a][cg * 4 + 2] * inv, o[a][cg * 4 + 3] * inv);
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (c + e < dk) dst[c + e] = o[a][cg * 4 + e] * inv;
            }
        }
        if (L && tx == 0) L[head * (int64_t)S + gi] = m_run[a] + logf(l_run[a]);
    }
}

int launch_sdpa_fwd(const float *Q, const float *K, const float *V, float *O, float *L, int64_t BH,
                    int64_t S, int64_t dk, float scale, int causal, cudaStream_t st)
{
    if (BH <= 0 || S <= 0) return 0;
    dim3 grid((unsigned)((S + BQ - 1) / BQ), (unsigned)BH);
    if (dk <= 64) {
        const size_t smem = (size_t)(BQ * 64 + 64 * BKV + BKV * 64 + BQ * PS_PITCH) * 4;
        static PerDeviceOnce once64;
        if (once64.first()) cudaFuncSetAttribute(sdpa_fwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        sdpa_fwd_kernel<64><<<grid, SD_THREADS, smem, st>>>(Q, K, V, O, L, (int)S, (int)dk, scale, causal);
    } else {
        const size_t smem = (size_t)(BQ * 128 + 128 * BKV + BKV * 128 + BQ * PS_PITCH) * 4;
        static PerDeviceOnce once128;
        if (once128.first()) cudaFuncSetAttribute(sdpa_fwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        sdpa_fwd_kernel<128><<<grid, SD_THREADS, smem, st>>>(Q, K, V, O, L, (int)S, (int)dk, scale, causal);
    }
    return (int)cudaGetLastError();
}

// P[bh,i,j] = exp(scale * q_i.k_j - L[bh,i]) (0 above the diagonal when causal): the soft-max probabilities the
// stock backend copies into P_save out of its score buffer (src/compute/backends/cuda/ops_attention.cu:366-370).
// The fused forward never forms them, so a caller that passes P_save gets them from this pass, after L is known.
// One CTA per 64x64 tile, fp32 FMA over dk in chunks of 32; tiles wholly above the diagonal are only cleared.
__global__ void __launch_bounds__(256) sdpa_probs_kernel(const float *__restrict__ Q, const float *__restrict__ K,
                                                         const float *__restrict__ L, float *__restrict__ P, int S,
                                                         int dk, float scale, int causal)
{
    __shared__ float Qs[64][33], Ks[64][33];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int j0 = blockIdx.x * 64, i0 = blockIdx.y * 64;
    const int64_t head = blockIdx.z;
    const float *Qh = Q + head * (int64_t)S * dk, *Kh = K + head * (int64_t)S * dk;
    float *Ph = P + head * (int64_t)S * S;
    float acc[4][4] = {};
    const bool dead = causal && j0 > i0 + 63;
    if (!dead) {
        for (int k0 = 0; k0 < dk; k0 += 32) {
            for (int e = tid; e < 64 * 32; e += 256) {
                const int r = e >> 5, c = e & 31;
                Qs[r][c] = (i0 + r < S && k0 + c < dk) ? __ldg(Qh + (int64_t)(i0 + r) * dk + k0 + c) : 0.0f;
                Ks[r][c] = (j0 + r < S && k0 + c < dk) ? __ldg(Kh + (int64_t)(j0 + r) * dk + k0 + c) : 0.0f;
            }
            __syncthreads();
#pragma unroll 8
            for (int k = 0; k < 32; ++k) {
                float q[4], kk[4];
#pragma unroll
                for (int a = 0; a < 4; ++a) q[a] = Qs[ty * 4 + a][k];
#pragma unroll
                for (int b = 0; b < 4; ++b) kk[b] = Ks[tx + 16 * b][k];
#pragma unroll
                for (int a = 0; a < 4; ++a)
#pragma unroll
                    for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(q[a], kk[b], acc[a][b]);
            }
            __syncthreads();
        }
    }
#pragma unroll
    for (int a = 0; a < 4; ++a) {
        const int i = i0 + ty * 4 + a;
        if (i >= S) continue;
        const float l = dead ? 0.0f : __ldg(L + head * (int64_t)S + i);
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int j = j0 + tx + 16 * b;
            if (j >= S) continue;
            Ph[(int64_t)i * S + j] = (dead || (causal && j > i)) ? 0.0f : expf(acc[a][b] * scale - l);
        }
    }
}

int launch_sdpa_probs(const float *Q, const float *K, const float *L, float *P, int64_t BH, int64_t S, int64_t dk,
                      float scale, int causal, cudaStream_t st)
{
    if (BH <= 0 || S <= 0) return 0;
    const unsigned t = (unsigned)((S + 63) / 64);
    sdpa_probs_kernel<<<dim3(t, t, (unsigned)BH), 256, 0, st>>>(Q, K, L, P, (int)S, (int)dk, scale, causal);
    return (int)cudaGetLastError();
}

}  // namespace axb
