// kv_attend.cu — attention of ONE new query token against a KV cache (autoregressive decode):
//     out[h,:] = softmax(scale * K[h,0:len,:] . q[h,:]) . V[h,0:len,:]
// on the cache layout [BH, max_seq, dk] of ax_kv_cache_t (include/axiom/attention.h:341-381; CPU path
// src/compute/backends/cpu_opt.c:9586-9654: two GEMVs and a softmax per head).  The reference has no device
// version.  The work is a single pass over K and V — HBM-bound like the skinny GEMV — so the cached rows of a
// head are cut into segments, one CTA each; the segments of a head form a thread-block cluster and are merged
// (running maximum, rescaled sums) in segment order out of each other's shared memory, which keeps the result
// deterministic.  Inside a CTA a group of lanes owns a row: 128-bit loads along dk, a shuffle tree for the dot
// product, and the same mapping for the p.V accumulation, so both passes read whole rows coalesced.
#include "kv_attend.cuh"

#include "ptx.cuh"

#include <math.h>
#include <stdint.h>

namespace axb {

static constexpr int KV_THREADS = 256, KV_WARPS = 8, KV_CHUNK = 2048;

struct KvArgs {
    const float *K, *V, *Q;
    float *out;
    int64_t max_seq;
    int cur_len, dk;
    float scale;
    int seg;  // cached rows per CTA
    int lpk;  // lanes per row (power of two)
};

// element e (0..3) of lane `li` of a row: contiguous float4 when VEC, else strided by 32
template <bool VEC>
__device__ __forceinline__ int kv_index(int li, int e)
{
    return VEC ? li * 4 + e : li + 32 * e;
}

template <bool VEC>
__device__ __forceinline__ void kv_load(const float *row, int li, int dk, float (&x)[4])
{
    if (VEC) {
        if (li * 4 < dk) {
            const float4 v = __ldg(reinterpret_cast<const float4 *>(row) + li);
            x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
        } else {
            x[0] = x[1] = x[2] = x[3] = 0.f;
        }
    } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) x[e] = (li + 32 * e < dk) ? __ldg(row + li + 32 * e) : 0.f;
    }
}

template <bool VEC>
__global__ void __launch_bounds__(KV_THREADS) kv_attend_kernel(const KvArgs a)
{
    __shared__ float sc[KV_CHUNK];
    __shared__ float4 accbuf[KV_WARPS * 32];
    __shared__ float lbuf[KV_WARPS * 32];
    __shared__ float wred[KV_WARPS];
    __shared__ float fin[2 + 128];   // m, l, acc[dk] of this segment

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int lpk = a.lpk, kpw = 32 / lpk;
    const int li = lane & (lpk - 1), g = lane / lpk;
    const int64_t head = blockIdx.x;
    const int nseg = gridDim.y, segi = blockIdx.y;
    const float *Kh = a.K + head * a.max_seq * a.dk, *Vh = a.V + head * a.max_seq * a.dk;
    const int seg0 = min(a.cur_len, segi * a.seg), seg1 = min(a.cur_len, seg0 + a.seg);

    float q[4];
    kv_load<VEC>(a.Q + head * a.dk, li, a.dk, q);

    float m_run = -INFINITY, l_part = 0.f;
    float acc[4] = { 0.f, 0.f, 0.f, 0.f };
    const int row_stride = KV_WARPS * kpw;

    for (int c0 = seg0; c0 < seg1; c0 += KV_CHUNK) {
        const int n = min(KV_CHUNK, seg1 - c0);
        // scores of this chunk
        float mx = -INFINITY;
        for (int jb = warp * kpw; jb < n; jb += 4 * row_stride) {   // warp-uniform bounds: the shuffles need every lane
            const int j0 = jb + g;
            float k[4][4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int j = j0 + u * row_stride;
                if (j < n) kv_load<VEC>(Kh + (int64_t)(c0 + j) * a.dk, li, a.dk, k[u]);
                else k[u][0] = k[u][1] = k[u][2] = k[u][3] = 0.f;
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int j = j0 + u * row_stride;
                float d = q[0] * k[u][0];
                d = fmaf(q[1], k[u][1], d);
                d = fmaf(q[2], k[u][2], d);
                d = fmaf(q[3], k[u][3], d);
                for (int off = lpk >> 1; off > 0; off >>= 1) d += __shfl_xor_sync(0xffffffffu, d, off);
                d *= a.scale;
                if (j < n) {
                    mx = fmaxf(mx, d);
                    if (li == 0) sc[j] = d;
                }
            }
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
        if (lane == 0) wred[warp] = mx;
        __syncthreads();
        float m_chunk = wred[0];
#pragma unroll
        for (int w = 1; w < KV_WARPS; ++w) m_chunk = fmaxf(m_chunk, wred[w]);
        const float m_new = fmaxf(m_run, m_chunk);
        const float corr = (m_run == -INFINITY) ? 0.f : expf(m_run - m_new);
        l_part *= corr;
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[e] *= corr;
        // p.V with the same row ownership (a group reads back the scores it wrote)
        for (int jb = warp * kpw; jb < n; jb += 4 * row_stride) {
            const int j0 = jb + g;
            float v[4][4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int j = j0 + u * row_stride;
                if (j < n) kv_load<VEC>(Vh + (int64_t)(c0 + j) * a.dk, li, a.dk, v[u]);
                else v[u][0] = v[u][1] = v[u][2] = v[u][3] = 0.f;
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int j = j0 + u * row_stride;
                if (j < n) {
                    const float p = expf(sc[j] - m_new);
                    if (li == 0) l_part += p;
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[e] = fmaf(p, v[u][e], acc[e]);
                }
            }
        }
        m_run = m_new;
        __syncthreads();   // the next chunk overwrites sc and wred
    }

    // segment totals, summed in a fixed order
    accbuf[tid] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    lbuf[tid] = l_part;
    __syncthreads();
    if (tid < lpk) {
        float s[4] = { 0.f, 0.f, 0.f, 0.f };
        for (int w = 0; w < KV_WARPS; ++w)
            for (int gg = 0; gg < kpw; ++gg) {
                const float4 t = accbuf[w * 32 + gg * lpk + tid];
                s[0] += t.x; s[1] += t.y; s[2] += t.z; s[3] += t.w;
            }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int d = kv_index<VEC>(tid, e);
            if (d < a.dk) fin[2 + d] = s[e];
        }
    }
    if (tid == 32) {
        float l = 0.f;
        for (int i = 0; i < KV_THREADS; ++i) l += lbuf[i];
        fin[0] = m_run;   // every thread holds the same running maximum
        fin[1] = l;
    }
    __syncthreads();

    if (nseg == 1) {
        if (tid < a.dk) a.out[head * a.dk + tid] = fin[2 + tid] / fin[1];
        return;
    }
    cluster_sync_all();
    if (segi == 0 && tid < a.dk) {
        float M = -INFINITY;
        for (int s = 0; s < nseg; ++s) {
            float ms;
            asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(ms) : "r"(map_to_cta(smem_u32(&fin[0]), (uint32_t)s)));
            M = fmaxf(M, ms);
        }
        float o = 0.f, L = 0.f;
        for (int s = 0; s < nseg; ++s) {
            float ms, ls, as;
            asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(ms) : "r"(map_to_cta(smem_u32(&fin[0]), (uint32_t)s)));
            asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(ls) : "r"(map_to_cta(smem_u32(&fin[1]), (uint32_t)s)));
            asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(as) : "r"(map_to_cta(smem_u32(&fin[2 + tid]), (uint32_t)s)));
            const float w = (ms == -INFINITY) ? 0.f : expf(ms - M);
            o = fmaf(as, w, o);
            L = fmaf(ls, w, L);
        }
        a.out[head * a.dk + tid] = o / L;
    }
    cluster_sync_all();   // the peers' shared memory must outlive the reads above
}

int launch_kv_cache_attend(const float *K_cache, const float *V_cache, const float *Q_new, float *out, int64_t BH,
                           int64_t cur_len, int64_t max_seq, int64_t dk, float scale, int sm_count, cudaStream_t st)
{
    if (BH <= 0) return 0;
    if (cur_len <= 0) return (int)cudaMemsetAsync(out, 0, (size_t)BH * dk * sizeof(float), st);
    const uintptr_t align = reinterpret_cast<uintptr_t>(K_cache) | reinterpret_cast<uintptr_t>(V_cache) |
                            reinterpret_cast<uintptr_t>(Q_new);
    const bool vec = (dk % 4 == 0) && ((align & 15) == 0);
    KvArgs a;
    a.K = K_cache; a.V = V_cache; a.Q = Q_new; a.out = out;
    a.max_seq = max_seq; a.cur_len = (int)cur_len; a.dk = (int)dk; a.scale = scale;
    int lpk = 32;
    if (vec) {
        lpk = 1;
        while (lpk * 4 < dk) lpk <<= 1;
    }
    a.lpk = lpk;
    // segments: about four CTAs per SM over all heads, at least 256 cached rows each, at most 8 (one cluster)
    int64_t splits = (4 * (int64_t)sm_count + BH - 1) / BH;
    if (splits > (cur_len + 255) / 256) splits = (cur_len + 255) / 256;
    if (splits > 8) splits = 8;
    if (splits < 1) splits = 1;
    a.seg = (int)(((cur_len + splits - 1) / splits + 7) / 8 * 8);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)BH, (unsigned)splits);
    cfg.blockDim = dim3(KV_THREADS);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute at;
    at.id = cudaLaunchAttributeClusterDimension;
    at.val.clusterDim.x = 1;
    at.val.clusterDim.y = (unsigned)splits;
    at.val.clusterDim.z = 1;
    cfg.attrs = &at;
    cfg.numAttrs = 1;
    return vec ? (int)cudaLaunchKernelEx(&cfg, kv_attend_kernel<true>, a) : (int)cudaLaunchKernelEx(&cfg, kv_attend_kernel<false>, a);
}

}  // namespace axb
