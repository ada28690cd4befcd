// skinny_tma.cu — the skinny-M route with the weight stream staged by TMA.
//
// Same arithmetic and the same fixed-order split-K reduction as skinny.cu, but
// W[K,N] reaches the SM through cp.async.bulk.tensor into a ring of 16 KB
// shared-memory stages filled by one producer thread.  The copy engine keeps
// the whole ring (64 KB per CTA) in flight no matter how many registers the
// FMA warps hold, which is what a stream of this size needs to get near the
// HBM rate: with plain loads the bytes in flight were capped by
// registers x occupancy and the kernel sat at ~45% of the copy bandwidth.
//
//   warp 8 (one lane)  producer: box = 16 rows x 256 columns (M <= 8) or
//                      32 rows x 128 columns (M > 8), completion on full[s]
//   warps 0..7         consumers: warp w takes rows w, w+8, .. of a stage; a lane
//                      reads its 4 (or 8) columns with 128-bit shared loads, X is
//                      broadcast from shared memory, all M outputs accumulate in
//                      registers; one arrive per warp on empty[s]
// Rows past K and columns past N are zero-filled by the tensor map.
#include "skinny.cuh"

#include "gemm_tc.cuh"
#include "ptx.cuh"

#include <cuda.h>
#include <stdint.h>

namespace axb {

static constexpr int ST_THREADS = 288;
static constexpr int ST_CONSUMERS = 8;
static constexpr int ST_MAX_STAGES = 8;
static constexpr int ST_STAGE_BYTES = 16384;
static constexpr int ST_HEADER = 128;

__device__ __forceinline__ float st_gelu(float v)
{
    const float inner = 0.7978845608028654f * (v + 0.044715f * v * v * v);
    return 0.5f * v * (1.0f + tanhf(inner));
}

__device__ __forceinline__ float st_epilogue(const SkinnyArgs &a, float v, int m, int64_t col)
{
    v *= a.alpha;
    if (a.beta != 0.0f) v += a.beta * a.Y[(int64_t)m * a.N + col];
    if (a.bias) v += __ldg(a.bias + col);
    if (a.act == 1) v = fmaxf(v, 0.0f);
    else if (a.act == 2) v = st_gelu(v);
    return v;
}

// floats of the region that holds the X slice [kchunk][mt] and later the CTA's strip sums [min(mt, 8)][<= 256]
__host__ __device__ inline int skinny_tma_x_floats(int mt, int kchunk)
{
    const int x = kchunk * mt, sums = (mt < 8 ? mt : 8) * 256;
    return ((x > sums ? x : sums) + 3) & ~3;
}

template <int MT, int CPL>
__global__ void __launch_bounds__(ST_THREADS) skinny_tma_kernel(const __grid_constant__ CUtensorMap tmW,
                                                                const SkinnyArgs a)
{
    constexpr int COLS = 128 * CPL;                     // columns of a strip
    constexpr int R = ST_STAGE_BYTES / (COLS * 4);      // rows per stage
    constexpr int RM = MT < 8 ? MT : 8;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ int s_last;
    const uint32_t base = (smem_u32(smem_raw) + 127u) & ~127u;
    uint8_t *gbase = smem_raw + (base - smem_u32(smem_raw));
    const int ST_STAGES = a.stages;  // ring depth chosen by the planner (<= ST_MAX_STAGES)
    const uint32_t bar_full = base, bar_empty = base + 8 * ST_MAX_STAGES;
    const uint32_t ring = base + ST_HEADER;
    float *ring_g = reinterpret_cast<float *>(gbase + ST_HEADER);
    float *xs = ring_g + ST_STAGES * ST_STAGE_BYTES / 4;  // [kchunk][MT]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int strip = blockIdx.x, ks = blockIdx.y;
    const int64_t k_begin = (int64_t)ks * a.kchunk;
    const int kc = (int)min((int64_t)a.kchunk, a.K - k_begin);
    const int nst = (kc + R - 1) / R;

    if (tid == 0) {
        for (int s = 0; s < ST_STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, ST_CONSUMERS);
        }
        mbar_fence_init();
        tma_prefetch_desc(&tmW);
    }
    __syncthreads();
    grid_dep_launch();   // a skinny call queued behind this one may start streaming ITS weights now

    // the producer puts the first stages in flight before anyone touches X
    if (warp == ST_CONSUMERS && lane == 0) {
        for (int st = 0; st < nst && st < ST_STAGES; ++st) {
            mbar_arrive_expect_tx(bar_full + 8 * st, ST_STAGE_BYTES);
            tma_load_2d(ring + st * ST_STAGE_BYTES, &tmW, bar_full + 8 * st, strip * COLS, (int)(k_begin + st * R));
        }
    }
    // the weights were requested while the kernel before this one may still be running (programmatic dependent
    // launch); X may be its output and Y its input, so everything else waits until it has finished
    grid_dep_wait();
    // X slice -> shared as [k][MT]; for MT >= 8 the float4 groups of a row are XOR-permuted with k so
    // the transposing stores spread over the banks (a lane stores one k, lanes differ in k).  Four consecutive k of
    // one row per 128-bit load when the rows allow it: the loads of a thread are independent and in flight together,
    // where one scalar load per (k, m) made the slice the longest wait before the first multiply (2.5 us at M = 8).
    {
        auto put = [&](int kk, int m, float v) {
            const int swz = MT >= 4 ? ((kk & 7) & (MT / 4 - 1)) : 0;
            const int pm = MT >= 4 ? ((((m >> 2) ^ swz) << 2) | (m & 3)) : m;
            xs[kk * MT + pm] = v;
        };
        const bool xvec = ((a.K | k_begin) & 3) == 0 && (reinterpret_cast<uintptr_t>(a.X) & 15) == 0;
        if (xvec) {
            const int kq = (kc + 3) >> 2;   // groups of four k
            constexpr int XB = 4;           // loads of a thread issued together, before any of them is stored
            for (int it0 = 0; it0 < kq * MT; it0 += XB * ST_THREADS) {
                float4 v[XB];
#pragma unroll
                for (int j = 0; j < XB; ++j) {
                    const int it = it0 + j * ST_THREADS + tid;
                    const int g = it / MT, m = it - g * MT, kk = g << 2;   // lanes run over the rows first
                    v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (it < kq * MT && m < a.M) {
                        const float *src = a.X + (int64_t)m * a.K + k_begin + kk;
                        if (kk + 4 <= kc) v[j] = __ldg(reinterpret_cast<const float4 *>(src));
                        else {
                            v[j].x = __ldg(src);
                            if (kk + 1 < kc) v[j].y = __ldg(src + 1);
                            if (kk + 2 < kc) v[j].z = __ldg(src + 2);
                        }
                    }
                }
#pragma unroll
                for (int j = 0; j < XB; ++j) {
                    const int it = it0 + j * ST_THREADS + tid;
                    if (it >= kq * MT) continue;
                    const int g = it / MT, m = it - g * MT, kk = g << 2;
                    put(kk, m, v[j].x);
                    if (kk + 1 < kc) put(kk + 1, m, v[j].y);
                    if (kk + 2 < kc) put(kk + 2, m, v[j].z);
                    if (kk + 3 < kc) put(kk + 3, m, v[j].w);
                }
            }
        } else {
            for (int kk = tid; kk < kc; kk += ST_THREADS) {
#pragma unroll
                for (int m = 0; m < MT; ++m) put(kk, m, (m < a.M) ? __ldg(a.X + (int64_t)m * a.K + k_begin + kk) : 0.0f);
            }
        }
    }
    __syncthreads();

    // accumulators: rows m = 2p and 2p+1 share one packed register pair, so one fma.rn.f32x2 feeds both
    constexpr int MP = MT >= 2 ? MT / 2 : 1;
    float2 acc[MP][4 * CPL];
#pragma unroll
    for (int p = 0; p < MP; ++p)
#pragma unroll
        for (int c = 0; c < 4 * CPL; ++c) acc[p][c] = make_float2(0.0f, 0.0f);

    bool ok = true;
    if (warp == ST_CONSUMERS) {
        if (lane == 0) {
            for (int st = ST_STAGES; st < nst; ++st) {
                const uint32_t s = st % ST_STAGES, ph = (st / ST_STAGES) & 1u;
                if (!mbar_wait_bounded(bar_empty + 8 * s, ph ^ 1u)) {
                    if (a.err) atomicCAS(a.err, 0, 11);
                    break;
                }
                mbar_arrive_expect_tx(bar_full + 8 * s, ST_STAGE_BYTES);
                tma_load_2d(ring + s * ST_STAGE_BYTES, &tmW, bar_full + 8 * s, strip * COLS, (int)(k_begin + st * R));
            }
        }
    } else {
        for (int st = 0; st < nst; ++st) {
            const uint32_t s = st % ST_STAGES, ph = (st / ST_STAGES) & 1u;
            const bool got = mbar_wait_bounded(bar_full + 8 * s, ph);
            if (!__all_sync(0xffffffffu, got)) {
                if (a.err && lane == 0) atomicCAS(a.err, 0, 12);
                ok = false;
                break;
            }
            const float *stage = ring_g + s * (ST_STAGE_BYTES / 4);
#pragma unroll
            for (int rr = 0; rr < R / ST_CONSUMERS; ++rr) {
                const int r = warp + rr * ST_CONSUMERS;
                const int kk = st * R + r;
                if (kk < kc) {
                    float4 w[CPL];
#pragma unroll
                    for (int c = 0; c < CPL; ++c)
                        w[c] = *reinterpret_cast<const float4 *>(stage + r * COLS + c * 128 + lane * 4);
                    const float *xr = xs + kk * MT;
                    if constexpr (MT == 1) {
                        const float xv = xr[0];
#pragma unroll
                        for (int c = 0; c < CPL; ++c) {
                            acc[0][4 * c + 0].x = fmaf(xv, w[c].x, acc[0][4 * c + 0].x);
                            acc[0][4 * c + 1].x = fmaf(xv, w[c].y, acc[0][4 * c + 1].x);
                            acc[0][4 * c + 2].x = fmaf(xv, w[c].z, acc[0][4 * c + 2].x);
                            acc[0][4 * c + 3].x = fmaf(xv, w[c].w, acc[0][4 * c + 3].x);
                        }
                    } else {
                        float2 wd[4 * CPL];  // each weight duplicated into both halves of a pair
#pragma unroll
                        for (int c = 0; c < CPL; ++c) {
                            wd[4 * c + 0] = make_float2(w[c].x, w[c].x);
                            wd[4 * c + 1] = make_float2(w[c].y, w[c].y);
                            wd[4 * c + 2] = make_float2(w[c].z, w[c].z);
                            wd[4 * c + 3] = make_float2(w[c].w, w[c].w);
                        }
                        if constexpr (MT == 2) {
                            const float2 xp = *reinterpret_cast<const float2 *>(xr);
#pragma unroll
                            for (int c = 0; c < 4 * CPL; ++c) acc[0][c] = __ffma2_rn(xp, wd[c], acc[0][c]);
                        } else {
                            const int swz = (kk & 7) & (MT / 4 - 1);
#pragma unroll
                            for (int g = 0; g < MT / 4; ++g) {
                                const float4 x4 = *reinterpret_cast<const float4 *>(xr + ((g ^ swz) << 2));
                                const float2 x01 = make_float2(x4.x, x4.y), x23 = make_float2(x4.z, x4.w);
#pragma unroll
                                for (int c = 0; c < 4 * CPL; ++c) {
                                    acc[2 * g][c] = __ffma2_rn(x01, wd[c], acc[2 * g][c]);
                                    acc[2 * g + 1][c] = __ffma2_rn(x23, wd[c], acc[2 * g + 1][c]);
                                }
                            }
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + 8 * s);
        }
    }
    (void)ok;
    __syncthreads();  // every stage consumed, no copy in flight: the ring now holds the warp sums

    float *red = ring_g;  // [ST_CONSUMERS][RM][COLS]
    float *part = a.partial ? a.partial + (int64_t)ks * a.M * a.N : nullptr;
#pragma unroll
    for (int m0 = 0; m0 < MT; m0 += RM) {
        if (warp < ST_CONSUMERS) {
#pragma unroll
            for (int mi = 0; mi < RM; ++mi)
#pragma unroll
                for (int c = 0; c < CPL; ++c)
                {
                    const int m = m0 + mi;
                    const float2 *row = acc[MT >= 2 ? m / 2 : 0];
                    const bool hi = (m & 1) != 0;
                    *reinterpret_cast<float4 *>(red + ((warp * RM + mi) * COLS + c * 128 + lane * 4)) =
                        hi ? make_float4(row[4 * c].y, row[4 * c + 1].y, row[4 * c + 2].y, row[4 * c + 3].y)
                           : make_float4(row[4 * c].x, row[4 * c + 1].x, row[4 * c + 2].x, row[4 * c + 3].x);
                }
        }
        __syncthreads();
        if (a.ksplit > 1 && a.cluster) {
            // the common case keeps the strip sums in shared memory for the cluster hand-over: four columns per thread
            // and pass (128-bit loads of the eight warp sums, one 128-bit store)
            for (int o4 = tid; o4 < RM * (COLS / 4); o4 += ST_THREADS) {
                const int mi = o4 / (COLS / 4), c = (o4 - mi * (COLS / 4)) * 4;
                float4 s4 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int w = 0; w < ST_CONSUMERS; ++w) {
                    const float4 v = *reinterpret_cast<const float4 *>(red + (w * RM + mi) * COLS + c);
                    s4.x += v.x; s4.y += v.y; s4.z += v.z; s4.w += v.w;
                }
                *reinterpret_cast<float4 *>(xs + (m0 + mi) * COLS + c) = s4;
            }
        } else
        for (int o = tid; o < RM * COLS; o += ST_THREADS) {
            const int mi = o / COLS, c = o - mi * COLS;
            const int m = m0 + mi;
            const int64_t gc = (int64_t)strip * COLS + c;
            if (m < a.M && gc < a.N) {
                float s = 0.0f;
#pragma unroll
                for (int w = 0; w < ST_CONSUMERS; ++w) s += red[(w * RM + mi) * COLS + c];
                if (a.ksplit == 1) a.Y[(int64_t)m * a.N + gc] = st_epilogue(a, s, m, gc);
                else if (a.cluster) xs[m * COLS + c] = s;   // X is dead: its space carries this CTA's strip sums
                else part[(int64_t)m * a.N + gc] = s;
            }
        }
        __syncthreads();
    }

    if (a.ksplit > 1 && a.cluster) {
        // The K-slices of this strip are the CTAs of one cluster and the strip's outputs are dealt out to them in
        // contiguous shares: slice r finishes outputs [r * per_owner, (r + 1) * per_owner).  Every slice PUSHES its sums into the owners' shared memory (remote
        // stores, fire and forget: slot [sender][o % per_owner] of a region behind X, which nobody reads any more), one
        // cluster barrier makes them visible, and each owner adds the slices in slice order out of its OWN memory — no
        // scratch in global memory, bitwise repeatable, and nobody reads a peer, so no second barrier keeps the
        // CTAs alive.  (Pulling the sums with remote loads needed that second barrier and a round trip: 2.9 us.)
        const int ncols = (int)min((int64_t)COLS, a.N - (int64_t)strip * COLS);
        const int total = a.M * ncols;
        const int per_owner = (total + a.ksplit - 1) / a.ksplit;
        // [ksplit][per_owner], behind the X slice: a peer that finishes early pushes while this CTA still reads X
        float *inbox = xs + skinny_tma_x_floats(MT, a.kchunk);
        const uint32_t me = cluster_cta_rank();
        if (((ncols | per_owner) & 3) == 0) {
            // whole strips: four outputs per remote store (an owner's share and a row both start at multiples of four)
            for (int o = tid * 4; o < total; o += ST_THREADS * 4) {
                const int m = o / ncols, c = o - m * ncols;
                const int owner = o / per_owner, idx = o - owner * per_owner;
                const uint32_t dst = map_to_cta(smem_u32(inbox + (int)me * per_owner + idx), (uint32_t)owner);
                const float4 v = *reinterpret_cast<const float4 *>(xs + m * COLS + c);
                asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
            }
        } else
        for (int o = tid; o < total; o += ST_THREADS) {
            const int m = o / ncols, c = o - m * ncols;
            const int owner = o / per_owner, idx = o - owner * per_owner;
            const uint32_t dst = map_to_cta(smem_u32(inbox + (int)me * per_owner + idx), (uint32_t)owner);
            asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(dst), "f"(xs[m * COLS + c]) : "memory");
        }
        cluster_sync_all();
        for (int idx = tid; idx < per_owner; idx += ST_THREADS) {
            const int o = (int)me * per_owner + idx;
            if (o < total) {
                float sum = 0.0f;
                for (int q = 0; q < a.ksplit; ++q) sum += inbox[q * per_owner + idx];
                const int m = o / ncols, c = o - m * ncols;
                const int64_t gc = (int64_t)strip * COLS + c;
                a.Y[(int64_t)m * a.N + gc] = st_epilogue(a, sum, m, gc);
            }
        }
    } else if (a.ksplit > 1) {
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            const int prev = atomicAdd(a.counters + strip, 1);
            s_last = (prev == a.ksplit - 1);
        }
        __syncthreads();
        if (s_last) {
            __threadfence();
            const int ncols = (int)min((int64_t)COLS, a.N - (int64_t)strip * COLS);
            for (int o = tid; o < a.M * ncols; o += ST_THREADS) {
                const int m = o / ncols;
                const int64_t gc = (int64_t)strip * COLS + (o - m * ncols);
                float s = 0.0f;
                for (int q = 0; q < a.ksplit; ++q) s += __ldcg(a.partial + ((int64_t)q * a.M + m) * a.N + gc);
                a.Y[(int64_t)m * a.N + gc] = st_epilogue(a, s, m, gc);
            }
            if (tid == 0) a.counters[strip] = 0;
        }
    }
}

template <int MT, int CPL>
static int launch_tma_inst(const CUtensorMap &tm, const SkinnyArgs &a, dim3 grid, size_t smem, cudaStream_t st)
{
    auto k = skinny_tma_kernel<MT, CPL>;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        attr_set[dev] = true;
    }
    if (a.cluster) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(ST_THREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = st;
        cudaLaunchAttribute at;
        at.id = cudaLaunchAttributeClusterDimension;
        at.val.clusterDim.x = 1;
        at.val.clusterDim.y = grid.y;   // all K-slices of a strip
        at.val.clusterDim.z = 1;
        cudaLaunchAttribute ats[2] = { at, {} };
        ats[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        ats[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = ats;
        cfg.numAttrs = a.pdl ? 2 : 1;
        return (int)cudaLaunchKernelEx(&cfg, k, tm, a);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(ST_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at;
    at.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &at;
    cfg.numAttrs = a.pdl ? 1 : 0;
    return (int)cudaLaunchKernelEx(&cfg, k, tm, a);
}

int skinny_tma_strip_cols(int mt, int cluster) { return (mt <= 8 && !cluster) ? 256 : 128; }
int skinny_tma_stage_rows(int mt, int cluster) { return ST_STAGE_BYTES / (skinny_tma_strip_cols(mt, cluster) * 4); }
size_t skinny_tma_smem_bytes(int mt, int kchunk, int stages)
{
    // header, ring, the X slice [kchunk][mt] (which later carries this CTA's strip sums, at most [8][256]) and, behind
    // it, the inbox of the cluster reduction: [ksplit][ceil(M * 128 / ksplit)] <= 8 * 128 + 8 floats
    return (size_t)ST_HEADER + 128 + (size_t)stages * ST_STAGE_BYTES + ((size_t)skinny_tma_x_floats(mt, kchunk) + 1024 + 8) * 4;
}

int launch_skinny_tma(const SkinnyArgs &a, const SkinnyPlan &plan, cudaStream_t st)
{
    alignas(64) CUtensorMap tm;
    const int cols = skinny_tma_strip_cols(plan.mt, plan.cluster), rows = skinny_tma_stage_rows(plan.mt, plan.cluster);
    int e = encode_f32_matrix_tmap(&tm, a.W, a.K, a.N, a.N, cols, rows);
    if (e) return e;
    dim3 grid((unsigned)plan.strips, (unsigned)plan.ksplit);
    const size_t smem = plan.smem_bytes;
    if (plan.cluster || plan.mt > 8) {
        switch (plan.mt) {
        case 1: return launch_tma_inst<1, 1>(tm, a, grid, smem, st);
        case 2: return launch_tma_inst<2, 1>(tm, a, grid, smem, st);
        case 4: return launch_tma_inst<4, 1>(tm, a, grid, smem, st);
        case 8: return launch_tma_inst<8, 1>(tm, a, grid, smem, st);
        case 16: return launch_tma_inst<16, 1>(tm, a, grid, smem, st);
        default: return launch_tma_inst<32, 1>(tm, a, grid, smem, st);
        }
    }
    switch (plan.mt) {
    case 1: return launch_tma_inst<1, 2>(tm, a, grid, smem, st);
    case 2: return launch_tma_inst<2, 2>(tm, a, grid, smem, st);
    case 4: return launch_tma_inst<4, 2>(tm, a, grid, smem, st);
    default: return launch_tma_inst<8, 2>(tm, a, grid, smem, st);
    }
}

}  // namespace axb
