// skinny_tc.cu — Y[M,N] = act(alpha * X[M,K].W[K,N] + beta*Y + bias) for 8 < M <= 32 on the tensor cores.
//
// The fp32-FMA skinny kernels stream W at the HBM rate only while M is small: at M = 32 every weight float4
// feeds 128 FMAs and the fp32 pipe, not memory, sets the pace (measured 16 % of the copy bandwidth).  Here the
// product is computed transposed, Y^T[N,M] = W^T.X^T, so that the 128 rows of the MMA are output COLUMNS and the
// few activation rows are its N.  Three tf32 products (hi.hi, hi.lo, lo.hi) keep fp32 accuracy; hi is the fp32
// value itself (the tensor core ignores the 13 low mantissa bits of a tf32 container), lo = tf32(x - trunc(x)).
//
// W is the A operand and is fed from TENSOR MEMORY: TMA lands the plain [32 k][128 n] tile in shared memory,
// each converter thread reads one column of it (its 32 k values for one output column — a warp reads 128
// contiguous bytes per k), computes the lo values in registers and stores hi and lo into tensor memory with
// tcgen05.st, where lane = output column and column = k is exactly the layout of a TS-form MMA's A operand.  So W
// crosses shared memory twice (TMA in, converter out) instead of six times (a version with W as a shared-memory
// operand, lo tiles written back to shared memory and three passes of the tensor core over them, was bound by
// shared-memory bandwidth at 35 % of the HBM rate).  X stays a K-major shared-memory B operand; its lo half is
// written right behind its hi half, so both are ONE operand of 2*M rows and W hi meets them in one pass.
//
// One CTA = 128 output columns x one K-slice; the K-slices of a column tile form a thread-block cluster and are
// summed through distributed shared memory in slice order (deterministic).  Roles: warp 0 TMA producer (ring of
// 8 stages of 32 k-rows — 128 KB of W in flight per SM), warps 1 and 10 MMA issuers for the even and the odd k-blocks
// (each into its own accumulator set), warps 2-5 and 6-9 two converter groups that take alternate k-blocks (a ring of
// four hi/lo tile pairs in tensor memory); warps 6-9 also drain the accumulators every 256 k (fresh TMEM
// accumulators per chunk: the tensor core truncates when it accumulates) and run the epilogue.
#include "skinny.cuh"

#include "gemm_tc.cuh"
#include "ptx.cuh"

#include <cuda.h>
#include <math.h>

namespace axb {

static constexpr int KT_THREADS = 352;   // producer, MMA issuer, 4 + 4 converter warps, second MMA issuer
static constexpr int KT_STAGES = 8;      // shared-memory ring (TMA destinations)
static constexpr int KT_T = 4;           // ring of W hi/lo tile pairs in tensor memory (64 columns each)
static constexpr int KT_ACC_COL = KT_T * 64;   // two accumulator buffers of two sets of 2*MP columns follow the ring
static constexpr int KT_KB = 32;        // k rows per stage
static constexpr int KT_BN = 128;       // output columns per CTA
static constexpr int KT_CHUNK = 8;      // stages per accumulator chunk (256 k)
static constexpr int KT_W_BYTES = KT_KB * KT_BN * 4;  // 16 KB: [32 k][128 n], rows of 512 bytes

struct alignas(64) SkinnyTcMaps {
    CUtensorMap w, x;
};

enum { KERR_PRODUCER = 21, KERR_CONVERT = 22, KERR_MMA = 23, KERR_DRAIN = 24 };

// KB_EMPTY + s completes when the MMAs of the block in stage s have retired: it frees the stage for the producer and,
// four blocks on, that block's tensor-memory slot for the converters
enum { KB_RAW = 0, KB_EMPTY = KT_STAGES, KB_T_FULL = 2 * KT_STAGES, KB_CHUNK_FULL = 2 * KT_STAGES + KT_T,
       KB_CHUNK_EMPTY = 2 * KT_STAGES + KT_T + 2 };


// one lane polls, the warp gets the outcome: 32 lanes spinning on a barrier cost shared-memory bandwidth that
// the MMA operands need
__device__ __forceinline__ bool kt_wait_warp(uint32_t bar, uint32_t parity)
{
    int ok = 1;
    if ((threadIdx.x & 31) == 0) ok = mbar_wait_bounded(bar, parity) ? 1 : 0;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

__device__ __forceinline__ void kt_report(int *err, int code)
{
    if (err) atomicCAS(err, 0, code);
}

__device__ __forceinline__ float kt_gelu(float v)
{
    const float inner = 0.7978845608028654f * (v + 0.044715f * v * v * v);
    return 0.5f * v * (1.0f + tanhf(inner));
}

__device__ __forceinline__ float kt_epilogue(const SkinnyArgs &a, float v, int m, int64_t col)
{
    v *= a.alpha;
    if (a.beta != 0.0f) v += a.beta * a.Y[(int64_t)m * a.N + col];
    if (a.bias) v += __ldg(a.bias + col);
    if (a.act == 1) v = fmaxf(v, 0.0f);
    else if (a.act == 2) v = kt_gelu(v);
    return v;
}

// lo = tf32(x - trunc_tf32(x)) for PER 16-byte groups per thread (group index first + 128*u) starting at `src`,
// written `lo_off` bytes further on.  All loads are issued before the first use: four warps convert a stage, so
// the loop must not serialise on shared-memory latency.
template <int PER>
__device__ __forceinline__ void kt_split(uint32_t src, uint32_t lo_off, int first)
{
    uint32_t x[PER][4];
#pragma unroll
    for (int u = 0; u < PER; ++u) {
        const uint32_t addr = src + (uint32_t)(first + 128 * u) * 16u;
        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(x[u][0]), "=r"(x[u][1]), "=r"(x[u][2]), "=r"(x[u][3]) : "r"(addr));
    }
#pragma unroll
    for (int u = 0; u < PER; ++u) {
        const uint32_t addr = src + (uint32_t)(first + 128 * u) * 16u;
        uint32_t l[4];
#pragma unroll
        for (int e = 0; e < 4; ++e)
            l[e] = (__float_as_uint(__uint_as_float(x[u][e]) - __uint_as_float(x[u][e] & 0xFFFFE000u)) + 0x1000u) & 0xFFFFE000u;
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr + lo_off), "r"(l[0]), "r"(l[1]), "r"(l[2]), "r"(l[3]) : "memory");
    }
}

template <int MP>
__global__ void __launch_bounds__(KT_THREADS, 1) skinny_tc_kernel(const __grid_constant__ SkinnyTcMaps tm,
                                                                   const SkinnyArgs a, int kb_total)
{
    constexpr uint32_t X_BYTES = MP * 128;                       // [MP rows][32 k] fp32
    // stage: W | X hi | X lo (the lo half of X is written by the converters right behind the hi half)
    constexpr uint32_t STAGE = KT_W_BYTES + 2 * X_BYTES;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *base_ptr = smem_raw + (base - raw);
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(base_ptr + 512);
    auto bar = [&](int i) -> uint32_t { return base + 8u * (uint32_t)i; };
    auto stage_addr = [&](int s) -> uint32_t { return base + 1024u + (uint32_t)s * STAGE; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x, slice = blockIdx.y, nslices = gridDim.y;
    const int64_t n0 = (int64_t)tile * KT_BN;
    const int per = (kb_total + nslices - 1) / nslices;
    const int kb0 = slice * per;
    const int nkb = max(0, min(per, kb_total - kb0));
    const int nchunks = (nkb + KT_CHUNK - 1) / KT_CHUNK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < KT_STAGES; ++s) {
            mbar_init(bar(KB_RAW + s), 1);
            mbar_init(bar(KB_EMPTY + s), 1);
        }
        for (int s = 0; s < KT_T; ++s) mbar_init(bar(KB_T_FULL + s), 128);
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar(KB_CHUNK_FULL + b), 2);      // one arrival per MMA issuer
            mbar_init(bar(KB_CHUNK_EMPTY + b), 128);
        }
        mbar_fence_init();
        // the first ring of tiles is requested before anything else happens in this CTA (tensor-memory allocation,
        // the block-wide barrier): the first HBM round trip is the longest wait of the kernel
        tma_prefetch_desc(&tm.w);
        tma_prefetch_desc(&tm.x);
        grid_dep_launch();   // a skinny call queued behind this one may start streaming ITS weights now
        for (int i = 0; i < nkb && i < KT_STAGES; ++i) {
            mbar_arrive_expect_tx(bar(KB_RAW + i), KT_W_BYTES + X_BYTES);
            tma_load_2d(stage_addr(i), &tm.w, bar(KB_RAW + i), (int32_t)n0, (kb0 + i) * KT_KB);
        }
        // the weights were requested while the kernel before this one may still be running (programmatic dependent
        // launch); the activations may be its output, so they are fetched only once it has finished
        grid_dep_wait();
        for (int i = 0; i < nkb && i < KT_STAGES; ++i)
            tma_load_3d(stage_addr(i) + KT_W_BYTES, &tm.x, bar(KB_RAW + i), (kb0 + i) * KT_KB, 0, 0);
    }
    if (warp == 1) {
        tmem_alloc(base + 512, 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    float acc[MP];
#pragma unroll
    for (int m = 0; m < MP; ++m) acc[m] = 0.f;
    const int t_row = 32 * (warp & 3) + lane;   // drain warps: TMEM lane = output column of the tile

    if (warp == 0) {
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            for (int i = KT_STAGES; i < nkb; ++i) {
                const int s = i % KT_STAGES, n = i / KT_STAGES;
                if (!mbar_wait_bounded(bar(KB_EMPTY + s), (n - 1) & 1)) { kt_report(a.err, KERR_PRODUCER); break; }
                const uint32_t st = stage_addr(s);
                const int k0 = (kb0 + i) * KT_KB;
                mbar_arrive_expect_tx(bar(KB_RAW + s), KT_W_BYTES + X_BYTES);
                tma_load_2d(st, &tm.w, bar(KB_RAW + s), (int32_t)n0, k0);
                tma_load_3d(st + KT_W_BYTES, &tm.x, bar(KB_RAW + s), k0, 0, 0);
            }
        }
    } else if (warp == 1 || warp == 10) {
        // --------------------------------------------------------- MMA issuers
        // TWO issuing threads: warp 1 takes the even k-blocks, warp 10 the odd ones, each into its own accumulator
        // set.  These MMAs are short (M128 x N<=64 x K8) and the tensor pipe is mostly idle; what a block costs is
        // the issuing thread's own time — about 70 cycles per tcgen05.mma and 120 per tcgen05.commit, 1.2 k cycles
        // per block of 8 + 2, measured with in-kernel time stamps — so a second thread doubles the rate.
        if (lane == 0) {
            const int par = warp == 1 ? 0 : 1;
            const uint64_t desc_x = smem_desc_kmajor(0, 128);
            // N = 2*MP for the pass of W hi over X hi and X lo side by side, MP for W lo over X hi
            const uint32_t idesc_hi = make_idesc<KIND_TF32>(KT_BN, 2 * MP);
            const uint32_t idesc_lo = make_idesc<KIND_TF32>(KT_BN, MP);
            bool ok = true;
            for (int ci = 0; ci < nchunks && ok; ++ci) {
                const int cb = ci & 1;
                if (ci >= 2 && !mbar_wait_bounded(bar(KB_CHUNK_EMPTY + cb), ((ci >> 1) - 1) & 1)) { ok = false; break; }
                // a SET = columns [0, MP): hi.hi, [MP, 2*MP): hi.lo + lo.hi (the second pass accumulates into the
                // columns of the first pass's second half: both are corrections of the same size)
                const uint32_t d = tmem + KT_ACC_COL + cb * (4 * MP) + par * (2 * MP);
                const int i_end = min(nkb, (ci + 1) * KT_CHUNK);
                bool issued = false;
                for (int i = ci * KT_CHUNK + par; i < i_end; i += 2) {
                    const int s = i % KT_STAGES, ts = i % KT_T;
                    if (!mbar_wait_bounded(bar(KB_T_FULL + ts), (i / KT_T) & 1)) { ok = false; break; }   // implies the stage's X
                    tc_fence_after_sync();
                    const uint32_t a_hi = tmem + ts * 64, a_lo = a_hi + 32;   // W^T: lane = output column, column = k
                    const uint32_t xb = stage_addr(s) + KT_W_BYTES;
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        const uint64_t bx = desc_x | (uint64_t)(((xb + ks * 32) & 0x3FFFFu) >> 4);
                        tc_mma_ts_tf32(d, a_hi + ks * 8, bx, idesc_hi, (!issued && ks == 0) ? 0u : 1u);
                    }
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        const uint64_t bx = desc_x | (uint64_t)(((xb + ks * 32) & 0x3FFFFu) >> 4);
                        tc_mma_ts_tf32(d + MP, a_lo + ks * 8, bx, idesc_lo, 1u);
                    }
                    issued = true;
                    // one barrier per block serves both rings: the converters wait on it for the tensor-memory slot of
                    // block i + 4, the producer for the shared-memory stage of block i + 8
                    tc_commit(bar(KB_EMPTY + s));
                }
                if (!ok) break;
                // every issuer arrives once per chunk — through the tensor pipe when it has MMAs in flight for it
                if (issued) tc_commit(bar(KB_CHUNK_FULL + cb));
                else mbar_arrive(bar(KB_CHUNK_FULL + cb));
            }
            if (!ok) kt_report(a.err, KERR_MMA);
        }
    } else {
        // ----------------------------------------------------- converters + drain
        // Two groups of four warps (each covers the four lane quarters of tensor memory): warps 2-5 convert the even
        // k-blocks, warps 6-9 the odd ones and, between two of theirs, drain the accumulator chunks.  In-kernel time
        // stamps of the version with ONE converter group (and four drain warps that idled seven blocks out of
        // eight) showed the conversion as the whole critical path: 1.4 k cycles per k-block, serial in its waits —
        // barrier, 32 shared-memory loads, the tensor-memory stores and their completion — against 0.5 k of MMA
        // issue, with the weight tiles in shared memory eight blocks ahead.
        const int grp = warp >= 6 ? 1 : 0;
        const int ct = threadIdx.x - 64 - grp * 128;  // 0..127 inside the group
        const int t_n = 32 * (warp & 3) + lane;       // the output column this thread carries into its TMEM lane
        const uint32_t st_lane = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        bool ok = true;
        auto drain = [&](int ci) -> bool {
            const int cb = ci & 1;
            if (!mbar_wait_warp_bounded(bar(KB_CHUNK_FULL + cb), (ci >> 1) & 1)) { kt_report(a.err, KERR_DRAIN); return false; }
            tc_fence_after_sync();
            const uint32_t abuf = st_lane + KT_ACC_COL + cb * (4 * MP);
            // a chunk of a single k-block (the tail of a slice) leaves the second set untouched: stale columns
            const bool two = min(nkb, (ci + 1) * KT_CHUNK) - ci * KT_CHUNK >= 2;
            if (MP == 32) {
                uint32_t r0[32], r1[32], r2[32], r3[32];   // set 0: hi.hi, corrections; set 1: the same
                tmem_ld_32x32(abuf, r0);
                tmem_ld_32x32(abuf + 32, r1);
                tmem_ld_32x32(abuf + 64, r2);
                tmem_ld_32x32(abuf + 96, r3);
                tmem_ld_wait();
                tc_fence_before_sync();
                mbar_arrive(bar(KB_CHUNK_EMPTY + cb));
#pragma unroll
                for (int m = 0; m < MP; ++m)
                    acc[m] += two ? (__uint_as_float(r1[m & 31]) + __uint_as_float(r3[m & 31])) + (__uint_as_float(r0[m & 31]) + __uint_as_float(r2[m & 31]))
                                  : __uint_as_float(r1[m & 31]) + __uint_as_float(r0[m & 31]);
            } else {
                uint32_t r0[32], r1[32];   // MP = 16: a set is 32 columns
                tmem_ld_32x32(abuf, r0);
                tmem_ld_32x32(abuf + 32, r1);
                tmem_ld_wait();
                tc_fence_before_sync();
                mbar_arrive(bar(KB_CHUNK_EMPTY + cb));
#pragma unroll
                for (int m = 0; m < MP; ++m)
                    acc[m] += two ? (__uint_as_float(r0[(MP + m) & 31]) + __uint_as_float(r1[(MP + m) & 31])) +
                                        (__uint_as_float(r0[m & 31]) + __uint_as_float(r1[m & 31]))
                                  : __uint_as_float(r0[(MP + m) & 31]) + __uint_as_float(r0[m & 31]);
            }
            return true;
        };
        int drained = 0;
        for (int i = grp; i < nkb && ok; i += 2) {
            // a chunk whose last block lies two blocks back has been through the tensor pipe (or is about to): it is
            // drained here, a whole chunk before the MMA issuer needs its buffer again
            while (grp == 1 && ok && drained < nchunks && (drained + 1) * KT_CHUNK + 1 <= i) ok = drain(drained++);
            if (!ok) break;
            const int s = i % KT_STAGES, n = i / KT_STAGES;
            if (!kt_wait_warp(bar(KB_RAW + s), n & 1)) { kt_report(a.err, KERR_CONVERT); ok = false; break; }
            const int ts = i % KT_T;
            // the tensor-memory slot is free when the MMAs of block i - 4 have retired (barrier of that block's stage)
            if (i >= KT_T && !kt_wait_warp(bar(KB_EMPTY + (i - KT_T) % KT_STAGES), ((i - KT_T) / KT_STAGES) & 1)) {
                kt_report(a.err, KERR_CONVERT);
                ok = false;
                break;
            }
            tc_fence_after_sync();
            const uint32_t st = stage_addr(s);
            uint32_t hi[32], lo[32];
#pragma unroll
            for (int k = 0; k < 32; ++k)
                asm volatile("ld.shared.b32 %0, [%1];" : "=r"(hi[k]) : "r"(st + (uint32_t)k * 512u + (uint32_t)t_n * 4u));
            kt_split<X_BYTES / 16 / 128>(st + KT_W_BYTES, X_BYTES, ct);
#pragma unroll
            for (int k = 0; k < 32; ++k)
                lo[k] = (__float_as_uint(__uint_as_float(hi[k]) - __uint_as_float(hi[k] & 0xFFFFE000u)) + 0x1000u) & 0xFFFFE000u;
            tmem_st_32x32(st_lane + ts * 64, hi);
            tmem_st_32x32(st_lane + ts * 64 + 32, lo);
            tmem_st_wait();
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // X lo, for the MMA's shared-memory reads
            tc_fence_before_sync();
            mbar_arrive(bar(KB_T_FULL + ts));
        }
        while (grp == 1 && ok && drained < nchunks) ok = drain(drained++);
    }

    // ------------------------------------------------------------ reduce + epilogue
    grid_dep_wait();   // Y and the bias are touched only after the kernel before this one has finished
    if (nslices == 1) {
        if (warp >= 6 && warp < 10 && n0 + t_row < a.N) {
#pragma unroll
            for (int m = 0; m < MP; ++m)
                if (m < a.M) a.Y[(int64_t)m * a.N + n0 + t_row] = kt_epilogue(a, acc[m], m, n0 + t_row);
        }
    } else {
        // The ring is idle (every MMA of this CTA has completed before the last chunk was drained): it carries this
        // slice's partial sums [MP][128].  Slice r finishes rows r, r + nslices, ...: its converter and drain warps
        // take one (row, four columns) item each and fetch the four values of every slice with ONE 128-bit load per
        // slice, all in flight together, and add them in slice order (bitwise deterministic).  One value per load,
        // one load after the other — the first version — cost a round trip per term; pushing the sums with remote
        // stores instead cost 2.8 us for 32 scalar stores per thread.
        float *red = reinterpret_cast<float *>(base_ptr + 1024);
        __syncthreads();
        if (warp >= 6 && warp < 10) {
#pragma unroll
            for (int m = 0; m < MP; ++m) red[m * KT_BN + t_row] = acc[m];
        }
        cluster_sync_all();
        if (warp >= 2 && warp < 10) {
            const int rows_owned = (a.M - slice + nslices - 1) / nslices;
            for (int it = threadIdx.x - 64; it < rows_owned * 32; it += 256) {
                const int m = slice + (it >> 5) * nslices, c4 = (it & 31) * 4;
                const uint32_t local = smem_u32(red + m * KT_BN + c4);
                float4 v[8];
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    v[q] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (q < nslices)
                        asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                                     : "=f"(v[q].x), "=f"(v[q].y), "=f"(v[q].z), "=f"(v[q].w)
                                     : "r"(map_to_cta(local, (uint32_t)q)));
                }
                float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int q = 0; q < 8; ++q)
                    if (q < nslices) { sum.x += v[q].x; sum.y += v[q].y; sum.z += v[q].z; sum.w += v[q].w; }
                const int64_t col = n0 + c4;
                const float out4[4] = { sum.x, sum.y, sum.z, sum.w };
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (col + e < a.N) a.Y[(int64_t)m * a.N + col + e] = kt_epilogue(a, out4[e], m, col + e);
            }
        }
        cluster_sync_all();   // the peers' shared memory must outlive the reads above
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, 512);
    }
}

// ---------------------------------------------------------------------- host

bool skinny_tc_applicable(int64_t M, int64_t N, int64_t K, const float *X, const float *W)
{
    // TMA reads X and W in place: rows must be multiples of 16 bytes on 16-byte aligned bases
    const uintptr_t align = reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(W);
    return M >= 1 && M <= 32 && N % 4 == 0 && K % 4 == 0 && (align & 15) == 0 && N >= 128 && K >= 256 &&
           N <= INT32_MAX && K <= INT32_MAX;
}

template <int MP>
static int launch_inst(const SkinnyTcMaps &tm, const SkinnyArgs &a, int kb_total, dim3 grid, cudaStream_t st)
{
    const size_t smem = 1024 + (size_t)KT_STAGES * (KT_W_BYTES + 2 * MP * 128) + 1024;
    auto kern = skinny_tc_kernel<MP>;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        attr_set[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(KT_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 1;
    at[0].val.clusterDim.y = grid.y;   // all K-slices of a column tile
    at[0].val.clusterDim.z = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // may start under the skinny call before it
    at[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = a.pdl ? 2 : 1;
    return (int)cudaLaunchKernelEx(&cfg, kern, tm, a, kb_total);
}

int launch_skinny_tc(const SkinnyArgs &a, int sm_count, cudaStream_t st)
{
    const int mp = a.M <= 16 ? 16 : 32;
    SkinnyTcMaps tm;
    int e = encode_f32_matrix_tmap(&tm.w, a.W, a.K, a.N, a.N, KT_BN, KT_KB);
    if (!e) e = encode_f32_batched_tmap(&tm.x, a.X, 1, a.M, a.K, a.K, mp, false);
    if (e) return e;
    const int tiles = (int)((a.N + KT_BN - 1) / KT_BN);
    const int kb_total = (int)((a.K + KT_KB - 1) / KT_KB);
    // K-slices: fill the GPU once, at most 8 per cluster, at least one accumulator chunk each
    int slices = sm_count / tiles;
    if (slices > 8) slices = 8;
    if (slices > kb_total / KT_CHUNK) slices = kb_total / KT_CHUNK;
    if (slices < 1) slices = 1;
    dim3 grid((unsigned)tiles, (unsigned)slices);
    return mp == 16 ? launch_inst<16>(tm, a, kb_total, grid, st) : launch_inst<32>(tm, a, kb_total, grid, st);
}

}  // namespace axb
