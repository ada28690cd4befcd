// qskinny_tc.cu — W8A32 for skinny activations on the integer tensor cores:
//     out[m,n] = act(scale[n] * sum_k a[m,k] * q[n,k] + bias[n]),   1 <= M <= 64.
//
// The reference multiplies fp32 activations into int8 weights with fp32 FMAs (src/core/quantize.c:100-177).  A
// GEMV written that way is paced by instruction issue and shared-memory reads as soon as M > 1: every weight byte
// costs a conversion and M FMAs.  Here the activations are put on a fixed-point grid instead: a pre-pass scales
// each activation row by a power of two so that its largest element lies in [2^29, 2^30), rounds to a 32-bit
// integer (absolute error <= 2^-30 of the row's largest element — finer than the fp32 rounding of the
// reference's products) and writes the four signed base-256 digits of that integer as four int8 planes.  Then
//     sum_k a*q = 2^-s * sum_j 256^j * (digit_j . q)
// and every digit_j . q is an int8 x int8 -> s32 product for tcgen05.mma kind::i8, exact.  The weights go from
// HBM to shared memory by TMA and from there straight into the MMA: no conversion, no register traffic, two
// shared-memory passes per weight byte.  The product is computed transposed — the 128 rows of the MMA are 128
// weight rows (output columns), its N the 4 x M digit rows — and accumulates in tensor memory over the whole K
// range of the CTA; the digits are recombined in 64-bit integers, so the result does not depend on how K is cut
// into slices or in which order the slices are added.
//
// One CTA = 128 weight rows x one K-slice; the K-slices of a tile form a thread-block cluster: every slice stores
// its integer partial sums of row m into the shared memory of slice m mod nslices, one cluster barrier, and each
// slice finishes the rows it owns.  Warp 0 is the TMA producer (a ring of 16 KB weight tiles plus the digit
// tiles, ~190 KB in flight per SM), warp 1 issues the MMAs, warps 2-17 read the accumulator and run the epilogue.
#include "qskinny_tc.cuh"

#include "gemm_tc.cuh"
#include "ptx.cuh"

#include <cuda.h>
#include <math.h>
#include <string.h>

namespace axb {

static constexpr int QT_THREADS = 608;   // warp 0: TMA producer, 1 and 18: MMA issuers, 2..17: drain
static constexpr int QT_BN = 128;                    // weight rows per CTA
static constexpr int QT_KB = 128;                    // k per stage: one 128-byte swizzled row
static constexpr int QT_W_BYTES = QT_BN * QT_KB;     // 16 KB

struct alignas(64) QtMaps {
    CUtensorMap w, x;
};

struct QtArgs {
    const float *scales, *bias, *inv_s;
    float *out;
    int *err;
    int M;
    int64_t N;
    int act;
    const float *x;   // FUSED kernels: the fp32 activations [M][K] themselves (no digit planes in memory)
    int K;
};

enum { QERR_PRODUCER = 31, QERR_MMA = 32, QERR_DRAIN = 33 };


__host__ __device__ constexpr int qt_stages(int mp)
{
    // (16 KB + 4*mp*128) * stages + (mp + 8) KB for the partial sums of the other K-slices <= 224 KB
    return mp <= 8 ? 10 : mp <= 16 ? 8 : mp <= 32 ? 5 : 3;
}

// ------------------------------------------------------------------------------------------------ pre-pass
// One CTA per activation row: largest magnitude, then the four digit planes digits[j][m][k] and 2^-s.  The row
// stays in registers between the two steps (up to 16384 elements; longer rows are read again), so the pre-pass
// costs one trip to memory, a block reduction and the stores.
// QX_THREADS x QX_CACHE float4 = 16384 elements stay in registers.  1024 threads: lowest latency for the few rows of
// the skinny kernel; 256 threads (eight CTAs per SM): one wave for the hundreds of rows of the GEMM route.
static constexpr int QX_CACHED_F4 = 4096;

__device__ __forceinline__ void qx_emit(uint32_t *dst, size_t plane4, int i, const float4 &v, float s)
{
    const float x[4] = { v.x, v.y, v.z, v.w };
    uint32_t pk[4] = { 0u, 0u, 0u, 0u };
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        int t = __float2int_rn(x[e] * s);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int d = (int)(int8_t)(t & 0xFF);
            t = (t - d) >> 8;
            pk[j] |= (uint32_t)(d & 0xFF) << (8 * e);
        }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) dst[j * plane4 + i] = pk[j];
}

__device__ __forceinline__ float qx_absmax(const float4 &v, bool &bad)
{
    bad |= !(v.x - v.x == 0.0f) | !(v.y - v.y == 0.0f) | !(v.z - v.z == 0.0f) | !(v.w - v.w == 0.0f);
    return fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
}

// MP > 0: digit plane j of row m at (j * MP + m) * K (four planes of MP rows); MP == 0: the four digit rows of a row
// side by side, digit j of row m at (4 * m + j) * K
template <int QX_THREADS>
__global__ void __launch_bounds__(QX_THREADS) qx_digits_kernel(const float *__restrict__ a, int K, int MP,
                                                               int8_t *__restrict__ digits, float *__restrict__ inv_s)
{
    constexpr int QX_CACHE = QX_CACHED_F4 / QX_THREADS;
    __shared__ float wmax[32];
    const int m = blockIdx.x, tid = threadIdx.x;
    grid_dep_launch();   // the tensor-core kernel may start streaming weights now; it waits before it reads the digits
    const float4 *row = reinterpret_cast<const float4 *>(a + (int64_t)m * K);
    const int k4n = K >> 2;
    float4 v[QX_CACHE];
    float mx = 0.0f;
    bool bad = false;
#pragma unroll
    for (int r = 0; r < QX_CACHE; ++r) {
        const int i = tid + QX_THREADS * r;
        v[r] = i < k4n ? __ldg(row + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int r = 0; r < QX_CACHE; ++r) mx = fmaxf(mx, qx_absmax(v[r], bad));
    for (int i = tid + QX_THREADS * QX_CACHE; i < k4n; i += QX_THREADS) mx = fmaxf(mx, qx_absmax(__ldg(row + i), bad));
    if (bad) mx = INFINITY;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    if ((tid & 31) == 0) wmax[tid >> 5] = mx;
    __syncthreads();
    mx = (tid & 31) < QX_THREADS / 32 ? wmax[tid & 31] : 0.0f;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));

    const bool finite = mx < INFINITY;
    int sexp = 0;
    if (mx > 0.0f && finite) {
        const int e = (int)(__float_as_uint(mx) >> 23) - 127;   // floor(log2 mx) for normal mx
        sexp = min(29 - e, 126);
    }
    const float s = finite ? __uint_as_float((uint32_t)(sexp + 127) << 23) : 0.0f;
    // a row with an infinity or a NaN comes out as NaN
    if (tid == 0) inv_s[m] = finite ? __uint_as_float((uint32_t)(127 - sexp) << 23) : __int_as_float(0x7FC00000);

    const size_t plane4 = MP > 0 ? ((size_t)MP * K) >> 2 : (size_t)K >> 2;
    uint32_t *dst = reinterpret_cast<uint32_t *>(digits + (size_t)m * K * (MP > 0 ? 1 : 4));
#pragma unroll
    for (int r = 0; r < QX_CACHE; ++r) {
        const int i = tid + QX_THREADS * r;
        if (i < k4n) qx_emit(dst, plane4, i, v[r], s);
    }
    for (int i = tid + QX_THREADS * QX_CACHE; i < k4n; i += QX_THREADS) qx_emit(dst, plane4, i, __ldg(row + i), s);
}

// ------------------------------------------------------------------------------------------------ main kernel
__device__ __forceinline__ void qt_report(int *err, int code)
{
    if (err) atomicCAS(err, 0, code);
}

// FUSED (used up to 4 rows): no digit pre-pass.  The sixteen drain warps, idle while the weights stream, make the digits
// themselves: every CTA finds the rows' largest magnitudes (M x K floats out of L2), then the warp that owns ring stage w
// writes the digit tiles of k-blocks w, w + stages, ... straight into the ring's X slots in the layout TMA would have left there (128-byte rows,
// 16-byte chunks XOR-ed with the row's low bits) and arrives on the stage's barrier beside the weight tile's bytes.
// One launch instead of two, and the ~2.7 us between the end of a pre-pass and the moment its dependents may read
// what it wrote are gone.
template <int MP, bool FUSED>
__global__ void __launch_bounds__(QT_THREADS, 1) qskinny_tc_kernel(const __grid_constant__ QtMaps tm, const QtArgs a,
                                                                   int kb_total)
{
    static_assert(!FUSED || MP == 8, "the fused digit maker serves the 8-row variant");
    constexpr int NB = 4 * MP;                                   // MMA N: digit plane j, row m at column j*MP + m
    constexpr uint32_t X_BYTES = NB * 128;
    constexpr uint32_t STAGE = QT_W_BYTES + X_BYTES;
    constexpr int STAGES = qt_stages(MP);
    // two MMA issuers with an accumulator set each up to 32 rows; at 64 rows (N = 256) the MMAs themselves fill the
    // issuing thread's time and a second set only lengthens the drain (measured: 26.5 us against 24.6)
    constexpr bool TWO = MP <= 32;
    constexpr uint32_t TCOLS = (TWO ? 2 : 1) * NB < 32 ? 32 : (TWO ? 2 : 1) * NB;
    enum { B_FULL = 0, B_EMPTY = STAGES, B_ACC = 2 * STAGES };

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *base_ptr = smem_raw + (base - raw);
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(base_ptr + 512);
    auto bar = [&](int i) -> uint32_t { return base + 8u * (uint32_t)i; };
    auto stage_addr = [&](int s) -> uint32_t { return base + 1024u + (uint32_t)s * STAGE; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x, slice = blockIdx.y, nslices = gridDim.y;
    const int64_t n0 = (int64_t)tile * QT_BN;
    const int per = (kb_total + nslices - 1) / nslices;
    const int kb0 = slice * per;
    const int nkb = max(0, min(per, kb_total - kb0));
    const int pre = min(nkb, STAGES);
    auto kpos = [&](int i) -> int { return (kb0 + i) * QT_KB; };

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar(B_FULL + s), FUSED ? 2 : 1);   // the weight tile's bytes (+ the warp that wrote the digits)
            mbar_init(bar(B_EMPTY + s), 1);
        }
        if (FUSED) {
#pragma unroll
            for (int m = 0; m < 10; ++m) reinterpret_cast<volatile uint32_t *>(base_ptr + 576)[m] = 0u;   // row maxima, bad-row mask
        }
        mbar_init(bar(B_ACC), TWO ? 2 : 1);   // one arrival per MMA issuer
        mbar_fence_init();
        // The weights depend on nothing this call computes: the first ring of weight tiles is requested before
        // anything else happens in this CTA — before tensor memory is allocated and long before the digits of the
        // pre-pass (which may still be running: this kernel is its programmatic dependent) are needed.
        tma_prefetch_desc(&tm.w);
        for (int i = 0; i < pre; ++i) {
            mbar_arrive_expect_tx(bar(B_FULL + i), FUSED ? QT_W_BYTES : STAGE);
            tma_load_3d(stage_addr(i), &tm.w, bar(B_FULL + i), kpos(i), (int32_t)n0, 0);
        }
        if (FUSED) grid_dep_launch();   // a call queued behind this one may request ITS weights now
        else tma_prefetch_desc(&tm.x);
    }
    if (warp == 1) {
        tmem_alloc(base + 512, TCOLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    // drain warps 2..17: TMEM lane quadrant warp & 3 (four warps per quadrant, `quarter` tells them apart)
    const int t_row = 32 * (warp & 3) + lane;   // TMEM lane = weight row of the tile
    const int quarter = (warp - 2) >> 2;
    const int64_t col = n0 + t_row;
    const bool col_ok = col < a.N;
    float col_scale = 0.0f, col_bias = 0.0f;    // inputs of the call, not of the pre-pass: loaded ahead of the K loop
    if (!FUSED && warp >= 2 && warp < 18 && col_ok) {
        col_scale = __ldg(a.scales + col);
        if (a.bias) col_bias = __ldg(a.bias + col);
    }
    float *s_inv = reinterpret_cast<float *>(base_ptr + 256);   // 2^-s per activation row
    // Partial sums of the other K-slices arrive here, behind the ring (a peer may be done while this CTA still
    // streams): recv[source slice][row owned by this CTA][weight row of the tile]
    long long *recv = reinterpret_cast<long long *>(base_ptr + 1024 + STAGES * STAGE);
    const int rows_owned = (a.M + nslices - 1) / nslices;

    if (warp == 0) {
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            if (!FUSED) {
                grid_dep_wait();   // the digits
                for (int i = 0; i < pre; ++i)
                    tma_load_3d(stage_addr(i) + QT_W_BYTES, &tm.x, bar(B_FULL + i), kpos(i), 0, 0);
            }
            for (int i = pre; i < nkb; ++i) {
                const int s = i % STAGES, n = i / STAGES;
                if (!mbar_wait_bounded(bar(B_EMPTY + s), (n - 1) & 1)) { qt_report(a.err, QERR_PRODUCER); break; }
                const uint32_t st = stage_addr(s);
                const int k0 = kpos(i);
                mbar_arrive_expect_tx(bar(B_FULL + s), FUSED ? QT_W_BYTES : STAGE);
                tma_load_3d(st, &tm.w, bar(B_FULL + s), k0, (int32_t)n0, 0);
                if (!FUSED) tma_load_3d(st + QT_W_BYTES, &tm.x, bar(B_FULL + s), k0, 0, 0);
            }
        }
    } else if (warp == 1 || warp == 18) {
        // --------------------------------------------------------- MMA issuers
        // Two threads, even and odd k-blocks, each into its own accumulator columns (the integer sums are added by the
        // drain warps): a k-block costs the issuing THREAD ~600 cycles — four MMAs at ~70, the commit ~120, barrier
        // and fence ~200 — while the tensor pipe needs a fraction of that, and with one issuer that, not the memory
        // system, paced the stream (16 KB per 0.4 us and SM: 5.1 TB/s over 128 SMs).
        if (lane == 0 && (TWO || warp == 1)) {
            const int par = warp == 1 ? 0 : 1;
            const uint64_t desc = smem_desc_kmajor(0, 128);
            const uint32_t idesc = make_idesc<KIND_I8>(QT_BN, NB);
            const uint32_t acc = tmem + (uint32_t)(par * NB);
            bool ok = true;
            uint32_t accf = 0u;
            for (int i = par; i < nkb; i += TWO ? 2 : 1) {
                const int s = i % STAGES;
                if (!mbar_wait_bounded(bar(B_FULL + s), (i / STAGES) & 1)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t st = stage_addr(s);
#pragma unroll
                for (int ks = 0; ks < QT_KB / 32; ++ks) {
                    tc_mma<KIND_I8>(acc, desc | (uint64_t)(((st + ks * 32) & 0x3FFFFu) >> 4),
                                    desc | (uint64_t)(((st + QT_W_BYTES + ks * 32) & 0x3FFFFu) >> 4), idesc, accf);
                    accf = 1u;
                }
                tc_commit(bar(B_EMPTY + s));
            }
            // both issuers arrive on the accumulator barrier: through the pipe when MMAs are in flight, plainly otherwise
            if (ok && accf) tc_commit(bar(B_ACC));
            else if (ok) mbar_arrive(bar(B_ACC));
            if (!ok) qt_report(a.err, QERR_MMA);
        }
    } else if (warp < 18) {
        // --------------------------------------------------------------- drain
        const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        grid_dep_wait();   // the row scales come from the pre-pass (FUSED: the activations from the kernel before)
        const int dt = threadIdx.x - 64;
        if constexpr (FUSED) {
            if (col_ok) {
                col_scale = __ldg(a.scales + col);
                if (a.bias) col_bias = __ldg(a.bias + col);
            }
            // ---- the rows' largest magnitudes (every CTA for itself: M x K floats, L2 hits after the first CTA)
            uint32_t *s_maxbits = reinterpret_cast<uint32_t *>(base_ptr + 576);   // [8] |x| bit patterns, [8] bad-row mask
            float *s_mul = reinterpret_cast<float *>(base_ptr + 640);             // [8] 2^s
            const int K = a.K, k4n = K >> 2;
            {
                // all rows' loads of a step are issued together: row after row, each row's loads waited for the previous
                // row's reduction and the pass took one trip to L2 per row
                float mx[MP];
                bool bad[MP];
#pragma unroll
                for (int m = 0; m < MP; ++m) { mx[m] = 0.0f; bad[m] = false; }
                const float4 *x4 = reinterpret_cast<const float4 *>(a.x);
                for (int i = dt; i < k4n; i += 512) {
#pragma unroll
                    for (int m = 0; m < MP; ++m)
                        if (m < a.M) mx[m] = fmaxf(mx[m], qx_absmax(__ldg(x4 + (int64_t)m * k4n + i), bad[m]));
                }
#pragma unroll
                for (int m = 0; m < MP; ++m) {
                    if (m < a.M) {
                        float v = bad[m] ? INFINITY : mx[m];
#pragma unroll
                        for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
                        if (lane == 0) atomicMax(s_maxbits + m, __float_as_uint(v));   // non-negative floats order like their bits
                    }
                }
            }
            asm volatile("bar.sync 1, 512;" ::: "memory");
            if (dt < MP) {
                const float mx = __uint_as_float(s_maxbits[dt]);
                const bool finite = mx < INFINITY;
                int sexp = 0;
                if (mx > 0.0f && finite) {
                    const int e = (int)(__float_as_uint(mx) >> 23) - 127;   // floor(log2 mx) for normal mx
                    sexp = min(29 - e, 126);
                }
                s_mul[dt] = (finite && dt < a.M) ? __uint_as_float((uint32_t)(sexp + 127) << 23) : 0.0f;
                // a row with an infinity or a NaN comes out as NaN
                s_inv[dt] = dt < a.M ? (finite ? __uint_as_float((uint32_t)(127 - sexp) << 23) : __int_as_float(0x7FC00000)) : 0.0f;
            }
            asm volatile("bar.sync 1, 512;" ::: "memory");
            // ---- digit tiles: warp w < STAGES owns ring stage w and makes k-blocks w, w + STAGES, ... (one warp per
            // stage, so that it sees every release of its stage in turn: a waiter that skipped a phase would be fooled
            // by the barrier's parity); lane l makes the four k at 4l of every row
            const int w16 = warp - 2;
            for (int i = w16; i < nkb && w16 < STAGES; i += STAGES) {
                const int s = i % STAGES, n = i / STAGES;
                if (n >= 1) {
                    const bool got = mbar_wait_warp_bounded(bar(B_EMPTY + s), (n - 1) & 1);
                    if (!got) { qt_report(a.err, QERR_PRODUCER); break; }
                }
                const int k = kpos(i) + 4 * lane;
                uint8_t *xs = base_ptr + 1024 + (size_t)s * STAGE + QT_W_BYTES;
                const int chunk = lane >> 2, within = (lane & 3) * 4;
#pragma unroll
                for (int m = 0; m < MP; ++m) {
                    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                    const bool live = m < a.M && k < K;   // padding rows and the K tail are zero digits
                    if (live) v = __ldg(reinterpret_cast<const float4 *>(a.x + (int64_t)m * K + k));
                    const float sc = s_mul[m];
                    const float xv[4] = { v.x, v.y, v.z, v.w };
                    uint32_t pk[4] = { 0u, 0u, 0u, 0u };
#pragma unroll
                    for (int e = 0; e < 4 && live; ++e) {
                        int t = __float2int_rn(xv[e] * sc);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int d = (int)(int8_t)(t & 0xFF);
                            t = (t - d) >> 8;
                            pk[j] |= (uint32_t)(d & 0xFF) << (8 * e);
                        }
                    }
                    // row j*MP + m of the tile: its low three bits are m (MP == 8), the chunk index is XOR-ed with them
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        *reinterpret_cast<uint32_t *>(xs + (j * MP + m) * 128 + ((chunk ^ m) << 4) + within) = pk[j];
                }
                fence_proxy_async_smem();   // generic-proxy writes before the tensor core reads them
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(B_FULL + s));
            }
        } else {
            if (dt < MP) s_inv[dt] = dt < a.M ? __ldg(a.inv_s + dt) : 0.0f;
        }
        asm volatile("bar.sync 1, 512;" ::: "memory");   // the sixteen drain warps
        bool have = nkb > 0;
        if (have && !mbar_wait_warp_bounded(bar(B_ACC), 0)) {
            qt_report(a.err, QERR_DRAIN);
            have = false;
        }
        tc_fence_after_sync();
#pragma unroll 1
        for (int g = quarter; g < MP / 4; g += 4) {
            if (4 * g >= a.M) break;
            uint32_t d[4][4];
            if (have) {
#pragma unroll
                for (int j = 0; j < 4; ++j) tmem_ld_32x32_x4(lane_base + (uint32_t)(j * MP + 4 * g), d[j]);
                tmem_ld_wait();
                if (TWO && nkb >= 2) {   // the odd k-blocks' sums (|sum| of both stays below 2^31 for K <= 65536)
                    uint32_t e[4][4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) tmem_ld_32x32_x4(lane_base + (uint32_t)(NB + j * MP + 4 * g), e[j]);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 4; ++j)
#pragma unroll
                        for (int u = 0; u < 4; ++u) d[j][u] += e[j][u];
                }
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
#pragma unroll
                    for (int u = 0; u < 4; ++u) d[j][u] = 0u;
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int m = 4 * g + u;
                const long long total = (long long)(int)d[0][u] + ((long long)(int)d[1][u] << 8) +
                                        ((long long)(int)d[2][u] << 16) + ((long long)(int)d[3][u] << 24);
                if (m < a.M) {
                    if (nslices == 1) {
                        if (col_ok) a.out[(int64_t)m * a.N + col] = qt_finish(total, s_inv[m], col_scale, col_bias, a.act);
                    } else {
                        // to the slice that finishes row m (m mod nslices): a store into its shared memory
                        const int owner = m % nslices, r = m / nslices;
                        const uint32_t dst = map_to_cta(smem_u32(recv + (slice * rows_owned + r) * QT_BN + t_row), (uint32_t)owner);
                        asm volatile("st.shared::cluster.b64 [%0], %1;" ::"r"(dst), "l"(total) : "memory");
                    }
                }
            }
        }
        tc_fence_before_sync();
    }

    if (nslices > 1) {
        cluster_sync_all();   // release / acquire: every slice's partial sums have landed
        if (warp >= 2 && warp < 18 && col_ok) {
            // integer sums of the rows this slice owns, out of its own shared memory: nobody reads a peer after the
            // barrier, so a CTA may leave as soon as it is done
            for (int r = quarter; r < rows_owned; r += 4) {
                const int m = slice + r * nslices;
                if (m >= a.M) break;
                long long sum = 0;
#pragma unroll
                for (int q = 0; q < 8; ++q)
                    if (q < nslices) sum += recv[(q * rows_owned + r) * QT_BN + t_row];
                a.out[(int64_t)m * a.N + col] = qt_finish(sum, s_inv[m], col_scale, col_bias, a.act);
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, TCOLS);
    }
}

// ---------------------------------------------------------------------------------------------------- host

bool qskinny_tc_applicable(int64_t M, int64_t N, int64_t K, const float *a, const int8_t *q)
{
    const uintptr_t align = reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(q);
    // TMA reads the weight rows in place; the s32 accumulator holds |digit.q| <= 2^14 * K
    return M >= 1 && M <= 64 && K % 16 == 0 && K >= 128 && K <= 65536 && N >= 1 && N <= INT32_MAX && (align & 15) == 0;
}

size_t qskinny_tc_workspace_bytes(int64_t M, int64_t K)
{
    const int mp = M <= 8 ? 8 : M <= 16 ? 16 : M <= 32 ? 32 : 64;
    return (size_t)4 * mp * K + 1024;
}

template <int MP, bool FUSED = false>
static int launch_inst(const QtMaps &tm, const QtArgs &a, int kb_total, dim3 grid, cudaStream_t st, int pdl = 1)
{
    const size_t smem = 1024 + (size_t)qt_stages(MP) * (QT_W_BYTES + 4 * MP * 128) + (size_t)(MP + 8) * 1024 + 1024;
    auto kern = qskinny_tc_kernel<MP, FUSED>;
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
    cfg.blockDim = dim3(QT_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 1;
    at[0].val.clusterDim.y = grid.y;   // all K-slices of a tile
    at[0].val.clusterDim.z = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // may start under the digit pre-pass
    at[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = pdl ? 2 : 1;
    return (int)cudaLaunchKernelEx(&cfg, kern, tm, a, kb_total);
}

int launch_qx_digits(const float *act_in, int64_t M, int64_t K, int64_t plane_rows, int8_t *digits, float *inv_s,
                     cudaStream_t st)
{
    if (M <= 64) qx_digits_kernel<1024><<<(unsigned)M, 1024, 0, st>>>(act_in, (int)K, (int)plane_rows, digits, inv_s);
    else qx_digits_kernel<256><<<(unsigned)M, 256, 0, st>>>(act_in, (int)K, (int)plane_rows, digits, inv_s);
    return (int)cudaGetLastError();
}

int launch_qskinny_tc(const float *act_in, const int8_t *q, const float *scales, const float *bias, int act, float *out,
                      int64_t M, int64_t N, int64_t K, void *workspace, int *err, int sm_count, cudaStream_t st, int pdl)
{
    const int mp = M <= 8 ? 8 : M <= 16 ? 16 : M <= 32 ? 32 : 64;
    // up to four rows the tensor-core kernel makes the digits itself, one launch (measured against the pre-pass form,
    // W[16384 x 4096]: M = 1 13.6 - 14.0 against 16.4 us, M = 2 14.4 / 16.4, M = 4 15.5 / 16.5, M = 8 17.1 / 16.6 — every
    // CTA converts all the rows, and at eight rows that is no faster than one pre-pass for all)
    const bool fused = M <= 4;
    float *inv_s = reinterpret_cast<float *>(workspace);
    int8_t *digits = reinterpret_cast<int8_t *>(workspace) + 1024;
    int e = 0;
    if (!fused) {
        qx_digits_kernel<1024><<<(unsigned)M, 1024, 0, st>>>(act_in, (int)K, mp, digits, inv_s);
        e = (int)cudaGetLastError();
        if (e) return e;
    }
    QtMaps tm;
    memset(&tm, 0, sizeof tm);
    e = encode_i8_batched_tmap(&tm.w, q, 1, N, K, K, N * K, QT_BN, 1);
    if (!e && !fused) e = encode_i8_batched_tmap(&tm.x, digits, 4, M, K, K, (int64_t)mp * K, mp, 4);
    if (e) return e;
    QtArgs a;
    a.scales = scales; a.bias = bias; a.inv_s = inv_s; a.out = out; a.err = err; a.M = (int)M; a.N = N; a.act = act;
    a.x = act_in; a.K = (int)K;
    const int tiles = (int)((N + QT_BN - 1) / QT_BN);
    const int kb_total = (int)((K + QT_KB - 1) / QT_KB);
    // K-slices: fill the GPU once, at most 8 per cluster, at least two k-blocks each, none empty
    int slices = sm_count / tiles;
    if (slices > 8) slices = 8;
    if (slices > kb_total / 2) slices = kb_total / 2;
    if (slices < 1) slices = 1;
    const int per = (kb_total + slices - 1) / slices;
    slices = (kb_total + per - 1) / per;
    dim3 grid((unsigned)tiles, (unsigned)slices);
    if (fused) return launch_inst<8, true>(tm, a, kb_total, grid, st, pdl);
    switch (mp) {
    case 8: return launch_inst<8>(tm, a, kb_total, grid, st);
    case 16: return launch_inst<16>(tm, a, kb_total, grid, st);
    case 32: return launch_inst<32>(tm, a, kb_total, grid, st);
    default: return launch_inst<64>(tm, a, kb_total, grid, st);
    }
}

}  // namespace axb
