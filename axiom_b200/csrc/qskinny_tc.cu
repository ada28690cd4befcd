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
// One CTA = 128 weight rows x one K-slice; the K-slices of a tile form a thread-block cluster and are added
// through distributed shared memory.  Warp 0 is the TMA producer (a ring of 16 KB weight tiles plus the digit
// tiles, ~190 KB in flight per SM), warp 1 issues the MMAs, warps 2-5 read the accumulator and run the epilogue.
#include "qskinny_tc.cuh"

#include "gemm_tc.cuh"
#include "ptx.cuh"

#include <cuda.h>
#include <math.h>

namespace axb {

static constexpr int QT_THREADS = 192;
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
};

enum { QERR_PRODUCER = 31, QERR_MMA = 32, QERR_DRAIN = 33 };

__host__ __device__ constexpr int qt_stages(int mp)
{
    return mp <= 8 ? 10 : mp <= 16 ? 8 : mp <= 32 ? 6 : 4;   // (16 KB + 4*mp*128) * stages <= 200 KB
}

// ------------------------------------------------------------------------------------------------ pre-pass
// One CTA per activation row: largest magnitude, then the four digit planes digits[j][m][k] and 2^-s.
__global__ void __launch_bounds__(256) qx_digits_kernel(const float *__restrict__ a, int K, int MP,
                                                        int8_t *__restrict__ digits, float *__restrict__ inv_s)
{
    __shared__ float wmax[8];
    const int m = blockIdx.x, tid = threadIdx.x;
    grid_dep_launch();   // the tensor-core kernel may start streaming weights now; it waits before it reads the digits
    const float4 *row = reinterpret_cast<const float4 *>(a + (int64_t)m * K);
    const int k4n = K >> 2;
    float mx = 0.0f;
    bool bad = false;
    for (int i = tid; i < k4n; i += 256) {
        const float4 v = __ldg(row + i);
        const float t = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
        bad |= !(v.x - v.x == 0.0f) | !(v.y - v.y == 0.0f) | !(v.z - v.z == 0.0f) | !(v.w - v.w == 0.0f);
        mx = fmaxf(mx, t);
    }
    if (bad) mx = INFINITY;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    if ((tid & 31) == 0) wmax[tid >> 5] = mx;
    __syncthreads();
    mx = wmax[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) mx = fmaxf(mx, wmax[w]);

    const bool finite = mx < INFINITY;
    int sexp = 0;
    if (mx > 0.0f && finite) {
        const int e = (int)(__float_as_uint(mx) >> 23) - 127;   // floor(log2 mx) for normal mx
        sexp = min(29 - e, 126);
    }
    const float s = finite ? __uint_as_float((uint32_t)(sexp + 127) << 23) : 0.0f;
    // a row with an infinity or a NaN comes out as NaN
    if (tid == 0) inv_s[m] = finite ? __uint_as_float((uint32_t)(127 - sexp) << 23) : __int_as_float(0x7FC00000);

    const size_t plane = (size_t)MP * K;
    uint32_t *dst = reinterpret_cast<uint32_t *>(digits + (size_t)m * K);
    for (int i = tid; i < k4n; i += 256) {
        const float4 v = __ldg(row + i);
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
        for (int j = 0; j < 4; ++j) dst[(j * plane >> 2) + i] = pk[j];
    }
}

// ------------------------------------------------------------------------------------------------ main kernel
__device__ __forceinline__ void qt_report(int *err, int code)
{
    if (err) atomicCAS(err, 0, code);
}

__device__ __forceinline__ float qt_finish(const QtArgs &a, long long total, int m, int64_t col)
{
    float v = (float)((double)total * (double)__ldg(a.inv_s + m) * (double)__ldg(a.scales + col));
    if (a.bias) v += __ldg(a.bias + col);
    if (a.act == 1) v = fmaxf(v, 0.0f);
    else if (a.act == 2) v = 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
    return v;
}

template <int MP>
__global__ void __launch_bounds__(QT_THREADS, 1) qskinny_tc_kernel(const __grid_constant__ QtMaps tm, const QtArgs a,
                                                                   int kb_total)
{
    constexpr int NB = 4 * MP;                                   // MMA N: digit plane j, row m at column j*MP + m
    constexpr uint32_t X_BYTES = NB * 128;
    constexpr uint32_t STAGE = QT_W_BYTES + X_BYTES;
    constexpr int STAGES = qt_stages(MP);
    constexpr uint32_t TCOLS = NB < 32 ? 32 : NB;
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

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar(B_FULL + s), 1);
            mbar_init(bar(B_EMPTY + s), 1);
        }
        mbar_init(bar(B_ACC), 1);
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(base + 512, TCOLS);
        tmem_relinquish();
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&tm.w);
        tma_prefetch_desc(&tm.x);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    const int t_row = 32 * (warp & 3) + lane;   // drain warps: TMEM lane = weight row of the tile
    long long *red = reinterpret_cast<long long *>(base_ptr + 1024);   // [MP][128], over the idle ring

    if (warp == 0) {
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            // The weights do not depend on the digit pre-pass: the first ring of weight tiles is requested before
            // this kernel waits for it, so the pre-pass and the launch overlap the first HBM round trips.
            const int pre = min(nkb, STAGES);
            for (int i = 0; i < pre; ++i) {
                mbar_arrive_expect_tx(bar(B_FULL + i), STAGE);
                tma_load_3d(stage_addr(i), &tm.w, bar(B_FULL + i), (kb0 + i) * QT_KB, (int32_t)n0, 0);
            }
            grid_dep_wait();
            for (int i = 0; i < pre; ++i)
                tma_load_3d(stage_addr(i) + QT_W_BYTES, &tm.x, bar(B_FULL + i), (kb0 + i) * QT_KB, 0, 0);
            for (int i = pre; i < nkb; ++i) {
                const int s = i % STAGES, n = i / STAGES;
                if (!mbar_wait_bounded(bar(B_EMPTY + s), (n - 1) & 1)) { qt_report(a.err, QERR_PRODUCER); break; }
                const uint32_t st = stage_addr(s);
                const int k0 = (kb0 + i) * QT_KB;
                mbar_arrive_expect_tx(bar(B_FULL + s), STAGE);
                tma_load_3d(st, &tm.w, bar(B_FULL + s), k0, (int32_t)n0, 0);
                tma_load_3d(st + QT_W_BYTES, &tm.x, bar(B_FULL + s), k0, 0, 0);
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------- MMA issuer
        if (lane == 0) {
            const uint64_t desc = smem_desc_kmajor(0, 128);
            const uint32_t idesc = make_idesc<KIND_I8>(QT_BN, NB);
            bool ok = true;
            uint32_t accf = 0u;
            for (int i = 0; i < nkb; ++i) {
                const int s = i % STAGES;
                if (!mbar_wait_bounded(bar(B_FULL + s), (i / STAGES) & 1)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t st = stage_addr(s);
#pragma unroll
                for (int ks = 0; ks < QT_KB / 32; ++ks) {
                    tc_mma<KIND_I8>(tmem, desc | (uint64_t)(((st + ks * 32) & 0x3FFFFu) >> 4),
                                    desc | (uint64_t)(((st + QT_W_BYTES + ks * 32) & 0x3FFFFu) >> 4), idesc, accf);
                    accf = 1u;
                }
                tc_commit(bar(B_EMPTY + s));
            }
            if (ok && nkb > 0) tc_commit(bar(B_ACC));
            if (!ok) qt_report(a.err, QERR_MMA);
        }
    } else {
        // --------------------------------------------------------------- drain
        const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        grid_dep_wait();   // the row scales come from the pre-pass
        bool have = nkb > 0;
        if (have && !mbar_wait_warp_bounded(bar(B_ACC), 0)) {
            qt_report(a.err, QERR_DRAIN);
            have = false;
        }
        tc_fence_after_sync();
        const bool col_ok = n0 + t_row < a.N;
#pragma unroll 1
        for (int g = 0; g < MP / 8; ++g) {
            uint32_t d[4][8];
            if (have) {
#pragma unroll
                for (int j = 0; j < 4; ++j) tmem_ld_32x32_x8(lane_base + (uint32_t)(j * MP + 8 * g), d[j]);
                tmem_ld_wait();
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
#pragma unroll
                    for (int u = 0; u < 8; ++u) d[j][u] = 0u;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int m = 8 * g + u;
                const long long total = (long long)(int)d[0][u] + ((long long)(int)d[1][u] << 8) +
                                        ((long long)(int)d[2][u] << 16) + ((long long)(int)d[3][u] << 24);
                if (nslices == 1) {
                    if (m < a.M && col_ok) a.out[(int64_t)m * a.N + n0 + t_row] = qt_finish(a, total, m, n0 + t_row);
                } else {
                    red[m * QT_BN + t_row] = total;   // every MMA of this CTA has completed: the ring is idle
                }
            }
        }
        tc_fence_before_sync();
    }

    if (nslices > 1) {
        cluster_sync_all();
        if (warp >= 2 && n0 + t_row < a.N) {
            // slice r finishes rows r, r + nslices, ...: integer sums straight out of the peers' shared memory
            for (int m = slice; m < a.M; m += nslices) {
                const uint32_t local = smem_u32(red + m * QT_BN + t_row);
                long long s = 0;
                for (int q = 0; q < nslices; ++q) {
                    long long v;
                    asm volatile("ld.shared::cluster.b64 %0, [%1];" : "=l"(v) : "r"(map_to_cta(local, (uint32_t)q)));
                    s += v;
                }
                a.out[(int64_t)m * a.N + n0 + t_row] = qt_finish(a, s, m, n0 + t_row);
            }
        }
        cluster_sync_all();   // the peers' shared memory must outlive the reads above
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

template <int MP>
static int launch_inst(const QtMaps &tm, const QtArgs &a, int kb_total, dim3 grid, cudaStream_t st)
{
    const size_t smem = 1024 + (size_t)qt_stages(MP) * (QT_W_BYTES + 4 * MP * 128) + 1024;
    auto kern = qskinny_tc_kernel<MP>;
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
    cfg.numAttrs = 2;
    return (int)cudaLaunchKernelEx(&cfg, kern, tm, a, kb_total);
}

int launch_qskinny_tc(const float *act_in, const int8_t *q, const float *scales, const float *bias, int act, float *out,
                      int64_t M, int64_t N, int64_t K, void *workspace, int *err, int sm_count, cudaStream_t st)
{
    const int mp = M <= 8 ? 8 : M <= 16 ? 16 : M <= 32 ? 32 : 64;
    float *inv_s = reinterpret_cast<float *>(workspace);
    int8_t *digits = reinterpret_cast<int8_t *>(workspace) + 1024;
    qx_digits_kernel<<<(unsigned)M, 256, 0, st>>>(act_in, (int)K, mp, digits, inv_s);
    int e = (int)cudaGetLastError();
    if (e) return e;

    QtMaps tm;
    e = encode_i8_batched_tmap(&tm.w, q, 1, N, K, K, N * K, QT_BN, 1);
    if (!e) e = encode_i8_batched_tmap(&tm.x, digits, 4, M, K, K, (int64_t)mp * K, mp, 4);
    if (e) return e;
    QtArgs a;
    a.scales = scales; a.bias = bias; a.inv_s = inv_s; a.out = out; a.err = err; a.M = (int)M; a.N = N; a.act = act;
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
    switch (mp) {
    case 8: return launch_inst<8>(tm, a, kb_total, grid, st);
    case 16: return launch_inst<16>(tm, a, kb_total, grid, st);
    case 32: return launch_inst<32>(tm, a, kb_total, grid, st);
    default: return launch_inst<64>(tm, a, kb_total, grid, st);
    }
}

}  // namespace axb
