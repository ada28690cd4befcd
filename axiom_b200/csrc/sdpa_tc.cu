// sdpa_tc.cu — attention forward on the tensor cores, fp32 in / fp32 out, head dim <= 64:
//     O = softmax(scale * Q.K^T [+ causal mask]) . V,   L = rowmax + log(rowsum)
//
// Both contractions run as three tf32 products over hi/lo planes (lo.hi + hi.lo + hi.hi), which keeps the
// result at fp32 accuracy (the reference computes this path in fp32, src/compute/backends/cpu_opt.c:7828-8071;
// its CUDA path uses one TF32 product and a materialised S x S buffer, cuda/ops_attention.cu:224-392).
//
// A pre-pass splits Q, K and V into planes [BH][S][pitch].  One CTA owns 128 query rows of one head and walks
// the keys in blocks of 128:
//   warp 4  : TMA producer — the Q tile once, then one K and one V block at a time (128-byte swizzle; V with
//             the 32-byte-chunk variant, the one layout an MN-major tf32 operand may have);
//   warp 5  : one thread issues tcgen05.mma.  S_j = Q.K_j^T (M128 x N128, operands from shared memory, both
//             K-major) goes to one of two TMEM score buffers; O_j = P_j.V_j takes P from TENSOR MEMORY (the TS
//             form) and V as an MN-major shared-memory operand, i.e. exactly as the TMA load leaves it — V is
//             never transposed.  N = 128 runs the tf32 pipe at its full rate (N = 64 does not: measured 48
//             cycles per instruction instead of 32), which is why the key block is 128 wide;
//   warps 0-3: thread t owns query row t.  Pass 1 reads the score row from TMEM in 32-column chunks and takes
//             the maximum; pass 2 re-reads it, forms p = 2^(c*s - m), and writes P back as tf32 hi (over the
//             scores it came from) and lo (a third buffer).  Every block's O_j lands in a fresh accumulator
//             (the tensor core's truncating accumulation never spans more than one block) and is folded into
//             the thread's fp32 register row with the usual rescale.  The chunk loops are rolled: the body
//             stays small enough for the instruction cache, which a fully unrolled row (the first version)
//             did not — its warps spent most of their time waiting for instructions.
// The score matrix never leaves the SM.  Issue order S_0 S_1 O_0 S_2 O_1 ...: the pipe computes the next
// block's scores while the softmax warps work on this one; in-order execution of the MMAs is what makes the
// score buffer (aliased by P hi) safe to overwrite two blocks later.
#include "sdpa.cuh"

#include "gemm_tc.cuh"
#include "ptx.cuh"

#include <cuda.h>
#include <math.h>

namespace axb {

static constexpr int TQ = 128, TKV = 128, ST_THREADS = 192;
static constexpr int ST_HEADER = 1024;
static constexpr int SLAB = 128 * 128;  // bytes of one 32-column slab of a 128-row tile

struct alignas(64) SdpaTmaps {
    CUtensorMap q[2], k[2], v[2];  // hi, lo
};

struct SdpaTcArgs {
    float *O, *L;
    int S, dk, causal;
    float c_log2;   // scale * log2(e), > 0
    int ksteps_qk;  // ceil(dk / 8) MMA steps along the head dim
    int n_pv;       // dk rounded up to 16: the N of the P.V product
    int vec_out;    // O rows are 16-byte aligned: 128-bit stores
    int *err;
};

enum { SERR_PRODUCER = 11, SERR_MMA = 12, SERR_SOFTMAX = 13 };

__device__ __forceinline__ void report_err(int *err, int code)
{
    if (err) atomicCAS(err, 0, code);
}

enum {
    B_Q_FULL = 0, B_K_FULL = 1, B_K_EMPTY = 2, B_V_FULL = 3, B_V_EMPTY = 4,
    B_S_FULL = 5, B_P_FULL = 7, B_O_FULL = 9, B_O_EMPTY = 11, B_COUNT = 13
};

// TMEM columns: two score buffers (P hi is written over the scores), P lo, two output buffers
enum { T_S = 0, T_PLO = 256, T_O = 384, T_COLS = 512 };

#ifdef AXB_SDPA_PROF
__device__ unsigned long long g_sdpa_prof[32];
#define PROF_DECL(n) long long prof_t[n] = {}; long long prof_c = clock64(); const bool prof_on = blockIdx.x == 0 && blockIdx.y == 0;
#define PROF_ADD(i) { const long long t_ = clock64(); prof_t[i] += t_ - prof_c; prof_c = t_; }
#define PROF_OUT(base, n) if (prof_on) { for (int i_ = 0; i_ < n; ++i_) g_sdpa_prof[base + i_] = (unsigned long long)prof_t[i_]; }
#else
#define PROF_DECL(n)
#define PROF_ADD(i)
#define PROF_OUT(base, n)
#endif

__device__ __forceinline__ bool wait_warp(uint32_t bar, uint32_t parity)
{
    return __all_sync(0xffffffffu, mbar_wait_bounded(bar, parity) ? 1 : 0) != 0;
}

// maximum of the raw scores of one row (masked entries excluded)
template <bool MASK>
__device__ __forceinline__ float row_max(uint32_t s_addr, int k0, int gi, int S, int causal)
{
    float mx[4] = { -INFINITY, -INFINITY, -INFINITY, -INFINITY };
#pragma unroll 1
    for (int c0 = 0; c0 < TKV; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(s_addr + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 32; ++c) {
            float v = __uint_as_float(r[c]);
            if (MASK) {
                const int gj = k0 + c0 + c;
                if ((causal && gj > gi) || gj >= S) v = -INFINITY;
            }
            mx[c & 3] = fmaxf(mx[c & 3], v);
        }
    }
    return fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
}

// p = 2^(c*s - m) for one row; P hi over the scores, P lo at plo_addr; returns the row sum
template <bool MASK>
__device__ __forceinline__ float row_exp(uint32_t s_addr, uint32_t plo_addr, float c_log2, float neg_m, int k0,
                                         int gi, int S, int causal)
{
    float sum[4] = { 0.f, 0.f, 0.f, 0.f };
#pragma unroll 1
    for (int c0 = 0; c0 < TKV; c0 += 32) {
        uint32_t r[32], lo[32];
        tmem_ld_32x32(s_addr + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 32; ++c) {
            float p = ex2_approx(fmaf(__uint_as_float(r[c]), c_log2, neg_m));
            if (MASK) {
                const int gj = k0 + c0 + c;
                if ((causal && gj > gi) || gj >= S) p = 0.f;
            }
            sum[c & 3] += p;
            const float ph = tf32_rna(p);
            r[c] = __float_as_uint(ph);
            lo[c] = __float_as_uint(p - ph);
        }
        tmem_st_32x32(s_addr + c0, r);
        tmem_st_32x32(plo_addr + c0, lo);
    }
    tmem_st_wait();
    return (sum[0] + sum[1]) + (sum[2] + sum[3]);
}

template <int NSLAB>
__global__ void __launch_bounds__(ST_THREADS, 1) sdpa_tc_kernel(const __grid_constant__ SdpaTmaps tm,
                                                                 const SdpaTcArgs a)
{
    constexpr int OW = 32 * NSLAB;             // accumulator columns of one output buffer
    constexpr uint32_t PLANE = NSLAB * SLAB;   // bytes of one plane of a 128-row tile
    constexpr uint32_t TILE = 2 * PLANE;       // hi + lo
    static_assert(2 * OW <= T_COLS - T_O, "output buffers exceed the TMEM allocation");

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *base_ptr = smem_raw + (base - raw);
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(base_ptr + 512);
    const uint32_t q_smem = base + ST_HEADER;
    const uint32_t k_smem = q_smem + TILE;
    const uint32_t v_smem = k_smem + TILE;
    auto bar = [&](int i) -> uint32_t { return base + 8u * (uint32_t)i; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qt = a.causal ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x;  // longest rows first
    const int head = blockIdx.y;
    const int q0 = qt * TQ;
    const int kv_end = a.causal ? min(a.S, q0 + TQ) : a.S;
    const int nb = (kv_end + TKV - 1) / TKV;

    if (threadIdx.x == 0) {
        mbar_init(bar(B_Q_FULL), 1);
        mbar_init(bar(B_K_FULL), 1);
        mbar_init(bar(B_K_EMPTY), 1);
        mbar_init(bar(B_V_FULL), 1);
        mbar_init(bar(B_V_EMPTY), 1);
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar(B_S_FULL + b), 1);
            mbar_init(bar(B_P_FULL + b), 128);
            mbar_init(bar(B_O_FULL + b), 1);
            mbar_init(bar(B_O_EMPTY + b), 128);
        }
        mbar_fence_init();
    }
    if (warp == 5) {
        tmem_alloc(base + 512, T_COLS);
        tmem_relinquish();
    }
    if (warp == 4 && lane == 0) {
        tma_prefetch_desc(&tm.q[0]); tma_prefetch_desc(&tm.q[1]);
        tma_prefetch_desc(&tm.k[0]); tma_prefetch_desc(&tm.k[1]);
        tma_prefetch_desc(&tm.v[0]); tma_prefetch_desc(&tm.v[1]);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp == 4) {
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            mbar_arrive_expect_tx(bar(B_Q_FULL), TILE);
#pragma unroll
            for (int pl = 0; pl < 2; ++pl)
#pragma unroll
                for (int s = 0; s < NSLAB; ++s)
                    tma_load_3d(q_smem + pl * PLANE + s * SLAB, &tm.q[pl], bar(B_Q_FULL), 32 * s, q0, head);
            // order K_0, K_1, V_0, K_2, V_1, ...: the K buffer frees early (its scores are computed one block
            // ahead), the V buffer only when the previous block's P.V has finished
            auto load_k = [&](int j) -> bool {
                if (j >= 1 && !mbar_wait_bounded(bar(B_K_EMPTY), (j - 1) & 1)) return false;
                mbar_arrive_expect_tx(bar(B_K_FULL), TILE);
#pragma unroll
                for (int pl = 0; pl < 2; ++pl)
#pragma unroll
                    for (int s = 0; s < NSLAB; ++s)
                        tma_load_3d(k_smem + pl * PLANE + s * SLAB, &tm.k[pl], bar(B_K_FULL), 32 * s, j * TKV, head);
                return true;
            };
            bool ok = load_k(0);
            for (int j = 0; ok && j < nb; ++j) {
                if (j + 1 < nb) ok = load_k(j + 1);
                if (!ok) break;
                if (j >= 1 && !mbar_wait_bounded(bar(B_V_EMPTY), (j - 1) & 1)) { ok = false; break; }
                mbar_arrive_expect_tx(bar(B_V_FULL), TILE);
#pragma unroll
                for (int pl = 0; pl < 2; ++pl)
#pragma unroll
                    for (int s = 0; s < NSLAB; ++s)
                        tma_load_3d(v_smem + pl * PLANE + s * SLAB, &tm.v[pl], bar(B_V_FULL), 32 * s, j * TKV, head);
            }
            if (!ok) report_err(a.err, SERR_PRODUCER);
        }
    } else if (warp == 5) {
        // ---------------------------------------------------------- MMA issuer
        if (lane == 0) {
            const uint64_t desc_k = smem_desc_kmajor(0, 128);
            const uint64_t desc_mn = smem_desc_mnmajor_sw128_32b(0, SLAB, 512);
            const uint32_t idesc_qk = make_idesc<KIND_TF32>(TQ, TKV);
            const uint32_t idesc_pv = make_idesc<KIND_TF32>(TQ, a.n_pv) | (1u << 16);  // B is MN-major
            const int ksteps = a.ksteps_qk;

            auto issue_qk = [&](int j) {
                const uint32_t d = tmem + T_S + (j & 1) * TKV;
                uint32_t acc = 0;
#pragma unroll
                for (int pr = 0; pr < 3; ++pr) {
                    const uint32_t qa = q_smem + (pr == 0 ? PLANE : 0);   // lo.hi, hi.lo, hi.hi
                    const uint32_t kk = k_smem + (pr == 1 ? PLANE : 0);
#pragma unroll
                    for (int ks = 0; ks < 4 * NSLAB; ++ks) {
                        if (ks < ksteps) {
                            const uint32_t off = (ks >> 2) * SLAB + (ks & 3) * 32;
                            tc_mma<KIND_TF32>(d, desc_k | (uint64_t)(((qa + off) & 0x3FFFFu) >> 4),
                                              desc_k | (uint64_t)(((kk + off) & 0x3FFFFu) >> 4), idesc_qk, acc);
                            acc = 1;
                        }
                    }
                }
                tc_commit(bar(B_S_FULL + (j & 1)));
                tc_commit(bar(B_K_EMPTY));
            };
            auto issue_pv = [&](int j) {
                const int b = j & 1;
                const uint32_t d = tmem + T_O + b * OW;
                const uint32_t phi = tmem + T_S + b * TKV, plo = tmem + T_PLO;
                uint32_t acc = 0;
#pragma unroll
                for (int pr = 0; pr < 3; ++pr) {
                    const uint32_t pa = pr == 0 ? plo : phi;                // lo.hi, hi.lo, hi.hi
                    const uint32_t vv = v_smem + (pr == 1 ? PLANE : 0);
#pragma unroll
                    for (int ks = 0; ks < TKV / 8; ++ks) {
                        tc_mma_ts_tf32(d, pa + ks * 8, desc_mn | (uint64_t)(((vv + ks * 1024) & 0x3FFFFu) >> 4), idesc_pv, acc);
                        acc = 1;
                    }
                }
                tc_commit(bar(B_O_FULL + b));
                tc_commit(bar(B_V_EMPTY));
            };

            PROF_DECL(8)
            bool ok = mbar_wait_bounded(bar(B_Q_FULL), 0) && mbar_wait_bounded(bar(B_K_FULL), 0);
            PROF_ADD(0)
            if (ok) {
                tc_fence_after_sync();
                issue_qk(0);
            }
            PROF_ADD(1)
            for (int j = 0; ok && j < nb; ++j) {
                if (j + 1 < nb) {
                    // the score buffer of block j+1 held P hi of block j-1: its P.V was issued before this
                    // point and MMAs execute in order, so nothing else has to be waited for
                    ok = mbar_wait_bounded(bar(B_K_FULL), (j + 1) & 1);
                    PROF_ADD(2)
                    if (!ok) break;
                    tc_fence_after_sync();
                    issue_qk(j + 1);
                    PROF_ADD(1)
                }
                const int b = j & 1, n = j >> 1;
                ok = mbar_wait_bounded(bar(B_P_FULL + b), n & 1);
                PROF_ADD(4)
                ok = ok && mbar_wait_bounded(bar(B_V_FULL), j & 1);
                PROF_ADD(5)
                ok = ok && (j < 2 || mbar_wait_bounded(bar(B_O_EMPTY + b), (n - 1) & 1));
                PROF_ADD(6)
                if (!ok) break;
                tc_fence_after_sync();
                issue_pv(j);
                PROF_ADD(7)
            }
            if (!ok) report_err(a.err, SERR_MMA);
            PROF_OUT(0, 8)
        }
    } else {
        // ------------------------------------------------------- softmax warps
        const int row = threadIdx.x;  // 0..127 = TMEM lane = query row of the tile
        const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
        const int gi = q0 + row;
        float o[OW];
#pragma unroll
        for (int c = 0; c < OW; ++c) o[c] = 0.f;
        float m = -INFINITY, l = 0.f;   // m in the scaled base-2 domain
        bool ok = true;

        auto fold = [&](int jb, float corr) {  // o = (o + O_jb) * corr
            const int b = jb & 1;
            tc_fence_after_sync();
            uint32_t r[OW / 32][32];
#pragma unroll
            for (int h = 0; h < OW / 32; ++h) tmem_ld_32x32(lane_base + T_O + b * OW + 32 * h, r[h]);
            tmem_ld_wait();
            tc_fence_before_sync();
            mbar_arrive(bar(B_O_EMPTY + b));
#pragma unroll
            for (int c = 0; c < OW; ++c) o[c] = (o[c] + __uint_as_float(r[c >> 5][c & 31])) * corr;
        };

        PROF_DECL(8)
        for (int j = 0; j < nb; ++j) {
            const int b = j & 1, n = j >> 1;
            if (!wait_warp(bar(B_S_FULL + b), n & 1)) { ok = false; break; }
            PROF_ADD(0)
            tc_fence_after_sync();
            const uint32_t s_addr = lane_base + T_S + b * TKV;
            const int k0 = j * TKV;
            const bool need_mask = (a.causal && k0 + TKV - 1 > q0) || (k0 + TKV > a.S);
            const float mx = need_mask ? row_max<true>(s_addr, k0, gi, a.S, a.causal)
                                       : row_max<false>(s_addr, k0, gi, a.S, a.causal);
            const float m_new = fmaxf(m, mx * a.c_log2);
            const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
            const float corr = ex2_approx(m - m_safe);  // 0 on the first block
            PROF_ADD(1)
            // P lo is a single buffer: the previous block's P.V must have finished reading it
            if (j > 0 && !wait_warp(bar(B_O_FULL + ((j - 1) & 1)), ((j - 1) >> 1) & 1)) { ok = false; break; }
            PROF_ADD(2)
            const float sum = need_mask ? row_exp<true>(s_addr, lane_base + T_PLO, a.c_log2, -m_safe, k0, gi, a.S, a.causal)
                                        : row_exp<false>(s_addr, lane_base + T_PLO, a.c_log2, -m_safe, k0, gi, a.S, a.causal);
            tc_fence_before_sync();
            mbar_arrive(bar(B_P_FULL + b));
            l = l * corr + sum;
            m = m_new;
            PROF_ADD(3)
            if (j > 0) fold(j - 1, corr);
            PROF_ADD(4)
        }
        if (ok && nb > 0) {
            if (wait_warp(bar(B_O_FULL + ((nb - 1) & 1)), ((nb - 1) >> 1) & 1)) fold(nb - 1, 1.0f);
            else ok = false;
        }
        if (!ok) report_err(a.err, SERR_SOFTMAX);
        if (threadIdx.x == 0) { PROF_OUT(8, 8) }

        if (ok && gi < a.S) {
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            float *dst = a.O + ((int64_t)head * a.S + gi) * a.dk;
            if (a.vec_out) {
#pragma unroll
                for (int c = 0; c < OW; c += 4)
                    if (c < a.dk)
                        *reinterpret_cast<float4 *>(dst + c) =
                            make_float4(o[c] * inv, o[c + 1] * inv, o[c + 2] * inv, o[c + 3] * inv);
            } else {
#pragma unroll
                for (int c = 0; c < OW; ++c)
                    if (c < a.dk) dst[c] = o[c] * inv;
            }
            if (a.L) a.L[(int64_t)head * a.S + gi] = m * 0.69314718055994531f + logf(l);
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 5) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, T_COLS);
    }
}

// Q, K, V [rows, dk] -> hi/lo tf32 planes [rows, pitch] (pitch = dk rounded up to 4; pad columns zero)
__global__ void __launch_bounds__(256) sdpa_split_kernel(const float *__restrict__ q, const float *__restrict__ k,
                                                         const float *__restrict__ v, float *planes,
                                                         int64_t plane_floats, int64_t rows, int dk, int pitch)
{
    const int t = blockIdx.y;
    const float *src = t == 0 ? q : (t == 1 ? k : v);
    float *hi = planes + (int64_t)(2 * t) * plane_floats, *lo = hi + plane_floats;
    const int p4 = pitch / 4;
    const int64_t total = rows * p4;
    const bool vec = (dk % 4 == 0) && ((reinterpret_cast<uintptr_t>(src) & 15) == 0);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / p4;
        const int c = (int)(i - r * p4) * 4;
        float x[4];
        if (vec) {
            const float4 w = __ldg(reinterpret_cast<const float4 *>(src + r * dk + c));
            x[0] = w.x; x[1] = w.y; x[2] = w.z; x[3] = w.w;
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) x[e] = (c + e < dk) ? __ldg(src + r * dk + c + e) : 0.f;
        }
        float4 h, d;
        h.x = tf32_rna(x[0]); d.x = tf32_rna(x[0] - h.x);
        h.y = tf32_rna(x[1]); d.y = tf32_rna(x[1] - h.y);
        h.z = tf32_rna(x[2]); d.z = tf32_rna(x[2] - h.z);
        h.w = tf32_rna(x[3]); d.w = tf32_rna(x[3] - h.w);
        *reinterpret_cast<float4 *>(hi + r * pitch + c) = h;
        *reinterpret_cast<float4 *>(lo + r * pitch + c) = d;
    }
}

// ---------------------------------------------------------------------- host

#ifdef AXB_SDPA_PROF
extern "C" __attribute__((visibility("default"))) int axb_debug_sdpa_prof(unsigned long long *out)
{
    return (int)cudaMemcpyFromSymbol(out, g_sdpa_prof, sizeof(unsigned long long) * 32);
}
#endif

bool sdpa_tc_applicable(int64_t BH, int64_t S, int64_t dk, float scale)
{
    // scale > 0: the row maximum is taken over the raw scores and scaled afterwards
    return dk >= 1 && dk <= 64 && S >= 128 && BH >= 1 && BH <= 65535 && scale > 0.f && scale < INFINITY;
}

static inline size_t plane_bytes(int64_t BH, int64_t S, int64_t dk)
{
    const int64_t pitch = (dk + 3) / 4 * 4;
    return ((size_t)BH * S * pitch * 4 + 1023) / 1024 * 1024;
}

size_t sdpa_tc_workspace_bytes(int64_t BH, int64_t S, int64_t dk) { return 6 * plane_bytes(BH, S, dk); }

template <int NSLAB>
static int launch_inst(const SdpaTmaps &tm, const SdpaTcArgs &a, dim3 grid, cudaStream_t st)
{
    const size_t smem = ST_HEADER + 3 * 2 * NSLAB * SLAB + 1024;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(sdpa_tc_kernel<NSLAB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        attr_set[dev] = true;
    }
    sdpa_tc_kernel<NSLAB><<<grid, ST_THREADS, smem, st>>>(tm, a);
    return (int)cudaGetLastError();
}

int launch_sdpa_tc_split(const float *Q, const float *K, const float *V, int64_t BH, int64_t S, int64_t dk,
                         void *workspace, int sm_count, cudaStream_t st)
{
    const int pitch = (int)((dk + 3) / 4 * 4);
    const size_t pb = plane_bytes(BH, S, dk);
    const int64_t rows = BH * S;
    int64_t blocks = (rows * (pitch / 4) + 255) / 256;
    const int64_t cap = (int64_t)sm_count * 8;
    if (blocks > cap) blocks = cap;
    sdpa_split_kernel<<<dim3((unsigned)blocks, 3), 256, 0, st>>>(Q, K, V, reinterpret_cast<float *>(workspace),
                                                                 (int64_t)(pb / 4), rows, (int)dk, pitch);
    return (int)cudaGetLastError();
}

int launch_sdpa_tc(const void *workspace, float *O, float *L, int64_t BH, int64_t S, int64_t dk, float scale,
                   int causal, int *err_word, cudaStream_t st)
{
    const int pitch = (int)((dk + 3) / 4 * 4);
    const size_t pb = plane_bytes(BH, S, dk);
    SdpaTmaps tm;
    for (int t = 0; t < 3; ++t)
        for (int pl = 0; pl < 2; ++pl) {
            CUtensorMap *dst = t == 0 ? &tm.q[pl] : (t == 1 ? &tm.k[pl] : &tm.v[pl]);
            int e = encode_f32_batched_tmap(dst, reinterpret_cast<const char *>(workspace) + (size_t)(2 * t + pl) * pb, BH, S,
                                            dk, pitch, 128, t == 2);
            if (e) return e;
        }
    SdpaTcArgs a;
    a.O = O; a.L = L;
    a.S = (int)S; a.dk = (int)dk; a.causal = causal ? 1 : 0;
    a.c_log2 = scale * 1.4426950408889634f;
    a.ksteps_qk = (int)((dk + 7) / 8);
    a.n_pv = (int)((dk + 15) / 16 * 16);
    a.vec_out = (dk % 4 == 0) && ((reinterpret_cast<uintptr_t>(O) & 15) == 0);
    a.err = err_word;
    dim3 grid((unsigned)((S + TQ - 1) / TQ), (unsigned)BH);
    return dk <= 32 ? launch_inst<1>(tm, a, grid, st) : launch_inst<2>(tm, a, grid, st);
}

}  // namespace axb
