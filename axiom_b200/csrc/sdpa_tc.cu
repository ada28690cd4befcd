// sdpa_tc.cu — attention forward on the tensor cores, fp32 in / fp32 out, head dim <= 64:
//     O = softmax(scale * Q.K^T [+ causal mask]) . V,   L = rowmax + log(rowsum)
//
// Both contractions run as three tf32 products over hi/lo planes (lo.hi + hi.lo + hi.hi), which keeps the
// result at fp32 accuracy (the reference computes this path in fp32, src/compute/backends/cpu_opt.c:7828-8071;
// its CUDA path uses one TF32 product and a materialised S x S buffer, cuda/ops_attention.cu:224-392).
//
// There is no pre-pass and no scratch: TMA loads the caller's fp32 tiles straight into the place of the hi
// plane, and converter warps split them where they lie (hi = the value cut to tf32, written back; lo = the
// exact remainder, rounded to tf32, written to the lo plane at the same swizzled offset).  Loading planes that
// a pre-pass had split cost 8 bytes per element from L2 for every key block of every query tile — the kernel
// was L2-bound on it — plus a pass over HBM; this costs 4.  One CTA owns 128 query rows of one head and walks
// the keys in blocks of 128:
//   warp 4   : TMA producer — the Q tile once, then one K and one V block at a time (128-byte swizzle; V with
//              the 32-byte-chunk variant, the one layout an MN-major tf32 operand may have);
//   warps 6-9: converters (above);
//   warps 5, 10: one thread each issues tcgen05.mma — warp 5 the scores, warp 10 the P.V products.
//              S_j = Q.K_j^T (M128 x N128, operands from shared memory, both
//              K-major) goes to one of two TMEM score buffers; O_j = P_j.V_j takes P from TENSOR MEMORY (the
//              TS form) and V as an MN-major shared-memory operand, i.e. exactly as the TMA load leaves it — V
//              is never transposed.  N = 128 runs the tf32 pipe at its full rate (N = 64 does not: measured
//              48 cycles per instruction instead of 32), which is why the key block is 128 wide;
//   warps 0-3: thread t owns query row t.  Pass 1 reads the score row from TMEM in 32-column chunks and takes
//              the maximum; pass 2 re-reads it, forms p = 2^(c*s - m), and writes P back as tf32 hi (over the
//              scores it came from) and lo (a third buffer).  Every block's O_j lands in a fresh accumulator
//              (the tensor core's truncating accumulation never spans more than one block) and is folded into
//              the thread's fp32 register row with the usual rescale.  The chunk loops are rolled: the body
//              stays small enough for the instruction cache, which a fully unrolled row (the first version)
//              did not — its warps spent most of their time waiting for instructions.  The split of P uses
//              integer masking, not cvt: conversions share the 16-lane pipe with ex2 and halved its rate.
// The score matrix never leaves the SM.  The scores run up to two blocks ahead of the softmax warps; the score
// buffer (aliased by P hi) of block j is overwritten by the scores of block j + 2 only once the P.V product that
// read it has retired (its completion barrier is what the score issuer waits for).
#include "sdpa.cuh"

#include "gemm_tc.cuh"
#include "ptx.cuh"

#include <cuda.h>
#include <math.h>

namespace axb {

static constexpr int TQ = 128, TKV = 128, ST_THREADS = 352;
static constexpr int ST_HEADER = 1024;
static constexpr int SLAB = 128 * 128;  // bytes of one 32-column slab of a 128-row tile

struct alignas(64) SdpaTmaps {
    CUtensorMap q, k, v;  // the caller's fp32 tensors [BH][S][dk]
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

enum { SERR_PRODUCER = 11, SERR_MMA = 12, SERR_SOFTMAX = 13, SERR_CONVERT = 14 };

__device__ __forceinline__ void report_err(int *err, int code)
{
    if (err) atomicCAS(err, 0, code);
}

enum {
    B_Q_RAW = 0, B_Q_FULL = 1, B_K_RAW = 2, B_K_FULL = 3, B_K_EMPTY = 4, B_V_RAW = 5, B_V_FULL = 6, B_V_EMPTY = 7,
    B_S_FULL = 8, B_P_FULL = 10, B_O_FULL = 12, B_O_EMPTY = 14, B_COUNT = 16
};

// TMEM columns: two score buffers (P hi is written over the scores), P lo, two output buffers
enum { T_S = 0, T_PLO = 256, T_O = 384, T_COLS = 512 };


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

// p = 2^(c*s - m) for one row, written over the scores it came from as full fp32: the tensor core reads
// the tf32 part of a 32-bit container and ignores the 13 low mantissa bits, so this IS the hi operand.
// Returns the row sum.
template <bool MASK>
__device__ __forceinline__ float row_exp(uint32_t s_addr, float c_log2, float neg_m, int k0, int gi, int S,
                                         int causal)
{
    float sum[4] = { 0.f, 0.f, 0.f, 0.f };
#pragma unroll 1
    for (int c0 = 0; c0 < TKV; c0 += 32) {
        uint32_t r[32];
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
            r[c] = __float_as_uint(p);
        }
        tmem_st_32x32(s_addr + c0, r);
    }
    tmem_st_wait();
    return (sum[0] + sum[1]) + (sum[2] + sum[3]);
}

// P lo = p - (p cut to tf32), exact, for one row
__device__ __forceinline__ void row_lo(uint32_t s_addr, uint32_t plo_addr)
{
#pragma unroll 1
    for (int c0 = 0; c0 < TKV; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(s_addr + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 32; ++c)
            r[c] = __float_as_uint(__uint_as_float(r[c]) - __uint_as_float(r[c] & 0xFFFFE000u));
        tmem_st_32x32(plo_addr + c0, r);
    }
    tmem_st_wait();
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
        mbar_init(bar(B_Q_RAW), 1);
        mbar_init(bar(B_Q_FULL), 128);
        mbar_init(bar(B_K_RAW), 1);
        mbar_init(bar(B_K_FULL), 128);
        mbar_init(bar(B_K_EMPTY), 1);
        mbar_init(bar(B_V_RAW), 1);
        mbar_init(bar(B_V_FULL), 128);
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
        tma_prefetch_desc(&tm.q);
        tma_prefetch_desc(&tm.k);
        tma_prefetch_desc(&tm.v);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp == 4) {
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            mbar_arrive_expect_tx(bar(B_Q_RAW), PLANE);
#pragma unroll
            for (int sl = 0; sl < NSLAB; ++sl) tma_load_3d(q_smem + sl * SLAB, &tm.q, bar(B_Q_RAW), 32 * sl, q0, head);
            // order K_0, K_1, V_0, K_2, V_1, ...: the K buffer frees early (its scores are computed one block
            // ahead), the V buffer only when the previous block's P.V has finished
            auto load_k = [&](int j) -> bool {
                if (j >= 1 && !mbar_wait_bounded(bar(B_K_EMPTY), (j - 1) & 1)) return false;
                mbar_arrive_expect_tx(bar(B_K_RAW), PLANE);
#pragma unroll
                for (int sl = 0; sl < NSLAB; ++sl) tma_load_3d(k_smem + sl * SLAB, &tm.k, bar(B_K_RAW), 32 * sl, j * TKV, head);
                if (j + 1 < nb) {   // the block after this one: into L2 now, so its load is short when its turn comes
#pragma unroll
                    for (int sl = 0; sl < NSLAB; ++sl) tma_prefetch_3d(&tm.k, 32 * sl, (j + 1) * TKV, head);
                }
                return true;
            };
            bool ok = load_k(0);
            for (int j = 0; ok && j < nb; ++j) {
                if (j + 1 < nb) ok = load_k(j + 1);
                if (!ok) break;
                if (j >= 1 && !mbar_wait_bounded(bar(B_V_EMPTY), (j - 1) & 1)) { ok = false; break; }
                mbar_arrive_expect_tx(bar(B_V_RAW), PLANE);
#pragma unroll
                for (int sl = 0; sl < NSLAB; ++sl) tma_load_3d(v_smem + sl * SLAB, &tm.v, bar(B_V_RAW), 32 * sl, j * TKV, head);
                if (j + 1 < nb) {
#pragma unroll
                    for (int sl = 0; sl < NSLAB; ++sl) tma_prefetch_3d(&tm.v, 32 * sl, (j + 1) * TKV, head);
                }
            }
            if (!ok) report_err(a.err, SERR_PRODUCER);
        }
    } else if (warp >= 6 && warp < 10) {
        // ---------------------------------------------------------- converters
        // lo = tf32(x - (x cut to tf32)) at the same offset of the lo plane.  x itself stays where TMA put it and
        // serves as the hi operand: the tensor core ignores the 13 low mantissa bits of a tf32 container
        // (results are bit-identical with the cut value written back, which costs a third of the traffic).
        const int ct = threadIdx.x - 192;  // 0..127
        auto split_tile = [&](uint32_t tile) {
#pragma unroll 4
            for (int i = ct; i < (int)(PLANE / 16); i += 128) {
                const uint32_t addr = tile + (uint32_t)i * 16u;
                uint32_t x0, x1, x2, x3;
                asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(x0), "=r"(x1), "=r"(x2), "=r"(x3) : "r"(addr));
                const uint32_t h0 = x0 & 0xFFFFE000u, h1 = x1 & 0xFFFFE000u, h2 = x2 & 0xFFFFE000u, h3 = x3 & 0xFFFFE000u;
                // remainder (exact), rounded to tf32 by adding half an ulp of its 13 dropped bits
                const uint32_t l0 = (__float_as_uint(__uint_as_float(x0) - __uint_as_float(h0)) + 0x1000u) & 0xFFFFE000u;
                const uint32_t l1 = (__float_as_uint(__uint_as_float(x1) - __uint_as_float(h1)) + 0x1000u) & 0xFFFFE000u;
                const uint32_t l2 = (__float_as_uint(__uint_as_float(x2) - __uint_as_float(h2)) + 0x1000u) & 0xFFFFE000u;
                const uint32_t l3 = (__float_as_uint(__uint_as_float(x3) - __uint_as_float(h3)) + 0x1000u) & 0xFFFFE000u;
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr + PLANE), "r"(l0), "r"(l1), "r"(l2), "r"(l3) : "memory");
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy stores -> visible to the MMA
        };
        bool ok = wait_warp(bar(B_Q_RAW), 0);
        if (ok) {
            split_tile(q_smem);
            mbar_arrive(bar(B_Q_FULL));
        }
        auto do_k = [&](int j) -> bool {
            if (!wait_warp(bar(B_K_RAW), j & 1)) return false;
            split_tile(k_smem);
            mbar_arrive(bar(B_K_FULL));
            return true;
        };
        ok = ok && do_k(0);
        for (int j = 0; ok && j < nb; ++j) {
            if (j + 1 < nb) ok = do_k(j + 1);
            if (!ok) break;
            if (!wait_warp(bar(B_V_RAW), j & 1)) { ok = false; break; }
            split_tile(v_smem);
            mbar_arrive(bar(B_V_FULL));
        }
        if (!ok) report_err(a.err, SERR_CONVERT);
    } else if (warp == 5 || warp == 10) {
        // --------------------------------------------------------- MMA issuers
        // Two issuing threads: warp 5 the score products, warp 10 the P.V products.  A tcgen05.mma of this size costs the
        // issuing thread more time than the tensor pipe (time stamps: 75 cycles per score MMA, 58 per P.V MMA with the
        // pipe 39 % busy), so one thread issuing both kinds in turn was one of the loop's long chains.
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
            bool ok = true;
            if (warp == 5) {
                ok = mbar_wait_bounded(bar(B_Q_FULL), 0);
                for (int j = 0; ok && j < nb; ++j) {
                    // score buffer j % 2 held P hi of block j - 2, the A operand of that block's P.V, which the other
                    // thread issues: wait until it has retired
                    if (j >= 2) ok = mbar_wait_bounded(bar(B_O_FULL + (j & 1)), ((j - 2) >> 1) & 1);
                    ok = ok && mbar_wait_bounded(bar(B_K_FULL), j & 1);
                    if (!ok) break;
                    tc_fence_after_sync();
                    issue_qk(j);
                }
            } else {
                for (int j = 0; ok && j < nb; ++j) {
                    const int b = j & 1, n = j >> 1;
                    ok = mbar_wait_bounded(bar(B_P_FULL + b), n & 1);
                    ok = ok && mbar_wait_bounded(bar(B_V_FULL), j & 1);
                    ok = ok && (j < 2 || mbar_wait_bounded(bar(B_O_EMPTY + b), (n - 1) & 1));
                    if (!ok) break;
                    tc_fence_after_sync();
                    issue_pv(j);
                }
            }
            if (!ok) report_err(a.err, SERR_MMA);
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
        for (int j = 0; j < nb; ++j) {
            const int b = j & 1, n = j >> 1;
            if (!wait_warp(bar(B_S_FULL + b), n & 1)) { ok = false; break; }
            tc_fence_after_sync();
            const uint32_t s_addr = lane_base + T_S + b * TKV;
            const int k0 = j * TKV;
            const bool need_mask = (a.causal && k0 + TKV - 1 > q0) || (k0 + TKV > a.S);
            const float mx = need_mask ? row_max<true>(s_addr, k0, gi, a.S, a.causal)
                                       : row_max<false>(s_addr, k0, gi, a.S, a.causal);
            const float m_new = fmaxf(m, mx * a.c_log2);
            const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
            const float corr = ex2_approx(m - m_safe);  // 0 on the first block
            const float sum = need_mask ? row_exp<true>(s_addr, a.c_log2, -m_safe, k0, gi, a.S, a.causal)
                                        : row_exp<false>(s_addr, a.c_log2, -m_safe, k0, gi, a.S, a.causal);
            // P lo is a single buffer: the previous block's P.V must have finished reading it.  Only this
            // short pass sits between that P.V and the next one; the exponentials above overlap it.
            if (j > 0 && !wait_warp(bar(B_O_FULL + ((j - 1) & 1)), ((j - 1) >> 1) & 1)) { ok = false; break; }
            row_lo(s_addr, lane_base + T_PLO);
            tc_fence_before_sync();
            mbar_arrive(bar(B_P_FULL + b));
            l = l * corr + sum;
            m = m_new;
            if (j > 0) fold(j - 1, corr);
        }
        if (ok && nb > 0) {
            if (wait_warp(bar(B_O_FULL + ((nb - 1) & 1)), ((nb - 1) >> 1) & 1)) fold(nb - 1, 1.0f);
            else ok = false;
        }
        if (!ok) report_err(a.err, SERR_SOFTMAX);

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

// ---------------------------------------------------------------------- host


bool sdpa_tc_applicable(const float *Q, const float *K, const float *V, int64_t BH, int64_t S, int64_t dk,
                        float scale)
{
    // TMA reads the caller's tensors: rows must be multiples of 16 bytes on 16-byte aligned bases.
    // scale > 0: the row maximum is taken over the raw scores and scaled afterwards.
    const uintptr_t align = reinterpret_cast<uintptr_t>(Q) | reinterpret_cast<uintptr_t>(K) | reinterpret_cast<uintptr_t>(V);
    return dk >= 4 && dk <= 64 && dk % 4 == 0 && (align & 15) == 0 && S >= 128 && BH >= 1 && BH <= 65535 &&
           scale > 0.f && scale < INFINITY;
}

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

int launch_sdpa_tc(const float *Q, const float *K, const float *V, float *O, float *L, int64_t BH, int64_t S,
                   int64_t dk, float scale, int causal, int *err_word, cudaStream_t st)
{
    SdpaTmaps tm;
    int e = encode_f32_batched_tmap(&tm.q, Q, BH, S, dk, dk, 128, false);
    if (!e) e = encode_f32_batched_tmap(&tm.k, K, BH, S, dk, dk, 128, false);
    if (!e) e = encode_f32_batched_tmap(&tm.v, V, BH, S, dk, dk, 128, true);
    if (e) return e;
    SdpaTcArgs a;
    a.O = O; a.L = L;
    a.S = (int)S; a.dk = (int)dk; a.causal = causal ? 1 : 0;
    a.c_log2 = scale * 1.4426950408889634f;
    a.ksteps_qk = (int)((dk + 7) / 8);
    a.n_pv = (int)((dk + 15) / 16 * 16);
    a.vec_out = (reinterpret_cast<uintptr_t>(O) & 15) == 0;
    a.err = err_word;
    dim3 grid((unsigned)((S + TQ - 1) / TQ), (unsigned)BH);
    return dk <= 32 ? launch_inst<1>(tm, a, grid, st) : launch_inst<2>(tm, a, grid, st);
}

}  // namespace axb
