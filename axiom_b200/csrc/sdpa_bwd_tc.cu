// sdpa_bwd_tc.cu — attention backward on the tensor cores, fp32 in / fp32 out, head dim <= 64
// (slot sdpa_bwd of ax_cuda_extension_t, include/axiom/internal/cuda_extension.h:96-100; the reference's CUDA
// path runs five strided-batched TF32 GEMMs over two BH*S*S buffers, src/compute/backends/cuda/ops_attention.cu:443-590):
//     P  = exp(scale*Q.K^T - L)            (L = row log-sum-exp from the forward; masked entries 0)
//     dV = P^T.dO      dP = dO.V^T      D_i = dO_i . O_i
//     dS = P o (dP - D) * scale          dQ = dS.K      dK = dS^T.Q
// Every contraction is three tf32 products over hi/lo planes (lo.hi + hi.lo + hi.hi), as in the forward kernel
// (sdpa_tc.cu), so the gradients keep fp32 accuracy; nothing of size S x S is stored and every output element has
// exactly one writer and a fixed summation order (no atomics: bitwise repeatable).
//
// ONE kernel in three roles.  A CTA owns 128 rows (the "fixed" side, operands F1 and F2, A operands of the MMAs) and
// walks the other side in blocks of 64 rows (the "stream", operands T1, T2, T3):
//   role DQ  fixed = 128 queries (F1 = Q, F2 = dO), stream = keys:    S  = F1.T1^T (T1 = K),  dP  = F2.T2^T (T2 = V),
//            dS from S, dP and the ROW's L and D;       dQ += dS.T3   (T3 = K again, as an MN-major operand)
//   role DK  fixed = 128 keys    (F1 = K, F2 = V),  stream = queries: S^T = F1.T1^T (T1 = Q), dP^T = F2.T2^T (T2 = dO),
//            dS^T from S^T, dP^T and the COLUMN's L and D; dK += dS^T.T3 (T3 = Q, MN-major)
//   role DV  fixed = 128 keys    (F1 = K),          stream = queries: S^T = F1.T1^T (T1 = Q),
//            P^T from S^T and the column's L;             dV += P^T.T3  (T3 = dO, MN-major)
// The score block lives in tensor memory; dS (or P) is written back over it as the tf32 hi operand (the raw fp32
// value: the tensor core ignores the 13 low mantissa bits) with the exact remainder as the lo operand over dP, and
// the third product reads both straight from tensor memory (the TS form of tcgen05.mma).  The stream tile of that
// product is the caller's row-major tile exactly as TMA leaves it (128-byte swizzle with 32-byte atoms, the one
// layout an MN-major tf32 operand may have): nothing is transposed.  Every block's product lands in a fresh
// accumulator and is added to the row's fp32 registers by its thread, so the tensor core's truncating accumulation
// never spans more than one block.
//   warp 4    TMA producer: one thread runs two independent chains — T1/T2 of block b+2 as soon as the score MMAs of
//             block b have retired (two buffers), T3 of block b+1 as soon as the output product of block b has
//   warps 6-9 converters: lo = tf32(x - trunc(x)).  Stream tiles: in place behind the hi plane.  Fixed tiles: into
//             TENSOR MEMORY (thread = row), where the lo.hi product reads them as its A operand (TS form) — that
//             frees the 64 KB of shared memory the second T1/T2 buffer needs
//   warp 5    one thread issues the score MMAs, up to two blocks ahead of the row threads (two score buffers);
//   warp 10   one thread issues the output products (dS from tensor memory) as the row threads finish a block
//   warps 0-3 thread t owns row t of the fixed side
// In-kernel time stamps of the single-buffered first version showed one serial cycle per block — load T1/T2, split,
// issue the scores, issue the output product, only then the next load — of 7.8 k cycles against 4.2 k of MMA issue;
// with the loads a block ahead the cycle is the MMA issue.
// The 64-row stream (not 128) is what fits: 64 KB fixed, 2 x 64 KB of T1/T2 and 32 KB of T3 are 224 KB at head dim 64;
// all 512 tensor-memory columns are in use (one CTA per SM, by shared memory).
#include "sdpa.cuh"

#include "errors.cuh"
#include "gemm_tc.cuh"
#include "ptx.cuh"

#include <cuda.h>
#include <math.h>

namespace axb {

namespace {

constexpr int BT_F = 128, BT_T = 64, BT_THREADS = 352;
constexpr int BT_HEADER = 2048;   // barriers, the TMEM slot, and the stream rows' L and D [2][64] each
constexpr uint32_t SLAB_F = 128 * 128;   // bytes of one 32-column slab of a 128-row tile
constexpr uint32_t SLAB_T = 64 * 128;    // ... of a 64-row tile

enum { ROLE_DQ = 0, ROLE_DK = 1, ROLE_DV = 2 };

struct alignas(64) BwdTmaps {
    CUtensorMap f1, f2;       // fixed side, boxes of 128 rows (K-major use)
    CUtensorMap t1, t2, t3;   // stream side, boxes of 64 rows; t3 with the 32-byte-atom swizzle (MN-major use)
};

struct BwdTcArgs {
    float *out;            // dQ, dK or dV [BH][S][dk]
    const float *L, *D;    // [BH][S]
    int S, dk, causal;
    float scale, c_log2;   // c_log2 = scale * log2(e)
    int ksteps;            // ceil(dk / 8): MMA steps of the score products
    int n_out;             // dk rounded up to 16: N of the output product
    int vec_out;
    int *err;
};

enum { BERR_PRODUCER = 21, BERR_MMA = 22, BERR_ROWS = 23, BERR_CONVERT = 24 };

enum {
    B_F_RAW = 0, B_F_FULL = 1, B_T12_RAW = 2, B_T12_FULL = 4, B_T12_EMPTY = 6, B_T3_RAW = 8, B_T3_FULL = 9, B_T3_EMPTY = 10,
    B_S_FULL = 12, B_DS_FULL = 14, B_ACC_FULL = 16, B_ACC_EMPTY = 18, B_COUNT = 20
};

// tensor-memory columns: two score buffers of 128 (S at +0 -> dS hi, dP at +64 -> dS lo), two output accumulators,
// and the lo planes of the two fixed tiles (row = lane, k = column)
enum { T_SC = 0, T_ACC = 256, T_FLO = 384, T_COLS = 512 };

__device__ __forceinline__ void bt_report(int *err, int code)
{
    if (err) atomicCAS(err, 0, code);
}

__device__ __forceinline__ bool bt_wait_warp(uint32_t bar, uint32_t parity)
{
    return __all_sync(0xffffffffu, mbar_wait_bounded(bar, parity) ? 1 : 0) != 0;
}

}  // namespace

template <int ROLE, int NSLAB>
__global__ void __launch_bounds__(BT_THREADS, 1) sdpa_bwd_tc_kernel(const __grid_constant__ BwdTmaps tm, const BwdTcArgs a)
{
    constexpr bool HAS2 = ROLE != ROLE_DV;                 // the second score product (dP) and its operands exist
    constexpr int NF = HAS2 ? 2 : 1;                       // fixed tiles
    constexpr uint32_t PLANE_F = NSLAB * SLAB_F;                     // fixed tiles: the hi plane only (lo in tensor memory)
    constexpr uint32_t PLANE_T = NSLAB * SLAB_T, TILE_T = 2 * PLANE_T;
    constexpr uint32_t T12_BYTES = (HAS2 ? 2 : 1) * TILE_T;           // one buffer of the T1 (and T2) tiles
    constexpr int OW = 32 * NSLAB;                         // accumulator columns in use

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *base_ptr = smem_raw + (base - raw);
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(base_ptr + 256);
    float *col_L = reinterpret_cast<float *>(base_ptr + 512);    // [2][64]: the stream rows' L (in the base-2 domain)
    float *col_D = col_L + 128;                                  // [2][64]: ... and D
    const uint32_t f1_smem = base + BT_HEADER;
    const uint32_t f2_smem = f1_smem + PLANE_F;
    const uint32_t t12_smem = f1_smem + NF * PLANE_F;               // [2 buffers][T1, T2]
    const uint32_t t3_smem = t12_smem + 2 * T12_BYTES;
    auto bar = [&](int i) -> uint32_t { return base + 8u * (uint32_t)i; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.y;
    // causal: the longest loops first (DQ: the last query tiles; DK/DV: the first key tiles)
    const int ft = (ROLE == ROLE_DQ && a.causal) ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x;
    const int f0 = ft * BT_F;
    int b_lo, b_hi;   // stream blocks [b_lo, b_hi) of 64 rows
    if (ROLE == ROLE_DQ) {
        b_lo = 0;
        b_hi = ((a.causal ? min(a.S, f0 + BT_F) : a.S) + BT_T - 1) / BT_T;
    } else {
        b_lo = a.causal ? f0 / BT_T : 0;
        b_hi = (a.S + BT_T - 1) / BT_T;
    }
    const int nb = max(0, b_hi - b_lo);

    if (threadIdx.x == 0) {
        mbar_init(bar(B_F_RAW), 1);
        mbar_init(bar(B_F_FULL), 128);
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar(B_T12_RAW + b), 1);
            mbar_init(bar(B_T12_FULL + b), 64);
            mbar_init(bar(B_T12_EMPTY + b), 1);
        }
        mbar_init(bar(B_T3_RAW), 1);
        mbar_init(bar(B_T3_FULL), 64);
        mbar_init(bar(B_T3_EMPTY), 1);
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar(B_S_FULL + b), 1);
            mbar_init(bar(B_DS_FULL + b), 128);
            mbar_init(bar(B_ACC_FULL + b), 1);
            mbar_init(bar(B_ACC_EMPTY + b), 128);
        }
        mbar_fence_init();
    }
    if (warp == 5) {
        tmem_alloc(base + 256, T_COLS);
        tmem_relinquish();
    }
    if (warp == 4 && lane == 0) {
        tma_prefetch_desc(&tm.f1);
        if (HAS2) tma_prefetch_desc(&tm.f2);
        tma_prefetch_desc(&tm.t1);
        if (HAS2) tma_prefetch_desc(&tm.t2);
        tma_prefetch_desc(&tm.t3);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp == 4) {
        // ------------------------------------------------------------ producer
        if (lane == 0 && nb > 0) {
            mbar_arrive_expect_tx(bar(B_F_RAW), NF * PLANE_F);
#pragma unroll
            for (int sl = 0; sl < NSLAB; ++sl) {
                tma_load_3d(f1_smem + sl * SLAB_F, &tm.f1, bar(B_F_RAW), 32 * sl, f0, head);
                if (HAS2) tma_load_3d(f2_smem + sl * SLAB_F, &tm.f2, bar(B_F_RAW), 32 * sl, f0, head);
            }
            // Two chains, polled in turn so that neither waits behind the other: T1/T2 of block n12 go into buffer
            // n12 % 2 once the scores of block n12 - 2 have retired; T3 of block n3 once the output product of block
            // n3 - 1 has.  A chain completes every phase of its barrier before the next can begin, so the parities
            // cannot alias.
            bool ok = true;
            int n12 = 0, n3 = 0;
            uint64_t t_idle = global_timer_ns();
            while (ok && (n12 < nb || n3 < nb)) {
                bool moved = false;
                if (n12 < nb && (n12 < 2 || mbar_test_wait(bar(B_T12_EMPTY + (n12 & 1)), ((n12 >> 1) - 1) & 1))) {
                    const int r0 = (b_lo + n12) * BT_T, b = n12 & 1;
                    const uint32_t t1 = t12_smem + b * T12_BYTES, t2 = t1 + TILE_T;
                    mbar_arrive_expect_tx(bar(B_T12_RAW + b), (HAS2 ? 2 : 1) * PLANE_T);
#pragma unroll
                    for (int sl = 0; sl < NSLAB; ++sl) {
                        tma_load_3d(t1 + sl * SLAB_T, &tm.t1, bar(B_T12_RAW + b), 32 * sl, r0, head);
                        if (HAS2) tma_load_3d(t2 + sl * SLAB_T, &tm.t2, bar(B_T12_RAW + b), 32 * sl, r0, head);
                    }
                    ++n12;
                    moved = true;
                }
                if (n3 < nb && (n3 < 1 || mbar_test_wait(bar(B_T3_EMPTY), (n3 - 1) & 1))) {
                    const int r0 = (b_lo + n3) * BT_T;
                    mbar_arrive_expect_tx(bar(B_T3_RAW), PLANE_T);
#pragma unroll
                    for (int sl = 0; sl < NSLAB; ++sl) tma_load_3d(t3_smem + sl * SLAB_T, &tm.t3, bar(B_T3_RAW), 32 * sl, r0, head);
                    if (ROLE == ROLE_DV && n3 + 1 < nb) {   // the next block into L2 now (DQ / DK: T3 is T1's data, loaded a block ahead)
#pragma unroll
                        for (int sl = 0; sl < NSLAB; ++sl) tma_prefetch_3d(&tm.t3, 32 * sl, r0 + BT_T, head);
                    }
                    ++n3;
                    moved = true;
                }
                if (moved) t_idle = global_timer_ns();
                else if (global_timer_ns() - t_idle > AXB_WAIT_LIMIT_NS) ok = false;
            }
            if (!ok) bt_report(a.err, BERR_PRODUCER);
        }
    } else if (warp >= 6 && warp < 10) {
        // ---------------------------------------------------------- converters
        // lo = tf32(x - (x cut to tf32)) at the same offset of the lo plane; x itself stays where TMA put it and is
        // the hi operand
        // After the fixed tiles the four warps part: warps 6-7 split every T1/T2 buffer as it lands, warps 8-9 every T3
        // — T3 of a block arrives a block later than T1/T2 of the next one, and one group walking both in order
        // would hold the early tile behind the late one.
        const int grp = (warp - 6) >> 1;
        const int ct = threadIdx.x - 192 - grp * 64;  // 0..63 inside the group
        auto split_tile = [&](uint32_t tile, uint32_t plane) {
#pragma unroll 4
            for (int i = ct; i < (int)(plane / 16); i += 64) {
                const uint32_t addr = tile + (uint32_t)i * 16u;
                uint32_t x0, x1, x2, x3;
                asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(x0), "=r"(x1), "=r"(x2), "=r"(x3) : "r"(addr));
                const uint32_t l0 = (__float_as_uint(__uint_as_float(x0) - __uint_as_float(x0 & 0xFFFFE000u)) + 0x1000u) & 0xFFFFE000u;
                const uint32_t l1 = (__float_as_uint(__uint_as_float(x1) - __uint_as_float(x1 & 0xFFFFE000u)) + 0x1000u) & 0xFFFFE000u;
                const uint32_t l2 = (__float_as_uint(__uint_as_float(x2) - __uint_as_float(x2 & 0xFFFFE000u)) + 0x1000u) & 0xFFFFE000u;
                const uint32_t l3 = (__float_as_uint(__uint_as_float(x3) - __uint_as_float(x3 & 0xFFFFE000u)) + 0x1000u) & 0xFFFFE000u;
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr + plane), "r"(l0), "r"(l1), "r"(l2), "r"(l3) : "memory");
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy stores -> visible to the MMA
        };
        // a fixed tile's lo plane goes to tensor memory: this thread's row (the lane quarter a warp may address is
        // warp % 4), 32 columns per slab, read through the 128-byte swizzle TMA wrote the tile with
        // (hi_cols >= 0: the raw values go to tensor memory as well — the role with one fixed tile has the columns to
        // spare, and then none of its score products reads the fixed tile from shared memory)
        auto split_fixed = [&](uint32_t tile, uint32_t t_cols, int hi_cols) {
            const int r = (warp & 3) * 32 + lane;
            const uint32_t taddr = tmem + ((uint32_t)((warp & 3) * 32) << 16) + t_cols;
#pragma unroll
            for (int sl = 0; sl < NSLAB; ++sl) {
                uint32_t v[32], h[32];
#pragma unroll
                for (int c4 = 0; c4 < 8; ++c4) {
                    const uint32_t addr = tile + sl * SLAB_F + (uint32_t)r * 128u + (uint32_t)((c4 ^ (r & 7)) << 4);
                    uint32_t x0, x1, x2, x3;
                    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(x0), "=r"(x1), "=r"(x2), "=r"(x3) : "r"(addr));
                    h[4 * c4 + 0] = x0; h[4 * c4 + 1] = x1; h[4 * c4 + 2] = x2; h[4 * c4 + 3] = x3;
                    v[4 * c4 + 0] = (__float_as_uint(__uint_as_float(x0) - __uint_as_float(x0 & 0xFFFFE000u)) + 0x1000u) & 0xFFFFE000u;
                    v[4 * c4 + 1] = (__float_as_uint(__uint_as_float(x1) - __uint_as_float(x1 & 0xFFFFE000u)) + 0x1000u) & 0xFFFFE000u;
                    v[4 * c4 + 2] = (__float_as_uint(__uint_as_float(x2) - __uint_as_float(x2 & 0xFFFFE000u)) + 0x1000u) & 0xFFFFE000u;
                    v[4 * c4 + 3] = (__float_as_uint(__uint_as_float(x3) - __uint_as_float(x3 & 0xFFFFE000u)) + 0x1000u) & 0xFFFFE000u;
                }
                tmem_st_32x32(taddr + 32 * sl, v);
                if (hi_cols >= 0) tmem_st_32x32(taddr - t_cols + (uint32_t)hi_cols + 32 * sl, h);
            }
        };
        bool ok = nb > 0 && bt_wait_warp(bar(B_F_RAW), 0);
        if (ok) {
            split_fixed(f1_smem, T_FLO, HAS2 ? -1 : T_FLO + 64);
            if (HAS2) split_fixed(f2_smem, T_FLO + 64, -1);
            tmem_st_wait();
            tc_fence_before_sync();
            mbar_arrive(bar(B_F_FULL));
        }
        if (grp == 0) {
            for (int bi = 0; ok && bi < nb; ++bi) {
                const int b = bi & 1;
                const uint32_t t1 = t12_smem + b * T12_BYTES;
                if (!bt_wait_warp(bar(B_T12_RAW + b), (bi >> 1) & 1)) { ok = false; break; }
                split_tile(t1, PLANE_T);
                if (HAS2) split_tile(t1 + TILE_T, PLANE_T);
                mbar_arrive(bar(B_T12_FULL + b));
            }
        } else {
            for (int bi = 0; ok && bi < nb; ++bi) {
                if (!bt_wait_warp(bar(B_T3_RAW), bi & 1)) { ok = false; break; }
                split_tile(t3_smem, PLANE_T);
                mbar_arrive(bar(B_T3_FULL));
            }
        }
        if (!ok && nb > 0) bt_report(a.err, BERR_CONVERT);
    } else if (warp == 5 || warp == 10) {
        // --------------------------------------------------------- MMA issuers
        // Two issuing threads: warp 5 the score products, warp 10 the output products.  A tcgen05.mma of this size costs
        // the issuing thread more time (70 - 90 cycles) than it costs the tensor pipe, so one thread issuing both kinds
        // in turn was the loop's critical path with the pipe a quarter busy.  (A third thread, for the dP products, was
        // measured: the row threads slowed down beside it and the backward took 0.90 ms instead of 0.83.)
        if (lane == 0 && nb > 0) {
            const uint64_t desc_k = smem_desc_kmajor(0, 128);
            const uint64_t desc_mn = smem_desc_mnmajor_sw128_32b(0, SLAB_T, 512);
            const uint32_t idesc_sc = make_idesc<KIND_TF32>(BT_F, BT_T);
            const uint32_t idesc_out = make_idesc<KIND_TF32>(BT_F, a.n_out) | (1u << 16);  // B is MN-major
            const int ksteps = a.ksteps;

            // D[128 x 64] = F . T^T, three products: lo.hi with F's lo plane from tensor memory (TS form), then hi.lo
            // and hi.hi with both operands K-major in shared memory
            // (!HAS2: the hi plane of the fixed tile is in tensor memory too, at f_lo + 64)
            auto issue_scores = [&](uint32_t d, uint32_t f_smem, uint32_t f_lo, uint32_t t_smem) {
                uint32_t acc = 0;
#pragma unroll
                for (int ks = 0; ks < 4 * NSLAB; ++ks) {
                    if (ks < ksteps) {
                        tc_mma_ts_tf32(d, f_lo + ks * 8,
                                       desc_k | (uint64_t)(((t_smem + (ks >> 2) * SLAB_T + (ks & 3) * 32) & 0x3FFFFu) >> 4), idesc_sc, acc);
                        acc = 1;
                    }
                }
#pragma unroll
                for (int pr = 1; pr < 3; ++pr) {
                    const uint32_t tb = t_smem + (pr == 1 ? PLANE_T : 0);
#pragma unroll
                    for (int ks = 0; ks < 4 * NSLAB; ++ks) {
                        if (ks < ksteps) {
                            const uint64_t db = desc_k | (uint64_t)(((tb + (ks >> 2) * SLAB_T + (ks & 3) * 32) & 0x3FFFFu) >> 4);
                            if (HAS2) tc_mma<KIND_TF32>(d, desc_k | (uint64_t)(((f_smem + (ks >> 2) * SLAB_F + (ks & 3) * 32) & 0x3FFFFu) >> 4), db, idesc_sc, acc);
                            else tc_mma_ts_tf32(d, f_lo + 64 + ks * 8, db, idesc_sc, acc);
                            acc = 1;
                        }
                    }
                }
            };
            auto issue_block_scores = [&](int bi) {
                const int b = bi & 1;
                const uint32_t d = tmem + T_SC + b * 128;
                const uint32_t t1 = t12_smem + b * T12_BYTES;
                issue_scores(d, f1_smem, tmem + T_FLO, t1);
                if (HAS2) issue_scores(d + 64, f2_smem, tmem + T_FLO + 64, t1 + TILE_T);
                tc_commit(bar(B_S_FULL + b));
                tc_commit(bar(B_T12_EMPTY + b));
            };
            auto issue_out = [&](int bi) {
                const int b = bi & 1;
                const uint32_t d = tmem + T_ACC + b * 64;
                const uint32_t hi = tmem + T_SC + b * 128, lo = hi + 64;
                uint32_t acc = 0;
#pragma unroll
                for (int pr = 0; pr < 3; ++pr) {
                    const uint32_t pa = pr == 0 ? lo : hi;                  // lo.hi, hi.lo, hi.hi
                    const uint32_t tb = t3_smem + (pr == 1 ? PLANE_T : 0);
#pragma unroll
                    for (int ks = 0; ks < BT_T / 8; ++ks) {
                        tc_mma_ts_tf32(d, pa + ks * 8, desc_mn | (uint64_t)(((tb + ks * 1024) & 0x3FFFFu) >> 4), idesc_out, acc);
                        acc = 1;
                    }
                }
                tc_commit(bar(B_ACC_FULL + b));
                tc_commit(bar(B_T3_EMPTY));
            };
            bool ok = true;
            if (warp == 5) {
                ok = mbar_wait_bounded(bar(B_F_FULL), 0);
                for (int bi = 0; ok && bi < nb; ++bi) {
                    // score buffer bi % 2 held dS of block bi - 2, the A operand of that block's output product, which
                    // the other thread issues: wait until it has retired
                    if (bi >= 2) ok = mbar_wait_bounded(bar(B_ACC_FULL + (bi & 1)), ((bi - 2) >> 1) & 1);
                    ok = ok && mbar_wait_bounded(bar(B_T12_FULL + (bi & 1)), (bi >> 1) & 1);
                    if (!ok) break;
                    tc_fence_after_sync();
                    issue_block_scores(bi);
                }
            } else {
                for (int bi = 0; ok && bi < nb; ++bi) {
                    const int b = bi & 1, n = bi >> 1;
                    ok = mbar_wait_bounded(bar(B_DS_FULL + b), n & 1);
                    ok = ok && mbar_wait_bounded(bar(B_T3_FULL), bi & 1);
                    ok = ok && (bi < 2 || mbar_wait_bounded(bar(B_ACC_EMPTY + b), (n - 1) & 1));
                    if (!ok) break;
                    tc_fence_after_sync();
                    issue_out(bi);
                }
            }
            if (!ok) bt_report(a.err, BERR_MMA);
        }
    } else {
        // ---------------------------------------------------------- row threads
        const int row = threadIdx.x;  // 0..127 = TMEM lane = row of the fixed tile
        const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
        const int gf = f0 + row;      // global index of this thread's row (query for DQ, key for DK / DV)
        float o[OW];
#pragma unroll
        for (int c = 0; c < OW; ++c) o[c] = 0.f;
        bool ok = true;
        const int64_t hoff = (int64_t)head * a.S;
        // DQ: the row's own L (base-2 domain) and D
        float row_L = INFINITY, row_D = 0.f;
        if (ROLE == ROLE_DQ && gf < a.S) {
            row_L = __ldg(a.L + hoff + gf) * 1.4426950408889634f;
            row_D = __ldg(a.D + hoff + gf);
        }

        auto fold = [&](int bi) {  // o += accumulator of block bi
            const int b = bi & 1;
            tc_fence_after_sync();
            uint32_t r[OW / 32][32];
#pragma unroll
            for (int h = 0; h < OW / 32; ++h) tmem_ld_32x32(lane_base + T_ACC + b * 64 + 32 * h, r[h]);
            tmem_ld_wait();
            tc_fence_before_sync();
            mbar_arrive(bar(B_ACC_EMPTY + b));
#pragma unroll
            for (int c = 0; c < OW; ++c) o[c] += __uint_as_float(r[c >> 5][c & 31]);
        };

        for (int bi = 0; bi < nb; ++bi) {
            const int b = bi & 1, n = bi >> 1;
            const int t0 = (b_lo + bi) * BT_T;   // first stream row of the block
            // (a warp whose wait ran out keeps walking the loop without working: the four warps meet at the barrier
            // below once per block, and one of them leaving early would strand the others there)
            if (ROLE != ROLE_DQ) {
                // the stream rows are queries: their L and D, once per block (two buffers: a thread may be one block
                // ahead of another, never two, because of the barrier below)
                if (row < 64) {
                    const int gi = t0 + row;
                    col_L[b * 64 + row] = gi < a.S ? __ldg(a.L + hoff + gi) * 1.4426950408889634f : INFINITY;
                } else if (ROLE == ROLE_DK) {
                    const int gi = t0 + row - 64;
                    col_D[b * 64 + row - 64] = gi < a.S ? __ldg(a.D + hoff + gi) : 0.f;
                }
                asm volatile("bar.sync 2, 128;" ::: "memory");
            }
            if (!ok) continue;
            if (!bt_wait_warp(bar(B_S_FULL + b), n & 1)) { ok = false; continue; }
            tc_fence_after_sync();
            const uint32_t s_addr = lane_base + T_SC + b * 128;
            // a block needs masking when it straddles the diagonal or the end of the sequence
            bool need_mask;
            if (ROLE == ROLE_DQ) need_mask = (a.causal && t0 + BT_T - 1 > f0) || (t0 + BT_T > a.S);
            else need_mask = (a.causal && t0 < f0 + BT_F - 1) || (t0 + BT_T > a.S);
#pragma unroll 1
            for (int c0 = 0; c0 < BT_T; c0 += 32) {
                uint32_t s[32], dp[32];
                tmem_ld_32x32(s_addr + c0, s);
                if (HAS2) tmem_ld_32x32(s_addr + 64 + c0, dp);
                tmem_ld_wait();
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    const int gt = t0 + c0 + c;   // global index of the stream row of this column
                    float Lc, Dc;
                    if (ROLE == ROLE_DQ) { Lc = row_L; Dc = row_D; }
                    else { Lc = col_L[b * 64 + c0 + c]; Dc = ROLE == ROLE_DK ? col_D[b * 64 + c0 + c] : 0.f; }
                    float p = ex2_approx(fmaf(__uint_as_float(s[c]), a.c_log2, -Lc));   // Lc = +inf past the sequence: p = 0
                    if (need_mask) {
                        const bool dead = ROLE == ROLE_DQ ? ((a.causal && gt > gf) || gt >= a.S)
                                                          : ((a.causal && gt < gf) || gt >= a.S);
                        if (dead) p = 0.f;
                    }
                    const float v = HAS2 ? p * (__uint_as_float(dp[c]) - Dc) * a.scale : p;
                    s[c] = __float_as_uint(v);                                           // hi: the raw value
                    dp[c] = __float_as_uint(v - __uint_as_float(__float_as_uint(v) & 0xFFFFE000u));   // lo: the exact remainder
                }
                tmem_st_32x32(s_addr + c0, s);
                tmem_st_32x32(s_addr + 64 + c0, dp);
            }
            tmem_st_wait();
            tc_fence_before_sync();
            mbar_arrive(bar(B_DS_FULL + b));
            if (bi > 0) {
                if (!bt_wait_warp(bar(B_ACC_FULL + ((bi - 1) & 1)), ((bi - 1) >> 1) & 1)) { ok = false; continue; }
                fold(bi - 1);
            }
        }
        if (ok && nb > 0) {
            if (bt_wait_warp(bar(B_ACC_FULL + ((nb - 1) & 1)), ((nb - 1) >> 1) & 1)) fold(nb - 1);
            else ok = false;
        }
        if (!ok) bt_report(a.err, BERR_ROWS);

        if (ok && gf < a.S) {
            float *dst = a.out + (hoff + gf) * a.dk;
            if (a.vec_out) {
#pragma unroll
                for (int c = 0; c < OW; c += 4)
                    if (c < a.dk) *reinterpret_cast<float4 *>(dst + c) = make_float4(o[c], o[c + 1], o[c + 2], o[c + 3]);
            } else {
#pragma unroll
                for (int c = 0; c < OW; ++c)
                    if (c < a.dk) dst[c] = o[c];
            }
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

bool sdpa_bwd_tc_applicable(const float *Q, const float *K, const float *V, const float *dO, int64_t BH, int64_t S, int64_t dk,
                            float scale)
{
    // TMA reads the caller's tensors: rows must be multiples of 16 bytes on 16-byte aligned bases
    const uintptr_t align = reinterpret_cast<uintptr_t>(Q) | reinterpret_cast<uintptr_t>(K) | reinterpret_cast<uintptr_t>(V) |
                            reinterpret_cast<uintptr_t>(dO);
    return dk >= 4 && dk <= 64 && dk % 4 == 0 && (align & 15) == 0 && S >= 128 && BH >= 1 && BH <= 65535 && scale > 0.f &&
           scale < INFINITY;
}

template <int ROLE, int NSLAB>
static int launch_role(const BwdTmaps &tm, const BwdTcArgs &a, dim3 grid, cudaStream_t st)
{
    constexpr int NF = ROLE != ROLE_DV ? 2 : 1, NT = ROLE != ROLE_DV ? 5 : 3;   // hi planes of the fixed tiles; T1(,T2) twice and T3
    const size_t smem = BT_HEADER + (size_t)NF * NSLAB * SLAB_F + (size_t)NT * 2 * NSLAB * SLAB_T + 1024;   // 227 KB at most
    auto kern = sdpa_bwd_tc_kernel<ROLE, NSLAB>;
    static PerDeviceOnce once;
    if (once.first()) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    kern<<<grid, BT_THREADS, smem, st>>>(tm, a);
    return (int)cudaGetLastError();
}

int launch_sdpa_bwd_tc(const float *Q, const float *K, const float *V, const float *dO, const float *L, const float *D,
                       float *dQ, float *dK, float *dV, int64_t BH, int64_t S, int64_t dk, float scale, int causal,
                       int *err_word, cudaStream_t st)
{
    BwdTcArgs a;
    a.L = L; a.D = D;
    a.S = (int)S; a.dk = (int)dk; a.causal = causal ? 1 : 0;
    a.scale = scale;
    a.c_log2 = scale * 1.4426950408889634f;
    a.ksteps = (int)((dk + 7) / 8);
    a.n_out = (int)((dk + 15) / 16 * 16);
    a.err = err_word;
    dim3 grid((unsigned)((S + BT_F - 1) / BT_F), (unsigned)BH);
    auto enc = [&](CUtensorMap *m, const float *p, int rows, bool atom32) {
        return encode_f32_batched_tmap(m, p, BH, S, dk, dk, rows, atom32);
    };
    int e;
    // dQ: fixed = queries (Q, dO), stream = keys (K, V, K)
    {
        BwdTmaps tm;
        e = enc(&tm.f1, Q, BT_F, false);
        if (!e) e = enc(&tm.f2, dO, BT_F, false);
        if (!e) e = enc(&tm.t1, K, BT_T, false);
        if (!e) e = enc(&tm.t2, V, BT_T, false);
        if (!e) e = enc(&tm.t3, K, BT_T, true);
        if (e) return e;
        a.out = dQ;
        a.vec_out = (reinterpret_cast<uintptr_t>(dQ) & 15) == 0;
        e = dk <= 32 ? launch_role<ROLE_DQ, 1>(tm, a, grid, st) : launch_role<ROLE_DQ, 2>(tm, a, grid, st);
        if (e) return e;
    }
    // dK: fixed = keys (K, V), stream = queries (Q, dO, Q)
    {
        BwdTmaps tm;
        e = enc(&tm.f1, K, BT_F, false);
        if (!e) e = enc(&tm.f2, V, BT_F, false);
        if (!e) e = enc(&tm.t1, Q, BT_T, false);
        if (!e) e = enc(&tm.t2, dO, BT_T, false);
        if (!e) e = enc(&tm.t3, Q, BT_T, true);
        if (e) return e;
        a.out = dK;
        a.vec_out = (reinterpret_cast<uintptr_t>(dK) & 15) == 0;
        e = dk <= 32 ? launch_role<ROLE_DK, 1>(tm, a, grid, st) : launch_role<ROLE_DK, 2>(tm, a, grid, st);
        if (e) return e;
    }
    // dV: fixed = keys (K), stream = queries (Q, dO)
    {
        BwdTmaps tm;
        memset(&tm, 0, sizeof tm);
        e = enc(&tm.f1, K, BT_F, false);
        if (!e) e = enc(&tm.t1, Q, BT_T, false);
        if (!e) e = enc(&tm.t3, dO, BT_T, true);
        if (e) return e;
        a.out = dV;
        a.vec_out = (reinterpret_cast<uintptr_t>(dV) & 15) == 0;
        e = dk <= 32 ? launch_role<ROLE_DV, 1>(tm, a, grid, st) : launch_role<ROLE_DV, 2>(tm, a, grid, st);
    }
    return e;
}

}  // namespace axb
