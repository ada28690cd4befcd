// gemm_tc.cu — the tcgen05 GEMM core.
//
// One persistent, warp-specialised kernel computes
//     D[M,N] = sum over products (pa,pb) of  Aplane[pa][M,K] . Bplane[pb][N,K]^T
// with every operand plane K-major.  A single product of bf16 planes is the
// fast bf16 mode; (hi,hi),(hi,lo),(lo,hi) over tf32 planes is 3xTF32; one
// product of int8 planes with s32 accumulators is the quantised GEMM.
//
//   warp 0 (one lane)  TMA producer: cp.async.bulk.tensor tiles with the 128-byte
//                      or 64-byte swizzle into a ring of shared-memory stages,
//                      completion counted in bytes on a per-stage mbarrier
//   warp 1 (one lane)  issues tcgen05.mma (M = 128, N = BN) into one of two
//                      TMEM accumulators; tcgen05.commit releases the stage
//                      and, after the last k-block, publishes the accumulator
//   warps 2..9         epilogue: tcgen05.ld the finished accumulator (a warp may
//                      read the 32-lane quarter warp%4; two warps share a
//                      quarter and split the columns), apply alpha/beta/bias/
//                      activation or the int8 requantisation, store to global;
//                      the second accumulator lets this overlap the MMAs that
//                      follow.  For the fp32 kinds K is cut into chunks that are
//                      summed in registers (see the MMA issuer).
//
// Tiles are walked in a grouped raster (GROUP_M row-tiles per column sweep) so
// the CTAs running at one time share operand panels in L2.  Edge tiles rely
// on TMA zero fill for loads and on masking for stores.
#include "gemm_tc.cuh"
#include "gemm_tc_internal.cuh"
#include "ptx.cuh"

#include <cuda.h>
#include <stdio.h>
#include "errors.cuh"
#include <stdlib.h>
#include <string.h>

namespace axb {


// SPLITK: compiled with the split-K hand-over (KernelArgs::ksplit > 1 allowed); the plain variant keeps the
// epilogue's registers for itself.
// Integer tiles of up to 128 columns have a SECOND MMA-issuing thread (warp 11, one warp more than the other
// instantiations): a 128-byte k-block of such a tile is four short MMAs, and what it costs is the issuing thread's own
// time — ~70 cycles per MMA, ~120 for the commit, ~200 for barrier and fence, 500-600 cycles against 256 of the tensor
// pipe.  The two threads take even and odd k-blocks into an accumulator set each; integer sums are exact, so the
// epilogue's addition of the two sets changes no bit.  (The fp32 kinds keep one issuer: two chains would change the
// order of the rounded additions and with it the bits that tile shapes otherwise share.)
template <int KIND, int BN>
struct TwoIssuers {
    static constexpr bool value = KIND == KIND_I8 && BN <= 128;
};

template <int KIND, int BN, int SWB, int NPROD, bool SPLITK>
__global__ void __launch_bounds__(NUM_THREADS + (TwoIssuers<KIND, BN>::value ? 32 : 0), 1)
gemm_tc_kernel(const __grid_constant__ TmapPack tm, const __grid_constant__ KernelArgs p)
{
    constexpr bool TWO = TwoIssuers<KIND, BN>::value;
    constexpr int ACC_STRIDE = TWO ? 2 * BN : BN;   // columns between the ping and the pong accumulator
    constexpr int A_BYTES = BM * SWB;   // one A plane of one stage
    constexpr int B_BYTES = BN * SWB;
    constexpr int ES = KIND == KIND_TF32 ? 4 : (KIND == KIND_BF16 ? 2 : 1);
    constexpr int BKE = SWB / ES;       // k elements per stage
    constexpr int KSTEPS = SWB / 32;    // one MMA consumes 32 bytes of K
    constexpr int TMEM_COLS = 2 * ACC_STRIDE;
    constexpr uint32_t IDESC = make_idesc<KIND>(BM, BN);

    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *gen_base = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bar_full = base;                 // MAX_STAGES x 8 B
    const uint32_t bar_empty = base + 64;           // MAX_STAGES x 8 B
    const uint32_t bar_tfull = base + 128;          // 2 x 8 B
    const uint32_t bar_tempty = base + 144;         // 2 x 8 B
    const uint32_t tmem_slot = base + 160;
    const uint32_t stage0 = base + HEADER_BYTES;
    const int stage_bytes = p.npa * A_BYTES + p.npb * B_BYTES;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    bool passed_cluster_barrier = false;   // split-K through the cluster: see the end of the kernel
    const int total_tiles = p.m_tiles * p.n_tiles;
    const int ksplit_all = SPLITK ? p.ksplit : 1;
    const int items = total_tiles * ksplit_all;   // work item = (tile, K-slice); one slice per tile unless K is split

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(bar_tfull + 8 * a, TWO ? 2 : 1);   // one arrival per MMA issuer
            mbar_init(bar_tempty + 8 * a, 8);
        }
        mbar_fence_init();
        *reinterpret_cast<volatile int *>(gen_base + HDR_SK_DEAD) = 0;
        *reinterpret_cast<volatile int *>(gen_base + HDR_SK_LAST) = 0;
        for (int i = 0; i < p.npa; ++i) tma_prefetch_desc(&tm.a[i]);
        for (int i = 0; i < p.npb; ++i) tma_prefetch_desc(&tm.b[i]);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(gen_base + 160);

    if (warp == 0 || warp == B_PRODUCER_WARP) {
        // ----------------------------------------------------- TMA producers
        // warp 0 fetches the A planes and posts the stage's byte count, warp 10 fetches the B
        // planes: two issuing threads keep up with the tensor pipe where one could not
        const bool do_a = warp == 0;
        if (lane == 0) {
            // ring position kept incrementally and every loop invariant in a register: the producer
            // has to turn a stage around faster than the tensor pipe drains one
            uint32_t s = 0, ph = 0;
            bool ok = true;
            const int k_blocks = p.k_blocks, stages = p.stages, npa = p.npa, npb = p.npb, ksplit = ksplit_all;
            const uint32_t sbytes = (uint32_t)stage_bytes;
            grid_dep_wait();   // the operand planes come from the kernel before this one
            if (!do_a && p.cv_taps > 0) {
                // implicit convolution: a stage of B is, per plane, one box per 64-pixel patch of the tile, taken
                // from the image at the window offset of the stage's tap (out-of-range coordinates read as zero)
                constexpr int NPATCH = BN / 64, PATCH_BYTES = 64 * SWB;
                const int cblocks = p.cv_cblocks, kw = p.cv_kw, pw = p.cv_pw, phh = 64 / p.cv_pw;
                for (int w = blockIdx.x; w < items && ok; w += gridDim.x) {
                    const int t = w / ksplit, kb_lo = (w - t * ksplit) * p.kb_per_slice, kb_hi = min(k_blocks, kb_lo + p.kb_per_slice);
                    int mt, nt;
                    tile_coords(t, p.m_tiles, p.n_tiles, mt, nt);
                    int x0[NPATCH], y0[NPATCH], n0[NPATCH];
#pragma unroll
                    for (int q = 0; q < NPATCH; ++q) {
                        // (a patch past the last one reads sample `batch`: outside the tensor, all zeros)
                        const int patch = nt * NPATCH + q, n = patch / p.cv_npatch_s, rem = patch - n * p.cv_npatch_s, py = rem / p.cv_px;
                        n0[q] = n;
                        x0[q] = (rem - py * p.cv_px) * pw - p.cv_pad_w;
                        y0[q] = py * phh - p.cv_pad_h;
                    }
                    int tap = kb_lo / cblocks, cb = kb_lo - tap * cblocks;
                    int ky = tap / kw, kx = tap - ky * kw;
                    for (int kb = kb_lo; kb < kb_hi; ++kb) {
                        if (!mbar_wait_bounded(bar_empty + 8 * s, ph ^ 1u)) {
                            report(p.err, ERR_PRODUCER_WAIT);
                            ok = false;
                            break;
                        }
                        const uint32_t fb = bar_full + 8 * s;
                        uint32_t dst = stage0 + s * sbytes + npa * A_BYTES;
                        for (int i = 0; i < npb; ++i)
#pragma unroll
                            for (int q = 0; q < NPATCH; ++q, dst += PATCH_BYTES)
                                tma_load_4d(dst, &tm.b[i], fb, cb * BKE, x0[q] + kx, y0[q] + ky, n0[q]);
                        if (++cb == cblocks) {
                            cb = 0;
                            if (++kx == kw) {
                                kx = 0;
                                ++ky;
                            }
                        }
                        if (++s == (uint32_t)stages) {
                            s = 0;
                            ph ^= 1u;
                        }
                    }
                }
            } else
            for (int w = blockIdx.x; w < items && ok; w += gridDim.x) {
                const int t = w / ksplit, kb_lo = (w - t * ksplit) * p.kb_per_slice, kb_hi = min(k_blocks, kb_lo + p.kb_per_slice);
                int mt, nt;
                tile_coords(t, p.m_tiles, p.n_tiles, mt, nt);
                const int row_a = mt * BM, row_b = nt * BN;
                for (int kb = kb_lo; kb < kb_hi; ++kb) {
                    if (!mbar_wait_bounded(bar_empty + 8 * s, ph ^ 1u)) {
                        report(p.err, ERR_PRODUCER_WAIT);
                        ok = false;
                        break;
                    }
                    const uint32_t fb = bar_full + 8 * s;
                    {
                        const int kcrd = kb * BKE;
                        if (do_a) {
                            mbar_arrive_expect_tx(fb, sbytes);
                            uint32_t dst = stage0 + s * sbytes;
                            for (int i = 0; i < npa; ++i, dst += A_BYTES) tma_load_2d(dst, &tm.a[i], fb, kcrd, row_a);
                        } else {
                            uint32_t dst = stage0 + s * sbytes + npa * A_BYTES;
                            for (int i = 0; i < npb; ++i, dst += B_BYTES) tma_load_2d(dst, &tm.b[i], fb, kcrd, row_b);
                        }
                    }
                    if (++s == (uint32_t)stages) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1 || (TWO && warp == B_PRODUCER_WARP + 1)) {
        // ------------------------------------------------------- MMA issuer(s)
        // K is cut into chunks of p.chunk_kb k-blocks; every chunk starts a
        // fresh TMEM accumulator (ping-pong) that the epilogue warps drain and
        // add up in registers.  The tensor core truncates when it accumulates,
        // an error that grows with the number of steps; bounding the steps per
        // chunk and summing the chunks with rounded fp32 adds keeps the result
        // inside the fp32 tolerance for any K.  Integer and plain bf16 runs use
        // a single chunk.
        if (lane == 0) {
            uint32_t s = 0, ph = 0, vt = 0;
            bool ok = true;
            // everything the issue loop needs lives in registers
            const int k_blocks = p.k_blocks, chunk_kb = p.chunk_kb, stages = p.stages, ksplit = ksplit_all;
            const uint32_t prod_a = p.prod_a, prod_b = p.prod_b;
            const uint64_t desc_hi = smem_desc_kmajor(0, SWB);
            const uint32_t npa_bytes = p.npa * A_BYTES, sbytes = (uint32_t)stage_bytes;
            const int par = (TWO && warp != 1) ? 1 : 0;   // with two issuers: this one's k-blocks of a chunk (even / odd)
            for (int w = blockIdx.x; w < items && ok; w += gridDim.x) {
                const int kb_lo = (w % ksplit) * p.kb_per_slice, kb_hi = min(k_blocks, kb_lo + p.kb_per_slice);
                for (int kb0 = kb_lo; kb0 < kb_hi && ok; kb0 += chunk_kb, ++vt) {
                    const uint32_t acc = vt & 1u, aph = (vt >> 1) & 1u;
                    if (!mbar_wait_bounded(bar_tempty + 8 * acc, aph ^ 1u)) {
                        report(p.err, ERR_MMA_WAIT_TMEM);
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t d_tmem = tmem_base + acc * ACC_STRIDE + par * BN;
                    const int kb1 = min(kb_hi, kb0 + chunk_kb);
                    bool issued = false;
                    for (int kb = kb0; kb < kb1; ++kb) {
                        if (!TWO || ((kb - kb0) & 1) == par) {
                            if (!mbar_wait_bounded(bar_full + 8 * s, ph)) {
                                report(p.err, ERR_MMA_WAIT_FULL);
                                ok = false;
                                break;
                            }
                            tc_fence_after_sync();
                            const uint32_t sa = stage0 + s * sbytes;
                            issue_stage_mmas<KIND, SWB, NPROD, false, A_BYTES, B_BYTES>(
                                d_tmem, sa, sa + npa_bytes, prod_a, prod_b, desc_hi, IDESC, !issued);
                            issued = true;
                            tc_commit(bar_empty + 8 * s);
                        }
                        if (++s == (uint32_t)stages) {
                            s = 0;
                            ph ^= 1u;
                        }
                    }
                    if (ok) {
                        // (an issuer without a k-block in this chunk arrives plainly: nothing of its own is in flight)
                        if (issued || !TWO) tc_commit(bar_tfull + 8 * acc);
                        else mbar_arrive(bar_tfull + 8 * acc);
                    }
                }
            }
        }
    } else if (warp < B_PRODUCER_WARP) {
        // ---------------------------------------------------------- epilogue
        // 8 warps: warp % 4 picks the TMEM lane quarter (a hardware rule), the
        // two warps of a quarter split the tile's columns in halves.
        constexpr int HALF = BN / 2;
        constexpr int PIECES = HALF / 32;
        const int q = warp & 3;
        const int half = (warp - 2) >> 2;
        uint32_t vt = 0;
        bool alive = true;
        const bool rows_aligned = KIND != KIND_I8 && epi_rows_aligned(p);
        const int ksplit = ksplit_all;
        for (int w = blockIdx.x; w < items && alive; w += gridDim.x) {
            const int t = w / ksplit, slice = w - t * ksplit;
            const int kb_lo = slice * p.kb_per_slice, kb_hi = min(p.k_blocks, kb_lo + p.kb_per_slice);
            const int nchunks = (kb_hi - kb_lo + p.chunk_kb - 1) / p.chunk_kb;
            int mt, nt;
            tile_coords(t, p.m_tiles, p.n_tiles, mt, nt);
            const long long row = (long long)mt * BM + q * 32 + lane;
            const bool row_ok = row < p.M;
            const int col_base = nt * BN + half * HALF;
            const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16) + half * HALF;

            if constexpr (KIND == KIND_I8) {
                // one chunk, exact integers
                const uint32_t acc = vt & 1u, aph = (vt >> 1) & 1u;
                ++vt;
                const bool got = __all_sync(0xffffffffu, mbar_wait_warp_bounded(bar_tfull + 8 * acc, aph));
                if (!got) report(p.err, ERR_EPI_WAIT);
                tc_fence_after_sync();
                if (!SPLITK || ksplit == 1) {
                    if (!got) {
                        alive = false;
                        break;
                    }
                    // stream 32 columns at a time
#pragma unroll 1
                    for (int c = 0; c < PIECES; ++c) {
                        const int col0 = col_base + c * 32;
                        if (col0 >= p.N) break;  // warp-uniform
                        uint32_t r[32];
                        __syncwarp();  // the TMEM load is warp-collective: reconverge after masked stores
                        tmem_ld_32x32(lane_addr + acc * ACC_STRIDE + c * 32, r);
                        tmem_ld_wait();
                        if (TWO && kb_hi - kb_lo >= 2) {   // the odd k-blocks' sums
                            uint32_t r2[32];
                            tmem_ld_32x32(lane_addr + acc * ACC_STRIDE + BN + c * 32, r2);
                            tmem_ld_wait();
#pragma unroll
                            for (int j = 0; j < 32; ++j) r[j] += r2[j];
                        }
                        store_piece_i8(p, reinterpret_cast<const int *>(r), row, row_ok, col0);
                    }
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_tempty + 8 * acc);
                } else if constexpr (SPLITK) {
                    // K is split: the whole partial row goes through the hand-over, the last slice stores
                    int v[HALF];
                    if (got) {
#pragma unroll
                        for (int c = 0; c < PIECES; ++c) {
                            uint32_t r[32];
                            tmem_ld_32x32(lane_addr + acc * ACC_STRIDE + c * 32, r);
                            tmem_ld_wait();
                            if (TWO && kb_hi - kb_lo >= 2) {
                                uint32_t r2[32];
                                tmem_ld_32x32(lane_addr + acc * ACC_STRIDE + BN + c * 32, r2);
                                tmem_ld_wait();
#pragma unroll
                                for (int j = 0; j < 32; ++j) r[j] += r2[j];
                            }
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[c * 32 + j] = (int)r[j];
                        }
                        tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar_tempty + 8 * acc);
                    }
                    const int st = splitk_exchange<int, HALF>(p, v, t, slice, warp, lane, gen_base, got);
                    if (st == SK_DEAD) {
                        alive = false;
                        break;
                    }
                    if (st == SK_LAST) {
#pragma unroll
                        for (int c = 0; c < PIECES; ++c) {
                            const int col0 = col_base + c * 32;
                            if (col0 < p.N) store_piece_i8(p, &v[c * 32], row, row_ok, col0);
                        }
                    }
                }
            } else {
                // fp32 kinds: add the chunks up in registers, then the fused epilogue
                float sum[HALF];
#pragma unroll
                for (int j = 0; j < HALF; ++j) sum[j] = 0.0f;
                bool got = true;
                for (int ch = 0; ch < nchunks; ++ch, ++vt) {
                    const uint32_t acc = vt & 1u, aph = (vt >> 1) & 1u;
                    if (!__all_sync(0xffffffffu, mbar_wait_warp_bounded(bar_tfull + 8 * acc, aph))) {
                        report(p.err, ERR_EPI_WAIT);
                        got = false;
                        break;
                    }
                    tc_fence_after_sync();
#pragma unroll
                    for (int c = 0; c < PIECES; ++c) {
                        uint32_t r[32];
                        tmem_ld_32x32(lane_addr + acc * ACC_STRIDE + c * 32, r);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; ++j) sum[c * 32 + j] += __uint_as_float(r[j]);
                    }
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_tempty + 8 * acc);
                }
                if (SPLITK && ksplit > 1 && p.sk_cluster) {
                    if constexpr (SPLITK) {
                        // The partner CTA holds the other K-slice of this tile.  This warp's 32 rows x HALF columns
                        // belong to column half `half`; the CTA of cluster rank `half` finishes them.  The staging
                        // area (untouched until the finishing pass) is the inbox: slot q, thread-private order.
                        const uint32_t rank = cluster_cta_rank();
                        uint8_t *stg0 = gen_base + HEADER_BYTES + (size_t)p.stages * stage_bytes;
                        volatile int *dead = reinterpret_cast<volatile int *>(gen_base + HDR_SK_DEAD);
                        if (!got) *dead = 1;
                        if (got && (uint32_t)half != rank) {
                            const uint32_t dst = map_to_cta(smem_u32(stg0) + (uint32_t)q * 8192u + (uint32_t)lane * 16u, (uint32_t)half);
#pragma unroll
                            for (int i = 0; i < HALF / 4; ++i)
                                asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(dst + (uint32_t)i * 512u),
                                             "f"(sum[4 * i]), "f"(sum[4 * i + 1]), "f"(sum[4 * i + 2]), "f"(sum[4 * i + 3])
                                             : "memory");
                        }
                        __syncwarp();
                        cluster_sync_all();          // every thread of both CTAs passes here exactly once
                        passed_cluster_barrier = true;
                        if ((uint32_t)half != rank) break;          // (one work item per CTA: the loop is over)
                        {
                            const float4 *in4 = reinterpret_cast<const float4 *>(stg0 + (size_t)q * 8192) + lane;
#pragma unroll
                            for (int i = 0; i < HALF / 4; ++i) {
                                const float4 o4 = in4[i * 32];
                                // slice order: rank 0's partial first
                                if (rank == 0) { sum[4 * i] += o4.x; sum[4 * i + 1] += o4.y; sum[4 * i + 2] += o4.z; sum[4 * i + 3] += o4.w; }
                                else { sum[4 * i] = o4.x + sum[4 * i]; sum[4 * i + 1] = o4.y + sum[4 * i + 1]; sum[4 * i + 2] = o4.z + sum[4 * i + 2]; sum[4 * i + 3] = o4.w + sum[4 * i + 3]; }
                            }
                        }
                        // the four finishing warps reuse the inbox as their staging tiles: all must have read it
                        asm volatile("bar.sync 2, 128;" ::: "memory");
                        if (*dead) {
                            alive = false;
                            break;
                        }
                    }
                } else if (SPLITK && ksplit > 1) {
                    if constexpr (SPLITK) {
                        const int st = splitk_exchange<float, HALF>(p, sum, t, slice, warp, lane, gen_base, got);
                        if (st == SK_DEAD) {
                            alive = false;
                            break;
                        }
                        if (st == SK_NOT_LAST) continue;
                    }
                } else if (!got) {
                    alive = false;
                    break;
                }
                {
                    // sums -> this warp's staging tile (row = lane) -> fused epilogue and whole-line stores
                    float4 *stg = reinterpret_cast<float4 *>(gen_base + HEADER_BYTES + (size_t)p.stages * stage_bytes) + (warp - 2) * 256;
                    const long long row0 = row - lane;
#pragma unroll
                    for (int c = 0; c < PIECES; ++c) {
                        const int col0 = col_base + c * 32;
                        if (col0 < p.N) {
                            if (p.tma_store && lane == 0) tma_store_wait_read();   // the engine has read the previous piece
                            __syncwarp();                      // ... and so has every lane
#pragma unroll
                            for (int j4 = 0; j4 < 8; ++j4)
                                stg[lane * 8 + (j4 ^ (lane & 7))] = make_float4(sum[c * 32 + 4 * j4], sum[c * 32 + 4 * j4 + 1],
                                                                                sum[c * 32 + 4 * j4 + 2], sum[c * 32 + 4 * j4 + 3]);
                            __syncwarp();
                            if (p.tma_store) store_piece_f32_tma(p, tm.c, stg, row0, col0, lane);
                            else if (p.cv_taps > 0) store_piece_f32_conv(p, stg, row0, col0, lane);
                            else store_piece_f32(p, stg, row0, col0, lane, rows_aligned);
                        }
                    }
                }
            }
        }
    }

    // split-K through the cluster: the warps that do not take part in the hand-over (producers, MMA issuer) meet the
    // epilogue warps at the cluster barrier, which counts every thread of both CTAs — each thread exactly once,
    // whatever happened before (a partner waiting there has no time limit)
    if constexpr (SPLITK) {
        if (p.sk_cluster && !passed_cluster_barrier) {
            __syncwarp();
            cluster_sync_all();
        }
    }

    // the staging tiles must have been read before the shared memory goes away; the global writes themselves are
    // complete when the kernel is
    if (p.tma_store && warp >= 2 && warp < B_PRODUCER_WARP && lane == 0) tma_store_wait_read();

    // ---------------------------------------------------------------- teardown
    // After a wait that ran out, give copies still in flight time to land in
    // this CTA's shared memory before it is released.
    if (p.err && *reinterpret_cast<volatile int *>(p.err) != 0) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---------------------------------------------------------------------- host

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static char g_err[256] = "";
const char *gemm_tc_last_error() { return g_err; }

static EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess)
            return nullptr;
        fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

static int encode_plane(CUtensorMap *out, int kind, const void *ptr, int64_t rows, int64_t k,
                        int64_t pitch_elems, int box_rows, int swb)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        snprintf(g_err, sizeof g_err, "cuTensorMapEncodeTiled entry point not found");
        return (int)cudaErrorSymbolNotFound;
    }
    const int es = kind == KIND_TF32 ? 4 : (kind == KIND_BF16 ? 2 : 1);
    const CUtensorMapDataType dt = kind == KIND_TF32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : kind == KIND_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                     : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    cuuint64_t dims[2] = { (cuuint64_t)k, (cuuint64_t)rows };
    cuuint64_t strides[1] = { (cuuint64_t)pitch_elems * es };
    cuuint32_t box[2] = { (cuuint32_t)(swb / es), (cuuint32_t)box_rows };
    cuuint32_t estr[2] = { 1, 1 };
    CUresult r = fn(out, dt, 2, const_cast<void *>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swb == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        snprintf(g_err, sizeof g_err,
                 "cuTensorMapEncodeTiled failed (%d): ptr=%p rows=%lld k=%lld pitch=%lld box=%ux%u", (int)r, ptr,
                 (long long)rows, (long long)k, (long long)pitch_elems, box[0], box[1]);
        return (int)cudaErrorInvalidValue;
    }
    return 0;
}

// Plain (unswizzled) fp32 matrix [rows, cols] with row pitch `pitch_elems`, box = box_cols x box_rows.
int encode_f32_matrix_tmap(void *tmap_out, const float *ptr, int64_t rows, int64_t cols, int64_t pitch_elems,
                           int box_cols, int box_rows)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        snprintf(g_err, sizeof g_err, "cuTensorMapEncodeTiled entry point not found");
        return (int)cudaErrorSymbolNotFound;
    }
    cuuint64_t dims[2] = { (cuuint64_t)cols, (cuuint64_t)rows };
    cuuint64_t strides[1] = { (cuuint64_t)pitch_elems * 4 };
    cuuint32_t box[2] = { (cuuint32_t)box_cols, (cuuint32_t)box_rows };
    cuuint32_t estr[2] = { 1, 1 };
    CUresult r = fn(reinterpret_cast<CUtensorMap *>(tmap_out), CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
                    const_cast<float *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        snprintf(g_err, sizeof g_err, "cuTensorMapEncodeTiled (fp32 matrix) failed (%d): ptr=%p rows=%lld cols=%lld box=%dx%d",
                 (int)r, (const void *)ptr, (long long)rows, (long long)cols, box_cols, box_rows);
        return (int)cudaErrorInvalidValue;
    }
    return 0;
}

// fp32 planes [batch][rows][pitch] with `cols` valid elements per row, 128-byte swizzle, box = 32 x box_rows x 1.
// Rows past `rows` inside a batch entry and columns past `cols` read as zero.  atom32: swizzle 32-byte chunks
// (the layout an MN-major tf32 MMA operand needs) instead of 16-byte chunks.
int encode_f32_batched_tmap(void *tmap_out, const void *ptr, int64_t batch, int64_t rows, int64_t cols,
                            int64_t pitch_elems, int box_rows, bool atom32)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        snprintf(g_err, sizeof g_err, "cuTensorMapEncodeTiled entry point not found");
        return (int)cudaErrorSymbolNotFound;
    }
    cuuint64_t dims[3] = { (cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batch };
    cuuint64_t strides[2] = { (cuuint64_t)pitch_elems * 4, (cuuint64_t)rows * (cuuint64_t)pitch_elems * 4 };
    cuuint32_t box[3] = { 32, (cuuint32_t)box_rows, 1 };
    cuuint32_t estr[3] = { 1, 1, 1 };
    CUresult r = fn(reinterpret_cast<CUtensorMap *>(tmap_out), CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3,
                    const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        snprintf(g_err, sizeof g_err,
                 "cuTensorMapEncodeTiled (batched planes) failed (%d): ptr=%p batch=%lld rows=%lld cols=%lld pitch=%lld",
                 (int)r, ptr, (long long)batch, (long long)rows, (long long)cols, (long long)pitch_elems);
        return (int)cudaErrorInvalidValue;
    }
    return 0;
}

// int8 planes [batch][rows][pitch] with `cols` valid bytes per row, 128-byte swizzle, box = 128 x box_rows x box_batch.
// Rows past `rows` and bytes past `cols` read as zero.
int encode_i8_batched_tmap(void *tmap_out, const void *ptr, int64_t batch, int64_t rows, int64_t cols,
                           int64_t pitch_bytes, int64_t batch_stride_bytes, int box_rows, int box_batch)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        snprintf(g_err, sizeof g_err, "cuTensorMapEncodeTiled entry point not found");
        return (int)cudaErrorSymbolNotFound;
    }
    cuuint64_t dims[3] = { (cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batch };
    cuuint64_t strides[2] = { (cuuint64_t)pitch_bytes, (cuuint64_t)batch_stride_bytes };
    cuuint32_t box[3] = { 128, (cuuint32_t)box_rows, (cuuint32_t)box_batch };
    cuuint32_t estr[3] = { 1, 1, 1 };
    CUresult r = fn(reinterpret_cast<CUtensorMap *>(tmap_out), CU_TENSOR_MAP_DATA_TYPE_UINT8, 3,
                    const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        snprintf(g_err, sizeof g_err,
                 "cuTensorMapEncodeTiled (int8 planes) failed (%d): ptr=%p batch=%lld rows=%lld cols=%lld pitch=%lld",
                 (int)r, ptr, (long long)batch, (long long)rows, (long long)cols, (long long)pitch_bytes);
        return (int)cudaErrorInvalidValue;
    }
    return 0;
}

// fp32 matrix [rows, cols] with row pitch pitch_elems as the destination of 32 x 32 TMA stores, 128-byte swizzle
static int encode_f32_store_tmap(CUtensorMap *out, float *ptr, int64_t rows, int64_t cols, int64_t pitch_elems)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        snprintf(g_err, sizeof g_err, "cuTensorMapEncodeTiled entry point not found");
        return (int)cudaErrorSymbolNotFound;
    }
    cuuint64_t dims[2] = { (cuuint64_t)cols, (cuuint64_t)rows };
    cuuint64_t strides[1] = { (cuuint64_t)pitch_elems * 4 };
    cuuint32_t box[2] = { 32, 32 };
    cuuint32_t estr[2] = { 1, 1 };
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        snprintf(g_err, sizeof g_err, "cuTensorMapEncodeTiled (output) failed (%d): ptr=%p rows=%lld cols=%lld pitch=%lld", (int)r,
                 (void *)ptr, (long long)rows, (long long)cols, (long long)pitch_elems);
        return (int)cudaErrorInvalidValue;
    }
    return 0;
}

// Image planes [batch][H][W][pitch] (C valid channels per pixel) as the B operand of an implicit convolution:
// box = swb bytes of channels x patch_w x patch_h pixels of one sample, swizzled like a K-major tile of
// patch_w * patch_h rows.
static int encode_conv_image_tmap(CUtensorMap *out, int kind, const void *ptr, int64_t batch, int64_t C, int64_t H, int64_t W,
                                  int64_t pitch_elems, int swb, int patch_w, int patch_h)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        snprintf(g_err, sizeof g_err, "cuTensorMapEncodeTiled entry point not found");
        return (int)cudaErrorSymbolNotFound;
    }
    const int es = kind == KIND_TF32 ? 4 : (kind == KIND_BF16 ? 2 : 1);
    const CUtensorMapDataType dt = kind == KIND_TF32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : kind == KIND_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                     : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    cuuint64_t dims[4] = { (cuuint64_t)C, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)batch };
    cuuint64_t strides[3] = { (cuuint64_t)pitch_elems * es, (cuuint64_t)W * (cuuint64_t)pitch_elems * es,
                              (cuuint64_t)H * (cuuint64_t)W * (cuuint64_t)pitch_elems * es };
    cuuint32_t box[4] = { (cuuint32_t)(swb / es), (cuuint32_t)patch_w, (cuuint32_t)patch_h, 1 };
    cuuint32_t estr[4] = { 1, 1, 1, 1 };
    CUresult r = fn(out, dt, 4, const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swb == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        snprintf(g_err, sizeof g_err, "cuTensorMapEncodeTiled (image planes) failed (%d): ptr=%p batch=%lld C=%lld H=%lld W=%lld pitch=%lld box=%ux%ux%u",
                 (int)r, ptr, (long long)batch, (long long)C, (long long)H, (long long)W, (long long)pitch_elems, box[0], box[1], box[2]);
        return (int)cudaErrorInvalidValue;
    }
    return 0;
}

template <int KIND, int BN, int SWB, int NPROD, bool SPLITK>
static int launch_inst(const TmapPack &tm, KernelArgs &ka, int stage_bytes, int grid, cudaStream_t stream)
{
    constexpr int STAGING = KIND == KIND_I8 ? 0 : EPI_STAGING_BYTES;
    int stages = (SMEM_BUDGET - HEADER_BYTES - 1024 - STAGING) / stage_bytes;
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    if (stages < 2) {
        snprintf(g_err, sizeof g_err, "stage of %d bytes leaves fewer than 2 pipeline stages", stage_bytes);
        return (int)cudaErrorInvalidConfiguration;
    }
    ka.stages = stages;
    const int smem = HEADER_BYTES + 1024 + stages * stage_bytes + STAGING;
    auto kern = gemm_tc_kernel<KIND, BN, SWB, NPROD, SPLITK>;
    static PerDeviceOnce once;
    if (once.first()) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BUDGET);
        if (e != cudaSuccess) {
            snprintf(g_err, sizeof g_err, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
            return (int)e;
        }
    }
    // programmatic dependent launch: when the kernel before this one in the stream is the operand pre-pass (which
    // releases its dependents as it starts), the barrier set-up and the TMEM allocation run under the pre-pass's
    // tail; the TMA producers wait for the pre-pass to have finished before the first load
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(NUM_THREADS + (TwoIssuers<KIND, BN>::value ? 32 : 0));
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = stream;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    if (SPLITK && ka.sk_cluster) {   // the two K-slices of a tile are consecutive CTAs: one cluster
        at[1].id = cudaLaunchAttributeClusterDimension;
        at[1].val.clusterDim.x = 2;
        at[1].val.clusterDim.y = 1;
        at[1].val.clusterDim.z = 1;
        cfg.numAttrs = 2;
    }
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tm, ka);
    if (e != cudaSuccess) snprintf(g_err, sizeof g_err, "gemm_tc launch: %s", cudaGetErrorString(e));
    return (int)e;
}

template <int KIND, int SWB, int NPROD>
static int launch_bn(int bn, const TmapPack &tm, KernelArgs &ka, int npa, int npb, int grid, cudaStream_t st)
{
    const int sb = npa * BM * SWB + npb * bn * SWB;
    const bool split = ka.ksplit > 1;
    switch (bn) {
    case 256: return split ? launch_inst<KIND, 256, SWB, NPROD, true>(tm, ka, sb, grid, st)
                           : launch_inst<KIND, 256, SWB, NPROD, false>(tm, ka, sb, grid, st);
    case 128: return split ? launch_inst<KIND, 128, SWB, NPROD, true>(tm, ka, sb, grid, st)
                           : launch_inst<KIND, 128, SWB, NPROD, false>(tm, ka, sb, grid, st);
    default: return split ? launch_inst<KIND, 64, SWB, NPROD, true>(tm, ka, sb, grid, st)
                          : launch_inst<KIND, 64, SWB, NPROD, false>(tm, ka, sb, grid, st);
    }
}

// How a problem is cut into work: tile shape, stage width, accumulator chunks and K-slices.
struct TcPlan {
    int bn;            // tile columns (256 for CTA pairs)
    bool pair;         // CTA pairs on 256 x 256 tiles (gemm_tc2.cu)
    int64_t mt, nt;    // tiles along M (of 256 rows for pairs) and along N
    int swb;           // bytes of K per stage row
    int k_blocks, chunk_kb;
    int ksplit, kb_per_slice;
};


static TcPlan make_plan(int kind, const TcProducts &prod, int64_t M, int64_t N, int64_t K, int sm_count, const TcSplitK *splitk,
                        bool allow_pair = true)
{
    TcPlan pl;
    const bool can_split = splitk && splitk->scratch && splitk->counters;
    // Tile shape.  CTA pairs when there are enough 256 x 256 tiles to fill the machine.  Otherwise one CTA per
    // 128 x bn tile; with split-K available the tile stays 128 columns wide and K is cut instead (every halving of
    // the width adds operand traffic — the A panel is loaded once per column tile — and an N = 64 MMA runs the
    // tensor pipe at two thirds of its rate); without it a width is given up only when it would leave more than half
    // of the SMs without a tile.
    int64_t mt = (M + BM - 1) / BM;
    int bn = 256;
    if (mt * ((N + 255) / 256) * 2 < sm_count) bn = 128;
    if (!can_split && bn == 128 && mt * ((N + 127) / 128) * 2 < sm_count) bn = 64;
    if (N <= 64) bn = 64;
    else if (N <= 128 && bn > 128) bn = 128;
    bool use_pair = allow_pair && ((M + 255) / 256) * ((N + 255) / 256) >= sm_count / 2 && N >= 256 && M >= 256;
    if (use_pair) {
        bn = 256;
        mt = (M + 255) / 256;
    }
    pl.bn = bn;
    pl.pair = use_pair;
    pl.mt = mt;
    pl.nt = (N + bn - 1) / bn;
    // 128-byte rows everywhere (fewer, larger stages: half the TMA and barrier traffic per unit of K) except
    // for the split-precision modes on single-CTA 128 x 256 tiles, where four operand planes of 128-byte rows
    // would leave a two-stage ring: those take 64-byte rows and keep four stages.
    pl.swb = (kind != KIND_I8 && prod.n > 1 && !use_pair && bn == 256) ? 64 : 128;
    const int es = kind == KIND_TF32 ? 4 : (kind == KIND_BF16 ? 2 : 1);
    const int bke = pl.swb / es;
    pl.k_blocks = (int)((K + bke - 1) / bke);
    pl.chunk_kb = pl.k_blocks;
    if (kind != KIND_I8 && prod.chunk_k > 0) {
        pl.chunk_kb = prod.chunk_k / bke;
        if (pl.chunk_kb < 1) pl.chunk_kb = 1;
        if (pl.chunk_kb > pl.k_blocks) pl.chunk_kb = pl.k_blocks;
    }
    // split-K: when the tiles would leave at least half of the SMs idle, K is cut into slices of whole accumulator
    // chunks (so the arithmetic of a slice is that of the same k range in an unsplit run) and tile x slice items fill
    // the machine; the partial tiles meet in scratch (splitk_exchange)
    pl.ksplit = 1;
    pl.kb_per_slice = pl.k_blocks;
    const int64_t tiles = pl.mt * pl.nt;
    const int64_t slots = sm_count;   // CTAs that run at once
    // (CTA pairs never split: measured, a problem with that few 256 x 256 tiles is faster on single-CTA tiles)
    if (can_split && !use_pair && bn <= 128 && tiles * 2 <= slots) {
        const int unit = (kind != KIND_I8 && pl.chunk_kb < pl.k_blocks) ? pl.chunk_kb : 4;   // k-blocks a slice is made of
        const int64_t units = (pl.k_blocks + unit - 1) / unit;
        const size_t slice_bytes = (size_t)BM * bn * 4;
        int64_t want = slots / tiles;
        if (want > units) want = units;
        if (want > 8) want = 8;
        const int64_t fit = (int64_t)(splitk->scratch_bytes / (slice_bytes * (size_t)tiles));
        if (want > fit) want = fit;
        if (tiles > splitk->n_counters) want = 1;
        if (want >= 2) {
            pl.kb_per_slice = (int)((units + want - 1) / want) * unit;
            pl.ksplit = (pl.k_blocks + pl.kb_per_slice - 1) / pl.kb_per_slice;
        }
    }
    // 256-column tiles that leave the last wave part empty (between half a wave and a whole one, e.g. the 96 tiles of a
    // 1024 x 3072 weight gradient on 148 SMs): K is cut so that tile x slice items fill whole waves — 96 x 3 = 288 items
    // are 1.95 rounds of a third of the work each instead of one round at 65 % occupancy.  Taken when it lifts the
    // occupancy of the rounds by a sixth or more AND a slice keeps at least eight accumulator chunks: the hand-over of a
    // 128 x 256 partial tile costs as much as several chunks (measured: K = 8192 254 -> 211 us; K = 4096 no gain; K = 2560
    // with four slices 85 -> 119 us).
    if (can_split && !use_pair && bn == 256 && pl.ksplit == 1 && tiles * 2 > slots && tiles < slots) {
        const int unit = (kind != KIND_I8 && pl.chunk_kb < pl.k_blocks) ? pl.chunk_kb : 4;
        const int64_t units = (pl.k_blocks + unit - 1) / unit;
        const size_t slice_bytes = (size_t)BM * bn * 4;
        auto occupancy = [&](int64_t ks) { return (double)(tiles * ks) / (double)(((tiles * ks + slots - 1) / slots) * slots); };
        int64_t best = 1;
        for (int64_t ks = 2; ks <= 4; ++ks) {
            if (units / ks < 8 || slice_bytes * (size_t)tiles * (size_t)ks > splitk->scratch_bytes || tiles > splitk->n_counters) break;
            if (occupancy(ks) > occupancy(best) + 1e-9) best = ks;
        }
        if (best > 1 && occupancy(best) >= occupancy(1) * (7.0 / 6.0)) {
            pl.kb_per_slice = (int)((units + best - 1) / best) * unit;
            pl.ksplit = (pl.k_blocks + pl.kb_per_slice - 1) / pl.kb_per_slice;
        }
    }
    return pl;
}

bool gemm_tc_splits_k(int kind, const TcProducts &prod, int64_t M, int64_t N, int64_t K, int sm_count)
{
    static int dummy_counter;
    const TcSplitK any = { &dummy_counter, (size_t)1 << 40, &dummy_counter, 1 << 30 };
    return make_plan(kind, prod, M, N, K, sm_count, &any).ksplit > 1;
}

// The 64-pixel patch of an implicit convolution: patch_w x 64/patch_w output pixels, the shape that wastes the
// fewest pixels past the image's right and bottom edges.
static int conv_patch_w(int64_t out_h, int64_t out_w)
{
    int best = 8;
    int64_t best_area = -1;
    for (int pw = 8; pw <= 32; pw *= 2) {
        const int ph = 64 / pw;
        const int64_t area = ((out_w + pw - 1) / pw) * ((out_h + ph - 1) / ph);
        if (best_area < 0 || area < best_area) {
            best = pw;
            best_area = area;
        }
    }
    return best;
}

int gemm_tc_conv_channel_pad(int kind) { return kind == KIND_TF32 ? 32 : (kind == KIND_BF16 ? 64 : 128); }

bool gemm_tc_conv_applicable(const TcConv &cv, int sh, int sw, const void *out)
{
    if (!(sh == 1 && sw == 1 && cv.out_w % 4 == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0 && cv.out_h > 0 &&
          cv.out_w > 0 && cv.batch >= 1 && cv.H < (1 << 30) && cv.W < (1 << 30) && cv.out_h < (1 << 30) &&
          cv.out_w < (1 << 30) && cv.kh * cv.kw < (1 << 20)))
        return false;
    // the GEMM's column count (64 per patch, samples back to back) must stay inside 31 bits
    const int64_t patches = ((cv.out_w + 7) / 8) * ((cv.out_h + 1) / 2) * cv.batch;   // the most any patch shape needs
    return patches < (1 << 24);
}

static int launch_common(int kind, const TcOperand &A, const TcOperand &B, const TcProducts &prod, int64_t M, int64_t N,
                         int64_t K, const TcEpilogue &ep, int *err_word, int sm_count, cudaStream_t stream,
                         const TcSplitK *splitk, const TcConv *cv);

int launch_gemm_tc(int kind, const TcOperand &A, const TcOperand &B, const TcProducts &prod,
                   int64_t M, int64_t N, int64_t K, const TcEpilogue &ep, int *err_word,
                   int sm_count, cudaStream_t stream, const TcSplitK *splitk)
{
    return launch_common(kind, A, B, prod, M, N, K, ep, err_word, sm_count, stream, splitk, nullptr);
}

int launch_gemm_tc_conv(int kind, const TcOperand &A, const TcOperand &B_image, const TcProducts &prod, int64_t M,
                        const TcConv &cv, const TcEpilogue &ep, int *err_word, int sm_count, cudaStream_t stream,
                        const TcSplitK *splitk)
{
    if (!gemm_tc_conv_applicable(cv, 1, 1, ep.C) || ep.out_mode != OUT_F32 || ep.beta != 0.0f || ep.n_extra != 0 ||
        ep.hs_dk != 0 || ep.bias || ep.colscale || kind == KIND_I8) {
        snprintf(g_err, sizeof g_err, "launch_gemm_tc_conv: geometry or epilogue outside the implicit path");
        return (int)cudaErrorInvalidValue;
    }
    const int pw = conv_patch_w(cv.out_h, cv.out_w), ph = 64 / pw;
    const int64_t npatch = ((cv.out_w + pw - 1) / pw) * ((cv.out_h + ph - 1) / ph) * cv.batch;
    const int cpad = gemm_tc_conv_channel_pad(kind);
    const int64_t c_pad = (cv.C + cpad - 1) / cpad * cpad;
    return launch_common(kind, A, B_image, prod, M, npatch * 64, (int64_t)cv.kh * cv.kw * c_pad, ep, err_word, sm_count,
                         stream, splitk, &cv);
}

static int launch_common(int kind, const TcOperand &A, const TcOperand &B, const TcProducts &prod, int64_t M, int64_t N,
                         int64_t K, const TcEpilogue &ep, int *err_word, int sm_count, cudaStream_t stream,
                         const TcSplitK *splitk, const TcConv *cv)
{
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || A.nplanes < 1 || B.nplanes < 1 || A.nplanes > TC_MAX_PLANES || B.nplanes > TC_MAX_PLANES ||
        prod.n < 1 || prod.n > TC_MAX_PRODUCTS) {
        snprintf(g_err, sizeof g_err, "launch_gemm_tc: bad operand description");
        return (int)cudaErrorInvalidValue;
    }
    // (a convolution takes CTA pairs too: each CTA's 128 columns of a tile are two whole patches)
    const TcPlan pl = make_plan(kind, prod, M, N, K, sm_count, splitk, cv == nullptr || kind != KIND_I8);
    const int bn = pl.bn, swb = pl.swb;
    const bool use_pair = pl.pair;
    const int64_t mt = pl.mt, nt = pl.nt;

    TmapPack tm;
    memset(&tm, 0, sizeof tm);
    for (int i = 0; i < A.nplanes; ++i) {
        int e = encode_plane(&tm.a[i], kind, A.plane[i], M, K, A.pitch_elems, BM, swb);
        if (e) return e;
    }
    const int cv_pw = cv ? conv_patch_w(cv->out_h, cv->out_w) : 0;
    for (int i = 0; i < B.nplanes; ++i) {
        int e = cv ? encode_conv_image_tmap(&tm.b[i], kind, B.plane[i], cv->batch, cv->C, cv->H, cv->W, B.pitch_elems, swb, cv_pw, 64 / cv_pw)
                   : encode_plane(&tm.b[i], kind, B.plane[i], N, K, B.pitch_elems, use_pair ? bn / 2 : bn, swb);
        if (e) return e;
    }
    KernelArgs ka;
    memset(&ka, 0, sizeof ka);
    ka.M = (int)M; ka.N = (int)N; ka.K = (int)K;
    ka.npa = A.nplanes; ka.npb = B.nplanes; ka.nprod = prod.n;
    for (int i = 0; i < prod.n; ++i) {
        ka.prod_a |= (uint32_t)(prod.a[i] & 15) << (4 * i);
        ka.prod_b |= (uint32_t)(prod.b[i] & 15) << (4 * i);
    }
    ka.m_tiles = (int)mt; ka.n_tiles = (int)nt;
    ka.k_blocks = pl.k_blocks;
    ka.chunk_kb = pl.chunk_kb;
    ka.ksplit = pl.ksplit;
    ka.kb_per_slice = pl.kb_per_slice;
    if (pl.ksplit > 1) {
        ka.sk_scratch = splitk->scratch;
        ka.sk_counters = splitk->counters;
        // two slices of an fp32 tile meet in shared memory (one work item per CTA: mt * nt * 2 <= sm_count by the plan)
        ka.sk_cluster = (pl.ksplit == 2 && kind != KIND_I8 && bn <= 128 && mt * nt * 2 <= sm_count) ? 1 : 0;
    }
    ka.alpha = ep.alpha; ka.beta = ep.beta; ka.bias = ep.bias; ka.colscale = ep.colscale;
    ka.dg_inv_s = ep.dg_inv_s; ka.dg_rows = ep.dg_rows;
    ka.rq_a_scale = ep.rq_a_scale; ka.rq_out_scale = ep.rq_out_scale;
    ka.act = ep.act; ka.out_mode = ep.out_mode; ka.C = ep.C; ka.acc_out = ep.acc_out;
    ka.ldc = ep.ldc; ka.err = err_word;
    ka.n_extra = ep.n_extra < 0 ? 0 : (ep.n_extra > TC_MAX_EXTRA ? TC_MAX_EXTRA : ep.n_extra);
    for (int i = 0; i < ka.n_extra; ++i) ka.c_extra[i] = ep.c_extra[i];
    if (ep.hs_dk > 0) {
        ka.hs_dk = ep.hs_dk; ka.hs_S = ep.hs_S; ka.hs_H = ep.hs_H;
        for (int i = 0; i < 3; ++i) ka.hs_out[i] = ep.hs_out[i];
        ka.n_extra = 0;   // beta applies to the scattered destinations (store_piece_f32 reads back where it writes)
    }
    if (cv) {
        const int es = kind == KIND_TF32 ? 4 : 2;
        const int cpad = gemm_tc_conv_channel_pad(kind);
        ka.cv_taps = cv->kh * cv->kw;
        ka.cv_kw = cv->kw;
        ka.cv_cblocks = (int)((cv->C + cpad - 1) / cpad * cpad / (swb / es));
        ka.cv_pw = cv_pw;
        ka.cv_px = (int)((cv->out_w + cv_pw - 1) / cv_pw);
        ka.cv_npatch = (int)(N / 64);
        ka.cv_npatch_s = (int)(N / 64 / cv->batch);
        ka.cv_pad_w = cv->pad_w;
        ka.cv_pad_h = cv->pad_h;
        // the output leaves through store_piece_f32_conv
        ka.ldc = cv->out_h * cv->out_w;
        ka.cv_out_w = (int)cv->out_w;
    }
    // aligned fp32 output that is not read back: the staging tiles leave through TMA stores; beta == 1 without bias and
    // activation (the accumulating calls of a backward pass) is a reduce-add of the same tiles
    const int tma_mode = cv ? 0 : (ep.beta == 0.0f ? 1 : ((ep.beta == 1.0f && !ep.bias && ep.act == ACT_NONE) ? 2 : 0));
    if (kind != KIND_I8 && ep.out_mode == OUT_F32 && ep.hs_dk == 0 && ka.n_extra == 0 && tma_mode && ep.C &&
        (reinterpret_cast<uintptr_t>(ep.C) & 15) == 0 && ep.ldc % 4 == 0) {
        int e = encode_f32_store_tmap(&tm.c[0], reinterpret_cast<float *>(ep.C), M, N, ep.ldc);
        if (e) return e;
        ka.tma_store = tma_mode;
    } else if (kind != KIND_I8 && ep.out_mode == OUT_F32 && ep.hs_dk > 0 && tma_mode && ep.hs_S % 32 == 0 &&
               ep.hs_dk % 32 == 0 && M % ep.hs_S == 0 && N % (ep.hs_H * ep.hs_dk) == 0 && N / (ep.hs_H * ep.hs_dk) <= 3) {
        // head-major scatter of whole 32 x 32 pieces: one store map per destination, each seen as a matrix of
        // B*H*S rows of dk floats (a piece never straddles a batch, S % 32 == 0, or a head, dk % 32 == 0)
        const int nwhich = (int)(N / (ep.hs_H * ep.hs_dk));
        bool ok = true;
        for (int i = 0; i < nwhich; ++i) ok = ok && ep.hs_out[i] && (reinterpret_cast<uintptr_t>(ep.hs_out[i]) & 15) == 0;
        if (ok && (M / ep.hs_S) * ep.hs_H * ep.hs_S <= INT32_MAX) {
            for (int i = 0; i < nwhich; ++i) {
                int e = encode_f32_store_tmap(&tm.c[i], ep.hs_out[i], (M / ep.hs_S) * ep.hs_H * ep.hs_S, ep.hs_dk, ep.hs_dk);
                if (e) return e;
            }
            ka.tma_store = tma_mode;
        }
    }
    const int64_t work = mt * nt * ka.ksplit;
    const int grid = (int)(work < sm_count ? work : sm_count);
    if (use_pair)
        return launch_gemm_tc_pair(kind, swb, prod.n, tm, ka, A.nplanes, B.nplanes, sm_count, stream, g_err, sizeof g_err);

    // instantiated combinations: split-precision modes (three products, 64-byte swizzle) and
    // single-product modes (128-byte swizzle)
    if (kind == KIND_TF32 && prod.n == 3 && swb == 64)
        return launch_bn<KIND_TF32, 64, 3>(bn, tm, ka, A.nplanes, B.nplanes, grid, stream);
    if (kind == KIND_BF16 && prod.n == 3 && swb == 64)
        return launch_bn<KIND_BF16, 64, 3>(bn, tm, ka, A.nplanes, B.nplanes, grid, stream);
    if (kind == KIND_TF32 && prod.n == 3 && swb == 128)
        return launch_bn<KIND_TF32, 128, 3>(bn, tm, ka, A.nplanes, B.nplanes, grid, stream);
    if (kind == KIND_BF16 && prod.n == 3 && swb == 128)
        return launch_bn<KIND_BF16, 128, 3>(bn, tm, ka, A.nplanes, B.nplanes, grid, stream);
    if (kind == KIND_BF16 && prod.n == 1 && swb == 128)
        return launch_bn<KIND_BF16, 128, 1>(bn, tm, ka, A.nplanes, B.nplanes, grid, stream);
    if (kind == KIND_I8 && prod.n == 1)
        return launch_bn<KIND_I8, 128, 1>(bn, tm, ka, A.nplanes, B.nplanes, grid, stream);
    snprintf(g_err, sizeof g_err, "launch_gemm_tc: no kernel for kind %d with %d products", kind, prod.n);
    return (int)cudaErrorInvalidValue;
}

}  // namespace axb
