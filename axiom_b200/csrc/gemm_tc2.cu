// gemm_tc2.cu — the tcgen05 GEMM core on CTA pairs (cta_group::2).
//
// Same contract as gemm_tc.cu, but a cluster of two CTAs computes one
// 256 x 256 output tile with MMAs of M = 256: each CTA stages ITS 128 rows of
// the A tile and ITS 128 rows of the B tile, and holds its 128 accumulator
// rows in its own TMEM.  Per SM this halves the shared-memory traffic of the B
// operand (both the TMA writes and the tensor-core reads), which is what
// limits the single-CTA kernel on int8 and bf16.
//
//   both CTAs, warp 0   TMA producer for the CTA's own halves; the byte counts
//                       of both CTAs land on the LEADER's full[s] barrier
//   leader, warp 1      issues tcgen05.mma.cta_group::2; tcgen05.commit with a
//                       two-CTA mask frees stage s in both CTAs and publishes
//                       the accumulator to both epilogues
//   both CTAs, warps 2..9  epilogue over the CTA's own 128 rows; accumulator
//                       release is an arrive on the leader's barrier (remote for
//                       the peer CTA)
// No multicast copies are used: every CTA fetches its own operand tiles.
#include "gemm_tc.cuh"
#include "gemm_tc_internal.cuh"
#include "errors.cuh"
#include "ptx.cuh"

#include <cuda.h>
#include <stdio.h>

namespace axb {



static constexpr int PAIR_BN = 256;
static constexpr int PAIR_TILE_M = 256;

template <int KIND, int SWB, int NPROD>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ TmapPack tm, const __grid_constant__ KernelArgs p)
{
    constexpr int BN = PAIR_BN;
    constexpr int A_BYTES = BM * SWB;          // this CTA's 128 rows of an A plane
    constexpr int B_BYTES = (BN / 2) * SWB;    // this CTA's 128 rows of a B plane
    constexpr int ES = KIND == KIND_TF32 ? 4 : (KIND == KIND_BF16 ? 2 : 1);
    constexpr int BKE = SWB / ES;
    constexpr int KSTEPS = SWB / 32;
    constexpr int TMEM_COLS = 2 * BN;
    constexpr uint32_t IDESC = make_idesc<KIND>(PAIR_TILE_M, BN);

    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *gen_base = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bar_full = base;            // leader's copy is the one in use
    const uint32_t bar_empty = base + 64;      // one per CTA, freed by the two-CTA commit
    const uint32_t bar_tfull = base + 128;     // one per CTA
    const uint32_t bar_tempty = base + 144;    // leader's copy is the one in use (16 arrivals)
    const uint32_t tmem_slot = base + 160;
    const uint32_t stage0 = base + HEADER_BYTES;
    const int stage_bytes = p.npa * A_BYTES + p.npb * B_BYTES;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    const int total_tiles = p.m_tiles * p.n_tiles;   // 256-row tiles

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(bar_tfull + 8 * a, 1);
            mbar_init(bar_tempty + 8 * a, 16);
        }
        mbar_fence_init();
        for (int i = 0; i < p.npa; ++i) tma_prefetch_desc(&tm.a[i]);
        for (int i = 0; i < p.npb; ++i) tma_prefetch_desc(&tm.b[i]);
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, TMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();   // both CTAs' barriers exist before anyone signals across the pair
    tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(gen_base + 160);

    if (warp == 0 || warp == B_PRODUCER_WARP) {
        // ----------------------------------------------------- TMA producers
        // warp 0 fetches the A planes and posts the stage's byte count, warp 10 fetches the B
        // planes: two issuing threads keep up with the tensor pipe where one could not
        const bool do_a = warp == 0;
        if (lane == 0) {
            uint32_t s = 0, ph = 0;
            bool ok = true;
            const int k_blocks = p.k_blocks, stages = p.stages, npa = p.npa, npb = p.npb;
            const uint32_t sbytes = (uint32_t)stage_bytes;
            grid_dep_wait();   // the operand planes come from the kernel before this one
            if (!do_a && p.cv_taps > 0) {
                // implicit convolution (see gemm_tc.cu): this CTA's 128 columns of the tile are two 64-pixel patches;
                // a stage of B is, per plane, one box per patch at the window offset of the stage's tap
                constexpr int NPATCH = (BN / 2) / 64, PATCH_BYTES = 64 * SWB;
                const int cblocks = p.cv_cblocks, kw = p.cv_kw, pw = p.cv_pw, phh = 64 / p.cv_pw;
                for (int t = pair; t < total_tiles && ok; t += npairs) {
                    int mt, nt;
                    tile_coords(t, p.m_tiles, p.n_tiles, mt, nt);
                    int x0[NPATCH], y0[NPATCH], n0[NPATCH];
#pragma unroll
                    for (int q = 0; q < NPATCH; ++q) {
                        // (a patch past the last one reads sample `batch`: outside the tensor, all zeros)
                        const int patch = (nt * BN + (int)rank * (BN / 2)) / 64 + q, n = patch / p.cv_npatch_s,
                                  rem = patch - n * p.cv_npatch_s, py = rem / p.cv_px;
                        n0[q] = n;
                        x0[q] = (rem - py * p.cv_px) * pw - p.cv_pad_w;
                        y0[q] = py * phh - p.cv_pad_h;
                    }
                    int cb = 0, ky = 0, kx = 0;
                    for (int kb = 0; kb < k_blocks; ++kb) {
                        if (!mbar_wait_bounded(bar_empty + 8 * s, ph ^ 1u)) {
                            report(p.err, ERR_PRODUCER_WAIT);
                            ok = false;
                            break;
                        }
                        const uint32_t fb = map_to_cta(bar_full + 8 * s, 0);
                        uint32_t dst = stage0 + s * sbytes + npa * A_BYTES;
                        for (int i = 0; i < npb; ++i)
#pragma unroll
                            for (int q = 0; q < NPATCH; ++q, dst += PATCH_BYTES)
                                tma_load_4d_pair(dst, &tm.b[i], fb, cb * BKE, x0[q] + kx, y0[q] + ky, n0[q]);
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
            for (int t = pair; t < total_tiles && ok; t += npairs) {
                int mt, nt;
                tile_coords(t, p.m_tiles, p.n_tiles, mt, nt);
                const int row_a = mt * PAIR_TILE_M + (int)rank * BM;
                const int row_b = nt * BN + (int)rank * (BN / 2);
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait_bounded(bar_empty + 8 * s, ph ^ 1u)) {
                        report(p.err, ERR_PRODUCER_WAIT);
                        ok = false;
                        break;
                    }
                    // the leader's barrier collects the bytes of both CTAs
                    const uint32_t fb = map_to_cta(bar_full + 8 * s, 0);
                    {
                        const int kcrd = kb * BKE;
                        if (do_a) {
                            if (leader) mbar_arrive_expect_tx(bar_full + 8 * s, 2u * sbytes);
                            uint32_t dst = stage0 + s * sbytes;
                            for (int i = 0; i < npa; ++i, dst += A_BYTES) tma_load_2d_pair(dst, &tm.a[i], fb, kcrd, row_a);
                        } else {
                            uint32_t dst = stage0 + s * sbytes + npa * A_BYTES;
                            for (int i = 0; i < npb; ++i, dst += B_BYTES) tma_load_2d_pair(dst, &tm.b[i], fb, kcrd, row_b);
                        }
                    }
                    if (++s == (uint32_t)stages) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------- MMA issuer
        if (leader && lane == 0) {
            uint32_t s = 0, ph = 0, vt = 0;
            bool ok = true;
            // everything the issue loop needs lives in registers
            const int k_blocks = p.k_blocks, chunk_kb = p.chunk_kb, stages = p.stages;
            const uint32_t prod_a = p.prod_a, prod_b = p.prod_b;
            const uint64_t desc_hi = smem_desc_kmajor(0, SWB);
            const uint32_t npa_bytes = p.npa * A_BYTES, sbytes = (uint32_t)stage_bytes;
            for (int t = pair; t < total_tiles && ok; t += npairs) {
                for (int kb0 = 0; kb0 < k_blocks && ok; kb0 += chunk_kb, ++vt) {
                    const uint32_t acc = vt & 1u, aph = (vt >> 1) & 1u;
                    if (!mbar_wait_bounded(bar_tempty + 8 * acc, aph ^ 1u)) {
                        report(p.err, ERR_MMA_WAIT_TMEM);
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t d_tmem = tmem_base + acc * BN;
                    const int kb1 = min(k_blocks, kb0 + chunk_kb);
                    for (int kb = kb0; kb < kb1; ++kb) {
                        if (!mbar_wait_bounded(bar_full + 8 * s, ph)) {
                            report(p.err, ERR_MMA_WAIT_FULL);
                            ok = false;
                            break;
                        }
                        tc_fence_after_sync();
                        const uint32_t sa = stage0 + s * sbytes;
                        issue_stage_mmas<KIND, SWB, NPROD, true, A_BYTES, B_BYTES>(
                            d_tmem, sa, sa + npa_bytes, prod_a, prod_b, desc_hi, IDESC, kb == kb0);
                        tc_commit_pair(bar_empty + 8 * s, 0x3);
                        if (++s == (uint32_t)stages) {
                            s = 0;
                            ph ^= 1u;
                        }
                    }
                    if (ok) tc_commit_pair(bar_tfull + 8 * acc, 0x3);
                }
            }
        }
    } else if (warp < B_PRODUCER_WARP) {
        // ---------------------------------------------------------- epilogue
        constexpr int HALF = BN / 2;
        constexpr int PIECES = HALF / 32;
        const int q = warp & 3;
        const int half = (warp - 2) >> 2;
        const int nchunks = (p.k_blocks + p.chunk_kb - 1) / p.chunk_kb;
        uint32_t vt = 0;
        bool alive = true;
        const bool rows_aligned = KIND != KIND_I8 && epi_rows_aligned(p);
        for (int t = pair; t < total_tiles && alive; t += npairs) {
            int mt, nt;
            tile_coords(t, p.m_tiles, p.n_tiles, mt, nt);
            const long long row = (long long)mt * PAIR_TILE_M + (long long)rank * BM + q * 32 + lane;
            const bool row_ok = row < p.M;
            const int col_base = nt * BN + half * HALF;
            const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16) + half * HALF;

            if constexpr (KIND == KIND_I8) {
                const uint32_t acc = vt & 1u, aph = (vt >> 1) & 1u;
                ++vt;
                const bool got = mbar_wait_warp_bounded(bar_tfull + 8 * acc, aph);
                if (!__all_sync(0xffffffffu, got)) {
                    report(p.err, ERR_EPI_WAIT);
                    alive = false;
                    break;
                }
                tc_fence_after_sync();
#pragma unroll 1
                for (int c = 0; c < PIECES; ++c) {
                    const int col0 = col_base + c * 32;
                    if (col0 >= p.N) break;
                    uint32_t r[32];
                    __syncwarp();
                    tmem_ld_32x32(lane_addr + acc * BN + c * 32, r);
                    tmem_ld_wait();
                    store_piece_i8(p, reinterpret_cast<const int *>(r), row, row_ok, col0);
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    if (leader) mbar_arrive(bar_tempty + 8 * acc);
                    else mbar_arrive_cluster(map_to_cta(bar_tempty + 8 * acc, 0));
                }
            } else {
                float sum[HALF];
#pragma unroll
                for (int j = 0; j < HALF; ++j) sum[j] = 0.0f;
                for (int ch = 0; ch < nchunks; ++ch, ++vt) {
                    const uint32_t acc = vt & 1u, aph = (vt >> 1) & 1u;
                    const bool got = mbar_wait_warp_bounded(bar_tfull + 8 * acc, aph);
                    if (!__all_sync(0xffffffffu, got)) {
                        report(p.err, ERR_EPI_WAIT);
                        alive = false;
                        break;
                    }
                    tc_fence_after_sync();
#pragma unroll
                    for (int c = 0; c < PIECES; ++c) {
                        uint32_t r[32];
                        tmem_ld_32x32(lane_addr + acc * BN + c * 32, r);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; ++j) sum[c * 32 + j] += __uint_as_float(r[j]);
                    }
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) {
                        if (leader) mbar_arrive(bar_tempty + 8 * acc);
                        else mbar_arrive_cluster(map_to_cta(bar_tempty + 8 * acc, 0));
                    }
                }
                if (!alive) break;
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

    // the staging tiles must have been read before the shared memory goes away; the global writes themselves are
    // complete when the kernel is
    if (p.tma_store && warp >= 2 && warp < B_PRODUCER_WARP && lane == 0) tma_store_wait_read();

    // ---------------------------------------------------------------- teardown
    if (p.err && *reinterpret_cast<volatile int *>(p.err) != 0) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();   // the peer's shared memory and barriers stay alive until both CTAs are done
    if (warp == 1) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

template <int KIND, int SWB, int NPROD>
static int launch_pair_inst(const TmapPack &tm, KernelArgs &ka, int npa, int npb, int sm_count, cudaStream_t stream,
                            char *err, size_t err_len)
{
    const int stage_bytes = npa * BM * SWB + npb * (PAIR_BN / 2) * SWB;
    constexpr int STAGING = KIND == KIND_I8 ? 0 : EPI_STAGING_BYTES;
    int stages = (SMEM_BUDGET - HEADER_BYTES - 1024 - STAGING) / stage_bytes;
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    if (stages < 2) {
        snprintf(err, err_len, "pair kernel: stage of %d bytes leaves fewer than 2 pipeline stages", stage_bytes);
        return (int)cudaErrorInvalidConfiguration;
    }
    ka.stages = stages;
    const int smem = HEADER_BYTES + 1024 + stages * stage_bytes + STAGING;
    auto kern = gemm_tc_pair_kernel<KIND, SWB, NPROD>;
    static PerDeviceOnce once;
    static int resident_pairs_dev[64] = {};
    if (once.first()) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BUDGET);
        if (e != cudaSuccess) {
            snprintf(err, err_len, "pair kernel: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
            return (int)e;
        }
    }
    int &resident_pairs = resident_pairs_dev[once.device()];
    // how many CTA pairs the device can hold at once (an SM without a free partner in its
    // cluster-scheduling group cannot host half a pair): persistent grid = that many pairs
    if (resident_pairs == 0) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(sm_count / 2 * 2));
        cfg.blockDim = dim3(NUM_THREADS);
        cfg.dynamicSmemBytes = (size_t)smem;
        cudaLaunchAttribute at;
        at.id = cudaLaunchAttributeClusterDimension;
        at.val.clusterDim.x = 2;
        at.val.clusterDim.y = 1;
        at.val.clusterDim.z = 1;
        cfg.attrs = &at;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) == cudaSuccess && n > 0) resident_pairs = n;
        else resident_pairs = sm_count / 2;
        (void)cudaGetLastError();
    }
    const long long tiles = (long long)ka.m_tiles * ka.n_tiles;
    long long pairs = resident_pairs;
    if (pairs > sm_count / 2) pairs = sm_count / 2;
    if (pairs > tiles) pairs = tiles;
    // programmatic dependent launch, as in the single-CTA launcher: set-up overlaps the operand pre-pass's tail
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3((unsigned)(2 * pairs));
    lc.blockDim = dim3(NUM_THREADS);
    lc.dynamicSmemBytes = (size_t)smem;
    lc.stream = stream;
    cudaLaunchAttribute lat;
    lat.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    lat.val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = &lat;
    lc.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&lc, kern, tm, ka);
    if (e != cudaSuccess) snprintf(err, err_len, "pair kernel launch: %s", cudaGetErrorString(e));
    return (int)e;
}

int launch_gemm_tc_pair(int kind, int swb, int nprod, const TmapPack &tm, KernelArgs &ka, int npa, int npb,
                        int sm_count, cudaStream_t stream, char *err, size_t err_len)
{
    if (kind == KIND_TF32 && nprod == 3 && swb == 64)
        return launch_pair_inst<KIND_TF32, 64, 3>(tm, ka, npa, npb, sm_count, stream, err, err_len);
    if (kind == KIND_BF16 && nprod == 3 && swb == 64)
        return launch_pair_inst<KIND_BF16, 64, 3>(tm, ka, npa, npb, sm_count, stream, err, err_len);
    if (kind == KIND_TF32 && nprod == 3 && swb == 128)
        return launch_pair_inst<KIND_TF32, 128, 3>(tm, ka, npa, npb, sm_count, stream, err, err_len);
    if (kind == KIND_BF16 && nprod == 3 && swb == 128)
        return launch_pair_inst<KIND_BF16, 128, 3>(tm, ka, npa, npb, sm_count, stream, err, err_len);
    if (kind == KIND_BF16 && nprod == 1 && swb == 128)
        return launch_pair_inst<KIND_BF16, 128, 1>(tm, ka, npa, npb, sm_count, stream, err, err_len);
    if (kind == KIND_I8 && nprod == 1)
        return launch_pair_inst<KIND_I8, 128, 1>(tm, ka, npa, npb, sm_count, stream, err, err_len);
    snprintf(err, err_len, "pair kernel: no instantiation for kind %d with %d products", kind, nprod);
    return (int)cudaErrorInvalidValue;
}

}  // namespace axb
