// gemm_tc_internal.cuh — definitions shared by the two tcgen05 GEMM kernels
// (gemm_tc.cu: one CTA per tile; gemm_tc2.cu: a CTA pair per tile).
#pragma once
#include "gemm_tc.cuh"
#include "qskinny_tc.cuh"
#include "ptx.cuh"

#include <cuda.h>
#include <type_traits>

namespace axb {

static constexpr int BM = 128;
static constexpr int GROUP_M = 16;
static constexpr int NUM_THREADS = 352;  // A-producer warp, MMA warp, 8 epilogue warps, B-producer warp
static constexpr int B_PRODUCER_WARP = 10;
static constexpr int HEADER_BYTES = 1024;
static constexpr int MAX_STAGES = 8;
static constexpr int SMEM_BUDGET = 227 * 1024;
static constexpr int EPI_STAGING_BYTES = 8 * 4096;   // fp32 kinds: one 32 x 32 fp32 tile per epilogue warp, after the ring

struct alignas(64) TmapPack {
    CUtensorMap a[TC_MAX_PLANES];
    CUtensorMap b[TC_MAX_PLANES];
    // fp32 output, box 32 x 32, 128-byte swizzle (valid when KernelArgs::tma_store): c[0] over C [M, N]; with the
    // head-major scatter c[which] over hs_out[which] seen as a matrix of B*H*S rows of hs_dk floats
    CUtensorMap c[3];
};

struct KernelArgs {
    int M, N, K;
    int npa, npb, nprod;
    uint32_t prod_a, prod_b;  // plane index of product i in bits [4i, 4i+4): registers, never indexed memory
    int m_tiles, n_tiles, k_blocks, stages;
    int chunk_kb;  // k-blocks accumulated in TMEM before the epilogue warps drain them
    float alpha, beta;
    const float *bias;
    const float *colscale;
    float rq_a_scale, rq_out_scale;   // int8 requantisation: multiplier = (rq_a_scale * colscale[n]) / rq_out_scale
    int act, out_mode;
    void *C;
    int32_t *acc_out;
    long long ldc;
    int *err;
    float *c_extra[TC_MAX_EXTRA];
    int n_extra;
    const float *dg_inv_s;   // OUT_DIGITS_T, see TcEpilogue
    int dg_rows;
    int hs_dk, hs_S, hs_H;   // head-major scatter of the output (hs_dk > 0), see TcEpilogue
    // fp32 output leaves through TMA copies of the staging tiles (aligned; plain C or head-major): 1 = stores (beta == 0),
    // 2 = reduce-adds (beta == 1 without bias and activation: C += alpha * sums, one rounded addition per element in
    // the memory system, C is never read into the SM)
    int tma_store;
    float *hs_out[3];
    // split-K (ksplit > 1): work item w = tile * ksplit + slice covers k-blocks [slice * kb_per_slice, ...); every
    // slice leaves its partial sums in sk_scratch and counts itself in on sk_counters[tile]; the slice that counts
    // last adds all of them in slice order and runs the epilogue (no CTA ever waits for another)
    int ksplit, kb_per_slice;
    void *sk_scratch;        // [tiles x CTAs per tile][ksplit][128 x BN] fp32 / s32
    int *sk_counters;        // [tiles x CTAs per tile], zero between launches
    // sk_cluster (fp32 kinds, ksplit == 2, one work item per CTA): the two slices of a tile are one thread-block
    // cluster and meet in shared memory instead of scratch — each CTA pushes the column half it does not finish into
    // its partner's epilogue staging area, one cluster barrier, and each finishes and stores its own half
    int sk_cluster;
    // implicit convolution (cv_taps > 0, see TcConv): the B maps are 4-D over the image planes [batch][H][W][C] with
    // one box per 64-pixel patch (cv_pw x 64/cv_pw pixels of one sample); output column j of the GEMM is pixel j % 64
    // of patch j / 64, patches numbered sample-major (cv_npatch_s per sample, cv_px per patch row), stored by
    // store_piece_f32_conv (ldc = out_h * out_w, samples M * ldc apart)
    int cv_taps, cv_kw, cv_cblocks, cv_pw, cv_px, cv_npatch, cv_npatch_s, cv_pad_w, cv_pad_h, cv_out_w;
};

// shared-memory header words used by the split-K hand-over (after the barriers and the TMEM slot)
static constexpr int HDR_SK_DEAD = 176, HDR_SK_LAST = 180;

// error words written to *err (first writer wins)
enum { ERR_PRODUCER_WAIT = 1, ERR_MMA_WAIT_FULL = 2, ERR_MMA_WAIT_TMEM = 3, ERR_EPI_WAIT = 4 };

__device__ __forceinline__ void report(int *err, int code)
{
    if (err) atomicCAS(err, 0, code);
}

__device__ __forceinline__ void tile_coords(int t, int m_tiles, int n_tiles, int &mt, int &nt)
{
    const int per_group = GROUP_M * n_tiles;
    const int g = t / per_group;
    const int first_m = g * GROUP_M;
    const int gm = min(GROUP_M, m_tiles - first_m);
    const int r = t - g * per_group;
    mt = first_m + r % gm;
    nt = r / gm;
}

// where the 32 output columns starting at col0 of output row `row` go
__device__ __forceinline__ float *out_piece_ptr(const KernelArgs &p, long long row, int col0)
{
    if (p.hs_dk == 0) return reinterpret_cast<float *>(p.C) + row * p.ldc + col0;
    const int D = p.hs_H * p.hs_dk;
    const int which = col0 / D, rem = col0 - which * D, h = rem / p.hs_dk, d0 = rem - h * p.hs_dk;
    const long long b = row / p.hs_S, s = row - b * p.hs_S;
    return p.hs_out[which] + ((b * p.hs_H + h) * p.hs_S + s) * p.hs_dk + d0;
}

// GELU, tanh form (ax_gelu: src/core/activations.c:267-333): 0.5 v (1 + tanh(u)) = v / (1 + exp(-2u)),
// u = 0.79788456 (v + 0.044715 v^3), on the fast exponential and reciprocal: eight dependent instructions, two of them
// on the special-function pipe, absolute error below 1e-6 * |v|.  exp(-2u) = 2^(-k w) with w = v + 0.044715 v^3 and
// k = 2 * 0.79788456 * log2(e); it overflows to +inf for very negative v (result -0) and underflows to 0 for large v
// (result v).
__device__ __forceinline__ float gelu_tanh(float v)
{
    const float w = fmaf(0.044715f * v * v, v, v);
    float t;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(-2.302208198f * w));
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + t));
    return v * r;
}

// fp32 epilogue of one warp's 32 x 32 piece.  The sums arrive row-per-lane (that is how TMEM is read); they are
// laid into a shared-memory tile (16-byte chunks XOR-swizzled, no bank conflicts either way) and read back so that
// eight lanes cover the 128 bytes of a row: every global access is whole 128-byte lines, C is read the same way
// when beta != 0, and the scale / bias / activation arithmetic sits in short ROLLED loops.  The first version kept
// a row per lane and unrolled everything: 170 KB of straight-line code per kernel (128 inlined tanh), fetched again
// for every tile through an L2 path the operand loads already saturate — 75 000 cycles per tile, longer than a
// K = 1024 main loop.
__device__ __forceinline__ float epi_act(float x, int act)
{
    if (act == ACT_RELU) return fmaxf(x, 0.0f);
    if (act == ACT_GELU) return gelu_tanh(x);
    return x;
}

// Scale, bias and activation applied IN a warp's staging tile (lane -> 16-byte column group lane & 7 of rows lane >> 3,
// + 4, ...).  One copy per kernel (not inlined: the piece loop around it is unrolled four times), the activation chosen
// once, and the eight groups of a lane handled four at a time — loads first, then sixteen independent chains, then the
// stores: with one group per step the exponential / reciprocal chains of the GELU ran one after the other and the pass
// (28 k cycles per tile with the stores' turn-around) outlasted the two accumulator chunks the MMAs can run ahead.
static __device__ __noinline__ void epi_staging_pass(float4 *stg, int lane, float alpha, float4 cs, float4 bs, int act)
{
    const int ch = lane & 7, r0 = lane >> 3;
#pragma unroll 1
    for (int h = 0; h < 2; ++h) {
        float4 v[4];
        int idx[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int r = (h * 4 + j) * 4 + r0;
            idx[j] = r * 8 + (ch ^ (r & 7));
            v[j] = stg[idx[j]];
            // (the same expression as the plain-store path, so that both give the same bits)
            v[j] = make_float4(v[j].x * alpha * cs.x + bs.x, v[j].y * alpha * cs.y + bs.y, v[j].z * alpha * cs.z + bs.z, v[j].w * alpha * cs.w + bs.w);
        }
        if (act == ACT_GELU) {
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = make_float4(gelu_tanh(v[j].x), gelu_tanh(v[j].y), gelu_tanh(v[j].z), gelu_tanh(v[j].w));
        } else if (act == ACT_RELU) {
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = make_float4(fmaxf(v[j].x, 0.0f), fmaxf(v[j].y, 0.0f), fmaxf(v[j].z, 0.0f), fmaxf(v[j].w, 0.0f));
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) stg[idx[j]] = v[j];
    }
}

static __device__ __forceinline__ void store_piece_f32(const KernelArgs &p, const float4 *stg, long long row0, int col0, int lane,
                                             bool aligned)
{
    if (aligned && col0 + 32 <= p.N) {
        const int ch = lane & 7, colv = col0 + ch * 4;
        float cs[4] = { 1.f, 1.f, 1.f, 1.f }, bs[4] = { 0.f, 0.f, 0.f, 0.f };
        if (p.colscale) { cs[0] = __ldg(p.colscale + colv); cs[1] = __ldg(p.colscale + colv + 1); cs[2] = __ldg(p.colscale + colv + 2); cs[3] = __ldg(p.colscale + colv + 3); }
        if (p.bias) { bs[0] = __ldg(p.bias + colv); bs[1] = __ldg(p.bias + colv + 1); bs[2] = __ldg(p.bias + colv + 2); bs[3] = __ldg(p.bias + colv + 3); }
        if (p.beta == 0.0f) {
            // nothing is read back: the arithmetic is done in the staging tile by the same pass the TMA-store path uses
            // (the same code, so the same bits), and what is left is a copy of finished 16-byte groups to every
            // destination — with the activation inline, a GELU in front of eight peer stores per group held the
            // epilogue warps longer than the two accumulator chunks the MMAs can run ahead
            if (p.alpha != 1.0f || p.colscale || p.bias || p.act != ACT_NONE)
                epi_staging_pass(const_cast<float4 *>(stg), lane, p.alpha, make_float4(cs[0], cs[1], cs[2], cs[3]),
                                 make_float4(bs[0], bs[1], bs[2], bs[3]), p.act);
#pragma unroll 2
            for (int it = 0; it < 8; ++it) {
                const int r = it * 4 + (lane >> 3);
                if (row0 + r >= p.M) continue;
                const float4 o = stg[r * 8 + (ch ^ (r & 7))];
                *reinterpret_cast<float4 *>(out_piece_ptr(p, row0 + r, col0) + ch * 4) = o;
                for (int e = 0; e < p.n_extra; ++e)
                    *reinterpret_cast<float4 *>(p.c_extra[e] + (row0 + r) * p.ldc + colv) = o;
            }
            return;
        }
#pragma unroll 2
        for (int it = 0; it < 8; ++it) {
            const int r = it * 4 + (lane >> 3);
            if (row0 + r >= p.M) continue;
            const float4 v = stg[r * 8 + (ch ^ (r & 7))];
            float *dst = out_piece_ptr(p, row0 + r, col0) + ch * 4;
            float x[4] = { v.x * p.alpha * cs[0], v.y * p.alpha * cs[1], v.z * p.alpha * cs[2], v.w * p.alpha * cs[3] };
            if (p.beta != 0.0f) {
                const float4 c = *reinterpret_cast<const float4 *>(dst);
                x[0] += p.beta * c.x; x[1] += p.beta * c.y; x[2] += p.beta * c.z; x[3] += p.beta * c.w;
            }
            const float4 o = make_float4(epi_act(x[0] + bs[0], p.act), epi_act(x[1] + bs[1], p.act),
                                         epi_act(x[2] + bs[2], p.act), epi_act(x[3] + bs[3], p.act));
            *reinterpret_cast<float4 *>(dst) = o;
            for (int e = 0; e < p.n_extra; ++e)
                *reinterpret_cast<float4 *>(p.c_extra[e] + (row0 + r) * p.ldc + colv) = o;
        }
    } else {
        // ragged last piece or unaligned rows: lane = column, one 128-byte row per iteration
        const int col = col0 + lane;
        const bool ok = col < p.N;
        const float cs = (p.colscale && ok) ? __ldg(p.colscale + col) : 1.0f;
        const float bs = (p.bias && ok) ? __ldg(p.bias + col) : 0.0f;
        const float *sf = reinterpret_cast<const float *>(stg);
#pragma unroll 1
        for (int r = 0; r < 32; ++r) {
            if (!ok || row0 + r >= p.M) continue;
            float *dst = out_piece_ptr(p, row0 + r, col0) + lane;
            float x = sf[r * 32 + (((lane >> 2) ^ (r & 7)) << 2) + (lane & 3)] * p.alpha * cs;
            if (p.beta != 0.0f) x += p.beta * *dst;
            x = epi_act(x + bs, p.act);
            *dst = x;
            for (int e = 0; e < p.n_extra; ++e) p.c_extra[e][(row0 + r) * p.ldc + col] = x;
        }
    }
}

// every row start of every fp32 destination is 16-byte aligned: the 128-bit path of store_piece_f32 may be used
__device__ __forceinline__ bool epi_rows_aligned(const KernelArgs &p)
{
    uintptr_t al;
    if (p.hs_dk > 0) {
        al = reinterpret_cast<uintptr_t>(p.hs_out[0]) | reinterpret_cast<uintptr_t>(p.hs_out[1]) | reinterpret_cast<uintptr_t>(p.hs_out[2]);
    } else {
        al = reinterpret_cast<uintptr_t>(p.C) | (uintptr_t)((p.ldc & 3) != 0 ? 4 : 0);
        for (int e = 0; e < p.n_extra; ++e) al |= reinterpret_cast<uintptr_t>(p.c_extra[e]);
    }
    return (al & 15) == 0;
}

// The same epilogue when C is a plain aligned matrix that is not read back: the arithmetic is done IN the staging
// tile (rolled loop, shared memory only) and the tile leaves as one TMA store — the staging layout is the 128-byte
// swizzle the tensor map names, rows and columns past M and N are clipped by the hardware, and the warp does not
// wait for the global writes, only (before it reuses the tile) for the engine to have read it.
static __device__ __forceinline__ void store_piece_f32_tma(const KernelArgs &p, const CUtensorMap *tmc, float4 *stg,
                                                           long long row0, int col0, int lane)
{
    if (p.alpha != 1.0f || p.colscale || p.bias || p.act != ACT_NONE) {
        const int ch = lane & 7, colv = col0 + ch * 4;
        float cs[4] = { 1.f, 1.f, 1.f, 1.f }, bs[4] = { 0.f, 0.f, 0.f, 0.f };
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            if (p.colscale && colv + e < p.N) cs[e] = __ldg(p.colscale + colv + e);
            if (p.bias && colv + e < p.N) bs[e] = __ldg(p.bias + colv + e);
        }
        epi_staging_pass(stg, lane, p.alpha, make_float4(cs[0], cs[1], cs[2], cs[3]), make_float4(bs[0], bs[1], bs[2], bs[3]), p.act);
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
        if (p.hs_dk > 0) {
            // head-major: the piece's 32 rows (b, s0..s0+31: hs_S % 32 == 0) and 32 columns (head h, d0..d0+31) are a
            // 32 x 32 box at row (b*H + h)*S + s0 of destination `which`
            const int D = p.hs_H * p.hs_dk;
            const int which = col0 / D, rem = col0 - which * D, h = rem / p.hs_dk, d0 = rem - h * p.hs_dk;
            const long long b = row0 / p.hs_S, s0 = row0 - b * p.hs_S;
            const int32_t r0 = (int32_t)((b * p.hs_H + h) * p.hs_S + s0);
            if (p.tma_store == 2) tma_reduce_add_2d(tmc + which, smem_u32(stg), d0, r0);
            else tma_store_2d(tmc + which, smem_u32(stg), d0, r0);
        } else if (p.tma_store == 2) {
            tma_reduce_add_2d(tmc, smem_u32(stg), col0, (int32_t)row0);
        } else {
            tma_store_2d(tmc, smem_u32(stg), col0, (int32_t)row0);
        }
        tma_store_commit();
    }
}

// The fp32 epilogue of an implicit convolution (alpha and activation only): the piece's 32 columns are 32 / cv_pw
// pixel rows of cv_pw pixels of one patch, so each 16-byte group of the staging tile goes to its own place in
// out[sample][row][oh][ow] (ldc = out_h * out_w; out_w % 4 == 0 keeps every group inside one pixel row and
// 16-byte aligned).  Pixels past the right and bottom edges of the image are dropped.
static __device__ __forceinline__ void store_piece_f32_conv(const KernelArgs &p, const float4 *stg, long long row0, int col0, int lane)
{
    const int patch = col0 >> 6;
    if (patch >= p.cv_npatch) return;
    const int n = patch / p.cv_npatch_s, rem = patch - n * p.cv_npatch_s, py = rem / p.cv_px, px = rem - py * p.cv_px;
    const int ch = lane & 7, j = (col0 & 63) + ch * 4;            // pixel index inside the patch of this lane's group
    const int out_w = p.cv_out_w, oh = py * (64 / p.cv_pw) + j / p.cv_pw, ow = px * p.cv_pw + j % p.cv_pw;
    if (ow >= out_w || (long long)oh * out_w >= p.ldc) return;
    float *dst0 = reinterpret_cast<float *>(p.C) + (long long)n * p.M * p.ldc + (long long)oh * out_w + ow;
#pragma unroll 2
    for (int it = 0; it < 8; ++it) {
        const int r = it * 4 + (lane >> 3);
        if (row0 + r >= p.M) continue;
        const float4 v = stg[r * 8 + (ch ^ (r & 7))];
        *reinterpret_cast<float4 *>(dst0 + (row0 + r) * p.ldc) =
            make_float4(epi_act(v.x * p.alpha, p.act), epi_act(v.y * p.alpha, p.act), epi_act(v.z * p.alpha, p.act),
                        epi_act(v.w * p.alpha, p.act));
    }
}

// All MMAs of one pipeline stage, fully unrolled.  tcgen05.mma holds the issuing thread while
// the tensor pipe is busy and the pipe queues next to nothing, so every scalar instruction
// between two MMAs is time the pipe idles: descriptors are one OR and one ADD away from
// registers, the product list is a bitfield, there are no loops, divisions or memory accesses.
template <int KIND, int SWB, int NPROD, bool PAIR, int A_BYTES, int B_BYTES>
__device__ __forceinline__ void issue_stage_mmas(uint32_t d_tmem, uint32_t sa, uint32_t sb, uint32_t prod_a,
                                                 uint32_t prod_b, uint64_t desc_hi, uint32_t idesc, bool first)
{
    // Order: per 64 bytes of K (two MMA steps) all products, then the next 64 bytes.  A 128-byte stage therefore
    // accumulates exactly like two 64-byte stages, so kernels with different stage widths (the tile heuristics pick
    // them by shape) give bit-identical results — what makes a row-chunked GEMM equal to the whole one.
    constexpr int KSTEPS = SWB / 32;
#pragma unroll
    for (int g = 0; g < KSTEPS / 2; ++g) {
#pragma unroll
        for (int pr = 0; pr < NPROD; ++pr) {
            const uint32_t ia = (prod_a >> (4 * pr)) & 15u, ib = (prod_b >> (4 * pr)) & 15u;
            const uint64_t da = desc_hi | (uint64_t)((sa + ia * A_BYTES) >> 4);
            const uint64_t db = desc_hi | (uint64_t)((sb + ib * B_BYTES) >> 4);
#pragma unroll
            for (int ks = 2 * g; ks < 2 * g + 2; ++ks) {
                const uint32_t accumulate = (g == 0 && pr == 0 && ks == 0) ? (first ? 0u : 1u) : 1u;
                if constexpr (PAIR) tc_mma_pair<KIND>(d_tmem, da + 2u * ks, db + 2u * ks, idesc, accumulate);
                else tc_mma<KIND>(d_tmem, da + 2u * ks, db + 2u * ks, idesc, accumulate);
            }
        }
    }
}

// barrier over the eight epilogue warps only (the producer and MMA warps never take part)
__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

enum { SK_DEAD = 0, SK_NOT_LAST = 1, SK_LAST = 2 };

// Split-K hand-over of one CTA's 128 x (2*HALF) partial tile.  `v` holds this thread's row (lane) x HALF columns.
// Every slice stores its partials to scratch in a thread-private order (the same thread of the same warp role reads
// them back, so the layout only has to be coalesced: consecutive lanes write consecutive 16-byte words), makes them
// visible device-wide and counts itself in.  The slice that counts last reloads ALL slices, its own included, and
// adds them in slice order, so the sum does not depend on which slice happened to finish last: results are bitwise
// repeatable.  Nobody waits for anybody.  `alive` = this warp's accumulator wait succeeded; a failed wait is
// agreed on by all eight warps here (they must keep meeting at the barrier) and ends the kernel's epilogue.
template <typename T, int HALF>
__device__ __forceinline__ int splitk_exchange(const KernelArgs &p, T (&v)[HALF], long long region, int slice, int warp,
                                               int lane, uint8_t *hdr, bool alive)
{
    constexpr int PIECES = HALF / 32;
    constexpr size_t SLICE_ELEMS = (size_t)BM * 2 * HALF;
    using V4 = typename std::conditional<std::is_same<T, float>::value, float4, int4>::type;
    volatile int *dead = reinterpret_cast<volatile int *>(hdr + HDR_SK_DEAD);
    volatile int *last = reinterpret_cast<volatile int *>(hdr + HDR_SK_LAST);
    T *tile0 = reinterpret_cast<T *>(p.sk_scratch) + (size_t)region * p.ksplit * SLICE_ELEMS;
    const size_t warp_off = (size_t)(warp - 2) * 32 * HALF;
    if (alive) {
        V4 *mine = reinterpret_cast<V4 *>(tile0 + (size_t)slice * SLICE_ELEMS + warp_off);
#pragma unroll
        for (int c = 0; c < PIECES; ++c)
#pragma unroll
            for (int j4 = 0; j4 < 8; ++j4) {
                V4 w;
                w.x = v[c * 32 + 4 * j4]; w.y = v[c * 32 + 4 * j4 + 1]; w.z = v[c * 32 + 4 * j4 + 2]; w.w = v[c * 32 + 4 * j4 + 3];
                mine[(c * 8 + j4) * 32 + lane] = w;
            }
        __threadfence();
    } else {
        *dead = 1;
    }
    epi_bar_sync();
    if (warp == 2 && lane == 0) {
        int is_last = 0;
        if (!*dead) {
            const int old = atomicAdd(p.sk_counters + region, 1);
            if (old == p.ksplit - 1) {
                is_last = 1;
                p.sk_counters[region] = 0;   // every slice has counted: ready for the next launch
            }
        }
        *last = is_last;
    }
    epi_bar_sync();
    if (*dead) return SK_DEAD;
    if (!*last) return SK_NOT_LAST;
    __threadfence();
#pragma unroll
    for (int j = 0; j < HALF; ++j) v[j] = T(0);
    for (int s = 0; s < p.ksplit; ++s) {
        const V4 *src = reinterpret_cast<const V4 *>(tile0 + (size_t)s * SLICE_ELEMS + warp_off);
#pragma unroll
        for (int c = 0; c < PIECES; ++c)
#pragma unroll
            for (int j4 = 0; j4 < 8; ++j4) {
                const V4 w = __ldcg(src + (c * 8 + j4) * 32 + lane);
                v[c * 32 + 4 * j4] += w.x; v[c * 32 + 4 * j4 + 1] += w.y; v[c * 32 + 4 * j4 + 2] += w.z; v[c * 32 + 4 * j4 + 3] += w.w;
            }
    }
    return SK_LAST;
}

// int8 epilogue of 32 accumulator columns of one row: raw s32 to acc_out and / or the requantised int8 to C.
// Called by all 32 lanes of a warp together (lane = row): lane j forms the multiplier of column col0 + j — one
// division per lane instead of 32 per thread — and the row loops fetch it with a shuffle.
__device__ __forceinline__ void store_piece_i8(const KernelArgs &p, const int *r, long long row, bool row_ok, int col0)
{
    if (p.out_mode == OUT_DIGITS_T) {
        // columns 4*m + j of this thread's accumulator row n are the four digit planes of activation row m: recombined
        // here in 64-bit integers (exact), scaled, and stored transposed — the lanes of a warp are 32 consecutive n of
        // one output row m, whole 128-byte lines
        const int m0 = col0 >> 2;
        const float sc = row_ok ? __ldg(p.colscale + row) : 0.0f, bs = (row_ok && p.bias) ? __ldg(p.bias + row) : 0.0f;
        float *out = reinterpret_cast<float *>(p.C);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int m = m0 + i;
            const long long t = (long long)r[4 * i] + ((long long)r[4 * i + 1] << 8) + ((long long)r[4 * i + 2] << 16) +
                                ((long long)r[4 * i + 3] << 24);
            if (row_ok && m < p.dg_rows) out[(long long)m * p.ldc + row] = qt_finish(t, __ldg(p.dg_inv_s + m), sc, bs, p.act);
        }
        return;
    }
    const bool full = col0 + 32 <= p.N;
    if (p.acc_out && row_ok) {
        int32_t *dst = p.acc_out + row * p.ldc + col0;
        if (full && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) *reinterpret_cast<int4 *>(dst + j) = make_int4(r[j], r[j + 1], r[j + 2], r[j + 3]);
        } else {
            for (int j = 0; j < 32 && col0 + j < p.N; ++j) dst[j] = r[j];
        }
    }
    if (p.out_mode == OUT_I8_REQUANT) {
        const int lane = threadIdx.x & 31;
        // (a_scale * b_scales[n]) / out_scale with one rounding per operation, as the CPU restatement does it
        const float my_mult = (col0 + lane < p.N) ? __fdiv_rn(__fmul_rn(p.rq_a_scale, __ldg(p.colscale + col0 + lane)), p.rq_out_scale) : 0.0f;
        uint32_t packed[8];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const float mult = __shfl_sync(0xffffffffu, my_mult, j);
            const float y = __fmul_rn(__int2float_rn(r[j]), mult);
            int v = __float2int_rn(y);
            v = max(-127, min(127, v));
            if ((j & 3) == 0) packed[j >> 2] = 0;
            packed[j >> 2] |= (uint32_t)(v & 0xff) << (8 * (j & 3));
        }
        if (row_ok) {
            int8_t *dst = reinterpret_cast<int8_t *>(p.C) + row * p.ldc + col0;
            if (full && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
                *reinterpret_cast<uint4 *>(dst) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                *reinterpret_cast<uint4 *>(dst + 16) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
            } else {
                for (int j = 0; j < 32 && col0 + j < p.N; ++j) dst[j] = (int8_t)((packed[j >> 2] >> (8 * (j & 3))) & 0xff);
            }
        }
    }
}

// gemm_tc2.cu: the CTA-pair kernel (256 x 256 tiles; ka.m_tiles counts 256-row tiles, the B maps have 128-row boxes)
int launch_gemm_tc_pair(int kind, int swb, int nprod, const TmapPack &tm, KernelArgs &ka, int npa, int npb, int sm_count,
                        cudaStream_t stream, char *err, size_t err_len);

}  // namespace axb
