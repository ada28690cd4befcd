// prepass.cu — operand preparation for the tcgen05 GEMM core, all HBM-bound:
//   * split an fp32 matrix into K-major tensor-core planes (tf32 hi/lo, or
//     bf16 hi/mid/lo), transposing on the way when the source is stored with
//     the contraction index outermost;
//   * widen int8 weights to an (exact) bf16 plane for the W8A32 path;
//   * re-pitch int8 operands whose row length is not a multiple of 16 bytes;
//   * the per-column requantisation multiplier and the row quantiser.
#include "prepass.cuh"
#include "ptx.cuh"

#include <cuda_bf16.h>
#include <stdint.h>

namespace axb {

__device__ __forceinline__ float tf32_round(float x)
{
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}

// value -> planes; MODE as SplitMode.  Every residual is exact in fp32, so the
// planes sum to the input up to the rounding of the LAST plane only.
template <int MODE>
__device__ __forceinline__ void split1(float x, float &t0, float &t1, __nv_bfloat16 &b0,
                                       __nv_bfloat16 &b1, __nv_bfloat16 &b2)
{
    if constexpr (MODE == SPLIT_TF32X2) {
        t0 = tf32_round(x);
        t1 = tf32_round(x - t0);
    } else {
        b0 = __float2bfloat16_rn(x);
        if constexpr (MODE >= SPLIT_BF16X2) {
            const float r1 = x - __bfloat162float(b0);
            b1 = __float2bfloat16_rn(r1);
            if constexpr (MODE >= SPLIT_BF16X3) b2 = __float2bfloat16_rn(r1 - __bfloat162float(b1));
        }
    }
}

template <int MODE>
__device__ __forceinline__ void store1(void *const *pl, int64_t idx, float x)
{
    float t0 = 0, t1 = 0;
    __nv_bfloat16 b0, b1, b2;
    split1<MODE>(x, t0, t1, b0, b1, b2);
    if constexpr (MODE == SPLIT_TF32X2) {
        reinterpret_cast<float *>(pl[0])[idx] = t0;
        reinterpret_cast<float *>(pl[1])[idx] = t1;
    } else {
        reinterpret_cast<__nv_bfloat16 *>(pl[0])[idx] = b0;
        if constexpr (MODE >= SPLIT_BF16X2) reinterpret_cast<__nv_bfloat16 *>(pl[1])[idx] = b1;
        if constexpr (MODE >= SPLIT_BF16X3) reinterpret_cast<__nv_bfloat16 *>(pl[2])[idx] = b2;
    }
}

// two k-adjacent values at an even index: one 8-byte (tf32) or 4-byte (bf16) store per plane
template <int MODE>
__device__ __forceinline__ void store2(void *const *pl, int64_t idx, float x, float y)
{
    float xt0 = 0, xt1 = 0, yt0 = 0, yt1 = 0;
    __nv_bfloat16 xb[3], yb[3];
    split1<MODE>(x, xt0, xt1, xb[0], xb[1], xb[2]);
    split1<MODE>(y, yt0, yt1, yb[0], yb[1], yb[2]);
    if constexpr (MODE == SPLIT_TF32X2) {
        *reinterpret_cast<float2 *>(reinterpret_cast<float *>(pl[0]) + idx) = make_float2(xt0, yt0);
        *reinterpret_cast<float2 *>(reinterpret_cast<float *>(pl[1]) + idx) = make_float2(xt1, yt1);
    } else {
        constexpr int NP = MODE == SPLIT_BF16X1 ? 1 : (MODE == SPLIT_BF16X2 ? 2 : 3);
#pragma unroll
        for (int q = 0; q < NP; ++q)
            *reinterpret_cast<uint32_t *>(reinterpret_cast<__nv_bfloat16 *>(pl[q]) + idx) =
                (uint32_t)__bfloat16_as_ushort(xb[q]) | ((uint32_t)__bfloat16_as_ushort(yb[q]) << 16);
    }
}

struct PlanePtrs {
    void *p[3];
};

// in [rows, k] (k contiguous, row pitch ld) -> planes [rows, pitch]; 4 elements / thread
template <int MODE>
__device__ __forceinline__ void split_rows_body(const float *__restrict__ in, int64_t rows, int64_t k, int64_t ld,
                                                const PlanePtrs &pl, int64_t pitch, int64_t chunk_k,
                                                int64_t chunk_stride, int vblock, int vgrid)
{
    const int64_t k4 = (k + 3) / 4;
    const int64_t total = rows * k4;
    const bool vec = (ld % 4 == 0) && ((reinterpret_cast<uintptr_t>(in) & 15) == 0);
    for (int64_t i = (int64_t)vblock * blockDim.x + threadIdx.x; i < total; i += (int64_t)vgrid * blockDim.x) {
        const int64_t r = i / k4, c = (i - r * k4) * 4;
        // chunk_k > 0: the k range is cut into chunks stored as separate [rows, chunk_k] blocks chunk_stride
        // apart (the layout an all-gather of column slabs leaves behind); chunk_k % 4 == 0
        const float *src = chunk_k > 0 ? in + (c / chunk_k) * chunk_stride + r * chunk_k + (c % chunk_k) : in + r * ld + c;
        float x[4];
        if (vec && c + 4 <= k) {
            const float4 v = __ldg(reinterpret_cast<const float4 *>(src));
            x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) x[j] = (c + j < k) ? __ldg(src + j) : 0.0f;
        }
        const int64_t o = r * pitch + c;  // pitch % 16 == 0, so 4-element groups never straddle
        if constexpr (MODE == SPLIT_TF32X2) {
            float4 hi, lo;
            hi.x = tf32_round(x[0]); lo.x = tf32_round(x[0] - hi.x);
            hi.y = tf32_round(x[1]); lo.y = tf32_round(x[1] - hi.y);
            hi.z = tf32_round(x[2]); lo.z = tf32_round(x[2] - hi.z);
            hi.w = tf32_round(x[3]); lo.w = tf32_round(x[3] - hi.w);
            *reinterpret_cast<float4 *>(reinterpret_cast<float *>(pl.p[0]) + o) = hi;
            *reinterpret_cast<float4 *>(reinterpret_cast<float *>(pl.p[1]) + o) = lo;
        } else {
            __nv_bfloat16 b[3][4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float t0, t1;
                split1<MODE>(x[j], t0, t1, b[0][j], b[1][j], b[2][j]);
            }
            constexpr int NP = MODE == SPLIT_BF16X1 ? 1 : (MODE == SPLIT_BF16X2 ? 2 : 3);
#pragma unroll
            for (int q = 0; q < NP; ++q) {
                uint2 w;
                w.x = (uint32_t)__bfloat16_as_ushort(b[q][0]) | ((uint32_t)__bfloat16_as_ushort(b[q][1]) << 16);
                w.y = (uint32_t)__bfloat16_as_ushort(b[q][2]) | ((uint32_t)__bfloat16_as_ushort(b[q][3]) << 16);
                *reinterpret_cast<uint2 *>(reinterpret_cast<__nv_bfloat16 *>(pl.p[q]) + o) = w;
            }
        }
    }
}

// in [k, rows] (rows contiguous, pitch ld) -> planes [rows, pitch] (k contiguous):
// 64(k) x 32(rows) tiles through shared memory.
template <int MODE>
__device__ __forceinline__ void split_transpose_body(const float *__restrict__ in0, int64_t rows, int64_t k, int64_t ld,
                                                     const PlanePtrs &pl, int64_t pitch, float (*tile)[33], int vblock,
                                                     int vgrid, int64_t batch = 1)
{
    // batch > 1: `batch` matrices [k, rows] k * ld apart; matrix b fills plane rows [b * rows, (b + 1) * rows)
    const int64_t tiles_r = (rows + 31) / 32, tiles_k = (k + 63) / 64, per = tiles_r * tiles_k;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
    for (int64_t tt = vblock; tt < per * batch; tt += vgrid) {
        const int64_t b = tt / per, t = tt - b * per;
        const float *in = in0 + b * k * ld;
        const int64_t tr = t % tiles_r, tk = t / tiles_r;
        const int64_t r0 = tr * 32, k0 = tk * 64;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int kk = ty + 8 * j;
            const int64_t gk = k0 + kk, gr = r0 + tx;
            tile[kk][tx] = (gk < k && gr < rows) ? __ldg(in + gk * ld + gr) : 0.0f;
        }
        __syncthreads();
        // each warp writes 4 rows; a lane covers k = 2*tx, 2*tx+1
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int rr = ty * 4 + j;
            const int64_t gr = r0 + rr;
            if (gr < rows) {
                const int kk = 2 * tx;
                const int64_t o = (b * rows + gr) * pitch + k0 + kk;
                if (k0 + kk + 1 < k) store2<MODE>(pl.p, o, tile[kk][rr], tile[kk + 1][rr]);
                else if (k0 + kk < k) store1<MODE>(pl.p, o, tile[kk][rr]);
            }
        }
        __syncthreads();
    }
}

template <int MODE>
__global__ void __launch_bounds__(256) split_rows_kernel(const float *__restrict__ in, int64_t rows, int64_t k, int64_t ld,
                                                         PlanePtrs pl, int64_t pitch, int64_t chunk_k, int64_t chunk_stride)
{
    grid_dep_launch();   // the GEMM that follows may set itself up now; its producers wait for this grid to finish
    split_rows_body<MODE>(in, rows, k, ld, pl, pitch, chunk_k, chunk_stride, blockIdx.x, gridDim.x);
}

template <int MODE>
__global__ void __launch_bounds__(256) split_transpose_kernel(const float *__restrict__ in, int64_t rows, int64_t k,
                                                              int64_t ld, PlanePtrs pl, int64_t pitch)
{
    __shared__ float tile[64][33];
    grid_dep_launch();
    split_transpose_body<MODE>(in, rows, k, ld, pl, pitch, tile, blockIdx.x, gridDim.x);
}

// Filter of an implicit convolution: weight [C_out][C_in][taps] (taps = kh * kw) -> planes [C_out][taps][c_pad],
// channel innermost and zero for c >= C_in, so that a k-block of the GEMM lies inside one window tap.
template <int MODE>
__device__ __forceinline__ void split_conv_weight_body(const float *__restrict__ w, int64_t C_out, int C_in, int taps, int c_pad,
                                                       const PlanePtrs &pl, int64_t pitch, int vblock, int vgrid)
{
    const int half = c_pad / 2;
    const int64_t total = C_out * taps * half;
    for (int64_t i = (int64_t)vblock * blockDim.x + threadIdx.x; i < total; i += (int64_t)vgrid * blockDim.x) {
        const int c = 2 * (int)(i % half);
        const int64_t rest = i / half;
        const int tap = (int)(rest % taps);
        const int64_t co = rest / taps;
        const float *src = w + (co * C_in + c) * taps + tap;
        const float v0 = c < C_in ? __ldg(src) : 0.0f, v1 = c + 1 < C_in ? __ldg(src + taps) : 0.0f;
        store2<MODE>(pl.p, co * pitch + (int64_t)tap * c_pad + c, v0, v1);
    }
}

// Both operands of one GEMM in ONE launch: blocks [0, ga) split operand A, the rest operand B; each operand is either
// row-major in k (rows body) or has k outermost (transpose body).  A 1024^3 GEMM is launch-bound: two pre-pass launches
// were a third of its step.
struct SplitTask {
    const float *in;
    int64_t rows, k, ld, pitch, chunk_k, chunk_stride;
    PlanePtrs pl;
    int transposed, blocks;
    int conv_taps, conv_cin, conv_cpad;   // conv_taps > 0: `in` is a filter [rows][conv_cin][conv_taps] (split_conv_weight_body)
    int64_t batch;                        // transposed tasks: matrices [k, rows] back to back (1 unless set)
};

template <int MODE>
__global__ void __launch_bounds__(256) split_pair_kernel(const SplitTask a, const SplitTask b)
{
    __shared__ float tile[64][33];
    grid_dep_launch();
    const bool first = (int)blockIdx.x < a.blocks;
    const SplitTask &t = first ? a : b;
    const int vblock = first ? (int)blockIdx.x : (int)blockIdx.x - a.blocks;
    if (t.conv_taps > 0) split_conv_weight_body<MODE>(t.in, t.rows, t.conv_cin, t.conv_taps, t.conv_cpad, t.pl, t.pitch, vblock, t.blocks);
    else if (t.transposed) split_transpose_body<MODE>(t.in, t.rows, t.k, t.ld, t.pl, t.pitch, tile, vblock, t.blocks, t.batch);
    else split_rows_body<MODE>(t.in, t.rows, t.k, t.ld, t.pl, t.pitch, t.chunk_k, t.chunk_stride, vblock, t.blocks);
}

// Implicit im2col: the B operand of a convolution-as-GEMM, written straight into K-major planes.  Row `pix` of
// the operand is output pixel (oh, ow); its element k = (c, ky, kx) is input[c][oh*sh + ky - ph][ow*sw + kx - pw]
// (zero outside the image) — the matrix k_im2col_sample materialises in the reference
// (src/compute/backends/cuda/ops_conv.cu:120-200) never exists here; the planes are the only intermediate.
template <int MODE>
__global__ void __launch_bounds__(256) split_im2col_kernel(const float *__restrict__ in, int64_t C_in, int64_t H, int64_t W,
                                                           int kh, int kw, int sh, int sw, int ph, int pw, int64_t out_h,
                                                           int64_t out_w, PlanePtrs pl, int64_t pitch, bool use_table)
{
    // One output pixel (= one row of the operand) per block pass, the threads run along k in pairs: the index
    // arithmetic per element is two 32-bit divisions and the stores are 8 bytes per plane.  (One element per thread
    // with the pixel recovered from a flat 64-bit index — the first version — spent its time in four 64-bit divisions
    // per element: 55 us for a 56x56x256 sample, 1 TB/s.)
    grid_dep_launch();
    const int K = (int)(C_in * kh * kw), khkw = kh * kw;
    const int64_t npix = out_h * out_w;
    // what depends on k alone — the offset of (c, ky, kx) inside the sample and the window position — is tabulated
    // once per block (when it fits) and reused for all of the block's pixels
    extern __shared__ int2 ktab[];   // { (c*H + ky)*W + kx, ky << 16 | kx }
    if (use_table) {
        for (int k = threadIdx.x; k < K; k += 256) {
            const int c = k / khkw, r = k - c * khkw, ky = r / kw, kx = r - ky * kw;
            ktab[k] = make_int2((int)((c * H + ky) * W + kx), (ky << 16) | kx);
        }
        __syncthreads();
    }
    for (int64_t pix = blockIdx.x; pix < npix; pix += gridDim.x) {
        const int oh = (int)(pix / out_w), ow = (int)(pix - (int64_t)oh * out_w);
        const int ih0 = oh * sh - ph, iw0 = ow * sw - pw;
        const int64_t row = pix * pitch;
        const float *base = in + (int64_t)ih0 * W + iw0;   // only dereferenced at offsets that land inside the sample
        for (int k = 2 * (int)threadIdx.x; k < K; k += 512) {
            float v[2] = { 0.0f, 0.0f };
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int kk = k + e;
                if (kk < K) {
                    int64_t off;
                    int ky, kx;
                    if (use_table) {
                        const int2 t = ktab[kk];
                        off = t.x; ky = t.y >> 16; kx = t.y & 0xFFFF;
                    } else {
                        const int c = kk / khkw, r = kk - c * khkw;
                        ky = r / kw; kx = r - ky * kw;
                        off = (c * H + ky) * W + kx;
                    }
                    const int ih = ih0 + ky, iw = iw0 + kx;
                    if (ih >= 0 && ih < H && iw >= 0 && iw < W) v[e] = __ldg(base + off);
                }
            }
            if (k + 1 < K && ((row + k) & 1) == 0) store2<MODE>(pl.p, row + k, v[0], v[1]);
            else {
                store1<MODE>(pl.p, row + k, v[0]);
                if (k + 1 < K) store1<MODE>(pl.p, row + k + 1, v[1]);
            }
        }
    }
}

// int8 [rows, k] -> bf16 plane [rows, pitch] (every int8 is exact in bf16)
__global__ void __launch_bounds__(256) widen_i8_bf16_kernel(const int8_t *__restrict__ in, int64_t rows,
                                                            int64_t k, __nv_bfloat16 *out, int64_t pitch)
{
    const int64_t total = rows * k;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / k, c = i - r * k;
        out[r * pitch + c] = __float2bfloat16_rn((float)in[i]);
    }
}

__global__ void __launch_bounds__(256) repitch_i8_kernel(const int8_t *__restrict__ in, int64_t rows,
                                                         int64_t k, int8_t *out, int64_t pitch)
{
    const int64_t total = rows * k;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / k, c = i - r * k;
        out[r * pitch + c] = in[i];
    }
}

// mult[n] = (a_scale * b_scales[n]) / out_scale with one rounding per operation
__global__ void requant_mult_kernel(float a_scale, const float *__restrict__ b_scales, float out_scale,
                                    int64_t n, float *mult)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) mult[i] = __fdiv_rn(__fmul_rn(a_scale, b_scales[i]), out_scale);
}

// one CTA per row: absmax, scale = absmax/127 (1 for a zero row), q = clamp(rint(w * (1/scale)))
__global__ void __launch_bounds__(256) quantize_rows_kernel(const float *__restrict__ w, int64_t k,
                                                            int8_t *q, float *scales)
{
    __shared__ float red[8];
    __shared__ float s_inv;
    const int64_t n = blockIdx.x;
    const float *row = w + n * k;
    float m = 0.0f;
    for (int64_t i = threadIdx.x; i < k; i += blockDim.x) m = fmaxf(m, fabsf(row[i]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        float a = red[0];
        for (int i = 1; i < (int)(blockDim.x >> 5); ++i) a = fmaxf(a, red[i]);
        const float scale = a > 0.0f ? __fdiv_rn(a, 127.0f) : 1.0f;
        scales[n] = scale;
        s_inv = __fdiv_rn(1.0f, scale);
    }
    __syncthreads();
    const float inv = s_inv;
    for (int64_t i = threadIdx.x; i < k; i += blockDim.x) {
        int v = __float2int_rn(__fmul_rn(row[i], inv));
        v = max(-127, min(127, v));
        q[n * k + i] = (int8_t)v;
    }
}

// ---------------------------------------------------------------------- host

static inline int grid_for(int64_t work_items, int threads, int sm_count)
{
    int64_t blocks = (work_items + threads - 1) / threads;
    const int64_t cap = (int64_t)sm_count * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

int split_planes(int mode, const float *in, int64_t rows, int64_t k, int64_t ld, bool in_is_k_major_outer,
                 void *const planes[3], int64_t pitch, int sm_count, cudaStream_t st, int64_t chunk_k,
                 int64_t chunk_stride)
{
    PlanePtrs pl;
    for (int i = 0; i < 3; ++i) pl.p[i] = planes[i];
    if (!in_is_k_major_outer) {
        const int g = grid_for(rows * ((k + 3) / 4), 256, sm_count);
        switch (mode) {
        case SPLIT_TF32X2: split_rows_kernel<SPLIT_TF32X2><<<g, 256, 0, st>>>(in, rows, k, ld, pl, pitch, chunk_k, chunk_stride); break;
        case SPLIT_BF16X1: split_rows_kernel<SPLIT_BF16X1><<<g, 256, 0, st>>>(in, rows, k, ld, pl, pitch, chunk_k, chunk_stride); break;
        case SPLIT_BF16X2: split_rows_kernel<SPLIT_BF16X2><<<g, 256, 0, st>>>(in, rows, k, ld, pl, pitch, chunk_k, chunk_stride); break;
        default: split_rows_kernel<SPLIT_BF16X3><<<g, 256, 0, st>>>(in, rows, k, ld, pl, pitch, chunk_k, chunk_stride); break;
        }
    } else {
        const int64_t tiles = ((rows + 31) / 32) * ((k + 63) / 64);
        const int64_t cap = (int64_t)sm_count * 8;
        const int g = (int)(tiles < cap ? (tiles > 0 ? tiles : 1) : cap);
        switch (mode) {
        case SPLIT_TF32X2: split_transpose_kernel<SPLIT_TF32X2><<<g, 256, 0, st>>>(in, rows, k, ld, pl, pitch); break;
        case SPLIT_BF16X1: split_transpose_kernel<SPLIT_BF16X1><<<g, 256, 0, st>>>(in, rows, k, ld, pl, pitch); break;
        case SPLIT_BF16X2: split_transpose_kernel<SPLIT_BF16X2><<<g, 256, 0, st>>>(in, rows, k, ld, pl, pitch); break;
        default: split_transpose_kernel<SPLIT_BF16X3><<<g, 256, 0, st>>>(in, rows, k, ld, pl, pitch); break;
        }
    }
    return (int)cudaGetLastError();
}

static SplitTask make_task(const float *in, int64_t rows, int64_t k, int64_t ld, bool transposed, void *const planes[3],
                           int64_t pitch, int64_t chunk_k, int64_t chunk_stride, int sm_count)
{
    SplitTask t;
    t.in = in; t.rows = rows; t.k = k; t.ld = ld; t.pitch = pitch; t.chunk_k = chunk_k; t.chunk_stride = chunk_stride;
    for (int i = 0; i < 3; ++i) t.pl.p[i] = planes[i];
    t.transposed = transposed ? 1 : 0;
    t.conv_taps = t.conv_cin = t.conv_cpad = 0;
    t.batch = 1;
    if (!transposed) {
        t.blocks = grid_for(rows * ((k + 3) / 4), 256, sm_count);
    } else {
        const int64_t tiles = ((rows + 31) / 32) * ((k + 63) / 64), cap = (int64_t)sm_count * 8;
        t.blocks = (int)(tiles < cap ? (tiles > 0 ? tiles : 1) : cap);
    }
    return t;
}

int split_planes_pair(int mode, const float *a_in, int64_t a_rows, int64_t a_ld, bool a_transposed, void *const a_planes[3],
                      int64_t a_pitch, int64_t a_chunk_k, int64_t a_chunk_stride, const float *b_in, int64_t b_rows,
                      int64_t b_ld, bool b_transposed, void *const b_planes[3], int64_t b_pitch, int64_t k, int sm_count,
                      cudaStream_t st)
{
    const SplitTask ta = make_task(a_in, a_rows, k, a_ld, a_transposed, a_planes, a_pitch, a_chunk_k, a_chunk_stride, sm_count);
    const SplitTask tb = make_task(b_in, b_rows, k, b_ld, b_transposed, b_planes, b_pitch, 0, 0, sm_count);
    const unsigned g = (unsigned)(ta.blocks + tb.blocks);
    switch (mode) {
    case SPLIT_TF32X2: split_pair_kernel<SPLIT_TF32X2><<<g, 256, 0, st>>>(ta, tb); break;
    case SPLIT_BF16X1: split_pair_kernel<SPLIT_BF16X1><<<g, 256, 0, st>>>(ta, tb); break;
    case SPLIT_BF16X2: split_pair_kernel<SPLIT_BF16X2><<<g, 256, 0, st>>>(ta, tb); break;
    default: split_pair_kernel<SPLIT_BF16X3><<<g, 256, 0, st>>>(ta, tb); break;
    }
    return (int)cudaGetLastError();
}

int split_im2col(int mode, const float *in, int64_t C_in, int64_t H, int64_t W, int kh, int kw, int sh, int sw, int ph,
                 int pw, int64_t out_h, int64_t out_w, void *const planes[3], int64_t pitch, int sm_count, cudaStream_t st)
{
    PlanePtrs pl;
    for (int i = 0; i < 3; ++i) pl.p[i] = planes[i];
    const int64_t npix = out_h * out_w, K = C_in * kh * kw;
    // the sample's element count must fit the table's 32-bit offsets; the table itself 48 KB of shared memory
    const bool table = K * 8 <= 48 * 1024 && C_in * H * W < INT32_MAX && kh < 32768 && kw < 32768;
    const int64_t cap = (int64_t)sm_count * (table ? 4 : 16);
    const int g = (int)(npix < cap ? npix : cap);
    const size_t sm = table ? (size_t)K * 8 : 0;
    switch (mode) {
    case SPLIT_TF32X2: split_im2col_kernel<SPLIT_TF32X2><<<g, 256, sm, st>>>(in, C_in, H, W, kh, kw, sh, sw, ph, pw, out_h, out_w, pl, pitch, table); break;
    case SPLIT_BF16X1: split_im2col_kernel<SPLIT_BF16X1><<<g, 256, sm, st>>>(in, C_in, H, W, kh, kw, sh, sw, ph, pw, out_h, out_w, pl, pitch, table); break;
    case SPLIT_BF16X2: split_im2col_kernel<SPLIT_BF16X2><<<g, 256, sm, st>>>(in, C_in, H, W, kh, kw, sh, sw, ph, pw, out_h, out_w, pl, pitch, table); break;
    default: split_im2col_kernel<SPLIT_BF16X3><<<g, 256, sm, st>>>(in, C_in, H, W, kh, kw, sh, sw, ph, pw, out_h, out_w, pl, pitch, table); break;
    }
    return (int)cudaGetLastError();
}

int split_conv_operands(int mode, const float *image, int64_t batch, int64_t C_in, int64_t HW, void *const image_planes[3],
                        int64_t image_pitch, const float *w, int64_t C_out, int taps, int c_pad, void *const w_planes[3],
                        int64_t w_pitch, int sm_count, cudaStream_t st)
{
    // a sample [C_in][HW] is a k-outermost operand: the transposing body writes it channel-innermost
    SplitTask ta = make_task(image, HW, C_in, HW, true, image_planes, image_pitch, 0, 0, sm_count);
    ta.batch = batch;
    {
        const int64_t tiles = ((HW + 31) / 32) * ((C_in + 63) / 64) * batch, cap = (int64_t)sm_count * 8;
        ta.blocks = (int)(tiles < cap ? (tiles > 0 ? tiles : 1) : cap);
    }
    SplitTask tb = make_task(w, C_out, (int64_t)taps * c_pad, 0, false, w_planes, w_pitch, 0, 0, sm_count);
    tb.conv_taps = taps; tb.conv_cin = (int)C_in; tb.conv_cpad = c_pad;
    tb.blocks = grid_for(C_out * taps * (c_pad / 2), 256, sm_count);
    const int g = ta.blocks + tb.blocks;
    switch (mode) {
    case SPLIT_TF32X2: split_pair_kernel<SPLIT_TF32X2><<<g, 256, 0, st>>>(ta, tb); break;
    case SPLIT_BF16X1: split_pair_kernel<SPLIT_BF16X1><<<g, 256, 0, st>>>(ta, tb); break;
    case SPLIT_BF16X2: split_pair_kernel<SPLIT_BF16X2><<<g, 256, 0, st>>>(ta, tb); break;
    default: split_pair_kernel<SPLIT_BF16X3><<<g, 256, 0, st>>>(ta, tb); break;
    }
    return (int)cudaGetLastError();
}

int widen_i8_to_bf16(const int8_t *in, int64_t rows, int64_t k, void *out, int64_t pitch, int sm_count,
                     cudaStream_t st)
{
    widen_i8_bf16_kernel<<<grid_for(rows * k, 256, sm_count), 256, 0, st>>>(
        in, rows, k, reinterpret_cast<__nv_bfloat16 *>(out), pitch);
    return (int)cudaGetLastError();
}

int repitch_i8(const int8_t *in, int64_t rows, int64_t k, int8_t *out, int64_t pitch, int sm_count,
               cudaStream_t st)
{
    repitch_i8_kernel<<<grid_for(rows * k, 256, sm_count), 256, 0, st>>>(in, rows, k, out, pitch);
    return (int)cudaGetLastError();
}

int requant_mult(float a_scale, const float *b_scales, float out_scale, int64_t n, float *mult,
                 cudaStream_t st)
{
    requant_mult_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(a_scale, b_scales, out_scale, n, mult);
    return (int)cudaGetLastError();
}

int quantize_rows(const float *w, int64_t n, int64_t k, int8_t *q, float *scales, cudaStream_t st)
{
    quantize_rows_kernel<<<(unsigned)n, 256, 0, st>>>(w, k, q, scales);
    return (int)cudaGetLastError();
}

}  // namespace axb
