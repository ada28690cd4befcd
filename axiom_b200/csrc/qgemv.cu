// qgemv.cu — W8A32 for skinny activations (M <= 8): out[m,n] = scale[n] * sum_k a[m,k] * q[n,k].
//
// The reference's quantised path exists for exactly this case (int8 weights quarter the bytes of a
// bandwidth-bound dense layer, src/core/quantize.c:100-177): the weight matrix [N,K] is streamed once, 16 int8
// per 128-bit load, converted to fp32 in registers and multiplied into fp32 accumulators — the same arithmetic
// as the reference's inner loop, summed in a different (fixed) order.  A warp owns whole weight rows: its lanes
// split K in 16-element pieces, the activations sit in shared memory, and a shuffle tree adds the lanes.
#include "qgemv.cuh"

#include <stdint.h>

namespace axb {

static constexpr int QV_THREADS = 256;
static constexpr int QV_WARPS = 8;

// int8 -> fp32 without the conversion pipe: flip the sign bits (s + 128 as an unsigned byte), drop the byte
// into the mantissa of 2^23 and subtract 2^23 + 128.  Exact for every int8 value.  The values come out as
// pairs so that the subtraction and the multiply-add run as packed f32x2 instructions: the kernel is paced by
// instruction issue (ncu: 60 % issue-active at 33 % of DRAM throughput), not by memory.
__device__ __forceinline__ void unpack16(const uint4 &w, float2 (&f)[8])
{
    const uint32_t v[4] = { w.x ^ 0x80808080u, w.y ^ 0x80808080u, w.z ^ 0x80808080u, w.w ^ 0x80808080u };
    const float2 bias = make_float2(-8388736.0f, -8388736.0f);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i + 0] = __fadd2_rn(make_float2(__uint_as_float(__byte_perm(v[i], 0x4B000000u, 0x7540)),
                                              __uint_as_float(__byte_perm(v[i], 0x4B000000u, 0x7541))), bias);
        f[2 * i + 1] = __fadd2_rn(make_float2(__uint_as_float(__byte_perm(v[i], 0x4B000000u, 0x7542)),
                                              __uint_as_float(__byte_perm(v[i], 0x4B000000u, 0x7543))), bias);
    }
}

static constexpr int QV_UNROLL = 8;   // 128-bit weight loads a lane keeps in flight

// K % 16 == 0, q 16-byte aligned, a 16-byte aligned.  Shared memory: a as [MT][K] floats.
template <int MT>
__global__ void __launch_bounds__(QV_THREADS) qgemv_w8a32_kernel(const float *__restrict__ a,
                                                                 const int8_t *__restrict__ q,
                                                                 const float *__restrict__ scales,
                                                                 const float *__restrict__ bias, int act,
                                                                 float *__restrict__ out, int M, int64_t N, int K)
{
    extern __shared__ __align__(16) float xs[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int pieces = K >> 4;                             // 16-element pieces per row
    const int64_t row_stride = (int64_t)gridDim.x * QV_WARPS;
    int64_t n = (int64_t)blockIdx.x * QV_WARPS + warp;

    // the first weight loads leave before the activations are staged
    constexpr int U = MT >= 8 ? 4 : QV_UNROLL;   // 16-byte loads per lane and buffer
    uint4 w[U], wb2[U];
    if (n < N) {
        const uint4 *row = reinterpret_cast<const uint4 *>(q + n * (int64_t)K);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int p = lane + 32 * u;
            w[u] = p < pieces ? __ldcs(row + p) : make_uint4(0, 0, 0, 0);
        }
    }

    // activations as [MT][K]; inside every 16-element piece p the four float4 are rotated by p/2 so that the
    // lanes of a quarter-warp (consecutive pieces, 64 bytes apart) hit eight different bank groups
    {
        const int k4n = K >> 2, total = MT * k4n;
        float4 *xs4 = reinterpret_cast<float4 *>(xs);
        for (int i0 = tid; i0 < total; i0 += QV_THREADS * 4) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * QV_THREADS;
                const int m = i / k4n;
                v[u] = (i < total && m < M) ? __ldg(reinterpret_cast<const float4 *>(a) + i)
                                            : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * QV_THREADS;
                if (i < total) {
                    const int m = i / k4n, k4 = i - m * k4n, pc = k4 >> 2, j = k4 & 3;
                    xs4[m * k4n + pc * 4 + ((j + (pc >> 1)) & 3)] = v[u];
                }
            }
        }
    }
    __syncthreads();

    // The rows of this warp as one stream of chunks (a chunk = QV_UNROLL 16-byte pieces per lane of one row).  The
    // loads of chunk c+1 are issued before chunk c is computed (two register buffers), so a warp always has weight
    // bytes in flight; with a single buffer the loads waited for the arithmetic and the kernel sat at half the
    // memory rate.
    const int cpr = (pieces + 32 * U - 1) / (32 * U);                 // chunks per row
    const int64_t my_rows = n < N ? (N - n + row_stride - 1) / row_stride : 0;
    const int64_t total = my_rows * cpr;
    float2 acc[MT];   // two partial sums per row (even and odd k), added at the end
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = make_float2(0.0f, 0.0f);

    auto load = [&](uint4 (&wb)[U], int64_t c) {
        const int64_t r = c / cpr;
        const int g = (int)(c - r * cpr);
        const uint4 *row = reinterpret_cast<const uint4 *>(q + (n + r * row_stride) * (int64_t)K);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int p = lane + 32 * (g * U + u);
            wb[u] = p < pieces ? __ldcs(row + p) : make_uint4(0, 0, 0, 0);
        }
    };
    auto compute = [&](const uint4 (&wb)[U], int64_t c) {
        const int64_t r = c / cpr;
        const int g = (int)(c - r * cpr);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int p = lane + 32 * (g * U + u);
            if (p < pieces) {
                float2 f[8];
                unpack16(wb[u], f);
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    const float4 *xv = reinterpret_cast<const float4 *>(xs + m * K + p * 16);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float4 x4 = xv[(j + (p >> 1)) & 3];
                        acc[m] = __ffma2_rn(make_float2(x4.x, x4.y), f[2 * j + 0], acc[m]);
                        acc[m] = __ffma2_rn(make_float2(x4.z, x4.w), f[2 * j + 1], acc[m]);
                    }
                }
            }
        }
        if (g == cpr - 1) {   // the row is complete
            const int64_t nr = n + r * row_stride;
            const float sc = __ldg(scales + nr);
            const float bn = bias ? __ldg(bias + nr) : 0.0f;
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                float v = acc[m].x + acc[m].y;
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
                if (lane == 0 && m < M) {
                    v = v * sc;                       // the reference's result (quantize.c:100-177) ...
                    if (bias) v += bn;                // ... and the dense layer's bias and activation on top
                    if (act == 1) v = fmaxf(v, 0.0f);
                    else if (act == 2) v = 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
                    out[(int64_t)m * N + nr] = v;
                }
                acc[m] = make_float2(0.0f, 0.0f);
            }
        }
    };

    for (int64_t c = 0; c < total; c += 2) {
        if (c + 1 < total) load(wb2, c + 1);
        compute(w, c);
        if (c + 1 < total) {
            if (c + 2 < total) load(w, c + 2);
            compute(wb2, c + 1);
        }
    }
}

bool qgemv_w8a32_applicable(int64_t M, int64_t N, int64_t K, const void *q)
{
    (void)N;
    const int64_t mt = M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : 8;
    return M >= 1 && M <= 8 && K % 16 == 0 && K * mt * 4 <= 160 * 1024 &&
           (reinterpret_cast<uintptr_t>(q) & 15) == 0;   // the caller checks the activations' alignment
}

template <int MT>
static int launch_qv(const float *a, const int8_t *q, const float *scales, const float *bias, int act, float *out, int M,
                     int64_t N, int64_t K, int sm_count, cudaStream_t st)
{
    auto k = qgemv_w8a32_kernel<MT>;
    const size_t smem = (size_t)MT * K * sizeof(float);
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        attr_set[dev] = true;
    }
    int64_t blocks = (N + QV_WARPS - 1) / QV_WARPS;
    const int64_t cap = (int64_t)sm_count * 2;   // two resident CTAs per SM (registers): one wave, rows strided over it
    if (blocks > cap) blocks = cap;
    k<<<(unsigned)blocks, QV_THREADS, smem, st>>>(a, q, scales, bias, act, out, M, N, (int)K);
    return (int)cudaGetLastError();
}

int launch_qgemv_w8a32(const float *a, const int8_t *q, const float *scales, const float *bias, int act, float *out,
                       int64_t M, int64_t N, int64_t K, int sm_count, cudaStream_t st)
{
    if (M <= 1) return launch_qv<1>(a, q, scales, bias, act, out, (int)M, N, K, sm_count, st);
    if (M <= 2) return launch_qv<2>(a, q, scales, bias, act, out, (int)M, N, K, sm_count, st);
    if (M <= 4) return launch_qv<4>(a, q, scales, bias, act, out, (int)M, N, K, sm_count, st);
    return launch_qv<8>(a, q, scales, bias, act, out, (int)M, N, K, sm_count, st);
}

}  // namespace axb
