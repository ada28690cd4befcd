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
// into the mantissa of 2^23 and subtract 2^23 + 128.  Exact for every int8 value.
__device__ __forceinline__ void unpack16(const uint4 &w, float (&f)[16])
{
    const uint32_t v[4] = { w.x ^ 0x80808080u, w.y ^ 0x80808080u, w.z ^ 0x80808080u, w.w ^ 0x80808080u };
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[4 * i + 0] = __uint_as_float(__byte_perm(v[i], 0x4B000000u, 0x7540)) - 8388736.0f;
        f[4 * i + 1] = __uint_as_float(__byte_perm(v[i], 0x4B000000u, 0x7541)) - 8388736.0f;
        f[4 * i + 2] = __uint_as_float(__byte_perm(v[i], 0x4B000000u, 0x7542)) - 8388736.0f;
        f[4 * i + 3] = __uint_as_float(__byte_perm(v[i], 0x4B000000u, 0x7543)) - 8388736.0f;
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
    uint4 w[QV_UNROLL];
    if (n < N) {
        const uint4 *row = reinterpret_cast<const uint4 *>(q + n * (int64_t)K);
#pragma unroll
        for (int u = 0; u < QV_UNROLL; ++u) {
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

    for (; n < N; n += row_stride) {
        const uint4 *row = reinterpret_cast<const uint4 *>(q + n * (int64_t)K);
        float acc[MT];
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[m] = 0.0f;
#pragma unroll 1
        for (int p0 = lane; p0 < pieces; p0 += 32 * QV_UNROLL) {
            if (p0 != lane) {
#pragma unroll
                for (int u = 0; u < QV_UNROLL; ++u) {
                    const int p = p0 + 32 * u;
                    w[u] = p < pieces ? __ldcs(row + p) : make_uint4(0, 0, 0, 0);
                }
            }
#pragma unroll
            for (int u = 0; u < QV_UNROLL; ++u) {
                const int p = p0 + 32 * u;
                if (p < pieces) {
                    float f[16];
                    unpack16(w[u], f);
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        const float4 *xv = reinterpret_cast<const float4 *>(xs + m * K + p * 16);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float4 x4 = xv[(j + (p >> 1)) & 3];
                            acc[m] = fmaf(x4.x, f[4 * j + 0], acc[m]);
                            acc[m] = fmaf(x4.y, f[4 * j + 1], acc[m]);
                            acc[m] = fmaf(x4.z, f[4 * j + 2], acc[m]);
                            acc[m] = fmaf(x4.w, f[4 * j + 3], acc[m]);
                        }
                    }
                }
            }
        }
        // the next row's first loads go out before this row's reduction
        const int64_t nn = n + row_stride;
        if (nn < N) {
            const uint4 *nrow = reinterpret_cast<const uint4 *>(q + nn * (int64_t)K);
#pragma unroll
            for (int u = 0; u < QV_UNROLL; ++u) {
                const int p = lane + 32 * u;
                w[u] = p < pieces ? __ldcs(nrow + p) : make_uint4(0, 0, 0, 0);
            }
        }
        const float sc = __ldg(scales + n);
        const float bn = bias ? __ldg(bias + n) : 0.0f;
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            float v = acc[m];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
            if (lane == 0 && m < M) {
                v = v * sc;                       // the reference's result (quantize.c:100-177) ...
                if (bias) v += bn;                // ... and the dense layer's bias and activation on top
                if (act == 1) v = fmaxf(v, 0.0f);
                else if (act == 2) v = 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
                out[(int64_t)m * N + n] = v;
            }
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
    const int64_t cap = (int64_t)sm_count * (smem > 48 * 1024 ? 2 : 4);
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
