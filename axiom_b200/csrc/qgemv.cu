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

__device__ __forceinline__ void unpack16(const uint4 &w, float (&f)[16])
{
    const uint32_t v[4] = { w.x, w.y, w.z, w.w };
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[4 * i + 0] = (float)(int8_t)(v[i] & 0xff);
        f[4 * i + 1] = (float)(int8_t)((v[i] >> 8) & 0xff);
        f[4 * i + 2] = (float)(int8_t)((v[i] >> 16) & 0xff);
        f[4 * i + 3] = (float)(int8_t)(v[i] >> 24);
    }
}

// K % 16 == 0, q 16-byte aligned.  Shared memory: a as [MT][K] floats.
template <int MT>
__global__ void __launch_bounds__(QV_THREADS) qgemv_w8a32_kernel(const float *__restrict__ a,
                                                                 const int8_t *__restrict__ q,
                                                                 const float *__restrict__ scales,
                                                                 float *__restrict__ out, int M, int64_t N, int64_t K)
{
    extern __shared__ __align__(16) float xs[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // activations as [MT][K]; inside every 16-element piece p the four float4 are rotated by p/2 so that the
    // lanes of a quarter-warp (consecutive pieces, 64 bytes apart) hit eight different bank groups
    for (int64_t i = tid; i < (int64_t)MT * K; i += QV_THREADS) {
        const int m = (int)(i / K);
        const int64_t k = i - (int64_t)m * K, pc = k >> 4;
        const int j = (int)((k >> 2) & 3), e = (int)(k & 3);
        xs[(int64_t)m * K + pc * 16 + (((j + (int)(pc >> 1)) & 3) << 2) + e] = m < M ? __ldg(a + i) : 0.0f;
    }
    __syncthreads();

    const int64_t pieces = K / 16;                         // 16-element pieces per row
    const int64_t row_stride = (int64_t)gridDim.x * QV_WARPS;
    for (int64_t n = (int64_t)blockIdx.x * QV_WARPS + warp; n < N; n += row_stride) {
        const uint4 *row = reinterpret_cast<const uint4 *>(q + n * K);
        float acc[MT];
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[m] = 0.0f;
        for (int64_t p0 = lane; p0 < pieces; p0 += 32 * 4) {
            uint4 w[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int64_t p = p0 + 32 * u;
                w[u] = p < pieces ? __ldcs(row + p) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int64_t p = p0 + 32 * u;
                if (p < pieces) {
                    float f[16];
                    unpack16(w[u], f);
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        const float4 *xv = reinterpret_cast<const float4 *>(xs + (int64_t)m * K + p * 16);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float4 x4 = xv[(j + (int)(p >> 1)) & 3];
                            acc[m] = fmaf(x4.x, f[4 * j + 0], acc[m]);
                            acc[m] = fmaf(x4.y, f[4 * j + 1], acc[m]);
                            acc[m] = fmaf(x4.z, f[4 * j + 2], acc[m]);
                            acc[m] = fmaf(x4.w, f[4 * j + 3], acc[m]);
                        }
                    }
                }
            }
        }
        const float sc = __ldg(scales + n);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            float v = acc[m];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
            if (lane == 0 && m < M) out[(int64_t)m * N + n] = v * sc;
        }
    }
}

bool qgemv_w8a32_applicable(int64_t M, int64_t N, int64_t K, const void *q)
{
    (void)N;
    const int64_t mt = M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : 8;
    return M >= 1 && M <= 8 && K % 16 == 0 && K * mt * 4 <= 160 * 1024 &&
           (reinterpret_cast<uintptr_t>(q) & 15) == 0;
}

template <int MT>
static int launch_qv(const float *a, const int8_t *q, const float *scales, float *out, int M, int64_t N, int64_t K,
                     int sm_count, cudaStream_t st)
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
    k<<<(unsigned)blocks, QV_THREADS, smem, st>>>(a, q, scales, out, M, N, K);
    return (int)cudaGetLastError();
}

int launch_qgemv_w8a32(const float *a, const int8_t *q, const float *scales, float *out, int64_t M, int64_t N,
                       int64_t K, int sm_count, cudaStream_t st)
{
    if (M <= 1) return launch_qv<1>(a, q, scales, out, (int)M, N, K, sm_count, st);
    if (M <= 2) return launch_qv<2>(a, q, scales, out, (int)M, N, K, sm_count, st);
    if (M <= 4) return launch_qv<4>(a, q, scales, out, (int)M, N, K, sm_count, st);
    return launch_qv<8>(a, q, scales, out, (int)M, N, K, sm_count, st);
}

}  // namespace axb
