// skinny.cu — the bandwidth-bound skinny-M route (M <= 32, bs=1 GEMV included):
//     Y[M,N] = act(alpha * X[M,K] . W[K,N] + beta * Y + bias[n])
// W is streamed from HBM exactly once with 128-bit loads; everything else is
// small.  A CTA owns a 128-column strip and a slice of K: its 8 warps walk
// interleaved rows of the slice (one float4 of W per lane per row, all M
// outputs of those 4 columns accumulated in registers, X broadcast from shared
// memory), then the warps' sums are combined through shared memory in a fixed
// order.  When K is split across CTAs each CTA writes its partial strip to
// scratch and the LAST CTA to arrive for a strip (a counter per strip) adds
// the partials in slice order and applies the epilogue, so results do not
// depend on scheduling: repeated calls are bitwise identical.
#include "skinny.cuh"

#include "../../include/axiom_b200.h"
#include "errors.cuh"

#include <stdint.h>
#include <stdlib.h>

namespace axb {

static constexpr int SK_THREADS = 256;
static constexpr int SK_WARPS = 8;
static constexpr int SK_STRIP = 128;  // columns per CTA

__device__ __forceinline__ float sk_gelu(float v)
{
    const float inner = 0.7978845608028654f * (v + 0.044715f * v * v * v);
    return 0.5f * v * (1.0f + tanhf(inner));
}

__device__ __forceinline__ float sk_epilogue(const SkinnyArgs &a, float v, int m, int col)
{
    v *= a.alpha;
    if (a.beta != 0.0f) v += a.beta * a.Y[(int64_t)m * a.N + col];
    if (a.bias) v += __ldg(a.bias + col);
    if (a.act == 1) v = fmaxf(v, 0.0f);
    else if (a.act == 2) v = sk_gelu(v);
    return v;
}

template <int MT, bool VEC>
__global__ void __launch_bounds__(SK_THREADS) skinny_kernel(const SkinnyArgs a)
{
    constexpr int RM = MT < 8 ? MT : 8;          // rows combined per reduction round
    constexpr int UNROLL = MT >= 32 ? 2 : (MT >= 16 ? 4 : 8);
    extern __shared__ float smem[];
    __shared__ int s_last;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int strip = blockIdx.x, ks = blockIdx.y;
    const int64_t k_begin = (int64_t)ks * a.kchunk;
    const int kc = (int)min((int64_t)a.kchunk, a.K - k_begin);  // rows of this slice (may be <= 0)
    const int col = strip * SK_STRIP + lane * 4;

    // X slice -> shared, transposed to [k][MT] so one k reads MT contiguous floats
    float *xs = smem;
    for (int i = tid; i < kc * MT; i += SK_THREADS) {
        const int m = i / kc, kk = i - m * kc;
        xs[kk * MT + m] = (m < a.M) ? __ldg(a.X + (int64_t)m * a.K + k_begin + kk) : 0.0f;
    }
    __syncthreads();

    float acc[MT][4];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.0f;

    if (col < a.N) {
        const float *wp = a.W + k_begin * a.N + col;
        for (int kk0 = warp; kk0 < kc; kk0 += SK_WARPS * UNROLL) {
            float4 w[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int kk = kk0 + u * SK_WARPS;
                if (kk < kc) {
                    const float *src = wp + (int64_t)kk * a.N;
                    if constexpr (VEC) {
                        w[u] = __ldcs(reinterpret_cast<const float4 *>(src));
                    } else {
                        w[u].x = __ldcs(src);
                        w[u].y = (col + 1 < a.N) ? __ldcs(src + 1) : 0.0f;
                        w[u].z = (col + 2 < a.N) ? __ldcs(src + 2) : 0.0f;
                        w[u].w = (col + 3 < a.N) ? __ldcs(src + 3) : 0.0f;
                    }
                } else {
                    w[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int kk = kk0 + u * SK_WARPS;
                if (kk < kc) {
                    const float *xr = xs + kk * MT;
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        const float xv = xr[m];
                        acc[m][0] = fmaf(xv, w[u].x, acc[m][0]);
                        acc[m][1] = fmaf(xv, w[u].y, acc[m][1]);
                        acc[m][2] = fmaf(xv, w[u].z, acc[m][2]);
                        acc[m][3] = fmaf(xv, w[u].w, acc[m][3]);
                    }
                }
            }
        }
    }
    __syncthreads();  // xs is dead from here: the same shared memory holds the warp sums

    float *red = smem;  // [SK_WARPS][RM][SK_STRIP]
    float *part = a.partial ? a.partial + (int64_t)ks * a.M * a.N : nullptr;
#pragma unroll  // m0 must be a compile-time constant: acc[] is indexed with it and has to stay in registers
    for (int m0 = 0; m0 < MT; m0 += RM) {
#pragma unroll
        for (int mi = 0; mi < RM; ++mi)
            *reinterpret_cast<float4 *>(red + ((warp * RM + mi) * SK_STRIP + lane * 4)) =
                make_float4(acc[m0 + mi][0], acc[m0 + mi][1], acc[m0 + mi][2], acc[m0 + mi][3]);
        __syncthreads();
        for (int o = tid; o < RM * SK_STRIP; o += SK_THREADS) {
            const int mi = o / SK_STRIP, c = o - mi * SK_STRIP;
            const int m = m0 + mi, gc = strip * SK_STRIP + c;
            if (m < a.M && gc < a.N) {
                float s = 0.0f;
#pragma unroll
                for (int w = 0; w < SK_WARPS; ++w) s += red[(w * RM + mi) * SK_STRIP + c];
                if (a.ksplit == 1) a.Y[(int64_t)m * a.N + gc] = sk_epilogue(a, s, m, gc);
                else part[(int64_t)m * a.N + gc] = s;
            }
        }
        __syncthreads();
    }

    if (a.ksplit > 1) {
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            const int prev = atomicAdd(a.counters + strip, 1);
            s_last = (prev == a.ksplit - 1);
        }
        __syncthreads();
        if (s_last) {
            __threadfence();
            const int ncols = min(SK_STRIP, (int)(a.N - (int64_t)strip * SK_STRIP));
            for (int o = tid; o < a.M * ncols; o += SK_THREADS) {
                const int m = o / ncols, gc = strip * SK_STRIP + (o - m * ncols);
                float s = 0.0f;
                for (int q = 0; q < a.ksplit; ++q)
                    s += __ldcg(a.partial + ((int64_t)q * a.M + m) * a.N + gc);
                a.Y[(int64_t)m * a.N + gc] = sk_epilogue(a, s, m, gc);
            }
            if (tid == 0) a.counters[strip] = 0;  // ready for the next call
        }
    }
}

template <int MT>
static int launch_mt(const SkinnyArgs &a, bool vec, dim3 grid, size_t smem, cudaStream_t st)
{
    auto kv = skinny_kernel<MT, true>;
    auto ks = skinny_kernel<MT, false>;
    // once per device and instantiation: allow the 64 KB X slice skinny_plan may ask for
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        cudaFuncSetAttribute(kv, cudaFuncAttributeMaxDynamicSharedMemorySize, 72 * 1024);
        cudaFuncSetAttribute(ks, cudaFuncAttributeMaxDynamicSharedMemorySize, 72 * 1024);
        attr_set[dev] = true;
    }
    if (vec) kv<<<grid, SK_THREADS, smem, st>>>(a);
    else ks<<<grid, SK_THREADS, smem, st>>>(a);
    return (int)cudaGetLastError();
}

static int mt_for(int64_t M) { return M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : M <= 8 ? 8 : M <= 16 ? 16 : 32; }

// The TMA-staged kernel needs what a tensor map needs: a 16-byte aligned base and row pitch.
static void skinny_plan_tma(int64_t M, int64_t N, int64_t K, int sm_count, SkinnyPlan *plan)
{
    const int mt = mt_for(M);
    const int stages = 4;
    plan->use_tma = 1;
    plan->mt = mt;
    plan->stages = stages;
    // Preferred: 128-column strips whose 8 K-slices form one cluster and reduce through shared memory
    // (no global scratch).  Needs enough strips to fill the machine and an X slice that fits.
    {
        const int rows = skinny_tma_stage_rows(mt, 1);
        const int strips = (int)((N + 127) / 128);
        int64_t ksplit = 8;
        int64_t kchunk = ((K + ksplit - 1) / ksplit + rows - 1) / rows * rows;
        ksplit = (K + kchunk - 1) / kchunk;
        const bool fits = kchunk * mt * 4 <= 64 * 1024 && kchunk >= 128;
        const bool fills = (int64_t)strips * ksplit >= sm_count;
        // (M > 8 holds one CTA per SM for its registers: a 256-CTA cluster grid would run in two waves)
        if (mt <= 8 && ksplit >= 2 && ksplit <= 8 && fits && fills) {
            plan->cluster = 1;
            plan->strips = strips;
            plan->ksplit = (int)ksplit;
            plan->kchunk = (int)kchunk;
            plan->partial_floats = 0;
            plan->smem_bytes = skinny_tma_smem_bytes(mt, (int)kchunk, stages);
            return;
        }
    }
    plan->cluster = 0;
    const int cols = skinny_tma_strip_cols(mt, 0), rows = skinny_tma_stage_rows(mt, 0);
    const int strips = (int)((N + cols - 1) / cols);
    const int ctas_per_sm = 2;
    int64_t ksplit = (ctas_per_sm * (int64_t)sm_count) / strips;
    if (ksplit < 1) ksplit = 1;
    const int64_t max_split = (K + 4 * rows - 1) / (4 * rows);  // at least one trip round the ring
    if (ksplit > max_split) ksplit = max_split;
    int64_t kchunk = (K + ksplit - 1) / ksplit;
    kchunk = (kchunk + rows - 1) / rows * rows;
    const int64_t max_chunk = (64 * 1024) / (4 * mt) / rows * rows;  // X slice within 64 KB
    if (kchunk > max_chunk) kchunk = max_chunk;
    ksplit = (K + kchunk - 1) / kchunk;
    plan->strips = strips;
    plan->ksplit = (int)ksplit;
    plan->kchunk = (int)kchunk;
    plan->partial_floats = ksplit > 1 ? ksplit * M * N : 0;
    plan->smem_bytes = skinny_tma_smem_bytes(mt, (int)kchunk, stages);
}

void skinny_plan(int64_t M, int64_t N, int64_t K, const float *W, int sm_count, SkinnyPlan *plan)
{
    if ((N % 4 == 0) && ((reinterpret_cast<uintptr_t>(W) & 15) == 0)) {
        skinny_plan_tma(M, N, K, sm_count, plan);
        return;
    }
    plan->use_tma = 0;
    plan->cluster = 0;
    plan->stages = 0;
    const int mt = mt_for(M);
    const int strips = (int)((N + SK_STRIP - 1) / SK_STRIP);
    int64_t ksplit = (2 * (int64_t)sm_count) / strips;
    if (ksplit < 1) ksplit = 1;
    const int64_t max_split = (K + 63) / 64;  // at least 8 rows per warp
    if (ksplit > max_split) ksplit = max_split;
    int64_t kchunk = (K + ksplit - 1) / ksplit;
    const int64_t max_chunk = (64 * 1024) / (4 * mt);  // keep the X slice within 64 KB of shared memory
    if (kchunk > max_chunk) kchunk = max_chunk;
    ksplit = (K + kchunk - 1) / kchunk;
    plan->mt = mt;
    plan->strips = strips;
    plan->ksplit = (int)ksplit;
    plan->kchunk = (int)kchunk;
    plan->partial_floats = ksplit > 1 ? ksplit * M * N : 0;
    const int rm = mt < 8 ? mt : 8;
    size_t sx = (size_t)kchunk * mt * 4, sr = (size_t)SK_WARPS * rm * SK_STRIP * 4;
    plan->smem_bytes = sx > sr ? sx : sr;
}

int launch_skinny(const SkinnyArgs &args, const SkinnyPlan &plan, cudaStream_t st)
{
    if (plan.use_tma) return launch_skinny_tma(args, plan, st);
    const bool vec = (args.N % 4 == 0) && ((reinterpret_cast<uintptr_t>(args.W) & 15) == 0);
    dim3 grid((unsigned)plan.strips, (unsigned)plan.ksplit);
    switch (plan.mt) {
    case 1: return launch_mt<1>(args, vec, grid, plan.smem_bytes, st);
    case 2: return launch_mt<2>(args, vec, grid, plan.smem_bytes, st);
    case 4: return launch_mt<4>(args, vec, grid, plan.smem_bytes, st);
    case 8: return launch_mt<8>(args, vec, grid, plan.smem_bytes, st);
    case 16: return launch_mt<16>(args, vec, grid, plan.smem_bytes, st);
    default: return launch_mt<32>(args, vec, grid, plan.smem_bytes, st);
    }
}

}  // namespace axb

// ------------------------------------------------- allocation-free entry point
//
// axb_skinny_gemm_static runs the same kernel as the skinny route above but
// takes its split-K scratch from a fixed array that is part of the library
// image, so the call itself never asks the driver for memory.  Every GPU that
// loads the library carries the array (AXB_STATIC_SCRATCH_BYTES) until exit.

namespace {

constexpr int64_t kStaticPartialFloats = (int64_t)1 << 20;   // 4 MiB of split-K partial sums
constexpr int kStaticCounters = 1023;                        // one arrival counter per 128-column strip
constexpr int kStaticWords = kStaticCounters + 1;            // ... and, after them, the word a timed-out wait reports in
constexpr int kMaxDevices = 64;

// In host code this name is only a handle for cudaGetSymbolAddress; the device
// address it stands for differs per GPU and is looked up once per device below.
static __device__ __align__(256) float g_static_scratch[kStaticPartialFloats + kStaticWords];

static float *s_scratch_addr[kMaxDevices];   // device address of g_static_scratch, per device ordinal
static int s_sm_count[kMaxDevices];

}  // namespace

extern "C" int axb_skinny_gemm_static(const float *X, const float *W, const float *bias, float *Y,
                                      int64_t M, int64_t N, int64_t K, float alpha, float beta, int act,
                                      void *cuda_stream)
{
    using namespace axb;
    if (!X || !W || !Y) return set_error(AXB_ERR_NULL_ARG, "skinny_gemm_static: NULL operand");
    if (M < 1 || M > 32 || N < 1 || K < 1)
        return set_error(AXB_ERR_INVALID_SHAPE, "skinny_gemm_static: needs 1 <= M <= 32, N >= 1, K >= 1 (got M=%lld N=%lld K=%lld)",
                         (long long)M, (long long)N, (long long)K);
    if (act < AXB_ACT_NONE || act > AXB_ACT_GELU)
        return set_error(AXB_ERR_INVALID_SHAPE, "skinny_gemm_static: unknown activation %d", act);
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return set_error(AXB_ERR_BACKEND, "skinny_gemm_static: cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return set_error(AXB_ERR_BACKEND, "skinny_gemm_static: device ordinal %d not supported", dev);
    if (!s_scratch_addr[dev]) {
        // first call on this device (it is the current one): resolve the array's device address
        void *addr = nullptr;
        e = cudaGetSymbolAddress(&addr, g_static_scratch);
        if (e != cudaSuccess || !addr)
            return set_error(AXB_ERR_BACKEND, "skinny_gemm_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        int sms = 0;
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess || sms <= 0)
            return set_error(AXB_ERR_BACKEND, "skinny_gemm_static: cudaDeviceGetAttribute: %s", cudaGetErrorString(e));
        // the word a timed-out wait reports in starts at zero (the image initialises the array to zero; a previous
        // process cannot have touched this context's copy, so this is belt and braces)
        e = cudaMemset(static_cast<float *>(addr) + kStaticPartialFloats + kStaticCounters, 0, sizeof(int));
        if (e != cudaSuccess) return set_error(AXB_ERR_BACKEND, "skinny_gemm_static: cudaMemset: %s", cudaGetErrorString(e));
        s_sm_count[dev] = sms;
        s_scratch_addr[dev] = static_cast<float *>(addr);
    }
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    float *scratch = s_scratch_addr[dev];
    int *counters = reinterpret_cast<int *>(scratch + kStaticPartialFloats);
    int *err_word = counters + kStaticCounters;
    SkinnyArgs a;
    a.X = X; a.W = W; a.bias = bias; a.Y = Y; a.M = (int)M; a.N = N; a.K = K;
    a.alpha = alpha; a.beta = beta; a.act = act;
    a.err = err_word;
    // the same choice of kernel as the skinny route of axb_gemm_bias_act: above 8 rows the tensor-core kernel,
    // which reduces inside its clusters and needs no scratch at all
    if (M >= 9 && skinny_tc_applicable(M, N, K, X, W)) {
        a.ksplit = 0; a.kchunk = 0; a.stages = 0; a.cluster = 0; a.partial = nullptr; a.counters = nullptr;
        int le = launch_skinny_tc(a, s_sm_count[dev], st);
        if (le) return set_error(AXB_ERR_BACKEND, "skinny_gemm_static: launch: %s", cudaGetErrorString((cudaError_t)le));
        return AXB_OK;
    }
    SkinnyPlan plan;
    skinny_plan(M, N, K, W, s_sm_count[dev], &plan);
    if (plan.partial_floats > kStaticPartialFloats || plan.strips > kStaticCounters)
        return set_error(AXB_ERR_INVALID_SHAPE,
                         "skinny_gemm_static: M=%lld N=%lld K=%lld needs %lld scratch floats and %d strip counters; the built-in "
                         "scratch holds %lld and %d (use axb_gemm_bias_act, which allocates)",
                         (long long)M, (long long)N, (long long)K, (long long)plan.partial_floats, plan.strips,
                         (long long)kStaticPartialFloats, kStaticCounters);
    // the array keeps whatever the previous call left: the arrival counters must start at zero
    e = cudaMemsetAsync(counters, 0, (size_t)plan.strips * sizeof(int), st);
    if (e != cudaSuccess) return set_error(AXB_ERR_BACKEND, "skinny_gemm_static: cudaMemsetAsync: %s", cudaGetErrorString(e));
    a.ksplit = plan.ksplit; a.kchunk = plan.kchunk; a.stages = plan.stages; a.cluster = plan.cluster;
    a.partial = (plan.ksplit > 1 && !plan.cluster) ? scratch : nullptr;
    a.counters = counters;
    int le = launch_skinny(a, plan, st);
    if (le) return set_error(AXB_ERR_BACKEND, "skinny_gemm_static: launch: %s", cudaGetErrorString((cudaError_t)le));
    return AXB_OK;
}

extern "C" int axb_skinny_gemm_static_error(void)
{
    using namespace axb;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices || !s_scratch_addr[dev]) return 0;
    int *err_word = reinterpret_cast<int *>(s_scratch_addr[dev] + kStaticPartialFloats) + kStaticCounters;
    int v = 0;
    if (cudaMemcpy(&v, err_word, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (v) {
        cudaMemset(err_word, 0, sizeof(int));
        set_error(AXB_ERR_BACKEND, "skinny_gemm_static: a kernel gave up on a bounded wait (code %d)", v);
    }
    return v;
}
