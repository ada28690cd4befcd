// api.cu — the C ABI declared in include/axiom_b200.h: argument checks, route
// selection (skinny-M / tcgen05 core), scratch management and error reporting.
// No arithmetic happens on the host and there is no host fallback: when a
// kernel cannot run the call fails with a status and a message.
#include "../../include/axiom_b200.h"

#include "elementwise.cuh"
#include "errors.cuh"
#include "gemm_tc.cuh"
#include "prepass.cuh"
#include "ptx.cuh"
#include "qgemv.cuh"
#include "qskinny_tc.cuh"
#include "kv_attend.cuh"
#include "sdpa.cuh"
#include "skinny.cuh"

#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

using namespace axb;

namespace {

struct Engine {
    bool ready = false;
    int device = 0;
    int sm_count = 148;
    cudaStream_t stream = 0;
    int fp32_mode = AXB_FP32_3XTF32;
    // K elements accumulated inside the tensor core per chunk in the split-precision modes
    int chunk_tf32 = 256, chunk_bf16 = 512;
    // grow-only scratch for operand planes (backend-owned, like the reference's
    // device scratch arena, src/compute/backends/cuda/internal.h:57-90)
    void *ws = nullptr;
    size_t ws_bytes = 0;
    // skinny route: split-K partials + per-strip arrival counters
    float *sk_partial = nullptr;
    size_t sk_partial_floats = 0;
    int *sk_counters = nullptr;
    int sk_counter_cap = 0;
    int *err_word = nullptr;
    int *gemm_counters = nullptr;   // split-K arrival counters of the tensor-core GEMM (zero between launches)
    // output range of the last skinny kernel, which lets the next one start under it: a skinny call whose WEIGHTS lie
    // in that range must not prefetch them early
    const char *chain_lo = nullptr, *chain_hi = nullptr;
    int64_t launches = 0;
    // grow-only buffer for intermediate results a fused route cannot avoid (the unfused qkv projection)
    void *aux = nullptr;
    size_t aux_bytes = 0;
    // host-operand GEMM: device staging (grow-only), copy streams and the events that order them
    void *hp_buf = nullptr;
    size_t hp_bytes = 0;
    cudaStream_t hp_in = nullptr, hp_out = nullptr;
    cudaEvent_t hp_ev[9] = {};
    // optional timing of the last GEMM-family call: events around its pre-pass and its core kernel
    bool profiling = false;
    static constexpr int EV_RING = 256;
    cudaEvent_t ev[EV_RING][3] = {};
    int ev_count = 0;   // calls recorded since the last summary (ring keeps the newest EV_RING)
    char msg[320] = "";
};

// One engine per device.  A host thread drives the device it selected with axb_init (a thread that never did uses
// the first device any thread initialised): one process per GPU sees exactly one engine, a host that walks several
// devices from one thread (the multi-GPU entry points, mgpu.cu) switches with axb_init(device).
constexpr int kMaxDevices = 16;
Engine g_engines[kMaxDevices];
thread_local int tl_device = -1;
int g_default_device = -1;

inline Engine &cur()
{
    const int d = tl_device >= 0 ? tl_device : (g_default_device >= 0 ? g_default_device : 0);
    return g_engines[d];
}

// split-K scratch of the tensor-core GEMM: one partial tile per work item (up to 147 tiles x 4 slices of 128 x 256 fp32 would be 74 MiB;
// the planner cuts K less finely when the scratch does not hold that)
constexpr size_t kSplitScratch = (size_t)64 << 20;
constexpr int kSplitCounters = 1024;

int fail(int status, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(cur().msg, sizeof cur().msg, fmt, ap);
    va_end(ap);
    return status;
}

int cuda_fail(const char *what, int err)
{
    return fail(AXB_ERR_BACKEND, "%s: %s%s%s", what, cudaGetErrorString((cudaError_t)err),
                gemm_tc_last_error()[0] ? " / " : "", gemm_tc_last_error());
}

inline size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

inline void mark(int i)
{
    if (!cur().profiling) return;
    cudaEvent_t *slot = cur().ev[cur().ev_count % Engine::EV_RING];
    if (!slot[i]) cudaEventCreate(&slot[i]);
    cudaEventRecord(slot[i], cur().stream);
    if (i == 2) cur().ev_count++;
}

int ensure_ready()
{
    if (cur().ready) return AXB_OK;
    return axb_init(-1);
}

int ensure_ws(size_t bytes)
{
    if (bytes <= cur().ws_bytes) return AXB_OK;
    if (cur().ws) {
        cudaStreamSynchronize(cur().stream);
        cudaFree(cur().ws);
        cur().ws = nullptr;
        cur().ws_bytes = 0;
    }
    const size_t want = round_up(bytes + bytes / 8, (size_t)1 << 20);
    cudaError_t e = cudaMalloc(&cur().ws, want);
    if (e != cudaSuccess) return fail(AXB_ERR_ALLOC, "scratch allocation of %zu bytes failed: %s", want, cudaGetErrorString(e));
    cur().ws_bytes = want;
    return AXB_OK;
}

struct Carver {
    char *p;
    size_t off = 0;
    void *take(size_t bytes)
    {
        void *r = p + off;
        off += round_up(bytes, 1024);
        return r;
    }
};

// the split-K scratch, carved behind a call's operand planes
TcSplitK take_splitk(Carver &c)
{
    TcSplitK sk;
    sk.scratch = c.take(kSplitScratch);
    sk.scratch_bytes = kSplitScratch;
    sk.counters = cur().gemm_counters;
    sk.n_counters = kSplitCounters;
    return sk;
}

// planes of one fp32 operand, written by the split pre-pass
struct SplitOperand {
    int mode;
    int64_t rows, k, pitch;
    size_t plane_bytes;
    size_t total() const { return (size_t)split_num_planes(mode) * round_up(plane_bytes, 1024); }
};

SplitOperand plan_split(int mode, int64_t rows, int64_t k)
{
    SplitOperand s;
    s.mode = mode;
    s.rows = rows;
    s.k = k;
    s.pitch = (int64_t)round_up((size_t)k, 16);
    s.plane_bytes = (size_t)rows * s.pitch * split_elem_bytes(mode);
    return s;
}

int run_split(const SplitOperand &s, const float *src, int64_t ld, bool transposed, Carver &c, TcOperand &op,
              int64_t chunk_k = 0, int64_t chunk_stride = 0)
{
    void *planes[3] = { nullptr, nullptr, nullptr };
    op.nplanes = split_num_planes(s.mode);
    for (int i = 0; i < op.nplanes; ++i) {
        planes[i] = c.take(s.plane_bytes);
        op.plane[i] = planes[i];
    }
    op.rows = s.rows;
    op.pitch_elems = s.pitch;
    int e = split_planes(s.mode, src, s.rows, s.k, ld, transposed, planes, s.pitch, cur().sm_count, cur().stream, chunk_k,
                         chunk_stride);
    cur().launches++;
    return e;
}

// operand split, MMA kind and product list of the current fp32 mode
void fp32_mode_plan(int &split_mode, int &kind, TcProducts &prod)
{
    memset(&prod, 0, sizeof prod);
    switch (cur().fp32_mode) {
    case AXB_FP32_BF16:
        split_mode = SPLIT_BF16X1; kind = KIND_BF16;
        prod.n = 1; prod.a[0] = 0; prod.b[0] = 0;
        prod.chunk_k = 0;
        break;
    case AXB_FP32_BF16X3:
        split_mode = SPLIT_BF16X2; kind = KIND_BF16;
        prod.n = 3; prod.a[0] = 1; prod.b[0] = 0; prod.a[1] = 0; prod.b[1] = 1; prod.a[2] = 0; prod.b[2] = 0;
        prod.chunk_k = cur().chunk_bf16;
        break;
    default:
        split_mode = SPLIT_TF32X2; kind = KIND_TF32;
        // small cross terms first, the hi.hi product last
        prod.n = 3; prod.a[0] = 1; prod.b[0] = 0; prod.a[1] = 0; prod.b[1] = 1; prod.a[2] = 0; prod.b[2] = 0;
        prod.chunk_k = cur().chunk_tf32;
        break;
    }
}

// the dense fp32 contraction on the tensor cores
int gemm_tc_f32(const float *A, const float *B, const float *bias, float *C, int64_t M, int64_t N, int64_t K,
                int ta, int tb, float alpha, float beta, int act, float *const *extra = nullptr, int n_extra = 0,
                int64_t a_chunk_k = 0, int64_t a_chunk_stride = 0, const int64_t *head_shape = nullptr,
                float *const *head_out = nullptr, const TcOperand *prepared_b = nullptr)
{
    int split_mode, kind;
    TcProducts prod;
    fp32_mode_plan(split_mode, kind, prod);
    const SplitOperand sa = plan_split(split_mode, M, K), sb = plan_split(split_mode, N, K);
    int st = ensure_ws(sa.total() + (prepared_b ? 0 : sb.total()) + kSplitScratch);
    if (st) return st;
    Carver carve{ (char *)cur().ws };
    const TcSplitK sk = take_splitk(carve);
    TcOperand opa, opb;
    mark(0);
    // A is [M,K] (k contiguous) unless trans_a, where it is stored [K,M];
    // B is [K,N] (k outermost) unless trans_b, where it is stored [N,K].
    void *pa[3] = { nullptr, nullptr, nullptr }, *pb[3] = { nullptr, nullptr, nullptr };
    opa.nplanes = split_num_planes(split_mode);
    for (int i = 0; i < opa.nplanes; ++i) opa.plane[i] = pa[i] = carve.take(sa.plane_bytes);
    opa.rows = sa.rows; opa.pitch_elems = sa.pitch;
    int e;
    if (prepared_b) {
        // the weight's planes exist already: only the left operand is split
        opb = *prepared_b;
        e = split_planes(split_mode, A, M, K, ta ? M : K, ta != 0, pa, sa.pitch, cur().sm_count, cur().stream, a_chunk_k,
                         a_chunk_stride);
    } else {
        // both operands in one pre-pass launch
        opb.nplanes = opa.nplanes;
        for (int i = 0; i < opb.nplanes; ++i) opb.plane[i] = pb[i] = carve.take(sb.plane_bytes);
        opb.rows = sb.rows; opb.pitch_elems = sb.pitch;
        e = split_planes_pair(split_mode, A, M, ta ? M : K, ta != 0, pa, sa.pitch, a_chunk_k, a_chunk_stride, B, N,
                              tb ? K : N, tb == 0, pb, sb.pitch, K, cur().sm_count, cur().stream);
    }
    cur().launches++;
    if (e) return cuda_fail("split operands", e);
    TcEpilogue ep;
    ep.n_extra = 0;
    ep.alpha = alpha; ep.beta = beta; ep.bias = bias; ep.colscale = nullptr; ep.act = act;
    ep.out_mode = OUT_F32; ep.C = C; ep.acc_out = nullptr; ep.ldc = N;
    ep.n_extra = n_extra;
    for (int i = 0; i < n_extra && i < TC_MAX_EXTRA; ++i) ep.c_extra[i] = extra[i];
    if (head_shape) {   // { S, H, dk }: the epilogue scatters into head_out[0..2] as [B*H, S, dk]
        ep.hs_S = (int)head_shape[0]; ep.hs_H = (int)head_shape[1]; ep.hs_dk = (int)head_shape[2];
        for (int i = 0; i < 3; ++i) ep.hs_out[i] = head_out[i];
    }
    mark(1);
    e = launch_gemm_tc(kind, opa, opb, prod, M, N, K, ep, cur().err_word, cur().sm_count, cur().stream, &sk);
    mark(2);
    cur().launches++;
    if (e) return cuda_fail("tcgen05 gemm", e);
    return AXB_OK;
}

int gemm_skinny(const float *X, const float *W, const float *bias, float *Y, int64_t M, int64_t N, int64_t K,
                float alpha, float beta, int act)
{
    // back-to-back skinny calls (a decode step walks a chain of them) overlap: this call may request its first weight
    // tiles while the previous one drains, unless those weights are what the previous call wrote
    const char *w_lo = reinterpret_cast<const char *>(W), *w_hi = w_lo + (size_t)K * N * sizeof(float);
    const int pdl = !(cur().chain_lo && w_lo < cur().chain_hi && cur().chain_lo < w_hi);
    cur().chain_lo = reinterpret_cast<const char *>(Y);
    cur().chain_hi = cur().chain_lo + (size_t)M * N * sizeof(float);
    // above 8 rows the fp32 pipe, not memory, paces the FMA kernels: the tensor-core variant takes over
    if (M >= 9 && skinny_tc_applicable(M, N, K, X, W)) {
        SkinnyArgs a;
        a.X = X; a.W = W; a.bias = bias; a.Y = Y; a.M = (int)M; a.N = N; a.K = K;
        a.alpha = alpha; a.beta = beta; a.act = act;
        a.ksplit = 0; a.kchunk = 0; a.stages = 0; a.cluster = 0; a.partial = nullptr; a.counters = nullptr;
        a.err = cur().err_word;
        a.pdl = pdl;
        mark(0);
        mark(1);
        int e = launch_skinny_tc(a, cur().sm_count, cur().stream);
        mark(2);
        cur().launches++;
        if (e) return cuda_fail("skinny tensor-core gemm", e);
        return AXB_OK;
    }
    SkinnyPlan plan;
    skinny_plan(M, N, K, W, cur().sm_count, &plan);
    if ((size_t)plan.partial_floats > cur().sk_partial_floats) {
        if (cur().sk_partial) { cudaStreamSynchronize(cur().stream); cudaFree(cur().sk_partial); cur().sk_partial = nullptr; }
        const size_t want = (size_t)plan.partial_floats + (size_t)plan.partial_floats / 4;
        cudaError_t e = cudaMalloc(&cur().sk_partial, want * sizeof(float));
        if (e != cudaSuccess) { cur().sk_partial_floats = 0; return fail(AXB_ERR_ALLOC, "skinny scratch: %s", cudaGetErrorString(e)); }
        cur().sk_partial_floats = want;
    }
    if (plan.strips > cur().sk_counter_cap) {
        if (cur().sk_counters) { cudaStreamSynchronize(cur().stream); cudaFree(cur().sk_counters); cur().sk_counters = nullptr; }
        const int want = plan.strips * 2 + 64;
        cudaError_t e = cudaMalloc(&cur().sk_counters, (size_t)want * sizeof(int));
        if (e != cudaSuccess) { cur().sk_counter_cap = 0; return fail(AXB_ERR_ALLOC, "skinny counters: %s", cudaGetErrorString(e)); }
        cudaMemsetAsync(cur().sk_counters, 0, (size_t)want * sizeof(int), cur().stream);
        cur().sk_counter_cap = want;
    }
    SkinnyArgs a;
    a.X = X; a.W = W; a.bias = bias; a.Y = Y; a.M = (int)M; a.N = N; a.K = K;
    a.alpha = alpha; a.beta = beta; a.act = act;
    a.ksplit = plan.ksplit; a.kchunk = plan.kchunk; a.stages = plan.stages; a.cluster = plan.cluster;
    a.partial = (plan.ksplit > 1 && !plan.cluster) ? cur().sk_partial : nullptr;
    a.counters = cur().sk_counters;
    a.err = cur().err_word;
    a.pdl = pdl;
    mark(0);
    mark(1);
    int e = launch_skinny(a, plan, cur().stream);
    mark(2);
    cur().launches++;
    if (e) return cuda_fail("skinny gemm", e);
    return AXB_OK;
}

}  // namespace

cudaStream_t axb::engine_stream() { return cur().stream; }
int axb::engine_device() { return tl_device >= 0 ? tl_device : g_default_device; }

int axb::set_error(int status, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(cur().msg, sizeof cur().msg, fmt, ap);
    va_end(ap);
    return status;
}

// ------------------------------------------------------------------ lifecycle

extern "C" int axb_init(int device)
{
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0)
        return fail(AXB_ERR_BACKEND, "no CUDA device: %s", e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
    if (device < 0) {
        if (tl_device >= 0) device = tl_device;
        else if (g_default_device >= 0) device = g_default_device;
        else if (cudaGetDevice(&device) != cudaSuccess) device = 0;
    }
    if (device >= count || device >= kMaxDevices)
        return fail(AXB_ERR_BACKEND, "device %d out of range (%d devices, at most %d engines)", device, count, kMaxDevices);
    if ((e = cudaSetDevice(device)) != cudaSuccess) return cuda_fail("cudaSetDevice", e);
    tl_device = device;
    if (g_default_device < 0) g_default_device = device;
    Engine &en = g_engines[device];
    if (en.ready) return AXB_OK;
    cudaDeviceProp prop;
    if ((e = cudaGetDeviceProperties(&prop, device)) != cudaSuccess) return cuda_fail("cudaGetDeviceProperties", e);
    if (prop.major != 10)
        return fail(AXB_ERR_BACKEND, "device %d is sm_%d%d; this engine holds sm_100a code only", device, prop.major, prop.minor);
    en.device = device;
    en.sm_count = prop.multiProcessorCount;
    if ((e = cudaMalloc(&en.err_word, sizeof(int))) != cudaSuccess) return cuda_fail("cudaMalloc", e);
    cudaMemset(en.err_word, 0, sizeof(int));
    if ((e = cudaMalloc(&en.gemm_counters, kSplitCounters * sizeof(int))) != cudaSuccess) return cuda_fail("cudaMalloc", e);
    cudaMemset(en.gemm_counters, 0, kSplitCounters * sizeof(int));
    const char *mode = getenv("AX_B200_FP32_MODE");
    if (mode) {
        if (!strcmp(mode, "bf16")) en.fp32_mode = AXB_FP32_BF16;
        else if (!strcmp(mode, "bf16x3")) en.fp32_mode = AXB_FP32_BF16X3;
        else if (!strcmp(mode, "3xtf32")) en.fp32_mode = AXB_FP32_3XTF32;
    }
    en.ready = true;
    if (getenv("AX_B200_VERBOSE"))
        fprintf(stderr, "axiom: b200 engine on device %d (%s, %d SMs), fp32 mode %d\n", device, prop.name,
                en.sm_count, en.fp32_mode);
    return AXB_OK;
}

extern "C" void axb_shutdown(void)
{
    for (int d = 0; d < kMaxDevices; ++d) {
        Engine &en = g_engines[d];
        if (!en.ready) continue;
        cudaSetDevice(d);
        cudaDeviceSynchronize();
        if (en.ws) cudaFree(en.ws);
        if (en.sk_partial) cudaFree(en.sk_partial);
        if (en.sk_counters) cudaFree(en.sk_counters);
        if (en.err_word) cudaFree(en.err_word);
        if (en.gemm_counters) cudaFree(en.gemm_counters);
        if (en.hp_buf) cudaFree(en.hp_buf);
        if (en.aux) cudaFree(en.aux);
        if (en.hp_in) cudaStreamDestroy(en.hp_in);
        if (en.hp_out) cudaStreamDestroy(en.hp_out);
        for (auto &ev : en.hp_ev)
            if (ev) cudaEventDestroy(ev);
        for (auto &slot : en.ev)
            for (auto &ev : slot)
                if (ev) cudaEventDestroy(ev);
        en = Engine();
    }
    tl_device = -1;
    g_default_device = -1;
}

extern "C" int axb_device_count(void)
{
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess) return 0;
    return count;
}

extern "C" void axb_synchronize(void)
{
    if (!cur().ready) return;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) cuda_fail("synchronize", e);
}

extern "C" void *axb_storage_alloc(size_t bytes)
{
    if (ensure_ready()) return nullptr;
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes ? bytes : 1);
    if (e != cudaSuccess) {
        fail(AXB_ERR_ALLOC, "storage_alloc(%zu): %s", bytes, cudaGetErrorString(e));
        return nullptr;
    }
    if (bytes) cudaMemsetAsync(p, 0, bytes, cur().stream);
    return p;
}

extern "C" void axb_storage_free(void *ptr)
{
    if (ptr) cudaFree(ptr);
}

extern "C" int axb_memcpy_h2d(void *dst, const void *src_host, size_t bytes)
{
    if (!dst || !src_host) return fail(AXB_ERR_NULL_ARG, "memcpy_h2d: NULL");
    if (ensure_ready()) return AXB_ERR_BACKEND;
    cudaError_t e = cudaMemcpyAsync(dst, src_host, bytes, cudaMemcpyHostToDevice, cur().stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(cur().stream);
    return e == cudaSuccess ? AXB_OK : cuda_fail("memcpy_h2d", e);
}

extern "C" int axb_memcpy_d2h(void *dst_host, const void *src, size_t bytes)
{
    if (!dst_host || !src) return fail(AXB_ERR_NULL_ARG, "memcpy_d2h: NULL");
    if (ensure_ready()) return AXB_ERR_BACKEND;
    cudaError_t e = cudaMemcpyAsync(dst_host, src, bytes, cudaMemcpyDeviceToHost, cur().stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(cur().stream);
    return e == cudaSuccess ? AXB_OK : cuda_fail("memcpy_d2h", e);
}

extern "C" int axb_memcpy_d2d(void *dst, const void *src, size_t bytes)
{
    if (!dst || !src) return fail(AXB_ERR_NULL_ARG, "memcpy_d2d: NULL");
    if (ensure_ready()) return AXB_ERR_BACKEND;
    cudaError_t e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, cur().stream);
    return e == cudaSuccess ? AXB_OK : cuda_fail("memcpy_d2d", e);
}

extern "C" void axb_set_stream(void *cuda_stream)
{
    cur().stream = (cudaStream_t)cuda_stream;
    cur().chain_lo = cur().chain_hi = nullptr;
}

extern "C" int axb_set_fp32_mode(int mode)
{
    if (mode < AXB_FP32_3XTF32 || mode > AXB_FP32_BF16) return fail(AXB_ERR_INVALID_SHAPE, "unknown fp32 mode %d", mode);
    cur().fp32_mode = mode;
    return AXB_OK;
}

extern "C" int axb_get_fp32_mode(void) { return cur().fp32_mode; }
extern "C" const char *axb_last_error(void) { return cur().msg; }

extern "C" int axb_device_error(void)
{
    if (!cur().ready || !cur().err_word) return 0;
    int v = 0;
    if (cudaMemcpy(&v, cur().err_word, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (v) {
        cudaMemset(cur().err_word, 0, sizeof(int));
        fail(AXB_ERR_BACKEND, "a kernel gave up on a bounded wait (code %d)", v);
    }
    return v;
}

extern "C" void axb_set_profiling(int on)
{
    cur().profiling = on != 0;
    cur().ev_count = 0;
}

extern "C" int axb_timing_summary(int *calls, float *prepass_ms_total, float *core_ms_total)
{
    if (!cur().profiling) return fail(AXB_ERR_BACKEND, "timing_summary: profiling is off");
    const int n = cur().ev_count < Engine::EV_RING ? cur().ev_count : Engine::EV_RING;
    float pre = 0.f, core = 0.f;
    for (int i = 0; i < n; ++i) {
        cudaEvent_t *slot = cur().ev[(cur().ev_count - 1 - i) % Engine::EV_RING];
        cudaError_t e = cudaEventSynchronize(slot[2]);
        if (e != cudaSuccess) return cuda_fail("timing_summary", e);
        float a = 0.f, b = 0.f;
        cudaEventElapsedTime(&a, slot[0], slot[1]);
        cudaEventElapsedTime(&b, slot[1], slot[2]);
        pre += a;
        core += b;
    }
    if (calls) *calls = n;
    if (prepass_ms_total) *prepass_ms_total = pre;
    if (core_ms_total) *core_ms_total = core;
    cur().ev_count = 0;
    return AXB_OK;
}

extern "C" int axb_timing_samples(float *prepass_ms, float *core_ms, int cap, int *n_out)
{
    if (!cur().profiling) return fail(AXB_ERR_BACKEND, "timing_samples: profiling is off");
    if (!n_out || cap < 0) return fail(AXB_ERR_NULL_ARG, "timing_samples: NULL");
    int n = cur().ev_count < Engine::EV_RING ? cur().ev_count : Engine::EV_RING;
    if (n > cap) n = cap;
    for (int i = 0; i < n; ++i) {   // oldest of the kept calls first
        cudaEvent_t *slot = cur().ev[(cur().ev_count - n + i) % Engine::EV_RING];
        cudaError_t e = cudaEventSynchronize(slot[2]);
        if (e != cudaSuccess) return cuda_fail("timing_samples", e);
        float a = 0.f, b = 0.f;
        cudaEventElapsedTime(&a, slot[0], slot[1]);
        cudaEventElapsedTime(&b, slot[1], slot[2]);
        if (prepass_ms) prepass_ms[i] = a;
        if (core_ms) core_ms[i] = b;
    }
    *n_out = n;
    return AXB_OK;
}

extern "C" int64_t axb_launch_count(int reset)
{
    const int64_t v = cur().launches;
    if (reset) cur().launches = 0;
    return v;
}

// ----------------------------------------------------------------- GEMM family

extern "C" int axb_gemm_bias_act(const float *A, const float *B, const float *bias, float *C, int64_t M,
                                 int64_t N, int64_t K, int trans_a, int trans_b, float alpha, float beta,
                                 int act)
{
    if (M < 0 || N < 0 || K < 0) return fail(AXB_ERR_INVALID_SHAPE, "gemm: negative dimension");
    if (M == 0 || N == 0) return AXB_OK;  // nothing to write; empty operands may legitimately be NULL
    if (!C || (K > 0 && (!A || !B))) return fail(AXB_ERR_NULL_ARG, "gemm: NULL operand");
    if (act < AXB_ACT_NONE || act > AXB_ACT_GELU) return fail(AXB_ERR_INVALID_SHAPE, "gemm: unknown activation %d", act);
    if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return fail(AXB_ERR_INVALID_SHAPE, "gemm: dimension exceeds 2^31-1");
    int st = ensure_ready();
    if (st) return st;
    if (K == 0) {
        // empty contraction: C = act(beta*C + bias) via the skinny kernel's epilogue is not
        // reachable (no rows to stream); express it as the bias/activation passes
        if (beta == 0.0f) cudaMemsetAsync(C, 0, (size_t)M * N * sizeof(float), cur().stream);
        else if (beta != 1.0f) return fail(AXB_ERR_NOT_IMPLEMENTED, "gemm: K == 0 with beta not in {0,1}");
        if (bias) { int e = launch_bias_add(C, bias, 1, C, M, N, cur().sm_count, cur().stream); cur().launches++; if (e) return cuda_fail("bias_add", e); }
        if (act) { int e = launch_unary(act == AXB_ACT_RELU ? 0 : 1, C, C, M * N, cur().sm_count, cur().stream); cur().launches++; if (e) return cuda_fail("activation", e); }
        return AXB_OK;
    }
    if (M <= 32 && !trans_a && !trans_b) return gemm_skinny(A, B, bias, C, M, N, K, alpha, beta, act);
    return gemm_tc_f32(A, B, bias, C, M, N, K, trans_a, trans_b, alpha, beta, act);
}

extern "C" int axb_gemm_bias_act_scatter(const float *A, const float *B, const float *bias, float *C,
                                         float *const *C_more, int n_more, int64_t M, int64_t N, int64_t K,
                                         int trans_a, int trans_b, float alpha, float beta, int act)
{
    if (M < 0 || N < 0 || K <= 0) return fail(AXB_ERR_INVALID_SHAPE, "gemm_scatter: bad shape");
    if (M == 0 || N == 0) return AXB_OK;
    if (!A || !B || !C || (n_more > 0 && !C_more)) return fail(AXB_ERR_NULL_ARG, "gemm_scatter: NULL operand");
    if (n_more < 0 || n_more > TC_MAX_EXTRA) return fail(AXB_ERR_INVALID_SHAPE, "gemm_scatter: at most %d extra destinations", TC_MAX_EXTRA);
    for (int i = 0; i < n_more; ++i)
        if (!C_more[i]) return fail(AXB_ERR_NULL_ARG, "gemm_scatter: NULL destination %d", i);
    if (act < AXB_ACT_NONE || act > AXB_ACT_GELU) return fail(AXB_ERR_INVALID_SHAPE, "gemm_scatter: unknown activation %d", act);
    if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return fail(AXB_ERR_INVALID_SHAPE, "gemm_scatter: dimension exceeds 2^31-1");
    int st = ensure_ready();
    if (st) return st;
    return gemm_tc_f32(A, B, bias, C, M, N, K, trans_a, trans_b, alpha, beta, act, C_more, n_more);
}

extern "C" int axb_gemm_gathered_scatter(const float *A_gathered, int chunks, int64_t chunk_k, const float *B,
                                         const float *bias, float *C, float *const *C_more, int n_more, int64_t M,
                                         int64_t N, float alpha, float beta, int act)
{
    if (chunks < 1 || chunk_k < 1 || (chunk_k % 4) != 0)
        return fail(AXB_ERR_INVALID_SHAPE, "gemm_gathered: needs chunks >= 1 and chunk_k a positive multiple of 4");
    if (M < 0 || N < 0) return fail(AXB_ERR_INVALID_SHAPE, "gemm_gathered: negative dimension");
    if (M == 0 || N == 0) return AXB_OK;
    if (!A_gathered || !B || !C || (n_more > 0 && !C_more)) return fail(AXB_ERR_NULL_ARG, "gemm_gathered: NULL operand");
    if (n_more < 0 || n_more > TC_MAX_EXTRA) return fail(AXB_ERR_INVALID_SHAPE, "gemm_gathered: at most %d extra destinations", TC_MAX_EXTRA);
    for (int i = 0; i < n_more; ++i)
        if (!C_more[i]) return fail(AXB_ERR_NULL_ARG, "gemm_gathered: NULL destination %d", i);
    if (act < AXB_ACT_NONE || act > AXB_ACT_GELU) return fail(AXB_ERR_INVALID_SHAPE, "gemm_gathered: unknown activation %d", act);
    const int64_t K = (int64_t)chunks * chunk_k;
    if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return fail(AXB_ERR_INVALID_SHAPE, "gemm_gathered: dimension exceeds 2^31-1");
    int st = ensure_ready();
    if (st) return st;
    return gemm_tc_f32(A_gathered, B, bias, C, M, N, K, 0, 0, alpha, beta, act, C_more, n_more, chunk_k, M * chunk_k);
}

extern "C" int axb_ipc_get_handle(const void *dev_ptr, void *handle_64_bytes)
{
    if (!dev_ptr || !handle_64_bytes) return fail(AXB_ERR_NULL_ARG, "ipc_get_handle: NULL");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, const_cast<void *>(dev_ptr));
    if (e != cudaSuccess) return cuda_fail("cudaIpcGetMemHandle", e);
    memcpy(handle_64_bytes, &h, 64);
    return AXB_OK;
}

extern "C" int axb_ipc_open_handle(const void *handle_64_bytes, void **dev_ptr_out)
{
    if (!handle_64_bytes || !dev_ptr_out) return fail(AXB_ERR_NULL_ARG, "ipc_open_handle: NULL");
    int st = ensure_ready();
    if (st) return st;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle_64_bytes, 64);
    cudaError_t e = cudaIpcOpenMemHandle(dev_ptr_out, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return cuda_fail("cudaIpcOpenMemHandle", e);
    return AXB_OK;
}

extern "C" int axb_ipc_close_handle(void *dev_ptr)
{
    if (!dev_ptr) return AXB_OK;
    cudaError_t e = cudaIpcCloseMemHandle(dev_ptr);
    return e == cudaSuccess ? AXB_OK : cuda_fail("cudaIpcCloseMemHandle", e);
}

extern "C" int axb_gemm(const float *A, const float *B, float *C, int64_t M, int64_t N, int64_t K)
{
    return axb_gemm_bias_act(A, B, nullptr, C, M, N, K, 0, 0, 1.0f, 0.0f, AXB_ACT_NONE);
}

extern "C" int axb_gemm_nt(const float *A, const float *B, float *C, int64_t M, int64_t N, int64_t K)
{
    return axb_gemm_bias_act(A, B, nullptr, C, M, N, K, 0, 1, 1.0f, 0.0f, AXB_ACT_NONE);
}

extern "C" int axb_gemm_tn(const float *A, const float *B, float *C, int64_t M, int64_t N, int64_t K)
{
    return axb_gemm_bias_act(A, B, nullptr, C, M, N, K, 1, 0, 1.0f, 0.0f, AXB_ACT_NONE);
}

extern "C" int axb_gemm_ex(const float *A, const float *B, float alpha, float beta, float *C, int64_t M,
                           int64_t N, int64_t K)
{
    return axb_gemm_bias_act(A, B, nullptr, C, M, N, K, 0, 0, alpha, beta, AXB_ACT_NONE);
}

extern "C" int axb_gemm_relu(const float *A, const float *B, const float *bias, float *C, int64_t M,
                             int64_t N, int64_t K)
{
    return axb_gemm_bias_act(A, B, bias, C, M, N, K, 0, 0, 1.0f, 0.0f, AXB_ACT_RELU);
}

// ---------------------------------------------------------------- prepared weights
//
// A dense layer multiplies by the same weight matrix call after call; its tensor-core operand planes (hi/lo tf32 or
// bf16, K-major) are the same every time.  A prepared weight holds them, so a product against it splits the left
// operand only.  The reference's CPU backend does the same thing behind the scenes: cpu_opt keeps packed B panels
// in a cache keyed on the storage pointer and its generation counter (src/compute/backends/cpu_opt.c, pack_b cache).
struct axb_weight {
    const float *src;     // the caller's matrix (borrowed: the skinny route streams it as it is)
    int64_t K, N;
    int trans;            // src is [N,K] instead of [K,N]
    int mode;             // fp32 mode the planes were made for
    int device;
    void *planes;         // owned
    TcOperand op;
};

extern "C" int axb_weight_prepare(const float *B, int64_t K, int64_t N, int trans_b, axb_weight **out)
{
    if (!out) return fail(AXB_ERR_NULL_ARG, "weight_prepare: NULL");
    *out = nullptr;
    if (!B) return fail(AXB_ERR_NULL_ARG, "weight_prepare: NULL");
    if (K <= 0 || N <= 0 || K > INT32_MAX || N > INT32_MAX) return fail(AXB_ERR_INVALID_SHAPE, "weight_prepare: bad shape");
    int st = ensure_ready();
    if (st) return st;
    int split_mode, kind;
    TcProducts prod;
    fp32_mode_plan(split_mode, kind, prod);
    const SplitOperand sb = plan_split(split_mode, N, K);
    axb_weight *w = new axb_weight();
    w->src = B; w->K = K; w->N = N; w->trans = trans_b != 0; w->mode = cur().fp32_mode; w->device = cur().device;
    cudaError_t ce = cudaMalloc(&w->planes, sb.total());
    if (ce != cudaSuccess) {
        delete w;
        return fail(AXB_ERR_ALLOC, "weight_prepare: %zu bytes of operand planes: %s", sb.total(), cudaGetErrorString(ce));
    }
    Carver carve{ (char *)w->planes };
    int e = run_split(sb, B, trans_b ? K : N, trans_b == 0, carve, w->op);
    if (e) {
        cudaFree(w->planes);
        delete w;
        return cuda_fail("weight_prepare: split", e);
    }
    *out = w;
    return AXB_OK;
}

extern "C" void axb_weight_release(axb_weight *w)
{
    if (!w) return;
    if (w->planes) {
        cudaStreamSynchronize(cur().stream);
        cudaFree(w->planes);
    }
    delete w;
}

extern "C" int axb_gemm_prepared(const float *A, const axb_weight *W, const float *bias, float *C, int64_t M, int trans_a,
                                 float alpha, float beta, int act)
{
    if (!W) return fail(AXB_ERR_NULL_ARG, "gemm_prepared: NULL weight");
    if (M < 0) return fail(AXB_ERR_INVALID_SHAPE, "gemm_prepared: negative dimension");
    if (M == 0) return AXB_OK;
    if (!A || !C) return fail(AXB_ERR_NULL_ARG, "gemm_prepared: NULL operand");
    if (act < AXB_ACT_NONE || act > AXB_ACT_GELU) return fail(AXB_ERR_INVALID_SHAPE, "gemm_prepared: unknown activation %d", act);
    if (M > INT32_MAX) return fail(AXB_ERR_INVALID_SHAPE, "gemm_prepared: dimension exceeds 2^31-1");
    int st = ensure_ready();
    if (st) return st;
    if (W->device != cur().device) return fail(AXB_ERR_BACKEND, "gemm_prepared: the weight was prepared on device %d", W->device);
    if (W->mode != cur().fp32_mode)
        return fail(AXB_ERR_BACKEND, "gemm_prepared: the weight was prepared in fp32 mode %d, the engine is in mode %d", W->mode, cur().fp32_mode);
    // the same routes as axb_gemm_bias_act, so the results are the same bits
    if (M <= 32 && !trans_a && !W->trans) return gemm_skinny(A, W->src, bias, C, M, W->N, W->K, alpha, beta, act);
    return gemm_tc_f32(A, W->src, bias, C, M, W->N, W->K, trans_a, W->trans, alpha, beta, act, nullptr, 0, 0, 0, nullptr, nullptr,
                       &W->op);
}

extern "C" int axb_gemm_prepared_scatter(const float *A, int chunks, int64_t chunk_k, const axb_weight *W, const float *bias,
                                         float *C, float *const *C_more, int n_more, int64_t M, float alpha, float beta, int act)
{
    if (!W) return fail(AXB_ERR_NULL_ARG, "gemm_prepared_scatter: NULL weight");
    if (W->trans) return fail(AXB_ERR_INVALID_SHAPE, "gemm_prepared_scatter: the weight must be prepared from its [K, N] form");
    if (chunks < 0 || (chunks > 0 && (chunk_k < 1 || (chunk_k % 4) != 0 || (int64_t)chunks * chunk_k != W->K)))
        return fail(AXB_ERR_INVALID_SHAPE, "gemm_prepared_scatter: chunks * chunk_k must equal the weight's K, chunk_k a multiple of 4");
    if (M < 0) return fail(AXB_ERR_INVALID_SHAPE, "gemm_prepared_scatter: negative dimension");
    if (M == 0) return AXB_OK;
    if (!A || !C || (n_more > 0 && !C_more)) return fail(AXB_ERR_NULL_ARG, "gemm_prepared_scatter: NULL operand");
    if (n_more < 0 || n_more > TC_MAX_EXTRA) return fail(AXB_ERR_INVALID_SHAPE, "gemm_prepared_scatter: at most %d extra destinations", TC_MAX_EXTRA);
    for (int i = 0; i < n_more; ++i)
        if (!C_more[i]) return fail(AXB_ERR_NULL_ARG, "gemm_prepared_scatter: NULL destination %d", i);
    if (act < AXB_ACT_NONE || act > AXB_ACT_GELU) return fail(AXB_ERR_INVALID_SHAPE, "gemm_prepared_scatter: unknown activation %d", act);
    if (M > INT32_MAX) return fail(AXB_ERR_INVALID_SHAPE, "gemm_prepared_scatter: dimension exceeds 2^31-1");
    int st = ensure_ready();
    if (st) return st;
    if (W->device != cur().device) return fail(AXB_ERR_BACKEND, "gemm_prepared_scatter: the weight was prepared on device %d", W->device);
    if (W->mode != cur().fp32_mode)
        return fail(AXB_ERR_BACKEND, "gemm_prepared_scatter: the weight was prepared in fp32 mode %d, the engine is in mode %d", W->mode, cur().fp32_mode);
    return gemm_tc_f32(A, W->src, bias, C, M, W->N, W->K, 0, 0, alpha, beta, act, C_more, n_more, chunks > 0 ? chunk_k : 0,
                       chunks > 0 ? M * chunk_k : 0, nullptr, nullptr, &W->op);
}

// C_host = A_host . B_host with the transfers pipelined against the tensor-core work: B goes up first and is
// split once; A goes up in row chunks on a copy stream, each chunk is split and multiplied as soon as it has
// landed, and its rows of C go back on a second copy stream while the next chunk is in flight.  Row chunks of
// a GEMM are independent, so the result is bit-identical to one call over the whole matrix.
extern "C" int axb_gemm_host(const float *A, const float *B, float *C, int64_t M, int64_t N, int64_t K,
                             int64_t row_chunk)
{
    if (M == 0 || N == 0) return AXB_OK;
    if (!A || !B || !C) return fail(AXB_ERR_NULL_ARG, "gemm_host: NULL");
    if (M < 0 || N < 0 || K <= 0 || row_chunk < 0) return fail(AXB_ERR_INVALID_SHAPE, "gemm_host: bad shape");
    if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return fail(AXB_ERR_INVALID_SHAPE, "gemm_host: dimension exceeds 2^31-1");
    int st = ensure_ready();
    if (st) return st;
    if (!cur().hp_in) {
        cudaError_t e = cudaStreamCreateWithFlags(&cur().hp_in, cudaStreamNonBlocking);
        if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&cur().hp_out, cudaStreamNonBlocking);
        for (auto &ev : cur().hp_ev)
            if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
        if (e != cudaSuccess) return cuda_fail("gemm_host: streams", e);
    }
    // the route follows the whole problem, as in axb_gemm (M <= 32 is the bandwidth-bound route), so that a
    // short last chunk is computed exactly as its rows would be in one call over the whole matrix
    const bool tensor_path = M > 32;
    {
        // a problem small enough for axb_gemm to split K over several CTAs is not worth a pipeline, and its row
        // blocks would add their partial sums in another order: upload, one axb_gemm, download
        int sm, kd;
        TcProducts pr;
        fp32_mode_plan(sm, kd, pr);
        if (tensor_path && gemm_tc_splits_k(kd, pr, M, N, K, cur().sm_count)) {
            const size_t ab = round_up((size_t)M * K * 4, 1024), bb = round_up((size_t)K * N * 4, 1024), cb = (size_t)M * N * 4;
            if (ab + bb + cb > cur().hp_bytes) {
                cudaDeviceSynchronize();
                if (cur().hp_buf) cudaFree(cur().hp_buf);
                cur().hp_buf = nullptr; cur().hp_bytes = 0;
                cudaError_t e = cudaMalloc(&cur().hp_buf, ab + bb + cb);
                if (e != cudaSuccess) return fail(AXB_ERR_ALLOC, "gemm_host: staging of %zu bytes: %s", ab + bb + cb, cudaGetErrorString(e));
                cur().hp_bytes = ab + bb + cb;
            }
            float *dA = (float *)cur().hp_buf, *dB = (float *)((char *)cur().hp_buf + ab), *dC = (float *)((char *)cur().hp_buf + ab + bb);
            cudaMemcpyAsync(dA, A, (size_t)M * K * 4, cudaMemcpyHostToDevice, cur().stream);
            cudaMemcpyAsync(dB, B, (size_t)K * N * 4, cudaMemcpyHostToDevice, cur().stream);
            st = axb_gemm(dA, dB, dC, M, N, K);
            if (st) { cudaStreamSynchronize(cur().stream); return st; }
            cudaMemcpyAsync(C, dC, cb, cudaMemcpyDeviceToHost, cur().stream);
            cudaError_t ce = cudaStreamSynchronize(cur().stream);
            return ce == cudaSuccess ? AXB_OK : cuda_fail("gemm_host", ce);
        }
    }
    // default: about 16 chunks (a short tail after the last upload), whole 128-row tiles, 256..1024 rows
    int64_t rc = row_chunk;
    if (rc <= 0) {
        rc = (M / 16 + 127) / 128 * 128;
        if (rc < 256) rc = 256;
        if (rc > 1024) rc = 1024;
    }
    if (rc > M) rc = M;
    const int64_t chunks = (M + rc - 1) / rc;
    // staging: B, two A chunks, two C chunks
    const size_t b_bytes = round_up((size_t)K * N * 4, 1024), a_bytes = round_up((size_t)rc * K * 4, 1024),
                 c_bytes = round_up((size_t)rc * N * 4, 1024);
    const size_t need = b_bytes + 2 * a_bytes + 2 * c_bytes;
    if (need > cur().hp_bytes) {
        cudaDeviceSynchronize();
        if (cur().hp_buf) cudaFree(cur().hp_buf);
        cur().hp_buf = nullptr; cur().hp_bytes = 0;
        cudaError_t e = cudaMalloc(&cur().hp_buf, need);
        if (e != cudaSuccess) return fail(AXB_ERR_ALLOC, "gemm_host: staging of %zu bytes: %s", need, cudaGetErrorString(e));
        cur().hp_bytes = need;
    }
    char *base = (char *)cur().hp_buf;
    float *dB = (float *)base;
    float *dA[2] = { (float *)(base + b_bytes), (float *)(base + b_bytes + a_bytes) };
    float *dC[2] = { (float *)(base + b_bytes + 2 * a_bytes), (float *)(base + b_bytes + 2 * a_bytes + c_bytes) };
    cudaEvent_t ev_b = cur().hp_ev[0], *ev_a = &cur().hp_ev[1], *ev_a_free = &cur().hp_ev[3], *ev_c = &cur().hp_ev[5], *ev_c_free = &cur().hp_ev[7];

    int split_mode, kind;
    TcProducts prod;
    fp32_mode_plan(split_mode, kind, prod);
    SplitOperand sb = plan_split(split_mode, N, K), sa = plan_split(split_mode, rc, K);
    TcOperand opb;
    Carver carve{ nullptr };
    if (tensor_path) {
        st = ensure_ws(sa.total() + sb.total());
        if (st) return st;
        carve.p = (char *)cur().ws;
    }
    // everything the engine's stream did before this call precedes the copies
    cudaEventRecord(ev_b, cur().stream);
    cudaStreamWaitEvent(cur().hp_in, ev_b, 0);
    cudaStreamWaitEvent(cur().hp_out, ev_b, 0);

    cudaMemcpyAsync(dB, B, (size_t)K * N * 4, cudaMemcpyHostToDevice, cur().hp_in);
    cudaEventRecord(ev_b, cur().hp_in);
    cudaStreamWaitEvent(cur().stream, ev_b, 0);
    // on a failure half way: let the copies already queued finish before the caller may free its buffers
    auto bail = [&](int status) {
        cudaStreamSynchronize(cur().hp_in);
        cudaStreamSynchronize(cur().hp_out);
        return status;
    };
    int e = 0;
    if (tensor_path) {
        e = run_split(sb, dB, N, true, carve, opb);
        if (e) return bail(cuda_fail("gemm_host: split B", e));
    }
    const size_t a_plane_off = carve.off;
    for (int64_t i = 0; i < chunks; ++i) {
        const int slot = (int)(i & 1);
        const int64_t r0 = i * rc, rows = (M - r0 < rc) ? M - r0 : rc;
        if (i >= 2) cudaStreamWaitEvent(cur().hp_in, ev_a_free[slot], 0);
        cudaMemcpyAsync(dA[slot], A + r0 * K, (size_t)rows * K * 4, cudaMemcpyHostToDevice, cur().hp_in);
        cudaEventRecord(ev_a[slot], cur().hp_in);
        cudaStreamWaitEvent(cur().stream, ev_a[slot], 0);
        if (i >= 2) cudaStreamWaitEvent(cur().stream, ev_c_free[slot], 0);
        if (tensor_path) {
            carve.off = a_plane_off;
            TcOperand opa;
            SplitOperand sai = plan_split(split_mode, rows, K);
            e = run_split(sai, dA[slot], K, false, carve, opa);
            if (e) return bail(cuda_fail("gemm_host: split A", e));
            cudaEventRecord(ev_a_free[slot], cur().stream);
            TcEpilogue ep;
            ep.alpha = 1.0f; ep.beta = 0.0f; ep.bias = nullptr; ep.colscale = nullptr; ep.act = ACT_NONE;
            ep.out_mode = OUT_F32; ep.C = dC[slot]; ep.acc_out = nullptr; ep.ldc = N; ep.n_extra = 0;
            e = launch_gemm_tc(kind, opa, opb, prod, rows, N, K, ep, cur().err_word, cur().sm_count, cur().stream);
            cur().launches++;
            if (e) return bail(cuda_fail("gemm_host: tcgen05 gemm", e));
        } else {
            st = axb_gemm(dA[slot], dB, dC[slot], rows, N, K);   // M <= 32: the skinny route
            if (st) return bail(st);
            cudaEventRecord(ev_a_free[slot], cur().stream);
        }
        cudaEventRecord(ev_c[slot], cur().stream);
        cudaStreamWaitEvent(cur().hp_out, ev_c[slot], 0);
        cudaMemcpyAsync(C + r0 * N, dC[slot], (size_t)rows * N * 4, cudaMemcpyDeviceToHost, cur().hp_out);
        cudaEventRecord(ev_c_free[slot], cur().hp_out);
    }
    cudaError_t ce = cudaStreamSynchronize(cur().hp_out);
    if (ce == cudaSuccess) ce = cudaStreamSynchronize(cur().hp_in);
    if (ce != cudaSuccess) return cuda_fail("gemm_host", ce);
    return AXB_OK;
}

// ------------------------------------------------------------------ elementwise

extern "C" int axb_bias_add(const float *in, const float *bias, int axis, float *out, int64_t M, int64_t N)
{
    if (!in || !bias || !out) return fail(AXB_ERR_NULL_ARG, "bias_add: NULL");
    if (axis != 0 && axis != 1) return fail(AXB_ERR_INVALID_AXIS, "bias_add: axis %d of a 2-D tensor", axis);
    if (M < 0 || N < 0) return fail(AXB_ERR_INVALID_SHAPE, "bias_add: negative dimension");
    int st = ensure_ready();
    if (st) return st;
    int e = launch_bias_add(in, bias, axis, out, M, N, cur().sm_count, cur().stream);
    cur().launches++;
    return e ? cuda_fail("bias_add", e) : AXB_OK;
}

extern "C" int axb_bias_add_nd(const float *in, const float *bias, float *out, int64_t outer, int64_t axis_len,
                               int64_t inner)
{
    if (!in || !bias || !out) return fail(AXB_ERR_NULL_ARG, "bias_add: NULL");
    if (outer < 0 || axis_len < 0 || inner < 0) return fail(AXB_ERR_INVALID_SHAPE, "bias_add: negative dimension");
    int st = ensure_ready();
    if (st) return st;
    // the broadcast axis last: a [outer, axis_len] matrix with one value per column; otherwise
    // [outer*axis_len, inner] with one value per row, repeating every axis_len rows
    int e = inner == 1 ? launch_bias_add(in, bias, 1, out, outer, axis_len, cur().sm_count, cur().stream)
                       : launch_bias_add(in, bias, 0, out, outer * axis_len, inner, cur().sm_count, cur().stream, axis_len);
    cur().launches++;
    return e ? cuda_fail("bias_add", e) : AXB_OK;
}

extern "C" int axb_relu(const float *in, float *out, int64_t n)
{
    if (!in || !out) return fail(AXB_ERR_NULL_ARG, "relu: NULL");
    int st = ensure_ready();
    if (st) return st;
    int e = launch_unary(0, in, out, n, cur().sm_count, cur().stream);
    cur().launches++;
    return e ? cuda_fail("relu", e) : AXB_OK;
}

extern "C" int axb_gelu(const float *in, float *out, int64_t n)
{
    if (!in || !out) return fail(AXB_ERR_NULL_ARG, "gelu: NULL");
    int st = ensure_ready();
    if (st) return st;
    int e = launch_unary(1, in, out, n, cur().sm_count, cur().stream);
    cur().launches++;
    return e ? cuda_fail("gelu", e) : AXB_OK;
}

// -------------------------------------------------------------------- quantised

extern "C" int axb_qgemm_w8a32(const float *a, const int8_t *q, const float *scales, float *out, int64_t M,
                               int64_t N, int64_t K)
{
    return axb_qdense_w8a32(a, q, scales, nullptr, AXB_ACT_NONE, out, M, N, K);
}

extern "C" int axb_qgemm_w8a32_qw(const float *a, const axb_qweight_t *qw, float *out, int64_t M)
{
    if (!a || !qw || !out || !qw->data || !qw->scales) return fail(AXB_ERR_NULL_ARG, "qgemm_w8a32: NULL");
    return axb_qdense_w8a32(a, qw->data, qw->scales, nullptr, AXB_ACT_NONE, out, M, qw->N, qw->K);
}

extern "C" int axb_qdense_w8a32(const float *a, const int8_t *q, const float *scales, const float *bias, int act,
                                float *out, int64_t M, int64_t N, int64_t K)
{
    if (!a || !q || !scales || !out) return fail(AXB_ERR_NULL_ARG, "qgemm_w8a32: NULL");
    if (act != AXB_ACT_NONE && act != AXB_ACT_RELU && act != AXB_ACT_GELU) return fail(AXB_ERR_INVALID_SHAPE, "qdense_w8a32: unknown activation %d", act);
    if (M < 0 || N <= 0 || K <= 0) return fail(AXB_ERR_INVALID_SHAPE, "qgemm_w8a32: bad shape");
    if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return fail(AXB_ERR_INVALID_SHAPE, "qgemm_w8a32: dimension exceeds 2^31-1");
    int st = ensure_ready();
    if (st) return st;
    if (M == 0) return AXB_OK;
    // a single activation row too once the layer is large: the fp32-FMA GEMV tops out at 3.7 TB/s (instruction issue),
    // the tensor-core kernel — one launch up to four rows, it makes the activations' digits itself — streams faster
    // from 2^24 weights on (measured: 16384 x 4096 13.6 us against 18.0, 8192 x 4096 9.3 against 13.0, 4096 x 4096
    // 8.0 against 8.8)
    const bool tc_route = M >= 2 ? N * K >= (1 << 20) : N * K >= (1 << 24);
    if (tc_route && qskinny_tc_applicable(M, N, K, a, q)) {
        // skinny activations as four int8 digit planes, weights streamed once into kind::i8 MMAs
        st = ensure_ws(qskinny_tc_workspace_bytes(M, K));
        if (st) return st;
        mark(0);
        mark(1);
        // (a call of up to 4 rows is one kernel that lets its successor start early: as on the fp32 skinny route, the
        // successor may only do so when this call's output is not what it streams as weights)
        const char *w_lo = reinterpret_cast<const char *>(q), *w_hi = w_lo + (size_t)N * K;
        const int pdl = !(cur().chain_lo && w_lo < cur().chain_hi && cur().chain_lo < w_hi);
        cur().chain_lo = reinterpret_cast<const char *>(out);
        cur().chain_hi = cur().chain_lo + (size_t)M * N * sizeof(float);
        int e = launch_qskinny_tc(a, q, scales, bias, act, out, M, N, K, cur().ws, cur().err_word, cur().sm_count, cur().stream, pdl);
        mark(2);
        cur().launches += M <= 4 ? 1 : 2;
        return e ? cuda_fail("w8a32 skinny", e) : AXB_OK;
    }
    if (qgemv_w8a32_applicable(M, N, K, q) && (reinterpret_cast<uintptr_t>(a) & 15) == 0) {
        // skinny activations: stream the int8 rows once, fp32 FMA (the reference's own arithmetic)
        mark(0);
        mark(1);
        int e = launch_qgemv_w8a32(a, q, scales, bias, act, out, M, N, K, cur().sm_count, cur().stream);
        mark(2);
        cur().launches++;
        return e ? cuda_fail("w8a32 gemv", e) : AXB_OK;
    }
    if (K % 16 == 0 && K <= 65536 && 4 * M <= INT32_MAX &&
        ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(q)) & 15) == 0) {
        // activations as four int8 digit rows per row, interleaved [M][4][K] = the B operand of one int8 GEMM whose A
        // operand is the weights as they are: the thread that holds accumulator row n has the four digit sums of an
        // output (m, n) side by side, recombines them with 64-bit integers (exact), applies scale, bias and activation
        // and stores out[m][n] — no s32 intermediate, no recombination pass
        const size_t dig_bytes = (size_t)4 * M * K;
        st = ensure_ws(round_up((size_t)M * sizeof(float), 1024) + round_up(dig_bytes, 1024) + kSplitScratch);
        if (st) return st;
        Carver carve{ (char *)cur().ws };
        const TcSplitK sk = take_splitk(carve);
        float *inv_s = (float *)carve.take((size_t)M * sizeof(float));
        int8_t *digits = (int8_t *)carve.take(dig_bytes);
        mark(0);
        int e = launch_qx_digits(a, M, K, 0, digits, inv_s, cur().stream);
        cur().launches++;
        if (e) return cuda_fail("w8a32 digits", e);
        TcOperand opa, opb;
        opa.nplanes = opb.nplanes = 1;
        opa.plane[0] = q; opa.rows = N; opa.pitch_elems = K;
        opb.plane[0] = digits; opb.rows = 4 * M; opb.pitch_elems = K;
        TcProducts prod;
        memset(&prod, 0, sizeof prod);
        prod.n = 1;
        TcEpilogue ep;
        ep.n_extra = 0;
        ep.alpha = 1.0f; ep.beta = 0.0f; ep.bias = bias; ep.colscale = scales; ep.act = act;
        ep.out_mode = OUT_DIGITS_T; ep.C = out; ep.acc_out = nullptr; ep.ldc = N;
        ep.dg_inv_s = inv_s; ep.dg_rows = (int)M;
        mark(1);
        e = launch_gemm_tc(KIND_I8, opa, opb, prod, N, 4 * M, K, ep, cur().err_word, cur().sm_count, cur().stream, &sk);
        mark(2);
        cur().launches++;
        return e ? cuda_fail("w8a32 digit gemm", e) : AXB_OK;
    }
    // activations: bf16 hi/mid/lo (exact to 24 bits); weights: int8 widened to bf16 (exact)
    const int amode = cur().fp32_mode == AXB_FP32_BF16 ? SPLIT_BF16X1 : SPLIT_BF16X3;
    const SplitOperand sa = plan_split(amode, M, K);
    const int64_t wpitch = (int64_t)round_up((size_t)K, 16);
    const size_t wbytes = (size_t)N * wpitch * 2;
    st = ensure_ws(sa.total() + round_up(wbytes, 1024));
    if (st) return st;
    Carver carve{ (char *)cur().ws };
    TcOperand opa, opb;
    mark(0);
    int e = run_split(sa, a, K, false, carve, opa);
    if (e) return cuda_fail("split activations", e);
    void *wplane = carve.take(wbytes);
    e = widen_i8_to_bf16(q, N, K, wplane, wpitch, cur().sm_count, cur().stream);
    cur().launches++;
    if (e) return cuda_fail("widen weights", e);
    opb.nplanes = 1; opb.plane[0] = wplane; opb.rows = N; opb.pitch_elems = wpitch;
    TcProducts prod;
    memset(&prod, 0, sizeof prod);
    prod.n = opa.nplanes;
    for (int i = 0; i < prod.n; ++i) { prod.a[i] = (int8_t)(prod.n - 1 - i); prod.b[i] = 0; }  // smallest plane first
    prod.chunk_k = prod.n > 1 ? cur().chunk_bf16 : 0;
    TcEpilogue ep;
    ep.n_extra = 0;
    ep.alpha = 1.0f; ep.beta = 0.0f; ep.bias = bias; ep.colscale = scales; ep.act = act;
    ep.out_mode = OUT_F32; ep.C = out; ep.acc_out = nullptr; ep.ldc = N;
    mark(1);
    e = launch_gemm_tc(KIND_BF16, opa, opb, prod, M, N, K, ep, cur().err_word, cur().sm_count, cur().stream);
    mark(2);
    cur().launches++;
    return e ? cuda_fail("w8a32 gemm", e) : AXB_OK;
}

extern "C" int axb_qgemm_w8a8(const int8_t *a_q, float a_scale, const int8_t *b_q, const float *b_scales,
                              float out_scale, int8_t *out_q, int32_t *acc_out, int64_t M, int64_t N, int64_t K)
{
    if (!a_q || !b_q) return fail(AXB_ERR_NULL_ARG, "qgemm_w8a8: NULL operand");
    if (out_q && !b_scales) return fail(AXB_ERR_NULL_ARG, "qgemm_w8a8: requantised output needs b_scales");
    if (!out_q && !acc_out) return fail(AXB_ERR_NULL_ARG, "qgemm_w8a8: no output requested");
    if (M < 0 || N <= 0 || K <= 0) return fail(AXB_ERR_INVALID_SHAPE, "qgemm_w8a8: bad shape");
    if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return fail(AXB_ERR_INVALID_SHAPE, "qgemm_w8a8: dimension exceeds 2^31-1");
    if (out_q && !(out_scale > 0.0f)) return fail(AXB_ERR_INVALID_SHAPE, "qgemm_w8a8: out_scale must be positive");
    int st = ensure_ready();
    if (st) return st;
    if (M == 0) return AXB_OK;
    // TMA needs 16-byte aligned bases and row pitches: operands that are not are re-pitched first
    const bool a_direct = (K % 16 == 0) && ((reinterpret_cast<uintptr_t>(a_q) & 15) == 0);
    const bool b_direct = (K % 16 == 0) && ((reinterpret_cast<uintptr_t>(b_q) & 15) == 0);
    const int64_t pitch = (int64_t)round_up((size_t)K, 16);
    size_t need = kSplitScratch;
    if (!a_direct) need += round_up((size_t)M * pitch, 1024);
    if (!b_direct) need += round_up((size_t)N * pitch, 1024);
    st = ensure_ws(need);
    if (st) return st;
    Carver carve{ (char *)cur().ws };
    const TcSplitK sk = take_splitk(carve);
    int e;
    mark(0);
    TcOperand opa, opb;
    opa.nplanes = opb.nplanes = 1;
    opa.rows = M; opb.rows = N;
    if (a_direct) { opa.plane[0] = a_q; opa.pitch_elems = K; }
    else {
        int8_t *p = (int8_t *)carve.take((size_t)M * pitch);
        e = repitch_i8(a_q, M, K, p, pitch, cur().sm_count, cur().stream);
        cur().launches++;
        if (e) return cuda_fail("repitch A", e);
        opa.plane[0] = p; opa.pitch_elems = pitch;
    }
    if (b_direct) { opb.plane[0] = b_q; opb.pitch_elems = K; }
    else {
        int8_t *p = (int8_t *)carve.take((size_t)N * pitch);
        e = repitch_i8(b_q, N, K, p, pitch, cur().sm_count, cur().stream);
        cur().launches++;
        if (e) return cuda_fail("repitch B", e);
        opb.plane[0] = p; opb.pitch_elems = pitch;
    }
    TcProducts prod;
    memset(&prod, 0, sizeof prod);
    prod.n = 1;
    TcEpilogue ep;
    ep.n_extra = 0;
    // the requantisation multiplier (a_scale * b_scales[n]) / out_scale is formed in the epilogue, rounding for rounding
    ep.alpha = 1.0f; ep.beta = 0.0f; ep.bias = nullptr; ep.colscale = b_scales; ep.act = ACT_NONE;
    ep.rq_a_scale = a_scale; ep.rq_out_scale = out_scale;
    ep.out_mode = out_q ? OUT_I8_REQUANT : OUT_S32_ONLY; ep.C = out_q; ep.acc_out = acc_out; ep.ldc = N;
    mark(1);
    e = launch_gemm_tc(KIND_I8, opa, opb, prod, M, N, K, ep, cur().err_word, cur().sm_count, cur().stream, &sk);
    mark(2);
    cur().launches++;
    return e ? cuda_fail("w8a8 gemm", e) : AXB_OK;
}

extern "C" int axb_quantize_rows(const float *w, int64_t N, int64_t K, int8_t *q, float *scales)
{
    if (!w || !q || !scales) return fail(AXB_ERR_NULL_ARG, "quantize_rows: NULL");
    if (N <= 0 || K <= 0) return fail(AXB_ERR_INVALID_SHAPE, "quantize_rows: bad shape");
    int st = ensure_ready();
    if (st) return st;
    int e = quantize_rows(w, N, K, q, scales, cur().stream);
    cur().launches++;
    return e ? cuda_fail("quantize_rows", e) : AXB_OK;
}

// -------------------------------------------------------------------- attention

extern "C" int axb_sdpa_fwd(const float *Q, const float *K, const float *V, float *out, float *L, int64_t BH,
                            int64_t S, int64_t dk, float scale, int causal, float *P_save)
{
    if (!Q || !K || !V || !out) return fail(AXB_ERR_NULL_ARG, "sdpa_fwd: NULL");
    if (BH < 0 || S < 0 || dk <= 0) return fail(AXB_ERR_INVALID_SHAPE, "sdpa_fwd: bad shape");
    if (dk > 128) return fail(AXB_ERR_NOT_IMPLEMENTED, "sdpa_fwd: head dim %lld > 128", (long long)dk);
    if (BH > 65535 || S > (1 << 24)) return fail(AXB_ERR_INVALID_SHAPE, "sdpa_fwd: BH > 65535 or S too large");
    int st = ensure_ready();
    if (st) return st;
    if (BH == 0 || S == 0) return AXB_OK;
    // the probabilities a caller wants kept are written after the fused pass from its log-sum-exp: O and L never
    // depend on them, and a caller that ignores the status (src/core/attention.c:335-342) still gets its output
    if (P_save && !L) {
        st = ensure_ws((size_t)BH * S * sizeof(float));
        if (st) return st;
        L = (float *)cur().ws;
    }
    mark(0);
    mark(1);
    int e;
    if (sdpa_tc_applicable(Q, K, V, BH, S, dk, scale)) e = launch_sdpa_tc(Q, K, V, out, L, BH, S, dk, scale, causal, cur().err_word, cur().stream);
    else e = launch_sdpa_fwd(Q, K, V, out, L, BH, S, dk, scale, causal, cur().stream);
    mark(2);
    cur().launches++;
    if (e) return cuda_fail("sdpa_fwd", e);
    if (P_save) {
        e = launch_sdpa_probs(Q, K, L, P_save, BH, S, dk, scale, causal, cur().stream);
        cur().launches++;
        if (e) return cuda_fail("sdpa_fwd: saved probabilities", e);
    }
    return AXB_OK;
}

extern "C" int axb_sdpa_bwd(const float *Q, const float *K, const float *V, const float *O, const float *dO,
                            const float *L, float *dQ, float *dK, float *dV, int64_t BH, int64_t S, int64_t dk,
                            float scale, int causal, const float *P_saved)
{
    if (!Q || !K || !V || !O || !dO || !L || !dQ || !dK || !dV) return fail(AXB_ERR_NULL_ARG, "sdpa_bwd: NULL");
    (void)P_saved;   // scores are always recomputed from Q, K and L: a saved P would only add S*S traffic
    if (BH < 0 || S < 0 || dk <= 0) return fail(AXB_ERR_INVALID_SHAPE, "sdpa_bwd: bad shape");
    if (dk > 128) return fail(AXB_ERR_NOT_IMPLEMENTED, "sdpa_bwd: head dim %lld > 128", (long long)dk);
    if (BH > 65535 || S > (1 << 24)) return fail(AXB_ERR_INVALID_SHAPE, "sdpa_bwd: BH > 65535 or S too large");
    int st = ensure_ready();
    if (st) return st;
    if (BH == 0 || S == 0) return AXB_OK;
    st = ensure_ws(sdpa_bwd_workspace_bytes(BH, S));
    if (st) return st;
    mark(0);
    mark(1);
    int n_launched = 0;
    int e = launch_sdpa_bwd(Q, K, V, O, dO, L, dQ, dK, dV, BH, S, dk, scale, causal, (float *)cur().ws, cur().sm_count,
                            cur().err_word, cur().stream, &n_launched);
    mark(2);
    cur().launches += n_launched;
    return e ? cuda_fail("sdpa_bwd", e) : AXB_OK;
}

// ---------------------------------------------------------------- convolution

// `batch` samples [C_in, H, W] back to back -> out [batch][C_out][out_h * out_w]
static int conv_gemm_any(const float *weight, const float *input, int64_t batch, int64_t C_out, int64_t C_in, int64_t H, int64_t W,
                         int kh, int kw, int sh, int sw, int ph, int pw, int64_t out_h, int64_t out_w, float *out)
{
    if (batch == 0) return AXB_OK;   // nothing to read or write (the pointers of an empty batch may be NULL)
    if (!weight || !input || !out) return fail(AXB_ERR_NULL_ARG, "conv_gemm: NULL");
    if (batch < 0 || C_out <= 0 || C_in <= 0 || H <= 0 || W <= 0 || kh <= 0 || kw <= 0 || sh <= 0 || sw <= 0 || ph < 0 || pw < 0 ||
        out_h < 0 || out_w < 0)
        return fail(AXB_ERR_INVALID_SHAPE, "conv_gemm: bad geometry");
    const int64_t K = C_in * kh * kw, P = out_h * out_w;
    if (C_out > INT32_MAX || K > INT32_MAX || P > INT32_MAX) return fail(AXB_ERR_INVALID_SHAPE, "conv_gemm: dimension exceeds 2^31-1");
    int st = ensure_ready();
    if (st) return st;
    if (P == 0) return AXB_OK;
    // out[C_out, P] = weight[C_out, K] . im2col(input)[K, P]: the weight rows are the A operand, the image patches
    // are gathered straight into the planes of the B operand
    int split_mode, kind;
    TcProducts prod;
    fp32_mode_plan(split_mode, kind, prod);
    TcConv cv;
    cv.C = C_in; cv.H = H; cv.W = W; cv.kh = kh; cv.kw = kw; cv.pad_h = ph; cv.pad_w = pw; cv.out_h = out_h; cv.out_w = out_w;
    cv.batch = batch;
    if (gemm_tc_conv_applicable(cv, sh, sw, out) && batch * H * W <= INT32_MAX) {
        // Stride 1: implicit GEMM.  The image is transposed once into channel-innermost planes (the same pre-pass
        // that transposes a [K, N] operand), the filter into [C_out][tap][channel] planes, and the GEMM's producer
        // reads shifted windows of the image planes — the patch matrix, kh * kw times the image, never exists.
        const int cpad = gemm_tc_conv_channel_pad(kind);
        const int64_t c_pad = (C_in + cpad - 1) / cpad * cpad, taps = (int64_t)kh * kw;
        const SplitOperand si = plan_split(split_mode, batch * H * W, C_in), sw_ = plan_split(split_mode, C_out, taps * c_pad);
        st = ensure_ws(si.total() + sw_.total() + kSplitScratch);
        if (st) return st;
        Carver carve{ (char *)cur().ws };
        const TcSplitK sk = take_splitk(carve);
        TcOperand opw, opi;
        mark(0);
        void *ip[3] = { nullptr, nullptr, nullptr }, *wp[3] = { nullptr, nullptr, nullptr };
        opi.nplanes = opw.nplanes = split_num_planes(split_mode);
        for (int i = 0; i < opi.nplanes; ++i) opi.plane[i] = ip[i] = carve.take(si.plane_bytes);
        for (int i = 0; i < opw.nplanes; ++i) opw.plane[i] = wp[i] = carve.take(sw_.plane_bytes);
        opi.rows = batch * H * W;
        opi.pitch_elems = si.pitch;
        opw.rows = C_out;
        opw.pitch_elems = sw_.pitch;
        int e = split_conv_operands(split_mode, input, batch, C_in, H * W, ip, si.pitch, weight, C_out, (int)taps, (int)c_pad, wp, sw_.pitch,
                                    cur().sm_count, cur().stream);
        cur().launches++;
        if (e) return cuda_fail("conv_gemm: operand planes", e);
        TcEpilogue ep;
        ep.alpha = 1.0f; ep.beta = 0.0f; ep.bias = nullptr; ep.colscale = nullptr; ep.act = ACT_NONE;
        ep.out_mode = OUT_F32; ep.C = out; ep.acc_out = nullptr; ep.ldc = P; ep.n_extra = 0;
        mark(1);
        e = launch_gemm_tc_conv(kind, opw, opi, prod, C_out, cv, ep, cur().err_word, cur().sm_count, cur().stream, &sk);
        mark(2);
        cur().launches++;
        return e ? cuda_fail("conv_gemm", e) : AXB_OK;
    }
    if (batch > 1) {
        // the gathered form (strided layers, output widths that are not a multiple of 4) takes the samples one by one
        for (int64_t n = 0; n < batch; ++n) {
            st = conv_gemm_any(weight, input + n * C_in * H * W, 1, C_out, C_in, H, W, kh, kw, sh, sw, ph, pw, out_h, out_w,
                               out + n * C_out * P);
            if (st) return st;
        }
        return AXB_OK;
    }
    const SplitOperand sa = plan_split(split_mode, C_out, K), sb = plan_split(split_mode, P, K);
    st = ensure_ws(sa.total() + sb.total() + kSplitScratch);
    if (st) return st;
    Carver carve{ (char *)cur().ws };
    const TcSplitK sk = take_splitk(carve);
    TcOperand opa, opb;
    mark(0);
    int e = run_split(sa, weight, K, false, carve, opa);
    if (e) return cuda_fail("conv_gemm: split weight", e);
    void *planes[3] = { nullptr, nullptr, nullptr };
    opb.nplanes = split_num_planes(split_mode);
    for (int i = 0; i < opb.nplanes; ++i) {
        planes[i] = carve.take(sb.plane_bytes);
        opb.plane[i] = planes[i];
    }
    opb.rows = P;
    opb.pitch_elems = sb.pitch;
    e = split_im2col(split_mode, input, C_in, H, W, kh, kw, sh, sw, ph, pw, out_h, out_w, planes, sb.pitch, cur().sm_count, cur().stream);
    cur().launches++;
    if (e) return cuda_fail("conv_gemm: im2col split", e);
    TcEpilogue ep;
    ep.alpha = 1.0f; ep.beta = 0.0f; ep.bias = nullptr; ep.colscale = nullptr; ep.act = ACT_NONE;
    ep.out_mode = OUT_F32; ep.C = out; ep.acc_out = nullptr; ep.ldc = P; ep.n_extra = 0;
    mark(1);
    e = launch_gemm_tc(kind, opa, opb, prod, C_out, P, K, ep, cur().err_word, cur().sm_count, cur().stream, &sk);
    mark(2);
    cur().launches++;
    return e ? cuda_fail("conv_gemm", e) : AXB_OK;
}

extern "C" int axb_conv_gemm(const float *weight, const float *input, int64_t C_out, int64_t C_in, int64_t H, int64_t W,
                             int kh, int kw, int sh, int sw, int ph, int pw, int64_t out_h, int64_t out_w, float *out)
{
    return conv_gemm_any(weight, input, 1, C_out, C_in, H, W, kh, kw, sh, sw, ph, pw, out_h, out_w, out);
}

extern "C" int axb_conv_gemm_batched(const float *weight, const float *input, int64_t batch, int64_t C_out, int64_t C_in, int64_t H,
                                     int64_t W, int kh, int kw, int sh, int sw, int ph, int pw, int64_t out_h, int64_t out_w,
                                     float *out)
{
    return conv_gemm_any(weight, input, batch, C_out, C_in, H, W, kh, kw, sh, sw, ph, pw, out_h, out_w, out);
}

// ------------------------------------------------------------------ KV cache

extern "C" int axb_kv_cache_append(float *K_cache, float *V_cache, const float *new_K, const float *new_V, int64_t BH,
                                   int64_t cur_len, int64_t max_seq, int64_t dk)
{
    if (!K_cache || !V_cache || !new_K || !new_V) return fail(AXB_ERR_NULL_ARG, "kv_cache_append: NULL");
    if (BH < 0 || dk <= 0 || max_seq <= 0 || cur_len < 0) return fail(AXB_ERR_INVALID_SHAPE, "kv_cache_append: bad shape");
    if (cur_len >= max_seq) return fail(AXB_ERR_INVALID_SHAPE, "kv_cache_append: cache full (%lld of %lld)", (long long)cur_len, (long long)max_seq);
    int st = ensure_ready();
    if (st) return st;
    if (BH == 0) return AXB_OK;
    // row cur_len of every head: [BH] rows of dk floats, max_seq*dk apart in the cache
    const size_t w = (size_t)dk * sizeof(float), pitch = (size_t)max_seq * w;
    cudaError_t e = cudaMemcpy2DAsync(K_cache + cur_len * dk, pitch, new_K, w, w, (size_t)BH, cudaMemcpyDeviceToDevice, cur().stream);
    if (e == cudaSuccess)
        e = cudaMemcpy2DAsync(V_cache + cur_len * dk, pitch, new_V, w, w, (size_t)BH, cudaMemcpyDeviceToDevice, cur().stream);
    return e == cudaSuccess ? AXB_OK : cuda_fail("kv_cache_append", e);
}

extern "C" int axb_kv_cache_attend(const float *K_cache, const float *V_cache, const float *Q_new, float *out, int64_t BH,
                                   int64_t cur_len, int64_t max_seq, int64_t dk, float scale)
{
    if (!K_cache || !V_cache || !Q_new || !out) return fail(AXB_ERR_NULL_ARG, "kv_cache_attend: NULL");
    if (BH < 0 || dk <= 0 || max_seq <= 0 || cur_len < 0 || cur_len > max_seq)
        return fail(AXB_ERR_INVALID_SHAPE, "kv_cache_attend: bad shape");
    if (dk > 128) return fail(AXB_ERR_NOT_IMPLEMENTED, "kv_cache_attend: head dim %lld > 128", (long long)dk);
    if (cur_len > INT32_MAX || BH > INT32_MAX) return fail(AXB_ERR_INVALID_SHAPE, "kv_cache_attend: dimension exceeds 2^31-1");
    int st = ensure_ready();
    if (st) return st;
    if (BH == 0) return AXB_OK;
    mark(0);
    mark(1);
    int e = launch_kv_cache_attend(K_cache, V_cache, Q_new, out, BH, cur_len, max_seq, dk, scale, cur().sm_count, cur().stream);
    mark(2);
    cur().launches++;
    return e ? cuda_fail("kv_cache_attend", e) : AXB_OK;
}

// ------------------------------------------------------- attention projections

// aux scratch of at least `need` bytes (grown on demand; the stream is drained before the old block is freed)
static int ensure_aux(const char *what, size_t need)
{
    if (need <= cur().aux_bytes) return AXB_OK;
    if (cur().aux) { cudaStreamSynchronize(cur().stream); cudaFree(cur().aux); cur().aux = nullptr; cur().aux_bytes = 0; }
    cudaError_t e = cudaMalloc(&cur().aux, need);
    if (e != cudaSuccess) return fail(AXB_ERR_ALLOC, "%s: scratch of %zu bytes: %s", what, need, cudaGetErrorString(e));
    cur().aux_bytes = need;
    return AXB_OK;
}

extern "C" int axb_qkv_head_gemm(const float *X, const float *Wqkv, const float *bqkv, int64_t B, int64_t S, int64_t H,
                                 int64_t dk, float *Qh, float *Kh, float *Vh)
{
    if (!X || !Wqkv || !Qh || !Kh || !Vh) return fail(AXB_ERR_NULL_ARG, "qkv_head_gemm: NULL");
    if (B < 0 || S < 0 || H <= 0 || dk <= 0) return fail(AXB_ERR_INVALID_SHAPE, "qkv_head_gemm: bad shape");
    const int64_t rows = B * S, D = H * dk;
    if (rows > INT32_MAX || 3 * D > INT32_MAX) return fail(AXB_ERR_INVALID_SHAPE, "qkv_head_gemm: dimension exceeds 2^31-1");
    int st = ensure_ready();
    if (st) return st;
    if (rows == 0) return AXB_OK;
    float *outs[3] = { Qh, Kh, Vh };
    if (rows > 32 && dk % 32 == 0) {
        // one launch: the tensor-core GEMM's epilogue adds the bias and stores head-major
        const int64_t shape[3] = { S, H, dk };
        return gemm_tc_f32(X, Wqkv, bqkv, nullptr, rows, 3 * D, D, 0, 0, 1.0f, 0.0f, AXB_ACT_NONE, nullptr, 0, 0, 0, shape, outs);
    }
    // other head dims and skinny inputs: the product (bias fused) into a scratch matrix, then the layout pass
    if ((st = ensure_aux("qkv_head_gemm", (size_t)rows * 3 * D * sizeof(float)))) return st;
    st = axb_gemm_bias_act(X, Wqkv, bqkv, (float *)cur().aux, rows, 3 * D, D, 0, 0, 1.0f, 0.0f, AXB_ACT_NONE);
    if (st) return st;
    int e = launch_head_layout(true, (float *)cur().aux, outs, nullptr, 3, B, S, H, dk, cur().sm_count, cur().stream);
    cur().launches++;
    return e ? cuda_fail("qkv_head_gemm: head split", e) : AXB_OK;
}

extern "C" int axb_dattn_head_gemm_nt(const float *dout, const float *Wo, int64_t B, int64_t S, int64_t H, int64_t dk, float *dO_head)
{
    if (!dout || !Wo || !dO_head) return fail(AXB_ERR_NULL_ARG, "dattn_head_gemm_nt: NULL");
    if (B < 0 || S < 0 || H <= 0 || dk <= 0) return fail(AXB_ERR_INVALID_SHAPE, "dattn_head_gemm_nt: bad shape");
    const int64_t rows = B * S, D = H * dk;
    if (rows > INT32_MAX || D > INT32_MAX) return fail(AXB_ERR_INVALID_SHAPE, "dattn_head_gemm_nt: dimension exceeds 2^31-1");
    int st = ensure_ready();
    if (st) return st;
    if (rows == 0) return AXB_OK;
    float *outs[3] = { dO_head, dO_head, dO_head };   // one D-wide column block: only the first destination is used
    if (rows > 32 && dk % 32 == 0) {
        // one launch: dout . Wo^T on the tensor cores, the epilogue stores head-major
        const int64_t shape[3] = { S, H, dk };
        return gemm_tc_f32(dout, Wo, nullptr, nullptr, rows, D, D, 0, 1, 1.0f, 0.0f, AXB_ACT_NONE, nullptr, 0, 0, 0, shape, outs);
    }
    if ((st = ensure_aux("dattn_head_gemm_nt", (size_t)rows * D * sizeof(float)))) return st;
    st = axb_gemm_bias_act(dout, Wo, nullptr, (float *)cur().aux, rows, D, D, 0, 1, 1.0f, 0.0f, AXB_ACT_NONE);
    if (st) return st;
    int e = launch_head_layout(true, (float *)cur().aux, outs, nullptr, 1, B, S, H, dk, cur().sm_count, cur().stream);
    cur().launches++;
    return e ? cuda_fail("dattn_head_gemm_nt: head layout", e) : AXB_OK;
}

// dW{q,k,v} += x^T . dQKV[:, {0,1,2}*D : +D]; `scratch_off` bytes at the start of aux are in use by the caller
static int dwqkv_split_acc_any(const char *what, const float *x_flat, const float *dQKV, int64_t rows, int64_t D, float *dWq,
                               float *dWk, float *dWv, size_t scratch_off)
{
    float *outs[3] = { dWq, dWk, dWv };
    if (D % 32 == 0) {
        // one launch: x^T . dQKV on the tensor cores; the epilogue treats the three D-wide column blocks as three
        // destinations (the head-major scatter with one head of D columns and D rows per "batch") and adds to them
        const int64_t shape[3] = { D, 1, D };
        return gemm_tc_f32(x_flat, dQKV, nullptr, nullptr, D, 3 * D, rows, 1, 0, 1.0f, 1.0f, AXB_ACT_NONE, nullptr, 0, 0, 0, shape, outs);
    }
    // other widths: the [D, 3D] product into scratch, then one pass that adds its column blocks to the gradients
    const size_t need = scratch_off + (size_t)D * 3 * D * sizeof(float);
    int st = ensure_aux(what, need);
    if (st) return st;
    float *prod = reinterpret_cast<float *>(reinterpret_cast<char *>(cur().aux) + scratch_off);
    st = axb_gemm_bias_act(x_flat, dQKV, nullptr, prod, D, 3 * D, rows, 1, 0, 1.0f, 0.0f, AXB_ACT_NONE);
    if (st) return st;
    int e = launch_head_layout(true, prod, outs, nullptr, 3, 1, D, 1, D, cur().sm_count, cur().stream, true);
    cur().launches++;
    return e ? cuda_fail(what, e) : AXB_OK;
}

extern "C" int axb_dwqkv_split_acc(const float *x_flat, const float *dQKV, int64_t rows, int64_t D, float *dWq, float *dWk,
                                   float *dWv)
{
    if (!x_flat || !dQKV || !dWq || !dWk || !dWv) return fail(AXB_ERR_NULL_ARG, "dwqkv_split_acc: NULL");
    if (rows < 0 || D <= 0) return fail(AXB_ERR_INVALID_SHAPE, "dwqkv_split_acc: bad shape");
    if (rows > INT32_MAX || 3 * D > INT32_MAX) return fail(AXB_ERR_INVALID_SHAPE, "dwqkv_split_acc: dimension exceeds 2^31-1");
    int st = ensure_ready();
    if (st) return st;
    if (rows == 0) return AXB_OK;   // an empty sum: the gradients keep their values
    return dwqkv_split_acc_any("dwqkv_split_acc", x_flat, dQKV, rows, D, dWq, dWk, dWv, 0);
}

extern "C" int axb_dwqkv_split_acc_hm(const float *x_flat, const float *dQh, const float *dKh, const float *dVh, int64_t B,
                                      int64_t S, int64_t H, int64_t dk, float *dWq, float *dWk, float *dWv)
{
    if (!x_flat || !dQh || !dKh || !dVh || !dWq || !dWk || !dWv) return fail(AXB_ERR_NULL_ARG, "dwqkv_split_acc_hm: NULL");
    if (B < 0 || S < 0 || H <= 0 || dk <= 0) return fail(AXB_ERR_INVALID_SHAPE, "dwqkv_split_acc_hm: bad shape");
    const int64_t rows = B * S, D = H * dk;
    if (rows > INT32_MAX || 3 * D > INT32_MAX) return fail(AXB_ERR_INVALID_SHAPE, "dwqkv_split_acc_hm: dimension exceeds 2^31-1");
    int st = ensure_ready();
    if (st) return st;
    if (rows == 0) return AXB_OK;
    // the three head-major gradients are gathered into the flat [rows, 3D] matrix the contraction walks
    const size_t merged = round_up((size_t)rows * 3 * D * sizeof(float), 256);
    st = ensure_aux("dwqkv_split_acc_hm", merged + (D % 32 == 0 ? 0 : (size_t)D * 3 * D * sizeof(float)));
    if (st) return st;
    float *heads[3] = { const_cast<float *>(dQh), const_cast<float *>(dKh), const_cast<float *>(dVh) };
    int e = launch_head_layout(false, (float *)cur().aux, heads, nullptr, 3, B, S, H, dk, cur().sm_count, cur().stream);
    cur().launches++;
    if (e) return cuda_fail("dwqkv_split_acc_hm: merge", e);
    return dwqkv_split_acc_any("dwqkv_split_acc_hm", x_flat, (const float *)cur().aux, rows, D, dWq, dWk, dWv, merged);
}

extern "C" int axb_mha_output_proj_fused(const float *attn_flat, const float *Wo, const float *bo, const float *dout, float *y,
                                         float *dattn, float *dWo_acc, float *dbo_acc, int64_t rows, int64_t D)
{
    if (!attn_flat || !Wo || !dout || !dattn || !dWo_acc) return fail(AXB_ERR_NULL_ARG, "mha_output_proj_fused: NULL");
    if (rows < 0 || D <= 0) return fail(AXB_ERR_INVALID_SHAPE, "mha_output_proj_fused: bad shape");
    if (rows > INT32_MAX || D > INT32_MAX) return fail(AXB_ERR_INVALID_SHAPE, "mha_output_proj_fused: dimension exceeds 2^31-1");
    int st = ensure_ready();
    if (st) return st;
    if (rows == 0) return AXB_OK;
    // forward: y = attn . Wo + bo (bias in the epilogue); skipped without y
    if (y && (st = axb_gemm_bias_act(attn_flat, Wo, bo, y, rows, D, D, 0, 0, 1.0f, 0.0f, AXB_ACT_NONE))) return st;
    // dattn = dout . Wo^T
    if ((st = axb_gemm_bias_act(dout, Wo, nullptr, dattn, rows, D, D, 0, 1, 1.0f, 0.0f, AXB_ACT_NONE))) return st;
    // dWo += attn^T . dout
    if ((st = axb_gemm_bias_act(attn_flat, dout, nullptr, dWo_acc, D, D, rows, 1, 0, 1.0f, 1.0f, AXB_ACT_NONE))) return st;
    if (dbo_acc) {
        // dbo += column sums of dout = ones[1, rows] . dout: the bandwidth-bound one-row route reads dout once
        if ((st = ensure_aux("mha_output_proj_fused", (size_t)rows * sizeof(float)))) return st;
        int e = launch_fill((float *)cur().aux, rows, 1.0f, cur().sm_count, cur().stream);
        cur().launches++;
        if (e) return cuda_fail("mha_output_proj_fused: fill", e);
        if ((st = axb_gemm_bias_act((const float *)cur().aux, dout, nullptr, dbo_acc, 1, D, rows, 0, 0, 1.0f, 1.0f, AXB_ACT_NONE))) return st;
    }
    return AXB_OK;
}

// ------------------------------------------------------- attention layout passes

static int head_layout_call(const char *what, bool to_head, const float *flat, float *const head[3], const float *bias,
                            int nslot, int64_t B, int64_t S, int64_t H, int64_t dk)
{
    if (!flat) return fail(AXB_ERR_NULL_ARG, "%s: NULL", what);
    for (int i = 0; i < nslot; ++i)
        if (!head[i]) return fail(AXB_ERR_NULL_ARG, "%s: NULL", what);
    if (B < 0 || S < 0 || H <= 0 || dk <= 0) return fail(AXB_ERR_INVALID_SHAPE, "%s: bad shape", what);
    if (S > INT32_MAX || H > INT32_MAX || dk > INT32_MAX) return fail(AXB_ERR_INVALID_SHAPE, "%s: dimension exceeds 2^31-1", what);
    int st = ensure_ready();
    if (st) return st;
    int e = launch_head_layout(to_head, const_cast<float *>(flat), head, bias, nslot, B, S, H, dk, cur().sm_count, cur().stream);
    cur().launches++;
    return e ? cuda_fail(what, e) : AXB_OK;
}

extern "C" int axb_head_interleave_qkv_split(const float *qkv, const float *bqkv, float *Qh, float *Kh, float *Vh,
                                             int64_t B, int64_t S, int64_t H, int64_t dk)
{
    float *head[3] = { Qh, Kh, Vh };
    return head_layout_call("head_interleave_qkv_split", true, qkv, head, bqkv, 3, B, S, H, dk);
}

extern "C" int axb_head_interleave(const float *src, float *dst, int64_t B, int64_t S, int64_t H, int64_t dk)
{
    float *head[3] = { dst, nullptr, nullptr };
    return head_layout_call("head_interleave", true, src, head, nullptr, 1, B, S, H, dk);
}

extern "C" int axb_head_deinterleave(const float *src, float *dst, int64_t B, int64_t S, int64_t H, int64_t dk)
{
    float *head[3] = { const_cast<float *>(src), nullptr, nullptr };
    return head_layout_call("head_deinterleave", false, dst, head, nullptr, 1, B, S, H, dk);
}

extern "C" int axb_head_deinterleave_qkv_merge(const float *dQ, const float *dK, const float *dV, float *dst, int64_t B,
                                               int64_t S, int64_t H, int64_t dk)
{
    float *head[3] = { const_cast<float *>(dQ), const_cast<float *>(dK), const_cast<float *>(dV) };
    return head_layout_call("head_deinterleave_qkv_merge", false, dst, head, nullptr, 3, B, S, H, dk);
}

// dst[rows, 3*cols] = [a | b | c] row by row (rows = cols = D for the weights; rows = 1 for the biases)
static int concat3(const char *what, float *dst, const float *a, const float *b, const float *c, int64_t rows, int64_t cols)
{
    if (!dst || !a || !b || !c) return fail(AXB_ERR_NULL_ARG, "%s: NULL", what);
    if (rows < 0 || cols < 0) return fail(AXB_ERR_INVALID_SHAPE, "%s: bad shape", what);
    int st = ensure_ready();
    if (st) return st;
    if (rows == 0 || cols == 0) return AXB_OK;
    const size_t w = (size_t)cols * sizeof(float);
    const float *src[3] = { a, b, c };
    for (int i = 0; i < 3; ++i) {
        cudaError_t e = cudaMemcpy2DAsync(dst + i * cols, 3 * w, src[i], w, w, (size_t)rows, cudaMemcpyDeviceToDevice, cur().stream);
        if (e != cudaSuccess) return cuda_fail(what, e);
    }
    return AXB_OK;
}

extern "C" int axb_qkv_cache_build(float *dst, const float *wq, const float *wk, const float *wv, int64_t D)
{
    return concat3("qkv_cache_build", dst, wq, wk, wv, D, D);
}

extern "C" int axb_bias_cache_build(float *dst, const float *bq, const float *bk, const float *bv, int64_t D)
{
    return concat3("bias_cache_build", dst, bq, bk, bv, 1, D);
}

extern "C" int axb_pointer_on_device(const void *p)
{
    if (!p) return 0;
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, p) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return (at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged) ? 1 : 0;
}
