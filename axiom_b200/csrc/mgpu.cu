// mgpu.cu — the large GEMMs and the chained MLP partitioned over the GPUs of one box, callable from a C host.
//
// axiom is single-device (no counterpart in the reference): these entry points are new.  One host thread walks
// the devices — every launch is asynchronous, so n devices run side by side without n host threads — and each
// device has its own engine (axb_init(device) selects it).  Two partitions:
//   rows (M)     every rank owns a block of rows of A and C, the weights are replicated: no communication.
//   columns (N)  every rank owns n = N / g output columns of a layer (its slab of W and of the bias), computes
//                its [M, n] slab with bias and activation fused in the GEMM epilogue, and ONE ncclAllGather per
//                layer leaves the full activation on every rank as [g][M][n] — each rank's slab contiguous, so the
//                collective is a plain contiguous all-gather — which the next layer reads in place as its
//                [M, g*n] operand (axb_gemm_gathered_scatter walks the g chunks; no re-layout pass).
// NCCL is bound at run time (dlopen of libnccl.so.2): a host that never creates a multi-GPU handle does not need it.
#include "../../include/axiom_b200.h"

#include "errors.cuh"

#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

using namespace axb;

namespace {

struct NcclApi {
    void *lib = nullptr;
    ncclResult_t (*CommInitAll)(ncclComm_t *, int, const int *) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
};

NcclApi g_nccl;

int load_nccl()
{
    if (g_nccl.lib) return AXB_OK;
    void *lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!lib) lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!lib) return set_error(AXB_ERR_BACKEND, "mgpu: libnccl.so.2 not found: %s", dlerror());
    NcclApi api;
    api.lib = lib;
    api.CommInitAll = reinterpret_cast<decltype(api.CommInitAll)>(dlsym(lib, "ncclCommInitAll"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(dlsym(lib, "ncclCommDestroy"));
    api.GroupStart = reinterpret_cast<decltype(api.GroupStart)>(dlsym(lib, "ncclGroupStart"));
    api.GroupEnd = reinterpret_cast<decltype(api.GroupEnd)>(dlsym(lib, "ncclGroupEnd"));
    api.AllGather = reinterpret_cast<decltype(api.AllGather)>(dlsym(lib, "ncclAllGather"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(dlsym(lib, "ncclGetErrorString"));
    if (!api.CommInitAll || !api.CommDestroy || !api.GroupStart || !api.GroupEnd || !api.AllGather || !api.GetErrorString)
        return set_error(AXB_ERR_BACKEND, "mgpu: libnccl lacks a required symbol");
    g_nccl = api;
    return AXB_OK;
}

constexpr int kMaxRanks = 16;

}  // namespace

struct axb_mgpu {
    int n = 0;
    int dev[kMaxRanks] = {};
    ncclComm_t comm[kMaxRanks] = {};
    bool have_comm = false;
};

namespace {

// selects rank r's device and engine for the calls that follow
int use_rank(const axb_mgpu *h, int r) { return axb_init(h->dev[r]); }

// puts the caller's device back when a multi-device call returns
struct DeviceGuard {
    int prev;
    DeviceGuard() : prev(engine_device()) {}
    ~DeviceGuard()
    {
        if (prev >= 0) axb_init(prev);
    }
};

int check_handle(const axb_mgpu *h, const char *what)
{
    if (!h || h->n < 1) return set_error(AXB_ERR_NULL_ARG, "%s: no multi-GPU handle", what);
    return AXB_OK;
}

}  // namespace

extern "C" int axb_mgpu_create(int n_devices, const int *devices, axb_mgpu **out)
{
    if (!out) return set_error(AXB_ERR_NULL_ARG, "mgpu_create: NULL");
    *out = nullptr;
    const int count = axb_device_count();
    if (n_devices < 1 || n_devices > kMaxRanks || n_devices > count)
        return set_error(AXB_ERR_INVALID_SHAPE, "mgpu_create: %d devices asked for, %d present (at most %d)", n_devices, count, kMaxRanks);
    axb_mgpu *h = new axb_mgpu();
    h->n = n_devices;
    DeviceGuard guard;
    for (int r = 0; r < n_devices; ++r) {
        h->dev[r] = devices ? devices[r] : r;
        for (int q = 0; q < r; ++q)
            if (h->dev[q] == h->dev[r]) {
                delete h;
                return set_error(AXB_ERR_INVALID_SHAPE, "mgpu_create: device %d listed twice", h->dev[r]);
            }
        int st = use_rank(h, r);
        if (st) {
            delete h;
            return st;
        }
    }
    if (n_devices > 1) {
        int st = load_nccl();
        if (st) {
            delete h;
            return st;
        }
        ncclResult_t nr = g_nccl.CommInitAll(h->comm, n_devices, h->dev);
        if (nr != ncclSuccess) {
            delete h;
            return set_error(AXB_ERR_BACKEND, "mgpu_create: ncclCommInitAll: %s", g_nccl.GetErrorString(nr));
        }
        h->have_comm = true;
    }
    *out = h;
    return AXB_OK;
}

extern "C" void axb_mgpu_destroy(axb_mgpu *h)
{
    if (!h) return;
    DeviceGuard guard;
    for (int r = 0; r < h->n; ++r) {
        if (use_rank(h, r) == AXB_OK) axb_synchronize();
        if (h->have_comm && h->comm[r]) g_nccl.CommDestroy(h->comm[r]);
    }
    delete h;
}

extern "C" int axb_mgpu_size(const axb_mgpu *h) { return h ? h->n : 0; }

extern "C" int axb_mgpu_device(const axb_mgpu *h, int rank) { return (h && rank >= 0 && rank < h->n) ? h->dev[rank] : -1; }

extern "C" void *axb_mgpu_alloc(axb_mgpu *h, int rank, size_t bytes)
{
    if (check_handle(h, "mgpu_alloc") || rank < 0 || rank >= h->n) return nullptr;
    DeviceGuard guard;
    if (use_rank(h, rank)) return nullptr;
    return axb_storage_alloc(bytes);
}

extern "C" void axb_mgpu_free(axb_mgpu *h, int rank, void *ptr)
{
    if (!h || rank < 0 || rank >= h->n || !ptr) return;
    DeviceGuard guard;
    if (use_rank(h, rank) == AXB_OK) axb_storage_free(ptr);
}

extern "C" int axb_mgpu_h2d(axb_mgpu *h, int rank, void *dst, const void *src_host, size_t bytes)
{
    int st = check_handle(h, "mgpu_h2d");
    if (st) return st;
    if (rank < 0 || rank >= h->n) return set_error(AXB_ERR_INVALID_SHAPE, "mgpu_h2d: rank %d of %d", rank, h->n);
    DeviceGuard guard;
    if ((st = use_rank(h, rank))) return st;
    return axb_memcpy_h2d(dst, src_host, bytes);
}

extern "C" int axb_mgpu_d2h(axb_mgpu *h, int rank, void *dst_host, const void *src, size_t bytes)
{
    int st = check_handle(h, "mgpu_d2h");
    if (st) return st;
    if (rank < 0 || rank >= h->n) return set_error(AXB_ERR_INVALID_SHAPE, "mgpu_d2h: rank %d of %d", rank, h->n);
    DeviceGuard guard;
    if ((st = use_rank(h, rank))) return st;
    return axb_memcpy_d2h(dst_host, src, bytes);
}

extern "C" int axb_mgpu_synchronize(axb_mgpu *h)
{
    int st = check_handle(h, "mgpu_synchronize");
    if (st) return st;
    DeviceGuard guard;
    int bad = 0;
    for (int r = 0; r < h->n; ++r) {
        if ((st = use_rank(h, r))) return st;
        axb_synchronize();
        if (axb_device_error() != 0) bad = AXB_ERR_BACKEND;
    }
    return bad;
}

extern "C" int axb_mgpu_gemm_rows(axb_mgpu *h, const float *const *A, const float *const *B, const float *const *bias,
                                  float *const *C, const int64_t *rows, int64_t N, int64_t K, int act)
{
    int st = check_handle(h, "mgpu_gemm_rows");
    if (st) return st;
    if (!A || !B || !C || !rows) return set_error(AXB_ERR_NULL_ARG, "mgpu_gemm_rows: NULL");
    DeviceGuard guard;
    for (int r = 0; r < h->n; ++r) {
        if ((st = use_rank(h, r))) return st;
        st = axb_gemm_bias_act(A[r], B[r], bias ? bias[r] : nullptr, C[r], rows[r], N, K, 0, 0, 1.0f, 0.0f, act);
        if (st) return st;
    }
    return AXB_OK;
}

extern "C" int axb_mgpu_qgemm_w8a8_rows(axb_mgpu *h, const int8_t *const *a_q, float a_scale, const int8_t *const *b_q,
                                        const float *const *b_scales, float out_scale, int8_t *const *out_q,
                                        const int64_t *rows, int64_t N, int64_t K)
{
    int st = check_handle(h, "mgpu_qgemm_w8a8_rows");
    if (st) return st;
    if (!a_q || !b_q || !b_scales || !out_q || !rows) return set_error(AXB_ERR_NULL_ARG, "mgpu_qgemm_w8a8_rows: NULL");
    DeviceGuard guard;
    for (int r = 0; r < h->n; ++r) {
        if ((st = use_rank(h, r))) return st;
        st = axb_qgemm_w8a8(a_q[r], a_scale, b_q[r], b_scales[r], out_scale, out_q[r], nullptr, rows[r], N, K);
        if (st) return st;
    }
    return AXB_OK;
}

extern "C" int axb_mgpu_gemm_cols_allgather(axb_mgpu *h, const float *const *X, int x_chunks, const float *const *W,
                                            const float *const *bias, float *const *slab, float *const *gathered,
                                            int64_t M, int64_t n, int64_t K, int act)
{
    int st = check_handle(h, "mgpu_gemm_cols_allgather");
    if (st) return st;
    if (!X || !W || !slab || !gathered) return set_error(AXB_ERR_NULL_ARG, "mgpu_gemm_cols_allgather: NULL");
    if (x_chunks < 1 || M < 0 || n < 0 || K < 1 || K % x_chunks != 0)
        return set_error(AXB_ERR_INVALID_SHAPE, "mgpu_gemm_cols_allgather: K must be a positive multiple of x_chunks");
    DeviceGuard guard;
    // every rank's slab: bias and activation in the GEMM epilogue
    for (int r = 0; r < h->n; ++r) {
        if ((st = use_rank(h, r))) return st;
        const float *b = bias ? bias[r] : nullptr;
        if (x_chunks == 1) st = axb_gemm_bias_act(X[r], W[r], b, slab[r], M, n, K, 0, 0, 1.0f, 0.0f, act);
        else st = axb_gemm_gathered_scatter(X[r], x_chunks, K / x_chunks, W[r], b, slab[r], nullptr, 0, M, n, 1.0f, 0.0f, act);
        if (st) return st;
    }
    if (M == 0 || n == 0) return AXB_OK;
    if (h->n == 1) {
        if ((st = use_rank(h, 0))) return st;
        return axb_memcpy_d2d(gathered[0], slab[0], (size_t)M * n * sizeof(float));
    }
    // one all-gather: rank r's slab lands at gathered[*][r] on every rank, behind that rank's GEMM on its stream
    ncclResult_t nr = g_nccl.GroupStart();
    for (int r = 0; r < h->n && nr == ncclSuccess; ++r) {
        if ((st = use_rank(h, r))) {
            g_nccl.GroupEnd();
            return st;
        }
        nr = g_nccl.AllGather(slab[r], gathered[r], (size_t)M * n, ncclFloat, h->comm[r], engine_stream());
    }
    const ncclResult_t ne = g_nccl.GroupEnd();
    if (nr == ncclSuccess) nr = ne;
    if (nr != ncclSuccess) return set_error(AXB_ERR_BACKEND, "mgpu_gemm_cols_allgather: ncclAllGather: %s", g_nccl.GetErrorString(nr));
    return AXB_OK;
}
