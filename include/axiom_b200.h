/* axiom_b200.h — C ABI of libaxiom_b200.so, a Blackwell (sm_100a) engine for
   axiom's matmul-dispatch hot path.

   Every entry point takes plain pointers and sizes.  Unless a parameter is
   named *_host, data pointers are DEVICE pointers on the device chosen by
   axb_init; matrices are dense row-major.  Work is enqueued asynchronously on
   the engine's stream (the legacy default stream unless axb_set_stream was
   called), exactly like the reference CUDA backend; results become visible to
   the host after axb_synchronize() or a blocking axb_memcpy_d2h().

   Return values are axiom's status codes (include/axiom/types.h:89-103 of the
   reference): 0 = AX_OK, 1 = NULL_ARG, 2 = ALLOC, 3 = SHAPE_MISMATCH,
   7 = INVALID_DTYPE, 9 = BACKEND, 10 = NOT_IMPLEMENTED ...  The engine never
   aborts and never falls back to host arithmetic; axb_last_error() returns
   the message of the most recent failure.  There is one engine per device;
   an engine is not thread-safe: one host thread drives it at a time, as with
   the reference backend (src/compute/backends/cuda/internal.h:70-74).

   Each declaration cites the reference interface it replaces as
   file:line within the axiom source tree. */
#ifndef AXIOM_B200_H
#define AXIOM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* exported from the shared library (everything else in it is hidden) */
#define AXB_API __attribute__((visibility("default")))

#define AXB_OK 0
#define AXB_ERR_NULL_ARG 1
#define AXB_ERR_ALLOC 2
#define AXB_ERR_SHAPE_MISMATCH 3
#define AXB_ERR_INVALID_AXIS 5
#define AXB_ERR_INVALID_SHAPE 6
#define AXB_ERR_BACKEND 9
#define AXB_ERR_NOT_IMPLEMENTED 10

/* activation selectors for the fused epilogues */
#define AXB_ACT_NONE 0
#define AXB_ACT_RELU 1
#define AXB_ACT_GELU 2 /* tanh approximation, src/core/activations.c:23-25 */

/* how fp32 GEMMs are computed on the tensor cores */
#define AXB_FP32_3XTF32 0 /* hi/lo TF32 split, 3 products: normalised error <= 1e-5 (default) */
#define AXB_FP32_BF16X3 1 /* hi/lo bf16 split, 3 products: same bound on well-scaled data, 2x faster */
#define AXB_FP32_BF16 2   /* single bf16 product: normalised error <= 5e-3 */

/* ---- lifecycle and device-owner hooks ------------------------------------
   Replace cuda_init_hook / cuda_shutdown_hook / cuda_sync_hook /
   cuda_device_count_hook (src/compute/backends/cuda/backend.cu:56-116) and the
   storage + memcpy hooks (src/compute/backends/cuda/memory.cu:80-140), i.e. the
   device-owner slots of ax_backend_ops_t
   (include/axiom/internal/backend_ops.h:262-296). */
AXB_API int axb_init(int device);      /* idempotent per device; selects the device (and its engine) for the calling thread;
                                          -1 = the thread's current choice; reads AX_B200_FP32_MODE = 3xtf32|bf16x3|bf16 */
AXB_API void axb_shutdown(void);       /* every device's engine */
AXB_API int axb_device_count(void);
AXB_API void axb_synchronize(void);    /* blocks; afterwards axb_device_error() is current */
AXB_API void *axb_storage_alloc(size_t bytes);   /* zero-filled, like the reference's pool allocator */
AXB_API void axb_storage_free(void *ptr);
AXB_API int axb_memcpy_h2d(void *dst, const void *src_host, size_t bytes); /* blocking */
AXB_API int axb_memcpy_d2h(void *dst_host, const void *src, size_t bytes); /* blocking */
AXB_API int axb_memcpy_d2d(void *dst, const void *src, size_t bytes);
AXB_API void axb_set_stream(void *cuda_stream); /* NULL = legacy default stream */
AXB_API int axb_set_fp32_mode(int mode);        /* AXB_FP32_* */
AXB_API int axb_get_fp32_mode(void);
AXB_API const char *axb_last_error(void);
/* Non-zero when a kernel gave up on a bounded wait (its code); reading clears it. */
AXB_API int axb_device_error(void);
/* Kernels enqueued by this library since the counter was last reset. */
AXB_API int64_t axb_launch_count(int reset);
/* Measurement aid (no reference counterpart): with profiling on, every GEMM-family,
   quantised-GEMM and attention call records CUDA events on the engine's stream
   around its operand pre-pass and around its main kernel (the newest 256 calls
   are kept).  axb_timing_summary blocks until they have finished, returns how
   many calls it covers and their summed pre-pass and main-kernel times in
   milliseconds, and starts a new window.  axb_set_profiling also starts one. */
AXB_API void axb_set_profiling(int on);
AXB_API int axb_timing_summary(int *calls, float *prepass_ms_total, float *core_ms_total);
/* The same window call by call (oldest first, at most cap entries, newest 256 kept): per-call pre-pass and
   main-kernel milliseconds, for medians and minima.  Does not start a new window. */
AXB_API int axb_timing_samples(float *prepass_ms, float *core_ms, int cap, int *n_out);

/* ---- dense fp32 GEMM family ----------------------------------------------
   Slots gemm / gemm_nt / gemm_tn / gemm_ex / gemm_relu of ax_backend_ops_t
   (backend_ops.h:54-65,156-165), reference CUDA implementations
   src/compute/backends/cuda/ops_gemm.cu:15-126 (cuBLAS) and CPU
   src/compute/backends/cpu_opt.c:3446,4842,5660,7401,7442. */

/* C[M,N] = A[M,K] . B[K,N]                        (ax_compute_gemm, dispatch.c:414) */
AXB_API int axb_gemm(const float *A, const float *B, float *C, int64_t M, int64_t N, int64_t K);
/* The same product on HOST operands (pinned memory for full transfer speed): C_host = A_host . B_host.
   In the reference a host caller pays ax_tensor_to_cuda + gemm + ax_tensor_to_cpu one after the other
   (src/core/tensor.c:1016-1090: three synchronous copies around the launch); this entry has no counterpart
   there.  B is uploaded and split once; A goes up in chunks of row_chunk rows (0 = about M/16) that are multiplied
   as they land while finished rows of C travel back, so the call costs about max(upload, compute, download)
   instead of their sum.  Synchronous: C_host is complete on return.  Bit-identical to axb_gemm on device
   copies of the same operands. */
AXB_API int axb_gemm_host(const float *A_host, const float *B_host, float *C_host, int64_t M, int64_t N, int64_t K,
                          int64_t row_chunk);
/* C[M,N] = A[M,K] . B[N,K]^T                      (ax_compute_gemm_nt, dispatch.c:419) */
AXB_API int axb_gemm_nt(const float *A, const float *B, float *C, int64_t M, int64_t N, int64_t K);
/* C[M,N] = A[K,M]^T . B[K,N]                      (ax_compute_gemm_tn, dispatch.c:430) */
AXB_API int axb_gemm_tn(const float *A, const float *B, float *C, int64_t M, int64_t N, int64_t K);
/* C = alpha * A.B + beta * C; beta == 0 never reads C   (ax_compute_gemm_ex, dispatch.c:642) */
AXB_API int axb_gemm_ex(const float *A, const float *B, float alpha, float beta, float *C,
                int64_t M, int64_t N, int64_t K);
/* C = max(A.B + bias[n], 0); bias may be NULL      (ax_compute_gemm_relu, dispatch.c:443) */
AXB_API int axb_gemm_relu(const float *A, const float *B, const float *bias, float *C,
                  int64_t M, int64_t N, int64_t K);
/* The general form all of the above reduce to:
     C = act(alpha * op(A).op(B) + beta * C + bias[n])
   trans_a: A stored [K,M]; trans_b: B stored [N,K]; act = AXB_ACT_*.
   This is the dense-layer path of src/core/ops.c:295-440 (matmul, bias, activation)
   in one launch; act = GELU fuses the separate ax_gelu pass
   (src/core/layer.c:110-114).  M <= 32 with B stored [K,N] takes the
   bandwidth-bound skinny route (the reference's tiny-M AXPY path,
   cpu_opt.c:3499-3567). */
AXB_API int axb_gemm_bias_act(const float *A, const float *B, const float *bias, float *C,
                      int64_t M, int64_t N, int64_t K, int trans_a, int trans_b,
                      float alpha, float beta, int act);

/* ---- prepared weights --------------------------------------------------------
   A dense layer multiplies by the same weight matrix call after call.  axb_weight_prepare makes the tensor-core
   operand planes of B once (device memory owned by the handle: 8 bytes per element in the 3xTF32 mode, 4 in bf16x3,
   2 in bf16); axb_gemm_prepared then splits only the left operand:
     C[M,N] = act(alpha * op(A) . op(B) + beta * C + bias[n])
   with the same routes and bit-identical results as axb_gemm_bias_act on the same operands.  B must stay allocated
   and unchanged until axb_weight_release (M <= 32 streams it directly); a weight belongs to the device and the fp32
   mode it was prepared under.  The reference's CPU backend keeps packed B panels across calls in the same spirit
   (pack_b cache keyed on storage pointer and generation, src/compute/backends/cpu_opt.c); its CUDA backend has no
   counterpart (cuBLAS repacks nothing). */
typedef struct axb_weight axb_weight_t;
AXB_API int axb_weight_prepare(const float *B, int64_t K, int64_t N, int trans_b, axb_weight_t **out);
AXB_API void axb_weight_release(axb_weight_t *w);
AXB_API int axb_gemm_prepared(const float *A, const axb_weight_t *W, const float *bias, float *C, int64_t M, int trans_a,
                              float alpha, float beta, int act);

/* ---- multi-GPU building blocks (no counterpart in the reference, which is single-device) ----
   axb_gemm_bias_act_scatter is axb_gemm_bias_act on the tensor cores whose epilogue stores each finished tile to C
   AND to n_more further buffers of the same shape and pitch (at most 8).  With C_more pointing into peers' gather
   buffers (mapped through the axb_ipc_* calls) a rank's output slab reaches every GPU over NVLink while the GEMM is
   still running, replacing the separate all-gather of a column-sharded layer; the caller still needs one small
   cross-rank synchronisation before the peers read.  beta reads C only. */
AXB_API int axb_gemm_bias_act_scatter(const float *A, const float *B, const float *bias, float *C,
                                      float *const *C_more, int n_more, int64_t M, int64_t N, int64_t K,
                                      int trans_a, int trans_b, float alpha, float beta, int act);
/* The same GEMM reading its left operand straight out of a gather buffer: A_gathered is [chunks][M][chunk_k]
   (what an all-gather of column slabs leaves behind) and stands for the [M, chunks*chunk_k] matrix whose
   columns chunk c occupy [c*chunk_k, (c+1)*chunk_k); B is [chunks*chunk_k, N].  No re-layout pass and no
   accumulating calls: the operand split reads the chunks in place.  chunk_k % 4 == 0.  C_more / n_more as above
   (n_more = 0 for a plain GEMM). */
AXB_API int axb_gemm_gathered_scatter(const float *A_gathered, int chunks, int64_t chunk_k, const float *B,
                                      const float *bias, float *C, float *const *C_more, int n_more, int64_t M,
                                      int64_t N, float alpha, float beta, int act);
/* Both of the above with the weight's operand planes prepared once (axb_weight_prepare from the [K, N] form): the
   tensor-core GEMM whose epilogue also stores to C_more, reading A either as a plain [M, K] matrix (chunks = 0) or out
   of a gather buffer [chunks][M][chunk_k] with chunks * chunk_k = K.  Same bits as the unprepared calls. */
AXB_API int axb_gemm_prepared_scatter(const float *A, int chunks, int64_t chunk_k, const axb_weight_t *W, const float *bias,
                                      float *C, float *const *C_more, int n_more, int64_t M, float alpha, float beta,
                                      int act);
/* Share a device allocation made with axb_storage_alloc with the other processes of the box:
   the owner exports a 64-byte handle, a peer opens it (peer access is enabled on first use) and gets a
   pointer valid on ITS device context; close before the owner frees. */
AXB_API int axb_ipc_get_handle(const void *dev_ptr, void *handle_64_bytes);
AXB_API int axb_ipc_open_handle(const void *handle_64_bytes, void **dev_ptr_out);
AXB_API int axb_ipc_close_handle(void *dev_ptr);

/* ---- one host thread, several GPUs (no counterpart in the reference) -----------------------------------
   Every device has its own engine; axb_init(device) initialises it on first use and makes it the one the
   calling thread's subsequent axb_* calls drive (it also makes that device the thread's current CUDA device).
   The entry points below walk the devices of a handle from the calling thread — every launch is asynchronous,
   so the devices work side by side — and put the caller's device back before they return.  Arrays are indexed
   by rank (0 .. n-1); rank r's pointers are device pointers on device axb_mgpu_device(h, r).
   NCCL (libnccl.so.2) is loaded when a handle with more than one device is created. */
typedef struct axb_mgpu axb_mgpu_t;
AXB_API int axb_mgpu_create(int n_devices, const int *devices /* NULL = 0 .. n-1 */, axb_mgpu_t **out);
AXB_API void axb_mgpu_destroy(axb_mgpu_t *h);
AXB_API int axb_mgpu_size(const axb_mgpu_t *h);
AXB_API int axb_mgpu_device(const axb_mgpu_t *h, int rank);
AXB_API void *axb_mgpu_alloc(axb_mgpu_t *h, int rank, size_t bytes);   /* zero-filled, on rank's device */
AXB_API void axb_mgpu_free(axb_mgpu_t *h, int rank, void *ptr);
AXB_API int axb_mgpu_h2d(axb_mgpu_t *h, int rank, void *dst, const void *src_host, size_t bytes);
AXB_API int axb_mgpu_d2h(axb_mgpu_t *h, int rank, void *dst_host, const void *src, size_t bytes);
AXB_API int axb_mgpu_synchronize(axb_mgpu_t *h);   /* all devices; AX_ERR_BACKEND if a kernel gave up on a bounded wait */
/* Rows (M) partitioned, weights replicated, no communication:
     rank r:  C[r][rows[r], N] = act(A[r][rows[r], K] . B[r][K, N] + bias[r][N])      (bias may be NULL)
   Each rank's result is bit-identical to the same rows of one axb_gemm_bias_act over the whole matrix whenever
   both take the same K-slicing (always for problems that fill a GPU). */
AXB_API int axb_mgpu_gemm_rows(axb_mgpu_t *h, const float *const *A, const float *const *B, const float *const *bias,
                               float *const *C, const int64_t *rows, int64_t N, int64_t K, int act);
/* The same partition for axb_qgemm_w8a8 (requantised int8 output). */
AXB_API int axb_mgpu_qgemm_w8a8_rows(axb_mgpu_t *h, const int8_t *const *a_q, float a_scale, const int8_t *const *b_q,
                                     const float *const *b_scales, float out_scale, int8_t *const *out_q,
                                     const int64_t *rows, int64_t N, int64_t K);
/* Output columns (N) partitioned, one NCCL all-gather: rank r holds W[r][K, n] and bias[r][n] (its n = N/g columns),
     slab[r][M, n] = act(X[r] . W[r] + bias[r]);   gathered[r][q][M][n] = slab[q] for every rank q
   so every rank ends up with the full activation as [g][M][n].  X[r] is the full input on rank r: a plain [M, K]
   matrix (x_chunks = 1) or the [x_chunks][M][K / x_chunks] buffer a previous call gathered, read in place.
   Chaining calls gives the column-sharded MLP with one all-gather per layer. */
AXB_API int axb_mgpu_gemm_cols_allgather(axb_mgpu_t *h, const float *const *X, int x_chunks, const float *const *W,
                                         const float *const *bias, float *const *slab, float *const *gathered,
                                         int64_t M, int64_t n, int64_t K, int act);

/* Skinny-M GEMM that never allocates (no counterpart in the reference).
     Y[M,N] = act(alpha * X[M,K] . W[K,N] + beta * Y + bias[n]),  1 <= M <= 32
   Takes the same kernel as the skinny route of axb_gemm_bias_act for the same arguments — the TMA-ringed FMA
   kernel up to 8 rows, the tensor-core kernel from 9 rows on (which needs no scratch), the plain-load kernel for
   operands a tensor map cannot describe — and gives bit-identical results, but the split-K scratch is a fixed
   4 MiB + 4 KiB array inside the library image (AXB_STATIC_SCRATCH_BYTES, resident on every GPU that loads the
   library) instead of memory obtained from cudaMalloc.  It is meant for callers that must not allocate once they
   are running: a host framework that handed the whole device to its own arena at start-up, a serving loop that
   cannot afford the device-wide stall an allocation may cause, or a process held to a fixed memory budget.
   The call uses neither the engine's state nor axb_init, and issues no cudaMalloc, cudaFree or other allocating
   call.
   - The device used is the calling thread's current CUDA device; work goes to
     cuda_stream (NULL = legacy default stream).
   - The first call on each device looks up the array's address on that device;
     make that first call during start-up, outside any stream capture.
   - The CUDA runtime loads a kernel's code onto the device the first time that kernel is launched, and each
     row bucket (1, 2, 4, 8, 16, 32 rows) and route is a kernel of its own.  A caller that may not see the
     driver touch device memory at all after start-up makes one call per row bucket and route it will use
     while starting up; later calls then change nothing on the device but Y and the array.
   - Most shapes reduce their K-slices inside a thread-block cluster and need no scratch at all.  Shapes
     that do need it (K too long for a cluster of 8 slices, i.e. roughly K * M > 131072, or N < 2400)
     and whose split-K partial sums exceed the array (slices * M * N > 2^20 floats), or with more than
     1023 column strips, are refused with AXB_ERR_INVALID_SHAPE and a message; nothing is launched.
   - All calls on a device share the one array and it keeps the previous call's
     contents (the counters are cleared on the stream before each launch).  Two
     calls that overlap on the GPU — different streams without ordering, or
     different threads — race on it; serialise them.
   - Every wait inside the kernels is bounded.  If one runs out (it should not), the kernel writes a code into
     the last word of the array and returns; Y is then incomplete.  axb_skinny_gemm_static_error() reads that
     word for the current device (a blocking 4-byte copy, no allocation), returns it and clears it; 0 = none. */
#define AXB_STATIC_SCRATCH_BYTES ((1u << 22) + 4096u)
AXB_API int axb_skinny_gemm_static(const float *X, const float *W, const float *bias, float *Y,
                                   int64_t M, int64_t N, int64_t K, float alpha, float beta, int act,
                                   void *cuda_stream);
AXB_API int axb_skinny_gemm_static_error(void);

/* ---- elementwise slots that remain as separate calls ---------------------- */
/* out = in + bias broadcast along axis (0: bias[M], 1: bias[N]); out may alias in.
   (bias_add slot, backend_ops.h:190; src/compute/backends/cuda/ops_fused.cu:260-292) */
AXB_API int axb_bias_add(const float *in, const float *bias, int axis, float *out, int64_t M, int64_t N);
/* The same slot for a tensor of any rank seen as [outer, axis_len, inner] (the products of the dimensions before
   and after the broadcast axis, ops_fused.cu:281-285): out[o,a,i] = in[o,a,i] + bias[a]. */
AXB_API int axb_bias_add_nd(const float *in, const float *bias, float *out, int64_t outer, int64_t axis_len,
                            int64_t inner);
/* (relu slot, backend_ops.h:235) */
AXB_API int axb_relu(const float *in, float *out, int64_t n);
/* (gelu_op slot, backend_ops.h:244; src/compute/backends/cuda/ops_activations.cu:12-24) */
AXB_API int axb_gelu(const float *in, float *out, int64_t n);

/* ---- quantised GEMM -------------------------------------------------------- */
/* W8A32: out[M,N] = scales[n] * sum_k a[m,k] * q[n,k], q int8 [N,K], fp32 result.
   Device-pointer form of ax_qgemm_w8a32 (include/axiom/quantize.h:75-79,
   src/core/quantize.c:100-177); q/scales/N/K are the fields of ax_qweight_t.
   M = 1 runs the reference's fp32 multiply-adds in a fixed order (layers under 2^24 weights).  Otherwise (K a
   multiple of 16 up to 65536, 16-byte aligned operands) each activation row is first rounded to a fixed-point grid of 2^-30 of its largest
   magnitude and the products are exact integer arithmetic on the tensor cores: the result is within 1e-7 of the
   exact sum and does not depend on summation order; a row that holds an infinity or a NaN comes out as NaN. */
AXB_API int axb_qgemm_w8a32(const float *a, const int8_t *q, const float *scales, float *out,
                    int64_t M, int64_t N, int64_t K);
/* The same call with axiom's own argument list, ax_qgemm_w8a32(a, qw, out, M) (include/axiom/quantize.h:75-79):
   qw points to a HOST struct laid out as ax_qweight_t (quantize.h:50-55) whose data and scales members are DEVICE
   pointers.  Status codes follow the reference (src/core/quantize.c:100-112): NULL_ARG for a NULL argument or
   member, INVALID_SHAPE for non-positive N or K. */
typedef struct {
    int8_t *data;   /* [N, K] int8 rows, device memory */
    float *scales;  /* [N] per-row scale, device memory */
    int64_t N, K;
} axb_qweight_t;
AXB_API int axb_qgemm_w8a32_qw(const float *a, const axb_qweight_t *qw, float *out, int64_t M);

/* The quantised dense layer the reference does not have ("raw kernel", docs/EMBEDDED.md:358: callers add bias and
   activation themselves after ax_qgemm_w8a32): out[m,n] = act(scale[n] * sum_k a[m,k]*q[n,k] + bias[n]), scale,
   bias and activation applied where the sums are finished (no pass over the output).  bias may be NULL; act is AXB_ACT_NONE / AXB_ACT_RELU / AXB_ACT_GELU.  axb_qgemm_w8a32 is this entry with
   no bias and no activation. */
AXB_API int axb_qdense_w8a32(const float *a, const int8_t *q, const float *scales, const float *bias, int act,
                             float *out, int64_t M, int64_t N, int64_t K);
/* W8A8: acc[m,n] = sum_k a_q[m,k] * b_q[n,k] in int32 (exact), then
     out_q[m,n] = clamp(rint(acc * ((a_scale * b_scales[n]) / out_scale)), -127, 127).
   acc_out (int32 [M,N]) and out_q (int8 [M,N]) may each be NULL.
   No counterpart in the reference (it has no int8 x int8 kernel); rounding and
   clamp follow its quantiser, src/core/quantize.c:45-54. */
AXB_API int axb_qgemm_w8a8(const int8_t *a_q, float a_scale, const int8_t *b_q, const float *b_scales,
                   float out_scale, int8_t *out_q, int32_t *acc_out,
                   int64_t M, int64_t N, int64_t K);
/* Per-row symmetric int8 quantiser on the device: scales[n] = absmax/127 (1 for a
   zero row), q = clamp(rint(w / scale)).  (ax_qweight_create_from_fp32,
   src/core/quantize.c:21-57) */
AXB_API int axb_quantize_rows(const float *w, int64_t N, int64_t K, int8_t *q, float *scales);

/* ---- attention ------------------------------------------------------------- */
/* O = softmax(scale * Q.K^T [+ causal mask]) . V per head on head-major
   [BH,S,dk] buffers; L[BH,S] = log-sum-exp per row or NULL.  P_save is NULL or a
   [BH,S,S] buffer that receives the soft-max probabilities (exactly 0 above the
   diagonal when causal), as the stock backend's copy of its score buffer does
   (ops_attention.cu:366-370).  O and L are always computed first by the fused
   kernel, which forms no S x S matrix; a non-NULL P_save costs one more pass
   that writes it from L.  axiom's caller ignores the returned status
   (src/core/attention.c:335-342), so no argument combination may skip O.
   axb_sdpa_bwd never reads the saved probabilities.
   (sdpa_fwd slot of ax_cuda_extension_t, include/axiom/internal/cuda_extension.h:89-92;
   src/compute/backends/cuda/ops_attention.cu:299-392; public CPU form
   ax_fused_attention_fwd[_causal], include/axiom/attention.h:273-280) */
AXB_API int axb_sdpa_fwd(const float *Q, const float *K, const float *V, float *out, float *L,
                 int64_t BH, int64_t S, int64_t dk, float scale, int causal, float *P_save);

/* Slot sdpa_bwd of ax_cuda_extension_t (include/axiom/internal/cuda_extension.h:96-100; reference CUDA
   implementation src/compute/backends/cuda/ops_attention.cu:443-590 with two BH*S*S scratch buffers, CPU
   implementation src/compute/backends/cpu_opt.c:9112-9180).  O, dO: [BH, S, dk]; L: [BH, S] from the forward.
   dQ, dK, dV are OVERWRITTEN (both reference implementations zero them first).  P_saved is accepted and
   ignored: the scores are recomputed block by block and nothing of size S*S is read or written.  dk <= 128. */
AXB_API int axb_sdpa_bwd(const float *Q, const float *K, const float *V, const float *O, const float *dO,
                         const float *L, float *dQ, float *dK, float *dV, int64_t BH, int64_t S, int64_t dk,
                         float scale, int causal, const float *P_saved);

/* ---- attention projections --------------------------------------------------
   Slot qkv_head_gemm of ax_backend_ops_t (include/axiom/internal/backend_ops.h:107-113; ax_compute_qkv_head_gemm,
   include/axiom/compute.h:150-170; CPU implementation src/compute/backends/cpu_opt.c:6160).  The reference CUDA
   backend leaves the slot NULL and runs gemm + k_head_interleave_qkv_split[_bias]
   (src/compute/backends/cuda/ops_attention.cu:74-137).
     qkv = X[B*S, D] . Wqkv[D, 3D] (+ bqkv[3D]),  D = H*dk
     Qh, Kh, Vh [B*H, S, dk] = the three D-wide column blocks of qkv, head-major; all three are overwritten.
   For dk % 32 == 0 the GEMM's epilogue stores head-major itself (one launch, no [B*S, 3D] intermediate). */
AXB_API int axb_qkv_head_gemm(const float *X, const float *Wqkv, const float *bqkv, int64_t B, int64_t S, int64_t H,
                              int64_t dk, float *Qh, float *Kh, float *Vh);
/* Slot dattn_head_gemm_nt of ax_backend_ops_t (include/axiom/internal/backend_ops.h:114-129; ax_compute_dattn_head_gemm_nt,
   src/compute/dispatch.c:553-567; CPU implementation src/compute/backends/cpu_opt.c:6506-6600) — the backward mirror:
     dattn = dout[B*S, D] . Wo[D, D]^T,   dO_head[B*H, S, dk] = dattn stored head-major (overwritten), D = H*dk.
   For dk % 32 == 0 one tensor-core launch whose epilogue stores head-major (no [B*S, D] intermediate); otherwise the
   product into scratch and the layout pass. */
AXB_API int axb_dattn_head_gemm_nt(const float *dout, const float *Wo, int64_t B, int64_t S, int64_t H, int64_t dk,
                                   float *dO_head);
/* Slots dwqkv_split_acc and dwqkv_split_acc_hm of ax_backend_ops_t (include/axiom/internal/backend_ops.h:66-95;
   ax_compute_dwqkv_split_acc[_hm], src/compute/dispatch.c:463-515; CPU implementations
   src/compute/backends/cpu_opt.c:6062-6119; caller mha_backward, src/core/attention.c:805-818) — the weight gradients of
   the fused q|k|v projection, ACCUMULATED into the three [D, D] gradients without a [D, 3D] intermediate:
     dWq += x_flat[rows, D]^T . dQKV[rows, 3D][:, 0:D],   dWk += ... [:, D:2D],   dWv += ... [:, 2D:3D].
   The _hm form takes the three gradients head-major (dQh, dKh, dVh each [B*H, S, dk], rows = B*S, D = H*dk) and gathers
   them into the flat matrix first.  For D % 32 == 0 one tensor-core launch whose epilogue adds each D-wide column block
   to its own destination; otherwise the product into scratch and one accumulating pass.  rows == 0 leaves the
   gradients as they are. */
AXB_API int axb_dwqkv_split_acc(const float *x_flat, const float *dQKV, int64_t rows, int64_t D, float *dWq, float *dWk,
                                float *dWv);
AXB_API int axb_dwqkv_split_acc_hm(const float *x_flat, const float *dQh, const float *dKh, const float *dVh, int64_t B,
                                   int64_t S, int64_t H, int64_t dk, float *dWq, float *dWk, float *dWv);
/* Slot mha_output_proj_fused of ax_backend_ops_t (include/axiom/internal/backend_ops.h:131-150;
   ax_compute_mha_output_proj_fused and ax_compute_output_proj_bwd_fused, src/compute/dispatch.c:577-634; CPU implementation
   src/compute/backends/cpu_opt.c:6819) — the output projection of the attention layer, forward and backward in one call:
     y[rows, D]     = attn_flat[rows, D] . Wo[D, D] + bo[D]      (skipped when y is NULL; bo may be NULL)
     dattn[rows, D] = dout[rows, D] . Wo^T                        (overwritten)
     dWo_acc[D, D] += attn_flat^T . dout                          (accumulated)
     dbo_acc[D]    += column sums of dout                         (accumulated; skipped when dbo_acc is NULL)
   Three tensor-core launches (bias and the accumulation in their epilogues) and, for dbo, one pass of the one-row
   bandwidth-bound route over dout. */
AXB_API int axb_mha_output_proj_fused(const float *attn_flat, const float *Wo, const float *bo, const float *dout, float *y,
                                      float *dattn, float *dWo_acc, float *dbo_acc, int64_t rows, int64_t D);

/* ---- attention layout passes and fused-parameter builders ---------------------
   The remaining attention slots of ax_cuda_extension_t (include/axiom/internal/cuda_extension.h:41-88; stock
   kernels src/compute/backends/cuda/ops_attention.cu:18-211), which axiom's multi-head attention layer calls
   between its GEMMs when its tensors live on a device (src/core/attention.c:234-261,368-375,665-716;
   src/core/attention/cache.c:43-80).  "flat" is the [B*S, H*dk] layout of a projection GEMM, "head-major" is
   [B*H, S, dk].  Each is one pass that reads and writes every element once. */
/* qkv [B*S, 3*H*dk] (+ bqkv[3*H*dk], may be NULL) -> Qh, Kh, Vh head-major   (head_interleave_qkv_split[_bias]) */
AXB_API int axb_head_interleave_qkv_split(const float *qkv, const float *bqkv, float *Qh, float *Kh, float *Vh,
                                          int64_t B, int64_t S, int64_t H, int64_t dk);
/* flat -> head-major                                                          (head_interleave) */
AXB_API int axb_head_interleave(const float *src, float *dst, int64_t B, int64_t S, int64_t H, int64_t dk);
/* head-major -> flat                                                          (head_deinterleave) */
AXB_API int axb_head_deinterleave(const float *src, float *dst, int64_t B, int64_t S, int64_t H, int64_t dk);
/* dQ, dK, dV head-major -> dst [B*S, 3*H*dk]                                  (head_deinterleave_qkv_merge) */
AXB_API int axb_head_deinterleave_qkv_merge(const float *dQ, const float *dK, const float *dV, float *dst, int64_t B,
                                            int64_t S, int64_t H, int64_t dk);
/* dst [D, 3D] = [wq | wk | wv] row by row, each [D, D]                        (qkv_cache_build) */
AXB_API int axb_qkv_cache_build(float *dst, const float *wq, const float *wk, const float *wv, int64_t D);
/* dst [3D] = bq | bk | bv                                                     (bias_cache_build) */
AXB_API int axb_bias_cache_build(float *dst, const float *bq, const float *bk, const float *bv, int64_t D);
/* 1 when p points into device (or managed) memory, else 0.  axiom labels some device buffers as CPU storage
   (the stack views of src/core/attention.c:71-89); the host layer asks the driver instead of trusting the label. */
AXB_API int axb_pointer_on_device(const void *p);

/* ---- convolution as GEMM -----------------------------------------------------
   Slot conv_gemm of ax_backend_ops_t (include/axiom/internal/backend_ops.h:199-202; ax_compute_conv_gemm,
   src/compute/dispatch.c:723; reference CUDA implementation src/compute/backends/cuda/ops_conv.cu:113-215:
   k_im2col_sample into a col buffer, then cuBLAS).  One [C_in, H, W] sample (ax_conv_params_t,
   include/axiom/compute.h:36-43):
     out[C_out, out_h*out_w] = weight[C_out, C_in*kh*kw] . im2col(input),  zero padding ph, pw; strides sh, sw.
   Stride-1 layers whose output width is a multiple of 4 run as an implicit GEMM (the producer of the tensor-core
   kernel reads shifted windows of the channel-innermost image; the padding is TMA's zero fill); for the rest the
   patches are gathered straight into the tensor-core operand planes.  No col matrix is materialised either way. */
AXB_API int axb_conv_gemm(const float *weight, const float *input, int64_t C_out, int64_t C_in, int64_t H, int64_t W,
                          int kh, int kw, int sh, int sw, int ph, int pw, int64_t out_h, int64_t out_w, float *out);
/* Slot conv_gemm_batched of ax_cuda_extension_t (include/axiom/internal/cuda_extension.h:102-108; caller
   src/core/conv/forward.c:529-560; reference implementation src/compute/backends/cuda/ops_conv.cu:213-290: one im2col
   launch per sample into an N*K*M col buffer, then one strided-batched cuBLAS GEMM).  `batch` samples [C_in, H, W]
   back to back in `input`, the filter shared: out[batch][C_out][out_h*out_w].  Stride-1 layers whose output width is
   a multiple of 4 run as ONE implicit GEMM over all samples (the pixels of all samples are its columns); other
   geometries take the samples one by one through axb_conv_gemm.  batch == 0 is a no-op. */
AXB_API int axb_conv_gemm_batched(const float *weight, const float *input, int64_t batch, int64_t C_out, int64_t C_in,
                                  int64_t H, int64_t W, int kh, int kw, int sh, int sw, int ph, int pw, int64_t out_h,
                                  int64_t out_w, float *out);

/* ---- KV cache (autoregressive decode) ---------------------------------------
   Device-pointer forms of ax_kv_cache_append / ax_kv_cache_attend (include/axiom/attention.h:341-381), whose
   only implementation in the reference is the CPU one (src/compute/backends/cpu_opt.c:9586-9654,
   ax_cpu_kv_cache_attend(K_cache, V_cache, Q_new, out, BH, cur_len, max_seq, dk, scale) — the same argument
   list).  K_cache, V_cache: [BH, max_seq, dk]; new_K, new_V, Q_new, out: [BH, dk].  The caller owns cur_len.
   append writes row cur_len of every head (cur_len < max_seq, else AX_ERR_INVALID_SHAPE where the reference
   returns false); attend reads rows [0, cur_len) and, like the reference, leaves out = 0 for an empty cache.
   dk <= 128. */
AXB_API int axb_kv_cache_append(float *K_cache, float *V_cache, const float *new_K, const float *new_V, int64_t BH,
                                int64_t cur_len, int64_t max_seq, int64_t dk);
AXB_API int axb_kv_cache_attend(const float *K_cache, const float *V_cache, const float *Q_new, float *out,
                                int64_t BH, int64_t cur_len, int64_t max_seq, int64_t dk, float scale);

#ifdef __cplusplus
}
#endif
#endif /* AXIOM_B200_H */
