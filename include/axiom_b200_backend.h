/* axiom_b200_backend.h — the axiom plug-in tables, as filled by libaxiom_b200_backend.so.

   axiom (v0.10.0) talks to a compute backend through two tables of function
   pointers: `ax_backend_ops_t` (include/axiom/internal/backend_ops.h:30-298) and
   `ax_cuda_extension_t` (include/axiom/internal/cuda_extension.h:41-130), whose
   operands are `ax_tensor_t` / `ax_storage_t` (include/axiom/tensor.h:29-70).
   This header describes the same binary layouts under `axb_`-prefixed names so
   that the host layer can be compiled without the axiom tree and so that both
   sets of headers can be included in one translation unit (tests do that to
   check every offset with _Static_assert).  Slots this engine does not provide
   are kept as opaque pointers so the layout stays identical; they are NULL in
   the exported table. */
#ifndef AXIOM_B200_BACKEND_H
#define AXIOM_B200_BACKEND_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AXB_AX_MAX_DIMS 8        /* AX_MAX_DIMS, include/axiom/types.h */
#define AXB_AX_FLOAT32 0         /* ax_dtype_t, include/axiom/types.h:52-60 */
#define AXB_AX_DEVICE_CPU 0      /* ax_device_t, include/axiom/types.h:105-110 */
#define AXB_AX_DEVICE_CUDA 1
#define AXB_AX_BACKEND_CUDA 3    /* ax_backend_id_t, include/axiom/compute.h:46-52 */

/* ax_storage_t (include/axiom/tensor.h:29-45) */
typedef struct {
    void *data;
    size_t size_bytes;
    int refcount;          /* atomic_int in axiom */
    int device;            /* ax_device_t */
    bool is_arena_temp;
    uint64_t generation;
} axb_ax_storage_t;

/* ax_tensor_t (include/axiom/tensor.h:53-70) */
typedef struct axb_ax_tensor {
    axb_ax_storage_t *storage;
    int64_t shape[AXB_AX_MAX_DIMS];
    int64_t strides[AXB_AX_MAX_DIMS];   /* in elements */
    int ndim;
    int dtype;                          /* ax_dtype_t */
    int64_t offset;                     /* in elements */
    bool requires_grad;
    struct axb_ax_tensor *grad;
    void *grad_fn;
    int layout;                         /* ax_layout_t */
} axb_ax_tensor_t;

/* ax_conv_params_t (include/axiom/compute.h:36-43): one [C_in, H, W] sample plus the kernel geometry */
typedef struct {
    const float *input;
    int64_t C_in, H, W;
    int kh, kw;
    int sh, sw;
    int ph, pw;
    int64_t out_h, out_w;
} axb_ax_conv_params_t;

typedef void (*axb_opaque_fn)(void);    /* a slot this engine leaves NULL */
typedef int axb_status;                 /* ax_status_t */

/* ax_backend_ops_t: one member per slot of the reference struct, in its order. */
typedef struct {
    const char *name;
    axb_opaque_fn add, sub, mul, div_op;
    axb_opaque_fn neg, abs_op, exp_op, log_op, sqrt_op, square;
    axb_opaque_fn add_scalar, mul_scalar;
    axb_status (*gemm)(const axb_ax_tensor_t *a, const axb_ax_tensor_t *b, axb_ax_tensor_t *out);
    axb_status (*gemm_nt)(const axb_ax_tensor_t *a, const axb_ax_tensor_t *b, axb_ax_tensor_t *out);
    axb_status (*gemm_tn)(const axb_ax_tensor_t *a, const axb_ax_tensor_t *b, axb_ax_tensor_t *out);
    axb_status (*dwqkv_split_acc)(const axb_ax_tensor_t *x_flat, const axb_ax_tensor_t *dQKV, axb_ax_tensor_t *dWq,
                                  axb_ax_tensor_t *dWk, axb_ax_tensor_t *dWv);   /* backend_ops.h:66-80 */
    axb_status (*dwqkv_split_acc_hm)(const axb_ax_tensor_t *x_flat, const axb_ax_tensor_t *dQh, const axb_ax_tensor_t *dKh,
                                     const axb_ax_tensor_t *dVh, int64_t B, int64_t S, int64_t H, int64_t dk,
                                     axb_ax_tensor_t *dWq, axb_ax_tensor_t *dWk, axb_ax_tensor_t *dWv);   /* backend_ops.h:82-95 */
    axb_status (*qkv_head_gemm)(const axb_ax_tensor_t *X, const axb_ax_tensor_t *Wqkv, const axb_ax_tensor_t *bqkv,
                                int64_t B, int64_t S, int64_t H, int64_t dk, axb_ax_tensor_t *Qh, axb_ax_tensor_t *Kh,
                                axb_ax_tensor_t *Vh);   /* backend_ops.h:107-113 */
    axb_status (*dattn_head_gemm_nt)(const axb_ax_tensor_t *dout, const axb_ax_tensor_t *Wo, int64_t B, int64_t S, int64_t H,
                                     int64_t dk, axb_ax_tensor_t *dO_head);   /* backend_ops.h:114-129 */
    axb_status (*mha_output_proj_fused)(const axb_ax_tensor_t *attn_flat, const axb_ax_tensor_t *Wo, const axb_ax_tensor_t *bo,
                                        const axb_ax_tensor_t *dout, axb_ax_tensor_t *y, axb_ax_tensor_t *dattn,
                                        axb_ax_tensor_t *dWo_acc, axb_ax_tensor_t *dbo_acc);   /* backend_ops.h:131-150 */
    axb_status (*gemm_relu)(const axb_ax_tensor_t *a, const axb_ax_tensor_t *b, const axb_ax_tensor_t *bias,
                            axb_ax_tensor_t *out);
    axb_status (*gemm_ex)(const axb_ax_tensor_t *a, const axb_ax_tensor_t *b, float alpha, float beta,
                          axb_ax_tensor_t *out);
    axb_opaque_fn add_relu, axpy, softmax_rowwise;
    axb_status (*bias_add)(const axb_ax_tensor_t *in, const axb_ax_tensor_t *bias, int axis, axb_ax_tensor_t *out);
    axb_status (*conv_gemm)(const axb_ax_tensor_t *weight, const axb_ax_conv_params_t *params, axb_ax_tensor_t *out);
    axb_opaque_fn conv_gemm_nt_dw;
    axb_opaque_fn sum, mean, max_op, min_op, argmax;
    axb_opaque_fn equal, greater;
    axb_opaque_fn fill, copy;
    axb_status (*relu)(const axb_ax_tensor_t *in, axb_ax_tensor_t *out);
    axb_opaque_fn sigmoid, tanh_op, leaky_relu, elu_op;
    axb_status (*gelu_op)(const axb_ax_tensor_t *in, axb_ax_tensor_t *out);
    axb_opaque_fn swish_op, adam_update, sgd_update;
    int device;                          /* ax_device_t this backend owns */
    axb_status (*init)(void);
    void (*shutdown)(void);
    void (*synchronize)(void);
    int (*device_count)(void);
    void *(*storage_alloc)(size_t size_bytes);
    void (*storage_free)(void *ptr);
    axb_status (*memcpy_h2d)(void *dst, const void *src, size_t bytes);
    axb_status (*memcpy_d2h)(void *dst, const void *src, size_t bytes);
    axb_status (*memcpy_d2d)(void *dst, const void *src, size_t bytes);
} axb_ax_backend_ops_t;

/* ax_cuda_extension_t (include/axiom/internal/cuda_extension.h:41-130): everything the attention layer calls on a
   device — the five head-layout passes, the two fused-parameter builders, sdpa_fwd and sdpa_bwd — is provided, and the
   batched convolution; the Winograd slots stay NULL (callers test them). */
typedef struct {
    void (*head_interleave_qkv_split)(const float *src, float *q, float *k, float *v, int64_t B, int64_t S, int64_t H,
                                      int64_t dk, int64_t D);
    void (*head_interleave_qkv_split_bias)(const float *src, const float *bqkv, float *q, float *k, float *v, int64_t B,
                                           int64_t S, int64_t H, int64_t dk, int64_t D);
    void (*head_interleave)(const float *src, float *dst, int64_t B, int64_t S, int64_t H, int64_t dk);
    void (*head_deinterleave)(const float *src, float *dst, int64_t B, int64_t S, int64_t H, int64_t dk);
    void (*head_deinterleave_qkv_merge)(const float *dQ, const float *dK, const float *dV, float *dst, int64_t B,
                                        int64_t S, int64_t H, int64_t dk, int64_t D);
    axb_status (*qkv_cache_build)(float *dst, const float *wq, const float *wk, const float *wv, int64_t D);
    axb_status (*bias_cache_build)(float *dst, const float *bq, const float *bk, const float *bv, int64_t D);
    axb_status (*sdpa_fwd)(const float *Q, const float *K, const float *V, float *out, float *L, int64_t BH,
                           int64_t S, int64_t dk, float scale, bool causal, float *P_save);
    axb_status (*sdpa_bwd)(const float *Q, const float *K, const float *V, const float *O, const float *dO,
                           const float *L, float *dQ, float *dK, float *dV, int64_t BH, int64_t S, int64_t dk,
                           float scale, bool causal, const float *P_saved);
    axb_status (*conv_gemm_batched)(const axb_ax_tensor_t *weight, const float *in_dev, int64_t N,
                                    const axb_ax_conv_params_t *single, axb_ax_tensor_t *out);
    axb_opaque_fn conv_winograd_f23, winograd_f23_prefer;
} axb_ax_cuda_extension_t;

#define AXB_BACKEND_API __attribute__((visibility("default")))

/* The tables.  Cast to `const ax_backend_ops_t *` / `const ax_cuda_extension_t *` on the
   axiom side (same layout) and hand them to ax_compute_register_backend(AX_BACKEND_CUDA, ...)
   (src/compute/dispatch.c:302-315) and ax_compute_register_cuda_extension (dispatch.c:290-296). */
AXB_BACKEND_API const axb_ax_backend_ops_t *axb_backend_ops(void);
AXB_BACKEND_API const axb_ax_cuda_extension_t *axb_cuda_extension(void);

/* Optional hooks into the host framework:
   skip_init  returns non-zero while the caller wants gemm/gemm_nt/gemm_tn to ACCUMULATE into
              `out` (axiom's ax_gemm_get_skip_init(), src/compute/dispatch.c:1284-1285);
   set_err    receives every failure (axiom's ax_err_set, src/core/error.c:23-38). */
AXB_BACKEND_API void axb_backend_set_hooks(int (*skip_init)(void), void (*set_err)(int status, const char *msg));

#ifdef __cplusplus
}
#endif
#endif /* AXIOM_B200_BACKEND_H */
