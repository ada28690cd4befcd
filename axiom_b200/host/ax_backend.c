/* ax_backend.c — the host side of the drop-in: axiom's backend vtable and CUDA
   extension table, filled in plain C on top of the C ABI of libaxiom_b200.so.

   Each function does what the corresponding function of the reference CUDA
   backend does before it reaches its kernel — validate the tensors, resolve
   `(float *)storage->data + offset`, read the sizes (for example
   src/compute/backends/cuda/ops_gemm.cu:15-37) — and then makes exactly one
   call into the engine.  No arithmetic happens here. */
#include "axiom_b200_backend.h"
#include "axiom_b200.h"

#include <stdio.h>

/* axiom status codes used below (include/axiom/types.h:89-103) */
enum { ST_OK = 0, ST_NULL_ARG = 1, ST_SHAPE = 3, ST_DTYPE = 4, ST_AXIS = 5, ST_INVALID_SHAPE = 6, ST_BACKEND = 9 };

static int (*hook_skip_init)(void);
static void (*hook_set_err)(int, const char *);

void axb_backend_set_hooks(int (*skip_init)(void), void (*set_err)(int status, const char *msg))
{
    hook_skip_init = skip_init;
    hook_set_err = set_err;
}

static axb_status report(axb_status st, const char *msg)
{
    if (st != ST_OK && hook_set_err) hook_set_err(st, msg);
    return st;
}

/* forward the engine's status together with its message */
static axb_status done(int st)
{
    return st == AXB_OK ? ST_OK : report(st, axb_last_error());
}

static int64_t numel(const axb_ax_tensor_t *t)
{
    int64_t n = 1;
    for (int i = 0; i < t->ndim; ++i) n *= t->shape[i];
    return n;
}

static int is_contiguous(const axb_ax_tensor_t *t)
{
    int64_t expect = 1;
    for (int i = t->ndim - 1; i >= 0; --i) {
        if (t->shape[i] != 1 && t->strides[i] != expect) return 0;
        expect *= t->shape[i];
    }
    return 1;
}

/* the reference's contract for every GEMM slot: fp32, contiguous, resident on the device */
static axb_status check_f32(const axb_ax_tensor_t *t, const char *what, int want_ndim)
{
    char msg[160];
    if (!t || !t->storage) {
        snprintf(msg, sizeof msg, "%s: NULL tensor", what);
        return report(ST_NULL_ARG, msg);
    }
    if (t->dtype != AXB_AX_FLOAT32) {
        snprintf(msg, sizeof msg, "%s: only float32 is supported", what);
        return report(ST_DTYPE, msg);
    }
    if (want_ndim > 0 && t->ndim != want_ndim) {
        snprintf(msg, sizeof msg, "%s: expected a %d-d tensor, got %d-d", what, want_ndim, t->ndim);
        return report(ST_SHAPE, msg);
    }
    if (!is_contiguous(t)) {
        snprintf(msg, sizeof msg, "%s: tensor must be contiguous", what);
        return report(ST_INVALID_SHAPE, msg);
    }
    /* axiom's attention layer wraps device buffers in stack views whose storage says CPU
       (mha_make_stack_view, src/core/attention.c:71-89), and the stock CUDA backend never looks at the field
       (src/compute/backends/cuda/ops_gemm.cu:15-27): trust the pointer, not the label, but never hand host
       memory to a kernel */
    if (t->storage->device != AXB_AX_DEVICE_CUDA && !axb_pointer_on_device(t->storage->data)) {
        snprintf(msg, sizeof msg, "%s: tensor is not on the CUDA device", what);
        return report(ST_BACKEND, msg);
    }
    return ST_OK;
}

static float *fptr(const axb_ax_tensor_t *t) { return (float *)t->storage->data + t->offset; }

/* ---- prepared-weight cache ------------------------------------------------------------------------------
   A dense layer hands the same weight tensor to `gemm` call after call.  The engine can keep a weight's
   tensor-core operand planes (axb_weight_prepare), so the second time a right-hand operand is seen with the
   same storage, generation counter and shape it is prepared, and from then on only the left operand is split.
   This is what axiom's own cpu_opt backend does with its packed-B cache, under the same contract: every
   in-place write to a tensor bumps its storage's generation (ax_storage_touch; the dispatcher does it for every
   op's output, src/compute/dispatch.c:347-350).  Writes that reach the device through this backend's own copy
   hooks and frees through its free hook drop the entries they touch.  Results are bit-identical with and
   without the cache. */
enum { WCACHE_SLOTS = 8 };
static const size_t WCACHE_MAX_BYTES = (size_t)2 << 30;   /* operand planes kept at most */
static const int64_t WCACHE_MIN_ELEMS = 1 << 16;          /* smaller weights are not worth a handle */

typedef struct {
    const void *data;     /* storage->data (+ offset folded into ptr below) */
    const float *ptr;
    uint64_t generation;
    int64_t K, N;
    axb_weight_t *w;      /* NULL: seen once, not prepared yet */
    size_t bytes;
    uint64_t stamp;
} wcache_entry;

static wcache_entry wcache[WCACHE_SLOTS];
static uint64_t wcache_clock;
static size_t wcache_bytes;

static void wcache_drop(wcache_entry *e)
{
    if (e->w) {
        axb_weight_release(e->w);
        wcache_bytes -= e->bytes;
    }
    e->data = NULL; e->ptr = NULL; e->w = NULL; e->bytes = 0; e->stamp = 0;
}

/* drops what lies in [lo, lo + bytes) or belongs to the storage whose base is lo */
static void wcache_drop_range(const void *lo, size_t bytes)
{
    const char *a = (const char *)lo, *b = a + (bytes ? bytes : 1);
    for (int i = 0; i < WCACHE_SLOTS; ++i) {
        wcache_entry *e = &wcache[i];
        if (!e->ptr) continue;
        const char *p = (const char *)e->ptr, *q = p + (size_t)(e->K * e->N) * sizeof(float);
        if (e->data == lo || (p < b && a < q)) wcache_drop(e);
    }
}

static void wcache_clear(void)
{
    for (int i = 0; i < WCACHE_SLOTS; ++i)
        if (wcache[i].ptr) wcache_drop(&wcache[i]);
}

/* the prepared form of right-hand operand b [K,N], or NULL (not seen before, too small, no room) */
static const axb_weight_t *wcache_lookup(const axb_ax_tensor_t *b, int64_t K, int64_t N)
{
    if (K * N < WCACHE_MIN_ELEMS) return NULL;
    const float *ptr = fptr(b);
    wcache_entry *hit = NULL, *victim = NULL;
    for (int i = 0; i < WCACHE_SLOTS; ++i) {
        wcache_entry *e = &wcache[i];
        if (e->ptr == ptr && e->K == K && e->N == N) hit = e;
        /* the slot a newcomer takes: an empty one, else the least recently used */
        if (!victim || (victim->ptr && (!e->ptr || e->stamp < victim->stamp))) victim = e;
    }
    if (hit && hit->generation != b->storage->generation) {   /* written since: start over */
        wcache_drop(hit);
        hit = NULL;
    }
    if (!hit) {                                                /* first sighting: remember it, prepare next time */
        if (victim->ptr) wcache_drop(victim);
        victim->data = b->storage->data; victim->ptr = ptr; victim->generation = b->storage->generation;
        victim->K = K; victim->N = N; victim->w = NULL; victim->bytes = 0; victim->stamp = ++wcache_clock;
        return NULL;
    }
    hit->stamp = ++wcache_clock;
    if (!hit->w) {
        const size_t bytes = (size_t)(K * N) * 8;              /* upper bound: two fp32-sized planes */
        while (wcache_bytes + bytes > WCACHE_MAX_BYTES) {
            wcache_entry *old = NULL;
            for (int i = 0; i < WCACHE_SLOTS; ++i)
                if (wcache[i].w && &wcache[i] != hit && (!old || wcache[i].stamp < old->stamp)) old = &wcache[i];
            if (!old) return NULL;
            wcache_drop(old);
        }
        if (axb_weight_prepare(ptr, K, N, 0, &hit->w) != AXB_OK) {
            hit->w = NULL;
            return NULL;
        }
        hit->bytes = bytes;
        wcache_bytes += bytes;
    }
    return hit->w;
}

/* shared body of gemm / gemm_nt / gemm_tn / gemm_relu / gemm_ex */
static axb_status gemm_common(const char *what, const axb_ax_tensor_t *a, const axb_ax_tensor_t *b,
                              const axb_ax_tensor_t *bias, axb_ax_tensor_t *out, int ta, int tb, float alpha,
                              float beta, int act)
{
    axb_status st;
    if ((st = check_f32(a, what, 2)) || (st = check_f32(b, what, 2)) || (st = check_f32(out, what, 2))) return st;
    const int64_t M = ta ? a->shape[1] : a->shape[0];
    const int64_t K = ta ? a->shape[0] : a->shape[1];
    const int64_t Kb = tb ? b->shape[1] : b->shape[0];
    const int64_t N = tb ? b->shape[0] : b->shape[1];
    if (K != Kb || out->shape[0] != M || out->shape[1] != N) {
        char msg[200];
        snprintf(msg, sizeof msg, "%s shape mismatch: op(a)=[%lld,%lld] op(b)=[%lld,%lld] out=[%lld,%lld]", what,
                 (long long)M, (long long)K, (long long)Kb, (long long)N, (long long)out->shape[0],
                 (long long)out->shape[1]);
        return report(ST_SHAPE, msg);
    }
    const float *bias_p = NULL;
    if (bias) {
        if ((st = check_f32(bias, what, 1))) return st;
        if (bias->shape[0] != N) return report(ST_SHAPE, "gemm bias length must equal the output columns");
        bias_p = fptr(bias);
    }
    if (!ta && !tb && M > 32) {
        const axb_weight_t *w = wcache_lookup(b, K, N);
        if (w) return done(axb_gemm_prepared(fptr(a), w, bias_p, fptr(out), M, 0, alpha, beta, act));
    }
    return done(axb_gemm_bias_act(fptr(a), fptr(b), bias_p, fptr(out), M, N, K, ta, tb, alpha, beta, act));
}

static float accumulate_beta(void) { return (hook_skip_init && hook_skip_init()) ? 1.0f : 0.0f; }

static axb_status be_gemm(const axb_ax_tensor_t *a, const axb_ax_tensor_t *b, axb_ax_tensor_t *out)
{
    return gemm_common("gemm", a, b, NULL, out, 0, 0, 1.0f, accumulate_beta(), AXB_ACT_NONE);
}

static axb_status be_gemm_nt(const axb_ax_tensor_t *a, const axb_ax_tensor_t *b, axb_ax_tensor_t *out)
{
    return gemm_common("gemm_nt", a, b, NULL, out, 0, 1, 1.0f, accumulate_beta(), AXB_ACT_NONE);
}

static axb_status be_gemm_tn(const axb_ax_tensor_t *a, const axb_ax_tensor_t *b, axb_ax_tensor_t *out)
{
    return gemm_common("gemm_tn", a, b, NULL, out, 1, 0, 1.0f, accumulate_beta(), AXB_ACT_NONE);
}

static axb_status be_gemm_relu(const axb_ax_tensor_t *a, const axb_ax_tensor_t *b, const axb_ax_tensor_t *bias,
                               axb_ax_tensor_t *out)
{
    return gemm_common("gemm_relu", a, b, bias, out, 0, 0, 1.0f, 0.0f, AXB_ACT_RELU);
}

static axb_status be_gemm_ex(const axb_ax_tensor_t *a, const axb_ax_tensor_t *b, float alpha, float beta,
                             axb_ax_tensor_t *out)
{
    return gemm_common("gemm_ex", a, b, NULL, out, 0, 0, alpha, beta, AXB_ACT_NONE);
}

/* shape rules of the reference's CPU implementation (src/compute/backends/cpu_opt.c:6165-6189) */
static axb_status be_qkv_head_gemm(const axb_ax_tensor_t *X, const axb_ax_tensor_t *Wqkv, const axb_ax_tensor_t *bqkv,
                                   int64_t B, int64_t S, int64_t H, int64_t dk, axb_ax_tensor_t *Qh, axb_ax_tensor_t *Kh,
                                   axb_ax_tensor_t *Vh)
{
    axb_status st;
    if ((st = check_f32(X, "qkv_head_gemm", 2)) || (st = check_f32(Wqkv, "qkv_head_gemm", 2)) ||
        (st = check_f32(Qh, "qkv_head_gemm", 3)) || (st = check_f32(Kh, "qkv_head_gemm", 3)) ||
        (st = check_f32(Vh, "qkv_head_gemm", 3)))
        return st;
    const int64_t D = X->shape[1];
    if (X->shape[0] != B * S || D != H * dk || Wqkv->shape[0] != D || Wqkv->shape[1] != 3 * D)
        return report(ST_SHAPE, "qkv_head_gemm: X must be [B*S, H*dk] and Wqkv [H*dk, 3*H*dk]");
    const axb_ax_tensor_t *outs[3] = { Qh, Kh, Vh };
    for (int i = 0; i < 3; ++i)
        if (outs[i]->shape[0] != B * H || outs[i]->shape[1] != S || outs[i]->shape[2] != dk)
            return report(ST_SHAPE, "qkv_head_gemm: Qh, Kh, Vh must be [B*H, S, dk]");
    const float *bias_p = NULL;
    if (bqkv) {
        if ((st = check_f32(bqkv, "qkv_head_gemm", 1))) return st;
        if (bqkv->shape[0] != 3 * D) return report(ST_SHAPE, "qkv_head_gemm: bqkv must have 3*H*dk elements");
        bias_p = fptr(bqkv);
    }
    return done(axb_qkv_head_gemm(fptr(X), fptr(Wqkv), bias_p, B, S, H, dk, fptr(Qh), fptr(Kh), fptr(Vh)));
}

/* shape rules of the CPU implementation (src/compute/backends/cpu_opt.c:6527-6560) */
static axb_status be_dattn_head_gemm_nt(const axb_ax_tensor_t *dout, const axb_ax_tensor_t *Wo, int64_t B, int64_t S, int64_t H,
                                        int64_t dk, axb_ax_tensor_t *dO_head)
{
    axb_status st;
    if ((st = check_f32(dout, "dattn_head_gemm_nt", 2)) || (st = check_f32(Wo, "dattn_head_gemm_nt", 2)) ||
        (st = check_f32(dO_head, "dattn_head_gemm_nt", 3)))
        return st;
    const int64_t D = H * dk;
    if (dout->shape[0] != B * S || dout->shape[1] != D || Wo->shape[0] != D || Wo->shape[1] != D)
        return report(ST_SHAPE, "dattn_head_gemm_nt: dout must be [B*S, H*dk] and Wo [H*dk, H*dk]");
    if (dO_head->shape[0] != B * H || dO_head->shape[1] != S || dO_head->shape[2] != dk)
        return report(ST_SHAPE, "dattn_head_gemm_nt: dO_head must be [B*H, S, dk]");
    return done(axb_dattn_head_gemm_nt(fptr(dout), fptr(Wo), B, S, H, dk, fptr(dO_head)));
}

/* shape rules of the CPU implementations (src/compute/backends/cpu_opt.c:6062-6119) */
static axb_status check_dw3(const char *what, int64_t D, axb_ax_tensor_t *dWq, axb_ax_tensor_t *dWk, axb_ax_tensor_t *dWv)
{
    axb_status st;
    if ((st = check_f32(dWq, what, 2)) || (st = check_f32(dWk, what, 2)) || (st = check_f32(dWv, what, 2))) return st;
    if (dWq->shape[0] != D || dWq->shape[1] != D || dWk->shape[0] != D || dWk->shape[1] != D || dWv->shape[0] != D ||
        dWv->shape[1] != D)
        return report(ST_SHAPE, "dwqkv_split_acc: the three gradients must be [D, D]");
    return 0;
}

static axb_status be_dwqkv_split_acc(const axb_ax_tensor_t *x_flat, const axb_ax_tensor_t *dQKV, axb_ax_tensor_t *dWq,
                                     axb_ax_tensor_t *dWk, axb_ax_tensor_t *dWv)
{
    axb_status st;
    if ((st = check_f32(x_flat, "dwqkv_split_acc", 2)) || (st = check_f32(dQKV, "dwqkv_split_acc", 2))) return st;
    const int64_t rows = x_flat->shape[0], D = x_flat->shape[1];
    if (dQKV->shape[0] != rows || dQKV->shape[1] != 3 * D)
        return report(ST_SHAPE, "dwqkv_split_acc: dQKV must be [rows, 3*D] for x_flat [rows, D]");
    if ((st = check_dw3("dwqkv_split_acc", D, dWq, dWk, dWv))) return st;
    return done(axb_dwqkv_split_acc(fptr(x_flat), fptr(dQKV), rows, D, fptr(dWq), fptr(dWk), fptr(dWv)));
}

static axb_status be_dwqkv_split_acc_hm(const axb_ax_tensor_t *x_flat, const axb_ax_tensor_t *dQh, const axb_ax_tensor_t *dKh,
                                        const axb_ax_tensor_t *dVh, int64_t B, int64_t S, int64_t H, int64_t dk,
                                        axb_ax_tensor_t *dWq, axb_ax_tensor_t *dWk, axb_ax_tensor_t *dWv)
{
    axb_status st;
    if ((st = check_f32(x_flat, "dwqkv_split_acc_hm", 2)) || (st = check_f32(dQh, "dwqkv_split_acc_hm", 3)) ||
        (st = check_f32(dKh, "dwqkv_split_acc_hm", 3)) || (st = check_f32(dVh, "dwqkv_split_acc_hm", 3)))
        return st;
    const int64_t D = H * dk;
    if (x_flat->shape[0] != B * S || x_flat->shape[1] != D)
        return report(ST_SHAPE, "dwqkv_split_acc_hm: x_flat must be [B*S, H*dk]");
    const axb_ax_tensor_t *hm[3] = { dQh, dKh, dVh };
    for (int i = 0; i < 3; i++)
        if (hm[i]->shape[0] != B * H || hm[i]->shape[1] != S || hm[i]->shape[2] != dk)
            return report(ST_SHAPE, "dwqkv_split_acc_hm: dQh, dKh, dVh must be [B*H, S, dk]");
    if ((st = check_dw3("dwqkv_split_acc_hm", D, dWq, dWk, dWv))) return st;
    return done(axb_dwqkv_split_acc_hm(fptr(x_flat), fptr(dQh), fptr(dKh), fptr(dVh), B, S, H, dk, fptr(dWq), fptr(dWk),
                                       fptr(dWv)));
}

/* shape rules of the CPU implementation (src/compute/backends/cpu_opt.c:6825-6857): y, bo and dbo_acc are optional */
static axb_status be_mha_output_proj_fused(const axb_ax_tensor_t *attn_flat, const axb_ax_tensor_t *Wo, const axb_ax_tensor_t *bo,
                                           const axb_ax_tensor_t *dout, axb_ax_tensor_t *y, axb_ax_tensor_t *dattn,
                                           axb_ax_tensor_t *dWo_acc, axb_ax_tensor_t *dbo_acc)
{
    static const char what[] = "mha_output_proj_fused";
    axb_status st;
    if ((st = check_f32(attn_flat, what, 2)) || (st = check_f32(Wo, what, 2)) || (st = check_f32(dout, what, 2)) ||
        (st = check_f32(dattn, what, 2)) || (st = check_f32(dWo_acc, what, 2)))
        return st;
    if ((y && (st = check_f32(y, what, 2))) || (bo && (st = check_f32(bo, what, 1))) || (dbo_acc && (st = check_f32(dbo_acc, what, 1))))
        return st;
    const int64_t rows = attn_flat->shape[0], D = attn_flat->shape[1];
    if (Wo->shape[0] != D || Wo->shape[1] != D || dout->shape[0] != rows || dout->shape[1] != D || dattn->shape[0] != rows ||
        dattn->shape[1] != D || dWo_acc->shape[0] != D || dWo_acc->shape[1] != D || (y && (y->shape[0] != rows || y->shape[1] != D)) ||
        (bo && bo->shape[0] != D) || (dbo_acc && dbo_acc->shape[0] != D))
        return report(ST_SHAPE, "mha_output_proj_fused: attn_flat, dout, y, dattn [rows, D]; Wo, dWo_acc [D, D]; bo, dbo_acc [D]");
    return done(axb_mha_output_proj_fused(fptr(attn_flat), fptr(Wo), (y && bo) ? fptr(bo) : NULL, fptr(dout), y ? fptr(y) : NULL,
                                          fptr(dattn), fptr(dWo_acc), dbo_acc ? fptr(dbo_acc) : NULL, rows, D));
}

/* shape rules of the reference's CUDA implementation (src/compute/backends/cuda/ops_conv.cu:113-142); params->input
   is a raw pointer into the (device-resident) batched input, as the conv layer passes it */
static axb_status be_conv_gemm(const axb_ax_tensor_t *weight, const axb_ax_conv_params_t *params, axb_ax_tensor_t *out)
{
    axb_status st;
    if (!params || !params->input) return report(ST_NULL_ARG, "conv_gemm: NULL params");
    if ((st = check_f32(weight, "conv_gemm", 2)) || (st = check_f32(out, "conv_gemm", 2))) return st;
    const int64_t C_out = weight->shape[0], K = weight->shape[1], M = params->out_h * params->out_w;
    if (K != params->C_in * params->kh * params->kw) return report(ST_SHAPE, "conv_gemm: weight columns must equal C_in*kh*kw");
    if (out->shape[0] != C_out || out->shape[1] != M) return report(ST_SHAPE, "conv_gemm: out must be [C_out, out_h*out_w]");
    return done(axb_conv_gemm(fptr(weight), params->input, C_out, params->C_in, params->H, params->W, params->kh, params->kw,
                              params->sh, params->sw, params->ph, params->pw, params->out_h, params->out_w, fptr(out)));
}

/* shape rules of the reference's CUDA implementation (src/compute/backends/cuda/ops_fused.cu:268-292): any rank,
   bias 1-d of length in->shape[axis], broadcast along that axis */
static axb_status be_bias_add(const axb_ax_tensor_t *in, const axb_ax_tensor_t *bias, int axis, axb_ax_tensor_t *out)
{
    axb_status st;
    if ((st = check_f32(in, "bias_add", 0)) || (st = check_f32(out, "bias_add", 0)) ||
        (st = check_f32(bias, "bias_add", 1)))
        return st;
    if (axis < 0) axis += in->ndim;
    if (axis < 0 || axis >= in->ndim) return report(ST_AXIS, "bias_add: axis out of range");
    if (out->ndim != in->ndim) return report(ST_SHAPE, "bias_add: out must have the shape of in");
    for (int d = 0; d < in->ndim; ++d)
        if (out->shape[d] != in->shape[d]) return report(ST_SHAPE, "bias_add: out must have the shape of in");
    if (bias->shape[0] != in->shape[axis]) return report(ST_SHAPE, "bias_add: bias length must equal in->shape[axis]");
    int64_t outer = 1, inner = 1;
    for (int d = 0; d < axis; ++d) outer *= in->shape[d];
    for (int d = axis + 1; d < in->ndim; ++d) inner *= in->shape[d];
    return done(axb_bias_add_nd(fptr(in), fptr(bias), fptr(out), outer, in->shape[axis], inner));
}

static axb_status unary(const char *what, const axb_ax_tensor_t *in, axb_ax_tensor_t *out, int gelu)
{
    axb_status st;
    if ((st = check_f32(in, what, 0)) || (st = check_f32(out, what, 0))) return st;
    if (numel(in) != numel(out)) return report(ST_SHAPE, "unary op: in and out must have the same number of elements");
    return done(gelu ? axb_gelu(fptr(in), fptr(out), numel(in)) : axb_relu(fptr(in), fptr(out), numel(in)));
}

static axb_status be_relu(const axb_ax_tensor_t *in, axb_ax_tensor_t *out) { return unary("relu", in, out, 0); }
static axb_status be_gelu(const axb_ax_tensor_t *in, axb_ax_tensor_t *out) { return unary("gelu", in, out, 1); }

/* ---- device-owner hooks (src/compute/backends/cuda/backend.cu:56-116, memory.cu:80-140) ---- */

static axb_status be_init(void) { return done(axb_init(-1)); }
static void be_shutdown(void)
{
    wcache_clear();
    axb_shutdown();
}
static void be_synchronize(void)
{
    axb_synchronize();
    if (axb_device_error() != 0) report(ST_BACKEND, axb_last_error());
}
static int be_device_count(void) { return axb_device_count(); }
static void *be_alloc(size_t bytes) { return axb_storage_alloc(bytes); }
static void be_free(void *p)
{
    if (p) wcache_drop_range(p, 1);   /* entries are keyed on pointers into live storage */
    axb_storage_free(p);
}
static axb_status be_h2d(void *dst, const void *src, size_t bytes)
{
    wcache_drop_range(dst, bytes);
    return done(axb_memcpy_h2d(dst, src, bytes));
}
static axb_status be_d2h(void *dst, const void *src, size_t bytes) { return done(axb_memcpy_d2h(dst, src, bytes)); }
static axb_status be_d2d(void *dst, const void *src, size_t bytes)
{
    wcache_drop_range(dst, bytes);
    return done(axb_memcpy_d2d(dst, src, bytes));
}

static axb_status ext_sdpa_fwd(const float *Q, const float *K, const float *V, float *out, float *L, int64_t BH,
                               int64_t S, int64_t dk, float scale, bool causal, float *P_save)
{
    return done(axb_sdpa_fwd(Q, K, V, out, L, BH, S, dk, scale, causal ? 1 : 0, P_save));
}

static axb_status ext_sdpa_bwd(const float *Q, const float *K, const float *V, const float *O, const float *dO,
                               const float *L, float *dQ, float *dK, float *dV, int64_t BH, int64_t S, int64_t dk,
                               float scale, bool causal, const float *P_saved)
{
    return done(axb_sdpa_bwd(Q, K, V, O, dO, L, dQ, dK, dV, BH, S, dk, scale, causal ? 1 : 0, P_saved));
}

/* ---- attention layout slots (include/axiom/internal/cuda_extension.h:41-88).  The five layout slots return
   void in axiom; a failure reaches the caller through the error hook only, as with the stock kernels' launch
   errors.  D is redundant (D = H*dk at every call site, src/core/attention.c:236-261,700-716). ---- */

static int d_matches(const char *what, int64_t H, int64_t dk, int64_t D)
{
    if (D == H * dk) return 1;
    char msg[120];
    snprintf(msg, sizeof msg, "%s: D must equal H*dk", what);
    report(ST_SHAPE, msg);
    return 0;
}

static void ext_qkv_split(const float *src, float *q, float *k, float *v, int64_t B, int64_t S, int64_t H, int64_t dk,
                          int64_t D)
{
    if (d_matches("head_interleave_qkv_split", H, dk, D)) done(axb_head_interleave_qkv_split(src, NULL, q, k, v, B, S, H, dk));
}

static void ext_qkv_split_bias(const float *src, const float *bqkv, float *q, float *k, float *v, int64_t B, int64_t S,
                               int64_t H, int64_t dk, int64_t D)
{
    if (!bqkv) { report(ST_NULL_ARG, "head_interleave_qkv_split_bias: NULL bias"); return; }
    if (d_matches("head_interleave_qkv_split_bias", H, dk, D)) done(axb_head_interleave_qkv_split(src, bqkv, q, k, v, B, S, H, dk));
}

static void ext_head_interleave(const float *src, float *dst, int64_t B, int64_t S, int64_t H, int64_t dk)
{
    done(axb_head_interleave(src, dst, B, S, H, dk));
}

static void ext_head_deinterleave(const float *src, float *dst, int64_t B, int64_t S, int64_t H, int64_t dk)
{
    done(axb_head_deinterleave(src, dst, B, S, H, dk));
}

static void ext_qkv_merge(const float *dQ, const float *dK, const float *dV, float *dst, int64_t B, int64_t S, int64_t H,
                          int64_t dk, int64_t D)
{
    if (d_matches("head_deinterleave_qkv_merge", H, dk, D)) done(axb_head_deinterleave_qkv_merge(dQ, dK, dV, dst, B, S, H, dk));
}

static axb_status ext_qkv_cache_build(float *dst, const float *wq, const float *wk, const float *wv, int64_t D)
{
    return done(axb_qkv_cache_build(dst, wq, wk, wv, D));
}

static axb_status ext_bias_cache_build(float *dst, const float *bq, const float *bk, const float *bv, int64_t D)
{
    return done(axb_bias_cache_build(dst, bq, bk, bv, D));
}

static const axb_ax_backend_ops_t ops_table = {
    .name = "b200_tcgen05",
    .gemm = be_gemm,
    .gemm_nt = be_gemm_nt,
    .gemm_tn = be_gemm_tn,
    .dwqkv_split_acc = be_dwqkv_split_acc,
    .dwqkv_split_acc_hm = be_dwqkv_split_acc_hm,
    .qkv_head_gemm = be_qkv_head_gemm,
    .dattn_head_gemm_nt = be_dattn_head_gemm_nt,
    .mha_output_proj_fused = be_mha_output_proj_fused,
    .gemm_relu = be_gemm_relu,
    .gemm_ex = be_gemm_ex,
    .bias_add = be_bias_add,
    .conv_gemm = be_conv_gemm,
    .relu = be_relu,
    .gelu_op = be_gelu,
    .device = AXB_AX_DEVICE_CUDA,
    .init = be_init,
    .shutdown = be_shutdown,
    .synchronize = be_synchronize,
    .device_count = be_device_count,
    .storage_alloc = be_alloc,
    .storage_free = be_free,
    .memcpy_h2d = be_h2d,
    .memcpy_d2h = be_d2h,
    .memcpy_d2d = be_d2d,
};

/* shape rules of the reference's implementation (src/compute/backends/cuda/ops_conv.cu:213-232): weight [C_out, K],
   out [N, C_out, out_h*out_w] contiguous, in_dev all N samples back to back */
static axb_status ext_conv_gemm_batched(const axb_ax_tensor_t *weight, const float *in_dev, int64_t N,
                                        const axb_ax_conv_params_t *single, axb_ax_tensor_t *out)
{
    axb_status st;
    if (!single || !in_dev) return report(ST_NULL_ARG, "conv_gemm_batched: NULL params");
    if ((st = check_f32(weight, "conv_gemm_batched", 2)) || (st = check_f32(out, "conv_gemm_batched", 3))) return st;
    const int64_t C_out = weight->shape[0], K = weight->shape[1], M = single->out_h * single->out_w;
    if (K != single->C_in * single->kh * single->kw) return report(ST_SHAPE, "conv_gemm_batched: weight columns must equal C_in*kh*kw");
    if (out->shape[0] != N || out->shape[1] != C_out || out->shape[2] != M)
        return report(ST_SHAPE, "conv_gemm_batched: out must be [N, C_out, out_h*out_w]");
    return done(axb_conv_gemm_batched(fptr(weight), in_dev, N, C_out, single->C_in, single->H, single->W, single->kh, single->kw,
                                      single->sh, single->sw, single->ph, single->pw, single->out_h, single->out_w, fptr(out)));
}

static const axb_ax_cuda_extension_t extension_table = {
    .head_interleave_qkv_split = ext_qkv_split,
    .head_interleave_qkv_split_bias = ext_qkv_split_bias,
    .head_interleave = ext_head_interleave,
    .head_deinterleave = ext_head_deinterleave,
    .head_deinterleave_qkv_merge = ext_qkv_merge,
    .qkv_cache_build = ext_qkv_cache_build,
    .bias_cache_build = ext_bias_cache_build,
    .sdpa_fwd = ext_sdpa_fwd,
    .sdpa_bwd = ext_sdpa_bwd,
    .conv_gemm_batched = ext_conv_gemm_batched,
};

const axb_ax_backend_ops_t *axb_backend_ops(void) { return &ops_table; }
const axb_ax_cuda_extension_t *axb_cuda_extension(void) { return &extension_table; }
