/* axb_oracle.c — CPU restatement of axiom's matmul-dispatch hot path.

   TEST INFRASTRUCTURE ONLY.  Nothing in the shipped library links, loads or
   calls this file; it exists so the parity tests, the smoke check and the
   cpu_baseline leg of the bench have an independent answer to compare the
   CUDA kernels with.  Build with `make -C oracle` (-ffp-contract=off so the
   float arithmetic below is executed exactly as written).

   Each function names the reference code it restates (paths are relative to
   the axiom source tree).  The arithmetic is written from those sources'
   behaviour, not copied: plain loops, no SIMD, OpenMP only across output
   elements so the per-element summation order never depends on the thread
   count.

   Pinning status:
     - gemm / gemm_nt / gemm_tn / gemm_ex / bias / relu / gelu / w8a32 / sdpa:
       pinned against the reference's own known-answer tests (tests/golden/)
       and against the compiled reference (oracle/_ref) on seeded inputs.
     - w8a8 (int8 x int8 -> s32 -> requantised int8): PARITY UNPINNED.  The
       reference has no such kernel; the restatement follows the reference
       quantiser's conventions (scale = absmax/127, lrintf, clamp +-127,
       src/core/quantize.c:36-56) and is pinned only by hand-checkable
       known-answer cases committed beside the tests. */

#include <float.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ---------------------------------------------------------------- inputs */

/* xorshift32 uniform fill in [-1, 1): same recurrence and scaling as the
   generator the reference's quantisation test uses (tests/test_quantize.c:23-29),
   so a seed names the same tensor in the reference's tests and in ours. */
ORC_API void orc_fill_uniform(float *buf, int64_t n, uint32_t seed)
{
    uint32_t s = seed;
    for (int64_t i = 0; i < n; i++) {
        s ^= s << 13; s ^= s >> 17; s ^= s << 5;
        buf[i] = ((float)(s & 0xFFFFu) / 32768.0f) - 1.0f;
    }
}

/* standard normal * sigma: Box-Muller over the same xorshift32 stream
   (two 24-bit uniforms per pair of normals). */
ORC_API void orc_fill_normal(float *buf, int64_t n, uint32_t seed, float sigma)
{
    uint32_t s = seed;
    for (int64_t i = 0; i < n; i += 2) {
        s ^= s << 13; s ^= s >> 17; s ^= s << 5;
        double u1 = ((double)(s >> 8) + 1.0) / 16777217.0;
        s ^= s << 13; s ^= s >> 17; s ^= s << 5;
        double u2 = (double)(s >> 8) / 16777216.0;
        double r = sqrt(-2.0 * log(u1));
        buf[i] = (float)(r * cos(6.283185307179586 * u2)) * sigma;
        if (i + 1 < n) buf[i + 1] = (float)(r * sin(6.283185307179586 * u2)) * sigma;
    }
}

/* int8 uniform in {-127..127} from the same stream. */
ORC_API void orc_fill_int8(int8_t *buf, int64_t n, uint32_t seed)
{
    uint32_t s = seed;
    for (int64_t i = 0; i < n; i++) {
        s ^= s << 13; s ^= s >> 17; s ^= s << 5;
        buf[i] = (int8_t)((int)((s >> 8) % 255u) - 127);
    }
}

/* uniform in [lo, hi) from the same stream (per-channel scales). */
ORC_API void orc_fill_range(float *buf, int64_t n, uint32_t seed, float lo, float hi)
{
    uint32_t s = seed;
    for (int64_t i = 0; i < n; i++) {
        s ^= s << 13; s ^= s >> 17; s ^= s << 5;
        buf[i] = lo + (hi - lo) * ((float)(s >> 8) / 16777216.0f);
    }
}

/* ---------------------------------------------------------------- GEMM */

/* C[M,N] = op(A) . op(B), fp32, every output element summed over p = 0..K-1 in
   order with one rounding per multiply and per add.  Restates the strided
   triple loop of src/compute/backends/cpu_naive.c:150-188 (which the
   reference's own property tests use as ground truth, tests/test_property.c:176-209).
   ta: A is stored [K,M] (gemm_tn, src/compute/backends/cuda/ops_gemm.cu:103-126);
   tb: B is stored [N,K] (gemm_nt, ops_gemm.cu:73-96). */
ORC_API void orc_gemm_f32(const float *A, const float *B, float *C,
                          int64_t M, int64_t N, int64_t K, int ta, int tb)
{
    const int64_t as_i = ta ? 1 : K, as_p = ta ? M : 1;
    const int64_t bs_p = tb ? 1 : N, bs_j = tb ? K : 1;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < M; i++) {
        float *row = (float *)malloc((size_t)(N > 0 ? N : 1) * sizeof(float));
        for (int64_t j = 0; j < N; j++) row[j] = 0.0f;
        if (!tb) {
            /* p outer / j inner: same per-element order, unit-stride B rows */
            for (int64_t p = 0; p < K; p++) {
                const float a = A[i * as_i + p * as_p];
                const float *b = B + p * N;
                for (int64_t j = 0; j < N; j++) row[j] = row[j] + a * b[j];
            }
        } else {
            for (int64_t j = 0; j < N; j++) {
                float sum = 0.0f;
                for (int64_t p = 0; p < K; p++)
                    sum = sum + A[i * as_i + p * as_p] * B[p * bs_p + j * bs_j];
                row[j] = sum;
            }
        }
        memcpy(C + i * N, row, (size_t)N * sizeof(float));
        free(row);
    }
}

/* Same contraction with a double accumulator: the "exact" answer both the
   reference's fp32 path and the GPU's split-precision path are measured
   against (normalised error max|x - ref| / max|ref|). */
ORC_API void orc_gemm_f64(const float *A, const float *B, double *C,
                          int64_t M, int64_t N, int64_t K, int ta, int tb)
{
    const int64_t as_i = ta ? 1 : K, as_p = ta ? M : 1;
    const int64_t bs_p = tb ? 1 : N, bs_j = tb ? K : 1;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < M; i++) {
        double *row = (double *)calloc((size_t)(N > 0 ? N : 1), sizeof(double));
        if (!tb) {
            for (int64_t p = 0; p < K; p++) {
                const double a = (double)A[i * as_i + p * as_p];
                const float *b = B + p * N;
                for (int64_t j = 0; j < N; j++) row[j] += a * (double)b[j];
            }
        } else {
            for (int64_t j = 0; j < N; j++) {
                double sum = 0.0;
                for (int64_t p = 0; p < K; p++)
                    sum += (double)A[i * as_i + p * as_p] * (double)B[p * bs_p + j * bs_j];
                row[j] = sum;
            }
        }
        memcpy(C + i * N, row, (size_t)N * sizeof(double));
        free(row);
    }
}

/* C = alpha * (A.B) + beta * C  (src/compute/backends/cpu_naive.c:272-306,
   ops_gemm.cu:43-65).  beta == 0 never reads C. */
ORC_API void orc_gemm_ex_f32(const float *A, const float *B, float alpha, float beta,
                             float *C, int64_t M, int64_t N, int64_t K)
{
    float *tmp = (float *)malloc((size_t)(M * N > 0 ? M * N : 1) * sizeof(float));
    orc_gemm_f32(A, B, tmp, M, N, K, 0, 0);
    for (int64_t i = 0; i < M * N; i++) {
        float v = alpha * tmp[i];
        if (beta != 0.0f) v = v + beta * C[i];
        C[i] = v;
    }
    free(tmp);
}

/* ------------------------------------------------------------ epilogues */

/* tanh-approximation GELU, constants as src/core/activations.c:23-25 and
   src/compute/backends/cuda/ops_activations.cu:12-24:
   0.5 v (1 + tanh(0.7978845608 (v + 0.044715 v^3))). */
static inline float orc_gelu1(float v)
{
    const float inner = 0.7978845608028654f * (v + 0.044715f * v * v * v);
    return 0.5f * v * (1.0f + tanhf(inner));
}

ORC_API void orc_gelu(const float *in, float *out, int64_t n)
{
    for (int64_t i = 0; i < n; i++) out[i] = orc_gelu1(in[i]);
}

ORC_API void orc_relu(const float *in, float *out, int64_t n)
{
    for (int64_t i = 0; i < n; i++) out[i] = in[i] > 0.0f ? in[i] : 0.0f;
}

/* out[i,j] = act(in[i,j] + bias[j]).  The per-COLUMN broadcast is the
   documented dense-layer meaning (include/axiom/ops.h:52-57) and what the
   reference's own fallback loop and its fused gemm_relu do
   (src/core/ops.c:359-364, src/compute/backends/cpu_opt.c:7412-7428).
   act: 0 none, 1 relu, 2 gelu.  bias may be NULL. */
ORC_API void orc_bias_act(const float *in, const float *bias, float *out,
                          int64_t M, int64_t N, int act)
{
    for (int64_t i = 0; i < M; i++)
        for (int64_t j = 0; j < N; j++) {
            float v = in[i * N + j];
            if (bias) v = v + bias[j];
            if (act == 1) v = v > 0.0f ? v : 0.0f;
            else if (act == 2) v = orc_gelu1(v);
            out[i * N + j] = v;
        }
}

/* out = in + bias broadcast along `axis` of a 2-D [M,N] tensor
   (bias_add slot: src/compute/backends/cuda/ops_fused.cu:260-292). */
ORC_API void orc_bias_add_axis(const float *in, const float *bias, int axis,
                               float *out, int64_t M, int64_t N)
{
    for (int64_t i = 0; i < M; i++)
        for (int64_t j = 0; j < N; j++)
            out[i * N + j] = in[i * N + j] + bias[axis == 0 ? i : j];
}

/* ---------------------------------------------------------- quantisation */

/* Per-row symmetric int8 quantiser (src/core/quantize.c:36-56):
   scale = absmax/127 (1.0 for an all-zero row), q = clamp(lrintf(w * (1/scale))). */
ORC_API void orc_quantize_rows(const float *w, int64_t N, int64_t K,
                               int8_t *q, float *scales)
{
    for (int64_t n = 0; n < N; n++) {
        const float *row = w + n * K;
        float absmax = 0.0f;
        for (int64_t k = 0; k < K; k++) {
            const float a = fabsf(row[k]);
            if (a > absmax) absmax = a;
        }
        const float scale = absmax > 0.0f ? absmax / 127.0f : 1.0f;
        const float inv = 1.0f / scale;
        scales[n] = scale;
        for (int64_t k = 0; k < K; k++) {
            long v = lrintf(row[k] * inv);
            if (v > 127) v = 127;
            if (v < -127) v = -127;
            q[n * K + k] = (int8_t)v;
        }
    }
}

ORC_API void orc_dequantize_rows(const int8_t *q, const float *scales,
                                 int64_t N, int64_t K, float *out)
{
    for (int64_t n = 0; n < N; n++)
        for (int64_t k = 0; k < K; k++)
            out[n * K + k] = (float)q[n * K + k] * scales[n];
}

/* W8A32: out[m,n] = scale[n] * sum_k a[m,k] * (float)q[n,k], fp32 accumulate
   in k order — the scalar branch of src/core/quantize.c:168-173. */
ORC_API void orc_qgemm_w8a32(const float *a, const int8_t *q, const float *scales,
                             float *out, int64_t M, int64_t N, int64_t K)
{
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; n++)
        for (int64_t m = 0; m < M; m++) {
            float acc = 0.0f;
            for (int64_t k = 0; k < K; k++)
                acc = acc + a[m * K + k] * (float)q[n * K + k];
            out[m * N + n] = acc * scales[n];
        }
}

/* Same sum carried in double: the exact value W8A32 results are normalised
   against. */
ORC_API void orc_qgemm_w8a32_f64(const float *a, const int8_t *q, const float *scales,
                                 double *out, int64_t M, int64_t N, int64_t K)
{
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; n++)
        for (int64_t m = 0; m < M; m++) {
            double acc = 0.0;
            for (int64_t k = 0; k < K; k++)
                acc += (double)a[m * K + k] * (double)q[n * K + k];
            out[m * N + n] = acc * (double)scales[n];
        }
}

/* W8A8 (PARITY UNPINNED — no reference kernel exists):
     acc[m,n]  = sum_k (int32)a_q[m,k] * (int32)b_q[n,k]          exact integer
     mult[n]   = (a_scale * b_scales[n]) / out_scale               fp32, two roundings
     out[m,n]  = clamp(lrintf((float)acc * mult[n]), -127, 127)    round-to-nearest-even
   Rounding and clamp follow the reference quantiser (src/core/quantize.c:50-54).
   acc_out and out_q may each be NULL. */
ORC_API void orc_qgemm_w8a8(const int8_t *a_q, float a_scale,
                            const int8_t *b_q, const float *b_scales, float out_scale,
                            int32_t *acc_out, int8_t *out_q,
                            int64_t M, int64_t N, int64_t K)
{
#pragma omp parallel for schedule(static)
    for (int64_t m = 0; m < M; m++)
        for (int64_t n = 0; n < N; n++) {
            int32_t acc = 0;
            for (int64_t k = 0; k < K; k++)
                acc += (int32_t)a_q[m * K + k] * (int32_t)b_q[n * K + k];
            if (acc_out) acc_out[m * N + n] = acc;
            if (out_q) {
                const float ab = a_scale * b_scales[n];
                const float mult = ab / out_scale;
                long v = lrintf((float)acc * mult);
                if (v > 127) v = 127;
                if (v < -127) v = -127;
                out_q[m * N + n] = (int8_t)v;
            }
        }
}

/* -------------------------------------------------------------- attention */

/* O = softmax(scale * Q.K^T + mask) . V per head on head-major [BH,S,dk]
   buffers, L = rowmax + log(rowsum) (nullable).  Restates the naive reference
   the attention tests compare against (tests/test_attention.c:19-49): scores in
   float, masked entries excluded, exp via expf.  The softmax weights are
   normalised before the P.V product exactly as there. */
ORC_API void orc_sdpa_fwd(const float *Q, const float *K, const float *V,
                          float *O, float *L,
                          int64_t BH, int64_t S, int64_t dk, float scale, int causal)
{
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t h = 0; h < BH; h++) {
        const float *q = Q + h * S * dk, *k = K + h * S * dk, *v = V + h * S * dk;
        float *o = O + h * S * dk;
        float *p = (float *)malloc((size_t)S * sizeof(float));
        for (int64_t i = 0; i < S; i++) {
            const int64_t jend = causal ? i + 1 : S;
            float mx = -INFINITY;
            for (int64_t j = 0; j < jend; j++) {
                float dot = 0.0f;
                for (int64_t d = 0; d < dk; d++) dot = dot + q[i * dk + d] * k[j * dk + d];
                dot = dot * scale;
                p[j] = dot;
                if (dot > mx) mx = dot;
            }
            float sum = 0.0f;
            for (int64_t j = 0; j < jend; j++) {
                p[j] = expf(p[j] - mx);
                sum = sum + p[j];
            }
            const float inv = 1.0f / sum;
            for (int64_t d = 0; d < dk; d++) {
                float acc = 0.0f;
                for (int64_t j = 0; j < jend; j++) acc = acc + p[j] * inv * v[j * dk + d];
                o[i * dk + d] = acc;
            }
            if (L) L[h * S + i] = mx + logf(sum);
        }
        free(p);
    }
}

/* The same attention carried in double (accuracy yardstick for both sides). */
ORC_API void orc_sdpa_fwd_f64(const float *Q, const float *K, const float *V,
                              double *O, double *L,
                              int64_t BH, int64_t S, int64_t dk, float scale, int causal)
{
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t h = 0; h < BH; h++) {
        const float *q = Q + h * S * dk, *k = K + h * S * dk, *v = V + h * S * dk;
        double *o = O + h * S * dk;
        double *p = (double *)malloc((size_t)S * sizeof(double));
        for (int64_t i = 0; i < S; i++) {
            const int64_t jend = causal ? i + 1 : S;
            double mx = -INFINITY;
            for (int64_t j = 0; j < jend; j++) {
                double dot = 0.0;
                for (int64_t d = 0; d < dk; d++) dot += (double)q[i * dk + d] * (double)k[j * dk + d];
                dot *= (double)scale;
                p[j] = dot;
                if (dot > mx) mx = dot;
            }
            double sum = 0.0;
            for (int64_t j = 0; j < jend; j++) { p[j] = exp(p[j] - mx); sum += p[j]; }
            for (int64_t d = 0; d < dk; d++) {
                double acc = 0.0;
                for (int64_t j = 0; j < jend; j++) acc += p[j] * (double)v[j * dk + d];
                o[i * dk + d] = acc / sum;
            }
            if (L) L[h * S + i] = mx + log(sum);
        }
        free(p);
    }
}

/* Convolution of one sample as the reference's conv_gemm slot defines it (include/axiom/internal/backend_ops.h:193-202,
   ax_conv_params_t in include/axiom/compute.h:36-43; CUDA path k_im2col_sample + GEMM,
   src/compute/backends/cuda/ops_conv.cu:120-215): out[co, oh*out_w + ow] = sum over (c, ky, kx) of
   weight[co, (c*kh + ky)*kw + kx] * input[c, oh*sh + ky - ph, ow*sw + kx - pw], zero outside the image.
   fp32, terms added in k order. */
ORC_API void orc_conv_gemm(const float *weight, const float *input, int64_t C_out, int64_t C_in, int64_t H, int64_t W,
                           int kh, int kw, int sh, int sw, int ph, int pw, int64_t out_h, int64_t out_w, float *out)
{
    const int64_t K = C_in * kh * kw, P = out_h * out_w;
#pragma omp parallel for schedule(static)
    for (int64_t co = 0; co < C_out; co++)
        for (int64_t pix = 0; pix < P; pix++) {
            const int64_t oh = pix / out_w, ow = pix - oh * out_w;
            float acc = 0.0f;
            for (int64_t c = 0; c < C_in; c++)
                for (int ky = 0; ky < kh; ky++)
                    for (int kx = 0; kx < kw; kx++) {
                        const int64_t ih = oh * sh + ky - ph, iw = ow * sw + kx - pw;
                        if (ih >= 0 && ih < H && iw >= 0 && iw < W)
                            acc += weight[co * K + (c * kh + ky) * kw + kx] * input[(c * H + ih) * W + iw];
                    }
            out[co * P + pix] = acc;
        }
}

/* Attention backward carried in double (src/compute/backends/cpu_opt.c:9112-9180 computes the same quantities
   tile by tile in fp32): P = softmax(scale*Q.K^T [+causal mask]) recomputed from the inputs,
   D_i = dO_i.O_i, dV = P^T.dO, dS = P o (dO.V^T - D) * scale, dQ = dS.K, dK = dS^T.Q.  O is the forward output
   of the same inputs (the caller passes what the forward produced).  Outputs are overwritten. */
ORC_API void orc_sdpa_bwd_f64(const float *Q, const float *K, const float *V, const float *O, const float *dO,
                              double *dQ, double *dK, double *dV,
                              int64_t BH, int64_t S, int64_t dk, float scale, int causal)
{
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t h = 0; h < BH; h++) {
        const float *q = Q + h * S * dk, *k = K + h * S * dk, *v = V + h * S * dk, *o = O + h * S * dk, *d_o = dO + h * S * dk;
        double *dq = dQ + h * S * dk, *dkk = dK + h * S * dk, *dv = dV + h * S * dk;
        for (int64_t i = 0; i < S * dk; i++) dq[i] = dkk[i] = dv[i] = 0.0;
        double *p = (double *)malloc((size_t)S * sizeof(double));
        for (int64_t i = 0; i < S; i++) {
            const int64_t jend = causal ? i + 1 : S;
            double mx = -INFINITY, sum = 0.0, Di = 0.0;
            for (int64_t j = 0; j < jend; j++) {
                double dot = 0.0;
                for (int64_t d = 0; d < dk; d++) dot += (double)q[i * dk + d] * (double)k[j * dk + d];
                p[j] = dot * (double)scale;
                if (p[j] > mx) mx = p[j];
            }
            for (int64_t j = 0; j < jend; j++) { p[j] = exp(p[j] - mx); sum += p[j]; }
            for (int64_t d = 0; d < dk; d++) Di += (double)d_o[i * dk + d] * (double)o[i * dk + d];
            for (int64_t j = 0; j < jend; j++) {
                const double pj = p[j] / sum;
                double dp = 0.0;
                for (int64_t d = 0; d < dk; d++) dp += (double)d_o[i * dk + d] * (double)v[j * dk + d];
                const double ds = pj * (dp - Di) * (double)scale;
                for (int64_t d = 0; d < dk; d++) {
                    dv[j * dk + d] += pj * (double)d_o[i * dk + d];
                    dq[i * dk + d] += ds * (double)k[j * dk + d];
                    dkk[j * dk + d] += ds * (double)q[i * dk + d];
                }
            }
        }
        free(p);
    }
}

/* QKV projection straight into the head-major layout (src/compute/backends/cpu_opt.c:6160-6260,
   ax_compute_qkv_head_gemm, include/axiom/compute.h:150-170): every output starts at its bias (or zero) and the
   products are accumulated on top in k order; column which*D + h*dk + d of row b*S + s lands in
   out[which][(b*H + h)*S + s][d]. */
ORC_API void orc_qkv_head_gemm(const float *X, const float *Wqkv, const float *bqkv, int64_t B, int64_t S,
                               int64_t H, int64_t dk, float *Qh, float *Kh, float *Vh)
{
    const int64_t D = H * dk, rows = B * S;
    float *outs[3] = { Qh, Kh, Vh };
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; r++) {
        const int64_t b = r / S, s = r - b * S;
        for (int64_t c = 0; c < 3 * D; c++) {
            const int64_t which = c / D, rem = c - which * D, h = rem / dk, d = rem - h * dk;
            float acc = bqkv ? bqkv[c] : 0.0f;
            for (int64_t k = 0; k < D; k++) acc += X[r * D + k] * Wqkv[k * 3 * D + c];
            outs[which][((b * H + h) * S + s) * dk + d] = acc;
        }
    }
}

/* Single-token attention against a KV cache (src/compute/backends/cpu_opt.c:9586-9654, reached from
   ax_kv_cache_attend, include/axiom/attention.h:373-381): per head, scores[j] = dot(q, K[j]) * scale over the
   cur_len cached rows, softmax with the maximum subtracted, out = sum_j p[j] * V[j].  The cache is laid out
   [BH, max_seq, dk]; rows past cur_len are not read.  fp32 with sequential sums, as the reference's scalar tail. */
ORC_API void orc_kv_cache_attend(const float *Kc, const float *Vc, const float *Qn, float *out,
                                 int64_t BH, int64_t cur_len, int64_t max_seq, int64_t dk, float scale)
{
#pragma omp parallel for schedule(static)
    for (int64_t h = 0; h < BH; h++) {
        const float *K_h = Kc + h * max_seq * dk, *V_h = Vc + h * max_seq * dk, *q = Qn + h * dk;
        float *o = out + h * dk;
        float *scores = (float *)malloc((size_t)(cur_len > 0 ? cur_len : 1) * sizeof(float));
        float mx = -FLT_MAX;
        for (int64_t j = 0; j < cur_len; j++) {
            float dot = 0.0f;
            for (int64_t d = 0; d < dk; d++) dot += q[d] * K_h[j * dk + d];
            scores[j] = dot * scale;
            if (scores[j] > mx) mx = scores[j];
        }
        float sum = 0.0f;
        for (int64_t j = 0; j < cur_len; j++) { scores[j] = expf(scores[j] - mx); sum += scores[j]; }
        const float inv = 1.0f / sum;
        for (int64_t d = 0; d < dk; d++) o[d] = 0.0f;
        for (int64_t j = 0; j < cur_len; j++) {
            const float w = scores[j] * inv;
            for (int64_t d = 0; d < dk; d++) o[d] += w * V_h[j * dk + d];
        }
        free(scores);
    }
}

/* The same in double (accuracy yardstick). */
ORC_API void orc_kv_cache_attend_f64(const float *Kc, const float *Vc, const float *Qn, double *out,
                                     int64_t BH, int64_t cur_len, int64_t max_seq, int64_t dk, float scale)
{
#pragma omp parallel for schedule(static)
    for (int64_t h = 0; h < BH; h++) {
        const float *K_h = Kc + h * max_seq * dk, *V_h = Vc + h * max_seq * dk, *q = Qn + h * dk;
        double *o = out + h * dk;
        double *scores = (double *)malloc((size_t)(cur_len > 0 ? cur_len : 1) * sizeof(double));
        double mx = -INFINITY;
        for (int64_t j = 0; j < cur_len; j++) {
            double dot = 0.0;
            for (int64_t d = 0; d < dk; d++) dot += (double)q[d] * (double)K_h[j * dk + d];
            scores[j] = dot * (double)scale;
            if (scores[j] > mx) mx = scores[j];
        }
        double sum = 0.0;
        for (int64_t j = 0; j < cur_len; j++) { scores[j] = exp(scores[j] - mx); sum += scores[j]; }
        for (int64_t d = 0; d < dk; d++) {
            double acc = 0.0;
            for (int64_t j = 0; j < cur_len; j++) acc += scores[j] * (double)V_h[j * dk + d];
            o[d] = acc / sum;
        }
        free(scores);
    }
}

ORC_API int orc_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
