// elementwise.cu — the vtable's bias_add / relu / gelu_op slots as stand-alone
// HBM-bound passes (float4 grid-stride loops).  The GEMM epilogues fuse the same
// math; these exist because callers may still invoke the slots on their own.
#include "elementwise.cuh"

namespace axb {

__device__ __forceinline__ float ew_gelu(float v)
{
    const float inner = 0.7978845608028654f * (v + 0.044715f * v * v * v);
    return 0.5f * v * (1.0f + tanhf(inner));
}

template <int OP>  // 0 relu, 1 gelu
__global__ void __launch_bounds__(256) unary_kernel(const float *__restrict__ in, float *__restrict__ out,
                                                    int64_t n, bool vec)
{
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (vec) {
        const int64_t n4 = n / 4;
        for (int64_t i = t; i < n4; i += stride) {
            float4 v = reinterpret_cast<const float4 *>(in)[i];
            if (OP == 0) { v.x = fmaxf(v.x, 0.f); v.y = fmaxf(v.y, 0.f); v.z = fmaxf(v.z, 0.f); v.w = fmaxf(v.w, 0.f); }
            else { v.x = ew_gelu(v.x); v.y = ew_gelu(v.y); v.z = ew_gelu(v.z); v.w = ew_gelu(v.w); }
            reinterpret_cast<float4 *>(out)[i] = v;
        }
        for (int64_t i = n4 * 4 + t; i < n; i += stride) out[i] = OP == 0 ? fmaxf(in[i], 0.f) : ew_gelu(in[i]);
    } else {
        for (int64_t i = t; i < n; i += stride) out[i] = OP == 0 ? fmaxf(in[i], 0.f) : ew_gelu(in[i]);
    }
}

// out[i,j] = in[i,j] + bias[axis == 0 ? i % period : j]; in-place safe (each element read then written by one
// thread).  period < M serves a broadcast axis in the middle of an n-d tensor viewed as [outer*axis_len, inner].
// IDX: 32-bit indices when the tensor has fewer than 2^31 accesses — the row / column split of every access is an
// integer division, and the 64-bit one costs enough instructions to hold the kernel at three quarters of the copy rate
template <typename IDX>
__global__ void __launch_bounds__(256) bias_add_kernel(const float *in, const float *__restrict__ bias,
                                                       int axis, float *out, int64_t M, int64_t N, int64_t period,
                                                       bool vec)
{
    const IDX stride = (IDX)gridDim.x * (IDX)blockDim.x;
    const IDX t = (IDX)blockIdx.x * (IDX)blockDim.x + (IDX)threadIdx.x;
    const IDX per = (IDX)period;
    if (vec) {  // N % 4 == 0 and 16-byte aligned pointers
        const IDX n4 = (IDX)(N / 4), total = (IDX)(M * (N / 4));
        for (IDX i = t; i < total; i += stride) {
            const IDX r = i / n4, c = (i - r * n4) * 4;
            float4 v = reinterpret_cast<const float4 *>(in)[i];
            if (axis == 0) {
                const float b = __ldg(bias + r % per);
                v.x += b; v.y += b; v.z += b; v.w += b;
            } else {
                const float4 b = __ldg(reinterpret_cast<const float4 *>(bias + c));
                v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
            }
            reinterpret_cast<float4 *>(out)[i] = v;
        }
    } else {
        const IDX n = (IDX)N, total = (IDX)(M * N);
        for (IDX i = t; i < total; i += stride) {
            const IDX r = i / n, c = i - r * n;
            out[i] = in[i] + __ldg(bias + (axis == 0 ? r % per : c));
        }
    }
}

static inline int ew_grid(int64_t items, int sm_count)
{
    int64_t b = (items + 255) / 256;
    const int64_t cap = (int64_t)sm_count * 8;
    if (b > cap) b = cap;
    return (int)(b < 1 ? 1 : b);
}

__global__ void __launch_bounds__(256) fill_kernel(float *__restrict__ out, int64_t n, float value)
{
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) out[i] = value;
}

static inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int launch_fill(float *out, int64_t n, float value, int sm_count, cudaStream_t st)
{
    if (n <= 0) return 0;
    fill_kernel<<<ew_grid(n, sm_count), 256, 0, st>>>(out, n, value);
    return (int)cudaGetLastError();
}

int launch_unary(int op, const float *in, float *out, int64_t n, int sm_count, cudaStream_t st)
{
    if (n <= 0) return 0;
    const bool vec = aligned16(in) && aligned16(out);
    const int g = ew_grid(vec ? (n + 3) / 4 : n, sm_count);
    if (op == 0) unary_kernel<0><<<g, 256, 0, st>>>(in, out, n, vec);
    else unary_kernel<1><<<g, 256, 0, st>>>(in, out, n, vec);
    return (int)cudaGetLastError();
}

int launch_bias_add(const float *in, const float *bias, int axis, float *out, int64_t M, int64_t N,
                    int sm_count, cudaStream_t st, int64_t period)
{
    if (M <= 0 || N <= 0) return 0;
    if (period <= 0) period = M;
    const bool vec = (N % 4 == 0) && aligned16(in) && aligned16(out) && aligned16(bias);
    const int g = ew_grid(vec ? M * N / 4 : M * N, sm_count);
    // (the loop index runs up to total + grid size: keep that inside 31 bits too)
    if (M * N < ((int64_t)1 << 30)) bias_add_kernel<uint32_t><<<g, 256, 0, st>>>(in, bias, axis, out, M, N, period, vec);
    else bias_add_kernel<int64_t><<<g, 256, 0, st>>>(in, bias, axis, out, M, N, period, vec);
    return (int)cudaGetLastError();
}

}  // namespace axb
